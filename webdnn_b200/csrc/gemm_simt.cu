// CUDA-core fp32 contraction kernel: strided/batched GEMM and implicit-GEMM convolution with the
// fused epilogues.  It is the path for shapes the tcgen05 kernel does not take (grouped or dilated
// convolutions, channel counts that are not a multiple of 32, tiny or oddly strided matrices).
// 64x64 output tile per CTA, K step 16, 256 threads, 4x4 accumulators per thread, fp32 FMA.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16
#define PAD 4

struct SimtProblem {
  int is_conv;
  int64_t batch, M, N, K;
  // gemm addressing
  int64_t sab, sa0, sa1, sbb, sb0, sb1, sc0, sc1;
  float alpha, beta;
  int has_c;
  int c_in_y;  // 1: the C operand IS the output (Y = alpha*A*B + beta*Y): read through Y with plain loads
  // conv addressing (x NHWC, w [ch_out][k_h][k_w][cig])
  int64_t in_h, in_w, ch_in, cig, cog, k_h, k_w, out_h, out_w, stride_h, stride_w, pad_t, pad_l,
      dil_h, dil_w, ch_out;
  int relu;
};

__global__ void __launch_bounds__(256) simt_contract_kernel(SimtProblem p, const float* __restrict__ A,
                                                            const float* __restrict__ B,
                                                            const float* __restrict__ C,
                                                            const float* __restrict__ scale,
                                                            const float* __restrict__ shift,
                                                            const float* __restrict__ residual,
                                                            float* __restrict__ Y) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  __shared__ int64_t row_base[BM];  // conv: element offset of (n, iy0, ix0) or -1
  __shared__ int row_iy[BM], row_ix[BM];

  const int t = threadIdx.x;
  const int64_t tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int64_t tiles = p.batch * tiles_m * tiles_n;
  const int tx = t & 15, ty = t >> 4;

  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t bz = tile / (tiles_m * tiles_n);
    const int64_t tr = tile % (tiles_m * tiles_n);
    const int64_t m0 = (tr / tiles_n) * BM, n0 = (tr % tiles_n) * BN;

    if (p.is_conv) {
      if (t < BM) {
        int64_t m = m0 + t;
        if (m < p.M) {
          int64_t ox = m % p.out_w, oy = (m / p.out_w) % p.out_h, n = m / (p.out_w * p.out_h);
          row_iy[t] = (int)(oy * p.stride_h - p.pad_t);
          row_ix[t] = (int)(ox * p.stride_w - p.pad_l);
          row_base[t] = n * p.in_h * p.in_w * p.ch_in + bz * p.cig;
        } else {
          row_base[t] = -1;
          row_iy[t] = row_ix[t] = 0;
        }
      }
      __syncthreads();
    }

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
      // ---- load A tile (BM x BK)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int e = t + i * 256;
        int mm, kk;
        if (p.is_conv || p.sa1 == 1) { kk = e & (BK - 1); mm = e >> 4; }
        else { mm = e & (BM - 1); kk = e >> 6; }
        int64_t m = m0 + mm, k = k0 + kk;
        float v = 0.f;
        if (m < p.M && k < p.K) {
          if (p.is_conv) {
            int64_t ci = k % p.cig, kx = (k / p.cig) % p.k_w, ky = k / (p.cig * p.k_w);
            int64_t iy = row_iy[mm] + ky * p.dil_h, ix = row_ix[mm] + kx * p.dil_w;
            if (iy >= 0 && iy < p.in_h && ix >= 0 && ix < p.in_w)
              v = __ldg(A + row_base[mm] + (iy * p.in_w + ix) * p.ch_in + ci);
          } else {
            v = __ldg(A + bz * p.sab + m * p.sa0 + k * p.sa1);
          }
        }
        As[kk][mm] = v;
      }
      // ---- load B tile (BK x BN)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int e = t + i * 256;
        int nn, kk;
        if (p.is_conv || p.sb0 == 1) { kk = e & (BK - 1); nn = e >> 4; }
        else { nn = e & (BN - 1); kk = e >> 6; }
        int64_t n = n0 + nn, k = k0 + kk;
        float v = 0.f;
        if (n < p.N && k < p.K) {
          if (p.is_conv) v = __ldg(B + (bz * p.cog + n) * p.K + k);
          else v = __ldg(B + bz * p.sbb + k * p.sb0 + n * p.sb1);
        }
        Bs[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < BK; kk++) {
        float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
        float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
        float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }

    // ---- epilogue
#pragma unroll
    for (int i = 0; i < 4; i++) {
      int64_t m = m0 + ty * 4 + i;
      if (m >= p.M) continue;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int64_t n = n0 + tx * 4 + j;
        if (n >= p.N) continue;
        float v = acc[i][j];
        int64_t o;
        if (p.is_conv) {
          int64_t c = bz * p.cog + n;
          float s = scale ? __ldg(scale + c) : 1.f, sh = shift ? __ldg(shift + c) : 0.f;
          v = fmaf(v, s, sh);
          o = m * p.ch_out + c;
          if (residual) v += __ldg(residual + o);
        } else {
          v *= p.alpha;
          o = (bz * p.M + m) * p.N + n;
          // In-place accumulation reads the old value through the output pointer itself: the read-only
          // data path (__ldg) and a second __restrict__ pointer must never see memory this kernel writes.
          if (p.c_in_y) v += Y[o] * p.beta;
          else if (p.has_c) v += __ldg(C + m * p.sc0 + n * p.sc1) * p.beta;
        }
        if (p.relu) v = v > 0.f ? v : (v == v ? 0.f : v);
        Y[o] = v;
      }
    }
    __syncthreads();
  }
}

static int launch_simt(wdc_context* ctx, const SimtProblem& p, const float* A, const float* B,
                       const float* C, const float* scale, const float* shift, const float* residual,
                       float* Y) {
  int64_t tiles = p.batch * ceil_div64(p.M, BM) * ceil_div64(p.N, BN);
  if (tiles == 0) return WDC_OK;
  int64_t cap = (int64_t)ctx->sm_count * 8;
  int grid = (int)(tiles < cap ? tiles : cap);
  simt_contract_kernel<<<grid, 256, 0, ctx->stream>>>(p, A, B, C, scale, shift, residual, Y);
  return wdc_check_launch(ctx, "simt_contract_kernel");
}

// Makes the driver load this file's module on the current device (lazy module loading would otherwise do it
// at the first launch).
int wdc_simt_preload(wdc_context* ctx) {
  cudaFuncAttributes fa;
  WDC_CUDA(ctx, cudaFuncGetAttributes(&fa, simt_contract_kernel));
  return WDC_OK;
}

int wdc_simt_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B, const float* C,
                  float* Y) {
  SimtProblem p = {};
  p.is_conv = 0;
  p.batch = d->batch; p.M = d->m; p.N = d->n; p.K = d->k;
  p.sab = d->sab; p.sa0 = d->sa0; p.sa1 = d->sa1;
  p.sbb = d->sbb; p.sb0 = d->sb0; p.sb1 = d->sb1;
  p.sc0 = d->sc0; p.sc1 = d->sc1;
  p.alpha = d->alpha; p.beta = d->beta; p.has_c = C != nullptr; p.relu = d->relu;
  if (C == Y && C != nullptr) {
    // accumulate into Y: only the element-for-element case is meaningful (each output reads its own old value)
    if (d->batch != 1 || d->sc0 != d->n || d->sc1 != 1)
      return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_gemm: C may alias Y only as a dense [m, n] matrix of a single batch");
    p.c_in_y = 1;
    p.has_c = 0;
    C = nullptr;
  }
  return launch_simt(ctx, p, A, B, C, nullptr, nullptr, nullptr, Y);
}

int wdc_simt_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w,
                    const float* scale, const float* shift, const float* residual, float* y) {
  SimtProblem p = {};
  p.is_conv = 1;
  p.batch = d->group;
  p.cig = d->ch_in / d->group; p.cog = d->ch_out / d->group;
  p.M = d->batch * d->out_h * d->out_w; p.N = p.cog; p.K = p.cig * d->k_h * d->k_w;
  p.in_h = d->in_h; p.in_w = d->in_w; p.ch_in = d->ch_in; p.ch_out = d->ch_out;
  p.k_h = d->k_h; p.k_w = d->k_w; p.out_h = d->out_h; p.out_w = d->out_w;
  p.stride_h = d->stride_h; p.stride_w = d->stride_w; p.pad_t = d->pad_t; p.pad_l = d->pad_l;
  p.dil_h = d->dil_h; p.dil_w = d->dil_w; p.relu = d->relu;
  return launch_simt(ctx, p, x, w, nullptr, scale, shift, residual, y);
}

// ------------------------------------------------------------------------ public entries
extern "C" int wdc_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B,
                        const float* C, float* Y) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_gemm: null context");
  wdc_note_write(ctx, Y);
  WDC_REQUIRE(ctx, d != nullptr, "wdc_gemm: null descriptor");
  WDC_REQUIRE(ctx, d->batch >= 0 && d->m >= 0 && d->n >= 0 && d->k >= 0, "wdc_gemm: negative shape");
  if (d->batch * d->m * d->n == 0) return WDC_OK;
  WDC_REQUIRE(ctx, Y && (d->k == 0 || (A && B)), "wdc_gemm: null buffer");
  DeviceGuard g(ctx->device);
  ProfScope prof(ctx, 2.0 * (double)d->batch * (double)d->m * (double)d->n * (double)d->k);
  // Y = alpha*A*B + beta*Y (C aliasing the output) is served by the CUDA-core kernel's in-place mode only
  int s = (C != nullptr && C == Y) ? WDC_ERR_UNSUPPORTED : wdc_tc_gemm(ctx, d, A, B, C, Y);
  if (s != WDC_ERR_UNSUPPORTED) return s;
  return wdc_simt_gemm(ctx, d, A, B, C, Y);
}

extern "C" int wdc_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w,
                          const float* scale, const float* shift, const float* residual, float* y) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_conv2d: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, d != nullptr, "wdc_conv2d: null descriptor");
  WDC_REQUIRE(ctx, d->batch >= 0 && d->ch_in > 0 && d->ch_out > 0 && d->in_h > 0 && d->in_w > 0 &&
                       d->k_h > 0 && d->k_w > 0 && d->stride_h > 0 && d->stride_w > 0 && d->dil_h > 0 &&
                       d->dil_w > 0 && d->group > 0 && d->out_h >= 0 && d->out_w >= 0,
              "wdc_conv2d: bad shape");
  WDC_REQUIRE(ctx, d->ch_in % d->group == 0 && d->ch_out % d->group == 0,
              "wdc_conv2d: channels (%lld, %lld) not divisible by group %lld", (long long)d->ch_in,
              (long long)d->ch_out, (long long)d->group);
  if (d->batch * d->out_h * d->out_w == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && w && y, "wdc_conv2d: null buffer");
  DeviceGuard g(ctx->device);
  ProfScope prof(ctx, 2.0 * (double)d->batch * (double)d->out_h * (double)d->out_w * (double)d->ch_out *
                          (double)(d->ch_in / d->group) * (double)d->k_h * (double)d->k_w);
  int s = wdc_tc_conv2d(ctx, d, x, w, scale, shift, residual, y);
  if (s != WDC_ERR_UNSUPPORTED) return s;
  if (d->x_nchw)
    return wdc_fail(ctx, WDC_ERR_UNSUPPORTED, "wdc_conv2d: an NCHW input is only taken by the first-layer path "
                    "(ch_in <= 4, k_w <= 8, ch_out %% 4 == 0, group 1)");
  return wdc_simt_conv2d(ctx, d, x, w, scale, shift, residual, y);
}

__global__ void pack_conv_weight_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                        int64_t ch_out, int64_t cig, int64_t khw) {
  int64_t n = ch_out * cig * khw;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    // dst index (co, tap, ci)
    int64_t ci = i % cig, tap = (i / cig) % khw, co = i / (cig * khw);
    dst[i] = src[(co * cig + ci) * khw + tap];
  }
}

extern "C" int wdc_pack_conv_weight(wdc_context* ctx, const float* w_onnx, float* w_packed, int64_t ch_out,
                                    int64_t cig, int64_t k_h, int64_t k_w) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_pack_conv_weight: null context");
  wdc_note_write(ctx, w_packed);
  WDC_REQUIRE(ctx, ch_out > 0 && cig > 0 && k_h > 0 && k_w > 0 && w_onnx && w_packed,
              "wdc_pack_conv_weight: bad argument");
  DeviceGuard g(ctx->device);
  int64_t n = ch_out * cig * k_h * k_w;
  pack_conv_weight_kernel<<<grid_for(ctx, n, 256, 8), 256, 0, ctx->stream>>>(w_onnx, w_packed, ch_out, cig,
                                                                            k_h * k_w);
  return wdc_check_launch(ctx, "pack_conv_weight_kernel");
}
