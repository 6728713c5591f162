// ConvTranspose and InstanceNormalization: operators of the reference's cpu backend that no benchmark
// configuration uses.  Both follow the reference's rounding points, not a fused formula, so that the
// results agree with its cpu backend to the last bit wherever the summation order allows.
#include <math.h>

#include "common.cuh"

// convtranspose.ts:30-263.  The reference computes, per input pixel, output channel and tap, the
// channel contraction in double and stores it as float32 (matmul, :218-240), then sums the taps that
// land on an output pixel in double and stores float32 (col2im, :139-196), then adds the bias
// (float32 + float32 -> float32).  One thread per output element does the same here.
// x [batch, group * cig, in_h, in_w]; w [group * cig, cog, k_h, k_w]; y [batch, group * cog, out_h, out_w].
__global__ void __launch_bounds__(256) conv_transpose2d_kernel(wdc_convt_desc d, const float* __restrict__ x,
                                                               const float* __restrict__ w,
                                                               const float* __restrict__ bias, float* __restrict__ y) {
  const int64_t cig = d.ch_in / d.group, cog = d.ch_out_per_group;
  const int64_t n = d.batch * d.group * cog * d.out_h * d.out_w;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    int64_t rem = i;
    const int64_t o1 = rem % d.out_w; rem /= d.out_w;
    const int64_t o0 = rem % d.out_h; rem /= d.out_h;
    const int64_t co = rem % cog; rem /= cog;
    const int64_t g = rem % d.group;
    const int64_t b = rem / d.group;
    double v = 0.0;
    for (int64_t k0 = 0; k0 < d.k_h; k0++) {
      const int64_t i0s = o0 + d.pad_t - k0 * d.dil_h;
      if (i0s % d.stride_h != 0) continue;
      const int64_t i0 = i0s / d.stride_h;
      if (i0 < 0 || i0 >= d.in_h) continue;
      for (int64_t k1 = 0; k1 < d.k_w; k1++) {
        const int64_t i1s = o1 + d.pad_l - k1 * d.dil_w;
        if (i1s % d.stride_w != 0) continue;
        const int64_t i1 = i1s / d.stride_w;
        if (i1 < 0 || i1 >= d.in_w) continue;
        double s = 0.0;
        for (int64_t ci = 0; ci < cig; ci++) {
          const float xv = x[((b * d.ch_in + g * cig + ci) * d.in_h + i0) * d.in_w + i1];
          const float wv = w[(((g * cig + ci) * cog + co) * d.k_h + k0) * d.k_w + k1];
          s += (double)xv * (double)wv;
        }
        v += (double)(float)s;
      }
    }
    float out = (float)v;
    if (bias) out = out + bias[g * cog + co];
    y[i] = out;
  }
}

// ---- the reference's own two steps (matmul, then col2im) on the device, for group 1 ----------------------
// col[(b, iy, ix), (ky, kx, co)] = sum_ci x[b, ci, iy, ix] * w[ci, co, ky, kx] is one tensor-core GEMM over the
// input pixels; col2im then sums, for every output element, the taps that land on it (in double, stored as
// float32, bias added in float32: the reference's rounding points, convtranspose.ts:139-196).  A 32 x 32
// (output column x channel) tile goes through shared memory so that col is read along co and y written along ox.
__global__ void __launch_bounds__(256) convt_col2im_kernel(wdc_convt_desc d, const float* __restrict__ col,
                                                           const float* __restrict__ bias, float* __restrict__ y) {
  __shared__ float tile[32][33];   // [ox][co]
  const int cog = (int)d.ch_out_per_group;
  const int64_t N = (int64_t)cog * d.k_h * d.k_w;
  const int tiles_x = (int)((d.out_w + 31) / 32), tiles_c = (cog + 31) / 32;
  const int64_t total = d.batch * d.out_h * tiles_x * tiles_c;
  const int cl = threadIdx.x & 31, sub = threadIdx.x >> 5;   // 32 x 8
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    int64_t rem = t;
    const int tc = (int)(rem % tiles_c); rem /= tiles_c;
    const int tx = (int)(rem % tiles_x); rem /= tiles_x;
    const int oy = (int)(rem % d.out_h);
    const int64_t b = rem / d.out_h;
    const int co = tc * 32 + cl;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int oxl = sub + 8 * j, ox = tx * 32 + oxl;
      double v = 0.0;
      if (co < cog && ox < d.out_w) {
        for (int ky = 0; ky < d.k_h; ky++) {
          const int i0s = oy + (int)d.pad_t - ky * (int)d.dil_h;
          if (i0s < 0 || i0s % (int)d.stride_h != 0) continue;
          const int iy = i0s / (int)d.stride_h;
          if (iy >= d.in_h) continue;
          for (int kx = 0; kx < d.k_w; kx++) {
            const int i1s = ox + (int)d.pad_l - kx * (int)d.dil_w;
            if (i1s < 0 || i1s % (int)d.stride_w != 0) continue;
            const int ix = i1s / (int)d.stride_w;
            if (ix >= d.in_w) continue;
            v += (double)__ldg(col + ((b * d.in_h + iy) * d.in_w + ix) * N + (int64_t)(ky * d.k_w + kx) * cog + co);
          }
        }
      }
      float out = (float)v;
      if (bias && co < cog) out = out + __ldg(bias + co);
      tile[oxl][cl] = out;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int c2 = tc * 32 + sub + 8 * j, ox = tx * 32 + cl;
      if (c2 < cog && ox < d.out_w) y[((b * cog + c2) * d.out_h + oy) * d.out_w + ox] = tile[cl][sub + 8 * j];
    }
    __syncthreads();
  }
}

static int conv_transpose_by_gemm(wdc_context* ctx, const wdc_convt_desc* d, const float* x, const float* w,
                                  const float* bias, float* y) {
  const int64_t cin = d->ch_in, cog = d->ch_out_per_group, taps = d->k_h * d->k_w;
  const int64_t pix = d->in_h * d->in_w, M = d->batch * pix, N = cog * taps;
  float* scratch = nullptr;
  int s = wdc_alloc(ctx, (M * cin + cin * N + M * N) * 4, (void**)&scratch);
  if (s != WDC_OK) return s;
  float *xt = scratch, *wp = xt + M * cin, *col = wp + cin * N;
  {   // x [b, cin, pix] -> xt [b, pix, cin]
    const int64_t dims[3] = {d->batch, pix, cin}, ss[3] = {cin * pix, 1, pix}, ds[3] = {pix * cin, cin, 1};
    s = wdc_strided_copy(ctx, x, xt, 3, dims, ss, 0, ds, 0);
  }
  if (s == WDC_OK && d->w_layout == 0) {   // w [cin, cog, taps] -> wp [cin, taps, cog]
    const int64_t dims[3] = {cin, taps, cog}, ss[3] = {cog * taps, 1, taps}, ds[3] = {taps * cog, cog, 1};
    s = wdc_strided_copy(ctx, w, wp, 3, dims, ss, 0, ds, 0);
  }
  if (d->w_layout == 1) wp = const_cast<float*>(w);   // the caller's own re-laid-out copy: its split stays cached
  if (s == WDC_OK) {
    wdc_gemm_desc g = {};
    g.batch = 1; g.m = M; g.n = N; g.k = cin;
    g.sa0 = cin; g.sa1 = 1; g.sb0 = N; g.sb1 = 1;
    g.alpha = 1.f; g.beta = 0.f;
    s = wdc_gemm(ctx, &g, xt, wp, nullptr, col);
  }
  if (s == WDC_OK) {
    const int64_t blocks = d->batch * d->out_h * ((d->out_w + 31) / 32) * ((cog + 31) / 32);
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    convt_col2im_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(*d, col, bias, y);
    s = wdc_check_launch(ctx, "convt_col2im_kernel");
  }
  wdc_free(ctx, scratch);   // stream-ordered
  return s;
}

extern "C" int wdc_conv_transpose2d(wdc_context* ctx, const wdc_convt_desc* d, const float* x, const float* w,
                                    const float* bias, float* y) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_conv_transpose2d: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, d != nullptr, "wdc_conv_transpose2d: null descriptor");
  WDC_REQUIRE(ctx, d->batch >= 0 && d->ch_in > 0 && d->group > 0 && d->ch_out_per_group > 0 && d->in_h > 0 &&
                       d->in_w > 0 && d->k_h > 0 && d->k_w > 0 && d->out_h >= 0 && d->out_w >= 0 && d->stride_h > 0 &&
                       d->stride_w > 0 && d->dil_h > 0 && d->dil_w > 0 && d->ch_in % d->group == 0 &&
                       (d->w_layout == 0 || d->w_layout == 1),
              "wdc_conv_transpose2d: bad shape");
  const int64_t n = d->batch * d->group * d->ch_out_per_group * d->out_h * d->out_w;
  if (n == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && w && y, "wdc_conv_transpose2d: null buffer");
  DeviceGuard g(ctx->device);
  // enough work for the tensor cores and shapes the contraction kernel takes: matmul + col2im; else one thread
  // per output element
  const int64_t M = d->batch * d->in_h * d->in_w, N = d->ch_out_per_group * d->k_h * d->k_w;
  if (d->group == 1 && d->ch_in % 4 == 0 && d->ch_in >= 32 && N % 4 == 0 && M >= 128 &&
      M * N < (1ll << 40) && d->out_w < (1ll << 30) && d->out_h < (1ll << 30))
    return conv_transpose_by_gemm(ctx, d, x, w, bias, y);
  WDC_REQUIRE(ctx, d->w_layout == 0, "wdc_conv_transpose2d: w_layout 1 is only taken by the tensor-core route");
  conv_transpose2d_kernel<<<grid_for(ctx, n, 256, 8), 256, 0, ctx->stream>>>(*d, x, w, bias, y);
  return wdc_check_launch(ctx, "conv_transpose2d_kernel");
}

// instancenormalization.ts:24-53: per (batch, channel) row of `area` elements, sum and sum of squares
// in double, mean = sum / area, variance = sqsum / area - mean^2, invstd = 1 / sqrt(variance + eps),
// y = x * (scale * invstd) + (bias - mean * scale * invstd), all in double, stored as float32.
// One block per row; the double sums are combined in a fixed tree, so the result does not depend on
// the launch (it can differ from the reference's left-to-right sum in the last bit of the double).
__global__ void __launch_bounds__(256) instance_norm_kernel(const float* __restrict__ x, const float* __restrict__ scale,
                                                            const float* __restrict__ bias, float* __restrict__ y,
                                                            int64_t rows, int64_t ch, int64_t area, double eps) {
  __shared__ double s_sum[256], s_sq[256];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float* xr = x + row * area;
    double sum = 0.0, sq = 0.0;
    for (int64_t r = threadIdx.x; r < area; r += blockDim.x) {
      const double v = (double)xr[r];
      sum += v;
      sq += v * v;
    }
    s_sum[threadIdx.x] = sum;
    s_sq[threadIdx.x] = sq;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if ((int)threadIdx.x < o) {
        s_sum[threadIdx.x] += s_sum[threadIdx.x + o];
        s_sq[threadIdx.x] += s_sq[threadIdx.x + o];
      }
      __syncthreads();
    }
    const double mean = s_sum[0] / (double)area;
    const double variance = s_sq[0] / (double)area - mean * mean;
    const double invstd = 1.0 / sqrt(variance + eps);
    const int64_t c = row % ch;
    const double chscale = (double)scale[c] * invstd;
    const double chbias = -mean * chscale + (double)bias[c];
    float* yr = y + row * area;
    for (int64_t r = threadIdx.x; r < area; r += blockDim.x) yr[r] = (float)((double)xr[r] * chscale + chbias);
    __syncthreads();
  }
}

extern "C" int wdc_instance_norm(wdc_context* ctx, const float* x, const float* scale, const float* bias, float* y,
                                 int64_t batch, int64_t ch, int64_t area, double eps) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_instance_norm: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, batch >= 0 && ch > 0 && area > 0, "wdc_instance_norm: bad shape");
  if (batch == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && scale && bias && y, "wdc_instance_norm: null buffer");
  DeviceGuard g(ctx->device);
  const int64_t rows = batch * ch;
  const int64_t cap = (int64_t)ctx->sm_count * 8;
  instance_norm_kernel<<<(int)(rows < cap ? rows : cap), 256, 0, ctx->stream>>>(x, scale, bias, y, rows, ch, area, eps);
  return wdc_check_launch(ctx, "instance_norm_kernel");
}
