// Pooling kernels.  Tensors are addressed through (n, c, h, w) element strides so that the
// channels-last tensors the convolution path produces and canonical NCHW tensors share the code.
// When channels are innermost (stride 1) and a multiple of 4, each thread handles 4 channels with
// 128-bit accesses.
#include <math.h>

#include "common.cuh"

template <bool IS_MAX, int VEC>
__global__ void __launch_bounds__(256) pool2d_kernel(wdc_pool_desc d, const float* __restrict__ x,
                                                     float* __restrict__ y, int c_fastest) {
  int64_t chv = d.ch / VEC;
  int64_t n = d.batch * chv * d.out_h * d.out_w;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    int64_t b, c, oy, ox, rem = i;
    if (c_fastest) {  // consecutive threads walk channels: coalesced for channels-last tensors
      c = (rem % chv) * VEC; rem /= chv;
      ox = rem % d.out_w; rem /= d.out_w;
      oy = rem % d.out_h; rem /= d.out_h;
      b = rem;
    } else {          // consecutive threads walk output columns: coalesced for NCHW
      ox = rem % d.out_w; rem /= d.out_w;
      oy = rem % d.out_h; rem /= d.out_h;
      c = (rem % chv) * VEC; rem /= chv;
      b = rem;
    }
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) acc[v] = IS_MAX ? -INFINITY : 0.f;
    double dacc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) dacc[v] = 0.0;
    int ctr = 0;
    for (int64_t ky = 0; ky < d.k_h; ky++) {
      int64_t iny = oy * d.stride_h - d.pad_t + ky * d.dil_h;
      if (iny < 0 || iny >= d.in_h) continue;
      for (int64_t kx = 0; kx < d.k_w; kx++) {
        int64_t inx = ox * d.stride_w - d.pad_l + kx * d.dil_w;
        if (inx < 0 || inx >= d.in_w) continue;
        const float* p = x + b * d.xs_n + c * d.xs_c + iny * d.xs_h + inx * d.xs_w;
        float val[VEC];
        if (VEC == 4) {
          float4 t = __ldg(reinterpret_cast<const float4*>(p));
          val[0] = t.x; val[1 % VEC] = t.y; val[2 % VEC] = t.z; val[3 % VEC] = t.w;
        } else {
          val[0] = __ldg(p);
        }
#pragma unroll
        for (int v = 0; v < VEC; v++) {
          if (IS_MAX) {
            if (val[v] > acc[v]) acc[v] = val[v];  // strict >, NaN never wins (maxpool.ts:96)
          } else {
            dacc[v] += (double)val[v];
          }
        }
        ctr++;
      }
    }
    float out[VEC];
#pragma unroll
    for (int v = 0; v < VEC; v++) {
      if (IS_MAX) out[v] = acc[v];
      else out[v] = (float)(d.count_include_pad ? dacc[v] / (double)(d.k_h * d.k_w) : dacc[v] / (double)ctr);
    }
    float* q = y + b * d.ys_n + c * d.ys_c + oy * d.ys_h + ox * d.ys_w;
    if (VEC == 4) *reinterpret_cast<float4*>(q) = make_float4(out[0], out[1 % VEC], out[2 % VEC], out[3 % VEC]);
    else *q = out[0];
  }
}

// Channels-last max pool with a window of at most 3x3 (dilation 1), dense NHWC on both sides, fewer
// than 2^31 elements: 32-bit index arithmetic, and the window's loads are issued together (out-of-
// image taps re-read the clamped pixel with a -inf substitute) before any comparison.
// One thread = 4 channels of one output pixel.
template <int KH, int KW>
__global__ void __launch_bounds__(256) maxpool_cl_small_kernel(const float4* __restrict__ x, float4* __restrict__ y,
                                                               int n_out, int chv, int in_h, int in_w, int out_h,
                                                               int out_w, int stride_h, int stride_w, int pad_t,
                                                               int pad_l) {
  const int step = gridDim.x * blockDim.x;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_out; i += step) {
    int rem = i;
    const int c = rem % chv; rem /= chv;
    const int ox = rem % out_w; rem /= out_w;
    const int oy = rem % out_h;
    const int b = rem / out_h;
    const int iy0 = oy * stride_h - pad_t, ix0 = ox * stride_w - pad_l;
    float4 v[KH * KW];
    bool in[KH * KW];
#pragma unroll
    for (int ky = 0; ky < KH; ky++) {
#pragma unroll
      for (int kx = 0; kx < KW; kx++) {
        const int iy = iy0 + ky, ix = ix0 + kx;
        const bool ok = (unsigned)iy < (unsigned)in_h && (unsigned)ix < (unsigned)in_w;
        const int cy = min(max(iy, 0), in_h - 1), cx = min(max(ix, 0), in_w - 1);
        in[ky * KW + kx] = ok;
        v[ky * KW + kx] = __ldg(x + ((size_t)(b * in_h + cy) * in_w + cx) * chv + c);
      }
    }
    float4 m = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
    for (int t = 0; t < KH * KW; t++) {
      if (in[t]) {  // strict >, NaN never wins (maxpool.ts:96)
        if (v[t].x > m.x) m.x = v[t].x;
        if (v[t].y > m.y) m.y = v[t].y;
        if (v[t].z > m.z) m.z = v[t].z;
        if (v[t].w > m.w) m.w = v[t].w;
      }
    }
    y[i] = m;
  }
}

static int pool_common(wdc_context* ctx, const wdc_pool_desc* d, const float* x, float* y, bool is_max,
                       const char* who) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "%s: null context", who);
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, d != nullptr, "%s: null descriptor", who);
  WDC_REQUIRE(ctx, d->batch >= 0 && d->ch >= 0 && d->in_h > 0 && d->in_w > 0 && d->out_h >= 0 &&
                       d->out_w >= 0 && d->k_h > 0 && d->k_w > 0 && d->stride_h > 0 && d->stride_w > 0 &&
                       d->dil_h > 0 && d->dil_w > 0,
              "%s: bad shape", who);
  int64_t n = d->batch * d->ch * d->out_h * d->out_w;
  if (n == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && y, "%s: null buffer", who);
  DeviceGuard g(ctx->device);
  bool cl = d->xs_c == 1 && d->ys_c == 1;
  bool vec = cl && d->ch % 4 == 0 && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0) && d->xs_n % 4 == 0 &&
             d->xs_h % 4 == 0 && d->xs_w % 4 == 0 && d->ys_n % 4 == 0 && d->ys_h % 4 == 0 && d->ys_w % 4 == 0;
  int64_t items = vec ? n / 4 : n;
  int grid = grid_for(ctx, items, 256, 8);
  const bool dense = d->xs_w == d->ch && d->xs_h == d->in_w * d->ch && d->xs_n == d->in_h * d->in_w * d->ch &&
                     d->ys_w == d->ch && d->ys_h == d->out_w * d->ch && d->ys_n == d->out_h * d->out_w * d->ch;
  if (is_max && vec && dense && d->dil_h == 1 && d->dil_w == 1 && d->k_h == d->k_w && (d->k_h == 2 || d->k_h == 3) &&
      d->batch * d->in_h * d->in_w * d->ch < (1ll << 31) && n < (1ll << 31)) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* y4 = reinterpret_cast<float4*>(y);
#define WDC_POOL_ARGS (int)items, (int)(d->ch / 4), (int)d->in_h, (int)d->in_w, (int)d->out_h, (int)d->out_w, \
                      (int)d->stride_h, (int)d->stride_w, (int)d->pad_t, (int)d->pad_l
    if (d->k_h == 3) maxpool_cl_small_kernel<3, 3><<<grid, 256, 0, ctx->stream>>>(x4, y4, WDC_POOL_ARGS);
    else maxpool_cl_small_kernel<2, 2><<<grid, 256, 0, ctx->stream>>>(x4, y4, WDC_POOL_ARGS);
#undef WDC_POOL_ARGS
    return wdc_check_launch(ctx, "maxpool_cl_small_kernel");
  }
  if (is_max) {
    if (vec) pool2d_kernel<true, 4><<<grid, 256, 0, ctx->stream>>>(*d, x, y, 1);
    else pool2d_kernel<true, 1><<<grid, 256, 0, ctx->stream>>>(*d, x, y, cl ? 1 : 0);
  } else {
    if (vec) pool2d_kernel<false, 4><<<grid, 256, 0, ctx->stream>>>(*d, x, y, 1);
    else pool2d_kernel<false, 1><<<grid, 256, 0, ctx->stream>>>(*d, x, y, cl ? 1 : 0);
  }
  return wdc_check_launch(ctx, "pool2d_kernel");
}

extern "C" int wdc_maxpool2d(wdc_context* ctx, const wdc_pool_desc* d, const float* x, float* y) {
  return pool_common(ctx, d, x, y, true, "wdc_maxpool2d");
}
extern "C" int wdc_avgpool2d(wdc_context* ctx, const wdc_pool_desc* d, const float* x, float* y) {
  return pool_common(ctx, d, x, y, false, "wdc_avgpool2d");
}

// Global average pool.  Channels-last: one thread per (b, c), walking pixels with stride xs_p,
// coalesced across c.  NCHW: one warp per (b, c), lanes stride the pixels.
__global__ void __launch_bounds__(256) gap_cl_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                     int64_t batch, int64_t ch, int64_t area,
                                                     int64_t xs_n, int64_t xs_p) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < batch * ch; i += step) {
    int64_t b = i / ch, c = i % ch;
    const float* p = x + b * xs_n + c;
    double s = 0;
    for (int64_t a = 0; a < area; a++) s += (double)__ldg(p + a * xs_p);
    y[i] = (float)(s / (double)area);
  }
}

__global__ void __launch_bounds__(256) gap_warp_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                       int64_t batch, int64_t ch, int64_t area,
                                                       int64_t xs_n, int64_t xs_c, int64_t xs_p) {
  int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int64_t rstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (; row < batch * ch; row += rstep) {
    int64_t b = row / ch, c = row % ch;
    const float* p = x + b * xs_n + c * xs_c;
    double s = 0;
    for (int64_t a = lane; a < area; a += 32) s += (double)__ldg(p + a * xs_p);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) y[row] = (float)(s / (double)area);
  }
}

// Short rows (a 7x7 map has 49 pixels): a whole warp per row leaves most lanes idle and one short load in flight,
// so L lanes (4, 8 or 16) share a row and a warp works on 32 / L rows at once.  All of a row's loads are issued
// before the first addition (up to 8 per lane), which is what keeps enough bytes in flight per SM.
template <int L>
__global__ void __launch_bounds__(256) gap_group_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                        int64_t rows, int64_t ch, int area, int64_t xs_n,
                                                        int64_t xs_c, int64_t xs_p) {
  constexpr int R = 2;                                   // rows per lane group and iteration: twice the loads in flight
  const int gl = threadIdx.x % L;
  const int64_t gid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / L;
  const int64_t gstep = (int64_t)gridDim.x * blockDim.x / L;
  const int64_t iters = (rows + R * gstep - 1) / (R * gstep);   // the same for every lane: the shuffles need the whole warp
  const double inv_area = 1.0 / (double)area;
  for (int64_t it = 0; it < iters; it++) {
    float v[R][8];
    int64_t row[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      row[r] = gid + (it * R + r) * gstep;
      const bool valid = row[r] < rows;
      // rows of consecutive channels and images are equally spaced in a dense tensor (xs_n == ch * xs_c): no
      // division then, and a 32-bit one otherwise (a 64-bit division costs more than the row's seven loads)
      const float* p = x;
      if (valid) {
        if (xs_n == ch * xs_c) p = x + row[r] * xs_c;
        else {
          const uint32_t b = (uint32_t)row[r] / (uint32_t)ch, c = (uint32_t)row[r] - b * (uint32_t)ch;
          p = x + (int64_t)b * xs_n + (int64_t)c * xs_c;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int a = gl + u * L;
        v[r][u] = (valid && a < area) ? __ldg(p + (int64_t)a * xs_p) : 0.f;
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
      double s = 0;
#pragma unroll
      for (int u = 0; u < 8; u++) s += (double)v[r][u];
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (row[r] < rows && gl == 0) y[row[r]] = (float)(s * inv_area);
    }
  }
}

// Dense NCHW maps of at most 96 pixels: the maps of consecutive (image, channel) pairs are one contiguous stretch of
// memory, so a CTA brings 128 of them into shared memory with full-width coalesced 16-byte loads (a 49-pixel map is
// 196 bytes: read map by map, no access is aligned) and 128 threads then add up one map each (a row stride of `area`
// words: conflict-free for odd areas, 2-way at worst for the even ones that matter).  Sums in double, like the others.
constexpr int GAP_MAPS = 128;
constexpr int GAP_MAX_AREA = 96;
__global__ void __launch_bounds__(GAP_MAPS) gap_dense_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                             int64_t rows, int area) {
  extern __shared__ __align__(16) float buf[];             // GAP_MAPS * area words: several CTAs per SM
  const double inv_area = 1.0 / (double)area;
  const int64_t chunks = (rows + GAP_MAPS - 1) / GAP_MAPS;
  for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    const int64_t row0 = c * GAP_MAPS;
    const int maps = (int)(rows - row0 < GAP_MAPS ? rows - row0 : GAP_MAPS);
    const int words = maps * area;
    const float* src = x + row0 * area;                    // 16-byte aligned: GAP_MAPS * area * 4 is a multiple of 16
    const int vec = words >> 2;
    // eight loads per thread in flight before the first store (a load-store loop would pay the memory latency
    // once per iteration)
    for (int base = 0; base < vec; base += GAP_MAPS * 8) {
      float4 r[8];
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * GAP_MAPS + (int)threadIdx.x;
        r[u] = i < vec ? __ldg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 8; u++) {
        const int i = base + u * GAP_MAPS + (int)threadIdx.x;
        if (i < vec) reinterpret_cast<float4*>(buf)[i] = r[u];
      }
    }
    for (int i = (vec << 2) + threadIdx.x; i < words; i += blockDim.x) buf[i] = __ldg(src + i);
    __syncthreads();
    if ((int)threadIdx.x < maps) {
      const float* m = buf + threadIdx.x * area;
      double s0 = 0, s1 = 0;
      int i = 0;
      for (; i + 1 < area; i += 2) {
        s0 += (double)m[i];
        s1 += (double)m[i + 1];
      }
      if (i < area) s0 += (double)m[i];
      y[row0 + threadIdx.x] = (float)((s0 + s1) * inv_area);
    }
    __syncthreads();
  }
}

extern "C" int wdc_global_avgpool(wdc_context* ctx, const float* x, float* y, int64_t batch, int64_t ch,
                                  int64_t area, int64_t xs_n, int64_t xs_c, int64_t xs_p) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_global_avgpool: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, batch >= 0 && ch >= 0 && area > 0, "wdc_global_avgpool: bad shape");
  if (batch * ch == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && y, "wdc_global_avgpool: null buffer");
  DeviceGuard g(ctx->device);
  if (xs_c == 1) {
    gap_cl_kernel<<<grid_for(ctx, batch * ch, 256, 8), 256, 0, ctx->stream>>>(x, y, batch, ch, area, xs_n, xs_p);
    return wdc_check_launch(ctx, "gap_cl_kernel");
  }
  if (area <= GAP_MAX_AREA && xs_p == 1 && xs_c == area && xs_n == ch * area && (((uintptr_t)x) & 15) == 0) {
    const int64_t rows = batch * ch;
    const int64_t chunks = (rows + GAP_MAPS - 1) / GAP_MAPS;
    const size_t smem = (size_t)GAP_MAPS * area * 4;       // 25 KB for 7x7 maps: eight CTAs per SM
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    gap_dense_kernel<<<(int)(chunks < cap ? chunks : cap), GAP_MAPS, smem, ctx->stream>>>(x, y, rows, (int)area);
    return wdc_check_launch(ctx, "gap_dense_kernel");
  }
  if (area <= 128 && batch * ch < (1ll << 31) && ch < (1ll << 31)) {
    const int64_t rows = batch * ch;
    const int a = (int)area;
    if (area <= 32) gap_group_kernel<4><<<grid_for(ctx, rows * 4, 256, 8), 256, 0, ctx->stream>>>(x, y, rows, ch, a, xs_n, xs_c, xs_p);
    else if (area <= 64) gap_group_kernel<8><<<grid_for(ctx, rows * 8, 256, 8), 256, 0, ctx->stream>>>(x, y, rows, ch, a, xs_n, xs_c, xs_p);
    else gap_group_kernel<16><<<grid_for(ctx, rows * 16, 256, 8), 256, 0, ctx->stream>>>(x, y, rows, ch, a, xs_n, xs_c, xs_p);
    return wdc_check_launch(ctx, "gap_group_kernel");
  }
  gap_warp_kernel<<<grid_for(ctx, batch * ch * 32, 256, 8), 256, 0, ctx->stream>>>(x, y, batch, ch, area,
                                                                                  xs_n, xs_c, xs_p);
  return wdc_check_launch(ctx, "gap_warp_kernel");
}
