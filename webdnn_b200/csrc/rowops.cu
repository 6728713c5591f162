// Row-wise kernels: softmax, single-axis reductions, layer normalisation, argmax.
// Each row is owned by one warp (rows up to 1024 elements are held in registers so the input is
// read from HBM exactly once) or by one CTA (longer rows, re-read through L2).
#include <math.h>

#include "common.cuh"

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------ softmax
// operators/cpu/operators/standard/softmax.ts:39-57: max, exp(v - max), sum, divide.
template <int ITEMS>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const float* __restrict__ x,
                                                           float* __restrict__ y, int64_t outer,
                                                           int len) {
  int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int64_t rstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (; row < outer; row += rstep) {
    const float* xr = x + row * len;
    float v[ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      int c = i * 32 + lane;
      v[i] = c < len ? xr[c] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      int c = i * 32 + lane;
      v[i] = c < len ? expf(v[i] - mx) : 0.f;
      s += v[i];
    }
    s = warp_sum(s);
    const float inv = 1.f / s;   // one division per row; e * (1 / s) is within an ulp of e / s
    float* yr = y + row * len;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      int c = i * 32 + lane;
      if (c < len) yr[c] = v[i] * inv;
    }
  }
}

__global__ void __launch_bounds__(512) softmax_block_kernel(const float* __restrict__ x,
                                                            float* __restrict__ y, int64_t outer,
                                                            int64_t len) {
  __shared__ float red[32];
  __shared__ float bcast;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    const float* xr = x + row * len;
    float* yr = y + row * len;
    float mx = -INFINITY;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) mx = fmaxf(mx, xr[c]);
    mx = warp_max(mx);
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    if (wid == 0) {
      float t = lane < nw ? red[lane] : -INFINITY;
      t = warp_max(t);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    mx = bcast;
    float s = 0.f;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
      float e = expf(xr[c] - mx);
      yr[c] = e;
      s += e;
    }
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) red[wid] = s;
    __syncthreads();
    if (wid == 0) {
      float t = lane < nw ? red[lane] : 0.f;
      t = warp_sum(t);
      if (lane == 0) bcast = t;
    }
    __syncthreads();
    s = 1.f / bcast;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) yr[c] = yr[c] * s;
    __syncthreads();
  }
}

// Rows of 1025 .. 256 * ITEMS elements: one CTA of 256 threads holds the row in registers (ITEMS per thread), so
// the input is read from HBM once and the output written once, like the warp kernel does for short rows.
__device__ __forceinline__ float block_reduce_f(float v, float* red, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();                 // red may still be read from the previous reduction
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < (int)(blockDim.x >> 5); i++) t = is_max ? fmaxf(t, red[i]) : t + red[i];   // same order in every thread
  return t;
}
template <int ITEMS>
__global__ void __launch_bounds__(256) softmax_block_reg_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                int64_t outer, int len) {
  __shared__ float red[8];
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    const float* xr = x + row * len;
    float v[ITEMS];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      v[i] = c < len ? xr[c] : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
    mx = block_reduce_f(mx, red, true);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      v[i] = c < len ? expf(v[i] - mx) : 0.f;
      s += v[i];
    }
    s = block_reduce_f(s, red, false);
    const float inv = 1.f / s;
    float* yr = y + row * len;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      if (c < len) yr[c] = v[i] * inv;
    }
  }
}

extern "C" int wdc_softmax(wdc_context* ctx, const float* x, float* y, int64_t outer, int64_t len) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_softmax: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, outer >= 0 && len >= 0, "wdc_softmax: negative shape");
  if (outer == 0 || len == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && y, "wdc_softmax: null buffer");
  DeviceGuard g(ctx->device);
  if (len <= 1024) {
    int wpb = 8;
    int grid = grid_for(ctx, outer * 32, wpb * 32, 8);
    int l = (int)len;
#define SM(IT) softmax_warp_kernel<IT><<<grid, wpb * 32, 0, ctx->stream>>>(x, y, outer, l)
    if (len <= 32) SM(1);
    else if (len <= 128) SM(4);
    else if (len <= 256) SM(8);
    else if (len <= 512) SM(16);
    else if (len <= 640) SM(20);
    else if (len <= 768) SM(24);
    else SM(32);
#undef SM
    return wdc_check_launch(ctx, "softmax_warp_kernel");
  }
  if (len <= 256 * 32) {
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    const int grid = (int)(outer < cap ? outer : cap);
    const int l = (int)len;
    if (len <= 256 * 8) softmax_block_reg_kernel<8><<<grid, 256, 0, ctx->stream>>>(x, y, outer, l);
    else if (len <= 256 * 16) softmax_block_reg_kernel<16><<<grid, 256, 0, ctx->stream>>>(x, y, outer, l);
    else softmax_block_reg_kernel<32><<<grid, 256, 0, ctx->stream>>>(x, y, outer, l);
    return wdc_check_launch(ctx, "softmax_block_reg_kernel");
  }
  int grid = (int)(outer < (int64_t)ctx->sm_count * 4 ? outer : (int64_t)ctx->sm_count * 4);
  softmax_block_kernel<<<grid, 512, 0, ctx->stream>>>(x, y, outer, len);
  return wdc_check_launch(ctx, "softmax_block_kernel");
}

// ------------------------------------------------------------------------------- reduce
// One pass of operators/cpu/operators/standard/reduce.ts:41-103 over [outer, red, inner].
// Sums are accumulated in double like the reference's JS numbers; the reference's per-pass
// application of abs/square/exp and its ReduceLogSum indexing (reduce.ts:288-312) are kept.
enum { R_SUM = 0, R_MEAN, R_MAX, R_MIN, R_PROD, R_L1, R_L2, R_LOGSUM, R_LOGSUMEXP, R_SUMSQUARE };

__device__ __forceinline__ double red_map(int kind, float v) {
  switch (kind) {
    case R_L1: return fabs((double)v);
    case R_L2:
    case R_SUMSQUARE: return (double)v * (double)v;
    case R_LOGSUMEXP: return exp((double)v);
    default: return (double)v;
  }
}
__device__ __forceinline__ double red_combine(int kind, double a, double b) {
  switch (kind) {
    case R_MAX: return b > a ? b : a;
    case R_MIN: return b < a ? b : a;
    case R_PROD: return a * b;
    default: return a + b;
  }
}
__device__ __forceinline__ double red_finish(int kind, int final, double s, int64_t total) {
  if (!final) return s;
  switch (kind) {
    case R_MEAN: return s / (double)total;
    case R_L2: return sqrt(s);
    case R_LOGSUM:
    case R_LOGSUMEXP: return log(s);
    default: return s;
  }
}

// inner == 1: one warp per output element, lanes stride the reduced axis.
__global__ void __launch_bounds__(256) reduce_rows_kernel(int kind, int final, const float* __restrict__ x,
                                                          float* __restrict__ y, int64_t outer,
                                                          int64_t red, int64_t total) {
  int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int64_t rstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (; row < outer; row += rstep) {
    const float* p = x + row * red;
    double ident = (kind == R_PROD) ? 1.0 : (kind == R_MAX ? -INFINITY : (kind == R_MIN ? INFINITY : 0.0));
    double s = ident;
    for (int64_t r = lane; r < red; r += 32) s = red_combine(kind, s, red_map(kind, p[r]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s = red_combine(kind, s, __shfl_xor_sync(0xffffffffu, s, o));
    if (lane == 0) y[row] = (float)red_finish(kind, final, s, total);
  }
}

// inner > 1: one thread per (outer, inner) output, coalesced across inner.
__global__ void __launch_bounds__(256) reduce_cols_kernel(int kind, int final, const float* __restrict__ x,
                                                          float* __restrict__ y, int64_t outer,
                                                          int64_t red, int64_t inner, int64_t total) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  int64_t n = outer * inner;
  for (; i < n; i += step) {
    int64_t o = i / inner, in = i % inner;
    const float* p = x + o * red * inner + in;
    double s;
    if (kind == R_LOGSUM) {
      s = 0;
      for (int64_t r = 0; r < red; r++) s += (double)x[o * red + r];
    } else if (kind == R_MAX || kind == R_MIN) {
      // an empty axis: the reference starts from element 0, which does not exist (undefined -> NaN in the typed array)
      s = red > 0 ? (double)p[0] : (double)NAN;
      for (int64_t r = 1; r < red; r++) s = red_combine(kind, s, (double)p[r * inner]);
    } else {
      s = (kind == R_PROD) ? 1.0 : 0.0;
      for (int64_t r = 0; r < red; r++) s = red_combine(kind, s, red_map(kind, p[r * inner]));
    }
    y[i] = (float)red_finish(kind, final, s, total);
  }
}

extern "C" int wdc_reduce_axis(wdc_context* ctx, int kind, int final, const float* x, float* y,
                               int64_t outer, int64_t red, int64_t inner, int64_t total) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_reduce_axis: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, kind >= R_SUM && kind <= R_SUMSQUARE, "wdc_reduce_axis: unknown kind %d", kind);
  WDC_REQUIRE(ctx, outer >= 0 && red >= 0 && inner >= 0, "wdc_reduce_axis: bad shape");
  if (outer == 0 || inner == 0) return WDC_OK;
  WDC_REQUIRE(ctx, y && (x || red == 0), "wdc_reduce_axis: null buffer");
  DeviceGuard g(ctx->device);
  if (inner == 1 && red >= 64) {
    reduce_rows_kernel<<<grid_for(ctx, outer * 32, 256, 8), 256, 0, ctx->stream>>>(kind, final, x, y,
                                                                                  outer, red, total);
    return wdc_check_launch(ctx, "reduce_rows_kernel");
  }
  reduce_cols_kernel<<<grid_for(ctx, outer * inner, 256, 8), 256, 0, ctx->stream>>>(
      kind, final, x, y, outer, red, inner, total);
  return wdc_check_launch(ctx, "reduce_cols_kernel");
}

// --------------------------------------------------------------------------- layer norm
// Equals the reference's decomposed chain ReduceMean -> Sub -> Mul(x,x) -> ReduceMean -> Add(eps)
// -> Sqrt -> Div -> Mul(gamma) -> Add(beta) with a float rounding after each node.
// Per-lane partial sums (at most 32 addends) are taken in fp32 and only the lanes' partials are added in double:
// converting every element to double made the conversion unit the limiter (63% of the HBM roofline for rows of
// 256); the result differs from the all-double sum by a few 1e-7 relative.  Two rows per warp iteration keep
// twice the loads in flight.
template <int ITEMS>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(const float* __restrict__ x,
                                                             const float* __restrict__ gamma,
                                                             const float* __restrict__ beta,
                                                             float* __restrict__ y, int64_t outer,
                                                             int len, float eps) {
  constexpr int R = ITEMS <= 8 ? 2 : 1;   // rows per warp iteration
  const double inv_len = 1.0 / (double)len;   // a double division per row costs more than the rest of the row
  int lane = threadIdx.x & 31;
  int64_t row0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
  int64_t rstep = (int64_t)gridDim.x * (blockDim.x >> 5) * R;
  for (; row0 < outer; row0 += rstep) {
    float v[R][ITEMS];
    float s[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const bool live = row0 + r < outer;
      const float* xr = x + (row0 + r) * len;
      s[r] = 0.f;
#pragma unroll
      for (int i = 0; i < ITEMS; i++) {
        int c = i * 32 + lane;
        v[r][i] = (live && c < len) ? xr[c] : 0.f;
        s[r] += v[r][i];
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
      if (row0 + r >= outer) continue;   // warp-uniform
      float mean = (float)(warp_sum_d((double)s[r]) * inv_len);
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < ITEMS; i++) {
        int c = i * 32 + lane;
        v[r][i] = v[r][i] - mean;                // Sub
        float sq = v[r][i] * v[r][i];            // Mul / Pow 2
        q += c < len ? sq : 0.f;
      }
      float var = (float)(warp_sum_d((double)q) * inv_len);  // ReduceMean
      float rden = 1.f / sqrtf(var + eps);                // Add, Sqrt; the Div as a multiplication (within an ulp)
      float* yr = y + (row0 + r) * len;
#pragma unroll
      for (int i = 0; i < ITEMS; i++) {
        int c = i * 32 + lane;
        if (c < len) {
          float o = v[r][i] * rden;              // Div
          if (gamma) o = o * gamma[c];           // Mul
          if (beta) o = o + beta[c];             // Add
          yr[c] = o;
        }
      }
    }
  }
}

// Rows longer than 1024 elements: one CTA of 256 threads per row, the row read three times (it stays in L2 / L1
// between the passes), the same rounding points as above.
__device__ __forceinline__ double block_sum_d(double v, double* scratch) {
  v = warp_sum_d(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();                 // scratch may still be read from the previous reduction
  if (lane == 0) scratch[w] = v;
  __syncthreads();
  double t = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += scratch[i];   // same order in every thread
  return t;
}
__global__ void __launch_bounds__(256) layernorm_block_kernel(const float* __restrict__ x,
                                                              const float* __restrict__ gamma,
                                                              const float* __restrict__ beta,
                                                              float* __restrict__ y, int64_t outer, int64_t len,
                                                              float eps) {
  __shared__ double scratch[8];
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    const float* xr = x + row * len;
    double s = 0;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) s += (double)xr[c];
    const float mean = (float)(block_sum_d(s, scratch) / (double)len);
    double q = 0;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
      const float d = xr[c] - mean;            // Sub
      const float sq = d * d;                  // Mul / Pow 2
      q += (double)sq;
    }
    const float var = (float)(block_sum_d(q, scratch) / (double)len);  // ReduceMean
    const float rden = 1.f / sqrtf(var + eps);                            // Add, Sqrt; Div as a multiplication
    float* yr = y + row * len;
    for (int64_t c = threadIdx.x; c < len; c += blockDim.x) {
      float r = (xr[c] - mean) * rden;         // Sub, Div
      if (gamma) r = r * gamma[c];             // Mul
      if (beta) r = r + beta[c];               // Add
      yr[c] = r;
    }
  }
}

// Rows of 1025 .. 256 * ITEMS elements with the row held in the CTA's registers (one read of x).
template <int ITEMS>
__global__ void __launch_bounds__(256) layernorm_block_reg_kernel(const float* __restrict__ x,
                                                                  const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta,
                                                                  float* __restrict__ y, int64_t outer, int len,
                                                                  float eps) {
  __shared__ double scratch[8];
  const double inv_len = 1.0 / (double)len;
  for (int64_t row = blockIdx.x; row < outer; row += gridDim.x) {
    const float* xr = x + row * len;
    float v[ITEMS];
    float s = 0.f;                             // per-thread partial (at most 32 addends) in fp32, then double
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      v[i] = c < len ? xr[c] : 0.f;
      s += v[i];
    }
    const float mean = (float)(block_sum_d((double)s, scratch) * inv_len);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      v[i] = v[i] - mean;                      // Sub
      const float sq = v[i] * v[i];            // Mul / Pow 2
      q += c < len ? sq : 0.f;
    }
    const float var = (float)(block_sum_d((double)q, scratch) * inv_len);  // ReduceMean
    const float rden = 1.f / sqrtf(var + eps);                            // Add, Sqrt; Div as a multiplication
    float* yr = y + row * len;
#pragma unroll
    for (int i = 0; i < ITEMS; i++) {
      const int c = i * 256 + threadIdx.x;
      if (c < len) {
        float r = v[i] * rden;                 // Div
        if (gamma) r = r * gamma[c];           // Mul
        if (beta) r = r + beta[c];             // Add
        yr[c] = r;
      }
    }
  }
}

extern "C" int wdc_layernorm(wdc_context* ctx, const float* x, const float* gamma, const float* beta,
                             float* y, int64_t outer, int64_t len, float eps) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_layernorm: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, outer >= 0 && len > 0, "wdc_layernorm: bad shape");
  if (outer == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && y, "wdc_layernorm: null buffer");
  DeviceGuard g(ctx->device);
  if (len > 1024 && len <= 256 * 32) {
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    const int grid = (int)(outer < cap ? outer : cap);
    const int l = (int)len;
    if (len <= 256 * 8) layernorm_block_reg_kernel<8><<<grid, 256, 0, ctx->stream>>>(x, gamma, beta, y, outer, l, eps);
    else if (len <= 256 * 16) layernorm_block_reg_kernel<16><<<grid, 256, 0, ctx->stream>>>(x, gamma, beta, y, outer, l, eps);
    else layernorm_block_reg_kernel<32><<<grid, 256, 0, ctx->stream>>>(x, gamma, beta, y, outer, l, eps);
    return wdc_check_launch(ctx, "layernorm_block_reg_kernel");
  }
  if (len > 1024) {
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    layernorm_block_kernel<<<(int)(outer < cap ? outer : cap), 256, 0, ctx->stream>>>(x, gamma, beta, y, outer, len, eps);
    return wdc_check_launch(ctx, "layernorm_block_kernel");
  }
  int grid = grid_for(ctx, outer * 32, 256, 8);
  int l = (int)len;
#define LN(IT) layernorm_warp_kernel<IT><<<grid, 256, 0, ctx->stream>>>(x, gamma, beta, y, outer, l, eps)
  if (len <= 32) LN(1);
  else if (len <= 128) LN(4);
  else if (len <= 256) LN(8);
  else if (len <= 512) LN(16);
  else LN(32);
#undef LN
  return wdc_check_launch(ctx, "layernorm_warp_kernel");
}

// ------------------------------------------------------------------------------- argmax
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ x, int32_t* __restrict__ y,
                                                     int64_t outer, int64_t len, int select_last) {
  int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  int64_t rstep = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (; row < outer; row += rstep) {
    const float* p = x + row * len;
    // NaN never wins a strict comparison; start from element 0 like a sequential scan
    float bv = p[0];
    int64_t bi = 0;
    for (int64_t r = lane; r < len; r += 32) {
      float v = p[r];
      if (v > bv || (v == bv && (select_last ? r > bi : r < bi))) {
        bv = v;
        bi = r;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && (select_last ? oi > bi : oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) y[row] = (int32_t)bi;
  }
}

extern "C" int wdc_argmax(wdc_context* ctx, const float* x, int32_t* y, int64_t outer, int64_t len,
                          int select_last) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_argmax: null context");
  wdc_note_write(ctx, y);
  WDC_REQUIRE(ctx, outer >= 0 && len > 0, "wdc_argmax: bad shape");
  if (outer == 0) return WDC_OK;
  WDC_REQUIRE(ctx, x && y, "wdc_argmax: null buffer");
  DeviceGuard g(ctx->device);
  argmax_kernel<<<grid_for(ctx, outer * 32, 256, 8), 256, 0, ctx->stream>>>(x, y, outer, len, select_last);
  return wdc_check_launch(ctx, "argmax_kernel");
}
