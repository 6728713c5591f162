// Data-movement kernels on 4-byte elements: general strided copy (<= 6-D) with a tiled
// shared-memory path for batched 2-D transposes (the NCHW <-> NHWC conversions), and gather.
#include "common.cuh"

struct CopyShape {
  int64_t dims[6];
  int64_t sstr[6];
  int64_t dstr[6];
};

// M = number of axes in use (the last M slots of the shape); I = the type the element index is split in: 32-bit
// division where the element count allows it (a 64-bit division per axis and element made a head split run at 43%
// of the HBM copy rate).
template <typename T, int M, typename I>
__global__ void __launch_bounds__(256) strided_copy_kernel(const T* __restrict__ src, T* __restrict__ dst, int64_t n,
                                                           CopyShape sh) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  I dims[M];
#pragma unroll
  for (int d = 0; d < M; d++) dims[d] = (I)sh.dims[6 - M + d];
  for (; i < n; i += step) {
    I rem = (I)i;
    int64_t is = 0, id = 0;
#pragma unroll
    for (int d = M - 1; d > 0; d--) {
      const I q = rem / dims[d];
      const I c = rem - q * dims[d];
      rem = q;
      is += (int64_t)c * sh.sstr[6 - M + d];
      id += (int64_t)c * sh.dstr[6 - M + d];
    }
    is += (int64_t)rem * sh.sstr[6 - M];
    id += (int64_t)rem * sh.dstr[6 - M];
    dst[id] = src[is];
  }
}

template <typename T>
static void launch_strided_copy(wdc_context* ctx, const T* s, T* d, int64_t n, const CopyShape& sh, int m) {
  const int grid = grid_for(ctx, n, 256, 8);
  const bool small = n < (1ll << 31);
#define WDC_COPY_CASE(MM)                                                                                   \
  case MM:                                                                                                  \
    if (small) strided_copy_kernel<T, MM, uint32_t><<<grid, 256, 0, ctx->stream>>>(s, d, n, sh);            \
    else strided_copy_kernel<T, MM, int64_t><<<grid, 256, 0, ctx->stream>>>(s, d, n, sh);                   \
    break;
  switch (m < 1 ? 1 : m) {
    WDC_COPY_CASE(1)
    WDC_COPY_CASE(2)
    WDC_COPY_CASE(3)
    WDC_COPY_CASE(4)
    WDC_COPY_CASE(5)
    default:
    WDC_COPY_CASE(6)
  }
#undef WDC_COPY_CASE
}

// dst[b][r][c] (dense, c innermost) <- src[b][c][r]: src element (b, r, c) at b*sb + c*rows + r.
// 32x32 tiles through shared memory (padded against bank conflicts): both sides coalesced.
__global__ void __launch_bounds__(256) transpose_tile_kernel(const uint32_t* __restrict__ src,
                                                             uint32_t* __restrict__ dst, int64_t batch,
                                                             int64_t rows, int64_t cols) {
  __shared__ uint32_t tile[32][33];
  int64_t tiles_r = (rows + 31) / 32, tiles_c = (cols + 31) / 32;
  int64_t ntiles = batch * tiles_r * tiles_c;
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    int64_t b = t / (tiles_r * tiles_c);
    int64_t rem = t % (tiles_r * tiles_c);
    int64_t r0 = (rem / tiles_c) * 32, c0 = (rem % tiles_c) * 32;
    const uint32_t* s = src + b * rows * cols;
    uint32_t* d = dst + b * rows * cols;
    // read: src is [cols][rows] with rows innermost
#pragma unroll
    for (int k = 0; k < 4; k++) {
      int64_t c = c0 + ty + k * 8, r = r0 + tx;
      if (c < cols && r < rows) tile[ty + k * 8][tx] = s[c * rows + r];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; k++) {
      int64_t r = r0 + ty + k * 8, c = c0 + tx;
      if (r < rows && c < cols) d[r * cols + c] = tile[tx][ty + k * 8];
    }
    __syncthreads();
  }
}

// The same transpose in 64x64 tiles with 16-byte accesses on both sides (rows and cols multiples of 4, 16-byte
// aligned buffers): a quarter of the memory instructions of the 32x32 kernel.  Shared-memory accesses are
// scalar with a pitch of 65 words: at most two-way bank conflicts on either side.
__global__ void __launch_bounds__(256) transpose_tile64_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                               int64_t batch, int64_t rows, int64_t cols) {
  __shared__ float tile[64][65];   // [c][r]
  const int64_t tiles_r = (rows + 63) / 64, tiles_c = (cols + 63) / 64;
  const int64_t ntiles = batch * tiles_r * tiles_c;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16
  for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const int64_t b = t / (tiles_r * tiles_c);
    const int64_t rem = t % (tiles_r * tiles_c);
    const int64_t r0 = (rem / tiles_c) * 64, c0 = (rem % tiles_c) * 64;
    const float* s = src + b * rows * cols;
    float* d = dst + b * rows * cols;
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {   // src is [cols][rows], rows innermost
      const int64_t c = c0 + ty + 16 * k, r = r0 + 4 * tx;
      v[k] = (c < cols && r < rows) ? __ldg(reinterpret_cast<const float4*>(s + c * rows + r))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float* p = &tile[ty + 16 * k][4 * tx];
      p[0] = v[k].x; p[1] = v[k].y; p[2] = v[k].z; p[3] = v[k].w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int rl = ty + 16 * k;
      const int64_t r = r0 + rl, c = c0 + 4 * tx;
      if (r < rows && c < cols)
        *reinterpret_cast<float4*>(d + r * cols + c) =
            make_float4(tile[4 * tx][rl], tile[4 * tx + 1][rl], tile[4 * tx + 2][rl], tile[4 * tx + 3][rl]);
    }
    __syncthreads();
  }
}

// Same transpose when one side is narrow (fewer than 8 columns or rows, e.g. the 3 channels of an
// image batch): one thread per position of the long axis, which is contiguous in src (narrow cols)
// or in dst (narrow rows), so that side is coalesced per step and the other is covered by the
// thread's short run of consecutive words.
__global__ void __launch_bounds__(256) transpose_narrow_cols_kernel(const uint32_t* __restrict__ src,
                                                                    uint32_t* __restrict__ dst, int64_t batch,
                                                                    int64_t rows, int cols) {
  int64_t n = batch * rows;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    int64_t b = i / rows, r = i - b * rows;
    const uint32_t* s = src + b * rows * cols + r;
    uint32_t* d = dst + i * cols;
    for (int c = 0; c < cols; c++) d[c] = __ldg(s + (int64_t)c * rows);
  }
}
__global__ void __launch_bounds__(256) transpose_narrow_rows_kernel(const uint32_t* __restrict__ src,
                                                                    uint32_t* __restrict__ dst, int64_t batch,
                                                                    int rows, int64_t cols) {
  int64_t n = batch * cols;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    int64_t b = i / cols, c = i - b * cols;
    const uint32_t* s = src + (b * cols + c) * rows;
    uint32_t* d = dst + b * rows * cols + c;
    for (int r = 0; r < rows; r++) d[(int64_t)r * cols] = __ldg(s + r);
  }
}

extern "C" int wdc_strided_copy(wdc_context* ctx, const void* src, void* dst, int ndim,
                                const int64_t* dims, const int64_t* sstr, int64_t src_off,
                                const int64_t* dstr, int64_t dst_off) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_strided_copy: null context");
  wdc_note_write(ctx, dst ? (const uint32_t*)dst + dst_off : nullptr);
  WDC_REQUIRE(ctx, ndim >= 0 && ndim <= 6, "wdc_strided_copy: rank %d not in 0..6", ndim);
  WDC_REQUIRE(ctx, ndim == 0 || (dims && sstr && dstr), "wdc_strided_copy: null shape");
  WDC_REQUIRE(ctx, src_off >= 0 && dst_off >= 0, "wdc_strided_copy: negative offset");
  // drop size-1 axes and merge axes that are contiguous on both sides
  int64_t md[6], ms[6], mt[6];
  int m = 0;
  int64_t n = 1;
  for (int i = 0; i < ndim; i++) {
    WDC_REQUIRE(ctx, dims[i] >= 0, "wdc_strided_copy: negative dim");
    n *= dims[i];
    if (dims[i] == 1) continue;
    if (m > 0 && ms[m - 1] == sstr[i] * dims[i] && mt[m - 1] == dstr[i] * dims[i]) {
      md[m - 1] *= dims[i];
      ms[m - 1] = sstr[i];
      mt[m - 1] = dstr[i];
    } else {
      md[m] = dims[i];
      ms[m] = sstr[i];
      mt[m] = dstr[i];
      m++;
    }
  }
  if (n == 0) return WDC_OK;
  WDC_REQUIRE(ctx, src && dst, "wdc_strided_copy: null buffer");
  DeviceGuard g(ctx->device);
  const uint32_t* s = (const uint32_t*)src + src_off;
  uint32_t* d = (uint32_t*)dst + dst_off;
  if (m == 0 || (m == 1 && ms[0] == 1 && mt[0] == 1)) return wdc_copy(ctx, d, s, n * 4);
  // batched 2-D transpose: dst dense [b][r][c], src [b][c][r]
  if ((m == 2 || m == 3) && mt[m - 1] == 1 && mt[m - 2] == md[m - 1] && ms[m - 2] == 1 &&
      ms[m - 1] == md[m - 2] && (m == 2 || (mt[0] == md[1] * md[2] && ms[0] == md[1] * md[2]))) {
    int64_t batch = m == 3 ? md[0] : 1, rows = md[m - 2], cols = md[m - 1];
    if (cols < 8) {
      transpose_narrow_cols_kernel<<<grid_for(ctx, batch * rows, 256, 8), 256, 0, ctx->stream>>>(s, d, batch, rows,
                                                                                                 (int)cols);
      return wdc_check_launch(ctx, "transpose_narrow_cols_kernel");
    }
    if (rows < 8) {
      transpose_narrow_rows_kernel<<<grid_for(ctx, batch * cols, 256, 8), 256, 0, ctx->stream>>>(s, d, batch,
                                                                                                 (int)rows, cols);
      return wdc_check_launch(ctx, "transpose_narrow_rows_kernel");
    }
    if (rows % 4 == 0 && cols % 4 == 0 && rows >= 32 && cols >= 32 && (((uintptr_t)s | (uintptr_t)d) & 15) == 0) {
      const int64_t nt = batch * ((rows + 63) / 64) * ((cols + 63) / 64);
      const int64_t cap64 = (int64_t)ctx->sm_count * 8;
      transpose_tile64_kernel<<<(int)(nt < cap64 ? nt : cap64), 256, 0, ctx->stream>>>(
          reinterpret_cast<const float*>(s), reinterpret_cast<float*>(d), batch, rows, cols);
      return wdc_check_launch(ctx, "transpose_tile64_kernel");
    }
    int64_t ntiles = batch * ((rows + 31) / 32) * ((cols + 31) / 32);
    int64_t cap = (int64_t)ctx->sm_count * 16;
    int grid = (int)(ntiles < cap ? ntiles : cap);
    transpose_tile_kernel<<<grid, 256, 0, ctx->stream>>>(s, d, batch, rows, cols);
    return wdc_check_launch(ctx, "transpose_tile_kernel");
  }
  CopyShape sh;
  for (int i = 0; i < 6; i++) {
    sh.dims[i] = 1;
    sh.sstr[i] = sh.dstr[i] = 0;
  }
  for (int i = 0; i < m; i++) {
    sh.dims[6 - m + i] = md[i];
    sh.sstr[6 - m + i] = ms[i];
    sh.dstr[6 - m + i] = mt[i];
  }
  // Innermost axis contiguous on both sides and everything a multiple of four elements (a head split, a Slice or
  // Concat along an outer axis): move 16-byte units, a quarter of the index arithmetic and full-width accesses.
  bool vec = m >= 1 && ms[m - 1] == 1 && mt[m - 1] == 1 && md[m - 1] % 4 == 0 &&
             (((uintptr_t)s | (uintptr_t)d) & 15) == 0;
  for (int i = 0; vec && i + 1 < m; i++) vec = ms[i] % 4 == 0 && mt[i] % 4 == 0;
  if (vec) {
    sh.dims[5] /= 4;
    for (int i = 0; i < 5; i++) {
      sh.sstr[i] /= 4;   // strides of the outer axes in 16-byte units (exact: multiples of 4, possibly negative)
      sh.dstr[i] /= 4;
    }
    launch_strided_copy<uint4>(ctx, reinterpret_cast<const uint4*>(s), reinterpret_cast<uint4*>(d), n / 4, sh, m);
    return wdc_check_launch(ctx, "strided_copy_kernel");
  }
  launch_strided_copy<uint32_t>(ctx, s, d, n, sh, m);
  return wdc_check_launch(ctx, "strided_copy_kernel");
}

__global__ void __launch_bounds__(256) gather_kernel(const uint32_t* __restrict__ data,
                                                     const int32_t* __restrict__ idx,
                                                     uint32_t* __restrict__ out, int64_t outer,
                                                     int64_t axis_len, int64_t inner, int64_t n_idx) {
  int64_t n = outer * n_idx * inner;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    int64_t in = i % inner, k = (i / inner) % n_idx, o = i / (inner * n_idx);
    int64_t j = idx[k];
    if (j < 0) j += axis_len;
    // out-of-range indices are clamped instead of read out of bounds
    j = j < 0 ? 0 : (j >= axis_len ? axis_len - 1 : j);
    out[i] = data[(o * axis_len + j) * inner + in];
  }
}

extern "C" int wdc_gather(wdc_context* ctx, const void* data, const int32_t* idx, void* out,
                          int64_t outer, int64_t axis_len, int64_t inner, int64_t n_idx) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_gather: null context");
  wdc_note_write(ctx, out);
  WDC_REQUIRE(ctx, outer >= 0 && axis_len > 0 && inner >= 0 && n_idx >= 0, "wdc_gather: bad shape");
  int64_t n = outer * n_idx * inner;
  if (n == 0) return WDC_OK;
  WDC_REQUIRE(ctx, data && idx && out, "wdc_gather: null buffer");
  DeviceGuard g(ctx->device);
  gather_kernel<<<grid_for(ctx, n, 256, 8), 256, 0, ctx->stream>>>((const uint32_t*)data, idx,
                                                                  (uint32_t*)out, outer, axis_len, inner, n_idx);
  return wdc_check_launch(ctx, "gather_kernel");
}
