// Implicit-GEMM convolution / GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   Y[m, n] = epilogue( sum_k A[m, k] * W[n, k] )       m = output pixel, n = output channel,
//                                                       k = (ky, kx, ci) over an NHWC input.
//
// fp32-class accuracy comes from the 3xTF32 split: every fp32 operand x is written as hi + lo with
// hi = tf32(x), lo = tf32(x - hi); the product is accumulated as A_lo*W_hi + A_hi*W_lo + A_hi*W_hi
// in fp32 TMEM accumulators (the lo*lo term, ~2^-22 relative, is dropped).
//
// One persistent CTA per SM, warp specialised:
//   warps 0-7   A producers: gather the im2col tile from global memory (128-bit loads, zero fill for
//               padding), split into hi/lo in registers and store both into 128B-swizzled shared
//               memory tiles (generic-proxy stores + fence.proxy.async).
//   warp  8     W producer: one lane issues two TMA tile loads per stage (pre-split W_hi, W_lo).
//   warp  9     MMA issuer: one lane issues tcgen05.mma.kind::tf32 (M=128, N=tile, K=8), 12 per
//               32-wide K block; tcgen05.commit releases the stage / publishes the accumulator.
//   warps 10-13 epilogue: tcgen05.ld the accumulator (double buffered in TMEM so the next tile's
//               main loop overlaps), apply scale/shift (bias, folded BatchNormalization), residual
//               add, Relu, and store NHWC with 128-bit stores.
// Every mbarrier wait is bounded in wall time; on expiry the kernel records an error code in the
// context's status word, raises a CTA-wide abort flag so the other roles stop too, frees its TMEM
// and returns.
#include <cuda.h>

#include <map>

#include "common.cuh"

namespace {

constexpr int TILE_M = 128;
constexpr int BLOCK_K = 32;           // fp32 elements per K block = one 128-byte swizzle row
constexpr int STAGES = 3;
constexpr int NUM_A_WARPS = 8;
constexpr int TMA_WARP = 8;
constexpr int MMA_WARP = 9;
constexpr int NUM_THREADS = 14 * 32;
constexpr int A_TILE_BYTES = TILE_M * BLOCK_K * 4;  // 16 KB
constexpr int PREFETCH = 3;                          // K blocks of A held in registers per thread
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct TcProblem {
  // implicit GEMM geometry
  int64_t M;          // batch * out_h * out_w
  int N;              // output channels
  int K;              // k_h * k_w * ch_in
  int ch_in, in_h, in_w, out_h, out_w, k_w;
  int stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int kblocks;        // ceil(K / 32)
  int cblocks;        // K blocks per filter tap = ceil(ch_in / 32)
  int tile_n;         // 32, 64 or 128
  int64_t tiles_m, tiles_n;
  // epilogue
  const float* scale;     // per channel or null
  const float* shift;     // per channel or null
  const float* residual;  // [M, res_stride] or null
  int64_t res_stride;
  float alpha, shift_mul, res_mul;
  int relu;
  int* status;
};

struct __align__(1024) SharedStorage {
  // tiles first: each must start on a 1024-byte boundary for the 128B swizzle
  unsigned char a_hi[STAGES][A_TILE_BYTES];
  unsigned char a_lo[STAGES][A_TILE_BYTES];
  unsigned char w_hi[STAGES][128 * BLOCK_K * 4];
  unsigned char w_lo[STAGES][128 * BLOCK_K * 4];
  unsigned long long full_bar[STAGES];
  unsigned long long empty_bar[STAGES];
  unsigned long long tmem_full_bar[2];
  unsigned long long tmem_empty_bar[2];
  unsigned int tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false if the wait was abandoned (time limit or CTA-wide abort).
__device__ __noinline__ bool mbar_wait_slow(unsigned long long* bar, uint32_t parity, SharedStorage* ss,
                                            int* status, int code) {
  unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (ss->abort_flag) return false;
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      ss->abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, SharedStorage* ss,
                                          int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ss, status, code);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024
// bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // version
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}

// instruction descriptor: D=f32, A=B=tf32, both K-major, dense, M=128, N=n
__device__ __forceinline__ uint32_t make_idesc(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_c, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_c), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, unsigned long long* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_igemm_kernel(const __grid_constant__ TcProblem p, const float* __restrict__ x,
                const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                float* __restrict__ y) {
  extern __shared__ unsigned char smem_raw[];
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&ss->full_bar[s], NUM_A_WARPS + 1);
      mbar_init(&ss->empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&ss->tmem_full_bar[b], 1);
      mbar_init(&ss->tmem_empty_bar[b], 4);
    }
    ss->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    // 256 columns: two accumulators of up to 128 fp32 columns each
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ss->tmem_base)),
                 "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ss->tmem_base;

  if (warp < NUM_A_WARPS) {
    // ===================================================================== A producers
    // Work items are (tile, K block) pairs in the order the MMA warp consumes them.  Loads run
    // PREFETCH items ahead of the shared-memory stores and cross tile boundaries, so the global
    // load latency is paid once per CTA, not once per tile.
    const int t = threadIdx.x;        // 0..255
    const int chunk = t & 7;          // 16-byte chunk of the 128-byte row
    const int rgrp = t >> 3;          // rows rgrp, rgrp+32, rgrp+64, rgrp+96
    const int64_t my_tiles = (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const int64_t items = my_tiles * p.kblocks;
    const int64_t hw = (int64_t)p.out_h * p.out_w;
    // load-side cursor
    int64_t ld_tile_i = -1;           // index into this CTA's tile sequence whose rows are cached
    long long rbase[4];
    int riy[4], rix[4];
    int ld_kb = 0;
    int64_t ld_tile_seq = 0;
    auto issue = [&](float4* dst) {
      if (ld_tile_seq != ld_tile_i) {
        ld_tile_i = ld_tile_seq;
        const int64_t tile = blockIdx.x + ld_tile_seq * gridDim.x;
        const int64_t m0 = (tile / p.tiles_n) * TILE_M;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int64_t m = m0 + rgrp + 32 * i;
          if (m < p.M) {
            const int64_t n = m / hw;
            const int rem = (int)(m - n * hw);
            const int oy = rem / p.out_w, ox = rem - oy * p.out_w;
            rbase[i] = n * (int64_t)p.in_h * p.in_w * p.ch_in;
            riy[i] = oy * p.stride_h - p.pad_t;
            rix[i] = ox * p.stride_w - p.pad_l;
          } else {
            rbase[i] = -1;
            riy[i] = rix[i] = 0;
          }
        }
      }
      const int tap = ld_kb / p.cblocks;
      const int c0 = (ld_kb - tap * p.cblocks) * BLOCK_K + chunk * 4;
      const int ky = tap / p.k_w, kx = tap - ky * p.k_w;
      const bool cok = c0 < p.ch_in;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int iy = riy[i] + ky * p.dil_h, ix = rix[i] + kx * p.dil_w;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cok && rbase[i] >= 0 && (unsigned)iy < (unsigned)p.in_h && (unsigned)ix < (unsigned)p.in_w)
          v = __ldg(reinterpret_cast<const float4*>(x + rbase[i] + ((long long)iy * p.in_w + ix) * p.ch_in + c0));
        dst[i] = v;
      }
      if (++ld_kb == p.kblocks) {
        ld_kb = 0;
        ld_tile_seq++;
      }
    };
    float4 ring[PREFETCH][4];
#pragma unroll
    for (int j = 0; j < PREFETCH; j++)
      if (j < items) issue(ring[j]);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int64_t g0 = 0; g0 < items; g0 += PREFETCH) {
#pragma unroll
      for (int j = 0; j < PREFETCH; j++) {
        const int64_t g = g0 + j;
        if (ok && g < items) {
          ok = mbar_wait(&ss->empty_bar[stage], phase ^ 1, ss, p.status, 12);
          if (ok) {
            unsigned char* ahi = ss->a_hi[stage];
            unsigned char* alo = ss->a_lo[stage];
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const int r = rgrp + 32 * i;
              const float4 v = ring[j][i];
              float4 h, l;
              h.x = to_tf32(v.x); h.y = to_tf32(v.y); h.z = to_tf32(v.z); h.w = to_tf32(v.w);
              l.x = to_tf32(v.x - h.x); l.y = to_tf32(v.y - h.y); l.z = to_tf32(v.z - h.z); l.w = to_tf32(v.w - h.w);
              const int off = r * 128 + ((chunk ^ (r & 7)) << 4);
              *reinterpret_cast<float4*>(ahi + off) = h;
              *reinterpret_cast<float4*>(alo + off) = l;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&ss->full_bar[stage]);
            if (g + PREFETCH < items) issue(ring[j]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == TMA_WARP) {
    // ===================================================================== W producer (TMA)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t bytes = 2u * (uint32_t)p.tile_n * BLOCK_K * 4u;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int n0 = (int)(tile % p.tiles_n) * p.tile_n;
        for (int kb = 0; kb < p.kblocks; kb++) {
          if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1, ss, p.status, 21)) { ok = false; break; }
          mbar_arrive_expect_tx(&ss->full_bar[stage], bytes);
          tma_load_2d(ss->w_hi[stage], &map_w_hi, &ss->full_bar[stage], kb * BLOCK_K, n0);
          tma_load_2d(ss->w_lo[stage], &map_w_lo, &ss->full_bar[stage], kb * BLOCK_K, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ===================================================================== MMA issuer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t idesc = make_idesc(p.tile_n);
      int64_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, it++) {
        const int acc = (int)(it & 1);
        const uint32_t acc_phase = (uint32_t)((it >> 1) & 1);
        if (!mbar_wait(&ss->tmem_empty_bar[acc], acc_phase ^ 1, ss, p.status, 31)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * 128);
        for (int kb = 0; kb < p.kblocks; kb++) {
          if (!mbar_wait(&ss->full_bar[stage], phase, ss, p.status, 32)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t da_hi = make_smem_desc(smem_u32(ss->a_hi[stage]));
          const uint64_t da_lo = make_smem_desc(smem_u32(ss->a_lo[stage]));
          const uint64_t dw_hi = make_smem_desc(smem_u32(ss->w_hi[stage]));
          const uint64_t dw_lo = make_smem_desc(smem_u32(ss->w_lo[stage]));
#pragma unroll
          for (int k = 0; k < BLOCK_K / 8; k++) {
            const uint64_t adv = (uint64_t)(k * 2);  // 8 tf32 = 32 bytes = 2 x 16-byte units
            umma_tf32(d_tmem, da_lo + adv, dw_hi + adv, idesc, (kb | k) ? 1u : 0u);
            umma_tf32(d_tmem, da_hi + adv, dw_lo + adv, idesc, 1u);
            umma_tf32(d_tmem, da_hi + adv, dw_hi + adv, idesc, 1u);
          }
          umma_commit(&ss->empty_bar[stage]);  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&ss->tmem_full_bar[acc]);
      }
    }
  } else {
    // ===================================================================== epilogue warps
    const int q = warp & 3;             // TMEM lane quadrant this warp may read
    const int row = q * 32 + lane;      // accumulator row (= TMEM lane) of this thread
    int64_t it = 0;
    bool ok = true;
    for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, it++) {
      const int buf = (int)(it & 1);
      const uint32_t bphase = (uint32_t)((it >> 1) & 1);
      const int64_t m0 = (tile / p.tiles_n) * TILE_M;
      const int n0 = (int)(tile % p.tiles_n) * p.tile_n;
      const int64_t m = m0 + row;
      if (!mbar_wait(&ss->tmem_full_bar[buf], bphase, ss, p.status, 42)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      for (int c0 = 0; c0 < p.tile_n; c0 += 32) {
        float v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 128 + c0), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (m < p.M) {
          const int nbase = n0 + c0;
          float* yrow = y + m * (int64_t)p.N + nbase;
          const float* rrow = p.residual ? p.residual + m * p.res_stride + nbase : nullptr;
          if (nbase + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float o[4];
#pragma unroll
              for (int e = 0; e < 4; e++) {
                const int c = nbase + j + e;
                float a = v[j + e] * (p.scale ? __ldg(p.scale + c) : p.alpha);
                if (p.shift) a = fmaf(p.shift_mul, __ldg(p.shift + c), a);
                o[e] = a;
              }
              if (rrow) {
                const float4 r4 = __ldg(reinterpret_cast<const float4*>(rrow + j));
                o[0] = fmaf(p.res_mul, r4.x, o[0]); o[1] = fmaf(p.res_mul, r4.y, o[1]);
                o[2] = fmaf(p.res_mul, r4.z, o[2]); o[3] = fmaf(p.res_mul, r4.w, o[3]);
              }
              if (p.relu) {
#pragma unroll
                for (int e = 0; e < 4; e++) o[e] = o[e] > 0.f ? o[e] : (o[e] == o[e] ? 0.f : o[e]);
              }
              *reinterpret_cast<float4*>(yrow + j) = make_float4(o[0], o[1], o[2], o[3]);
            }
          } else {
            for (int j = 0; j < 32; j++) {
              const int c = nbase + j;
              if (c >= p.N) break;
              float a = v[j] * (p.scale ? __ldg(p.scale + c) : p.alpha);
              if (p.shift) a = fmaf(p.shift_mul, __ldg(p.shift + c), a);
              if (rrow) a = fmaf(p.res_mul, __ldg(rrow + j), a);
              if (p.relu) a = a > 0.f ? a : (a == a ? 0.f : a);
              yrow[j] = a;
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss->tmem_empty_bar[buf]);
    }
  }

  // ------------------------------------------------------------------------------- teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256));
  }
}

// ---------------------------------------------------------------------------- host side
__global__ void split_tf32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo,
                                  int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    float v = w[i];
    float h = to_tf32(v);
    hi[i] = h;
    lo[i] = to_tf32(v - h);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct WeightEntry {
  float* hi = nullptr;
  float* lo = nullptr;
  int64_t rows = 0, k = 0;
  int tile_n = 0;
  CUtensorMap map_hi, map_lo;
};

struct TcState {
  EncodeTiledFn encode = nullptr;
  bool unavailable = false;
  bool attr_set = false;
  std::map<const void*, WeightEntry> weights;
};

TcState* tc_state(wdc_context* ctx) {
  if (!ctx->tc_state) ctx->tc_state = new TcState();
  return (TcState*)ctx->tc_state;
}

int pick_tile_n(int64_t n) { return n > 64 ? 128 : (n > 32 ? 64 : 32); }

int encode_map(TcState* st, CUtensorMap* map, float* base, int64_t rows, int64_t k, int tile_n) {
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)k * 4};
  cuuint32_t box[2] = {BLOCK_K, (cuuint32_t)tile_n};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Looks up (or builds) the hi/lo split and the tensor maps of a [rows, k] K-major weight matrix.
int get_weight(wdc_context* ctx, const float* w, int64_t rows, int64_t k, WeightEntry** out) {
  TcState* st = tc_state(ctx);
  auto it = st->weights.find(w);
  if (it != st->weights.end() && it->second.rows == rows && it->second.k == k) {
    *out = &it->second;
    return WDC_OK;
  }
  if (it != st->weights.end()) {
    wdc_free(ctx, it->second.hi);
    wdc_free(ctx, it->second.lo);
    st->weights.erase(it);
  }
  WeightEntry e;
  e.rows = rows;
  e.k = k;
  e.tile_n = pick_tile_n(rows);
  int s = wdc_alloc(ctx, rows * k * 4, (void**)&e.hi);
  if (s != WDC_OK) return s;
  s = wdc_alloc(ctx, rows * k * 4, (void**)&e.lo);
  if (s != WDC_OK) {
    wdc_free(ctx, e.hi);
    return s;
  }
  split_tf32_kernel<<<grid_for(ctx, rows * k, 256, 8), 256, 0, ctx->stream>>>(w, e.hi, e.lo, rows * k);
  s = wdc_check_launch(ctx, "split_tf32_kernel");
  int r1 = encode_map(st, &e.map_hi, e.hi, rows, k, e.tile_n);
  int r2 = encode_map(st, &e.map_lo, e.lo, rows, k, e.tile_n);
  if (s != WDC_OK || r1 || r2) {
    wdc_free(ctx, e.hi);
    wdc_free(ctx, e.lo);
    if (s != WDC_OK) return s;
    return wdc_fail(ctx, WDC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d, %d) for a [%lld, %lld] weight", r1, r2,
                    (long long)rows, (long long)k);
  }
  auto ins = st->weights.emplace(w, e);
  *out = &ins.first->second;
  return WDC_OK;
}

bool tc_ready(wdc_context* ctx) {
  TcState* st = tc_state(ctx);
  if (st->unavailable) return false;
  if (!st->encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
      cudaGetLastError();
      st->unavailable = true;
      return false;
    }
    st->encode = (EncodeTiledFn)fn;
  }
  if (!st->attr_set) {
    cudaError_t e = cudaFuncSetAttribute(tc_igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(SharedStorage) + 1024);
    if (e != cudaSuccess) {
      cudaGetLastError();
      st->unavailable = true;
      return false;
    }
    st->attr_set = true;
  }
  return true;
}

int launch_tc(wdc_context* ctx, TcProblem& p, const float* x, const float* w, float* y) {
  WeightEntry* we = nullptr;
  int s = get_weight(ctx, w, p.N, p.K, &we);
  if (s != WDC_OK) return s;
  p.tile_n = we->tile_n;
  p.tiles_m = ceil_div64(p.M, TILE_M);
  p.tiles_n = ceil_div64(p.N, p.tile_n);
  p.kblocks = (p.K + BLOCK_K - 1) / BLOCK_K;
  p.status = ctx->status_word;
  int64_t tiles = p.tiles_m * p.tiles_n;
  int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  tc_igemm_kernel<<<grid, NUM_THREADS, sizeof(SharedStorage) + 1024, ctx->stream>>>(p, x, we->map_hi, we->map_lo, y);
  ctx->n_tc_launch++;
  return wdc_check_launch(ctx, "tc_igemm_kernel");
}

bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

}  // namespace

void wdc_tc_evict(wdc_context* ctx, const void* ptr) {
  if (!ctx->tc_state) return;
  TcState* st = (TcState*)ctx->tc_state;
  auto it = st->weights.find(ptr);
  if (it == st->weights.end()) return;
  WeightEntry e = it->second;
  st->weights.erase(it);
  wdc_free(ctx, e.hi);
  wdc_free(ctx, e.lo);
}

void wdc_tc_destroy(wdc_context* ctx) {
  if (!ctx->tc_state) return;
  delete (TcState*)ctx->tc_state;  // the split buffers die with the arena slabs
  ctx->tc_state = nullptr;
}

int wdc_tc_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w, const float* scale,
                  const float* shift, const float* residual, float* y) {
  if (d->group != 1 || d->ch_in % BLOCK_K != 0 || d->ch_out % 4 != 0) return WDC_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (residual && !aligned16(residual))) return WDC_ERR_UNSUPPORTED;
  const int64_t K = d->ch_in * d->k_h * d->k_w;
  if (K > (1 << 30) || d->ch_out > (1 << 24)) return WDC_ERR_UNSUPPORTED;
  if (!tc_ready(ctx)) return WDC_ERR_UNSUPPORTED;
  TcProblem p = {};
  p.M = d->batch * d->out_h * d->out_w;
  p.N = (int)d->ch_out;
  p.K = (int)K;
  p.ch_in = (int)d->ch_in; p.in_h = (int)d->in_h; p.in_w = (int)d->in_w;
  p.out_h = (int)d->out_h; p.out_w = (int)d->out_w; p.k_w = (int)d->k_w;
  p.stride_h = (int)d->stride_h; p.stride_w = (int)d->stride_w; p.pad_t = (int)d->pad_t; p.pad_l = (int)d->pad_l;
  p.dil_h = (int)d->dil_h; p.dil_w = (int)d->dil_w;
  p.cblocks = (int)(d->ch_in / BLOCK_K);
  p.scale = scale; p.shift = shift; p.residual = residual; p.res_stride = d->ch_out;
  p.alpha = 1.f; p.shift_mul = 1.f; p.res_mul = 1.f; p.relu = d->relu;
  return launch_tc(ctx, p, x, w, y);
}

int wdc_tc_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B, const float* C,
                float* Y) {
  // A [m, k] with k contiguous, B given as [n, k] with k contiguous (Gemm transB=1, LSTM weights)
  if (d->batch != 1 || d->sa1 != 1 || d->sb0 != 1 || d->sb1 != d->k || d->sa0 != d->k) return WDC_ERR_UNSUPPORTED;
  if (d->k % 4 != 0 || d->sa0 % 4 != 0 || d->k < 32 || d->m < 32) return WDC_ERR_UNSUPPORTED;
  if (!aligned16(A) || !aligned16(B) || !aligned16(Y)) return WDC_ERR_UNSUPPORTED;
  const float* shift = nullptr;
  const float* residual = nullptr;
  int64_t res_stride = 0;
  if (C) {
    if (d->sc0 == 0 && d->sc1 == 1) shift = C;                                      // row vector (bias)
    else if (d->sc1 == 1 && d->sc0 >= d->n && d->sc0 % 4 == 0 && aligned16(C)) {    // full matrix
      residual = C;
      res_stride = d->sc0;
    } else return WDC_ERR_UNSUPPORTED;
  }
  if (d->k > (1 << 30) || d->n > (1 << 24)) return WDC_ERR_UNSUPPORTED;
  if (!tc_ready(ctx)) return WDC_ERR_UNSUPPORTED;
  TcProblem p = {};
  p.M = d->m;
  p.N = (int)d->n;
  p.K = (int)d->k;
  p.ch_in = (int)d->k; p.in_h = 1; p.in_w = 1; p.out_h = 1; p.out_w = 1; p.k_w = 1;
  p.stride_h = p.stride_w = 1; p.dil_h = p.dil_w = 1;
  p.cblocks = (int)((d->k + BLOCK_K - 1) / BLOCK_K);
  p.shift = shift; p.residual = residual; p.res_stride = res_stride;
  p.alpha = d->alpha; p.shift_mul = d->beta; p.res_mul = d->beta; p.relu = d->relu;
  return launch_tc(ctx, p, A, B, Y);
}
