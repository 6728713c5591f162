// Fused scaled-dot-product attention on the 5th-generation tensor cores (tcgen05, sm_100a):
//   y = softmax(scale * q k^T) v   per (batch, head), the score matrix kept on chip.
//
// One CTA owns 128 query rows of one head and walks the keys in chunks of 64:
//   S  = Q K_chunk^T            tcgen05.mma.kind::tf32, M = 128, N = 64, K = head size; Q is the A operand in TENSOR
//                               MEMORY (raw fp32 as the high part: the tensor core truncates it to TF32; low part
//                               x - truncate(x)), K_chunk the B operand in shared memory
//   P  = exp2(S' - max)         by the 128 "row" threads (thread r = query row r = TMEM lane r): tcgen05.ld of the
//                               row's 64 scores, running maximum and sum (one-pass softmax), P written back to
//                               tensor memory over S as the next A operand (high part raw, low part beside it)
//   Oc = P V_chunk              M = 128, N = head size, K = 64; V_chunk^T the B operand in shared memory
//   O  = O * alpha + Oc         in the row threads' registers (fp32, round to nearest): the tensor core only ever
//                               accumulates 64 keys, like the convolution kernel's segments
// Every product is 3xTF32 (lo*hi + hi*lo + hi*hi), which keeps the result within 1e-4 of the reference's
// double-accumulating operator chain (matmul.ts:63-111, binary7.ts:16-68, softmax.ts:39-57).
//
// K and V are split into high and low parts once per call by a small pre-pass (the B operand must be in shared
// memory in the tensor core's K-major layout, so V is transposed there as well): K_hi/K_lo [batch*heads, tk, dh]
// and Vt_hi/Vt_lo [batch*heads, dh, tk rounded up to 4] in arena scratch; TMA brings 64-key tiles of them into
// 128B-swizzled shared memory, two stages deep.  Keys past tk read as zero or as the next head's rows; their
// scores are replaced by -inf before the maximum, so they contribute nothing.
//
// Warps: 0-3 row threads, 4 TMA producer, 5 MMA issuer (one elected lane each).  With a head size of 32 a CTA needs
// 256 TMEM columns and 64 KB of shared memory, so two CTAs share an SM and one's softmax overlaps the other's MMAs.
// Every mbarrier wait is bounded (2 s): on expiry the CTA records a status code, raises its abort flag, frees its
// TMEM and returns.  No cluster, no multicast.
#include <cuda.h>

#include <math.h>

#include "common.cuh"

namespace {

constexpr int BQ = 128;           // query rows per CTA = TMEM lanes
constexpr int BK = 64;            // keys per chunk
constexpr int ATT_THREADS = 192;
constexpr int STAGES = 2;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct AttTcProblem {
  const float* q;
  float* y;
  int64_t q_sb, q_sh, q_st, y_sb, y_sh, y_st;
  int heads, tq, tk;
  float scale_log2;   // scale * log2(e): the softmax runs on exp2
  int* status;
};

struct AttShared {
  unsigned long long kv_full[STAGES], kv_empty[STAGES];
  unsigned long long q_ready, s_full, p_ready, o_full;
  unsigned int tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __noinline__ bool mbar_wait_slow(unsigned long long* bar, uint32_t parity, AttShared* sh, int* status, int code) {
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 1024; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (sh->abort_flag) return false;
    if (global_ns() - t0 > WAIT_LIMIT_NS) {
      sh->abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, AttShared* sh, int* status, int code) {
  for (int i = 0; i < 2048; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 4) __nanosleep(64);
  }
  return mbar_wait_slow(bar, parity, sh, status, code);
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
// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// instruction descriptor: D = f32, A = B = tf32, both K-major, dense, M = 128, N = n
__device__ __forceinline__ uint32_t make_idesc(int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_c, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_c), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ float low_part(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

// ------------------------------------------------------------------------------------------- pre-pass
// K [.., tk, dh] (strided) -> k_hi, k_lo [bh, tk, dh];  V -> vt_hi, vt_lo [bh, dh, tkp] (transposed, zero for
// keys tk .. tkp-1).  One CTA per (head, 32 keys).
template <int DH>
__global__ void __launch_bounds__(256) attn_split_kv_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                                            float* __restrict__ k_hi, float* __restrict__ k_lo,
                                                            float* __restrict__ vt_hi, float* __restrict__ vt_lo,
                                                            int heads, int tk, int tkp, int64_t k_sb, int64_t k_sh,
                                                            int64_t k_st, int64_t v_sb, int64_t v_sh, int64_t v_st) {
  __shared__ float tile[32][DH + 1];
  const int bh = blockIdx.y, b = bh / heads, h = bh - b * heads;
  const int t0 = blockIdx.x * 32;
  const float* kp = k + (int64_t)b * k_sb + (int64_t)h * k_sh;
  const float* vp = v + (int64_t)b * v_sb + (int64_t)h * v_sh;
  for (int i = threadIdx.x; i < 32 * DH; i += 256) {
    const int j = i / DH, c = i - j * DH, t = t0 + j;
    if (t < tk) {
      const float x = kp[(int64_t)t * k_st + c];
      const float hi = to_tf32(x);
      const int64_t o = ((int64_t)bh * tk + t) * DH + c;
      k_hi[o] = hi;
      k_lo[o] = to_tf32(x - hi);
      tile[j][c] = vp[(int64_t)t * v_st + c];
    } else {
      tile[j][c] = 0.f;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * DH; i += 256) {
    const int c = i >> 5, j = i & 31, t = t0 + j;
    if (t < tkp) {
      const float x = tile[j][c];
      const float hi = to_tf32(x);
      const int64_t o = ((int64_t)bh * DH + c) * tkp + t;
      vt_hi[o] = hi;
      vt_lo[o] = to_tf32(x - hi);
    }
  }
}

// ------------------------------------------------------------------------------------------- main kernel
template <int DH>
struct AttLayout {
  static constexpr int KB = DH / 32;                       // 32-wide K blocks of the head size
  static constexpr int K_TILE = BK * 128;                  // 64 keys x 32 floats = 8 KB
  static constexpr int V_TILE = DH * 128;                  // DH rows x 32 keys
  static constexpr int K_HI = 0, K_LO = KB * K_TILE, V_HI = 2 * KB * K_TILE, V_LO = V_HI + 2 * V_TILE;
  static constexpr int STAGE_BYTES = V_LO + 2 * V_TILE;    // 32 KB (DH = 32) or 64 KB (DH = 64)
  // tensor-memory columns
  static constexpr int Q_HI = 0, Q_LO = DH, S = 2 * DH, P_LO = S + BK, O = P_LO + BK;
  static constexpr int TMEM_COLS = DH == 32 ? 256 : 512;   // 224 or 320 used; a power of two must be allocated
};

template <int DH>
__global__ void __launch_bounds__(ATT_THREADS, DH == 32 ? 2 : 1)
attention_tc_kernel(const AttTcProblem p, const __grid_constant__ CUtensorMap map_k_hi,
                    const __grid_constant__ CUtensorMap map_k_lo, const __grid_constant__ CUtensorMap map_vt_hi,
                    const __grid_constant__ CUtensorMap map_vt_lo) {
  using L = AttLayout<DH>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stage_base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  AttShared* sh = reinterpret_cast<AttShared*>(stage_base + STAGES * L::STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.y, b = bh / p.heads, h = bh - b * p.heads;
  const int q0 = blockIdx.x * BQ;
  const int nck = (p.tk + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&sh->kv_full[s], 1);
      mbar_init(&sh->kv_empty[s], 1);
    }
    mbar_init(&sh->q_ready, 4);
    mbar_init(&sh->s_full, 1);
    mbar_init(&sh->p_ready, 4);
    mbar_init(&sh->o_full, 1);
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_k_hi) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_k_lo) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_vt_hi) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_vt_lo) : "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(L::TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = sh->tmem_base;
  // the pre-pass (the grid before this one) wrote the split operands this kernel is about to load
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp < 4) {
    // ============================================================================ row threads
    const int r = threadIdx.x;                              // query row inside the tile = TMEM lane
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    const int qrow = q0 + r;
    {
      // Q row -> tensor memory: high part raw (the tensor core truncates), low part x - truncate(x)
      const float* qp = p.q + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)qrow * p.q_st;
#pragma unroll
      for (int c0 = 0; c0 < DH; c0 += 16) {
        float hi[16], lo[16];
#pragma unroll
        for (int j = 0; j < 16; j += 4) {
          float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
          if (qrow < p.tq) x = __ldg(reinterpret_cast<const float4*>(qp + c0 + j));
          hi[j] = x.x; hi[j + 1] = x.y; hi[j + 2] = x.z; hi[j + 3] = x.w;
          lo[j] = low_part(x.x); lo[j + 1] = low_part(x.y); lo[j + 2] = low_part(x.z); lo[j + 3] = low_part(x.w);
        }
        tmem_st16(lane_base + (uint32_t)(L::Q_HI + c0), hi);
        tmem_st16(lane_base + (uint32_t)(L::Q_LO + c0), lo);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->q_ready);
    }
    float o[DH];
#pragma unroll
    for (int c = 0; c < DH; c++) o[c] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nck && ok; j++) {
      const uint32_t ph = (uint32_t)(j & 1);
      ok = mbar_wait(&sh->s_full, ph, sh, p.status, 71);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float s[BK];
#pragma unroll
      for (int c0 = 0; c0 < BK; c0 += 16) tmem_ld16(lane_base + (uint32_t)(L::S + c0), s + c0);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int valid = p.tk - j * BK;                      // columns of this chunk that are real keys
      float mc = -INFINITY;
#pragma unroll
      for (int c = 0; c < BK; c++) {
        s[c] = c < valid ? s[c] * p.scale_log2 : -INFINITY;
        mc = fmaxf(mc, s[c]);
      }
      const float m_new = fmaxf(m, mc);
      const float alpha = exp2f(m - m_new);                 // 0 for the first chunk (m = -inf)
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < BK; c++) {
        s[c] = exp2f(s[c] - m_new);
        sum += s[c];
      }
      l = l * alpha + sum;
      m = m_new;
      // P over S (high part, raw) and beside it (low part)
#pragma unroll
      for (int c0 = 0; c0 < BK; c0 += 16) {
        float lo[16];
#pragma unroll
        for (int c = 0; c < 16; c++) lo[c] = low_part(s[c0 + c]);
        tmem_st16(lane_base + (uint32_t)(L::S + c0), s + c0);
        tmem_st16(lane_base + (uint32_t)(L::P_LO + c0), lo);
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->p_ready);
      // O = O * alpha + P V_chunk
      ok = mbar_wait(&sh->o_full, ph, sh, p.status, 72);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < DH; c0 += 16) {
        float oc[16];
        tmem_ld16(lane_base + (uint32_t)(L::O + c0), oc);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 16; c++) o[c0 + c] = fmaf(o[c0 + c], alpha, oc[c]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (ok && qrow < p.tq) {
      const float inv = 1.f / l;
      float* yp = p.y + (int64_t)b * p.y_sb + (int64_t)h * p.y_sh + (int64_t)qrow * p.y_st;
#pragma unroll
      for (int c = 0; c < DH; c += 4)
        *reinterpret_cast<float4*>(yp + c) = make_float4(o[c] * inv, o[c + 1] * inv, o[c + 2] * inv, o[c + 3] * inv);
    }
  } else if (warp == 4) {
    // ============================================================================ TMA producer
    if (elect_one()) {
      bool ok = true;
      for (int j = 0; j < nck && ok; j++) {
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        ok = mbar_wait(&sh->kv_empty[st], ph ^ 1, sh, p.status, 73);
        if (!ok) break;
        unsigned char* sb = stage_base + st * L::STAGE_BYTES;
        mbar_arrive_expect_tx(&sh->kv_full[st], (uint32_t)L::STAGE_BYTES);
        const int krow = bh * p.tk + j * BK;
#pragma unroll
        for (int kb = 0; kb < L::KB; kb++) {
          tma_load_2d(sb + L::K_HI + kb * L::K_TILE, &map_k_hi, &sh->kv_full[st], kb * 32, krow);
          tma_load_2d(sb + L::K_LO + kb * L::K_TILE, &map_k_lo, &sh->kv_full[st], kb * 32, krow);
        }
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
          tma_load_2d(sb + L::V_HI + blk * L::V_TILE, &map_vt_hi, &sh->kv_full[st], j * BK + blk * 32, bh * DH);
          tma_load_2d(sb + L::V_LO + blk * L::V_TILE, &map_vt_lo, &sh->kv_full[st], j * BK + blk * 32, bh * DH);
        }
      }
    }
  } else {
    // ============================================================================ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(BK), idesc_o = make_idesc(DH);
      const uint32_t t_qhi = tmem_base + L::Q_HI, t_qlo = tmem_base + L::Q_LO, t_s = tmem_base + L::S,
                     t_plo = tmem_base + L::P_LO, t_o = tmem_base + L::O;
      bool ok = mbar_wait(&sh->q_ready, 0, sh, p.status, 74);
      for (int j = 0; j < nck && ok; j++) {
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)(j & 1);
        ok = mbar_wait(&sh->kv_full[st], (uint32_t)((j / STAGES) & 1), sh, p.status, 75);
        if (!ok) break;
        // S shares its columns with the previous chunk's P: wait until that chunk's P V has completed (its O has
        // been produced), which the o_full barrier of the previous chunk says
        if (j > 0) {
          ok = mbar_wait(&sh->o_full, ph ^ 1, sh, p.status, 76);
          if (!ok) break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sb = smem_u32(stage_base + st * L::STAGE_BYTES);
#pragma unroll
        for (int kb = 0; kb < L::KB; kb++) {
          const uint64_t d_hi = make_smem_desc(sb + L::K_HI + kb * L::K_TILE);
          const uint64_t d_lo = make_smem_desc(sb + L::K_LO + kb * L::K_TILE);
#pragma unroll
          for (int k8 = 0; k8 < 4; k8++) {
            const uint32_t acol = (uint32_t)(kb * 32 + k8 * 8);
            const uint64_t adv = (uint64_t)(k8 * 2);
            umma_tf32_ts(t_s, t_qlo + acol, d_hi + adv, idesc_s, (kb | k8) ? 1u : 0u);
            umma_tf32_ts(t_s, t_qhi + acol, d_lo + adv, idesc_s, 1u);
            umma_tf32_ts(t_s, t_qhi + acol, d_hi + adv, idesc_s, 1u);
          }
        }
        umma_commit(&sh->s_full);
        ok = mbar_wait(&sh->p_ready, ph, sh, p.status, 77);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
          const uint64_t d_hi = make_smem_desc(sb + L::V_HI + blk * L::V_TILE);
          const uint64_t d_lo = make_smem_desc(sb + L::V_LO + blk * L::V_TILE);
#pragma unroll
          for (int k8 = 0; k8 < 4; k8++) {
            const uint32_t acol = (uint32_t)(blk * 32 + k8 * 8);
            const uint64_t adv = (uint64_t)(k8 * 2);
            umma_tf32_ts(t_o, t_plo + acol, d_hi + adv, idesc_o, (blk | k8) ? 1u : 0u);
            umma_tf32_ts(t_o, t_s + acol, d_lo + adv, idesc_o, 1u);
            umma_tf32_ts(t_o, t_s + acol, d_hi + adv, idesc_o, 1u);
          }
        }
        umma_commit(&sh->kv_empty[st]);   // the stage's tiles have been read
        umma_commit(&sh->o_full);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)f;
    else
      cudaGetLastError();
  }
  return fn;
}

// [rows, cols] fp32 row-major matrix cut into boxes of box_rows x 32 columns, 128B-swizzled
bool encode_2d(CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int DH>
int launch(wdc_context* ctx, const wdc_attention_desc* d, const float* q, const float* k, const float* v, float* y) {
  using L = AttLayout<DH>;
  const int64_t bh = d->batch * d->heads;
  const int tk = (int)d->tk, tkp = (tk + 3) & ~3;
  static bool attr_set[64] = {};
  const int smem = STAGES * L::STAGE_BYTES + (int)sizeof(AttShared) + 1024;
  if (ctx->device < 0 || ctx->device >= 64) return WDC_ERR_UNSUPPORTED;
  if (!attr_set[ctx->device]) {
    if (cudaFuncSetAttribute(attention_tc_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      cudaGetLastError();
      return WDC_ERR_UNSUPPORTED;
    }
    attr_set[ctx->device] = true;
  }
  // scratch: the split copies of K and of V transposed
  const int64_t n_k = bh * tk * DH, n_v = bh * DH * tkp;
  float* scratch = nullptr;
  int s = wdc_alloc(ctx, (2 * n_k + 2 * n_v) * 4, (void**)&scratch);
  if (s != WDC_OK) return s;
  float *k_hi = scratch, *k_lo = k_hi + n_k, *vt_hi = k_lo + n_k, *vt_lo = vt_hi + n_v;
  CUtensorMap m_k_hi, m_k_lo, m_vt_hi, m_vt_lo;
  if (!encode_2d(&m_k_hi, k_hi, bh * tk, DH, BK) || !encode_2d(&m_k_lo, k_lo, bh * tk, DH, BK) ||
      !encode_2d(&m_vt_hi, vt_hi, bh * DH, tkp, DH) || !encode_2d(&m_vt_lo, vt_lo, bh * DH, tkp, DH)) {
    wdc_free(ctx, scratch);
    return WDC_ERR_UNSUPPORTED;
  }
  attn_split_kv_kernel<DH><<<dim3((unsigned)((tk + 31) / 32), (unsigned)bh), 256, 0, ctx->stream>>>(
      k, v, k_hi, k_lo, vt_hi, vt_lo, (int)d->heads, tk, tkp, d->k_sb, d->k_sh, d->k_st, d->v_sb, d->v_sh, d->v_st);
  s = wdc_check_launch(ctx, "attn_split_kv_kernel");
  if (s == WDC_OK) {
    AttTcProblem p;
    p.q = q; p.y = y;
    p.q_sb = d->q_sb; p.q_sh = d->q_sh; p.q_st = d->q_st;
    p.y_sb = d->y_sb; p.y_sh = d->y_sh; p.y_st = d->y_st;
    p.heads = (int)d->heads; p.tq = (int)d->tq; p.tk = tk;
    p.scale_log2 = d->scale * 1.4426950408889634f;
    p.status = ctx->status_word;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((d->tq + BQ - 1) / BQ), (unsigned)bh);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = ctx->stream;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
    const AttTcProblem& pc = p;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attention_tc_kernel<DH>, pc, m_k_hi, m_k_lo, m_vt_hi, m_vt_lo);
    ctx->n_launch++;
    ctx->n_tc_launch++;
    s = wdc_check_cuda(ctx, e, "attention_tc_kernel");
    if (s == WDC_OK) s = wdc_check_cuda(ctx, cudaGetLastError(), "attention_tc_kernel");
  }
  wdc_free(ctx, scratch);   // stream-ordered: reused only by work queued after the kernel
  return s;
}

}  // namespace

// Tensor-core form of wdc_attention.  WDC_ERR_UNSUPPORTED (nothing written): the caller runs the CUDA-core kernel.
int wdc_attention_tc(wdc_context* ctx, const wdc_attention_desc* d, const float* q, const float* k, const float* v,
                     float* y) {
  if (!encode_fn()) return WDC_ERR_UNSUPPORTED;
  if (d->batch * d->heads > 65535 || d->batch * d->heads * d->tk >= (1ll << 31) - 64 || d->tq >= (1ll << 31) - BQ)
    return WDC_ERR_UNSUPPORTED;
  if (d->batch * d->heads * 64 * ((d->tk + 3) / 4 * 4) >= (1ll << 40)) return WDC_ERR_UNSUPPORTED;
  if (d->dh == 32) return launch<32>(ctx, d, q, k, v, y);
  if (d->dh == 64) return launch<64>(ctx, d, q, k, v, y);
  return WDC_ERR_UNSUPPORTED;
}
