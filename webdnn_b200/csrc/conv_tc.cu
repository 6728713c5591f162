// Implicit-GEMM convolution / GEMM on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   Y[m, n] = epilogue( sum_k A[m, k] * W[n, k] )       m = output pixel, n = output channel,
//                                                       k = (ky, kx, ci) over an NHWC input.
//
// fp32-class accuracy comes from the 3xTF32 split: every fp32 operand x is written as hi + lo and the
// product is accumulated as A_lo*W_hi + A_hi*W_lo + A_hi*W_hi in fp32 TMEM accumulators (the lo*lo
// term, ~2^-22 relative, is dropped).  Weights are split once (hi = tf32(w), lo = tf32(w - hi), after
// the per-channel scale has been multiplied in) and cached.  For activations the tensor core's own
// operand truncation is the split: the raw fp32 value is the high operand (the MMA ignores its low
// 13 mantissa bits) and lo = x - (x & 0xffffe000), exact in fp32.
//
// The tensor core's fp32 accumulator truncates when it aligns addends, which biases long sums
// toward zero (measured ~0.15 ulp of the running sum per MMA).  To keep fp32-class accuracy through
// 50+ layers the accumulation has two levels: TMEM holds the partial sum of one SEGMENT of 4 K blocks
// (K = 128; a unit's last segment also takes a remainder of 1-3), and the epilogue warps add each
// finished segment into fp32 registers with round-to-nearest while the next segment runs into the
// other TMEM buffer.
//
// Shared memory bandwidth (128 B/clk) is the scarce resource of a 3xTF32 kernel: with both operands
// in shared memory a 128x128x8 MMA reads 8 KB per 64 clocks, which alone saturates it.  So the A
// operand lives in TENSOR MEMORY (tcgen05.st by the splitter threads; the MMA takes A from TMEM, W
// from shared memory) and shared memory carries the weight tiles, the raw A tiles on their way to the
// splitters, and the epilogue's staging buffers.
//
// One persistent CTA per SM, warp specialised, 16 warps (4 per SM sub-partition, so that every
// thread can have 128 registers).  tc_igemm_kernel<true> (A tiles by TMA):
//   warp  6     A loader: one im2col-mode TMA load per K block brings the raw 128-pixel x 32-channel
//               tile of the NHWC input (padding and rows past M arrive as zeros) into a 128B-swizzled
//               stage; first-layer mode (4 channels per pixel) loads one plane per tap or tap pair.
//   warps 0-3   A splitters: thread (w, l) owns row 32w+l of the tile (= TMEM lane); per K block it
//               reads its row from the stage (8 conflict-free 16-byte reads) and writes raw / lo into
//               32 + 32 TMEM columns with tcgen05.st.
//   warp  4     W loader: one lane issues two TMA tile loads per stage (pre-split W_hi, W_lo).
//   warp  5     MMA issuer: one lane issues tcgen05.mma.kind::tf32 (M=128, N=tile, K=8, A from TMEM),
//               12 per 32-wide K block; tcgen05.commit releases the stage / publishes the segment.
//   warps 8-15  accumulate + epilogue: each warp owns one TMEM lane quadrant and half of the tile's
//               columns; accumulators start at the per-channel shift; per segment tcgen05.ld + add into
//               registers; at the end of a tile the residual tile (brought by TMA into the warp's
//               staging buffer) is added, Relu applied, the result written over it and stored by TMA.
//               Tiles of at most 64 columns with at least 4 K blocks: warps 8-11 only (all of the tile's
//               columns each); warps 12-15 are then a second group of A splitters, and the two groups
//               take alternate K blocks (duo_mode).
// A barrier operation takes about 150 cycles to answer on this part even when its phase is long over,
// so the roles on the serial path ask ahead with the non-blocking mbarrier.test_wait while they have
// work in flight (the splitters while their shared-memory loads return, the MMA issuer between the k
// steps of a K block) and fall back to the bounded blocking wait only when they asked too early.
// tc_igemm_kernel<false> keeps the earlier producers for geometries an im2col tensor map cannot
// express: warps 0-3 gather A from global memory themselves (8 x 128-bit loads per row and K block,
// running 2 K blocks ahead).  Outputs whose row pitch is not a multiple of 16 bytes use the plain
// epilogue (transpose through shared memory, per-thread loads and stores).
// TMEM columns: [0,256) two segment accumulators of up to 128 columns, [256,448) three A stages of
// 32 (raw) + 32 (lo) columns.
// Every mbarrier wait is bounded in wall time; on expiry the kernel records an error code in the
// context's status word, raises a CTA-wide abort flag so the other roles stop too, frees its TMEM
// and returns.
#include <cuda.h>

#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "common.cuh"

namespace {

constexpr int TILE_M = 128;
constexpr int BLOCK_K = 32;           // fp32 elements per K block = one 128-byte swizzle row of W
constexpr int STAGES = 3;             // W tiles in shared memory and A (hi, lo) column groups in TMEM
constexpr int A_STAGES = 3;           // raw A tiles in shared memory (kTmaA)
constexpr int A_STAGES_MAX = 6;       // tiles of at most 64 columns leave half of the W region free: 3 more A stages
constexpr int PROBE_AFTER_K = 1;      // the MMA issuer probes its next barriers after this k step of a K block (0..3)
constexpr int DUO_MIN_KBLOCKS = 4;    // shortest reduction that runs with two splitter groups (see duo_mode)
constexpr int NUM_A_WARPS = 4;
constexpr int TMA_WARP = 4;
constexpr int MMA_WARP = 5;
constexpr int ATMA_WARP = 6;          // issues the im2col tile loads of A (kTmaA kernels only)
constexpr int A_TILE_BYTES = TILE_M * BLOCK_K * 4;  // 16 KB of raw fp32 A per stage
constexpr int EPI_WARP0 = 8;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 16 * 32;
constexpr int RES_L2_KBLOCKS = 4;   // residual L2 prefetch for launches with at most this many K blocks
constexpr int SEG_KBLOCKS = 4;        // K blocks accumulated in TMEM before the partial sum is drained; a unit's last
                                      // segment also takes a remainder of 1-3 blocks (see segments_of)
constexpr int NBUF = 2;               // TMEM segment accumulators of 128 columns
constexpr int EPI_BUF_BYTES = 32 * 32 * 4;   // epilogue staging: 32 rows x 32 columns per buffer, 2 per warp
constexpr int TMEM_A_COL0 = NBUF * 128;  // first column of the A stages
constexpr int W_TILE_BYTES = 128 * BLOCK_K * 4;  // 16 KB (hi) + 16 KB (lo) per stage
constexpr int PREFETCH = 2;           // K blocks of A held in registers per thread
constexpr int SHIFT_TAB = 2048;        // per-column addends kept in shared memory when N fits
constexpr int KTAB = 512;             // K blocks whose gather offsets are tabulated in shared memory
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// Development knock-out switches exist only in a build with -DWDC_TC_DEVELOP; the shipped kernel has none.
#ifdef WDC_TC_DEVELOP
#define TC_DBG(p, bit) (((p).dbg & (bit)) != 0)
#else
#define TC_DBG(p, bit) false
#endif

struct TcProblem {
  // implicit GEMM geometry
  int64_t M;          // batch * out_h * out_w
  int N;              // output channels
  int K;              // k_h * k_w * ch_in
  int ch_in, in_h, in_w, out_h, out_w, k_h, k_w;
  int stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int kblocks;        // ceil(K / 32)
  int cblocks;        // K blocks per filter tap = ceil(ch_in / 32)
  int tile_n;         // 32, 64 or 128
  // Work units.  The first `full_tiles` tiles (a whole number of waves of the grid, possibly none) are computed
  // by one unit each and leave through the fused epilogue.  Each of the remaining tiles (fewer than one wave) is
  // cut into `splits` ranges of `kbs` K blocks that run as separate units, so that the last, partly filled wave
  // becomes ceil(rest * splits / grid) rounds of 1 / splits of a tile instead of one whole tile per CTA.  A range's
  // raw partial sums go to block (rest_index * splits + range) of a workspace of 128-row x tile_n blocks; a second
  // kernel adds the ranges in ascending order and applies the epilogue.  splits == 1: every tile is a full tile.
  int full_tiles;
  int splits;
  int kbs;
  int tma_epi;        // 1: residual tiles and output tiles move by TMA (map_res, map_y)
  int c4;             // 1: input has 4 channels per pixel, one K block per filter row, chunk j = tap kx;
                      // 2: the same with the row physically padded on the left and stride_w 2, so that taps
                      //    (2j, 2j+1) are one 32-byte pixel pair: 4 loads of 128 x 32 bytes per K block
  int in_w_pad;       // c4 == 2: pixels per padded input row (even)
  int tiles_m, tiles_n;   // their product fits 31 bits (checked on the host)
  // epilogue
  const float* scale;     // per channel or null
  const float* shift;     // per channel or null
  const float* residual;  // [M, res_stride] or null
  int64_t res_stride;
  float alpha, shift_mul, res_mul;
  int relu;
  int single_pass;    // 1: precision tf32x1 (one MMA per multiply-add on the truncated operands; no low parts)
  uint32_t nap_ns;    // sleep between failed barrier polls (0: spin)
#ifdef WDC_TC_DEVELOP
  long long* prof;    // [grid][16] cycle counters of the warp roles (WDC_TC_PROF), or null
  int dbg;  // development knock-outs (WDC_TC_DEBUG): 1 = no A loads, 2 = no epilogue memory traffic, 4 = no MMAs
#endif
  int* status;
};

// Gather recipe of one K block, the same for every row of every tile: computed once per launch so
// that the producers' inner loop has no integer division.
struct KEntry {
  int off;       // element offset inside the image: (ky*dil_h*in_w + kx*dil_w)*ch_in + c0
  short dy, dx;  // tap displacement, for the bounds check
  int nchunks;   // valid 16-byte chunks of the block (8 unless the channel count ends inside it)
};

struct __align__(1024) SharedStorage {
  // weight tiles first: each must start on a 1024-byte boundary for the 128B swizzle
  // W_hi stages then W_lo stages, each tile_n x 128 bytes (16 KB slots for 128-column tiles; 8 KB slots for
  // narrower tiles, whose unused 48 KB then hold three more raw A stages)
  unsigned char w_region[2 * STAGES * W_TILE_BYTES];
  union {
    unsigned char a_raw[A_STAGES][A_TILE_BYTES];  // kTmaA: raw A tiles, 128B-swizzled rows of 32 floats
    KEntry ktab[KTAB];                          // gather kernels: per-K-block gather recipes
  };
  union {
    unsigned char epi_buf[NUM_EPI_WARPS][2][EPI_BUF_BYTES];  // TMA epilogue: residual in, result out
    float epi_stage[NUM_EPI_WARPS][32][20];  // plain epilogue: per-warp transpose buffer, 32 rows x 16 columns (+4 pad)
  };
  float shift_tab[SHIFT_TAB + 128];          // shift_mul * shift[col], zero past N (TMA epilogue, N <= SHIFT_TAB)
  unsigned long long full_bar[STAGES];
  unsigned long long empty_bar[STAGES];
  unsigned long long seg_full_bar[NBUF];
  unsigned long long seg_empty_bar[NBUF];
  unsigned long long a_full_bar[A_STAGES_MAX];
  unsigned long long a_empty_bar[A_STAGES_MAX];
  unsigned long long res_bar[NUM_EPI_WARPS][2];
  unsigned int tmem_base;
  volatile int abort_flag;
};

static_assert(offsetof(SharedStorage, a_raw) == offsetof(SharedStorage, w_region) + 2 * STAGES * W_TILE_BYTES,
              "the raw A tiles follow the W region without a gap");

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
// Non-blocking probe of a phase (try_wait may suspend the thread; this never does).
__device__ __forceinline__ bool mbar_test(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
__device__ __noinline__ bool mbar_wait_timed(unsigned long long* bar, uint32_t parity, SharedStorage* ss,
                                             int* status, int code) {
  // reached only after a few thousand failed polls: now watch the clock and the abort flag
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 1024; i++)
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
                                          int* status, int code, uint32_t nap_ns = 100) {
  // Hot path: plain polling, no timer read.  After two failed polls the thread sleeps ~100 ns between
  // polls: under a sustained load the GPU runs at its power cap, and warps that spin at full issue rate
  // cost clock frequency for the tensor pipe (measured: 0.7% of a ResNet-50 step).
  for (int i = 0; i < 4096; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 2 && nap_ns) __nanosleep(nap_ns);
  }
  return mbar_wait_timed(bar, parity, ss, status, code);
}

#ifdef WDC_TC_DEVELOP
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = clock64(); const long long prof_t0 = prof_t
#define PROF_ADD(slot) do { const long long n_ = clock64(); prof_acc[slot] += n_ - prof_t; prof_t = n_; } while (0)
#define PROF_OUT(base, n) do { if (p.prof) { for (int i_ = 0; i_ < (n); i_++) p.prof[blockIdx.x * 16 + (base) + i_] = prof_acc[i_]; \
                                 p.prof[blockIdx.x * 16 + (base) + (n)] = clock64() - prof_t0; } } while (0)
#define PROF_CNT(slot, cond) do { if (p.prof && (cond)) p.prof[blockIdx.x * 16 + (slot)] += 1; } while (0)
#define PROF_EV(type, g) do { if (p.prof && blockIdx.x == 0 && (g) < 64) p.prof[2368 + (type) * 64 + (int)(g)] = clock64(); } while (0)
#else
#define PROF_EV(type, g)
#define PROF_CNT(slot, cond)
#define PROF_DECL(n)
#define PROF_ADD(slot)
#define PROF_OUT(base, n)
#endif

// Narrow tiles with a reduction long enough for the operand split to matter run with two splitter groups and four
// epilogue warps; short reductions are bound by the epilogue's memory traffic and keep all eight epilogue warps.
__host__ __device__ __forceinline__ bool duo_mode(const TcProblem& p, bool a_by_tma) {
  return a_by_tma && p.tile_n <= 64 && p.kblocks >= DUO_MIN_KBLOCKS && !TC_DBG(p, 8192);
}

// Segments of a work unit of kbn K blocks: floor(kbn / 4) of them (at least one), 4 K blocks each, the last one
// with the remainder as well (up to 7): a short trailing segment would cost a whole accumulator drain for little
// accuracy (the stem's 7 K blocks are one segment instead of 4 + 3).
__host__ __device__ __forceinline__ int segments_of(int kbn) {
  return kbn < 2 * SEG_KBLOCKS ? 1 : kbn / SEG_KBLOCKS;
}

// Work unit u of a launch: a full tile (sp = -1, all K blocks), or range sp of one of the remaining tiles
// (K blocks kb0 .. kb0 + kbn - 1); `rest` is the tile's index among the remaining tiles.
__device__ __forceinline__ void unit_of(const TcProblem& p, int u, int& tile, int& sp, int& kb0, int& kbn) {
  if (u < p.full_tiles) {
    tile = u;
    sp = -1;
    kb0 = 0;
    kbn = p.kblocks;
    return;
  }
  const int r = u - p.full_tiles;
  const int rest = r / p.splits;
  tile = p.full_tiles + rest;
  sp = r - rest * p.splits;
  kb0 = sp * p.kbs;
  kbn = p.kblocks - kb0 < p.kbs ? p.kblocks - kb0 : p.kbs;
}

// Programmatic dependent launch.  wait: everything the grids before this one wrote is visible afterwards (a no-op
// for a launch without the attribute).  launch_dependents: the next grid of the stream may start its own set-up.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// max(x, 0) that keeps a NaN input (Math.max semantics), one instruction
__device__ __forceinline__ float relu_nan(float x) {
  float r;
  asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(r) : "f"(x));
  return r;
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

// D[tmem] (+)= A[tmem] * B[smem], the shared-memory descriptor given as its two 32-bit halves (only the low one, which holds the start
// address, changes from MMA to MMA) and the accumulate flag as a compile-time constant where it is one: the issuing
// thread is a single lane whose instruction count per K block is part of the kernel's serial path.
template <bool kAccumulate>
__device__ __forceinline__ void umma_tf32_ts2(uint32_t tmem_c, uint32_t tmem_a, uint32_t desc_lo, uint32_t desc_hi,
                                              uint32_t idesc, uint32_t accumulate = 1) {
  if (kAccumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\t"
        "mov.b64 d, {%2, %3};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d, %4, p;\n\t}"
        :
        : "r"(tmem_c), "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\t"
        "mov.b64 d, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d, %4, p;\n\t}"
        :
        : "r"(tmem_c), "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit_addr(uint32_t bar_saddr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_saddr) : "memory");
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
// Asks L2 to fetch the box at (x, y) of a 2-D tensor map; nothing lands in shared memory.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               :
               : "l"((unsigned long long)map), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"((unsigned long long)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
// im2col-mode tile load of an NHWC tensor: TILE_M pixels x BLOCK_K channels starting at base pixel
// (w, h, n) and channel c, each pixel displaced by the filter tap (off_w, off_h).  The base pixel
// walks the bounding box of the tensor map W-first with the convolution's strides; positions that
// fall outside the image (padding) or past the last image read as zero.
__device__ __forceinline__ void tma_load_im2col(void* smem_dst, const CUtensorMap* map, unsigned long long* bar,
                                                int c, int w, int h, int n, int off_w, int off_h) {
  const unsigned short ow = (unsigned short)off_w, oh = (unsigned short)off_h;
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
      :
      : "r"(smem_u32(smem_dst)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
        "h"(ow), "h"(oh)
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

// kTmaA = true: A tiles arrive by im2col TMA in shared memory (map_a) and the producer warps only
// split them into TMEM.  kTmaA = false: the producer warps gather A from global memory themselves
// (first-layer mode with 4 channels per pixel, and geometries an im2col tensor map cannot express).
template <bool kTmaA>
__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_igemm_kernel(const __grid_constant__ TcProblem p, const float* __restrict__ x,
                const __grid_constant__ CUtensorMap map_w_hi, const __grid_constant__ CUtensorMap map_w_lo,
                const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_y,
                const __grid_constant__ CUtensorMap map_res, const __grid_constant__ CUtensorMap map_ws,
                float* __restrict__ y) {
  extern __shared__ unsigned char smem_raw[];
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = p.tiles_m * p.tiles_n;
  const int total_units = p.full_tiles + (total_tiles - p.full_tiles) * p.splits;
  // shared-memory stage addresses
  const bool narrow = p.tile_n <= 64;
  // Narrow tiles: the operand split, not the tensor pipe, is the serial path (a barrier or shared-memory round trip
  // costs about 150 cycles, and a K block needs several).  Their epilogue is light (at most 64 columns), so four
  // warps do it instead of eight and the other four become a second group of splitters: the groups take alternate
  // K blocks.
  const bool duo = duo_mode(p, kTmaA);
  const int n_epi = duo ? NUM_EPI_WARPS / 2 : NUM_EPI_WARPS;
  const uint32_t w_slot = narrow ? W_TILE_BYTES / 2 : W_TILE_BYTES;
  const int a_stages = (kTmaA && narrow) ? A_STAGES_MAX : A_STAGES;
  auto w_hi_ptr = [&](int st) { return ss->w_region + (uint32_t)st * w_slot; };
  auto w_lo_ptr = [&](int st) { return ss->w_region + (uint32_t)(STAGES + st) * w_slot; };
  // (the upper half of the W region and the raw A tiles behind it are one contiguous block of 96 KB)
  auto a_ptr = [&](int st) {
    return st < A_STAGES ? ss->a_raw[st] : ss->w_region + 2 * STAGES * (W_TILE_BYTES / 2) + (st - A_STAGES) * A_TILE_BYTES;
  };

  {
    // one barrier per thread (38 of them): a single thread initialising them all costs half a microsecond per launch
    const int t = threadIdx.x;
    unsigned long long* bar = nullptr;
    int count = 1;
    if (t < STAGES) { bar = &ss->full_bar[t]; count = NUM_A_WARPS + 1; }
    else if (t < 2 * STAGES) { bar = &ss->empty_bar[t - STAGES]; }
    else if (t < 2 * STAGES + A_STAGES_MAX) { bar = &ss->a_full_bar[t - 2 * STAGES]; }
    else if (t < 2 * STAGES + 2 * A_STAGES_MAX) { bar = &ss->a_empty_bar[t - 2 * STAGES - A_STAGES_MAX]; count = NUM_A_WARPS; }
    else if (t < 2 * STAGES + 2 * A_STAGES_MAX + 2 * NUM_EPI_WARPS) {
      const int i = t - 2 * STAGES - 2 * A_STAGES_MAX;
      bar = &ss->res_bar[i >> 1][i & 1];
    } else if (t < 2 * STAGES + 2 * A_STAGES_MAX + 2 * NUM_EPI_WARPS + NBUF) {
      bar = &ss->seg_full_bar[t - 2 * STAGES - 2 * A_STAGES_MAX - 2 * NUM_EPI_WARPS];
    } else if (t < 2 * STAGES + 2 * A_STAGES_MAX + 2 * NUM_EPI_WARPS + 2 * NBUF) {
      bar = &ss->seg_empty_bar[t - 2 * STAGES - 2 * A_STAGES_MAX - 2 * NUM_EPI_WARPS - NBUF];
      count = n_epi;
    }
    if (bar) {
      mbar_init(bar, count);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (t == 0) ss->abort_flag = 0;
  }
  for (int kb = threadIdx.x; !kTmaA && kb < p.kblocks && kb < KTAB; kb += NUM_THREADS) {
    KEntry e;
    if (p.c4) {
      e.off = kb * p.dil_h * p.in_w * 4;
      e.dy = (short)(kb * p.dil_h);
      e.dx = 0;
      e.nchunks = p.k_w;
    } else {
      const int tap = kb / p.cblocks;
      const int c0 = (kb - tap * p.cblocks) * BLOCK_K;
      const int ky = tap / p.k_w, kx = tap - ky * p.k_w;
      e.off = (ky * p.dil_h * p.in_w + kx * p.dil_w) * p.ch_in + c0;
      e.dy = (short)(ky * p.dil_h);
      e.dx = (short)(kx * p.dil_w);
      const int left = (p.ch_in - c0 + 3) >> 2;
      e.nchunks = left < 8 ? left : 8;
    }
    ss->ktab[kb] = e;
  }
  const bool use_shift_tab = p.tma_epi && p.N <= SHIFT_TAB;
  if (threadIdx.x == 32) {
    // descriptor fetches of the first TMA operations overlap the rest of the set-up
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_w_hi) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_w_lo) : "memory");
    if (kTmaA) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_a) : "memory");
    if (p.tma_epi) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_y) : "memory");
    if (p.splits > 1) asm volatile("prefetch.tensormap [%0];" ::"l"((unsigned long long)&map_ws) : "memory");
  }
  if (kTmaA && p.c4) {
    // 4-channel mode: planes of taps past the filter width are never loaded; their weights are zero,
    // so the operand only has to be finite
    for (int st = 0; st < a_stages; st++)
      for (int i = threadIdx.x; i < A_TILE_BYTES / 16; i += NUM_THREADS)
        reinterpret_cast<float4*>(a_ptr(st))[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    // all 512 columns: NBUF segment accumulators + STAGES x (A_hi, A_lo)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ss->tmem_base)),
                 "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = ss->tmem_base;
  // Everything above touched only this CTA's own state, kernel parameters and constants of the model, so under
  // programmatic dependent launch it overlaps the tail of the previous grid.  From here on the kernel reads what
  // earlier grids wrote (activations, the residual) and writes memory they may still be reading (the arena reuses
  // freed blocks in stream order): wait for them.  The next grid may begin its own set-up right away; its CTAs
  // become resident as this grid's CTAs exit, and it waits for this grid's completion at the same point.
  grid_dependency_wait();
  grid_launch_dependents();
  // (the table of per-column addends is filled by the epilogue warps themselves, after this wait: the addends may
  // have been produced by an earlier grid, and the producer warps need not wait for the table)
  // Each CTA walks the K blocks of a full tile from a different starting point so that the CTAs, which all need
  // the same weight tiles, do not ask the same L2 lines at the same moment (split ranges start at their first block).
  const int rot_full = (int)(((int64_t)blockIdx.x * p.kblocks) / gridDim.x);

  if (kTmaA && (warp < NUM_A_WARPS || (duo && warp >= EPI_WARP0 + NUM_EPI_WARPS / 2))) {
    // ===================================================================== A producers (split only)
    // Thread (w, l) owns row 32w+l of the tile = TMEM lane.  Per K block: read the row's 32 raw
    // values from the swizzled shared-memory tile, write them unchanged as the high operand (the
    // tensor core ignores the low 13 bits of a tf32 operand, i.e. it truncates) and
    // lo = x - truncate(x), exact in fp32, as the low operand.
    const int q4 = warp & 3;                       // TMEM lane quadrant of this warp
    const int row = q4 * 32 + lane;
    const int group = warp < NUM_A_WARPS ? 0 : 1;  // second group: narrow tiles only
    const int ngroups = duo ? 2 : 1;
    const bool t0 = threadIdx.x == 0;
    int64_t items = 0;   // K blocks of all work units of this CTA
    for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
      int tile, sp, kb0, kbn;
      unit_of(p, u, tile, sp, kb0, kbn);
      items += kbn;
    }
    const uint32_t lane_base = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)TMEM_A_COL0;
    // normal mode: 128-byte rows, 16-byte chunks XOR-swizzled by the row; 4-channel mode: 8 planes
    // (one per filter tap of the row) of 128 rows x 16 bytes, or 4 planes (one per tap pair) of 128
    // rows x 32 bytes with the 32B swizzle (chunk ^= bit 2 of the row)
    const uint32_t row_off = (uint32_t)row * (p.c4 == 1 ? 16u : p.c4 == 2 ? 32u : 128u);
    const uint32_t sw = (uint32_t)(row & 7);
    // ring positions of K block g: TMEM / W stage g % STAGES, raw tile g % a_stages
    int stage = group % STAGES, as = group % a_stages;
    uint32_t phase = 0, aphase = 0;
    bool a_tok = false;   // answer of the probe made one iteration earlier
    PROF_DECL(5);
    for (int64_t g = group; g < items; g += ngroups) {
      PROF_ADD(4);
      if (t0) PROF_CNT(13, !a_tok);
      if (!a_tok && !mbar_wait(&ss->a_full_bar[as], aphase, ss, p.status, 11, p.nap_ns)) break;
      PROF_ADD(0);
      if (t0) PROF_EV(0, g);
      float4 v[8];
      const unsigned char* tile = a_ptr(as) + row_off;
#pragma unroll
      for (int j = 0; j < 8; j++)
        v[j] = *reinterpret_cast<const float4*>(
            tile + (p.c4 == 1   ? (uint32_t)j * (TILE_M * 16u)
                    : p.c4 == 2 ? (uint32_t)(j >> 1) * (TILE_M * 32u) + ((((uint32_t)j & 1u) ^ ((uint32_t)(row >> 2) & 1u)) << 4)
                                : (((uint32_t)j ^ sw) << 4)));
      // A barrier operation takes about 150 cycles to answer even when the phase is long over.  So both barriers
      // are probed without blocking while the shared-memory loads above are in flight: this K block's TMEM stage,
      // and the raw tile of the group's NEXT K block (looked at one iteration later).  A probe that came too early
      // falls back to the blocking wait.
      int as_n = as + ngroups, stage_n = stage + ngroups;
      uint32_t aphase_n = aphase, phase_n = phase;
      if (as_n >= a_stages) { as_n -= a_stages; aphase_n ^= 1; }
      if (stage_n >= STAGES) { stage_n -= STAGES; phase_n ^= 1; }
      bool a_tok_n = false, e_tok = false;
      if (!TC_DBG(p, 4096)) {
        e_tok = mbar_test(&ss->empty_bar[stage], phase ^ 1);
        if (g + ngroups < items) a_tok_n = mbar_test(&ss->a_full_bar[as_n], aphase_n);
      }
      if (t0) PROF_CNT(14, !e_tok);
      if (!e_tok && !mbar_wait(&ss->empty_bar[stage], phase ^ 1, ss, p.status, 12, p.nap_ns)) break;
      PROF_ADD(1);
      if (t0) PROF_EV(1, g);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_hi = lane_base + (uint32_t)(stage * 64);
#pragma unroll
      for (int h = 0; h < 2; h++) {
        float hi[16], lo[16];
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const float4 q = v[h * 4 + c];
          const float e[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int t = 0; t < 4; t++) {
            hi[c * 4 + t] = e[t];
            lo[c * 4 + t] = e[t] - __uint_as_float(__float_as_uint(e[t]) & 0xffffe000u);
          }
        }
        tmem_st16(a_hi + (uint32_t)(h * 16), hi);
        if (!p.single_pass) tmem_st16(a_hi + 32u + (uint32_t)(h * 16), lo);
      }
      // the shared-memory tile has been read into registers: hand the slot back to the loader
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss->a_empty_bar[as]);
      PROF_ADD(2);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      PROF_ADD(3);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss->full_bar[stage]);
      if (t0) PROF_EV(2, g);
      stage = stage_n; phase = phase_n;
      as = as_n; aphase = aphase_n;
      a_tok = a_tok_n;
    }
    if (t0) PROF_OUT(0, 5);
  } else if (kTmaA && warp == ATMA_WARP) {
    // ===================================================================== A loader (im2col TMA)
    // One lane issues the loads; in 4-channel mode lane j issues the load of tap j of the filter row.
    if (p.c4 ? lane < 8 : lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t hw = (uint32_t)p.out_h * (uint32_t)p.out_w;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int tile, sp, kb0, kbn;
        unit_of(p, u, tile, sp, kb0, kbn);
        // base pixel of the tile's first row
        const int64_t m0 = (int64_t)(tile / p.tiles_n) * TILE_M;
        const int64_t n = m0 / hw;
        const uint32_t rem = (uint32_t)(m0 - n * hw);
        const int oy = (int)(rem / (uint32_t)p.out_w), ox = (int)rem - oy * p.out_w;
        const int cw = p.c4 == 2 ? ox : ox * p.stride_w - p.pad_l, ch = oy * p.stride_h - p.pad_t;
        // first K block: this CTA's rotation, or the start of the unit's range (no rotation then)
        const int kfirst = kb0 + (sp < 0 ? rot_full : 0);
        const int tap = kfirst / p.cblocks;
        int c0 = (kfirst - tap * p.cblocks) * BLOCK_K;
        int ky = tap / p.k_w, kx = tap - ky * p.k_w;
        if (p.c4) ky = kfirst;
        for (int kb = 0; kb < kbn; kb++) {
          if (!mbar_wait(&ss->a_empty_bar[stage], phase ^ 1, ss, p.status, 22, p.nap_ns)) { ok = false; break; }
          if (TC_DBG(p, 256)) {   // no A loads
            if (lane == 0) mbar_arrive(&ss->a_full_bar[stage]);
            if (++stage == a_stages) { stage = 0; phase ^= 1; }
            continue;
          }
          if (p.c4) {
            // K block = filter row ky; one load of 128 pixels x 4 channels per tap of the row, or of 128
            // pixel pairs x 8 channels per tap pair
            const int nload = p.c4 == 2 ? (p.k_w + 1) >> 1 : p.k_w;
            const int plane = p.c4 == 2 ? TILE_M * 32 : TILE_M * 16;
            if (lane == 0) mbar_arrive_expect_tx(&ss->a_full_bar[stage], (uint32_t)(nload * plane));
            __syncwarp(0xffu);
            if (lane < nload)
              tma_load_im2col(a_ptr(stage) + lane * plane, &map_a, &ss->a_full_bar[stage], 0, cw, ch, (int)n,
                              p.c4 == 2 ? lane : lane * p.dil_w, ky * p.dil_h);
            if (++ky == p.k_h) ky = 0;
          } else {
            mbar_arrive_expect_tx(&ss->a_full_bar[stage], (uint32_t)A_TILE_BYTES);
            tma_load_im2col(a_ptr(stage), &map_a, &ss->a_full_bar[stage], c0, cw, ch, (int)n, kx * p.dil_w,
                            ky * p.dil_h);
            c0 += BLOCK_K;
            if (c0 >= p.ch_in) {
              c0 = 0;
              if (++kx == p.k_w) {
                kx = 0;
                if (++ky == p.k_h) ky = 0;
              }
            }
          }
          if (++stage == a_stages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (!kTmaA && warp < NUM_A_WARPS) {
    // ===================================================================== A producers (gather)
    // Work items are (tile, K block) pairs in the order the MMA warp consumes them.  Loads run
    // PREFETCH items ahead of the TMEM stores and cross tile boundaries, so the global load latency
    // is paid once per CTA, not once per tile.
    const int row = threadIdx.x;      // 0..127: tile row and TMEM lane of this thread
    const int64_t my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int64_t items = my_tiles * p.kblocks;
    const uint32_t hw = (uint32_t)p.out_h * (uint32_t)p.out_w;
    const int64_t img_elems = (int64_t)p.in_h * p.in_w * p.ch_in;
    // load-side cursor
    const float* rsrc = nullptr;      // address of input pixel (n, iy0, ix0, channel 0); null for rows past M
    int riy = 0, rix = 0;
    int ld_kb = p.kblocks;            // forces the row set-up on the first call
    int ld_tile = (int)blockIdx.x - (int)gridDim.x;
    auto issue = [&](float4* dst) {
      if (ld_kb == p.kblocks) {       // next tile: locate this thread's output pixel
        ld_kb = 0;
        ld_tile += gridDim.x;
        const int64_t m = (int64_t)(ld_tile / p.tiles_n) * TILE_M + row;
        if (m < p.M) {
          uint32_t n, rem;
          if (p.M <= 0x7fffffffll) {  // 32-bit division is several times cheaper
            n = (uint32_t)m / hw;
            rem = (uint32_t)m - n * hw;
          } else {
            n = (uint32_t)(m / hw);
            rem = (uint32_t)(m - (int64_t)n * hw);
          }
          const int oy = (int)(rem / (uint32_t)p.out_w), ox = (int)rem - oy * p.out_w;
          riy = oy * p.stride_h - p.pad_t;
          rix = ox * p.stride_w - p.pad_l;
          rsrc = x + ((int64_t)n * img_elems + (int64_t)(riy * p.in_w + rix) * p.ch_in);
        } else {
          rsrc = nullptr;
        }
      }
      int kb = ld_kb + rot_full;   // (this kernel never splits a tile)
      if (kb >= p.kblocks) kb -= p.kblocks;
      ld_kb++;
      KEntry e;
      if (kb < KTAB) {
        e = ss->ktab[kb];
      } else {  // very long reductions: compute the entry instead of looking it up
        const int tap = kb / p.cblocks;
        const int c0 = (kb - tap * p.cblocks) * BLOCK_K;
        const int ky = tap / p.k_w, kx = tap - ky * p.k_w;
        e.off = (ky * p.dil_h * p.in_w + kx * p.dil_w) * p.ch_in + c0;
        e.dy = (short)(ky * p.dil_h);
        e.dx = (short)(kx * p.dil_w);
        const int left = (p.ch_in - c0 + 3) >> 2;
        e.nchunks = left < 8 ? left : 8;
      }
      const int iy = riy + e.dy;
      const bool rowok = !TC_DBG(p, 1) && rsrc != nullptr && (unsigned)iy < (unsigned)p.in_h;
      const float* src = rsrc + e.off;
      if (p.c4) {
        // one K block = one filter row: chunk j is tap kx = j (the 4 channels of one pixel)
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int ix = rix + j * p.dil_w;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (rowok && j < e.nchunks && (unsigned)ix < (unsigned)p.in_w)
            v = __ldg(reinterpret_cast<const float4*>(src + j * p.dil_w * 4));
          dst[j] = v;
        }
      } else {
        const int ix = rix + e.dx;
        const bool ok2 = rowok && (unsigned)ix < (unsigned)p.in_w;
        if (ok2 && e.nchunks == 8) {
#pragma unroll
          for (int j = 0; j < 8; j++) dst[j] = __ldg(reinterpret_cast<const float4*>(src) + j);
        } else {
#pragma unroll
          for (int j = 0; j < 8; j++) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ok2 && j < e.nchunks) v = __ldg(reinterpret_cast<const float4*>(src) + j);
            dst[j] = v;
          }
        }
      }
    };
    float4 ring[PREFETCH][8];
#pragma unroll
    for (int j = 0; j < PREFETCH; j++)
      if (j < items) issue(ring[j]);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)TMEM_A_COL0;
    for (int64_t g0 = 0; g0 < items; g0 += PREFETCH) {
#pragma unroll
      for (int j = 0; j < PREFETCH; j++) {
        const int64_t g = g0 + j;
        if (ok && g < items) {
          ok = mbar_wait(&ss->empty_bar[stage], phase ^ 1, ss, p.status, 12, p.nap_ns);
          if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi = lane_base + (uint32_t)(stage * 64);
#pragma unroll
            for (int h = 0; h < 2; h++) {
              float hi[16], lo[16];
#pragma unroll
              for (int c = 0; c < 4; c++) {
                const float4 v = ring[j][h * 4 + c];
                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int t = 0; t < 4; t++) {
                  if (p.single_pass) { hi[c * 4 + t] = e[t]; lo[c * 4 + t] = 0.f; continue; }
                  // hi = e rounded to TF32 (add half an ulp of the 10-bit mantissa, clear the low 13
                  // bits): two full-rate integer ops instead of a quarter-rate cvt.  lo = e - hi is
                  // exact in fp32; the tensor core ignores the low 13 bits of a tf32 operand, which
                  // costs lo at most 2^-10 of its own size (2^-21 of e).
                  const float hh = __uint_as_float((__float_as_uint(e[t]) + 0x1000u) & 0xffffe000u);
                  hi[c * 4 + t] = hh;
                  lo[c * 4 + t] = e[t] - hh;
                }
              }
              if (TC_DBG(p, 16)) continue;
              tmem_st16(a_hi + (uint32_t)(h * 16), hi);
              if (!p.single_pass) tmem_st16(a_hi + 32u + (uint32_t)(h * 16), lo);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
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
      const uint32_t bytes = (p.single_pass ? 1u : 2u) * (uint32_t)p.tile_n * BLOCK_K * 4u;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int tile, sp, kb0, kbn;
        unit_of(p, u, tile, sp, kb0, kbn);
        const int n0 = (int)(tile % p.tiles_n) * p.tile_n;
        for (int kb = 0; kb < kbn; kb++) {
          if (!mbar_wait(&ss->empty_bar[stage], phase ^ 1, ss, p.status, 21, p.nap_ns)) { ok = false; break; }
          if (TC_DBG(p, 128)) {   // no W loads: the MMAs read whatever the stage holds
            mbar_arrive(&ss->full_bar[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          mbar_arrive_expect_tx(&ss->full_bar[stage], bytes);
          int kr = kb0 + kb + (sp < 0 ? rot_full : 0);
          if (kr >= kb0 + kbn) kr -= kbn;
          // K offset of the block in a weight row: blocks are counted per filter tap, and when the channel
          // count is not a multiple of 32 a tap's last block is short (its tail columns meet zeros of A)
          int kx0 = kr * BLOCK_K;
          if (!p.c4 && p.cblocks * BLOCK_K != p.ch_in) {
            const int tap = kr / p.cblocks;
            kx0 = tap * p.ch_in + (kr - tap * p.cblocks) * BLOCK_K;
          }
          tma_load_2d(w_hi_ptr(stage), &map_w_hi, &ss->full_bar[stage], kx0, n0);
          if (!p.single_pass) tma_load_2d(w_lo_ptr(stage), &map_w_lo, &ss->full_bar[stage], kx0, n0);
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
      // per-stage operand addresses from a few bases: descriptor low words (start address in 16-byte units) of the
      // W_hi / W_lo slots, the high word all descriptors share, TMEM column of the stage's A, barrier addresses
      const uint64_t desc0 = make_smem_desc(smem_u32(w_hi_ptr(0)));
      const uint32_t desc_hi32 = (uint32_t)(desc0 >> 32);
      const uint32_t dwh0 = (uint32_t)desc0, dwl0 = (uint32_t)make_smem_desc(smem_u32(w_lo_ptr(0)));
      const uint32_t dslot = w_slot >> 4;
      const uint32_t a_col0 = tmem_base + (uint32_t)TMEM_A_COL0;
      const uint32_t empty0 = smem_u32(&ss->empty_bar[0]);
      int64_t seg = 0;  // segments issued by this CTA so far
      bool ok = true;
      bool f_tok = false;   // answer of the probe made one K block earlier
      bool s_tok = false;   // the same for the next segment's accumulator
      PROF_DECL(5);
      int gk = 0;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int tile, sp, kb0, kbn;
        unit_of(p, u, tile, sp, kb0, kbn);
        uint32_t d_tmem = 0;
        int buf = 0;
        int in_seg = 0;
        for (int kb = 0; kb < kbn; kb++) {
          const bool seg_last = kb == kbn - 1 || (in_seg == SEG_KBLOCKS - 1 && kbn - (kb + 1) >= SEG_KBLOCKS);
          PROF_ADD(2);
          if (in_seg == 0) {
            buf = (int)(seg % NBUF);
            if (!s_tok && !mbar_wait(&ss->seg_empty_bar[buf], (uint32_t)((seg / NBUF) & 1) ^ 1, ss, p.status, 31, p.nap_ns)) { ok = false; break; }
            s_tok = false;
            PROF_ADD(0);
            PROF_EV(5, gk);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            d_tmem = tmem_base + (uint32_t)(buf * 128);
          }
          PROF_CNT(15, !f_tok);
          if (!f_tok && !mbar_wait(&ss->full_bar[stage], phase, ss, p.status, 32, p.nap_ns)) { ok = false; break; }
          f_tok = false;
          PROF_ADD(1);
          PROF_EV(3, gk);
          const int stage_n = stage + 1 == STAGES ? 0 : stage + 1;
          const uint32_t phase_n = stage_n ? phase : phase ^ 1;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_hi = a_col0 + (uint32_t)(stage * 64);
          const uint32_t a_lo = a_hi + 32u;
          const uint32_t dw_hi = dwh0 + (uint32_t)stage * dslot;
          const uint32_t dw_lo = dwl0 + (uint32_t)stage * dslot;
#pragma unroll
          for (int k = 0; k < BLOCK_K / 8; k++) {
            const uint32_t adv = (uint32_t)(k * 2);  // 8 tf32 = 32 bytes = 2 x 16-byte units of W
            const uint32_t acol = (uint32_t)(k * 8); // 8 TMEM columns of A
            if (TC_DBG(p, 4)) continue;
            if (p.single_pass) {
              if (k == 0) umma_tf32_ts2<false>(d_tmem, a_hi, dw_hi, desc_hi32, idesc, in_seg ? 1u : 0u);
              else umma_tf32_ts2<true>(d_tmem, a_hi + acol, dw_hi + adv, desc_hi32, idesc);
              continue;
            }
            if (k == 0) umma_tf32_ts2<false>(d_tmem, a_lo, dw_hi, desc_hi32, idesc, in_seg ? 1u : 0u);
            else umma_tf32_ts2<true>(d_tmem, a_lo + acol, dw_hi + adv, desc_hi32, idesc);
            umma_tf32_ts2<true>(d_tmem, a_hi + acol, dw_lo + adv, desc_hi32, idesc);
            umma_tf32_ts2<true>(d_tmem, a_hi + acol, dw_hi + adv, desc_hi32, idesc);
            if (k == PROBE_AFTER_K && !TC_DBG(p, 4096)) {
              // Probe the next stage's barrier (see the operand splitters) with MMAs of this stage already queued:
              // the answer takes about 150 cycles, during which this lane issues nothing and the tensor pipe works on
              // what is queued.  On a segment's last K block also the accumulator the next segment will use.
              f_tok = mbar_test(&ss->full_bar[stage_n], phase_n);
              if (seg_last)
                s_tok = mbar_test(&ss->seg_empty_bar[(int)((seg + 1) % NBUF)], (uint32_t)(((seg + 1) / NBUF) & 1) ^ 1);
            }
          }
          PROF_ADD(3);
          umma_commit_addr(empty0 + (uint32_t)stage * 8u);  // stage reusable once these MMAs have read it

          PROF_ADD(4);
          PROF_EV(4, gk);
          gk++;
          stage = stage_n; phase = phase_n;
          if (seg_last) {
            umma_commit(&ss->seg_full_bar[buf]);  // partial sum of this segment is complete
            seg++;
            in_seg = 0;
          } else {
            in_seg++;
          }
        }
      }
      PROF_OUT(6, 5);
    }
  } else if (warp >= EPI_WARP0) {
    // ===================================================================== accumulate + epilogue warps
    const int ew = warp - EPI_WARP0;
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    const int half = ew >> 2;                     // which half of the tile's columns (eight warps)
    const int ncols = duo ? p.tile_n : p.tile_n >> 1;   // 16, 32 or 64 columns per warp
    const int col0 = half * ncols;
    int nseg = segments_of(p.kblocks);
    int64_t seg = 0;
    bool ok = true;
    if (use_shift_tab) {
      // entries a warp can touch: its first column (< tiles_n * tile_n) plus 64; the epilogue warps fill the
      // table and meet at a barrier of their own (id 1, 256 threads), so the producers are not held up
      const int used = p.tiles_n * p.tile_n + 64;
      for (int i = threadIdx.x - EPI_WARP0 * 32; i < used; i += n_epi * 32)
        ss->shift_tab[i] = (p.shift && i < p.N) ? p.shift_mul * __ldg(p.shift + i) : 0.f;
      asm volatile("bar.sync 1, %0;" ::"r"(n_epi * 32) : "memory");
    }
    if (p.tma_epi) {
      // ------------------------------------------------------------------ epilogue through TMA
      // The warp's 32 rows x ncols columns leave in chunks of 32 rows x cw columns.  Per chunk: the
      // residual tile (if any) has been loaded by TMA into one of the warp's two staging buffers;
      // lane r reads row r of it, applies scale/shift, residual and Relu to its accumulators, writes
      // the result over the residual and one lane hands the buffer to a TMA store, which clips at
      // the matrix edges.  The residual of the following chunk (of this or of the next tile) is
      // requested right after, into the other buffer.
      const int cw = ncols < 32 ? ncols : 32;
      const int nch = ncols / cw;                       // 1 or 2
      const uint32_t chunk_bytes = 32u * (uint32_t)cw * 4u;
      const uint32_t swz = cw == 32 ? (uint32_t)(lane & 7) : 0u;   // 128B swizzle only for 128-byte rows
      const uint32_t row_off = (uint32_t)lane * (uint32_t)cw * 4u;
      const bool use_res = p.residual != nullptr && !TC_DBG(p, 2);
      // residual tiles exist for full tiles only; a CTA's full tiles all come before its split ranges
      int64_t k = 0;                                    // residual chunks handled by this warp so far
      int64_t ks = 0;                                   // staging buffers used so far (parity picks the buffer)
      if (use_res && lane == 0 && (int)blockIdx.x < p.full_tiles) {
        const int t0 = blockIdx.x;
        mbar_arrive_expect_tx(&ss->res_bar[ew][0], chunk_bytes);
        tma_load_2d(ss->epi_buf[ew][0], &map_res, &ss->res_bar[ew][0], (int)(t0 % p.tiles_n) * p.tile_n + col0,
                    (int)((t0 / p.tiles_n) * TILE_M + q * 32));
        if (nch == 2 && p.kblocks <= RES_L2_KBLOCKS)
          tma_prefetch_l2_2d(&map_res, (int)(t0 % p.tiles_n) * p.tile_n + col0 + 32,
                             (int)((t0 / p.tiles_n) * TILE_M + q * 32));
      }
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        int tile, sp, kb0, kbn;
        unit_of(p, u, tile, sp, kb0, kbn);
        const bool direct = sp < 0;                     // full tile: fused epilogue; else raw partial sums
        const bool res_u = use_res && direct;
        nseg = segments_of(kbn);
        // Short-K (memory-bound) launches: while this tile accumulates, L2 fetches the residual chunks of
        // the warp's next tile.  Each staging buffer holds one chunk, so without this every chunk waits
        // for a full trip to HBM.  Long-K launches hide that trip behind the MMAs and skip the extra requests.
        if (res_u && lane == 0 && p.kblocks <= RES_L2_KBLOCKS && tile + (int)gridDim.x < p.full_tiles) {
          const int nt = tile + (int)gridDim.x;
          for (int c = 0; c < nch; c++)
            tma_prefetch_l2_2d(&map_res, (int)(nt % p.tiles_n) * p.tile_n + col0 + c * 32,
                               (int)((nt / p.tiles_n) * TILE_M + q * 32));
        }
        const int64_t mrow0 = (int64_t)(tile / p.tiles_n) * TILE_M + q * 32;   // first row of this warp
        // split ranges: block (rest * splits + sp) of the workspace, 128 rows x tile_n columns each
        const int64_t ws_row = ((int64_t)(tile - p.full_tiles) * p.splits + sp) * TILE_M + q * 32;
        const int nbase = (int)(tile % p.tiles_n) * p.tile_n + col0;
        // The accumulators of a full tile start at the per-column addend (bias / folded BatchNormalization
        // shift); the per-column multiplier is already in the weights.  Warp-uniform 16-byte loads from the
        // table in shared memory (from global memory when N exceeds the table).  Split ranges start at zero.
        float acc[64];
        if (!direct) {
#pragma unroll
          for (int j = 0; j < 64; j++) acc[j] = 0.f;
        } else if (p.N <= SHIFT_TAB) {
          // branch-free: the table is zero past N, and 64 entries past any warp's first column exist
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(&ss->shift_tab[nbase + j]);
            acc[j] = b4.x;
            acc[j + 1] = b4.y;
            acc[j + 2] = b4.z;
            acc[j + 3] = b4.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; j += 4) {
            float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.shift && j < ncols && nbase + j < p.N) {
              b4 = __ldg(reinterpret_cast<const float4*>(p.shift + nbase + j));
              b4.x *= p.shift_mul; b4.y *= p.shift_mul; b4.z *= p.shift_mul; b4.w *= p.shift_mul;
            }
            acc[j] = b4.x;
            acc[j + 1] = b4.y;
            acc[j + 2] = b4.z;
            acc[j + 3] = b4.w;
          }
        }
        for (int s = 0; s < nseg && ok; s++, seg++) {
          const int buf = (int)(seg % NBUF);
          ok = mbar_wait(&ss->seg_full_bar[buf], (uint32_t)((seg / NBUF) & 1), ss, p.status, 42, p.nap_ns);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 128 + col0);
#pragma unroll
          for (int c = 0; c < 4; c++) {
            if (c * 16 < ncols) {
              float v[16];
              tmem_ld16(taddr + (uint32_t)(c * 16), v);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 16; j++) acc[c * 16 + j] += v[j];
            }
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&ss->seg_empty_bar[buf]);
        }
        if (!ok) break;

#pragma unroll
        for (int c = 0; c < 2; c++) {
          if (c < nch && ok) {
            const int b = (int)(ks & 1);
            unsigned char* sbuf = ss->epi_buf[ew][b];
            // buffer b is free: with a residual, its load was issued after the store that last read
            // the buffer had finished; without, lane 0 has waited for that store before this point
            if (res_u) ok = mbar_wait(&ss->res_bar[ew][b], (uint32_t)((k >> 1) & 1), ss, p.status, 43, p.nap_ns);
            __syncwarp();
            if (ok) {
              // 4 cells (16 columns) at a time: residual reads first, then arithmetic and writes, so
              // that the shared-memory reads of a batch do not queue behind the writes one by one.
#pragma unroll
              for (int jb = 0; jb < 8; jb += 4) {
                if (jb * 4 < cw) {
                  float4 r4[4];
                  if (res_u) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                      r4[j] = *reinterpret_cast<const float4*>(sbuf + row_off + (((uint32_t)(jb + j) ^ swz) << 4));
                  }
#pragma unroll
                  for (int j = 0; j < 4; j++) {
                    const float* av = &acc[c * 32 + (jb + j) * 4];
                    float o[4] = {av[0], av[1], av[2], av[3]};
                    if (res_u) {
                      o[0] = fmaf(p.res_mul, r4[j].x, o[0]);
                      o[1] = fmaf(p.res_mul, r4[j].y, o[1]);
                      o[2] = fmaf(p.res_mul, r4[j].z, o[2]);
                      o[3] = fmaf(p.res_mul, r4[j].w, o[3]);
                    }
                    if (p.relu && direct) {
#pragma unroll
                      for (int e = 0; e < 4; e++) o[e] = relu_nan(o[e]);
                    }
                    *reinterpret_cast<float4*>(sbuf + row_off + (((uint32_t)(jb + j) ^ swz) << 4)) =
                        make_float4(o[0], o[1], o[2], o[3]);
                  }
                }
              }
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                const int col = nbase + c * 32;
                if (!TC_DBG(p, 2) && mrow0 < p.M && col < p.N) {
                  if (direct) tma_store_2d(&map_y, sbuf, col, (int)mrow0);
                  else tma_store_2d(&map_ws, sbuf, col0 + c * 32, (int)ws_row);
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the other buffer's store has read it
                if (res_u) {
                  int nt = tile;
                  int nc = c + 1;
                  if (nc == nch) { nc = 0; nt += gridDim.x; }
                  if (nt < p.full_tiles) {
                    mbar_arrive_expect_tx(&ss->res_bar[ew][b ^ 1], chunk_bytes);
                    tma_load_2d(ss->epi_buf[ew][b ^ 1], &map_res, &ss->res_bar[ew][b ^ 1],
                                (int)(nt % p.tiles_n) * p.tile_n + col0 + nc * 32,
                                (int)((nt / p.tiles_n) * TILE_M + q * 32));
                  }
                }
              }
              if (res_u) k++;
              ks++;
            }
          }
        }
      }
      // the staging buffers must have been read before the CTA's shared memory goes away; the stores' arrival in
      // global memory is covered by the grid's completion
      if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    } else {
      // ------------------------------------------------------------------ plain epilogue
    const int nchunks = ncols >> 4;
    float (*stg)[20] = ss->epi_stage[ew];
    // After the transpose through shared memory a lane owns 4 consecutive columns of 4 rows, so that a
    // warp-wide access touches 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
    const int tr = lane >> 2;                     // rows tr, tr+8, tr+16, tr+24 of the warp's 32
    const int tc = (lane & 3) * 4;                // first of this lane's 4 columns inside a 16-column chunk
    const bool vec = (p.N & 3) == 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int64_t mrow0 = (int64_t)(tile / p.tiles_n) * TILE_M + q * 32;   // first row of this warp
      const int nbase = (int)(tile % p.tiles_n) * p.tile_n + col0;
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; j++) acc[j] = 0.f;
      float4 rcur[4];
      auto load_res = [&](int c, float4* dst) {
        const int col = nbase + c * 16 + tc;
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int64_t m = mrow0 + tr + 8 * i;
          float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.residual && !TC_DBG(p, 2) && m < p.M && col < p.N) {
            const float* rp = p.residual + m * p.res_stride + col;
            if (vec) r = __ldg(reinterpret_cast<const float4*>(rp));
            else {
              r.x = __ldg(rp);
              if (col + 1 < p.N) r.y = __ldg(rp + 1);
              if (col + 2 < p.N) r.z = __ldg(rp + 2);
              if (col + 3 < p.N) r.w = __ldg(rp + 3);
            }
          }
          dst[i] = r;
        }
      };
      for (int s = 0; s < nseg && ok; s++, seg++) {
        const int buf = (int)(seg % NBUF);
        if (s == nseg - 1) {
          load_res(0, rcur);  // in flight while the last segment finishes
          if (p.residual && !TC_DBG(p, 2)) {  // pull the rest of the residual tile towards L2
            for (int c = 1; c < nchunks; c++) {
              const int col = nbase + c * 16 + tc;
#pragma unroll
              for (int i = 0; i < 4; i++) {
                const int64_t m = mrow0 + tr + 8 * i;
                if (m < p.M && col < p.N)
                  asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + m * p.res_stride + col));
              }
            }
          }
        }
        ok = mbar_wait(&ss->seg_full_bar[buf], (uint32_t)((seg / NBUF) & 1), ss, p.status, 42, p.nap_ns);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 128 + col0);
#pragma unroll
        for (int c = 0; c < 4; c++) {
          if (c < nchunks) {
            float v[16];
            tmem_ld16(taddr + (uint32_t)(c * 16), v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) acc[c * 16 + j] += v[j];
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&ss->seg_empty_bar[buf]);
      }
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        if (c < nchunks) {
          // row-per-lane -> shared memory
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4*>(&stg[lane][j]) =
                make_float4(acc[c * 16 + j], acc[c * 16 + j + 1], acc[c * 16 + j + 2], acc[c * 16 + j + 3]);
          __syncwarp();
          const int col = nbase + c * 16 + tc;
          if (col < p.N && !TC_DBG(p, 2)) {
            float sc[4] = {p.alpha, p.alpha, p.alpha, p.alpha}, sh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int e = 0; e < 4; e++) {
              if (col + e < p.N) {
                if (p.scale) sc[e] = __ldg(p.scale + col + e);
                if (p.shift) sh[e] = p.shift_mul * __ldg(p.shift + col + e);
              }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const int64_t m = mrow0 + tr + 8 * i;
              if (m < p.M) {
                const float4 a = *reinterpret_cast<const float4*>(&stg[tr + 8 * i][tc]);
                float o[4] = {a.x, a.y, a.z, a.w};
                const float rr[4] = {rcur[i].x, rcur[i].y, rcur[i].z, rcur[i].w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                  float t = fmaf(o[e], sc[e], sh[e]);
                  if (p.residual) t = fmaf(p.res_mul, rr[e], t);
                  if (p.relu) t = relu_nan(t);
                  o[e] = t;
                }
                float* yp = y + m * (int64_t)p.N + col;
                if (vec) *reinterpret_cast<float4*>(yp) = make_float4(o[0], o[1], o[2], o[3]);
                else {
#pragma unroll
                  for (int e = 0; e < 4; e++)
                    if (col + e < p.N) yp[e] = o[e];
                }
              }
            }
          }
          __syncwarp();
          if (c + 1 < nchunks) load_res(c + 1, rcur);
        }
      }
    }
    }
  }

  // ------------------------------------------------------------------------------- teardown
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
}

// ---------------------------------------------------------------------------- host side
// Row r of the weight matrix is multiplied by alpha * scale[r] (scale null = 1) before the split, so
// that the kernel's epilogue has no per-channel multiply left.
__global__ void split_tf32_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo,
                                  int64_t n, int64_t k, const float* __restrict__ scale, float alpha) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) {
    float v = w[i] * (scale ? alpha * scale[i / k] : alpha);
    float h = to_tf32(v);
    hi[i] = h;
    lo[i] = to_tf32(v - h);
  }
}

// Same split for a weight matrix stored [k][rows] (rows contiguous, MatMul's B): 32x32 tiles through
// shared memory so that both the reads (along rows) and the writes (along k) are coalesced.
__global__ void __launch_bounds__(256) split_tf32_transpose_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                                                   float* __restrict__ lo, int64_t rows, int64_t k,
                                                                   const float* __restrict__ scale, float alpha) {
  __shared__ float tile[32][33];
  const int64_t tiles_r = (rows + 31) / 32, tiles_k = (k + 31) / 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int64_t t = blockIdx.x; t < tiles_r * tiles_k; t += gridDim.x) {
    const int64_t r0 = (t / tiles_k) * 32, k0 = (t % tiles_k) * 32;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t kk = k0 + ty + i * 8, r = r0 + tx;
      if (kk < k && r < rows) tile[ty + i * 8][tx] = w[kk * rows + r];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int64_t r = r0 + ty + i * 8, kk = k0 + tx;
      if (r < rows && kk < k) {
        const float v = tile[tx][ty + i * 8] * (scale ? alpha * scale[r] : alpha);
        const float h = to_tf32(v);
        hi[r * k + kk] = h;
        lo[r * k + kk] = to_tf32(v - h);
      }
    }
    __syncthreads();
  }
}

// Second pass for the tiles whose reduction was cut into ranges: for tile `full_tiles + r`, block (r * splits + s)
// of the workspace holds the raw partial sums of range s as 128 rows x tile_n columns.  The ranges are added in
// ascending order (deterministic), then shift, residual and Relu are applied as in the fused epilogue.  N % 4 == 0.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, float* __restrict__ y,
                                                            const float* __restrict__ shift, float shift_mul,
                                                            const float* __restrict__ residual, int64_t res_stride,
                                                            float res_mul, int relu, int64_t M, int N, int tile_n,
                                                            int tiles_n, int full_tiles, int rest_tiles, int splits) {
  grid_dependency_wait();   // launched as a programmatic dependent of the contraction kernel
  const int tv = tile_n / 4;                       // float4 cells per tile row
  const int64_t total = (int64_t)rest_tiles * TILE_M * tv;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const int c4 = (int)(i % tv);
    const int row = (int)((i / tv) % TILE_M);
    const int r = (int)(i / ((int64_t)tv * TILE_M));
    const int tile = full_tiles + r;
    const int64_t m = (int64_t)(tile / tiles_n) * TILE_M + row;
    const int n = (tile % tiles_n) * tile_n + c4 * 4;
    if (m >= M || n >= N) continue;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shift) {
      const float4 b = __ldg(reinterpret_cast<const float4*>(shift + n));
      acc = make_float4(shift_mul * b.x, shift_mul * b.y, shift_mul * b.z, shift_mul * b.w);
    }
    const float* src = ws + (((int64_t)r * splits) * TILE_M + row) * tile_n + c4 * 4;
    // all ranges' loads first (at most 8 in flight per thread), then the additions in ascending order
    float4 v[8];
#pragma unroll
    for (int s = 0; s < 8; s++)
      v[s] = s < splits ? __ldcg(reinterpret_cast<const float4*>(src + (int64_t)s * TILE_M * tile_n))
                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; s++) {
      if (s < splits) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
    }
    if (residual) {
      const float4 rr = __ldg(reinterpret_cast<const float4*>(residual + m * res_stride + n));
      acc.x = fmaf(res_mul, rr.x, acc.x); acc.y = fmaf(res_mul, rr.y, acc.y);
      acc.z = fmaf(res_mul, rr.z, acc.z); acc.w = fmaf(res_mul, rr.w, acc.w);
    }
    if (relu) {
      acc.x = relu_nan(acc.x); acc.y = relu_nan(acc.y); acc.z = relu_nan(acc.z); acc.w = relu_nan(acc.w);
    }
    *reinterpret_cast<float4*>(y + m * N + n) = acc;
  }
}

// Stem mode operand preparation: 4 channels per pixel, 8 taps per filter row.
// `plane` = 0: x is NHWC (a pixel's channels are adjacent); > 0: x is NCHW with `plane` pixels per channel plane.
__global__ void pad_channels4_kernel(const float* __restrict__ x, float* __restrict__ x4, int64_t pixels, int cin,
                                     int64_t plane) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < pixels; i += step) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* s = plane ? x + (i / plane) * plane * cin + i % plane : x + i * cin;
    const int64_t cs = plane ? plane : 1;
    v.x = s[0];
    if (cin > 1) v.y = s[cs];
    if (cin > 2) v.z = s[2 * cs];
    if (cin > 3) v.w = s[3 * cs];
    reinterpret_cast<float4*>(x4)[i] = v;
  }
}
// Same with every image row shifted right by pad_l pixels into a zero-filled row of wp pixels: pixel pair
// (2j, 2j+1) of the padded row is then the pair of taps (2j, 2j+1) of output column j for stride 2.
// With hp > h the images are padded vertically too: pad_t zero rows above, hp - pad_t - h below.
__global__ void pad_channels4_rows_kernel(const float* __restrict__ x, float* __restrict__ x4, int64_t images, int h,
                                          int hp, int pad_t, int w, int wp, int pad_l, int cin, int nchw) {
  int64_t total = images * hp * wp;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const int64_t rp = i / wp;
    const int px = (int)(i - rp * wp) - pad_l;
    const int64_t img = rp / hp;
    const int yy = (int)(rp - img * hp) - pad_t;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (px >= 0 && px < w && yy >= 0 && yy < h) {
      // NHWC rows, or NCHW planes of h x w
      const int64_t plane = (int64_t)h * w;
      const float* s = nchw ? x + img * plane * cin + (int64_t)yy * w + px : x + ((img * h + yy) * w + px) * cin;
      const int64_t cs = nchw ? plane : 1;
      v.x = s[0];
      if (cin > 1) v.y = s[cs];
      if (cin > 2) v.z = s[2 * cs];
      if (cin > 3) v.w = s[3 * cs];
    }
    reinterpret_cast<float4*>(x4)[i] = v;
  }
}
// w [n][k_h][k_w][cin] -> hi/lo of [n][k_h][8][4] (zero where kx >= k_w or c >= cin)
__global__ void split_tf32_c4_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo,
                                     int64_t rows, int k_h, int k_w, int cin, const float* __restrict__ scale,
                                     float alpha) {
  int64_t total = rows * k_h * 32;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    int c = (int)(i & 3), kx = (int)((i >> 2) & 7);
    int64_t r = i >> 5;  // n * k_h + ky
    float v = (kx < k_w && c < cin) ? w[(r * k_w + kx) * cin + c] : 0.f;
    v *= scale ? alpha * scale[r / k_h] : alpha;
    float h = to_tf32(v);
    hi[i] = h;
    lo[i] = to_tf32(v - h);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct WeightKey {
  const void* w;
  const void* scale;
  uint32_t alpha_bits;
  int k_major;  // 1: source stored [rows][k]; 0: stored [k][rows]
  bool operator<(const WeightKey& o) const {
    if (w != o.w) return w < o.w;
    if (scale != o.scale) return scale < o.scale;
    if (alpha_bits != o.alpha_bits) return alpha_bits < o.alpha_bits;
    return k_major < o.k_major;
  }
};

struct WeightEntry {
  float* hi = nullptr;
  float* lo = nullptr;
  int64_t rows = 0, k = 0;
  int64_t src_bytes = 0;  // size of the caller's weight buffer the split was made from
  int64_t born = 0;       // creation number (wdc_context::split_seq), for the staleness of captured graphs
  // tensor maps of the split copies for tile heights of 32, 64 and 128 weight rows (index log2(n / 32)),
  // encoded when a launch first asks for that height
  CUtensorMap map_hi[3], map_lo[3];
  bool has_map[3] = {false, false, false};
};

struct TcState {
  EncodeTiledFn encode = nullptr;
  EncodeIm2colFn encode_im2col = nullptr;  // may stay null: then every launch gathers A itself
  bool unavailable = false;
  bool attr_set = false;
  std::map<WeightKey, WeightEntry> weights;
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

// [rows, cols] fp32 matrix with a row pitch of `pitch` elements, cut into boxes of 32 rows x cw columns
// (128B-swizzled when a box row is 128 bytes).
int encode_rows_map(TcState* st, CUtensorMap* map, const float* base, int64_t rows, int64_t cols, int64_t pitch,
                    int cw) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch * 4};
  cuuint32_t box[2] = {(cuuint32_t)cw, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE,
                          cw == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Looks up (or builds) the hi/lo split and the tensor maps of a [rows, k] K-major weight matrix.
int get_weight(wdc_context* ctx, const float* w, const float* scale, float alpha, int64_t rows, int64_t k,
               WeightEntry** out, int c4_kh = 0, int c4_kw = 0, int c4_cin = 0, bool k_major = true) {
  TcState* st = tc_state(ctx);
  WeightKey key = {w, scale, 0, k_major ? 1 : 0};
  memcpy(&key.alpha_bits, &alpha, 4);
  auto it = st->weights.find(key);
  if (it != st->weights.end() && it->second.rows == rows && it->second.k == k) {
    *out = &it->second;
    return WDC_OK;
  }
  if (ctx->capture_arena)
    return wdc_fail(ctx, WDC_ERR_INVALID,
                    "a weight operand was seen for the first time while capturing: run the sequence once before "
                    "wdc_capture_begin, so that the one-time split is not part of the recorded run");
  if (it != st->weights.end()) {
    WeightEntry old = it->second;
    st->weights.erase(it);
    wdc_graphs_note_evicted(ctx, old.born);
    wdc_free(ctx, old.hi);
    wdc_free(ctx, old.lo);
  }
  WeightEntry e;
  e.rows = rows;
  e.k = k;
  e.src_bytes = (c4_kh ? rows * c4_kh * c4_kw * c4_cin : rows * k) * 4;
  int s = wdc_alloc(ctx, rows * k * 4, (void**)&e.hi);
  if (s != WDC_OK) return s;
  s = wdc_alloc(ctx, rows * k * 4, (void**)&e.lo);
  if (s != WDC_OK) {
    wdc_free(ctx, e.hi);
    return s;
  }
  if (c4_kh)
    split_tf32_c4_kernel<<<grid_for(ctx, rows * k, 256, 8), 256, 0, ctx->stream>>>(w, e.hi, e.lo, rows, c4_kh, c4_kw,
                                                                                    c4_cin, scale, alpha);
  else if (!k_major)
    split_tf32_transpose_kernel<<<grid_for(ctx, ((rows + 31) / 32) * ((k + 31) / 32) * 256, 256, 16), 256, 0,
                                  ctx->stream>>>(w, e.hi, e.lo, rows, k, scale, alpha);
  else
    split_tf32_kernel<<<grid_for(ctx, rows * k, 256, 8), 256, 0, ctx->stream>>>(w, e.hi, e.lo, rows * k, k, scale, alpha);
  s = wdc_check_launch(ctx, "split_tf32_kernel");
  if (s != WDC_OK) {
    wdc_free(ctx, e.hi);
    wdc_free(ctx, e.lo);
    return s;
  }
  e.born = ++ctx->split_seq;
  auto ins = st->weights.emplace(key, e);
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
    fn = nullptr;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess && fn) st->encode_im2col = (EncodeIm2colFn)fn;
    else cudaGetLastError();
  }
  if (!st->attr_set) {
    cudaError_t e = cudaFuncSetAttribute(tc_igemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(SharedStorage) + 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(tc_igemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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

// Describes the NHWC input as an im2col tensor map: box = TILE_M pixels x BLOCK_K channels, bounding
// box = the positions the filter's first tap takes (from -pad to the position of the last output
// pixel), traversal strides = the convolution's strides.  Returns false when the geometry does not
// fit the map's fields; the caller then launches the gathering kernel.
bool encode_a_map(TcState* st, const TcProblem& p, const float* x, CUtensorMap* map) {
  if (!st->encode_im2col || TC_DBG(p, 32)) return false;
  if (p.c4 && p.k_w > 8) return false;
  const int64_t hw = (int64_t)p.out_h * p.out_w;
  const int64_t images = (p.M + hw - 1) / hw;
  if (p.c4 == 2) {
    // pixel pairs of the physically padded rows: 8 channels per position, in_w_pad / 2 positions per row,
    // horizontal stride 1 and no horizontal padding; vertical geometry as given
    const int wpos = p.in_w_pad / 2;
    const int lower2[2] = {0, -p.pad_t};
    const int upper2[2] = {(p.out_w - 1) - (wpos - 1), -p.pad_t + (p.out_h - 1) * p.stride_h - (p.in_h - 1)};
    for (int i = 0; i < 2; i++)
      if (lower2[i] < -128 || upper2[i] < -128 || upper2[i] > 127) return false;
    if (p.stride_h < 1 || p.stride_h > 8 || (p.k_h - 1) * p.dil_h > 255 || images >= (1ll << 31)) return false;
    cuuint64_t dims2[4] = {8, (cuuint64_t)wpos, (cuuint64_t)p.in_h, (cuuint64_t)images};
    cuuint64_t strides2[3] = {32, (cuuint64_t)32 * wpos, (cuuint64_t)32 * wpos * p.in_h};
    cuuint32_t estr2[4] = {1, 1, (cuuint32_t)p.stride_h, 1};
    CUresult r2 = st->encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)x, dims2, strides2, lower2, upper2,
                                    8, TILE_M, estr2, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r2 == CUDA_SUCCESS;
  }
  const int lower[2] = {-p.pad_l, -p.pad_t};
  const int upper[2] = {-p.pad_l + (p.out_w - 1) * p.stride_w - (p.in_w - 1),
                        -p.pad_t + (p.out_h - 1) * p.stride_h - (p.in_h - 1)};
  for (int i = 0; i < 2; i++)
    if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return false;
  if (p.stride_w < 1 || p.stride_w > 8 || p.stride_h < 1 || p.stride_h > 8) return false;
  if ((p.k_w - 1) * p.dil_w > 255 || (p.k_h - 1) * p.dil_h > 255) return false;
  if ((p.ch_in & 3) || images >= (1ll << 31)) return false;
  cuuint64_t dims[4] = {(cuuint64_t)p.ch_in, (cuuint64_t)p.in_w, (cuuint64_t)p.in_h, (cuuint64_t)images};
  cuuint64_t strides[3] = {(cuuint64_t)p.ch_in * 4, (cuuint64_t)p.ch_in * 4 * p.in_w,
                           (cuuint64_t)p.ch_in * 4 * p.in_w * p.in_h};
  if (strides[2] >= (1ull << 40)) return false;
  cuuint32_t estr[4] = {1, (cuuint32_t)p.stride_w, (cuuint32_t)p.stride_h, 1};
  CUresult r = st->encode_im2col(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)x, dims, strides, lower, upper,
                                 p.c4 ? 4 : BLOCK_K, TILE_M, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 p.c4 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tile width and the treatment of the last, partly filled wave for an [M, N] output with `kblocks` K blocks.
// The widest tile is the cheapest per column (a 64-column MMA costs about 0.65 of a 128-column one, a 32-column
// one about 0.45), but tiles are dealt to the SMs in waves, and the tiles of the last wave (`rest`, fewer than the
// SMs) cost a whole tile time however few they are.  Those tiles can cut their reduction into `splits` ranges that
// run as separate work units (each at least 4 K blocks long, at most 8 ranges): the last wave then takes
// ceil(rest * splits / SMs) / splits of a tile time, plus a second, memory-bound pass over the rest tiles' partial
// sums, charged as a fixed 5 us (measured on ResNet-50's layers at batch 32: shorter reductions than about 20 K
// blocks lose more to that launch than the split wins).  The estimate picks width and split.
void choose_tiling(const wdc_context* ctx, int64_t m, int64_t n, int kblocks, bool may_split, int* tile_n,
                   int* splits, int* full_tiles) {
  const int widest = pick_tile_n(n);
  const double cost[3] = {0.45, 0.65, 1.0};
  const int sms = ctx->sm_count;
  double best_t = 1e300;
  *tile_n = widest;
  *splits = 1;
  *full_tiles = 0;
  for (int t = widest, i = widest == 128 ? 2 : widest == 64 ? 1 : 0; t >= 32; t >>= 1, i--) {
    const int64_t tiles = ceil_div64(m, TILE_M) * ceil_div64(n, t);
    if (tiles >= (1ll << 31) - 65536) continue;
    const int64_t waves = tiles / sms, rest = tiles - waves * sms;
    const double whole = (double)ceil_div64(tiles, sms) * cost[i];
    if (whole < best_t - 1e-9) {
      best_t = whole;
      *tile_n = t;
      *splits = 1;
      *full_tiles = (int)tiles;
    }
    if (!may_split || rest == 0) continue;
    for (int sp = 2; sp <= 8 && kblocks / sp >= 4; sp++) {
      const int kbs = (kblocks + sp - 1) / sp;
      if ((sp - 1) * kbs >= kblocks) continue;   // an empty last range
      // the second pass is a launch of its own: about 5 us, i.e. 12 / kblocks of a 128-column tile's time (a K block
      // of such a tile takes ~0.42 us), whatever the tile width
      const double est = ((double)waves + (double)ceil_div64(rest * sp, sms) * kbs / kblocks) * cost[i] + 12.0 / kblocks;
      if (est < best_t - 1e-9) {
        best_t = est;
        *tile_n = t;
        *splits = sp;
        *full_tiles = (int)(waves * sms);
      }
    }
  }
}

int launch_tc(wdc_context* ctx, TcProblem& p, const float* x, const float* w, float* y, int c4_kw = 0,
              int c4_cin = 0, bool w_k_major = true) {
  WeightEntry* we = nullptr;
  int s = get_weight(ctx, w, p.scale, p.alpha, p.N, p.K, &we, p.c4 ? p.K / 32 : 0, c4_kw, c4_cin, w_k_major);
  if (s != WDC_OK) return s;
  p.scale = nullptr;  // folded into the split weights
  p.alpha = 1.f;
  p.kblocks = p.c4 ? p.K / BLOCK_K : p.k_h * p.k_w * p.cblocks;   // K blocks are counted per filter tap
  {
    // a split reduction needs the TMA paths on both sides (checked again below) and no first-layer mode
    const bool may_split = !p.c4 && p.N % 4 == 0 && p.M < (1ll << 27) && tc_state(ctx)->encode_im2col != nullptr &&
                           (((uintptr_t)p.shift | (uintptr_t)p.residual | (uintptr_t)y) & 15) == 0 &&
                           (!p.residual || p.res_stride % 4 == 0) && ctx->opt_split_k;
    choose_tiling(ctx, p.M, p.N, p.kblocks, may_split, &p.tile_n, &p.splits, &p.full_tiles);
  }
  const int mi = p.tile_n == 128 ? 2 : p.tile_n == 64 ? 1 : 0;
  if (!we->has_map[mi]) {
    const int r1 = encode_map(tc_state(ctx), &we->map_hi[mi], we->hi, we->rows, we->k, p.tile_n);
    const int r2 = encode_map(tc_state(ctx), &we->map_lo[mi], we->lo, we->rows, we->k, p.tile_n);
    if (r1 || r2)
      return wdc_fail(ctx, WDC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d, %d) for a [%lld, %lld] weight", r1, r2,
                      (long long)we->rows, (long long)we->k);
    we->has_map[mi] = true;
  }
  const CUtensorMap& w_map_hi = we->map_hi[mi];
  const CUtensorMap& w_map_lo = we->map_lo[mi];
  if (ceil_div64(p.M, TILE_M) * ceil_div64(p.N, p.tile_n) >= (1ll << 31) - 65536) return WDC_ERR_UNSUPPORTED;
  p.tiles_m = (int)ceil_div64(p.M, TILE_M);
  p.tiles_n = (int)ceil_div64(p.N, p.tile_n);
  p.status = ctx->status_word;
  p.nap_ns = 100;
#ifdef WDC_TC_DEVELOP
  {
    static int dbg = -1;
    if (dbg < 0) {
      const char* e = getenv("WDC_TC_DEBUG");
      dbg = e ? atoi(e) : 0;
    }
    p.dbg = dbg;
    static int nap = -2;
    if (nap == -2) {
      const char* e = getenv("WDC_TC_NAP");
      nap = e ? atoi(e) : -1;
    }
    if (nap >= 0) p.nap_ns = (uint32_t)nap;
  }
  static long long* prof_buf = nullptr;
  static int prof_on = -1;
  if (prof_on < 0) prof_on = getenv("WDC_TC_PROF") ? 1 : 0;
  if (prof_on) {
    if (!prof_buf) cudaMalloc(&prof_buf, 256 * 16 * sizeof(long long));
    cudaMemsetAsync(prof_buf, 0, 256 * 16 * sizeof(long long), ctx->stream);
    p.prof = prof_buf;
  }
#endif
  p.single_pass = ctx->opt_precision == 1 ? 1 : 0;
  TcState* st = tc_state(ctx);
  const int total_tiles = p.tiles_m * p.tiles_n;
  float* ws = nullptr;
  CUtensorMap map_a;
  bool a_by_tma = encode_a_map(st, p, x, &map_a);
  if (!a_by_tma) p.splits = 1;   // geometry outside the im2col map: gathering producers, whole tiles only
  if (p.splits == 1) p.full_tiles = total_tiles;
  p.kbs = (p.kblocks + p.splits - 1) / p.splits;
  const int rest_tiles = total_tiles - p.full_tiles;
  // output, residual and split-range workspace as row-major matrices cut into 32-row x cw-column boxes for the
  // epilogue warps
  CUtensorMap map_y = w_map_hi, map_res = w_map_hi, map_ws = w_map_hi;
  {
    // (narrow tiles fed by TMA have four epilogue warps of tile_n columns each, all others eight of tile_n / 2)
    const int ncols = duo_mode(p, a_by_tma) ? p.tile_n : p.tile_n / 2, cw = ncols < 32 ? ncols : 32;
    bool can = (p.N % 4 == 0) && p.M < (1ll << 31) && !TC_DBG(p, 64) && (((uintptr_t)p.scale | (uintptr_t)p.shift) & 15) == 0;
    if (can) can = encode_rows_map(st, &map_y, y, p.M, p.N, p.N, cw) == 0;
    if (can && p.residual)
      can = p.res_stride % 4 == 0 && encode_rows_map(st, &map_res, p.residual, p.M, p.N, p.res_stride, cw) == 0;
    p.tma_epi = can ? 1 : 0;
    if (!can && p.splits > 1) {   // split ranges leave through the TMA epilogue only
      p.splits = 1;
      p.full_tiles = total_tiles;
      p.kbs = p.kblocks;
    }
    if (p.splits > 1) {
      const int64_t ws_rows = (int64_t)rest_tiles * p.splits * TILE_M;
      s = wdc_alloc(ctx, ws_rows * p.tile_n * 4, (void**)&ws);
      if (s != WDC_OK) return s;
      if (encode_rows_map(st, &map_ws, ws, ws_rows, p.tile_n, p.tile_n, cw) != 0) {
        wdc_free(ctx, ws);
        return wdc_fail(ctx, WDC_ERR_CUDA, "tensor map for the split-reduction workspace could not be encoded");
      }
    }
  }
  const int64_t units = (int64_t)p.full_tiles + (int64_t)(total_tiles - p.full_tiles) * p.splits;
  const int grid = (int)(units < ctx->sm_count ? units : ctx->sm_count);
  const size_t smem = sizeof(SharedStorage) + 1024;
  if (!a_by_tma && p.c4 == 2) {   // the paired layout exists only for the TMA path
    if (ws) wdc_free(ctx, ws);
    return WDC_ERR_UNSUPPORTED;
  }
  // Programmatic dependent launch: the grid may start while the previous grid of the stream drains; the kernel
  // itself waits (griddepcontrol.wait) before it touches anything an earlier grid wrote or still reads.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->opt_pdl ? 1 : 0;
  const TcProblem& pc = p;
  cudaError_t le;
  if (a_by_tma)
    le = cudaLaunchKernelEx(&cfg, tc_igemm_kernel<true>, pc, x, w_map_hi, w_map_lo, map_a, map_y, map_res, map_ws, y);
  else
    le = cudaLaunchKernelEx(&cfg, tc_igemm_kernel<false>, pc, x, w_map_hi, w_map_lo, w_map_hi, map_y, map_res, map_ws, y);
  ctx->n_tc_launch++;
  ctx->n_launch++;
  s = wdc_check_cuda(ctx, le, "tc_igemm_kernel");
  if (s == WDC_OK) s = wdc_check_cuda(ctx, cudaGetLastError(), "tc_igemm_kernel");
#ifdef WDC_TC_DEVELOP
  if (p.prof) {
    static long long host[256 * 16];
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(host, p.prof, sizeof(host), cudaMemcpyDeviceToHost);
    double acc[16] = {};
    for (int b = 0; b < grid; b++)
      for (int i = 0; i < 16; i++) acc[i] += (double)host[b * 16 + i] / grid;
    const double steps = (double)units * p.kbs / grid;   // K blocks per CTA (about)
    if (getenv("WDC_TC_TIMELINE")) {
      const long long* ev = host + 2368;
      const long long t0 = ev[0 * 64 + 8];
      fprintf(stderr, "timeline CTA 0 (cycles from K block 8): g | split a_full, empty, arrived | mma seg_empty, full, issued\n");
      for (int g = 8; g < 40; g++)
        fprintf(stderr, "  %2d | %6lld %6lld %6lld | %6lld %6lld %6lld\n", g, ev[g] - t0, ev[64 + g] - t0, ev[128 + g] - t0,
                ev[5 * 64 + g] ? ev[5 * 64 + g] - t0 : -1, ev[3 * 64 + g] - t0, ev[4 * 64 + g] - t0);
    }
    fprintf(stderr, "prof M=%lld N=%d kb=%d tile_n=%d c4=%d | per K block, cycles: split[a_full %.0f empty %.0f ld+st %.0f wait_st %.0f "
            "loop %.0f total %.0f] mma[seg_empty %.0f full %.0f loop %.0f mmas %.0f commit %.0f total %.0f]\n", (long long)p.M, p.N, p.kblocks, p.tile_n,
            p.c4, acc[0] / steps, acc[1] / steps, acc[2] / steps, acc[3] / steps, acc[4] / steps, acc[5] / steps, acc[6] / steps,
            acc[7] / steps, acc[8] / steps, acc[9] / steps, acc[10] / steps, acc[11] / steps);
    fprintf(stderr, "   blocking waits per K block: a_full %.2f empty %.2f full %.2f\n", acc[13] / steps, acc[14] / steps, acc[15] / steps);
  }
#endif
  if (p.splits > 1) {
    if (s == WDC_OK) {
      cudaLaunchConfig_t rc = {};
      rc.gridDim = dim3((unsigned)grid_for(ctx, (int64_t)rest_tiles * TILE_M * (p.tile_n / 4), 256, 8));
      rc.blockDim = dim3(256);
      rc.stream = ctx->stream;
      rc.attrs = attr;
      rc.numAttrs = ctx->opt_pdl ? 1 : 0;
      le = cudaLaunchKernelEx(&rc, splitk_reduce_kernel, (const float*)ws, y, p.shift, p.shift_mul, p.residual,
                              p.res_stride, p.res_mul, p.relu, p.M, p.N, p.tile_n, p.tiles_n, p.full_tiles, rest_tiles,
                              p.splits);
      ctx->n_launch++;
      s = wdc_check_cuda(ctx, le, "splitk_reduce_kernel");
      if (s == WDC_OK) s = wdc_check_cuda(ctx, cudaGetLastError(), "splitk_reduce_kernel");
    }
    wdc_free(ctx, ws);   // stream-ordered: reused only by work queued after the reduction
  }
  return s;
}

bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

}  // namespace

void wdc_tc_evict(wdc_context* ctx, const void* ptr, int64_t bytes) {
  if (!ctx->tc_state) return;
  TcState* st = (TcState*)ctx->tc_state;
  if (st->weights.empty()) return;
  // written extent: the byte range, widened to the arena allocation that contains its start
  const char* lo = (const char*)ptr;
  const char* hi = lo + (bytes > 0 ? bytes : 1);
  const char *blo, *bhi;
  if (wdc_arena_extent(ctx, ptr, &blo, &bhi)) {
    if (blo < lo) lo = blo;
    if (bhi > hi) hi = bhi;
  }
  // entries whose weight buffer or per-channel scale vector overlaps [lo, hi)
  std::vector<WeightEntry> dropped;
  for (auto it = st->weights.begin(); it != st->weights.end();) {
    const char* w = (const char*)it->first.w;
    const char* sc = (const char*)it->first.scale;
    const bool hit = (w < hi && lo < w + it->second.src_bytes) || (sc && sc < hi && lo < sc + it->second.rows * 4);
    if (hit) {
      dropped.push_back(it->second);
      it = st->weights.erase(it);
    } else {
      ++it;
    }
  }
  for (const WeightEntry& e : dropped) {   // wdc_free re-enters this function: the map is already consistent
    wdc_graphs_note_evicted(ctx, e.born);
    wdc_free(ctx, e.hi);
    wdc_free(ctx, e.lo);
  }
}

void wdc_tc_destroy(wdc_context* ctx) {
  if (!ctx->tc_state) return;
  delete (TcState*)ctx->tc_state;  // the split buffers die with the arena slabs
  ctx->tc_state = nullptr;
}

int wdc_tc_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w, const float* scale,
                  const float* shift, const float* residual, float* y) {
  const bool stem = d->group == 1 && d->ch_in <= 4 && d->k_w <= 8 && d->ch_out % 4 == 0;
  if (d->x_nchw && !stem) return WDC_ERR_UNSUPPORTED;
  if (!stem && (d->group != 1 || d->ch_in % 4 != 0 || d->ch_out % 4 != 0)) return WDC_ERR_UNSUPPORTED;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (residual && !aligned16(residual))) return WDC_ERR_UNSUPPORTED;
  const int64_t K = d->ch_in * d->k_h * d->k_w;
  if (K > (1 << 30) || d->ch_out > (1 << 24)) return WDC_ERR_UNSUPPORTED;
  if (!tc_ready(ctx)) return WDC_ERR_UNSUPPORTED;
  TcProblem p = {};
  p.M = d->batch * d->out_h * d->out_w;
  p.N = (int)d->ch_out;
  p.K = (int)K;
  p.ch_in = (int)d->ch_in; p.in_h = (int)d->in_h; p.in_w = (int)d->in_w;
  p.out_h = (int)d->out_h; p.out_w = (int)d->out_w; p.k_h = (int)d->k_h; p.k_w = (int)d->k_w;
  p.stride_h = (int)d->stride_h; p.stride_w = (int)d->stride_w; p.pad_t = (int)d->pad_t; p.pad_l = (int)d->pad_l;
  p.dil_h = (int)d->dil_h; p.dil_w = (int)d->dil_w;
  p.cblocks = (int)((d->ch_in + BLOCK_K - 1) / BLOCK_K);
  p.scale = scale; p.shift = shift; p.residual = residual; p.res_stride = d->ch_out;
  p.alpha = 1.f; p.shift_mul = 1.f; p.res_mul = 1.f; p.relu = d->relu;
  if (!stem) return launch_tc(ctx, p, x, w, y);
  // Few input channels (the network's first convolution): pad the pixels to 4 channels so that one
  // 16-byte chunk is one pixel, and lay the filter out as 8 taps x 4 channels per filter row.
  float* x4 = nullptr;
  // stride-2 stems: pad the rows physically so that two taps are one 32-byte pixel pair
  const bool pairs = d->stride_w == 2 && d->dil_w == 1 && tc_state(ctx)->encode_im2col != nullptr;
  const int wp = pairs ? (int)(2 * d->out_w + 6) : (int)d->in_w;
  const int hp = (int)d->in_h;
  const int64_t pixels = d->batch * hp * wp;
  int s = wdc_alloc(ctx, pixels * 16, (void**)&x4);
  if (s != WDC_OK) return s;
  if (pairs)
    pad_channels4_rows_kernel<<<grid_for(ctx, pixels, 256, 8), 256, 0, ctx->stream>>>(
        x, x4, d->batch, (int)d->in_h, hp, 0, (int)d->in_w, wp, (int)d->pad_l, (int)d->ch_in,
        d->x_nchw ? 1 : 0);
  else
    pad_channels4_kernel<<<grid_for(ctx, pixels, 256, 8), 256, 0, ctx->stream>>>(x, x4, pixels, (int)d->ch_in,
                                                                                 d->x_nchw ? d->in_h * d->in_w : 0);
  s = wdc_check_launch(ctx, "pad_channels4_kernel");
  if (s == WDC_OK) {
    p.c4 = pairs ? 2 : 1;
    p.in_w_pad = wp;
    p.ch_in = 4;
    p.K = (int)d->k_h * 32;
    p.cblocks = 1;
    s = launch_tc(ctx, p, x4, w, y, (int)d->k_w, (int)d->ch_in);
  }
  wdc_free(ctx, x4);
  return s;
}

int wdc_tc_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B, const float* C,
                float* Y) {
  // A [m, k] with k contiguous; B either [n, k] with k contiguous (Gemm transB=1, LSTM weights) or [k, n] with n
  // contiguous (MatMul, Gemm transB=0: transposed while it is split).  A batch whose B is shared (stride 0) and
  // whose A and Y are stacked without gaps is one tall matrix.
  int64_t m = d->m;
  if (d->batch != 1) {
    if (d->sbb != 0 || d->sab != d->m * d->sa0 || C) return WDC_ERR_UNSUPPORTED;
    m = d->batch * d->m;
  }
  const bool b_k_major = d->sb0 == 1 && d->sb1 == d->k;
  const bool b_n_major = d->sb1 == 1 && d->sb0 == d->n;
  if (d->sa1 != 1 || d->sa0 != d->k || !(b_k_major || b_n_major)) return WDC_ERR_UNSUPPORTED;
  if (d->k % 4 != 0 || d->k < 32 || m < 32) return WDC_ERR_UNSUPPORTED;
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
  p.M = m;
  p.N = (int)d->n;
  p.K = (int)d->k;
  p.ch_in = (int)d->k; p.in_h = 1; p.in_w = 1; p.out_h = 1; p.out_w = 1; p.k_h = 1; p.k_w = 1;
  p.stride_h = p.stride_w = 1; p.dil_h = p.dil_w = 1;
  p.cblocks = (int)((d->k + BLOCK_K - 1) / BLOCK_K);
  p.shift = shift; p.residual = residual; p.res_stride = res_stride;
  p.alpha = d->alpha; p.shift_mul = d->beta; p.res_mul = d->beta; p.relu = d->relu;
  return launch_tc(ctx, p, A, B, Y, 0, 0, b_k_major);
}
