// ONNX LSTM recurrence (forward, default activations, gate order i,o,f,c) as ONE persistent kernel.
//
// The input projection P[T, B, 4H] = X * W^T of all steps is a tensor-core GEMM done beforehand; what
// is left is the serial part: for t = 0..T-1, G = h_{t-1} * R^T + P_t, gates, c_t, h_t.  Launched per
// step it costs two launches and a round trip through HBM for G; here the whole recurrence is one
// cooperative launch:
//   * CTA g owns U hidden units (U = 4 or 8) and keeps their 4*U rows of R in shared memory for the
//     whole sequence (R is read from HBM once), and the cell state c of its units in registers;
//   * per step it loads h_{t-1} [B, H] (written by all CTAs into Y[t-1]) into shared memory, computes
//     its B x 4U pre-activations with fp32 FMAs (thread tile 8 batch rows x 4 gates of one unit, K split
//     over 8 thread groups, 16-byte shared-memory reads: 12 per 128 FMAs), reduces the partial sums, applies the gate
//     non-linearities for its units (a thread holds all four gates of its (row, unit) pair, so no
//     exchange is needed), and writes its U columns of h_t straight into Y[t];
//   * the CTAs meet at a per-step counter in global memory (release: __syncthreads + fence + atomicAdd;
//     acquire: polling load + __syncthreads), one counter per step so nothing is ever reset.
// The launch is cooperative, so all CTAs are resident at once, which the counter protocol needs.
// Every wait is bounded (2 s of %globaltimer): on expiry the CTA sets the context's status word and
// an abort word that every other CTA's polling loop also watches, and all CTAs return.
//
// Shapes it takes: B <= 64, H % 32 == 0, H / U <= number of SMs for U in {4, 8}, and
// (B + 4U) * (H + 4) * 4 + 128 * B * U bytes of shared memory <= 226 KB (config: B = 64, H = 512).
// Everything else returns WDC_ERR_UNSUPPORTED and wdc_lstm runs its per-step path.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kMaxDynSmem = 226 * 1024;   // the opt-in maximum minus room for the kernel's static shared memory
constexpr int KS = 8;                     // K slices (thread groups) per CTA
constexpr unsigned long long WAIT_NS = 2000000000ull;

struct LstmArgs {
  const float* P;      // [T, B, 4H] input projection without bias
  const float* R;      // [4H, H]
  const float* bias;   // [8H] or null
  const float* h0;     // [B, H] or null
  const float* c0;     // [B, H] or null
  float* Y;            // [T, B, H]
  float* Yh;           // [B, H]
  float* Yc;           // [B, H]
  unsigned int* counters;  // [T + 1]: arrivals per step; last word = abort flag
  int* status;
  int T, B, H;
  unsigned long long wait_ns;   // limit of every wait (WAIT_NS; the self-test passes about a millisecond)
  unsigned int arrivals;        // arrivals that complete a step: the grid size (the self-test asks for one more)
};

__device__ __forceinline__ float sigmoid_ref(float x) { return (tanhf(x * 0.5f) + 1.f) * 0.5f; }

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits until `*counter >= target`.  Returns false if the wait was abandoned.
__device__ bool wait_counter(const unsigned int* counter, unsigned int target, unsigned int* abort_word, int* status,
                             int code, unsigned long long limit_ns) {
  for (int i = 0; i < 4096; i++)
    if (ld_acquire(counter) >= target) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; i++)
      if (ld_acquire(counter) >= target) return true;
    if (ld_acquire(abort_word) != 0) return false;
    if (global_ns() - t0 > limit_ns) {
      atomicExch(abort_word, 1u);
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

// Bounded wait for the bulk copies of one step.  Returns false if the wait was abandoned.
__device__ bool wait_copies(unsigned long long* bar, uint32_t parity, unsigned int* abort_word, int* status, int code,
                            unsigned long long limit_ns) {
  for (int i = 0; i < 4096; i++)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 256; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (ld_acquire(abort_word) != 0) return false;
    if (global_ns() - t0 > limit_ns) {
      atomicExch(abort_word, 1u);
      atomicCAS(status, 0, code);
      return false;
    }
  }
}

template <int U>
__global__ void __launch_bounds__(64 * U, 1) lstm_persistent_kernel(const LstmArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = a.H, B = a.B, T = a.T;
  const int ld = H + 4;                                  // row pitch: (H + 4) / 4 is odd -> conflict-free 16-byte reads
  float* h_s = reinterpret_cast<float*>(smem_raw);       // [B][ld]
  float* r_s = h_s + (size_t)B * ld;                     // [4 * U][ld], row = gate * U + unit
  float4* part = reinterpret_cast<float4*>(r_s + (size_t)4 * U * ld);  // [KS][B * U] (4 gates each)
  __shared__ int s_ok, s_ok_copies;   // outcomes of the two bounded waits of a step (thread 0 decides for the CTA)
  __shared__ __align__(8) unsigned long long h_bar;   // completion of the bulk copies of h_{t-1}

  const int tid = threadIdx.x;
  const int u0 = blockIdx.x * U;
  unsigned int* abort_word = a.counters + T;

  // thread roles for the dot products: 8 lanes = 8 row groups of one unit (rows bg, bg+8, ..), so that the
  // 8 lanes of a quarter warp read 8 different 16-byte bank groups of h_s and one address of r_s
  const int ks = tid / (8 * U);
  const int r = tid % (8 * U);
  const int bg = r % 8, u = r / 8;
  int rows[8];
#pragma unroll
  for (int i = 0; i < 8; i++) rows[i] = min(bg + 8 * i, B - 1);   // rows past B repeat the last one; never stored
  const int kbeg = ks * (H / KS), kend = kbeg + H / KS;
  // thread role for the gate stage: one (row, unit) pair, cell state in a register
  const bool fin = tid < B * U;
  const int fb = tid / U, fu = tid % U;
  float c_reg = 0.f, h_reg = 0.f;
  float bsum[4] = {0.f, 0.f, 0.f, 0.f};
  if (fin) {
    if (a.c0) c_reg = a.c0[(size_t)fb * H + u0 + fu];
    if (a.bias) {
#pragma unroll
      for (int g = 0; g < 4; g++) bsum[g] = a.bias[g * H + u0 + fu] + a.bias[(4 + g) * H + u0 + fu];
    }
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&h_bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // this CTA's rows of R stay in shared memory for the whole sequence
  for (int i = tid; i < 4 * U * (H / 4); i += blockDim.x) {
    const int row = i / (H / 4), k4 = i % (H / 4);
    const int g = row / U, uu = row % U;
    const float4 v = __ldg(reinterpret_cast<const float4*>(a.R + ((size_t)g * H + u0 + uu) * H) + k4);
    *reinterpret_cast<float4*>(r_s + (size_t)row * ld + k4 * 4) = v;
  }
  __syncthreads();   // r_s filled, h_bar initialised

  int copies = 0;   // bulk-copy rounds completed on h_bar
  for (int t = 0; t < T; t++) {
    // projected input of this step for the (row, unit) pair: in flight during the wait and the dot products
    float pin[4] = {0.f, 0.f, 0.f, 0.f};
    if (fin) {
      const float* p = a.P + ((size_t)t * B + fb) * 4 * H + u0 + fu;
#pragma unroll
      for (int g = 0; g < 4; g++) pin[g] = __ldg(p + (size_t)g * H);
    }
    // h_{t-1}: h0 (or zero) for the first step, else Y[t-1] once every CTA has written its columns
    if (t > 0) {
      if (tid == 0)
        s_ok = wait_counter(a.counters + (t - 1), a.arrivals, abort_word, a.status, 61, a.wait_ns) ? 1 : 0;
      __syncthreads();
      if (!s_ok) return;
    }
    const float* hsrc = t > 0 ? a.Y + (size_t)(t - 1) * B * H : a.h0;
    if (hsrc) {
      // one bulk copy per row (global -> shared, 16-byte aligned on both sides), issued by the lanes
      // of warp 0; the rows were written by other SMs with ordinary stores, so order the async proxy
      // after the acquire above
      if (tid < 32) {
        asm volatile("fence.proxy.async;" ::: "memory");
        if (tid == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&h_bar)),
                       "r"((uint32_t)(B * H * 4))
                       : "memory");
        __syncwarp();
        for (int b = tid; b < B; b += 32)
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                  smem_addr(h_s + (size_t)b * ld)),
              "l"(hsrc + (size_t)b * H), "r"((uint32_t)(H * 4)), "r"(smem_addr(&h_bar))
              : "memory");
      }
      // One thread runs the bounded wait and the whole CTA follows its outcome, so that on expiry every thread
      // leaves together (no thread is left behind at a later __syncthreads).  After the barrier each thread
      // observes the completed phase itself, which is what orders its reads after the copies' writes; the
      // phase cannot advance before the next step's expect_tx, so this returns at the first poll.
      if (tid == 0)
        s_ok_copies = wait_copies(&h_bar, (uint32_t)(copies & 1), abort_word, a.status, 62, a.wait_ns) ? 1 : 0;
      __syncthreads();
      if (!s_ok_copies) return;
      for (int i = 0; i < (1 << 20) && !mbar_try_wait(&h_bar, (uint32_t)(copies & 1)); i++) {}
      copies++;
    } else {
      for (int i = tid; i < B * (H / 4); i += blockDim.x) {
        const int b = i / (H / 4), k4 = i % (H / 4);
        *reinterpret_cast<float4*>(h_s + (size_t)b * ld + k4 * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      __syncthreads();
    }

    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
      for (int g = 0; g < 4; g++) acc[i][g] = 0.f;
#pragma unroll 2
    for (int k = kbeg; k < kend; k += 4) {
      float4 hv[8], rv[4];
#pragma unroll
      for (int i = 0; i < 8; i++) hv[i] = *reinterpret_cast<const float4*>(h_s + (size_t)rows[i] * ld + k);
#pragma unroll
      for (int g = 0; g < 4; g++) rv[g] = *reinterpret_cast<const float4*>(r_s + (size_t)(g * U + u) * ld + k);
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int g = 0; g < 4; g++) {
          acc[i][g] = fmaf(hv[i].x, rv[g].x, acc[i][g]);
          acc[i][g] = fmaf(hv[i].y, rv[g].y, acc[i][g]);
          acc[i][g] = fmaf(hv[i].z, rv[g].z, acc[i][g]);
          acc[i][g] = fmaf(hv[i].w, rv[g].w, acc[i][g]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int b = bg + 8 * i;
      if (b < B) part[(size_t)ks * B * U + b * U + u] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    }
    __syncthreads();

    if (fin) {
      float g4[4] = {pin[0] + bsum[0], pin[1] + bsum[1], pin[2] + bsum[2], pin[3] + bsum[3]};
#pragma unroll
      for (int s = 0; s < KS; s++) {
        const float4 v = part[(size_t)s * B * U + fb * U + fu];
        g4[0] += v.x; g4[1] += v.y; g4[2] += v.z; g4[3] += v.w;
      }
      const float it = sigmoid_ref(g4[0]), ot = sigmoid_ref(g4[1]), ft = sigmoid_ref(g4[2]), ct = tanhf(g4[3]);
      c_reg = ft * c_reg + it * ct;
      h_reg = ot * tanhf(c_reg);
      a.Y[((size_t)t * B + fb) * H + u0 + fu] = h_reg;
    }
    // publish this CTA's columns of h_t
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      atomicAdd(a.counters + t, 1u);
    }
  }
  if (fin) {
    if (T == 0) {
      h_reg = a.h0 ? a.h0[(size_t)fb * H + u0 + fu] : 0.f;
    }
    a.Yh[(size_t)fb * H + u0 + fu] = h_reg;
    a.Yc[(size_t)fb * H + u0 + fu] = c_reg;
  }
}

template <int U>
int launch_persistent(wdc_context* ctx, LstmArgs& args, size_t smem) {
  static bool attr_set[64] = {};
  auto kernel = lstm_persistent_kernel<U>;
  if (!attr_set[ctx->device & 63]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) !=
        cudaSuccess) {
      cudaGetLastError();
      return WDC_ERR_UNSUPPORTED;
    }
    attr_set[ctx->device & 63] = true;
  }
  const int grid = args.H / U;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 64 * U, smem) != cudaSuccess || per_sm < 1 ||
      (int64_t)per_sm * ctx->sm_count < grid) {
    cudaGetLastError();
    return WDC_ERR_UNSUPPORTED;  // not all CTAs would be resident at once
  }
  void* params[] = {(void*)&args};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)kernel, dim3(grid), dim3(64 * U), params, smem, ctx->stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return WDC_ERR_UNSUPPORTED;
  }
  return wdc_check_launch(ctx, "lstm_persistent_kernel");
}

}  // namespace

// Runs the recurrence on the projected input P.  WDC_ERR_UNSUPPORTED: shape outside the kernel's range
// (nothing has been written); any other non-zero status is an error.
int wdc_lstm_persistent(wdc_context* ctx, const float* P, const float* R, const float* bias, const float* h0,
                        const float* c0, float* Y, float* Yh, float* Yc, int64_t T, int64_t Bt, int64_t H,
                        int64_t selftest_wait_ns) {
  if (Bt > 64 || H % 32 != 0 || T > (1 << 24) || T < 1) return WDC_ERR_UNSUPPORTED;
  if ((((uintptr_t)P | (uintptr_t)R | (uintptr_t)Y | (uintptr_t)h0) & 15) != 0) return WDC_ERR_UNSUPPORTED;
  int U = 0;
  for (int cand : {4, 8})
    if (!U && H % cand == 0 && H / cand <= ctx->sm_count) U = cand;
  if (!U) return WDC_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(Bt + 4 * U) * (H + 4) * 4 + (size_t)KS * Bt * U * 16;
  if (smem > (size_t)kMaxDynSmem) return WDC_ERR_UNSUPPORTED;
  static int coop[64] = {};  // 0 unknown, 1 yes, -1 no
  if (!coop[ctx->device & 63]) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, ctx->device);
    coop[ctx->device & 63] = v ? 1 : -1;
  }
  if (coop[ctx->device & 63] < 0) return WDC_ERR_UNSUPPORTED;
  unsigned int* counters = nullptr;
  int s = wdc_alloc(ctx, (T + 1) * 4, (void**)&counters);
  if (s != WDC_OK) return s;
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)(T + 1) * 4, ctx->stream);
  if (e != cudaSuccess) {
    wdc_free(ctx, counters);
    return wdc_check_cuda(ctx, e, "cudaMemsetAsync");
  }
  LstmArgs args = {P, R, bias, h0, c0, Y, Yh, Yc, counters, ctx->status_word, (int)T, (int)Bt, (int)H,
                   WAIT_NS, (unsigned)(H / U)};
  if (selftest_wait_ns > 0) {   // wdc_selftest_device_wait: a step that can never complete, and a short limit
    args.wait_ns = (unsigned long long)selftest_wait_ns;
    args.arrivals = (unsigned)(H / U) + 1u;
  }
  s = U == 4 ? launch_persistent<4>(ctx, args, smem) : launch_persistent<8>(ctx, args, smem);
  wdc_free(ctx, counters);  // stream-ordered arena: reused only by work queued after this launch
  return s;
}
