// ONNX LSTM (forward, default activations, gate order i,o,f,c).
// Step 1: one GEMM projects all T steps of the input: P[T*Bt, 4H] = X * W^T.
// Step 2: the recurrence, as one persistent cooperative kernel (lstm_persistent.cu) when the shape
// fits it; otherwise per time step G = h_{t-1} * R^T + P_t (GEMM with P_t as the C operand) and a
// fused gate kernel that applies bias, sigmoid/tanh, updates c and h and writes Y_t.
// Scratch (P, G, and the running h/c state) comes from the context arena.
#include <math.h>

#include "common.cuh"

int wdc_simt_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B, const float* C,
                  float* Y);
int wdc_simt_preload(wdc_context* ctx);
int wdc_lstm_persistent(wdc_context* ctx, const float* P, const float* R, const float* bias, const float* h0,
                        const float* c0, float* Y, float* Yh, float* Yc, int64_t T, int64_t Bt, int64_t H,
                        int64_t selftest_wait_ns = 0);

__device__ __forceinline__ float sigmoid_ref(float x) { return (tanhf(x * 0.5f) + 1.f) * 0.5f; }

// G [Bt, 4H] holds pre-activations without bias.  bias [8H] = Wb (i,o,f,c) then Rb (i,o,f,c).
__global__ void __launch_bounds__(256) lstm_gate_kernel(const float* __restrict__ G,
                                                        const float* __restrict__ bias,
                                                        float* __restrict__ c, float* __restrict__ h,
                                                        float* __restrict__ y_t, int64_t Bt, int64_t H) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (; i < Bt * H; i += step) {
    int64_t b = i / H, j = i % H;
    const float* g = G + b * 4 * H;
    float gi = g[j], go = g[H + j], gf = g[2 * H + j], gc = g[3 * H + j];
    if (bias) {
      gi += bias[j] + bias[4 * H + j];
      go += bias[H + j] + bias[5 * H + j];
      gf += bias[2 * H + j] + bias[6 * H + j];
      gc += bias[3 * H + j] + bias[7 * H + j];
    }
    float it = sigmoid_ref(gi), ot = sigmoid_ref(go), ft = sigmoid_ref(gf), ct = tanhf(gc);
    float cn = ft * c[i] + it * ct;
    float hn = ot * tanhf(cn);
    c[i] = cn;
    h[i] = hn;
    y_t[i] = hn;
  }
}

extern "C" int wdc_lstm(wdc_context* ctx, const float* X, const float* W, const float* R, const float* bias,
                        const float* h0, const float* c0, float* Y, float* Yh, float* Yc, int64_t T,
                        int64_t Bt, int64_t I, int64_t H) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_lstm: null context");
  wdc_note_write(ctx, Yc);
  wdc_note_write(ctx, Yh);
  wdc_note_write(ctx, Y);
  WDC_REQUIRE(ctx, T >= 0 && Bt > 0 && I > 0 && H > 0, "wdc_lstm: bad shape");
  WDC_REQUIRE(ctx, X && W && R && Yh && Yc && (T == 0 || Y), "wdc_lstm: null buffer");
  DeviceGuard g(ctx->device);
  float *P = nullptr, *G = nullptr;
  int s = wdc_alloc(ctx, (T > 0 ? T : 1) * Bt * 4 * H * 4, (void**)&P);
  if (s != WDC_OK) return s;
  if (T > 0) {
    wdc_gemm_desc d = {};
    d.batch = 1; d.m = T * Bt; d.n = 4 * H; d.k = I;
    d.sa0 = I; d.sa1 = 1; d.sb0 = 1; d.sb1 = I;  // B = W^T
    d.alpha = 1.f; d.beta = 0.f;
    s = wdc_gemm(ctx, &d, X, W, nullptr, P);
    if (s != WDC_OK) {
      wdc_free(ctx, P);
      return s;
    }
    // the whole recurrence as one persistent kernel when the shape fits it
    s = wdc_lstm_persistent(ctx, P, R, bias, h0, c0, Y, Yh, Yc, T, Bt, H);
    if (s != WDC_ERR_UNSUPPORTED) {
      wdc_free(ctx, P);
      return s;
    }
  }
  s = wdc_alloc(ctx, Bt * 4 * H * 4, (void**)&G);
  if (s != WDC_OK) {
    wdc_free(ctx, P);
    return s;
  }
  // running state lives directly in the Yh / Yc outputs
  if (h0) s = wdc_copy(ctx, Yh, h0, Bt * H * 4);
  else s = wdc_fill_u32(ctx, Yh, 0u, Bt * H);
  if (s == WDC_OK) {
    if (c0) s = wdc_copy(ctx, Yc, c0, Bt * H * 4);
    else s = wdc_fill_u32(ctx, Yc, 0u, Bt * H);
  }
  for (int64_t t = 0; t < T && s == WDC_OK; t++) {
    wdc_gemm_desc d = {};
    d.batch = 1; d.m = Bt; d.n = 4 * H; d.k = H;
    d.sa0 = H; d.sa1 = 1; d.sb0 = 1; d.sb1 = H;  // B = R^T
    d.sc0 = 4 * H; d.sc1 = 1;
    d.alpha = 1.f; d.beta = 1.f;
    s = wdc_gemm(ctx, &d, Yh, R, P + t * Bt * 4 * H, G);
    if (s != WDC_OK) break;
    lstm_gate_kernel<<<grid_for(ctx, Bt * H, 256, 4), 256, 0, ctx->stream>>>(G, bias, Yc, Yh,
                                                                            Y + t * Bt * H, Bt, H);
    s = wdc_check_launch(ctx, "lstm_gate_kernel");
  }
  wdc_free(ctx, G);
  wdc_free(ctx, P);
  return s;
}

// Self-test of the bounded device waits: runs the persistent recurrence kernel on a small zero-filled problem
// (2 steps, batch 8, hidden 128: 32 CTAs) whose first step is told to wait for one arrival more than there are
// CTAs, with `limit_ns` as the limit of every wait.  The wait runs out, the kernel records its status, raises its
// abort word, every CTA returns, and the context stays usable: the next wdc_sync reports WDC_ERR_DEVICE_WAIT once.
extern "C" int wdc_selftest_device_wait(wdc_context* ctx, int64_t limit_ns) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_selftest_device_wait: null context");
  WDC_REQUIRE(ctx, limit_ns >= 1000 && limit_ns <= 1000000000ll,
              "wdc_selftest_device_wait: limit of %lld ns is outside 1 us .. 1 s", (long long)limit_ns);
  DeviceGuard g(ctx->device);
  const int64_t T = 2, Bt = 8, H = 128;
  const int64_t n_p = T * Bt * 4 * H, n_r = 4 * H * H, n_y = T * Bt * H, n_s = Bt * H;
  float* buf = nullptr;
  int s = wdc_alloc(ctx, (n_p + n_r + n_y + 2 * n_s) * 4, (void**)&buf);
  if (s != WDC_OK) return s;
  s = wdc_fill_u32(ctx, buf, 0u, n_p + n_r + n_y + 2 * n_s);
  if (s == WDC_OK) {
    float *P = buf, *R = P + n_p, *Y = R + n_r, *Yh = Y + n_y, *Yc = Yh + n_s;
    s = wdc_lstm_persistent(ctx, P, R, nullptr, nullptr, nullptr, Y, Yh, Yc, T, Bt, H, limit_ns);
    if (s == WDC_ERR_UNSUPPORTED)
      s = wdc_fail(ctx, WDC_ERR_UNSUPPORTED, "wdc_selftest_device_wait: the persistent kernel cannot run on this device");
  }
  wdc_free(ctx, buf);   // stream-ordered
  return s;
}

// ------------------------------------------------------------------------------------------------
// wdc_lstm_static: the same LSTM for callers that must not allocate.
//
// Some hosts of this library cannot take a device allocation in the middle of their work: a runtime
// that has handed all of the GPU's memory to its own pool, a real-time loop that may not block in
// the driver's allocator, a plug-in sandbox that forbids cudaMalloc after start-up.  wdc_lstm needs
// scratch (the projected inputs of all steps and one step's gate pre-activations) and takes it from
// the context arena, which may have to grow.  This variant keeps its scratch in a fixed array that
// is part of the loaded library image instead: kLstmStaticFloats floats (4 MiB) per GPU that loads
// the library, held until the process exits.  To stay inside that budget it projects the input one
// step at a time, so the scratch is one [batch, 4*hidden] block, and it runs both contractions on
// the CUDA-core kernel, whose launch allocates nothing (the tensor-core path caches a split copy of
// its weights in the arena).
//
// In host code the array's name is only a handle for the symbol, not a device address; the address
// comes from cudaGetSymbolAddress, asked once per device with that device current.  wdc_create does
// that lookup for its device (wdc_lstm_static_setup below), because the lookup is also the moment
// the CUDA driver loads this file's module and sets the 4 MiB array aside: a context created at
// start-up has therefore paid for the array before the first wdc_lstm_static call, and that call
// touches no allocator at all, not even the driver's module loader.  Should the address of a device
// still be unknown when wdc_lstm_static runs (it cannot be after a successful wdc_create), the call
// looks it up itself; such a first call must come before any stream capture.
// All calls on a device share the one array: it holds whatever the previous call left (nothing here
// needs to start at zero: every step overwrites the block before reading it), and two calls that
// overlap on the GPU (different streams or contexts of one device) would race on it.
constexpr int64_t kLstmStaticFloats = 1 << 20;
static __device__ __align__(256) float g_lstm_static_scratch[kLstmStaticFloats];

static float* g_lstm_static_ptr[64] = {};  // per-device address of the array, filled by wdc_lstm_static_setup

// Resolves the array's device address for the context's device (which must be current).  Called by
// wdc_create; the first lookup on a device makes the driver load this module and reserve the array.
int wdc_lstm_static_setup(wdc_context* ctx) {
  if (ctx->device < 0 || ctx->device >= 64) return WDC_OK;   // wdc_lstm_static refuses such a device itself
  if (g_lstm_static_ptr[ctx->device]) return WDC_OK;
  float* p = nullptr;
  WDC_CUDA(ctx, cudaGetSymbolAddress((void**)&p, g_lstm_static_scratch));
  // the kernels wdc_lstm_static launches live in three modules; with lazy module loading a module's code is
  // placed in device memory at its first use, so touch them now as well
  cudaFuncAttributes fa;
  WDC_CUDA(ctx, cudaFuncGetAttributes(&fa, lstm_gate_kernel));
  int s = wdc_simt_preload(ctx);
  if (s != WDC_OK) return s;
  g_lstm_static_ptr[ctx->device] = p;
  return WDC_OK;
}

extern "C" int wdc_lstm_static(wdc_context* ctx, const float* X, const float* W, const float* R,
                               const float* bias, const float* h0, const float* c0, float* Y, float* Yh,
                               float* Yc, int64_t T, int64_t Bt, int64_t I, int64_t H) {
  if (!ctx) return wdc_fail(ctx, WDC_ERR_INVALID, "wdc_lstm_static: null context");
  wdc_note_write(ctx, Yc);
  wdc_note_write(ctx, Yh);
  wdc_note_write(ctx, Y);
  WDC_REQUIRE(ctx, T >= 0 && Bt > 0 && I > 0 && H > 0, "wdc_lstm_static: bad shape");
  WDC_REQUIRE(ctx, X && W && R && Yh && Yc && (T == 0 || Y), "wdc_lstm_static: null buffer");
  if (Bt * 4 * H > kLstmStaticFloats)
    return wdc_fail(ctx, WDC_ERR_UNSUPPORTED,
                    "wdc_lstm_static: batch * 4 * hidden_size = %lld exceeds the static scratch of %lld floats; "
                    "use wdc_lstm",
                    (long long)(Bt * 4 * H), (long long)kLstmStaticFloats);
  WDC_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "wdc_lstm_static: device index out of range");
  DeviceGuard g(ctx->device);
  {
    int s0 = wdc_lstm_static_setup(ctx);   // a no-op after wdc_create
    if (s0 != WDC_OK) return s0;
  }
  float* G = g_lstm_static_ptr[ctx->device];
  int s;
  if (h0) s = wdc_copy(ctx, Yh, h0, Bt * H * 4);
  else s = wdc_fill_u32(ctx, Yh, 0u, Bt * H);
  if (s == WDC_OK) {
    if (c0) s = wdc_copy(ctx, Yc, c0, Bt * H * 4);
    else s = wdc_fill_u32(ctx, Yc, 0u, Bt * H);
  }
  for (int64_t t = 0; t < T && s == WDC_OK; t++) {
    wdc_gemm_desc d = {};
    d.batch = 1; d.m = Bt; d.n = 4 * H; d.k = I;
    d.sa0 = I; d.sa1 = 1; d.sb0 = 1; d.sb1 = I;   // G = X_t * W^T
    d.alpha = 1.f; d.beta = 0.f;
    s = wdc_simt_gemm(ctx, &d, X + t * Bt * I, W, nullptr, G);
    if (s != WDC_OK) break;
    d.k = H; d.sa0 = H; d.sb1 = H;                // G += h * R^T: C == Y selects the kernel's in-place mode, which
    d.sc0 = 4 * H; d.sc1 = 1; d.beta = 1.f;       // reads the old value through the output pointer with a plain load
    s = wdc_simt_gemm(ctx, &d, Yh, R, G, G);
    if (s != WDC_OK) break;
    lstm_gate_kernel<<<grid_for(ctx, Bt * H, 256, 4), 256, 0, ctx->stream>>>(G, bias, Yc, Yh, Y + t * Bt * H, Bt, H);
    s = wdc_check_launch(ctx, "lstm_gate_kernel");
  }
  return s;
}
