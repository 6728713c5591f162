// ONNX LSTM (forward, default activations, gate order i,o,f,c).
// Step 1: one GEMM projects all T steps of the input: P[T*Bt, 4H] = X * W^T.
// Step 2: per time step, G = h_{t-1} * R^T + P_t (GEMM with P_t as the C operand), then a fused
// gate kernel applies bias, sigmoid/tanh, updates c and h and writes Y_t.
// Scratch (P, G, and the running h/c state) comes from the context arena.
#include <math.h>

#include "common.cuh"

int wdc_simt_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B, const float* C,
                  float* Y);

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
  WDC_REQUIRE(ctx, T >= 0 && Bt > 0 && I > 0 && H > 0, "wdc_lstm: bad shape");
  WDC_REQUIRE(ctx, X && W && R && Yh && Yc && (T == 0 || Y), "wdc_lstm: null buffer");
  DeviceGuard g(ctx->device);
  float *P = nullptr, *G = nullptr;
  int s = wdc_alloc(ctx, (T > 0 ? T : 1) * Bt * 4 * H * 4, (void**)&P);
  if (s != WDC_OK) return s;
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
  if (s == WDC_OK && T > 0) {
    wdc_gemm_desc d = {};
    d.batch = 1; d.m = T * Bt; d.n = 4 * H; d.k = I;
    d.sa0 = I; d.sa1 = 1; d.sb0 = 1; d.sb1 = I;  // B = W^T
    d.alpha = 1.f; d.beta = 0.f;
    s = wdc_gemm(ctx, &d, X, W, nullptr, P);
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
