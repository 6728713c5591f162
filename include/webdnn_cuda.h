/*
 * webdnn_cuda.h — C ABI of libwebdnn_cuda.so, the sm_100a device layer of WebDNN's "cuda" backend.
 *
 * The ABI mirrors the verbs WebDNN's wasm backend sends to its worker
 * (src/shader/wasm/pre.js:4-92: alloc / destroy / write / read / runKernel) with one typed entry
 * point per kernel family instead of name dispatch.  Every device pointer is a plain `void*`
 * into the context's arena; every size is int64_t; every call returns a wdc_status and never
 * throws.  All work of a context is enqueued on that context's single in-order stream; only
 * wdc_download() and wdc_sync() wait for the device.  Asynchronous device errors surface at the
 * next waiting call.
 *
 * Tensors are dense row-major unless a call takes explicit strides (in elements).
 * dtype codes: 0 = float32, 1 = int32, 2 = bool (uint8).
 */
#ifndef WEBDNN_CUDA_H_
#define WEBDNN_CUDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct wdc_context wdc_context;

enum wdc_status {
  WDC_OK = 0,
  WDC_ERR_INVALID = 1,      /* bad argument, shape or dtype */
  WDC_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed */
  WDC_ERR_OOM = 3,          /* arena byte budget or device memory exhausted */
  WDC_ERR_UNSUPPORTED = 4,  /* valid ONNX semantics this library does not implement */
  WDC_ERR_DEVICE_WAIT = 5   /* a bounded device-side wait expired (reported at sync) */
};

/* ---- context, arena, transfers ------------------------------------------------------------
 * Replaces WebDNNWasmContextImpl / WebDNNWebGPUContextImpl device ownership
 * (backend/wasm/wasmContextImpl.ts:39-163, backend/webgpu/webgpuContextImpl.ts:85-189) and the
 * wasm heap (src/shader/wasm/src/core/allocation.cpp:6-14). */
int wdc_device_count(int* count);
/* arena_limit_bytes <= 0 means "no budget below device memory". */
int wdc_create(int device, int64_t arena_limit_bytes, wdc_context** out);
int wdc_destroy(wdc_context* ctx);
/* Message of the last failing call on this context (ctx may be NULL for wdc_create failures). */
const char* wdc_last_error(wdc_context* ctx);
int wdc_alloc(wdc_context* ctx, int64_t bytes, void** dptr);
int wdc_free(wdc_context* ctx, void* dptr);
/* Pinned host staging memory (page-locked), for callers that want true async H2D. */
int wdc_host_alloc(wdc_context* ctx, int64_t bytes, void** hptr);
int wdc_host_free(wdc_context* ctx, void* hptr);
int wdc_upload(wdc_context* ctx, void* dst, const void* host, int64_t bytes);
int wdc_download(wdc_context* ctx, void* host, const void* src, int64_t bytes); /* waits */
/* Host-to-device transfer on the context's second stream, so that the next batch's input moves
 * while the current batch's kernels run (no counterpart in the reference, whose tensor upload,
 * webgpuContextImpl.ts moveTensor / queue.writeBuffer, is ordered with the compute queue).
 * `host` should be pinned (wdc_host_alloc) and must stay valid until the transfer has run.
 * The transfer starts after the work already queued on the compute stream.  *ticket identifies it;
 * wdc_wait_upload makes the compute stream (not the host) wait for that transfer: call it before
 * the first launch that reads dst. */
/* Replay of a whole run without per-launch host work (the reference has no counterpart: its runner
 * re-issues every operator on every run, runnerImpl.ts:315-596).  Between wdc_capture_begin and
 * wdc_capture_end every launch on the context's stream is recorded instead of executed, and every
 * wdc_alloc / wdc_free is served by a private arena that the resulting graph keeps, so the recorded
 * launches find their buffers at the same addresses on every wdc_graph_launch.  Rules for the calls made
 * while capturing: no host<->device transfer, no wdc_sync, per-launch profiling off; buffers that were
 * allocated while capturing (the run's outputs) must be freed before wdc_graph_destroy; run the same
 * sequence once normally first, so that one-time work (weight packing and splitting) is not recorded. */
typedef struct wdc_graph wdc_graph;
int wdc_capture_begin(wdc_context* ctx);
int wdc_capture_end(wdc_context* ctx, wdc_graph** graph);
int wdc_graph_launch(wdc_context* ctx, wdc_graph* graph);
int wdc_graph_destroy(wdc_context* ctx, wdc_graph* graph);
int wdc_upload_async(wdc_context* ctx, void* dst, const void* host, int64_t bytes, int64_t* ticket);
int wdc_wait_upload(wdc_context* ctx, int64_t ticket);
/* wdc_upload_async for a destination that no queued work has touched since wdc_alloc returned it (a tensor created
 * for this transfer, the usual case of moveTensor, runnerImpl.ts:420-447): only a previous tenant of the memory can
 * still be in use, so the transfer waits for the compute stream's position at the arena's most recent wdc_free
 * instead of for everything queued so far, and can overlap a run that was queued before the call. */
int wdc_upload_fresh_async(wdc_context* ctx, void* dst, const void* host, int64_t bytes, int64_t* ticket);
/* Device-to-host transfer on a third stream, for callers that queue the next run before they read the result of
 * this one (the reference's getData, webgpuTensorImpl.ts:31-53, maps a staging buffer and awaits it; its runner
 * has one run in flight).  The transfer starts after the work queued so far on the compute stream and does not
 * hold up work queued later; wdc_wait_download blocks the host until that transfer has arrived (and reports an
 * expired device wait like wdc_download).  `host` should be pinned; `src` must not be freed or overwritten before
 * wdc_wait_download has returned. */
int wdc_download_async(wdc_context* ctx, void* host, const void* src, int64_t bytes, int64_t* ticket);
int wdc_wait_download(wdc_context* ctx, int64_t ticket);
int wdc_copy(wdc_context* ctx, void* dst, const void* src, int64_t bytes);
int wdc_fill_u32(wdc_context* ctx, void* dst, uint32_t value, int64_t count);
int wdc_sync(wdc_context* ctx);
/* Per-context options, the device side of `backendOptions.cuda` (InitOption.backendOptions, index.ts:26-30):
 *   "precision" 0 = tf32x3: every fp32 multiply-add of a tensor-core contraction is three TF32 MMAs on split
 *                   operands (fp32-class accuracy, the default); 1 = tf32x1: one MMA on truncated operands
 *                   (three times the tensor-pipe rate, about 1e-3 relative error per layer);
 *   "split_k"   1 = small outputs with long reductions may be cut into K ranges (default), 0 = never;
 *   "pdl"       1 = contraction launches are programmatic dependent launches, so that a launch's set-up
 *                   overlaps the tail of the launch before it (default), 0 = plain stream order;
 *   "nvtx"      1 = wdc_range_push / wdc_range_pop emit NVTX ranges (default 0).
 * Unknown names and out-of-range values return WDC_ERR_INVALID.  A captured graph keeps the options that were
 * in force while it was captured. */
int wdc_set_option(wdc_context* ctx, const char* name, int64_t value);
/* Named ranges around a caller's work (one per graph node: "name(opType)"), the counterpart of the per-node
 * records the reference's runner logs (core/runnerImpl.ts:487-489, 534-541).  No-ops unless option "nvtx" is 1. */
int wdc_range_push(wdc_context* ctx, const char* name);
int wdc_range_pop(wdc_context* ctx);
/* cudaStream_t of the context, for callers that record their own events around launches. */
void* wdc_stream(wdc_context* ctx);
/* out[0..n): bytes_in_use, high_water_bytes, reserved_bytes, allocs, frees, launches,
 * h2d_bytes, d2h_bytes, tensor_core_launches (launches of the tcgen05 contraction kernel),
 * then, only when n > 9 (it costs a driver call): device_free_bytes, device_total_bytes as
 * cudaMemGetInfo reports them for the context's GPU (-1 if that query fails). */
int wdc_stats(wdc_context* ctx, int64_t* out, int n);
int wdc_reset_stats(wdc_context* ctx);
/* Per-family device timing.  While enabled, every contraction launch (wdc_gemm / wdc_conv2d) is
 * bracketed by CUDA events on the context's stream; wdc_profile_read waits for the stream and
 * returns, for family 0 (contractions), the summed kernel milliseconds, the number of launches
 * and the summed algorithmic FLOPs since the last read, then clears the record. */
int wdc_profile_enable(wdc_context* ctx, int on);
int wdc_profile_read(wdc_context* ctx, int family, double* ms, int64_t* launches, double* flops);
/* Copy between buffers of two contexts (possibly on different GPUs) ordered after src's stream
 * and before later work on dst's stream; used to gather replica outputs over NVLink. */
int wdc_peer_copy(wdc_context* dst_ctx, void* dst, wdc_context* src_ctx, const void* src,
                  int64_t bytes);

/* ---- pointwise ------------------------------------------------------------------------------
 * wdc_unary replaces kernel_{ceil,exp,floor,relu,sigmoid,sqrt,tanh} and kernel_leakyrelu
 * (src/shader/wasm/src/kernels/standard/unarys.cpp:9-17, dynamic_unarys.cpp:8-11) and covers the
 * cpu backend's list (operators/cpu/operators/standard/unary.ts:34-211, dynamicunary.ts:156-189,
 * clip.ts).  Op codes: see wdc_unary_op.  p0/p1 are the op's attributes (alpha, beta/gamma,
 * or clip min/max). */
enum wdc_unary_op {
  WDC_U_ABS = 0, WDC_U_ACOS, WDC_U_ACOSH, WDC_U_ASIN, WDC_U_ASINH, WDC_U_ATAN, WDC_U_ATANH,
  WDC_U_CEIL, WDC_U_COS, WDC_U_COSH, WDC_U_EXP, WDC_U_FLOOR, WDC_U_HARDSWISH, WDC_U_LOG,
  WDC_U_NEG, WDC_U_RECIPROCAL, WDC_U_RELU, WDC_U_ROUND, WDC_U_SIGMOID, WDC_U_SIGN, WDC_U_SIN,
  WDC_U_SOFTPLUS, WDC_U_SOFTSIGN, WDC_U_SQRT, WDC_U_TAN, WDC_U_TANH,
  WDC_U_ELU = 32, WDC_U_HARDSIGMOID, WDC_U_LEAKYRELU, WDC_U_SELU, WDC_U_THRESHOLDEDRELU,
  WDC_U_CLIP = 40, WDC_U_IDENTITY = 41
};
int wdc_unary(wdc_context* ctx, int op, int dtype, const void* src, void* dst, int64_t n,
              float p0, float p1);

/* wdc_binary replaces kernel_{add,sub,mul,div,pow}_d{0..6}
 * (src/shader/wasm/src/kernels/standard/binary7s.cpp:9-22) and binary_*_add*.wgsl; semantics of
 * operators/cpu/operators/standard/binary7.ts:16-255 including int32 (computed in double, stored
 * with ToInt32).  dims are the broadcast output dims (ndim <= 6); sa/sb are input strides with 0
 * on broadcast axes (operatorUtil.ts:211-245). */
enum wdc_binary_op { WDC_B_ADD = 0, WDC_B_SUB, WDC_B_MUL, WDC_B_DIV, WDC_B_POW, WDC_B_MAX, WDC_B_MIN };
int wdc_binary(wdc_context* ctx, int op, int dtype, const void* a, const void* b, void* out,
               int ndim, const int64_t* dims, const int64_t* sa, const int64_t* sb);

/* Cast between float32 and int32 with the typed-array store semantics of
 * operators/cpu/operators/standard/cast.ts:43-45 (truncate, wrap mod 2^32, NaN -> 0). */
int wdc_cast(wdc_context* ctx, int src_dtype, int dst_dtype, const void* src, void* dst, int64_t n);

/* y = x * scale[c] + shift[c]; channel index c = (i / inner) % channels.  Used for
 * BatchNormalization in inference form (not in the reference; ONNX operator spec). */
int wdc_channel_affine(wdc_context* ctx, const float* x, const float* scale, const float* shift,
                       float* y, int64_t outer, int64_t channels, int64_t inner, int relu);

/* ---- contractions ---------------------------------------------------------------------------
 * wdc_gemm replaces kernel_gemm_transa{0,1}_transb{0,1}[_c]
 * (src/shader/wasm/src/kernels/standard/gemm.cpp:9-103) and gemm.wgsl:22-43; semantics of
 * operators/cpu/operators/standard/gemm.ts:21-61: Y[m,n] = alpha * sum_k A[i*sa0+k*sa1] *
 * B[k*sb0+j*sb1] (+ beta * C[i*sc0+j*sc1] when C != NULL), optional fused Relu.
 * batch > 1 with batch strides serves MatMul (operators/cpu/operators/standard/matmul.ts:63-111). */
typedef struct wdc_gemm_desc {
  int64_t batch, m, n, k;
  int64_t sab, sa0, sa1; /* A strides: batch, row(m), col(k) */
  int64_t sbb, sb0, sb1; /* B strides: batch, row(k), col(n) */
  int64_t sc0, sc1;      /* C strides (0 = broadcast); ignored when C == NULL */
  float alpha, beta;
  int relu;
} wdc_gemm_desc;
int wdc_gemm(wdc_context* ctx, const wdc_gemm_desc* d, const float* A, const float* B,
             const float* C, float* Y);

/* wdc_conv2d replaces the conv_im2col / conv_matmul / conv_transpose / conv_bias pipeline
 * (src/shader/webgpu/shadersources/standard/conv_*.wgsl, operators/webgpu/operators/standard/
 * conv.ts:13-120) with one implicit-GEMM launch; semantics of operators/cpu/operators/standard/
 * conv.ts:134-333 and base/conv.ts:31-79.
 * Layouts: x is NHWC [batch, in_h, in_w, ch_in]; w is [ch_out, k_h, k_w, ch_in/group] (use
 * wdc_pack_conv_weight to produce it from ONNX [ch_out, ch_in/group, k_h, k_w]); y is NHWC.
 * Epilogue per output channel c: v = acc * scale[c] + shift[c] (scale NULL = 1, shift NULL = 0;
 * bias and folded BatchNormalization go here), then v += residual (NHWC, same shape as y, or
 * NULL), then Relu when relu != 0. */
typedef struct wdc_conv_desc {
  int64_t batch, ch_in, in_h, in_w;
  int64_t ch_out, k_h, k_w, out_h, out_w;
  int64_t stride_h, stride_w, pad_t, pad_l, dil_h, dil_w, group;
  int relu;
  int x_nchw; /* 1: x is NCHW [batch, ch_in, in_h, in_w] instead of NHWC.  Accepted only where the input is
               * re-laid out anyway (ch_in <= 4, the network's first layer: the padding pass reads the planes
               * directly and the separate NCHW -> NHWC conversion is saved); WDC_ERR_UNSUPPORTED elsewhere. */
} wdc_conv_desc;
int wdc_conv2d(wdc_context* ctx, const wdc_conv_desc* d, const float* x, const float* w,
               const float* scale, const float* shift, const float* residual, float* y);
/* ONNX weight [ch_out, cig, k_h, k_w] -> [ch_out, k_h, k_w, cig]. */
int wdc_pack_conv_weight(wdc_context* ctx, const float* w_onnx, float* w_packed, int64_t ch_out,
                         int64_t cig, int64_t k_h, int64_t k_w);

/* ---- pooling --------------------------------------------------------------------------------
 * Semantics of operators/cpu/operators/standard/maxpool.ts:56-112 and
 * operators/cpu/rawcomputation/averagepool.ts:1-46.  x/y strides are given in elements for the
 * (n, c, h, w) axes so that NCHW and NHWC tensors use the same entry point. */
typedef struct wdc_pool_desc {
  int64_t batch, ch, in_h, in_w, out_h, out_w;
  int64_t k_h, k_w, stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int64_t xs_n, xs_c, xs_h, xs_w; /* input strides */
  int64_t ys_n, ys_c, ys_h, ys_w; /* output strides */
  int count_include_pad;          /* average pool only */
} wdc_pool_desc;
int wdc_maxpool2d(wdc_context* ctx, const wdc_pool_desc* d, const float* x, float* y);
int wdc_avgpool2d(wdc_context* ctx, const wdc_pool_desc* d, const float* x, float* y);
/* GlobalAveragePool (operators/cpu/operators/standard/globalaveragepool.ts:12-41):
 * y[b, c] = mean over area; x strides for (n, c, pixel). */
int wdc_global_avgpool(wdc_context* ctx, const float* x, float* y, int64_t batch, int64_t ch,
                       int64_t area, int64_t xs_n, int64_t xs_c, int64_t xs_p);

/* ---- row ops --------------------------------------------------------------------------------
 * Softmax over the last axis (operators/cpu/operators/standard/softmax.ts:15-59). */
int wdc_softmax(wdc_context* ctx, const float* x, float* y, int64_t outer, int64_t len);
/* One reduction pass over the middle axis of [outer, red, inner]
 * (operators/cpu/operators/standard/reduce.ts:41-103; one call per reduced axis).
 * kind: 0 sum, 1 mean, 2 max, 3 min, 4 prod, 5 l1, 6 l2, 7 logsum, 8 logsumexp, 9 sumsquare.
 * final != 0 applies the finishing function (mean divides by `total`). */
int wdc_reduce_axis(wdc_context* ctx, int kind, int final, const float* x, float* y,
                    int64_t outer, int64_t red, int64_t inner, int64_t total);
/* LayerNormalization over the last axis (not in the reference; equals its decomposed
 * ReduceMean/Sub/Mul/ReduceMean/Add/Sqrt/Div/Mul/Add chain).  gamma/beta may be NULL. */
int wdc_layernorm(wdc_context* ctx, const float* x, const float* gamma, const float* beta,
                  float* y, int64_t outer, int64_t len, float eps);
/* ArgMax over the last axis of [outer, len] -> int32 (not in the reference; ONNX spec). */
int wdc_argmax(wdc_context* ctx, const float* x, int32_t* y, int64_t outer, int64_t len,
               int select_last);

/* ---- data movement --------------------------------------------------------------------------
 * dst (dense row-major over dims, starting at element dst_off with strides dstr) <- src at
 * element src_off with strides sstr (source strides may be negative: Slice with a negative step);
 * 4-byte elements, ndim <= 6.  Serves Transpose
 * (operators/cpu/operators/standard/transpose.ts:12-169), Slice (slice.ts:12-90), Concat
 * (concat.ts:21-77), Split, Tile and NCHW<->NHWC conversion; replaces kernel_copy
 * (src/shader/wasm/src/kernels/standard/copy.cpp:6-8) where a layout really changes. */
int wdc_strided_copy(wdc_context* ctx, const void* src, void* dst, int ndim, const int64_t* dims,
                     const int64_t* sstr, int64_t src_off, const int64_t* dstr, int64_t dst_off);
/* Gather along axis: data [outer, axis_len, inner], idx int32 [n_idx] (negative wraps). */
int wdc_gather(wdc_context* ctx, const void* data, const int32_t* idx, void* out, int64_t outer,
               int64_t axis_len, int64_t inner, int64_t n_idx);

/* ConvTranspose, 2-D, NCHW (operators/cpu/operators/standard/convtranspose.ts:30-263, shape rule
 * base/convtranspose.ts:34-104): x [batch, ch_in, in_h, in_w], w [ch_in, ch_out_per_group, k_h, k_w],
 * bias [group * ch_out_per_group] or NULL, y [batch, group * ch_out_per_group, out_h, out_w].  Rounding
 * points as in the reference: channel contraction per tap -> float32, taps summed in
 * double -> float32, bias added in float32.  Large enough group-1 shapes run as the reference's own two steps on
 * the device: one tensor-core GEMM over the input pixels (3xTF32) into arena scratch, then col2im. */
typedef struct wdc_convt_desc {
  int64_t batch, ch_in, in_h, in_w;
  int64_t ch_out_per_group, group, k_h, k_w, out_h, out_w;
  int64_t stride_h, stride_w, pad_t, pad_l, dil_h, dil_w;
  int64_t w_layout; /* 0: w as in ONNX, [ch_in, ch_out_per_group, k_h, k_w].  1: w re-laid out once by the caller as
                     * [ch_in, k_h, k_w, ch_out_per_group] (a wdc_strided_copy), which the tensor-core route (group 1,
                     * ch_in a multiple of 4 and at least 32, ch_out_per_group * k_h * k_w a multiple of 4, at least 128
                     * input pixels) multiplies by directly; WDC_ERR_INVALID where that route does not apply. */
} wdc_convt_desc;
int wdc_conv_transpose2d(wdc_context* ctx, const wdc_convt_desc* d, const float* x, const float* w,
                         const float* bias, float* y);
/* InstanceNormalization over NCHW rows (operators/cpu/operators/standard/instancenormalization.ts:24-53):
 * per (batch, channel): y = x * (scale[c] * invstd) + (bias[c] - mean * scale[c] * invstd), statistics and
 * arithmetic in double.  eps is passed as the reference evaluates it (see CudaInstanceNormalization). */
int wdc_instance_norm(wdc_context* ctx, const float* x, const float* scale, const float* bias, float* y,
                      int64_t batch, int64_t ch, int64_t area, double eps);

/* Fused scaled-dot-product attention: y = softmax(scale * q k^T) v for every (batch, head), the [tq, tk]
 * score matrix kept on chip (one pass over the keys with a running row maximum and sum).  Not an operator of
 * the reference: it replaces the chain MatMul -> Mul -> Softmax -> MatMul that its graphs contain
 * (operators/cpu/operators/standard/matmul.ts:11-111, binary7.ts:16-68, softmax.ts:15-59) and is checked
 * against that chain.  Both contractions run on the tensor cores (tcgen05, 3xTF32: scores and the running
 * output live in tensor memory, K and V^T tiles arrive by TMA from a split copy made by a pre-pass in arena
 * scratch); a CUDA-core kernel takes over when the tensor-map entry point or the scratch is unavailable.
 * Element (b, h, t, c) of q sits at q[b * q_sb + h * q_sh + t * q_st + c] (likewise k, v
 * with tk rows and y with tq rows): head-split views of [batch, tokens, heads * dh] tensors need no transpose.
 * dh is 32 or 64 (else WDC_ERR_UNSUPPORTED); strides are multiples of 4 floats, buffers 16-byte aligned. */
typedef struct wdc_attention_desc {
  int64_t batch, heads, tq, tk, dh;
  int64_t q_sb, q_sh, q_st;
  int64_t k_sb, k_sh, k_st;
  int64_t v_sb, v_sh, v_st;
  int64_t y_sb, y_sh, y_st;
  float scale;
} wdc_attention_desc;
int wdc_attention(wdc_context* ctx, const wdc_attention_desc* d, const float* q, const float* k, const float* v,
                  float* y);

/* 8-bit weight codec of the WDN2 tensor container (core/tensorDecoder/decodeTensorEightbit.ts:36-61): `codes`
 * holds one byte per element (the inflated zlib stream, uploaded as bytes); out[i] = level[codes[i] & 127] * scale,
 * negated when bit 7 is set, bit-identical to the reference's table lookup.  Both buffers 16-byte aligned. */
int wdc_decode_eightbit(wdc_context* ctx, const void* codes, float* out, int64_t n, float scale);

/* ---- LSTM -----------------------------------------------------------------------------------
 * ONNX LSTM, forward direction, default activations, no peepholes (not in the reference; ONNX
 * operator spec).  X [T, Bt, I], W [4H, I], R [4H, H], bias [8H] or NULL, h0/c0 [Bt, H] or NULL;
 * Y [T, 1, Bt, H], Yh/Yc [Bt, H].  Gate order i, o, f, c.  One tensor-core GEMM projects the
 * inputs of all steps; the recurrence runs as one persistent cooperative kernel with R resident in
 * shared memory across the SMs when Bt <= 64 and H % 32 == 0 (and the slices fit), else as one
 * GEMM + one gate kernel per step. */
int wdc_lstm(wdc_context* ctx, const float* X, const float* W, const float* R, const float* bias,
             const float* h0, const float* c0, float* Y, float* Yh, float* Yc, int64_t T,
             int64_t Bt, int64_t I, int64_t H);

/* Self-test of the error path of bounded device waits (the reference's counterpart is the exception path of
 * core/runnerImpl.ts:511-520: a failing operator is reported, the runner object stays usable).  Enqueues the
 * persistent LSTM kernel on a small internal problem whose first step can never complete, with limit_ns
 * (1 us .. 1 s) as the limit of its waits: the kernel gives up after that time, records its status and returns.
 * The call itself returns WDC_OK; the next wdc_sync / wdc_download returns WDC_ERR_DEVICE_WAIT once, and the
 * context keeps working afterwards. */
int wdc_selftest_device_wait(wdc_context* ctx, int64_t limit_ns);

/* wdc_lstm for callers that cannot allocate device memory while they run (a host that owns all GPU memory in
 * its own pool, a real-time loop, a sandbox without cudaMalloc): same arguments and results as wdc_lstm, but the
 * scratch is a fixed 4 MiB array inside the library image (held on every GPU that loads the library, until exit)
 * and no cudaMalloc / cudaFree / allocating routine is called.  Limit: batch * 4 * hidden_size <= 1 048 576,
 * otherwise WDC_ERR_UNSUPPORTED.  The array's address is looked up, and the modules of the kernels this entry
 * point launches are loaded, by wdc_create for its device: that is the moment the driver sets the 4 MiB aside, so
 * create the context at start-up.  (If a device's address is still unknown when the call runs, the call looks it
 * up itself; such a first call must come before any stream capture.)  Calls on one device share the array: calls
 * that overlap on the GPU race.  This entry point has no counterpart in the reference. */
int wdc_lstm_static(wdc_context* ctx, const float* X, const float* W, const float* R, const float* bias,
                    const float* h0, const float* c0, float* Y, float* Yh, float* Yc, int64_t T,
                    int64_t Bt, int64_t I, int64_t H);

#ifdef __cplusplus
}
#endif
#endif /* WEBDNN_CUDA_H_ */
