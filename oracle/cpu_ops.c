/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the arithmetic of WebDNN's "cpu" backend
 * (src/descriptor_runner/operators/cpu/) for the operator-execution path.  Nothing in the
 * shipped CUDA backend links, imports or calls this file; only tests, the smoke check and the
 * benchmark's CPU-baseline leg do, and only as the checker / the timed CPU baseline.
 *
 * Numerics follow the JavaScript the reference runs: tensors are Float32Array / Int32Array,
 * every accumulator is an IEEE double ("number"), and a value is rounded to float exactly where
 * the JS stores into a Float32Array.  Loop orders match the cited loops so that the double sums
 * are formed in the same sequence.
 *
 * Pinning status: the reference ships no golden tensors for these ops beyond the tiny known
 * answers restated in tests/golden/reference_known_answers.json (Relu vector, tensor strides);
 * the reference itself cannot run in the build environment (needs Node.js).  Parity of Relu and
 * of tensor indexing is pinned by those answers; everything else is checked against float64
 * PyTorch/numpy results, which is what the reference's own test generators use as expectations
 * (test/model_test/make_models.py, test/fixtures/generate_fixtures.py).  BatchNormalization,
 * LSTM, ArgMax and fused LayerNormalization do not exist in the reference at all: they are
 * restated from the ONNX operator specification and are "parity unpinned".
 *
 * OpenMP (when compiled with -fopenmp) only distributes independent output elements over
 * threads; the sequence of operations forming each output value is unchanged, so results are
 * identical for any thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* JS ToInt32: what a store of a double into an Int32Array does. */
static int32_t to_int32(double d) {
  if (!isfinite(d)) return 0;
  double t = trunc(d);
  double m = fmod(t, 4294967296.0);
  if (m < 0) m += 4294967296.0;
  if (m >= 2147483648.0) m -= 4294967296.0;
  return (int32_t)m;
}

/* JS Math.round: nearest integer, ties toward +Infinity. */
static double js_round(double x) {
  if (!isfinite(x) || fabs(x) >= 4503599627370496.0) return x;
  double r = floor(x + 0.5);
  if (r == 0.0 && (x < 0.0 || (x == 0.0 && signbit(x)))) return -0.0;
  return r;
}

static double js_sign(double x) {
  if (x != x) return x;
  if (x > 0) return 1.0;
  if (x < 0) return -1.0;
  return x; /* keeps -0 */
}

/* JS Math.max(v, 0): NaN propagates, max(-0, 0) = +0. */
static double js_max0(double v) {
  if (v != v) return v;
  return v > 0 ? v : 0.0;
}

/* JS `**` / Math.pow deviations from C pow(). */
static double js_pow(double a, double b) {
  if (b != b) return NAN;
  if ((a == 1.0 || a == -1.0) && isinf(b)) return NAN;
  return pow(a, b);
}

/* ---------------------------------------------------------------- unary ----
 * operators/cpu/operators/standard/unary.ts:10-32 (loop) and :34-211 (functions);
 * dynamicunary.ts:41-154 for the parameterised ones. Codes are shared with the CUDA library. */
enum {
  U_ABS = 0, U_ACOS, U_ACOSH, U_ASIN, U_ASINH, U_ATAN, U_ATANH, U_CEIL, U_COS, U_COSH, U_EXP,
  U_FLOOR, U_HARDSWISH, U_LOG, U_NEG, U_RECIPROCAL, U_RELU, U_ROUND, U_SIGMOID, U_SIGN, U_SIN,
  U_SOFTPLUS, U_SOFTSIGN, U_SQRT, U_TAN, U_TANH,
  U_ELU = 32, U_HARDSIGMOID, U_LEAKYRELU, U_SELU, U_THRESHOLDEDRELU,
  U_CLIP = 40, U_IDENTITY = 41
};

static double unary_eval(int op, double v, double p0, double p1) {
  switch (op) {
    case U_ABS: return fabs(v);
    case U_ACOS: return acos(v);
    case U_ACOSH: return acosh(v);
    case U_ASIN: return asin(v);
    case U_ASINH: return asinh(v);
    case U_ATAN: return atan(v);
    case U_ATANH: return atanh(v);
    case U_CEIL: return ceil(v);
    case U_COS: return cos(v);
    case U_COSH: return cosh(v);
    case U_EXP: return exp(v);
    case U_FLOOR: return floor(v);
    case U_HARDSWISH: /* unary.ts:110-126 */
      if (v <= -3) return 0;
      if (v >= 3) return v;
      return (v * (v + 3)) / 6;
    case U_LOG: return log(v);
    case U_NEG: return -v;
    case U_RECIPROCAL: return 1 / v;
    case U_RELU: return js_max0(v);
    case U_ROUND: return js_round(v);
    case U_SIGMOID: return (tanh(v / 2) + 1) / 2; /* unary.ts:163 */
    case U_SIGN: return js_sign(v);
    case U_SIN: return sin(v);
    case U_SOFTPLUS: return log(exp(v) + 1);
    case U_SOFTSIGN: return v / (1 + fabs(v));
    case U_SQRT: return sqrt(v);
    case U_TAN: return tan(v);
    case U_TANH: return tanh(v);
    case U_ELU: return v >= 0 ? v : (exp(v) - 1) * p0;
    case U_HARDSIGMOID: {
      /* Math.max(0, Math.min(1, v*alpha+beta)); NaN propagates through both */
      double t = v * p0 + p1;
      if (t != t) return t;
      double m = t < 1 ? t : 1;
      return m > 0 ? m : 0;
    }
    case U_LEAKYRELU: return v >= 0 ? v : v * p0;
    case U_SELU: return v > 0 ? p1 * v : p1 * (p0 * exp(v) - p0); /* p0=alpha p1=gamma */
    case U_THRESHOLDEDRELU: return v > p0 ? v : 0;
    case U_CLIP: { /* clip.ts (opset < 11): Math.min(max, Math.max(v, min)) */
      if (v != v) return v;
      double t = v > p0 ? v : p0;
      return t < p1 ? t : p1;
    }
    case U_IDENTITY: return v;
  }
  return NAN;
}

/* dtype: 0 = float32, 1 = int32 */
int orc_unary(int op, int dtype, const void* src, void* dst, int64_t n, double p0, double p1) {
  if (dtype == 0) {
    const float* s = (const float*)src;
    float* d = (float*)dst;
#pragma omp parallel for if (n > 65536)
    for (int64_t i = 0; i < n; i++) d[i] = (float)unary_eval(op, (double)s[i], p0, p1);
  } else if (dtype == 1) {
    if (!(op == U_ABS || op == U_NEG || op == U_RELU || op == U_SIGN || op == U_IDENTITY)) return 1;
    const int32_t* s = (const int32_t*)src;
    int32_t* d = (int32_t*)dst;
    for (int64_t i = 0; i < n; i++) d[i] = to_int32(unary_eval(op, (double)s[i], p0, p1));
  } else {
    return 1;
  }
  return 0;
}

/* --------------------------------------------------------------- binary ----
 * operators/cpu/operators/standard/binary7.ts:16-68 (dispatch), :70-255 (rank loops);
 * eachelementwise.ts for Max/Min (op codes 5, 6 here take exactly two operands). */
enum { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MAX, B_MIN };

static double binary_eval(int op, double l, double r) {
  switch (op) {
    case B_ADD: return l + r;
    case B_SUB: return l - r;
    case B_MUL: return l * r;
    case B_DIV: return l / r;
    case B_POW: return js_pow(l, r);
    case B_MAX: if (l != l || r != r) return NAN; return l > r ? l : r;
    case B_MIN: if (l != l || r != r) return NAN; return l < r ? l : r;
  }
  return NAN;
}

int orc_binary(int op, int dtype, const void* a, const void* b, void* out, int ndim,
               const int64_t* dims, const int64_t* sa, const int64_t* sb) {
  if (ndim > 6 || ndim < 0) return 1;
  int64_t d[6] = {1, 1, 1, 1, 1, 1}, xa[6] = {0}, xb[6] = {0};
  for (int i = 0; i < ndim; i++) {
    d[6 - ndim + i] = dims[i];
    xa[6 - ndim + i] = sa[i];
    xb[6 - ndim + i] = sb[i];
  }
  int64_t idx = 0;
  for (int64_t i0 = 0; i0 < d[0]; i0++)
  for (int64_t i1 = 0; i1 < d[1]; i1++)
  for (int64_t i2 = 0; i2 < d[2]; i2++)
  for (int64_t i3 = 0; i3 < d[3]; i3++)
  for (int64_t i4 = 0; i4 < d[4]; i4++)
  for (int64_t i5 = 0; i5 < d[5]; i5++) {
    int64_t ia = i0 * xa[0] + i1 * xa[1] + i2 * xa[2] + i3 * xa[3] + i4 * xa[4] + i5 * xa[5];
    int64_t ib = i0 * xb[0] + i1 * xb[1] + i2 * xb[2] + i3 * xb[3] + i4 * xb[4] + i5 * xb[5];
    if (dtype == 0) {
      ((float*)out)[idx] = (float)binary_eval(op, ((const float*)a)[ia], ((const float*)b)[ib]);
    } else {
      ((int32_t*)out)[idx] =
          to_int32(binary_eval(op, ((const int32_t*)a)[ia], ((const int32_t*)b)[ib]));
    }
    idx++;
  }
  return 0;
}

/* ----------------------------------------------------------------- gemm ----
 * operators/cpu/operators/standard/gemm.ts:37-47 (product, alpha) and :49-58 (C, beta). */
int orc_gemm(const float* A, const float* B, const float* C, float* Y, int64_t m, int64_t n,
             int64_t k, int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, int has_c,
             int64_t sc0, int64_t sc1, double alpha, double beta) {
#pragma omp parallel for
  for (int64_t i = 0; i < m; i++) {
    for (int64_t j = 0; j < n; j++) {
      double sum = 0;
      for (int64_t x = 0; x < k; x++)
        sum += (double)A[i * sa0 + x * sa1] * (double)B[x * sb0 + j * sb1];
      sum *= alpha;
      float y = (float)sum;
      if (has_c) y = (float)((double)y + (double)C[i * sc0 + j * sc1] * beta);
      Y[i * n + j] = y;
    }
  }
  return 0;
}

/* --------------------------------------------------------------- matmul ----
 * operators/cpu/operators/standard/matmul.ts:63-111 with the strides of base/matmul.ts:56-70;
 * a 2-D result is the batch == 1 case. */
int orc_matmul(const float* A, const float* B, float* Y, int64_t batch, int64_t m, int64_t n,
               int64_t k, int64_t sab, int64_t sam, int64_t sak, int64_t sbb, int64_t sbk,
               int64_t sbn) {
#pragma omp parallel for collapse(2)
  for (int64_t o = 0; o < batch; o++) {
    for (int64_t i = 0; i < m; i++) {
      for (int64_t j = 0; j < n; j++) {
        double sum = 0;
        for (int64_t x = 0; x < k; x++)
          sum += (double)A[o * sab + i * sam + x * sak] * (double)B[o * sbb + x * sbk + j * sbn];
        Y[(o * m + i) * n + j] = (float)sum;
      }
    }
  }
  return 0;
}

/* ----------------------------------------------------------------- conv ----
 * operators/cpu/operators/standard/conv.ts: im2col :223-270 (zero fill outside the image, K order
 * ci,ky,kx), matmul :272-295 (double sum stored to float), transpose :297-316 (to NCHW),
 * bias :318-333 (float += bias).  Output shape per base/conv.ts:31-79 is computed by the caller. */
int orc_conv2d(const float* X, const float* W, const float* Bias, float* Y, int64_t batch,
               int64_t chIn, int64_t inH, int64_t inW, int64_t chOut, int64_t kH, int64_t kW,
               int64_t outH, int64_t outW, int64_t strideH, int64_t strideW, int64_t padT,
               int64_t padL, int64_t dilH, int64_t dilW, int64_t group) {
  const int64_t cig = chIn / group, cog = chOut / group, K = cig * kH * kW;
#pragma omp parallel
  {
    float* patch = (float*)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
#pragma omp for collapse(3)
    for (int64_t g = 0; g < group; g++) {
      for (int64_t b = 0; b < batch; b++) {
        for (int64_t oy = 0; oy < outH; oy++) {
          for (int64_t ox = 0; ox < outW; ox++) {
            int64_t p = 0;
            for (int64_t ci = 0; ci < cig; ci++)
              for (int64_t ky = 0; ky < kH; ky++)
                for (int64_t kx = 0; kx < kW; kx++) {
                  int64_t iny = oy * strideH - padT + ky * dilH;
                  int64_t inx = ox * strideW - padL + kx * dilW;
                  float v = 0;
                  if (iny >= 0 && iny < inH && inx >= 0 && inx < inW)
                    v = X[((b * chIn + g * cig + ci) * inH + iny) * inW + inx];
                  patch[p++] = v;
                }
            int64_t co = 0;
            /* four independent accumulators; each one is still a strictly sequential sum */
            for (; co + 4 <= cog; co += 4) {
              const float* w0 = W + (g * cog + co) * K;
              const float *w1 = w0 + K, *w2 = w1 + K, *w3 = w2 + K;
              double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
              for (int64_t ip = 0; ip < K; ip++) {
                double a = patch[ip];
                s0 += a * (double)w0[ip];
                s1 += a * (double)w1[ip];
                s2 += a * (double)w2[ip];
                s3 += a * (double)w3[ip];
              }
              double ss[4] = {s0, s1, s2, s3};
              for (int q = 0; q < 4; q++) {
                int64_t c = g * cog + co + q;
                float y = (float)ss[q];
                if (Bias) y = (float)((double)y + (double)Bias[c]);
                Y[((b * chOut + c) * outH + oy) * outW + ox] = y;
              }
            }
            for (; co < cog; co++) {
              const float* w0 = W + (g * cog + co) * K;
              double s = 0;
              for (int64_t ip = 0; ip < K; ip++) s += (double)patch[ip] * (double)w0[ip];
              int64_t c = g * cog + co;
              float y = (float)s;
              if (Bias) y = (float)((double)y + (double)Bias[c]);
              Y[((b * chOut + c) * outH + oy) * outW + ox] = y;
            }
          }
        }
      }
    }
    free(patch);
  }
  return 0;
}

/* ------------------------------------------------------------- max pool ----
 * operators/cpu/operators/standard/maxpool.ts:56-112: -Infinity start, strict `>` (NaN never
 * wins), padding excluded. */
int orc_maxpool(const float* X, float* Y, int64_t batch, int64_t ch, int64_t inH, int64_t inW,
                int64_t kH, int64_t kW, int64_t outH, int64_t outW, int64_t strideH,
                int64_t strideW, int64_t padT, int64_t padL, int64_t dilH, int64_t dilW) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < batch; b++)
    for (int64_t c = 0; c < ch; c++)
      for (int64_t oy = 0; oy < outH; oy++)
        for (int64_t ox = 0; ox < outW; ox++) {
          float mv = -INFINITY;
          for (int64_t ky = 0; ky < kH; ky++)
            for (int64_t kx = 0; kx < kW; kx++) {
              int64_t iny = oy * strideH - padT + ky * dilH, inx = ox * strideW - padL + kx * dilW;
              if (iny >= 0 && iny < inH && inx >= 0 && inx < inW) {
                float v = X[((b * ch + c) * inH + iny) * inW + inx];
                if (v > mv) mv = v;
              }
            }
          Y[((b * ch + c) * outH + oy) * outW + ox] = mv;
        }
  return 0;
}

/* --------------------------------------------------------- average pool ----
 * operators/cpu/rawcomputation/averagepool.ts:13-46.  GlobalAveragePool calls it with the
 * kernel equal to the image, no pads, count_include_pad = true
 * (operators/cpu/operators/standard/globalaveragepool.ts:23-34). */
int orc_avgpool(const float* X, float* Y, int count_include_pad, int64_t batch, int64_t ch,
                int64_t inH, int64_t inW, int64_t kH, int64_t kW, int64_t outH, int64_t outW,
                int64_t strideH, int64_t strideW, int64_t padT, int64_t padL) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < batch; b++)
    for (int64_t c = 0; c < ch; c++)
      for (int64_t oy = 0; oy < outH; oy++)
        for (int64_t ox = 0; ox < outW; ox++) {
          double sum = 0;
          int64_t ctr = 0;
          for (int64_t ky = 0; ky < kH; ky++)
            for (int64_t kx = 0; kx < kW; kx++) {
              int64_t iny = oy * strideH - padT + ky, inx = ox * strideW - padL + kx;
              if (iny >= 0 && iny < inH && inx >= 0 && inx < inW) {
                sum += (double)X[((b * ch + c) * inH + iny) * inW + inx];
                ctr++;
              }
            }
          Y[((b * ch + c) * outH + oy) * outW + ox] =
              (float)(count_include_pad ? sum / (double)(kH * kW) : sum / (double)ctr);
        }
  return 0;
}

/* -------------------------------------------------------------- softmax ----
 * operators/cpu/operators/standard/softmax.ts:39-57: exp stored as float, the sum keeps the
 * unrounded doubles, the division reads back the stored float. */
int orc_softmax(const float* X, float* Y, int64_t outer, int64_t len) {
#pragma omp parallel for if (outer * len > 65536)
  for (int64_t o = 0; o < outer; o++) {
    double mx = -INFINITY;
    for (int64_t r = 0; r < len; r++) {
      double v = X[o * len + r];
      if (v > mx) mx = v;
    }
    double expsum = 0;
    for (int64_t r = 0; r < len; r++) {
      double e = exp((double)X[o * len + r] - mx);
      Y[o * len + r] = (float)e;
      expsum += e;
    }
    for (int64_t r = 0; r < len; r++) Y[o * len + r] = (float)((double)Y[o * len + r] / expsum);
  }
  return 0;
}

/* --------------------------------------------------------------- reduce ----
 * operators/cpu/operators/standard/reduce.ts:41-103: one pass per (sorted) axis, every pass
 * stores floats; the last pass applies the finishing function (:206-493).  `kind` selects the
 * op; `final` is 1 on the last axis; total = product of all reduced lengths so far.  The
 * reference applies abs / square / exp on EVERY pass of a multi-axis reduction and its
 * ReduceLogSum indexes the input without the inner offset (:288-312); both are restated as
 * they are, since the contract is "same result as the reference". */
enum { R_SUM = 0, R_MEAN, R_MAX, R_MIN, R_PROD, R_L1, R_L2, R_LOGSUM, R_LOGSUMEXP, R_SUMSQUARE };

int orc_reduce_axis(int kind, int final, const float* X, float* Y, int64_t outer,
                    int64_t red, int64_t inner, int64_t total) {
#pragma omp parallel for collapse(2) if (outer * inner * red > 65536)
  for (int64_t o = 0; o < outer; o++)
    for (int64_t in = 0; in < inner; in++) {
      double s;
      const float* p = X + o * red * inner + in;
      switch (kind) {
        case R_MAX:
          s = red > 0 ? p[0] : NAN;   /* empty axis: element 0 is undefined in the reference -> NaN */
          for (int64_t r = 1; r < red; r++) { double v = p[r * inner]; if (v > s) s = v; }
          break;
        case R_MIN:
          s = red > 0 ? p[0] : NAN;
          for (int64_t r = 1; r < red; r++) { double v = p[r * inner]; if (v < s) s = v; }
          break;
        case R_PROD:
          s = 1;
          for (int64_t r = 0; r < red; r++) s *= (double)p[r * inner];
          break;
        case R_L1:
          s = 0;
          for (int64_t r = 0; r < red; r++) s += fabs((double)p[r * inner]);
          break;
        case R_L2:
        case R_SUMSQUARE:
          s = 0;
          for (int64_t r = 0; r < red; r++) {
            double v = p[r * inner];
            s += v * v;
          }
          if (kind == R_L2 && final) s = sqrt(s);
          break;
        case R_LOGSUMEXP:
          s = 0;
          for (int64_t r = 0; r < red; r++) s += exp((double)p[r * inner]);
          if (final) s = log(s);
          break;
        case R_LOGSUM:
          s = 0;
          for (int64_t r = 0; r < red; r++) s += (double)X[o * red + r];
          if (final) s = log(s);
          break;
        default: /* R_SUM, R_MEAN */
          s = 0;
          for (int64_t r = 0; r < red; r++) s += (double)p[r * inner];
          if (kind == R_MEAN && final) s = s / (double)total;
          break;
      }
      Y[o * inner + in] = (float)s;
    }
  return 0;
}

/* ------------------------------------------------------ strided copies ----
 * operators/cpu/operators/standard/transpose.ts:49-169 (copyNd: output row-major, input strided)
 * also serves Slice (slice.ts) and Concat/Split pieces; elements are 4 bytes wide. */
int orc_strided_copy(const void* src, void* dst, int ndim, const int64_t* dims,
                     const int64_t* sstr, int64_t soff) {
  if (ndim > 6 || ndim < 0) return 1;
  int64_t d[6] = {1, 1, 1, 1, 1, 1}, s[6] = {0};
  for (int i = 0; i < ndim; i++) {
    d[6 - ndim + i] = dims[i];
    s[6 - ndim + i] = sstr[i];
  }
  const uint32_t* in = (const uint32_t*)src + soff;
  uint32_t* out = (uint32_t*)dst;
  int64_t idx = 0;
  for (int64_t i0 = 0; i0 < d[0]; i0++)
  for (int64_t i1 = 0; i1 < d[1]; i1++)
  for (int64_t i2 = 0; i2 < d[2]; i2++)
  for (int64_t i3 = 0; i3 < d[3]; i3++)
  for (int64_t i4 = 0; i4 < d[4]; i4++)
  for (int64_t i5 = 0; i5 < d[5]; i5++)
    out[idx++] = in[i0 * s[0] + i1 * s[1] + i2 * s[2] + i3 * s[3] + i4 * s[4] + i5 * s[5]];
  return 0;
}

/* Cast float -> int32 as an Int32Array store does (cast.ts:43-45). */
int orc_cast_f32_i32(const float* src, int32_t* dst, int64_t n) {
  for (int64_t i = 0; i < n; i++) dst[i] = to_int32((double)src[i]);
  return 0;
}

/* ------------------------------------------------- ops not in reference ----
 * Restated from the ONNX operator specification; parity unpinned. */

/* BatchNormalization (inference form): y = (x - mean) / sqrt(var + eps) * scale + bias, NCHW. */
int orc_batchnorm(const float* X, const float* scale, const float* bias, const float* mean,
                  const float* var, float* Y, int64_t batch, int64_t ch, int64_t area,
                  double eps) {
#pragma omp parallel for collapse(2)
  for (int64_t b = 0; b < batch; b++)
    for (int64_t c = 0; c < ch; c++) {
      double inv = 1.0 / sqrt((double)var[c] + eps);
      for (int64_t i = 0; i < area; i++) {
        int64_t o = (b * ch + c) * area + i;
        Y[o] = (float)(((double)X[o] - (double)mean[c]) * inv * (double)scale[c] + (double)bias[c]);
      }
    }
  return 0;
}

static double sigm(double x) { return (tanh(x / 2) + 1) / 2; }

/* LSTM, forward direction, default activations, no peepholes, gate order i,o,f,c.
 * X [T,Bt,I], W [4H,I], R [4H,H], Bias [8H] or NULL, h0/c0 [Bt,H] or NULL.
 * Y [T,1,Bt,H], Yh/Yc [Bt,H].  State is held as float between steps. */
int orc_lstm(const float* X, const float* W, const float* R, const float* Bias, const float* h0,
             const float* c0, float* Y, float* Yh, float* Yc, int64_t T, int64_t Bt, int64_t I,
             int64_t H) {
  float* h = (float*)calloc((size_t)(Bt * H), sizeof(float));
  float* c = (float*)calloc((size_t)(Bt * H), sizeof(float));
  float* hn = (float*)calloc((size_t)(Bt * H), sizeof(float));
  if (h0) memcpy(h, h0, sizeof(float) * (size_t)(Bt * H));
  if (c0) memcpy(c, c0, sizeof(float) * (size_t)(Bt * H));
  for (int64_t t = 0; t < T; t++) {
#pragma omp parallel for collapse(2)
    for (int64_t b = 0; b < Bt; b++)
      for (int64_t j = 0; j < H; j++) {
        double g[4];
        for (int q = 0; q < 4; q++) {
          int64_t row = q * H + j;
          double s = 0;
          const float* x = X + (t * Bt + b) * I;
          const float* w = W + row * I;
          for (int64_t i = 0; i < I; i++) s += (double)x[i] * (double)w[i];
          const float* hp = h + b * H;
          const float* r = R + row * H;
          for (int64_t i = 0; i < H; i++) s += (double)hp[i] * (double)r[i];
          if (Bias) s += (double)Bias[row] + (double)Bias[4 * H + row];
          g[q] = s;
        }
        double it = sigm(g[0]), ot = sigm(g[1]), ft = sigm(g[2]), ct = tanh(g[3]);
        float cn = (float)(ft * (double)c[b * H + j] + it * ct);
        float hv = (float)(ot * tanh((double)cn));
        c[b * H + j] = cn;
        hn[b * H + j] = hv;
        Y[(t * Bt + b) * H + j] = hv;
      }
    memcpy(h, hn, sizeof(float) * (size_t)(Bt * H));
  }
  memcpy(Yh, h, sizeof(float) * (size_t)(Bt * H));
  memcpy(Yc, c, sizeof(float) * (size_t)(Bt * H));
  free(h); free(c); free(hn);
  return 0;
}

/* ArgMax over the last axis after the caller moved the axis last; first maximum wins
 * (select_last_index = 0), or last when select_last != 0. */
int orc_argmax(const float* X, int32_t* Y, int64_t outer, int64_t len, int select_last) {
  for (int64_t o = 0; o < outer; o++) {
    int64_t best = 0;
    float bv = X[o * len];
    for (int64_t r = 1; r < len; r++) {
      float v = X[o * len + r];
      if (v > bv || (select_last && v == bv)) { bv = v; best = r; }
    }
    Y[o] = (int32_t)best;
  }
  return 0;
}
