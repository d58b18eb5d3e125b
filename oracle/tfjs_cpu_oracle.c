/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the tfjs-backend-cpu kernels
 * that sit on the inference hot path.  Nothing in the shipped CUDA path may
 * link or call this file; it is the checker used by tests/, by
 * __graft_entry__.smoke() and by the cpu_baseline / reference legs of bench.py.
 *
 * Parity status: pinned.  tests/test_oracle_golden.py checks every function
 * here against known-answer vectors taken from the reference's own op tests
 * (tests/golden/ts_goldens.json, produced by tests/golden/make_ts_goldens.py)
 * and against fixtures produced by importing the reference's quantization.py.
 *
 * JavaScript numerics are reproduced exactly: every arithmetic operation is an
 * IEEE double operation, and every store into a Float32Array rounds to fp32.
 * Loops over independent output elements are OpenMP-parallel; the order of
 * accumulation for one output element is always the reference's order, so the
 * result does not depend on the thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- conv2D: tfjs-backend-cpu/src/kernels/Conv2D.ts:64-100 -----------------
 * NHWC x, HWIO filter.  The reference's loop nest is b,yR,wR,yC,wC,d1,d2 with
 * `yVals[..] += xVal * w` on a Float32Array, so for one output element the
 * MACs arrive in (wR,wC,d1) order and each one rounds the running value to
 * fp32: y = fl32(double(y) + double(x)*double(w)).  Taps that fall outside the
 * image are skipped (Conv2D.ts:72-74, :82-84). */
void orc_conv2d(const float* x, const float* w, float* y, int batch, int inH,
                int inW, int inC, int outH, int outW, int outC, int fH, int fW,
                int strideH, int strideW, int dilH, int dilW, int padTop,
                int padLeft) {
  const long total = (long)batch * outH * outW;
#pragma omp parallel for schedule(static)
  for (long p = 0; p < total; ++p) {
    const int yC = (int)(p % outW);
    const int yR = (int)((p / outW) % outH);
    const int b = (int)(p / ((long)outW * outH));
    float* yo = y + p * outC;
    for (int d2 = 0; d2 < outC; ++d2) yo[d2] = 0.0f;
    const int xRCorner = yR * strideH - padTop;
    const int xCCorner = yC * strideW - padLeft;
    for (int wR = 0; wR < fH; ++wR) {
      const int xR = xRCorner + wR * dilH;
      if (xR < 0 || xR >= inH) continue;
      for (int wC = 0; wC < fW; ++wC) {
        const int xC = xCCorner + wC * dilW;
        if (xC < 0 || xC >= inW) continue;
        const float* xp = x + (((long)b * inH + xR) * inW + xC) * inC;
        const float* wp = w + ((long)wR * fW + wC) * inC * outC;
        for (int d1 = 0; d1 < inC; ++d1) {
          const double xv = (double)xp[d1];
          const float* wrow = wp + (long)d1 * outC;
          for (int d2 = 0; d2 < outC; ++d2)
            yo[d2] = (float)((double)yo[d2] + xv * (double)wrow[d2]);
        }
      }
    }
  }
}

/* ---- depthwiseConv2dNative: DepthwiseConv2dNative.ts:62-99 ----------------
 * Filter [fH,fW,inC,chMul]; output channel = d1*chMul + q (:87-94).  Same
 * per-MAC fp32 rounding (:90), order (wR,wC) per output element. */
void orc_depthwise_conv2d(const float* x, const float* w, float* y, int batch,
                          int inH, int inW, int inC, int chMul, int outH,
                          int outW, int fH, int fW, int strideH, int strideW,
                          int dilH, int dilW, int padTop, int padLeft) {
  const long total = (long)batch * outH * outW;
  const int outC = inC * chMul;
#pragma omp parallel for schedule(static)
  for (long p = 0; p < total; ++p) {
    const int yC = (int)(p % outW);
    const int yR = (int)((p / outW) % outH);
    const int b = (int)(p / ((long)outW * outH));
    float* yo = y + p * outC;
    for (int c = 0; c < outC; ++c) yo[c] = 0.0f;
    const int xRCorner = yR * strideH - padTop;
    const int xCCorner = yC * strideW - padLeft;
    for (int wR = 0; wR < fH; ++wR) {
      const int xR = xRCorner + wR * dilH;
      if (xR < 0 || xR >= inH) continue;
      for (int wC = 0; wC < fW; ++wC) {
        const int xC = xCCorner + wC * dilW;
        if (xC < 0 || xC >= inW) continue;
        const float* xp = x + (((long)b * inH + xR) * inW + xC) * inC;
        const float* wp = w + ((long)wR * fW + wC) * inC * chMul;
        for (int d1 = 0; d1 < inC; ++d1) {
          const double xv = (double)xp[d1];
          for (int q = 0; q < chMul; ++q) {
            float* o = yo + d1 * chMul + q;
            *o = (float)((double)*o + xv * (double)wp[d1 * chMul + q]);
          }
        }
      }
    }
  }
}

/* ---- batchMatMul: BatchMatMul.ts:95-125 ------------------------------------
 * a3d is [batchA, M, K] (or [batchA, K, M] when transposeA), b3d likewise.
 * Blocks of 48 (backend_cpu.ts:38) over i, j, k; inside a k-block the products
 * are summed in a JS double and then added once into the fp32 result
 * (:108-119).  Batch broadcast is `bi % batchDim` (:96-97). */
void orc_batch_matmul(const float* a, const float* b, float* out, int batchA,
                      int batchB, int M, int N, int K, int transA,
                      int transB) {
  const int blockSize = 48;
  const int batch = batchA > batchB ? batchA : batchB;
  const long aBatch = (long)M * K, bBatch = (long)K * N;
  const long aOuter = transA ? 1 : K, aInner = transA ? M : 1;
  const long bInner = transB ? 1 : N, bOuter = transB ? K : 1;
  const long rows = (long)batch * M;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) {
    const int bi = (int)(r / M);
    const int i = (int)(r % M);
    const float* ap = a + (long)(bi % batchA) * aBatch + i * aOuter;
    const float* bp = b + (long)(bi % batchB) * bBatch;
    float* o = out + r * N;
    for (int j = 0; j < N; ++j) {
      float res = 0.0f;
      for (int k0 = 0; k0 < K; k0 += blockSize) {
        const int kEnd = k0 + blockSize < K ? k0 + blockSize : K;
        double sum = 0.0;
        for (int k = k0; k < kEnd; ++k)
          sum += (double)ap[k * aInner] * (double)bp[k * bInner + j * bOuter];
        res = (float)((double)res + sum);
      }
      o[j] = res;
    }
  }
}

/* ---- pool: utils/pool_utils.ts:20-87 ---------------------------------------
 * Window clipped to the image (:51-59).  Max starts at -inf and only updates
 * on `pixel > max`, so NaN taps are never selected (:68-69).  Avg divides the
 * double sum by the count of in-bounds taps (:70-73, :80-81). */
void orc_pool2d(const float* x, float* y, int isMax, int batch, int inH,
                int inW, int C, int outH, int outW, int effFH, int effFW,
                int strideH, int strideW, int dilH, int dilW, int padTop,
                int padLeft) {
  const long total = (long)batch * outH * outW;
#pragma omp parallel for schedule(static)
  for (long p = 0; p < total; ++p) {
    const int yC = (int)(p % outW);
    const int yR = (int)((p / outW) % outH);
    const int b = (int)(p / ((long)outW * outH));
    const int xRCorner = yR * strideH - padTop;
    const int xCCorner = yC * strideW - padLeft;
    const int xRMin = xRCorner > 0 ? xRCorner : 0;
    const int xRMax = inH < effFH + xRCorner ? inH : effFH + xRCorner;
    const int xCMin = xCCorner > 0 ? xCCorner : 0;
    const int xCMax = inW < effFW + xCCorner ? inW : effFW + xCCorner;
    for (int d = 0; d < C; ++d) {
      double mm = isMax ? -INFINITY : INFINITY;
      double avg = 0.0;
      int count = 0;
      for (int xR = xRMin; xR < xRMax; xR += dilH) {
        for (int xC = xCMin; xC < xCMax; xC += dilW) {
          const double pixel =
              (double)x[(((long)b * inH + xR) * inW + xC) * C + d];
          if (isMax) {
            if (pixel > mm) mm = pixel;
          } else {
            avg += pixel;
            count++;
          }
        }
        if (isnan(mm)) break;
      }
      y[p * C + d] = (float)(isMax ? mm : avg / (double)count);
    }
  }
}

/* ---- unary ops: utils/unary_impl.ts:25-36 with the per-op scalar functions ---
 * One double-precision evaluation per element, then an fp32 store. */
enum {
  ORC_U_RELU = 0,    /* Relu.ts:22      Math.max(0, x)            */
  ORC_U_RELU6 = 1,   /* Relu6.ts:22-23  Math.min(Math.max(0,x),6) */
  ORC_U_ELU = 2,     /* Elu.ts:22-23    x >= 0 ? x : exp(x) - 1   */
  ORC_U_SIGMOID = 3, /* Sigmoid.ts:23-26 1 / (1 + exp(-x))        */
  ORC_U_LEAKYRELU = 4, /* LeakyRelu.ts:38-40 x < 0 ? alpha*x : x  */
  ORC_U_EXP = 5,
  ORC_U_SQRT = 6,
  ORC_U_RSQRT = 7, /* Rsqrt.ts  1 / Math.sqrt(x) */
  ORC_U_SQUARE = 8,
  ORC_U_TANH = 9,
  ORC_U_NEG = 10,
  ORC_U_CLIP = 11, /* ClipByValue.ts  x > max ? max : (x < min ? min : x) */
  ORC_U_ERF = 12,  /* Erf.ts:29-40 */
  ORC_U_ABS = 13,
  ORC_U_LOG = 14,
  ORC_U_IDENTITY = 15
};

/* JS Math.max / Math.min: NaN if either operand is NaN; +0 beats -0 for max,
 * -0 beats +0 for min. */
static double js_max(double a, double b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a == 0.0 && b == 0.0) return signbit(a) ? b : a;
  return a > b ? a : b;
}
static double js_min(double a, double b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a == 0.0 && b == 0.0) return signbit(a) ? a : b;
  return a < b ? a : b;
}

static double orc_unary_scalar(int op, double x, double p0, double p1) {
  switch (op) {
    case ORC_U_RELU: return js_max(0.0, x);
    case ORC_U_RELU6: return js_min(js_max(0.0, x), 6.0);
    case ORC_U_ELU: return x >= 0.0 ? x : exp(x) - 1.0;
    case ORC_U_SIGMOID: return 1.0 / (1.0 + exp(-x));
    case ORC_U_LEAKYRELU: return x < 0.0 ? p0 * x : x;
    case ORC_U_EXP: return exp(x);
    case ORC_U_SQRT: return sqrt(x);
    case ORC_U_RSQRT: return 1.0 / sqrt(x);
    case ORC_U_SQUARE: return x * x;
    case ORC_U_TANH: return tanh(x);
    case ORC_U_NEG: return -x;
    case ORC_U_CLIP: return x > p1 ? p1 : (x < p0 ? p0 : x);
    case ORC_U_ERF: {
      /* Abramowitz-Stegun 7.1.26 with the constants of
       * tfjs-core/src/ops/erf_util.ts:18-23, evaluated as Erf.ts:31-39. */
      const double p = 0.3275911, a1 = 0.254829592, a2 = -0.284496736,
                   a3 = 1.421413741, a4 = -1.453152027, a5 = 1.061405429;
      const double sign = x > 0.0 ? 1.0 : (x < 0.0 ? -1.0 : x); /* Math.sign */
      const double v = fabs(x);
      const double t = 1.0 / (1.0 + p * v);
      return sign *
             (1.0 - (((((a5 * t + a4) * t) + a3) * t + a2) * t + a1) * t *
                        exp(-v * v));
    }
    case ORC_U_ABS: return fabs(x);
    case ORC_U_LOG: return log(x);
    default: return x;
  }
}

void orc_unary(int op, const float* x, float* y, long n, double p0, double p1) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i)
    y[i] = (float)orc_unary_scalar(op, (double)x[i], p0, p1);
}

/* ---- binary ops with numpy-style broadcasting: utils/binary_impl.ts:25-69 ----
 * The caller passes shapes already left-padded with 1s to a common rank; the
 * result index decomposes into a location and broadcast dims read index 0,
 * which is what the reference's loc arithmetic does (:52-64). */
enum {
  ORC_B_ADD = 0,
  ORC_B_SUB = 1,
  ORC_B_MUL = 2,
  ORC_B_DIV = 3,
  ORC_B_MAX = 4,  /* Maximum.ts  Math.max */
  ORC_B_MIN = 5,  /* Minimum.ts  Math.min */
  ORC_B_POW = 6,
  ORC_B_SQDIFF = 7, /* SquaredDifference.ts (a-b)*(a-b) */
  ORC_B_PRELU = 8   /* Prelu.ts:24-25 x < 0 ? a*x : x */
};

static double orc_binary_scalar(int op, double a, double b) {
  switch (op) {
    case ORC_B_ADD: return a + b;
    case ORC_B_SUB: return a - b;
    case ORC_B_MUL: return a * b;
    case ORC_B_DIV: return a / b;
    case ORC_B_MAX: return js_max(a, b);
    case ORC_B_MIN: return js_min(a, b);
    case ORC_B_POW: return pow(a, b);
    case ORC_B_SQDIFF: { const double d = a - b; return d * d; }
    case ORC_B_PRELU: return a < 0.0 ? b * a : a;
    default: return a;
  }
}

static void orc_bcast_strides(const long* shape, const long* outShape, int rank,
                              long* strides) {
  (void)outShape;
  long s = 1;
  for (int d = rank - 1; d >= 0; --d) {
    strides[d] = shape[d] == 1 ? 0 : s;
    s *= shape[d];
  }
}

void orc_binary_f32(int op, const float* a, const long* aShape, const float* b,
                    const long* bShape, float* out, const long* outShape,
                    int rank) {
  long as[8], bs[8], n = 1;
  orc_bcast_strides(aShape, outShape, rank, as);
  orc_bcast_strides(bShape, outShape, rank, bs);
  for (int d = 0; d < rank; ++d) n *= outShape[d];
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    long rem = i, ai = 0, bi = 0;
    for (int d = rank - 1; d >= 0; --d) {
      const long c = rem % outShape[d];
      rem /= outShape[d];
      ai += c * as[d];
      bi += c * bs[d];
    }
    out[i] = (float)orc_binary_scalar(op, (double)a[ai], (double)b[bi]);
  }
}

/* int32 flavour: the JS double result is stored into an Int32Array (ToInt32:
 * truncation, wrap modulo 2^32). */
static int32_t js_to_int32(double v) {
  if (isnan(v) || isinf(v)) return 0;
  double t = trunc(v);
  double m = fmod(t, 4294967296.0);
  if (m < 0) m += 4294967296.0;
  return (int32_t)(uint32_t)m;
}

void orc_binary_i32(int op, const int32_t* a, const long* aShape,
                    const int32_t* b, const long* bShape, int32_t* out,
                    const long* outShape, int rank) {
  long as[8], bs[8], n = 1;
  orc_bcast_strides(aShape, outShape, rank, as);
  orc_bcast_strides(bShape, outShape, rank, bs);
  for (int d = 0; d < rank; ++d) n *= outShape[d];
  for (long i = 0; i < n; ++i) {
    long rem = i, ai = 0, bi = 0;
    for (int d = rank - 1; d >= 0; --d) {
      const long c = rem % outShape[d];
      rem /= outShape[d];
      ai += c * as[d];
      bi += c * bs[d];
    }
    out[i] = js_to_int32(orc_binary_scalar(op, (double)a[ai], (double)b[bi]));
  }
}

/* ---- reductions over the innermost axis of a [rows, reduceSize] view --------
 * Sum.ts:67-74: a JS double accumulator, one fp32 store.
 * Max_impl.ts:26-36: starts from the first element; NaN is sticky. */
void orc_sum_rows(const float* x, float* y, long rows, long reduceSize) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < rows; ++i) {
    double s = 0.0;
    for (long j = 0; j < reduceSize; ++j) s += (double)x[i * reduceSize + j];
    y[i] = (float)s;
  }
}

void orc_max_rows(const float* x, float* y, long rows, long reduceSize) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < rows; ++i) {
    float m = x[i * reduceSize];
    for (long j = 0; j < reduceSize; ++j) {
      const float v = x[i * reduceSize + j];
      if (isnan(v) || v > m) m = v;
    }
    y[i] = m;
  }
}

/* Mean.ts:37-48: every element is first divided by the reduce size (an fp32
 * tensor), then the quotients are summed as in Sum. */
void orc_mean_rows(const float* x, float* y, long rows, long reduceSize) {
  const double n = (double)(float)reduceSize;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < rows; ++i) {
    double s = 0.0;
    for (long j = 0; j < reduceSize; ++j)
      s += (double)(float)((double)x[i * reduceSize + j] / n);
    y[i] = (float)s;
  }
}

/* ArgMax.ts:55-66: first index of the strict maximum. */
void orc_argmax_rows(const float* x, int32_t* y, long rows, long reduceSize) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < rows; ++i) {
    float m = x[i * reduceSize];
    int32_t mi = 0;
    for (long j = 0; j < reduceSize; ++j) {
      const float v = x[i * reduceSize + j];
      if (v > m) { m = v; mi = (int32_t)j; }
    }
    y[i] = mi;
  }
}

/* ---- softmax over the last axis: Softmax.ts:50-67 ---------------------------
 * max (NaN-sticky), a = x - max (fp32), b = exp(a) (fp32), sum in double
 * (fp32 store), out = b / sum (fp32). */
void orc_softmax_rows(const float* x, float* y, long rows, long cols) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < rows; ++i) {
    const float* xr = x + i * cols;
    float* yr = y + i * cols;
    float m = xr[0];
    for (long j = 0; j < cols; ++j)
      if (isnan(xr[j]) || xr[j] > m) m = xr[j];
    double s = 0.0;
    for (long j = 0; j < cols; ++j) {
      const float a = (float)((double)xr[j] - (double)m);
      const float e = (float)exp((double)a);
      yr[j] = e;
      s += (double)e;
    }
    const float sf = (float)s;
    for (long j = 0; j < cols; ++j)
      yr[j] = (float)((double)yr[j] / (double)sf);
  }
}

/* ---- batchNorm: BatchNorm.ts:69-87 ------------------------------------------
 * Parameter indices cycle modulo each parameter's own length. */
void orc_batchnorm(const float* x, const float* mean, long nMean,
                   const float* var, long nVar, const float* scale, long nScale,
                   const float* off, long nOff, double eps, float* y, long n) {
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    const double o = off ? (double)off[i % nOff] : 0.0;
    const double s = scale ? (double)scale[i % nScale] : 1.0;
    y[i] = (float)(o + ((double)x[i] - (double)mean[i % nMean]) * s /
                           sqrt((double)var[i % nVar] + eps));
  }
}

/* JS Math.round: nearest integer, ties toward +infinity. */
static double js_round(double v) {
  double r = floor(v);
  if (v - r >= 0.5) r += 1.0;
  return r;
}

/* ---- cast to int32: Cast.ts:30-33 (Int32Array.from => ToInt32) -------------- */
void orc_cast_f32_i32(const float* x, int32_t* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = js_to_int32((double)x[i]);
}

/* ---- weight dequantisation: tfjs-core/src/io/io_utils.ts:221-227, :243-247 ---
 * float32 target: fl32(v * scale + min) in double.  int32 target:
 * Math.round (round half up) of the same double. */
void orc_dequant_f32(const void* q, int isU16, double scale, double min,
                     float* out, long n) {
  for (long i = 0; i < n; ++i) {
    const double v = isU16 ? (double)((const uint16_t*)q)[i]
                           : (double)((const uint8_t*)q)[i];
    out[i] = (float)(v * scale + min);
  }
}

void orc_dequant_i32(const void* q, int isU16, double scale, double min,
                     int32_t* out, long n) {
  for (long i = 0; i < n; ++i) {
    const double v = isU16 ? (double)((const uint16_t*)q)[i]
                           : (double)((const uint8_t*)q)[i];
    out[i] = js_to_int32(js_round(v * scale + min));
  }
}
