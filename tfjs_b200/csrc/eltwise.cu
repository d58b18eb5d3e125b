// Bandwidth-bound elementwise and data-movement kernels: unary, broadcasting
// binary, batch-norm, cast, fill, strided copy (Concat/Slice/PadV2/Tile),
// transpose, gather and load-time weight dequantisation.
//
// All are SIMT kernels with grid-stride loops over 128-bit vectors where the
// layout allows; grids are capped at a multiple of the SM count.
#include "common.cuh"
#include <mutex>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxRank = 6;

struct Dims {
  long long v[kMaxRank];
};

// ---------------------------------------------------------------- unary ----
// One double-precision evaluation per element and one fp32 rounding, like the
// reference's scalar loops over a Float32Array
// (tfjs-backend-cpu/src/utils/unary_impl.ts:25-36).
template <int OP>
__device__ __forceinline__ float unary_eval(float x, double p0, double p1) {
  if (OP == TFJS_CUDA_RELU) return js_relu(x);
  if (OP == TFJS_CUDA_RELU6) return js_relu6(x);
  if (OP == TFJS_CUDA_ELU) return js_elu(x);
  if (OP == TFJS_CUDA_SIGMOID) return js_sigmoid(x);
  if (OP == TFJS_CUDA_LEAKYRELU) return js_leakyrelu(x, p0);
  if (OP == TFJS_CUDA_EXP) return (float)exp_fast((double)x);
  if (OP == TFJS_CUDA_SQRT) return sqrtf(x);
  if (OP == TFJS_CUDA_RSQRT) return (float)(1.0 / sqrt((double)x));
  if (OP == TFJS_CUDA_SQUARE) return x * x;
  if (OP == TFJS_CUDA_TANH) return (float)tanh((double)x);
  if (OP == TFJS_CUDA_NEG) return -x;
  if (OP == TFJS_CUDA_CLIP) {
    const double v = (double)x;
    return (float)(v > p1 ? p1 : (v < p0 ? p0 : v));
  }
  if (OP == TFJS_CUDA_ERF) return js_erf(x);
  if (OP == TFJS_CUDA_ABS) return fabsf(x);
  if (OP == TFJS_CUDA_LOG) return (float)log((double)x);
  if (OP == TFJS_CUDA_EXP_F32) return expf(x);
  if (OP == TFJS_CUDA_ERF_F32) return erf_f32(x);
  if (OP == TFJS_CUDA_SIGMOID_F32) return sigmoid_f32(x);
  if (OP == TFJS_CUDA_TANH_F32) return tanhf(x);
  if (OP == TFJS_CUDA_ELU_F32) return elu_f32(x);
  return x;
}

template <int OP>
__global__ void unary_kernel(const float* __restrict__ x, float* __restrict__ y,
                             uint64_t n, double p0, double p1) {
  const uint64_t n4 = n >> 2;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  float4* y4 = reinterpret_cast<float4*>(y);
  for (uint64_t i = tid; i < n4; i += stride) {
    float4 v = x4[i];
    if (OP == TFJS_CUDA_ERF) {
      const float in[4] = {v.x, v.y, v.z, v.w};
      float out[4];
      js_erf_vec<4>(in, out);
      y4[i] = make_float4(out[0], out[1], out[2], out[3]);
      continue;
    }
    v.x = unary_eval<OP>(v.x, p0, p1);
    v.y = unary_eval<OP>(v.y, p0, p1);
    v.z = unary_eval<OP>(v.z, p0, p1);
    v.w = unary_eval<OP>(v.w, p0, p1);
    y4[i] = v;
  }
  for (uint64_t i = (n4 << 2) + tid; i < n; i += stride)
    y[i] = unary_eval<OP>(x[i], p0, p1);
}

// --------------------------------------------------------------- binary ----
// JS semantics: Math.max / Math.min propagate NaN and order signed zeros.
__device__ __forceinline__ float js_maxf(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  if (a == 0.0f && b == 0.0f) return signbit(a) ? b : a;
  return a > b ? a : b;
}
__device__ __forceinline__ float js_minf(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  if (a == 0.0f && b == 0.0f) return signbit(a) ? a : b;
  return a < b ? a : b;
}

template <int OP>
__device__ __forceinline__ float binary_eval(float a, float b) {
  // +, -, *, / on two fp32 values rounded once equal the reference's double
  // operation followed by an fp32 store (double rounding is innocuous here).
  if (OP == TFJS_CUDA_ADD) return __fadd_rn(a, b);
  if (OP == TFJS_CUDA_SUB) return __fsub_rn(a, b);
  if (OP == TFJS_CUDA_MUL) return __fmul_rn(a, b);
  if (OP == TFJS_CUDA_DIV) return __fdiv_rn(a, b);
  if (OP == TFJS_CUDA_MAXIMUM) return js_maxf(a, b);
  if (OP == TFJS_CUDA_MINIMUM) return js_minf(a, b);
  if (OP == TFJS_CUDA_POW) return (float)pow((double)a, (double)b);
  if (OP == TFJS_CUDA_SQUARED_DIFFERENCE) {
    const double d = (double)a - (double)b;
    return (float)(d * d);
  }
  if (OP == TFJS_CUDA_PRELU) return a < 0.0f ? __fmul_rn(b, a) : a;
  return a;
}

__device__ __forceinline__ int32_t js_to_int32(double v) {
  if (!isfinite(v)) return 0;
  double t = trunc(v);
  if (t >= -2147483648.0 && t <= 2147483647.0) return (int32_t)t;
  double m = fmod(t, 4294967296.0);
  if (m < 0) m += 4294967296.0;
  return (int32_t)(uint32_t)m;
}

template <int OP>
__device__ __forceinline__ int32_t binary_eval_i32(int32_t a, int32_t b) {
  const double x = (double)a, y = (double)b;
  double r;
  if (OP == TFJS_CUDA_ADD) r = x + y;
  else if (OP == TFJS_CUDA_SUB) r = x - y;
  else if (OP == TFJS_CUDA_MUL) r = x * y;
  else if (OP == TFJS_CUDA_DIV) r = x / y;
  else if (OP == TFJS_CUDA_MAXIMUM) r = x > y ? x : y;
  else if (OP == TFJS_CUDA_MINIMUM) r = x < y ? x : y;
  else if (OP == TFJS_CUDA_POW) r = pow(x, y);
  else if (OP == TFJS_CUDA_SQUARED_DIFFERENCE) r = (x - y) * (x - y);
  else if (OP == TFJS_CUDA_PRELU) r = x < 0 ? y * x : x;
  else r = x;
  return js_to_int32(r);
}

// a and b have the same number of elements as out.
template <int OP>
__global__ void binary_same_kernel(const float* __restrict__ a,
                                   const float* __restrict__ b,
                                   float* __restrict__ o, uint64_t n) {
  const uint64_t n4 = n >> 2;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(o);
  for (uint64_t i = tid; i < n4; i += stride) {
    const float4 u = a4[i], v = b4[i];
    float4 r;
    r.x = binary_eval<OP>(u.x, v.x);
    r.y = binary_eval<OP>(u.y, v.y);
    r.z = binary_eval<OP>(u.z, v.z);
    r.w = binary_eval<OP>(u.w, v.w);
    o4[i] = r;
  }
  for (uint64_t i = (n4 << 2) + tid; i < n; i += stride)
    o[i] = binary_eval<OP>(a[i], b[i]);
}

// out = act(a + b) for equal shapes: the residual Add followed by Relu of a
// bottleneck block, in one pass (3 tensor transfers instead of 5).
template <int ACT>
__global__ void add_act_kernel(const float* __restrict__ a, const float* __restrict__ b,
                               float* __restrict__ o, uint64_t n) {
  const uint64_t n4 = n >> 2;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(o);
  auto f = [](float x, float y) {
    const float s = __fadd_rn(x, y);
    return ACT == TFJS_CUDA_ACT_RELU ? js_relu(s) : (ACT == TFJS_CUDA_ACT_RELU6 ? js_relu6(s) : s);
  };
  for (uint64_t i = tid; i < n4; i += stride) {
    const float4 u = a4[i], v = b4[i];
    o4[i] = make_float4(f(u.x, v.x), f(u.y, v.y), f(u.z, v.z), f(u.w, v.w));
  }
  for (uint64_t i = (n4 << 2) + tid; i < n; i += stride) o[i] = f(a[i], b[i]);
}

// ---- chains of elementwise ops in one pass -------------------------------------------
// Interpreter over a small program (tfjs_cuda_ew_program): a thread owns V consecutive
// output elements, keeps every value slot in a per-thread array and evaluates the ops in
// order with the same device functions as the separate kernels, so every intermediate is
// rounded to fp32 exactly as if it had been written to memory.
struct EwArgs {
  int n_inputs, n_ops;
  uint64_t n;
  uint32_t cols;
  const float* in[TFJS_CUDA_EW_MAX_INPUTS];
  int mode[TFJS_CUDA_EW_MAX_INPUTS];
  uint32_t period[TFJS_CUDA_EW_MAX_INPUTS];
  uint32_t aux[TFJS_CUDA_EW_MAX_INPUTS];
  // divisions by cols / period / aux as multiply-shift, valid for indices below 2^31
  // (the launcher sends larger tensors through the separate kernels)
  uint32_t cols_mul, cols_shr;
  uint32_t period_mul[TFJS_CUDA_EW_MAX_INPUTS], period_shr[TFJS_CUDA_EW_MAX_INPUTS];
  uint32_t aux_mul[TFJS_CUDA_EW_MAX_INPUTS], aux_shr[TFJS_CUDA_EW_MAX_INPUTS];
  tfjs_cuda_ew_op ops[TFJS_CUDA_EW_MAX_OPS];
  float* out;
};

// n / d for 0 <= n < 2^31 as umulhi(n, mul) >> shr, mul = ceil(2^(32 + shr) / d); mul = 0: d = 1.
__device__ __forceinline__ uint32_t ew_div(uint32_t n, uint32_t mul, uint32_t shr) {
  return mul ? __umulhi(n, mul) >> shr : n;
}
static void ew_div_setup(uint32_t d, uint32_t* mul, uint32_t* shr) {
  if (d <= 1) { *mul = 0; *shr = 0; return; }
  int lg = 0;
  while ((1ull << lg) < d) ++lg;
  const int p = 31 + lg;
  *mul = (uint32_t)(((1ull << p) + d - 1) / d);
  *shr = (uint32_t)(p - 32);
}

// Address of input k for the thread whose first element is e0.
__device__ __forceinline__ const float* ew_input_ptr(const EwArgs& g, int k, uint32_t e0) {
  const float* src = g.in[k];
  const int mode = g.mode[k];
  if (mode == TFJS_CUDA_EW_FULL) return src + e0;
  if (mode == TFJS_CUDA_EW_PERIODIC)
    return src + (e0 - ew_div(e0, g.period_mul[k], g.period_shr[k]) * g.period[k]);
  if (mode == TFJS_CUDA_EW_ROW) return src + ew_div(e0, g.cols_mul, g.cols_shr);
  if (mode == TFJS_CUDA_EW_BATCHED)
    return src + ew_div(e0, g.aux_mul[k], g.aux_shr[k]) * g.period[k] +
           (e0 - ew_div(e0, g.period_mul[k], g.period_shr[k]) * g.period[k]);
  return src;
}

// One decode per op: the switch is outside the loop over the thread's V elements.
template <int V>
__device__ __forceinline__ void ew_eval(int code, const float* a, const float* b, float* r) {
#define EW_BIN(OP)                                                    \
  case OP:                                                            \
    _Pragma("unroll") for (int t = 0; t < V; ++t) r[t] = binary_eval<OP>(a[t], b[t]); \
    break;
#define EW_UN(OP)                                                     \
  case TFJS_CUDA_EW_UNARY + OP:                                       \
    _Pragma("unroll") for (int t = 0; t < V; ++t) r[t] = unary_eval<OP>(a[t], 0.0, 0.0); \
    break;
  switch (code) {
    EW_BIN(TFJS_CUDA_ADD)
    EW_BIN(TFJS_CUDA_SUB)
    EW_BIN(TFJS_CUDA_MUL)
    EW_BIN(TFJS_CUDA_DIV)
    EW_BIN(TFJS_CUDA_MAXIMUM)
    EW_BIN(TFJS_CUDA_MINIMUM)
    EW_BIN(TFJS_CUDA_SQUARED_DIFFERENCE)
    EW_UN(TFJS_CUDA_RELU)
    EW_UN(TFJS_CUDA_RELU6)
    EW_UN(TFJS_CUDA_ELU)
    EW_UN(TFJS_CUDA_SIGMOID)
    EW_UN(TFJS_CUDA_EXP)
    EW_UN(TFJS_CUDA_SQRT)
    EW_UN(TFJS_CUDA_RSQRT)
    EW_UN(TFJS_CUDA_TANH)
    EW_UN(TFJS_CUDA_NEG)
    EW_UN(TFJS_CUDA_ABS)
    EW_UN(TFJS_CUDA_LOG)
    EW_UN(TFJS_CUDA_EXP_F32)
    EW_UN(TFJS_CUDA_ERF_F32)
    EW_UN(TFJS_CUDA_SIGMOID_F32)
    EW_UN(TFJS_CUDA_TANH_F32)
    EW_UN(TFJS_CUDA_ELU_F32)
    case TFJS_CUDA_EW_UNARY + TFJS_CUDA_ERF:
      js_erf_vec<V>(a, r);
      break;
    case TFJS_CUDA_EW_UNARY + TFJS_CUDA_SQUARE:
#pragma unroll
      for (int t = 0; t < V; ++t) r[t] = __fmul_rn(a[t], a[t]);
      break;
    default:
#pragma unroll
      for (int t = 0; t < V; ++t) r[t] = a[t];
      break;
  }
#undef EW_BIN
#undef EW_UN
}

// V = 4: n, cols and every period are multiples of 4 (or the period is 1) and every pointer
// is 16-byte aligned; V = 1 otherwise.  Indices fit 32 bits (checked by the launcher).
template <int V>
__global__ void __launch_bounds__(256)
fused_elementwise_kernel(const __grid_constant__ EwArgs g) {
  const uint32_t nv = (uint32_t)(g.n / V);
  const uint32_t stride = gridDim.x * blockDim.x;
  constexpr int kSlots = TFJS_CUDA_EW_MAX_INPUTS + TFJS_CUDA_EW_MAX_OPS;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float vals[kSlots][V];
    const uint32_t e0 = i * V;  // first element of this thread
    for (int k = 0; k < g.n_inputs; ++k) {
      const float* src = ew_input_ptr(g, k, e0);
      const int mode = g.mode[k];
      if (mode == TFJS_CUDA_EW_ROW || mode == TFJS_CUDA_EW_SCALAR) {
        const float sv = __ldg(src);
#pragma unroll
        for (int t = 0; t < V; ++t) vals[k][t] = sv;
      } else if (V == 4) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(src));
        vals[k][0] = q.x; vals[k][1 % V] = q.y; vals[k][2 % V] = q.z; vals[k][3 % V] = q.w;
      } else {
        vals[k][0] = __ldg(src);
      }
    }
    for (int j = 0; j < g.n_ops; ++j) {
      const tfjs_cuda_ew_op op = g.ops[j];
      float r[V];
      ew_eval<V>(op.opcode, vals[op.a], vals[op.b], r);
#pragma unroll
      for (int t = 0; t < V; ++t) vals[g.n_inputs + j][t] = r[t];
    }
    const int last = g.n_inputs + g.n_ops - 1;
    if (V == 4) {
      *reinterpret_cast<float4*>(g.out + e0) =
          make_float4(vals[last][0], vals[last][1 % V], vals[last][2 % V], vals[last][3 % V]);
    } else {
      g.out[e0] = vals[last][0];
    }
  }
}

// One operand is the full tensor, the other repeats with period `period`
// (bias over the innermost axis, or a scalar when period == 1).  period % 4 == 0
// or period == 1.  SWAP: the periodic operand is the left one.
template <int OP, bool SWAP>
__global__ void binary_periodic_kernel(const float* __restrict__ full,
                                       const float* __restrict__ per,
                                       float* __restrict__ o, uint64_t n,
                                       uint32_t period) {
  const uint64_t n4 = n >> 2;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const float4* f4 = reinterpret_cast<const float4*>(full);
  const float4* p4 = reinterpret_cast<const float4*>(per);
  float4* o4 = reinterpret_cast<float4*>(o);
  const float s = per[0];
  // position inside the period in float4 units, advanced without a division per element
  const uint32_t per4 = period == 1 ? 1u : period >> 2;
  const uint32_t step = (uint32_t)(stride % per4);
  uint32_t r = (uint32_t)(tid % per4);
  for (uint64_t i = tid; i < n4; i += stride) {
    const float4 u = f4[i];
    const float4 v = period == 1 ? make_float4(s, s, s, s) : __ldg(p4 + r);
    r += step;
    if (r >= per4) r -= per4;
    float4 q;
    q.x = SWAP ? binary_eval<OP>(v.x, u.x) : binary_eval<OP>(u.x, v.x);
    q.y = SWAP ? binary_eval<OP>(v.y, u.y) : binary_eval<OP>(u.y, v.y);
    q.z = SWAP ? binary_eval<OP>(v.z, u.z) : binary_eval<OP>(u.z, v.z);
    q.w = SWAP ? binary_eval<OP>(v.w, u.w) : binary_eval<OP>(u.w, v.w);
    o4[i] = q;
  }
  for (uint64_t i = (n4 << 2) + tid; i < n; i += stride) {
    const float v = per[period == 1 ? 0 : i % period];
    o[i] = SWAP ? binary_eval<OP>(v, full[i]) : binary_eval<OP>(full[i], v);
  }
}

// out[o][m][i] = full[o][m][i] op small[o][i]: the small operand equals the output shape on
// a leading and a trailing group of axes and is 1 in between (an attention mask
// [B,1,1,S] against scores [B,H,S,S]).  inner % 4 == 0; sizes in float4 units fit 32 bits.
template <int OP, bool SWAP>
__global__ void binary_batched_periodic_kernel(const float* __restrict__ full,
                                               const float* __restrict__ small_op,
                                               float* __restrict__ o, uint32_t n4,
                                               uint32_t inner4, uint32_t mid_inner4) {
  const uint32_t stride = gridDim.x * blockDim.x;
  const float4* f4 = reinterpret_cast<const float4*>(full);
  const float4* s4 = reinterpret_cast<const float4*>(small_op);
  float4* o4 = reinterpret_cast<float4*>(o);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const uint32_t outer = i / mid_inner4;
    const uint32_t in4 = (i - outer * mid_inner4) % inner4;
    const float4 u = f4[i];
    const float4 v = __ldg(s4 + outer * inner4 + in4);
    float4 q;
    q.x = SWAP ? binary_eval<OP>(v.x, u.x) : binary_eval<OP>(u.x, v.x);
    q.y = SWAP ? binary_eval<OP>(v.y, u.y) : binary_eval<OP>(u.y, v.y);
    q.z = SWAP ? binary_eval<OP>(v.z, u.z) : binary_eval<OP>(u.z, v.z);
    q.w = SWAP ? binary_eval<OP>(v.w, u.w) : binary_eval<OP>(u.w, v.w);
    o4[i] = q;
  }
}

// One operand is the full tensor viewed as [rows, cols]; the other has one value
// per row (shape [..., 1], e.g. the mean / rsqrt terms of a layer norm).  cols % 4 == 0.
template <int OP>
__global__ void binary_rowscalar_kernel(const float* __restrict__ full,
                                        const float* __restrict__ per_row,
                                        float* __restrict__ o, uint64_t n, uint32_t cols,
                                        bool swap) {
  const uint64_t n4 = n >> 2;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const float4* f4 = reinterpret_cast<const float4*>(full);
  float4* o4 = reinterpret_cast<float4*>(o);
  const uint32_t c4 = cols >> 2;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 u = f4[i];
    const float v = __ldg(per_row + i / c4);
    float4 r;
    r.x = swap ? binary_eval<OP>(v, u.x) : binary_eval<OP>(u.x, v);
    r.y = swap ? binary_eval<OP>(v, u.y) : binary_eval<OP>(u.y, v);
    r.z = swap ? binary_eval<OP>(v, u.z) : binary_eval<OP>(u.z, v);
    r.w = swap ? binary_eval<OP>(v, u.w) : binary_eval<OP>(u.w, v);
    o4[i] = r;
  }
}

// I is the index type: uint32_t when every extent fits, which keeps the per-element
// div/mod chain in 32-bit arithmetic.
template <int OP, typename T, typename I>
__global__ void binary_general_kernel(const T* __restrict__ a,
                                      const T* __restrict__ b, T* __restrict__ o,
                                      uint64_t n, int rank, Dims oshape,
                                      Dims astride, Dims bstride) {
  const I stride = (I)gridDim.x * blockDim.x;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < (I)n; i += stride) {
    I rem = i;
    I ai = 0, bi = 0;
    for (int d = rank - 1; d >= 0; --d) {
      const I ext = (I)oshape.v[d];
      const I q = rem / ext;
      const I c = rem - q * ext;
      rem = q;
      ai += c * (I)astride.v[d];
      bi += c * (I)bstride.v[d];
    }
    if ((T)0.5f != (T)0)  // T is float
      o[i] = (T)binary_eval<OP>((float)a[ai], (float)b[bi]);
    else
      o[i] = (T)binary_eval_i32<OP>((int32_t)a[ai], (int32_t)b[bi]);
  }
}

// ------------------------------------------------------------ batch norm ----
// tfjs-backend-cpu/src/kernels/BatchNorm.ts:69-87.
__global__ void batchnorm_kernel(const float* __restrict__ x, uint64_t n,
                                 const float* __restrict__ mean, uint64_t n_mean,
                                 const float* __restrict__ var, uint64_t n_var,
                                 const float* __restrict__ scale,
                                 uint64_t n_scale, const float* __restrict__ off,
                                 uint64_t n_off, double eps,
                                 float* __restrict__ y) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const double o = off ? (double)off[i % n_off] : 0.0;
    const double s = scale ? (double)scale[i % n_scale] : 1.0;
    y[i] = (float)(o + ((double)x[i] - (double)mean[i % n_mean]) * s /
                           sqrt((double)var[i % n_var] + eps));
  }
}

// The same arithmetic on a [rows, cols] view of x whose parameters are rows or columns of
// it: tfjs-layers' LayerNormalization tiles the moments (one value per row) and gamma / beta
// (one per column) to the input's shape and calls batchNorm on the tiles
// (tfjs-layers/src/layers/normalization.ts:578-622); with the tiles left unmaterialised the
// kernel indexes the untiled tensors.  Parameter modes: 0 absent, 1 one value per column,
// 2 one value per row, 3 one value per element, 4 a single value.
struct BnParam {
  const float* p;
  int mode;
};
__device__ __forceinline__ double bn_fetch(const BnParam& q, uint64_t i, uint32_t r,
                                           uint32_t c, double absent) {
  switch (q.mode) {
    case 1: return (double)__ldg(q.p + c);
    case 2: return (double)__ldg(q.p + r);
    case 3: return (double)__ldg(q.p + i);
    case 4: return (double)__ldg(q.p);
    default: return absent;
  }
}
__global__ void batchnorm_rows_kernel(const float* __restrict__ x, uint32_t rows, uint32_t cols,
                                      BnParam mean, BnParam var, BnParam scale, BnParam off,
                                      double eps, float* __restrict__ y) {
  const uint64_t n = (uint64_t)rows * cols;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const uint32_t r = (uint32_t)(i / cols), c = (uint32_t)(i - (uint64_t)r * cols);
    const double o = bn_fetch(off, i, r, c, 0.0);
    const double sc = bn_fetch(scale, i, r, c, 1.0);
    y[i] = (float)(o + ((double)x[i] - bn_fetch(mean, i, r, c, 0.0)) * sc /
                           sqrt(bn_fetch(var, i, r, c, 1.0) + eps));
  }
}

// ------------------------------------------------------------------ cast ----
// tfjs-backend-cpu/src/kernels/Cast.ts:30-45.
template <typename TI, typename TO, int MODE>  // 0 convert, 1 to-int32 (JS), 2 to-bool
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y,
                            uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    if (MODE == 1) y[i] = (TO)js_to_int32((double)x[i]);
    else if (MODE == 2) y[i] = (TO)(x[i] != (TI)0 ? 1 : 0);
    else y[i] = (TO)x[i];
  }
}

__global__ void fill32_kernel(uint32_t* __restrict__ y, uint32_t bits, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride)
    y[i] = bits;
}

// --------------------------------------------------------- strided copy ----
template <typename T>
__global__ void copy_strided_kernel(const T* __restrict__ x, T* __restrict__ o,
                                    uint64_t n, int rank, Dims extent,
                                    long long x_off, Dims xs, Dims xw,
                                    long long o_off, Dims os) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    uint64_t rem = i;
    long long xi = x_off, oi = o_off;
    for (int d = rank - 1; d >= 0; --d) {
      const long long c = (long long)(rem % (uint64_t)extent.v[d]);
      rem /= (uint64_t)extent.v[d];
      xi += (c % xw.v[d]) * xs.v[d];
      oi += c * os.v[d];
    }
    o[oi] = x[xi];
  }
}

// ------------------------------------------------------------- transpose ----
// Output-major traversal: writes are coalesced, reads are gathered through L2.
// T is the moved unit (1, 4 or 16 bytes; 16 when the innermost axis stays put).
template <typename T, typename I>
__global__ void transpose_kernel(const T* __restrict__ x, T* __restrict__ o,
                                 uint64_t n, int rank, Dims oshape,
                                 Dims xstride_for_out) {
  const I stride = (I)gridDim.x * blockDim.x;
  for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < (I)n; i += stride) {
    I rem = i;
    I xi = 0;
    for (int d = rank - 1; d >= 0; --d) {
      const I ext = (I)oshape.v[d];
      const I q = rem / ext;
      xi += (rem - q * ext) * (I)xstride_for_out.v[d];
      rem = q;
    }
    o[i] = x[xi];
  }
}

// 2-D tiled transpose of the two innermost axes of a [batch, rows, cols] view
// through shared memory (both sides coalesced).
__global__ void transpose2d_kernel(const float* __restrict__ x,
                                   float* __restrict__ o, int rows, int cols) {
  __shared__ float tile[32][33];
  const uint64_t base = (uint64_t)blockIdx.z * rows * cols;
  int c = blockIdx.x * 32 + threadIdx.x;
  int r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int r = r0 + j;
    if (r < rows && c < cols) tile[j][threadIdx.x] = x[base + (uint64_t)r * cols + c];
  }
  __syncthreads();
  const int orow0 = blockIdx.x * 32;  // output rows = input cols
  const int oc = blockIdx.y * 32 + threadIdx.x;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    const int orow = orow0 + j;
    if (orow < cols && oc < rows)
      o[base + (uint64_t)orow * rows + oc] = tile[threadIdx.x][j];
  }
}

// ---------------------------------------------------------------- gather ----
// out[b, o, i, :] = x[b, o, idx[b, i], :]
// (tfjs-backend-cpu/src/kernels/GatherV2_impl.ts:20-41).  An index outside
// [0, dim-1] is reported through `bad` and the slice is zero-filled instead of
// being read.
template <typename T>
__global__ void gather_kernel(const T* __restrict__ x,
                              const int32_t* __restrict__ idx, T* __restrict__ o,
                              uint64_t n, uint64_t outer, uint64_t dim,
                              uint64_t slice, uint64_t n_idx,
                              long long* __restrict__ bad) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const uint64_t s = i % slice;
    uint64_t rem = i / slice;
    const uint64_t ii = rem % n_idx;
    rem /= n_idx;
    const uint64_t oo = rem % outer;
    const uint64_t b = rem / outer;
    const long long g = idx[b * n_idx + ii];
    if (g < 0 || g >= (long long)dim) {
      if (bad) atomicCAS((unsigned long long*)bad, (unsigned long long)-1LL,
                         (unsigned long long)g);
      T z;
      memset(&z, 0, sizeof(T));
      o[i] = z;
    } else {
      o[i] = x[((b * outer + oo) * dim + (uint64_t)g) * slice + s];
    }
  }
}

// --------------------------------------------------------------- dequant ----
// tfjs-core/src/io/io_utils.ts:221-227: values[i] = v * scale + min.  The table
// holds fl32(v*scale+min) for every possible v, computed on the host in double.
template <typename TO>
__global__ void dequant_u8_kernel(const uint8_t* __restrict__ q,
                                  const TO* __restrict__ table,
                                  TO* __restrict__ o, uint64_t n) {
  __shared__ TO lut[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = table[i];
  __syncthreads();
  const uint64_t n16 = n >> 4;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* q16 = reinterpret_cast<const uint4*>(q);
  for (uint64_t i = tid; i < n16; i += stride) {
    const uint4 w = q16[i];
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      TO r[4];
      r[0] = lut[words[j] & 0xff];
      r[1] = lut[(words[j] >> 8) & 0xff];
      r[2] = lut[(words[j] >> 16) & 0xff];
      r[3] = lut[words[j] >> 24];
      *reinterpret_cast<uint4*>(o + (i << 4) + (j << 2)) =
          *reinterpret_cast<const uint4*>(r);
    }
  }
  for (uint64_t i = (n16 << 4) + tid; i < n; i += stride) o[i] = lut[q[i]];
}

template <typename TO>
__global__ void dequant_u16_kernel(const uint16_t* __restrict__ q,
                                   const TO* __restrict__ table,
                                   TO* __restrict__ o, uint64_t n) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride)
    o[i] = table[q[i]];
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

// ---- catalogued chains: straight-line kernels ------------------------------------------
// The chains the graph models actually contain are compiled ahead of time: the program is
// a compile-time constant, so the loop over ops unrolls, every value slot is a register and
// each op is the inlined device function of the separate kernel.  A program matches an
// entry when its ops and operand slots are identical (the host layer brings programs into
// a canonical order first); input addressing modes stay run-time values.
struct StaticOp {
  int code, a, b;
};
#define EW_B(OP, A, B) StaticOp{TFJS_CUDA_##OP, A, B}
#define EW_U(OP, A) StaticOp{TFJS_CUDA_EW_UNARY + TFJS_CUDA_##OP, A, A}
// slots: inputs first, then one per op
struct ProgLayerNormTail {  // ((x - mean) * rstd) * gamma + beta
  static constexpr int n_in = 5, n_ops = 4;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[4] = {EW_B(SUB, 0, 1), EW_B(MUL, 5, 2), EW_B(MUL, 6, 3),
                               EW_B(ADD, 7, 4)};
    return t[j];
  }
};
struct ProgLayerNormTailBn {  // x * (rstd * gamma) + (beta - mean * (rstd * gamma))
  static constexpr int n_in = 5, n_ops = 6;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[6] = {EW_B(MUL, 1, 2), EW_B(MUL, 5, 3), EW_B(SUB, 0, 6),
                                      EW_B(MUL, 1, 2), EW_B(MUL, 8, 4), EW_B(ADD, 7, 9)};
    return t[j];
  }
};
struct ProgGeluErf {  // (x * 0.5) * (erf(x * c) + 1)
  static constexpr int n_in = 4, n_ops = 5;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(MUL, 0, 1), EW_U(ERF, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 0, 3), EW_B(MUL, 6, 7)};
    return t[j];
  }
};
struct ProgGeluErfDiv {  // (x * 0.5) * (erf(x / c) + 1)
  static constexpr int n_in = 4, n_ops = 5;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(DIV, 0, 1), EW_U(ERF, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 0, 3), EW_B(MUL, 6, 7)};
    return t[j];
  }
};
struct ProgGeluErfF32 {  // the same chain with the fp32 erf (TF32 math mode)
  static constexpr int n_in = 4, n_ops = 5;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(MUL, 0, 1), EW_U(ERF_F32, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 0, 3), EW_B(MUL, 6, 7)};
    return t[j];
  }
};
struct ProgGeluErfDivF32 {
  static constexpr int n_in = 4, n_ops = 5;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(DIV, 0, 1), EW_U(ERF_F32, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 0, 3), EW_B(MUL, 6, 7)};
    return t[j];
  }
};
struct ProgGeluLayers {  // x * (0.5 * (erf(x / c) + 1)): the Gelu activation of tfjs-layers
  static constexpr int n_in = 4, n_ops = 5;   // (tfjs-layers/src/activations.ts:223-233)
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(DIV, 0, 1), EW_U(ERF, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 6, 3), EW_B(MUL, 7, 0)};
    return t[j];
  }
};
struct ProgGeluLayersF32 {
  static constexpr int n_in = 4, n_ops = 5;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[5] = {EW_B(DIV, 0, 1), EW_U(ERF_F32, 4), EW_B(ADD, 5, 2),
                                      EW_B(MUL, 6, 3), EW_B(MUL, 7, 0)};
    return t[j];
  }
};
struct ProgBiasGeluLayers {  // t = x + bias; t * (0.5 * (erf(t / c) + 1)): a Dense layer of
  static constexpr int n_in = 5, n_ops = 6;   // tfjs-layers with the gelu activation
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[6] = {EW_B(ADD, 0, 1), EW_B(DIV, 5, 2), EW_U(ERF, 6), EW_B(ADD, 7, 3),
                                      EW_B(MUL, 8, 4), EW_B(MUL, 5, 9)};
    return t[j];
  }
};
struct ProgBiasGeluLayersF32 {
  static constexpr int n_in = 5, n_ops = 6;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[6] = {EW_B(ADD, 0, 1), EW_B(DIV, 5, 2), EW_U(ERF_F32, 6),
                                      EW_B(ADD, 7, 3), EW_B(MUL, 8, 4), EW_B(MUL, 5, 9)};
    return t[j];
  }
};
struct ProgScaleShift {  // x * a + b (attention scores * scale + mask, affine maps)
  static constexpr int n_in = 3, n_ops = 2;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[2] = {EW_B(MUL, 0, 1), EW_B(ADD, 3, 2)};
    return t[j];
  }
};
struct ProgAddAdd {  // (a + b) + c (residual + bias)
  static constexpr int n_in = 3, n_ops = 2;
  __host__ __device__ static constexpr StaticOp op(int j) {
    constexpr StaticOp t[2] = {EW_B(ADD, 0, 1), EW_B(ADD, 3, 2)};
    return t[j];
  }
};
#undef EW_B
#undef EW_U

// SIMPLE: every input is either a full tensor or a scalar; the scalars are fetched once,
// ahead of the loop, and no index arithmetic is left in it.
template <class P, int V, bool SIMPLE>
__global__ void __launch_bounds__(256)
fused_elementwise_static_kernel(const __grid_constant__ EwArgs g) {
  const uint32_t nv = (uint32_t)(g.n / V);
  const uint32_t stride = gridDim.x * blockDim.x;
  float scalar[P::n_in];
  bool is_scalar[P::n_in];
  if (SIMPLE) {
#pragma unroll
    for (int k = 0; k < P::n_in; ++k) {
      is_scalar[k] = g.mode[k] == TFJS_CUDA_EW_SCALAR;
      scalar[k] = is_scalar[k] ? __ldg(g.in[k]) : 0.0f;
    }
  }
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const uint32_t e0 = i * V;
    float vals[P::n_in + P::n_ops][V];
#pragma unroll
    for (int k = 0; k < P::n_in; ++k) {
      if (SIMPLE) {
        if (is_scalar[k]) {
#pragma unroll
          for (int t = 0; t < V; ++t) vals[k][t] = scalar[k];
        } else if (V == 4) {
          const float4 q = __ldg(reinterpret_cast<const float4*>(g.in[k] + e0));
          vals[k][0] = q.x; vals[k][1 % V] = q.y; vals[k][2 % V] = q.z; vals[k][3 % V] = q.w;
        } else {
          vals[k][0] = __ldg(g.in[k] + e0);
        }
        continue;
      }
      const float* src = ew_input_ptr(g, k, e0);
      const int mode = g.mode[k];
      if (mode == TFJS_CUDA_EW_ROW || mode == TFJS_CUDA_EW_SCALAR) {
        const float sv = __ldg(src);
#pragma unroll
        for (int t = 0; t < V; ++t) vals[k][t] = sv;
      } else if (V == 4) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(src));
        vals[k][0] = q.x; vals[k][1 % V] = q.y; vals[k][2 % V] = q.z; vals[k][3 % V] = q.w;
      } else {
        vals[k][0] = __ldg(src);
      }
    }
#pragma unroll
    for (int j = 0; j < P::n_ops; ++j)
      ew_eval<V>(P::op(j).code, vals[P::op(j).a], vals[P::op(j).b], vals[P::n_in + j]);
    constexpr int last = P::n_in + P::n_ops - 1;
    if (V == 4) {
      *reinterpret_cast<float4*>(g.out + e0) =
          make_float4(vals[last][0], vals[last][1 % V], vals[last][2 % V], vals[last][3 % V]);
    } else {
      g.out[e0] = vals[last][0];
    }
  }
}

template <class P>
static bool ew_matches(const EwArgs& g) {
  if (g.n_inputs != P::n_in || g.n_ops != P::n_ops) return false;
  for (int j = 0; j < P::n_ops; ++j)
    if (g.ops[j].opcode != P::op(j).code || g.ops[j].a != P::op(j).a ||
        g.ops[j].b != P::op(j).b)
      return false;
  return true;
}

template <class P>
static void ew_launch_static(tfjs_cuda_ctx* ctx, const EwArgs& g, bool vec) {
  bool simple = true;
  for (int k = 0; k < g.n_inputs; ++k)
    simple = simple && (g.mode[k] == TFJS_CUDA_EW_FULL || g.mode[k] == TFJS_CUDA_EW_SCALAR);
  const unsigned grid = grid_for(vec ? g.n / 4 : g.n, kThreads, ctx->sm_count);
  if (vec && simple)
    fused_elementwise_static_kernel<P, 4, true><<<grid, kThreads, 0, ctx->stream>>>(g);
  else if (vec)
    fused_elementwise_static_kernel<P, 4, false><<<grid, kThreads, 0, ctx->stream>>>(g);
  else
    fused_elementwise_static_kernel<P, 1, false><<<grid, kThreads, 0, ctx->stream>>>(g);
}

// Launches the catalogue entry that matches g (dry_run: only reports whether one does).
static bool ew_launch_catalogued(tfjs_cuda_ctx* ctx, const EwArgs& g, bool vec,
                                 bool dry_run = false) {
#define EW_TRY(P)                                  \
  if (ew_matches<P>(g)) {                          \
    if (!dry_run) ew_launch_static<P>(ctx, g, vec); \
    return true;                                   \
  }
  EW_TRY(ProgLayerNormTail)
  EW_TRY(ProgLayerNormTailBn)
  EW_TRY(ProgGeluErf)
  EW_TRY(ProgGeluErfDiv)
  EW_TRY(ProgGeluErfF32)
  EW_TRY(ProgGeluErfDivF32)
  EW_TRY(ProgGeluLayers)
  EW_TRY(ProgGeluLayersF32)
  EW_TRY(ProgBiasGeluLayers)
  EW_TRY(ProgBiasGeluLayersF32)
  EW_TRY(ProgScaleShift)
  EW_TRY(ProgAddAdd)
#undef EW_TRY
  return false;
}

extern "C" {

int tfjs_cuda_unary(tfjs_cuda_ctx* ctx, int32_t op, double p0, double p1,
                    int32_t x_id, uint64_t n, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *x, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, n * 4, "unary x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "unary out", &y))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for((n + 3) / 4, kThreads, ctx->sm_count);
  const float* xp = (const float*)x->ptr;
  float* yp = (float*)y->ptr;
  if (op < 0 || op > TFJS_CUDA_LOG)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "unary: unknown op %d", op);
  // the default math mode evaluates exp / erf / sigmoid / tanh / elu in fp32
  if (ctx->math_mode == TFJS_CUDA_MATH_TF32) op = fast_unary_op(op);
#define UN(OP) case OP: unary_kernel<OP><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, n, p0, p1); break;
  switch (op) {
    UN(TFJS_CUDA_RELU) UN(TFJS_CUDA_RELU6) UN(TFJS_CUDA_ELU) UN(TFJS_CUDA_SIGMOID)
    UN(TFJS_CUDA_LEAKYRELU) UN(TFJS_CUDA_EXP) UN(TFJS_CUDA_SQRT) UN(TFJS_CUDA_RSQRT)
    UN(TFJS_CUDA_SQUARE) UN(TFJS_CUDA_TANH) UN(TFJS_CUDA_NEG) UN(TFJS_CUDA_CLIP)
    UN(TFJS_CUDA_ERF) UN(TFJS_CUDA_ABS) UN(TFJS_CUDA_LOG)
    UN(TFJS_CUDA_EXP_F32) UN(TFJS_CUDA_ERF_F32) UN(TFJS_CUDA_SIGMOID_F32)
    UN(TFJS_CUDA_TANH_F32) UN(TFJS_CUDA_ELU_F32)
    default: return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "unary: unknown op %d", op);
  }
#undef UN
  LAUNCH_CHECK(ctx, "unary_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_binary(tfjs_cuda_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                     int32_t a_id, const int64_t* a_shape, int32_t b_id,
                     const int64_t* b_shape, int32_t out_id,
                     const int64_t* out_shape) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (rank < 0 || rank > kMaxRank)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "binary: rank %d > %d", rank, kMaxRank);
  if (dtype != TFJS_CUDA_FLOAT32 && dtype != TFJS_CUDA_INT32)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "binary: dtype %d", dtype);
  uint64_t na = 1, nb = 1, n = 1;
  Dims os, as, bs;
  for (int d = 0; d < kMaxRank; ++d) os.v[d] = 1, as.v[d] = 0, bs.v[d] = 0;
  for (int d = 0; d < rank; ++d) {
    if (a_shape[d] != out_shape[d] && a_shape[d] != 1)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "binary: a not broadcastable");
    if (b_shape[d] != out_shape[d] && b_shape[d] != 1)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "binary: b not broadcastable");
    na *= a_shape[d]; nb *= b_shape[d]; n *= out_shape[d];
    os.v[d] = out_shape[d];
  }
  long long sa = 1, sb = 1;
  for (int d = rank - 1; d >= 0; --d) {
    as.v[d] = a_shape[d] == 1 ? 0 : sa;
    bs.v[d] = b_shape[d] == 1 ? 0 : sb;
    sa *= a_shape[d];
    sb *= b_shape[d];
  }
  Buffer *a, *b, *o;
  int rc;
  if ((rc = ctx_get(ctx, a_id, na * 4, "binary a", &a))) return rc;
  if ((rc = ctx_get(ctx, b_id, nb * 4, "binary b", &b))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "binary out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  // Classify: same-size, or one side periodic over a suffix of the out shape.
  int mode = 2;  // general
  uint32_t period = 0, bp_inner4 = 0, bp_mid_inner4 = 0;
  bool swap = false;
  if (dtype == TFJS_CUDA_FLOAT32) {
    auto suffix_period = [&](const int64_t* s, uint64_t cnt) -> bool {
      // true when s is 1 on a prefix and equals out_shape on the rest
      int d = 0;
      while (d < rank && s[d] == 1) ++d;
      for (int e = d; e < rank; ++e)
        if (s[e] != out_shape[e]) return false;
      return cnt <= 0xffffffffu;
    };
    auto row_scalar = [&](const int64_t* s, uint64_t cnt) -> bool {
      // s equals out_shape except for a trailing 1, and rows of 4k floats
      if (rank < 1 || s[rank - 1] != 1 || out_shape[rank - 1] % 4 != 0 ||
          out_shape[rank - 1] > 0xffffffffll)
        return false;
      for (int e = 0; e < rank - 1; ++e)
        if (s[e] != out_shape[e]) return false;
      return cnt * (uint64_t)out_shape[rank - 1] == n;
    };
    auto batched_period = [&](const int64_t* sh) -> bool {
      // equal to out_shape on axes [0, p) and [q, rank), 1 on [p, q), with 0 < p < q < rank
      int p = 0;
      while (p < rank && sh[p] == out_shape[p]) ++p;
      int q = p;
      while (q < rank && sh[q] == 1) ++q;
      if (p == 0 || q == p || q == rank) return false;
      uint64_t inner = 1, mid = 1;
      for (int e = q; e < rank; ++e) {
        if (sh[e] != out_shape[e]) return false;
        inner *= (uint64_t)out_shape[e];
      }
      for (int e = p; e < q; ++e) mid *= (uint64_t)out_shape[e];
      if (inner % 4 != 0 || mid < 2 || n / 4 > 0xffffffffull) return false;
      bp_inner4 = (uint32_t)(inner / 4);
      bp_mid_inner4 = (uint32_t)(mid * inner / 4);
      return true;
    };
    if (na == n && nb == n) mode = 0;
    else if (na == n && nb > 1 && row_scalar(b_shape, nb)) {
      mode = 3; period = (uint32_t)out_shape[rank - 1]; swap = false;
    } else if (nb == n && na > 1 && row_scalar(a_shape, na)) {
      mode = 3; period = (uint32_t)out_shape[rank - 1]; swap = true;
    }
    else if (na == n && nb > 1 && batched_period(b_shape)) {
      mode = 4; swap = false;
    } else if (nb == n && na > 1 && batched_period(a_shape)) {
      mode = 4; swap = true;
    }
    else if (na == n && suffix_period(b_shape, nb) && (nb == 1 || nb % 4 == 0)) {
      mode = 1; period = (uint32_t)nb; swap = false;
    } else if (nb == n && suffix_period(a_shape, na) && (na == 1 || na % 4 == 0)) {
      mode = 1; period = (uint32_t)na; swap = true;
    }
  }
  const float* ap = (const float*)a->ptr;
  const float* bp = (const float*)b->ptr;
  float* op_ = (float*)o->ptr;
  const bool small = n < 0x7fffffffull && na < 0x7fffffffull && nb < 0x7fffffffull;
#define BIN_CASE(OP)                                                              \
  case OP:                                                                        \
    if (mode == 0)                                                                \
      binary_same_kernel<OP><<<grid_for((n + 3) / 4, kThreads, ctx->sm_count),    \
                               kThreads, 0, ctx->stream>>>(ap, bp, op_, n);       \
    else if (mode == 1 && !swap)                                                  \
      binary_periodic_kernel<OP, false>                                           \
          <<<grid_for((n + 3) / 4, kThreads, ctx->sm_count), kThreads, 0,         \
             ctx->stream>>>(ap, bp, op_, n, period);                              \
    else if (mode == 1)                                                           \
      binary_periodic_kernel<OP, true>                                            \
          <<<grid_for((n + 3) / 4, kThreads, ctx->sm_count), kThreads, 0,         \
             ctx->stream>>>(bp, ap, op_, n, period);                              \
    else if (mode == 4 && !swap)                                                  \
      binary_batched_periodic_kernel<OP, false>                                   \
          <<<grid_for(n / 4, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>( \
              ap, bp, op_, (uint32_t)(n / 4), bp_inner4, bp_mid_inner4);           \
    else if (mode == 4)                                                           \
      binary_batched_periodic_kernel<OP, true>                                    \
          <<<grid_for(n / 4, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>( \
              bp, ap, op_, (uint32_t)(n / 4), bp_inner4, bp_mid_inner4);           \
    else if (mode == 3)                                                           \
      binary_rowscalar_kernel<OP><<<grid_for((n + 3) / 4, kThreads, ctx->sm_count), \
                                    kThreads, 0, ctx->stream>>>(                  \
          swap ? bp : ap, swap ? ap : bp, op_, n, period, swap);                  \
    else if (dtype == TFJS_CUDA_FLOAT32 && small)                                 \
      binary_general_kernel<OP, float, uint32_t>                                  \
          <<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(   \
              ap, bp, op_, n, rank, os, as, bs);                                  \
    else if (dtype == TFJS_CUDA_FLOAT32)                                          \
      binary_general_kernel<OP, float, uint64_t>                                  \
          <<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(   \
              ap, bp, op_, n, rank, os, as, bs);                                  \
    else                                                                          \
      binary_general_kernel<OP, int32_t, uint64_t>                                \
          <<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(   \
              (const int32_t*)a->ptr, (const int32_t*)b->ptr, (int32_t*)o->ptr,   \
              n, rank, os, as, bs);                                               \
    break;
  switch (op) {
    BIN_CASE(TFJS_CUDA_ADD) BIN_CASE(TFJS_CUDA_SUB) BIN_CASE(TFJS_CUDA_MUL)
    BIN_CASE(TFJS_CUDA_DIV) BIN_CASE(TFJS_CUDA_MAXIMUM) BIN_CASE(TFJS_CUDA_MINIMUM)
    BIN_CASE(TFJS_CUDA_POW) BIN_CASE(TFJS_CUDA_SQUARED_DIFFERENCE)
    BIN_CASE(TFJS_CUDA_PRELU)
    default: return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "binary: unknown op %d", op);
  }
#undef BIN_CASE
  LAUNCH_CHECK(ctx, "binary_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_fused_elementwise(tfjs_cuda_ctx* ctx, const tfjs_cuda_ew_program* p,
                                int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (!p || p->n_inputs < 1 || p->n_inputs > TFJS_CUDA_EW_MAX_INPUTS || p->n_ops < 1 ||
      p->n_ops > TFJS_CUDA_EW_MAX_OPS || p->cols < 1)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_elementwise: bad program header");
  if (p->n >= (1ull << 31))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "fused_elementwise: 2^31 elements or more");
  EwArgs g;
  memset(&g, 0, sizeof g);
  g.n_inputs = p->n_inputs;
  g.n_ops = p->n_ops;
  g.n = p->n;
  g.cols = p->cols;
  ew_div_setup(g.cols, &g.cols_mul, &g.cols_shr);
  bool vec = (p->n % 4) == 0 && (p->cols % 4) == 0;
  int rc;
  for (int k = 0; k < p->n_inputs; ++k) {
    uint64_t need;
    const int mode = p->input_mode[k];
    if (mode == TFJS_CUDA_EW_FULL) need = p->n;
    else if (mode == TFJS_CUDA_EW_PERIODIC) {
      need = p->input_period[k];
      if (need == 0 || p->n % need != 0)
        return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                        "fused_elementwise: period %u of input %d does not divide the output",
                        p->input_period[k], k);
      if (need % 4 != 0) vec = false;
    } else if (mode == TFJS_CUDA_EW_ROW) {
      if (p->n % p->cols != 0)
        return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_elementwise: cols does not divide n");
      need = p->n / p->cols;
    } else if (mode == TFJS_CUDA_EW_SCALAR) need = 1;
    else if (mode == TFJS_CUDA_EW_BATCHED) {
      const uint64_t per = p->input_period[k], aux = p->input_aux[k];
      if (per == 0 || aux == 0 || aux % per != 0 || p->n % aux != 0)
        return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                        "fused_elementwise: batched input %d has period %u, aux %u", k,
                        p->input_period[k], p->input_aux[k]);
      need = p->n / aux * per;
      if (per % 4 != 0) vec = false;
    }
    else return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_elementwise: input mode %d", mode);
    Buffer* b;
    if ((rc = ctx_get(ctx, p->input_id[k], need * 4, "fused_elementwise input", &b))) return rc;
    g.in[k] = (const float*)b->ptr;
    g.mode[k] = mode;
    g.period[k] = p->input_period[k];
    g.aux[k] = p->input_aux[k];
    ew_div_setup(g.period[k], &g.period_mul[k], &g.period_shr[k]);
    ew_div_setup(g.aux[k], &g.aux_mul[k], &g.aux_shr[k]);
    if (!aligned16(b->ptr)) vec = false;
  }
  for (int j = 0; j < p->n_ops; ++j) {
    const tfjs_cuda_ew_op& op = p->ops[j];
    const int limit = p->n_inputs + j;  // an op reads inputs and earlier results only
    const bool unary = op.opcode >= TFJS_CUDA_EW_UNARY;
    const int code = unary ? op.opcode - TFJS_CUDA_EW_UNARY : op.opcode;
    const bool known = unary ? (code >= TFJS_CUDA_RELU && code <= TFJS_CUDA_LOG &&
                                code != TFJS_CUDA_LEAKYRELU && code != TFJS_CUDA_CLIP)
                             : (code >= TFJS_CUDA_ADD && code <= TFJS_CUDA_SQUARED_DIFFERENCE &&
                                code != TFJS_CUDA_POW);
    if (!known || op.a >= limit || (!unary && op.b >= limit))
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_elementwise: op %d is malformed", j);
    g.ops[j] = op;
    if (unary) {
      g.ops[j].b = op.a;
      if (ctx->math_mode == TFJS_CUDA_MATH_TF32)
        g.ops[j].opcode = (int16_t)(TFJS_CUDA_EW_UNARY + fast_unary_op(code));
    }
  }
  Buffer* o;
  if ((rc = ctx_get(ctx, out_id, p->n * 4, "fused_elementwise out", &o))) return rc;
  if (p->n == 0) return TFJS_CUDA_OK;
  g.out = (float*)o->ptr;
  if (!aligned16(o->ptr)) vec = false;
  cudaSetDevice(ctx->device);
  if (!ew_launch_catalogued(ctx, g, vec)) {
    // not in the catalogue: the interpreter (slower than the separate kernels for short
    // chains; the host layer asks tfjs_cuda_fused_elementwise_catalogued first)
    if (vec)
      fused_elementwise_kernel<4><<<grid_for(p->n / 4, kThreads, ctx->sm_count), kThreads, 0,
                                    ctx->stream>>>(g);
    else
      fused_elementwise_kernel<1><<<grid_for(p->n, kThreads, ctx->sm_count), kThreads, 0,
                                    ctx->stream>>>(g);
  }
  LAUNCH_CHECK(ctx, "fused_elementwise_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_fused_elementwise_catalogued(tfjs_cuda_ctx* ctx, const tfjs_cuda_ew_program* p,
                                           int32_t* out_yes) {
  if (!ctx || !p || !out_yes) return TFJS_CUDA_INVALID_ARG;
  *out_yes = 0;
  if (p->n_inputs < 1 || p->n_inputs > TFJS_CUDA_EW_MAX_INPUTS || p->n_ops < 1 ||
      p->n_ops > TFJS_CUDA_EW_MAX_OPS)
    return TFJS_CUDA_OK;
  EwArgs g;
  memset(&g, 0, sizeof g);
  g.n_inputs = p->n_inputs;
  g.n_ops = p->n_ops;
  for (int j = 0; j < p->n_ops; ++j) {
    g.ops[j] = p->ops[j];
    if (g.ops[j].opcode >= TFJS_CUDA_EW_UNARY) {
      g.ops[j].b = g.ops[j].a;
      // every catalogued chain with a transcendental op exists in both forms, so the answer
      // does not depend on the math mode in force
      if (ctx->math_mode == TFJS_CUDA_MATH_TF32 &&
          g.ops[j].opcode <= TFJS_CUDA_EW_UNARY + TFJS_CUDA_LOG)
        g.ops[j].opcode = (int16_t)(TFJS_CUDA_EW_UNARY +
                                    fast_unary_op(g.ops[j].opcode - TFJS_CUDA_EW_UNARY));
    }
  }
  *out_yes = ew_launch_catalogued(ctx, g, true, true) ? 1 : 0;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_add_activation(tfjs_cuda_ctx* ctx, int32_t activation, int32_t a_id,
                             int32_t b_id, uint64_t n, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (activation != TFJS_CUDA_ACT_LINEAR && activation != TFJS_CUDA_ACT_RELU &&
      activation != TFJS_CUDA_ACT_RELU6)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "add_activation: activation %d", activation);
  Buffer *a, *b, *o;
  int rc;
  if ((rc = ctx_get(ctx, a_id, n * 4, "add_activation a", &a))) return rc;
  if ((rc = ctx_get(ctx, b_id, n * 4, "add_activation b", &b))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "add_activation out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for((n + 3) / 4, kThreads, ctx->sm_count);
  const float* ap = (const float*)a->ptr;
  const float* bp = (const float*)b->ptr;
  float* op = (float*)o->ptr;
  if (activation == TFJS_CUDA_ACT_RELU)
    add_act_kernel<TFJS_CUDA_ACT_RELU><<<grid, kThreads, 0, ctx->stream>>>(ap, bp, op, n);
  else if (activation == TFJS_CUDA_ACT_RELU6)
    add_act_kernel<TFJS_CUDA_ACT_RELU6><<<grid, kThreads, 0, ctx->stream>>>(ap, bp, op, n);
  else
    add_act_kernel<TFJS_CUDA_ACT_LINEAR><<<grid, kThreads, 0, ctx->stream>>>(ap, bp, op, n);
  LAUNCH_CHECK(ctx, "add_act_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_batchnorm(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t n,
                        int32_t mean_id, uint64_t n_mean, int32_t var_id,
                        uint64_t n_var, int32_t scale_id, uint64_t n_scale,
                        int32_t offset_id, uint64_t n_offset, double epsilon,
                        int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *x, *m, *v, *s = nullptr, *o = nullptr, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, n * 4, "batchnorm x", &x))) return rc;
  if ((rc = ctx_get(ctx, mean_id, n_mean * 4, "batchnorm mean", &m))) return rc;
  if ((rc = ctx_get(ctx, var_id, n_var * 4, "batchnorm variance", &v))) return rc;
  if (scale_id && (rc = ctx_get(ctx, scale_id, n_scale * 4, "batchnorm scale", &s))) return rc;
  if (offset_id && (rc = ctx_get(ctx, offset_id, n_offset * 4, "batchnorm offset", &o))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "batchnorm out", &y))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  if (n_mean == 0 || n_var == 0 || (s && n_scale == 0) || (o && n_offset == 0))
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "batchnorm: empty parameter");
  cudaSetDevice(ctx->device);
  batchnorm_kernel<<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      (const float*)x->ptr, n, (const float*)m->ptr, n_mean, (const float*)v->ptr,
      n_var, s ? (const float*)s->ptr : nullptr, n_scale ? n_scale : 1,
      o ? (const float*)o->ptr : nullptr, n_offset ? n_offset : 1, epsilon,
      (float*)y->ptr);
  LAUNCH_CHECK(ctx, "batchnorm_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_batchnorm_rows(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows, uint64_t cols,
                             int32_t mean_id, int32_t mean_mode, int32_t var_id,
                             int32_t var_mode, int32_t scale_id, int32_t scale_mode,
                             int32_t offset_id, int32_t offset_mode, double epsilon,
                             int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (rows > 0xffffffffull || cols > 0xffffffffull)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "batchnorm_rows: view too large");
  const uint64_t n = rows * cols;
  Buffer *x, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, n * 4, "batchnorm_rows x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "batchnorm_rows out", &y))) return rc;
  const int32_t ids[4] = {mean_id, var_id, scale_id, offset_id};
  const int32_t modes[4] = {mean_mode, var_mode, scale_mode, offset_mode};
  BnParam q[4];
  for (int k = 0; k < 4; ++k) {
    q[k].p = nullptr;
    q[k].mode = modes[k];
    if (modes[k] < 0 || modes[k] > 4 || (k < 2 && modes[k] == 0))
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "batchnorm_rows: parameter %d has mode %d", k,
                      modes[k]);
    if (modes[k] == 0) continue;
    const uint64_t need = modes[k] == 1 ? cols : modes[k] == 2 ? rows : modes[k] == 3 ? n : 1;
    Buffer* b;
    if ((rc = ctx_get(ctx, ids[k], need * 4, "batchnorm_rows parameter", &b))) return rc;
    q[k].p = (const float*)b->ptr;
  }
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  batchnorm_rows_kernel<<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      (const float*)x->ptr, (uint32_t)rows, (uint32_t)cols, q[0], q[1], q[2], q[3], epsilon,
      (float*)y->ptr);
  LAUNCH_CHECK(ctx, "batchnorm_rows_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

static uint64_t dtype_bytes(int dt) { return dt == TFJS_CUDA_BOOL ? 1 : 4; }

int tfjs_cuda_cast(tfjs_cuda_ctx* ctx, int32_t from, int32_t to, int32_t x_id,
                   uint64_t n, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (from < 0 || from > 2 || to < 0 || to > 2)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "cast: unknown dtype");
  Buffer *x, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, n * dtype_bytes(from), "cast x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * dtype_bytes(to), "cast out", &y))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for(n, kThreads, ctx->sm_count);
#define CAST(TI, TO, MODE) cast_kernel<TI, TO, MODE><<<grid, kThreads, 0, ctx->stream>>>((const TI*)x->ptr, (TO*)y->ptr, n)
  const int key = from * 3 + to;
  switch (key) {
    case 0: CAST(float, float, 0); break;
    case 1: CAST(float, int32_t, 1); break;
    case 2: CAST(float, uint8_t, 2); break;
    case 3: CAST(int32_t, float, 0); break;
    case 4: CAST(int32_t, int32_t, 0); break;
    case 5: CAST(int32_t, uint8_t, 2); break;
    case 6: CAST(uint8_t, float, 0); break;
    case 7: CAST(uint8_t, int32_t, 0); break;
    default: CAST(uint8_t, uint8_t, 0); break;
  }
#undef CAST
  LAUNCH_CHECK(ctx, "cast_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_fill(tfjs_cuda_ctx* ctx, int32_t elem_bytes, uint32_t bits,
                   int32_t out_id, uint64_t n) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (elem_bytes != 1 && elem_bytes != 4)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fill: elem_bytes %d", elem_bytes);
  Buffer* y;
  int rc;
  if ((rc = ctx_get(ctx, out_id, n * elem_bytes, "fill out", &y))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (elem_bytes == 1) {
    CUDA_TRY(ctx, cudaMemsetAsync(y->ptr, (int)(bits & 0xff), n, ctx->stream));
  } else {
    fill32_kernel<<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (uint32_t*)y->ptr, bits, n);
    LAUNCH_CHECK(ctx, "fill32_kernel");
  }
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_copy_strided(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t rank,
                           const int64_t* extent, int32_t x_id, int64_t x_off,
                           const int64_t* x_strides, const int64_t* x_wrap,
                           int32_t out_id, int64_t o_off,
                           const int64_t* o_strides) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (rank < 0 || rank > kMaxRank)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "copy_strided: rank %d", rank);
  if (elem_bytes != 1 && elem_bytes != 4)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "copy_strided: elem_bytes %d", elem_bytes);
  Dims ex, xs, xw, os;
  uint64_t n = 1;
  long long x_max = x_off, o_max = o_off;
  for (int d = 0; d < kMaxRank; ++d) ex.v[d] = 1, xs.v[d] = 0, xw.v[d] = 1, os.v[d] = 0;
  for (int d = 0; d < rank; ++d) {
    if (extent[d] < 0 || x_wrap[d] <= 0 || x_strides[d] < 0 || o_strides[d] < 0)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "copy_strided: bad dims");
    ex.v[d] = extent[d]; xs.v[d] = x_strides[d]; xw.v[d] = x_wrap[d]; os.v[d] = o_strides[d];
    n *= extent[d];
    if (extent[d] > 0) {
      long long top = extent[d] - 1;
      if (top > x_wrap[d] - 1) top = x_wrap[d] - 1;
      x_max += top * x_strides[d];
      o_max += (extent[d] - 1) * o_strides[d];
    }
  }
  if (n == 0) return TFJS_CUDA_OK;
  if (x_off < 0 || o_off < 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "copy_strided: negative offset");
  Buffer *x, *o;
  int rc;
  if ((rc = ctx_get(ctx, x_id, (uint64_t)(x_max + 1) * elem_bytes, "copy_strided x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, (uint64_t)(o_max + 1) * elem_bytes, "copy_strided out", &o))) return rc;
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for(n, kThreads, ctx->sm_count);
  if (elem_bytes == 4)
    copy_strided_kernel<uint32_t><<<grid, kThreads, 0, ctx->stream>>>(
        (const uint32_t*)x->ptr, (uint32_t*)o->ptr, n, rank, ex, x_off, xs, xw, o_off, os);
  else
    copy_strided_kernel<uint8_t><<<grid, kThreads, 0, ctx->stream>>>(
        (const uint8_t*)x->ptr, (uint8_t*)o->ptr, n, rank, ex, x_off, xs, xw, o_off, os);
  LAUNCH_CHECK(ctx, "copy_strided_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_transpose(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t rank,
                        int32_t x_id, const int64_t* x_shape,
                        const int32_t* perm, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (rank < 0 || rank > kMaxRank)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "transpose: rank %d", rank);
  if (elem_bytes != 1 && elem_bytes != 4)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "transpose: elem_bytes %d", elem_bytes);
  uint64_t n = 1;
  long long xstr[kMaxRank];
  bool seen[kMaxRank] = {false, false, false, false, false, false};
  for (int d = 0; d < rank; ++d) {
    if (perm[d] < 0 || perm[d] >= rank || seen[perm[d]])
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "transpose: bad perm");
    seen[perm[d]] = true;
    n *= x_shape[d];
  }
  long long s = 1;
  for (int d = rank - 1; d >= 0; --d) { xstr[d] = s; s *= x_shape[d]; }
  Buffer *x, *o;
  int rc;
  if ((rc = ctx_get(ctx, x_id, n * elem_bytes, "transpose x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * elem_bytes, "transpose out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  // Drop size-1 axes and merge axes that stay adjacent, then pick a kernel.
  int64_t oshape[kMaxRank];
  long long ostr_x[kMaxRank];
  int r2 = 0;
  for (int d = 0; d < rank; ++d) {
    const int src = perm[d];
    if (x_shape[src] == 1) continue;
    if (r2 > 0 && ostr_x[r2 - 1] == xstr[src] * x_shape[src]) {
      oshape[r2 - 1] *= x_shape[src];
      ostr_x[r2 - 1] = xstr[src];
    } else {
      oshape[r2] = x_shape[src];
      ostr_x[r2] = xstr[src];
      ++r2;
    }
  }
  if (r2 <= 1) {  // pure copy
    CUDA_TRY(ctx, cudaMemcpyAsync(o->ptr, x->ptr, n * elem_bytes,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
    ctx_mark_written(ctx, out_id);
    return TFJS_CUDA_OK;
  }
  Dims os, xs;
  for (int d = 0; d < kMaxRank; ++d) os.v[d] = 1, xs.v[d] = 0;
  if (elem_bytes == 4 && r2 <= 3 && ostr_x[r2 - 2] == 1 &&
      ostr_x[r2 - 1] == oshape[r2 - 2] &&
      (r2 == 2 || ostr_x[0] == oshape[1] * oshape[2]) && oshape[r2 - 1] <= 0x7fffffff &&
      oshape[r2 - 2] <= 0x7fffffff && (r2 == 2 || oshape[0] <= 65535)) {
    // [batch, rows, cols] -> [batch, cols, rows]
    const int rows = (int)oshape[r2 - 1], cols = (int)oshape[r2 - 2];
    const unsigned batch = r2 == 3 ? (unsigned)oshape[0] : 1u;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
    if (grid.y <= 65535) {
      transpose2d_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(
          (const float*)x->ptr, (float*)o->ptr, rows, cols);
      LAUNCH_CHECK(ctx, "transpose2d_kernel");
      ctx_mark_written(ctx, out_id);
      return TFJS_CUDA_OK;
    }
  }
  for (int d = 0; d < r2; ++d) { os.v[d] = oshape[d]; xs.v[d] = ostr_x[d]; }
  const bool inner_kept = ostr_x[r2 - 1] == 1;
  if (elem_bytes == 4 && inner_kept && oshape[r2 - 1] % 4 == 0) {
    bool ok = aligned16(x->ptr) && aligned16(o->ptr);
    for (int d = 0; d < r2 - 1; ++d) ok = ok && (ostr_x[d] % 4 == 0);
    if (ok) {
      os.v[r2 - 1] /= 4;
      for (int d = 0; d < r2 - 1; ++d) xs.v[d] /= 4;
      const uint64_t n4 = n / 4;
      if (n < 0x7fffffffull)
        transpose_kernel<uint4, uint32_t><<<grid_for(n4, kThreads, ctx->sm_count), kThreads, 0,
                                            ctx->stream>>>((const uint4*)x->ptr,
                                                           (uint4*)o->ptr, n4, r2, os, xs);
      else
        transpose_kernel<uint4, uint64_t><<<grid_for(n4, kThreads, ctx->sm_count), kThreads, 0,
                                            ctx->stream>>>((const uint4*)x->ptr,
                                                           (uint4*)o->ptr, n4, r2, os, xs);
      LAUNCH_CHECK(ctx, "transpose_kernel<uint4>");
      ctx_mark_written(ctx, out_id);
      return TFJS_CUDA_OK;
    }
  }
  const unsigned grid = grid_for(n, kThreads, ctx->sm_count);
  if (elem_bytes == 4 && n < 0x7fffffffull)
    transpose_kernel<uint32_t, uint32_t><<<grid, kThreads, 0, ctx->stream>>>(
        (const uint32_t*)x->ptr, (uint32_t*)o->ptr, n, r2, os, xs);
  else if (elem_bytes == 4)
    transpose_kernel<uint32_t, uint64_t><<<grid, kThreads, 0, ctx->stream>>>(
        (const uint32_t*)x->ptr, (uint32_t*)o->ptr, n, r2, os, xs);
  else
    transpose_kernel<uint8_t, uint64_t><<<grid, kThreads, 0, ctx->stream>>>(
        (const uint8_t*)x->ptr, (uint8_t*)o->ptr, n, r2, os, xs);
  LAUNCH_CHECK(ctx, "transpose_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_gather(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t x_id,
                     int32_t indices_id, uint64_t batch, uint64_t outer,
                     uint64_t dim, uint64_t slice, uint64_t n_idx,
                     int32_t out_id, int32_t check_indices,
                     int64_t* out_bad_index) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (elem_bytes != 1 && elem_bytes != 4)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "gather: elem_bytes %d", elem_bytes);
  const uint64_t n = batch * outer * n_idx * slice;
  Buffer *x, *idx, *o;
  int rc;
  if ((rc = ctx_get(ctx, x_id, batch * outer * dim * slice * elem_bytes, "gather x", &x))) return rc;
  if ((rc = ctx_get(ctx, indices_id, batch * n_idx * 4, "gather indices", &idx))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * elem_bytes, "gather out", &o))) return rc;
  if (out_bad_index) *out_bad_index = -1;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  long long* bad = nullptr;
  if (check_indices) {
    CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_bad_index, 0xff, sizeof(long long), ctx->stream));
    bad = ctx->d_bad_index;
  }
  const int32_t* ip = (const int32_t*)idx->ptr;
  if (elem_bytes == 4 && slice % 4 == 0 && aligned16(x->ptr) && aligned16(o->ptr)) {
    const uint64_t n4 = n / 4;
    gather_kernel<uint4><<<grid_for(n4, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const uint4*)x->ptr, ip, (uint4*)o->ptr, n4, outer, dim, slice / 4, n_idx, bad);
  } else if (elem_bytes == 4) {
    gather_kernel<uint32_t><<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const uint32_t*)x->ptr, ip, (uint32_t*)o->ptr, n, outer, dim, slice, n_idx, bad);
  } else {
    gather_kernel<uint8_t><<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const uint8_t*)x->ptr, ip, (uint8_t*)o->ptr, n, outer, dim, slice, n_idx, bad);
  }
  LAUNCH_CHECK(ctx, "gather_kernel");
  ctx_mark_written(ctx, out_id);
  if (check_indices && ctx->capturing) {
    // a captured step cannot stop for the answer: the kernel writes zeros for a bad index
    // (as it always does) and replays do not raise the reference's error for it
    return TFJS_CUDA_OK;
  }
  if (check_indices) {
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->h_bad_index, ctx->d_bad_index, sizeof(long long),
                                  cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    const long long g = *ctx->h_bad_index;
    if (out_bad_index) *out_bad_index = g;
    if (g != -1)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                      "GatherV2: the index value %lld is not in [0, %llu]", g,
                      (unsigned long long)(dim - 1));
  }
  return TFJS_CUDA_OK;
}

}  // extern "C"

// Pointer-level form shared with the weight loader: table built on the host in double,
// uploaded, looked up by the kernel.  Everything is queued on the context's compute stream.
int dequant_enqueue(tfjs_cuda_ctx* ctx, const void* q, int q_bytes, int to_dtype, double scale,
                    double min, uint64_t n, void* out) {
  const int entries = q_bytes == 1 ? 256 : 65536;
  std::vector<uint32_t> table(entries);
  for (int v = 0; v < entries; ++v) {
    const double d = (double)v * scale + min;
    if (to_dtype == TFJS_CUDA_FLOAT32) {
      const float f = (float)d;
      memcpy(&table[v], &f, 4);
    } else {
      double r = floor(d);  // Math.round: ties toward +infinity
      if (d - r >= 0.5) r += 1.0;
      int32_t iv = 0;
      if (isfinite(r)) {
        double m = fmod(r, 4294967296.0);
        if (m < 0) m += 4294967296.0;
        iv = (int32_t)(uint32_t)m;
      }
      memcpy(&table[v], &iv, 4);
    }
  }
  void* d_table = nullptr;
  CUDA_TRY(ctx, cudaMallocAsync(&d_table, entries * 4, ctx->stream));
  // Pageable source: the driver stages the bytes before this call returns.
  CUDA_TRY(ctx, cudaMemcpyAsync(d_table, table.data(), entries * 4,
                                cudaMemcpyHostToDevice, ctx->stream));
  if (q_bytes == 1) {
    dequant_u8_kernel<uint32_t><<<grid_for((n + 15) / 16, kThreads, ctx->sm_count),
                                  kThreads, 0, ctx->stream>>>(
        (const uint8_t*)q, (const uint32_t*)d_table, (uint32_t*)out, n);
  } else {
    dequant_u16_kernel<uint32_t><<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0,
                                   ctx->stream>>>(
        (const uint16_t*)q, (const uint32_t*)d_table, (uint32_t*)out, n);
  }
  LAUNCH_CHECK(ctx, "dequant_kernel");
  CUDA_TRY(ctx, cudaFreeAsync(d_table, ctx->stream));
  return TFJS_CUDA_OK;
}

extern "C" {

int tfjs_cuda_dequantize(tfjs_cuda_ctx* ctx, int32_t q_bytes, int32_t to_dtype,
                         int32_t q_id, double scale, double min, uint64_t n,
                         int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "dequantising weights");
  if (q_bytes != 1 && q_bytes != 2)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "dequantize: q_dtype_bytes %d", q_bytes);
  if (to_dtype != TFJS_CUDA_FLOAT32 && to_dtype != TFJS_CUDA_INT32)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "dequantize: target dtype %d", to_dtype);
  Buffer *q, *o;
  int rc;
  if ((rc = ctx_get(ctx, q_id, n * q_bytes, "dequantize q", &q))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "dequantize out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if ((rc = dequant_enqueue(ctx, q->ptr, q_bytes, to_dtype, scale, min, n, o->ptr))) return rc;
  Buffer* ob = ctx_buf(ctx, out_id);
  ob->version++;
  ob->from_host = true;  // dequantised weights are constants
  ctx_drop_packed(ctx, out_id);
  return TFJS_CUDA_OK;
}

// ---- float16-stored weights: exact widening to float32 ------------------------------
// tfjs-core/src/io/io_utils.ts:228-231 decodes 'float16' quantised weights with the
// table method of van der Zijp ("Fast Half Float Conversions"), which is the exact IEEE
// widening: subnormals are normalised, infinities stay, a NaN keeps its payload in the
// upper mantissa bits.  Done here with integer arithmetic, eight values per thread.
__device__ __forceinline__ uint32_t half_bits_to_float_bits(uint32_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 31u;
  uint32_t m = h & 0x3ffu;
  if (e == 0) {
    if (m == 0) return sign;
    const int shift = __clz(m) - 21;  // bring the leading one to bit 10
    m = (m << shift) & 0x3ffu;
    return sign | ((uint32_t)(113 - shift) << 23) | (m << 13);
  }
  if (e == 31) return sign | 0x7f800000u | (m << 13);
  return sign | ((e + 112u) << 23) | (m << 13);
}

__global__ void decode_f16_kernel(const uint16_t* __restrict__ q, uint32_t* __restrict__ o,
                                  uint64_t n) {
  const uint64_t n8 = n >> 3;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint4* q8 = reinterpret_cast<const uint4*>(q);
  uint4* o4 = reinterpret_cast<uint4*>(o);
  for (uint64_t i = tid; i < n8; i += stride) {
    const uint4 v = __ldg(q8 + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t r[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      r[2 * k] = half_bits_to_float_bits(w[k] & 0xffffu);
      r[2 * k + 1] = half_bits_to_float_bits(w[k] >> 16);
    }
    o4[2 * i] = make_uint4(r[0], r[1], r[2], r[3]);
    o4[2 * i + 1] = make_uint4(r[4], r[5], r[6], r[7]);
  }
  for (uint64_t i = (n8 << 3) + tid; i < n; i += stride) o[i] = half_bits_to_float_bits(q[i]);
}

}  // extern "C"

int decode_f16_enqueue(tfjs_cuda_ctx* ctx, const void* q, uint64_t n, void* out) {
  decode_f16_kernel<<<grid_for((n + 7) / 8, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      (const uint16_t*)q, (uint32_t*)out, n);
  LAUNCH_CHECK(ctx, "decode_f16_kernel");
  return TFJS_CUDA_OK;
}

extern "C" {

int tfjs_cuda_decode_float16(tfjs_cuda_ctx* ctx, int32_t q_id, uint64_t n, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *q, *o;
  int rc;
  if ((rc = ctx_get(ctx, q_id, n * 2, "decode_float16 q", &q))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "decode_float16 out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if ((rc = decode_f16_enqueue(ctx, q->ptr, n, o->ptr))) return rc;
  Buffer* ob = ctx_buf(ctx, out_id);
  ob->version++;
  ob->from_host = true;  // decoded weights are constants
  ctx_drop_packed(ctx, out_id);
  return TFJS_CUDA_OK;
}

// ---- dequantisation without any allocation --------------------------------------
// The lookup table lives in a fixed device array instead of a pool allocation.
// 65536 entries cover the widest quantised type (uint16); 256 KiB per GPU, held
// from library load until the process exits.
#define TFJS_CUDA_STATIC_TABLE_ENTRIES 65536
static __device__ __align__(256) uint32_t g_static_dequant_table[TFJS_CUDA_STATIC_TABLE_ENTRIES];
// In host code the name above is only a handle for the symbol, not an address a
// kernel can use; the real device address is looked up once per device.
static uint32_t* g_static_table_addr[64];
// Host staging for the table (no heap use on the call path).  One array for the whole
// process, so host threads that dequantise at the same time (on the same GPU or on
// different ones) take turns filling it: the lock is held from the fill until the copy
// out of it has been staged by the driver, which is before cudaMemcpyAsync returns for a
// pageable source.
static uint32_t g_static_table_host[TFJS_CUDA_STATIC_TABLE_ENTRIES];
static std::mutex g_static_table_lock;

int tfjs_cuda_dequantize_static(tfjs_cuda_ctx* ctx, int32_t q_bytes, int32_t to_dtype,
                                int32_t q_id, double scale, double min, uint64_t n,
                                int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "dequantising weights");
  if (q_bytes < 1)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "dequantize_static: q_dtype_bytes %d", q_bytes);
  if (q_bytes > 2)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "dequantize_static: a %d-byte quantised type needs a lookup table larger "
                    "than the fixed %d-entry table; the widest supported type is uint16",
                    q_bytes, TFJS_CUDA_STATIC_TABLE_ENTRIES);
  if (to_dtype != TFJS_CUDA_FLOAT32 && to_dtype != TFJS_CUDA_INT32)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "dequantize_static: target dtype %d", to_dtype);
  if (ctx->device < 0 || ctx->device >= 64)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "dequantize_static: device ordinal %d",
                    ctx->device);
  Buffer *q, *o;
  int rc;
  if ((rc = ctx_get(ctx, q_id, n * q_bytes, "dequantize_static q", &q))) return rc;
  if ((rc = ctx_get(ctx, out_id, n * 4, "dequantize_static out", &o))) return rc;
  if (n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  std::lock_guard<std::mutex> hold(g_static_table_lock);
  uint32_t* table = g_static_table_addr[ctx->device];
  if (!table) {
    // First call on this device: resolve the symbol with this device current.
    void* addr = nullptr;
    CUDA_TRY(ctx, cudaGetSymbolAddress(&addr, g_static_dequant_table));
    table = g_static_table_addr[ctx->device] = (uint32_t*)addr;
  }
  const int entries = q_bytes == 1 ? 256 : 65536;
  for (int v = 0; v < entries; ++v) {
    const double d = (double)v * scale + min;
    if (to_dtype == TFJS_CUDA_FLOAT32) {
      const float f = (float)d;
      memcpy(&g_static_table_host[v], &f, 4);
    } else {
      double r = floor(d);  // Math.round: ties toward +infinity
      if (d - r >= 0.5) r += 1.0;
      int32_t iv = 0;
      if (isfinite(r)) {
        double m = fmod(r, 4294967296.0);
        if (m < 0) m += 4294967296.0;
        iv = (int32_t)(uint32_t)m;
      }
      memcpy(&g_static_table_host[v], &iv, 4);
    }
  }
  // Every entry a kernel can index is rewritten here, so nothing left over from
  // an earlier call is ever read.  Pageable source: staged before the call returns.
  CUDA_TRY(ctx, cudaMemcpyAsync(table, g_static_table_host, (size_t)entries * 4,
                                cudaMemcpyHostToDevice, ctx->stream));
  if (q_bytes == 1) {
    dequant_u8_kernel<uint32_t><<<grid_for((n + 15) / 16, kThreads, ctx->sm_count),
                                  kThreads, 0, ctx->stream>>>(
        (const uint8_t*)q->ptr, (const uint32_t*)table, (uint32_t*)o->ptr, n);
  } else {
    dequant_u16_kernel<uint32_t><<<grid_for(n, kThreads, ctx->sm_count), kThreads, 0,
                                   ctx->stream>>>(
        (const uint16_t*)q->ptr, (const uint32_t*)table, (uint32_t*)o->ptr, n);
  }
  LAUNCH_CHECK(ctx, "dequant_kernel (static table)");
  o->version++;           // any packed copy of the old contents is now stale
  o->from_host = true;    // dequantised weights are constants
  ctx_packed_contents_changed(ctx, out_id);  // so are captured steps that read that copy
  return TFJS_CUDA_OK;
}

int tfjs_cuda_flush_l2(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "flushing L2");
  cudaSetDevice(ctx->device);
  const uint64_t bytes = 256ull << 20;
  if (!ctx->l2_scratch) {
    CUDA_TRY(ctx, cudaMallocAsync(&ctx->l2_scratch, bytes, ctx->stream));
    ctx->l2_scratch_bytes = bytes;
  }
  fill32_kernel<<<grid_for(bytes / 4, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
      (uint32_t*)ctx->l2_scratch, 0u, bytes / 4);
  ctx->launches--;  // hygiene helper, not part of the measured path
  LAUNCH_CHECK(ctx, "flush_l2");
  return TFJS_CUDA_OK;
}

}  // extern "C"
