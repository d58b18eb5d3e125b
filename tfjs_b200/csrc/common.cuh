// Internal declarations shared by the translation units of libtfjs_cuda.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "tfjs_cuda.h"

struct Buffer {
  void* ptr = nullptr;
  uint64_t bytes = 0;
  bool live = false;
  bool from_host = false;  // last filled by write()/dequantize(): weight-like
  uint32_t version = 0;    // bumped whenever the contents are (re)written
  cudaEvent_t ready = nullptr;  // set while an upload on the copy stream is pending
  bool uploaded = false;        // block came from tfjs_cuda_upload: recycled for uploads
  bool in_arena = false;        // lives in the arena of a captured graph
};

// A captured step (tfjs_cuda_capture_begin .. _end): the instantiated graph and the
// arena its intermediate and output tensors live in.
struct ReplayGraph {
  cudaGraphExec_t exec = nullptr;
  void* arena = nullptr;
  uint64_t arena_bytes = 0;
  uint64_t launches = 0;  // kernels per replay
  // Memory outside the arena whose address the recorded kernels carry: the packed copies
  // of these weight ids and, if uses_scratch, the context's scratch buffer.  When one of
  // them is freed or re-allocated the graph is stale and graph_launch refuses it.
  std::vector<int32_t> packed_ids;
  bool uses_scratch = false;
  bool stale = false;
};
struct ArenaSpan {
  uint64_t off, size;
};

// A block released by an uploaded tensor, kept for the next upload of that size: the
// copy stream waits for `released` (the compute stream's position when the tensor was
// freed) instead of the compute stream's tail.
struct UploadBlock {
  void* ptr;
  uint64_t bytes;
  cudaEvent_t released;
};

// A filter repacked for the tensor-core kernels: [rows = out channels][k_pad]
// with K contiguous, values rounded to TF32 (round-to-nearest).
struct PackedWeight {
  float* ptr = nullptr;
  uint64_t bytes = 0;
  uint32_t version = 0;
  int rows = 0, k_pad = 0;
  int layout = 0;
};

struct tfjs_cuda_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaStream_t copy_stream = nullptr;       // uploads that overlap compute
  cudaStream_t read_stream = nullptr;       // large downloads that overlap the next kernels
  std::vector<cudaEvent_t> event_pool;      // recycled upload-completion events
  // Exact-size cache of freed blocks.  A graph model asks for the same sizes every
  // step; handing a freed block straight to the next request of that size keeps the
  // driver's allocator (and its occasional re-mapping of large blocks) off the step.
  // Safe without fences because every cached block is reused on the same in-order
  // compute stream that last touched it.
  std::unordered_map<uint64_t, std::vector<void*>> block_cache;
  uint64_t cached_bytes = 0;
  std::vector<UploadBlock> upload_cache;  // oldest first
  // stream capture of a whole step
  bool capturing = false;
  bool capture_failed = false;
  void* arena = nullptr;
  uint64_t arena_bytes = 0;
  std::vector<ArenaSpan> arena_free;  // sorted by offset, coalesced
  uint64_t capture_launches0 = 0;
  std::vector<int32_t> capture_packed;  // weight ids whose packed copy the capture reads
  bool capture_scratch = false;         // the capture reads or writes ctx->scratch
  std::vector<ReplayGraph> graphs;    // index + 1 = graph id
  cudaMemPool_t pool = nullptr;
  std::vector<Buffer> bufs;  // index = id; slot 0 unused
  std::vector<int32_t> free_ids;
  std::unordered_map<int32_t, PackedWeight> packed;
  std::string err;
  uint64_t in_use = 0, high_water = 0, n_live = 0;
  uint64_t launches = 0;
  // names of the kernel instantiations launched while tfjs_cuda_launch_log is on (string
  // literals or statics: the pointers stay valid)
  bool log_launches = false;
  std::vector<const char*> launch_log;
  int math_mode = TFJS_CUDA_MATH_TF32;
  int* d_flag = nullptr;  // device error word written by bounded waits
  int* h_flag = nullptr;  // pinned mirror
  long long* d_bad_index = nullptr;
  long long* h_bad_index = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::vector<cudaEvent_t> prof_events;  // numbered events for per-kernel timing
  std::vector<cudaEvent_t> read_events;  // tickets of tfjs_cuda_read_begin (index + 1)
  std::vector<cudaEvent_t> read_order;   // per ticket: orders the read stream behind the compute stream
  std::vector<int*> read_flags;          // one pinned copy of the device error word per ticket
  std::vector<int> read_free;            // ticket slots free for reuse
  void* l2_scratch = nullptr;
  uint64_t l2_scratch_bytes = 0;
  // workspace of the GEMM's K-split tail: partial accumulator tiles and their flags
  void* sk_ws = nullptr;
  unsigned* sk_flags = nullptr;
  // grow-only scratch for im2col / operand transposes
  void* scratch = nullptr;
  uint64_t scratch_bytes = 0;
};

int ctx_fail(tfjs_cuda_ctx* ctx, int code, const char* fmt, ...);
int ctx_check(tfjs_cuda_ctx* ctx, cudaError_t e, const char* what);
Buffer* ctx_buf(tfjs_cuda_ctx* ctx, int32_t id);
// Returns the buffer of `id` after checking it holds at least `need` bytes.
int ctx_get(tfjs_cuda_ctx* ctx, int32_t id, uint64_t need, const char* name,
            Buffer** out);
int ctx_scratch(tfjs_cuda_ctx* ctx, uint64_t bytes, void** out);
void ctx_mark_written(tfjs_cuda_ctx* ctx, int32_t id);
void ctx_drop_packed(tfjs_cuda_ctx* ctx, int32_t id);
// Marks captured steps that read the packed copy of weight `id` as stale (no memory call).
void ctx_packed_contents_changed(tfjs_cuda_ctx* ctx, int32_t id);

// Weight decoding on raw device pointers, queued on the compute stream (eltwise.cu); the
// tensor-id entry points and the weight loader share them.
int dequant_enqueue(tfjs_cuda_ctx* ctx, const void* q, int q_bytes, int to_dtype, double scale,
                    double min, uint64_t n, void* out);
int decode_f16_enqueue(tfjs_cuda_ctx* ctx, const void* q, uint64_t n, void* out);
// Drops the weight loaders of a context that is being destroyed (loader.cu).
void loaders_drop(tfjs_cuda_ctx* ctx);

#define CUDA_TRY(ctx, expr)                                   \
  do {                                                        \
    int _rc = ctx_check((ctx), (expr), #expr);                \
    if (_rc != TFJS_CUDA_OK) return _rc;                      \
  } while (0)

// Entry points that cannot be part of a captured step (host transfers, waits, new
// pool allocations) refuse and mark the capture as failed; the host layer then runs
// that model eagerly.
#define NOT_WHILE_CAPTURING(ctx, what)                                                    \
  do {                                                                                    \
    if ((ctx)->capturing) {                                                               \
      (ctx)->capture_failed = true;                                                       \
      return ctx_fail((ctx), TFJS_CUDA_UNSUPPORTED,                                       \
                      what " cannot be part of a captured step");                         \
    }                                                                                     \
  } while (0)

#define LAUNCH_CHECK(ctx, name)                               \
  do {                                                        \
    (ctx)->launches++;                                        \
    if ((ctx)->log_launches) (ctx)->launch_log.push_back(name); \
    int _rc = ctx_check((ctx), cudaGetLastError(), name);     \
    if (_rc != TFJS_CUDA_OK) return _rc;                      \
  } while (0)

static inline unsigned grid_for(uint64_t work_items, int threads, int sm_count,
                                int waves = 8) {
  uint64_t blocks = (work_items + threads - 1) / threads;
  uint64_t cap = (uint64_t)sm_count * waves;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return (unsigned)blocks;
}

// ---- device helpers -------------------------------------------------------
// Activations with JavaScript semantics (tfjs-backend-cpu/src/kernels/Relu.ts,
// Relu6.ts, Elu.ts, Sigmoid.ts, LeakyRelu.ts, Prelu.ts): Math.max/Math.min
// propagate NaN, which fmaxf/fminf do not, so comparisons are written so that
// NaN falls through unchanged.  elu and sigmoid go through double exp so the
// fp32 result matches a double evaluation rounded once.
struct ActParams {
  int act;
  int prelu_len;        // 0, 1, or channel count
  const float* prelu;   // device pointer or null
  double alpha;         // leakyrelu
  float gelu_scale, gelu_half, gelu_one;  // TFJS_CUDA_ACT_GELU_ERF
  int gelu_divide;
};

// exp(x) in double for results that are rounded to fp32 afterwards.  The library's exp
// costs about twice the instructions for its last few bits; this one is good to ~2^-47
// relative (Cody-Waite reduction by ln 2, Taylor series to r^11 on |r| <= ln 2 / 2), which
// changes the fp32 rounding of about one result in 2^22.  Arguments beyond +-700 (and
// NaN) take the library path.
__device__ __forceinline__ double exp_fast(double x) {
  if (!(fabs(x) <= 700.0)) return exp(x);
  const double kMagic = 6755399441055744.0;  // 1.5 * 2^52: adding it rounds to an integer
  const double t = fma(x, 1.4426950408889634074, kMagic);
  const int n = __double2loint(t);
  const double nd = t - kMagic;
  double r = fma(nd, -6.93147180369123816490e-01, x);
  r = fma(nd, -1.90821492927058770002e-10, r);
  double p = 2.50521083854417187751e-08;          // 1/11!
  p = fma(p, r, 2.75573192239858906526e-07);      // 1/10!
  p = fma(p, r, 2.75573192239858906526e-06);      // 1/9!
  p = fma(p, r, 2.48015873015873015873e-05);      // 1/8!
  p = fma(p, r, 1.98412698412698412698e-04);      // 1/7!
  p = fma(p, r, 1.38888888888888888889e-03);      // 1/6!
  p = fma(p, r, 8.33333333333333333333e-03);      // 1/5!
  p = fma(p, r, 4.16666666666666666667e-02);      // 1/4!
  p = fma(p, r, 1.66666666666666666667e-01);      // 1/3!
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  // p in [0.70, 1.42], |n| <= 1010: scaling by 2^n is an add to the exponent field
  return __hiloint2double(__double2hiint(p) + (n << 20), __double2loint(p));
}

// erf as the reference evaluates it (tfjs-core/src/ops/erf_util.ts:18-23,
// tfjs-backend-cpu/src/kernels/Erf.ts:31-39): Abramowitz-Stegun 7.1.26 in double, rounded
// to fp32 once.  js_erf_exact is that sequence operation by operation.  1 - poly(t) * t *
// exp(-v^2) cancels for small v, so the short form (approximate reciprocal with one Newton
// step, exp_fast; relative error ~2^-45) serves 2^-13 <= |x| <= 26, where it leaves the
// fp32 result within one part in 2^30 of the exact sequence; it has no branches, and
// reports arguments outside that range (zero, NaN and infinity among them) through `slow`
// for the caller to redo.
__device__ __forceinline__ float js_erf_exact(float x) {
  const double p = 0.3275911, a1 = 0.254829592, a2 = -0.284496736,
               a3 = 1.421413741, a4 = -1.453152027, a5 = 1.061405429;
  const double xd = (double)x;
  const double v = fabs(xd);
  const double sign = xd > 0.0 ? 1.0 : (xd < 0.0 ? -1.0 : xd);
  // every product and sum rounded on its own, as JavaScript does (no contraction to
  // FMA): near zero the result is the 1e-9 left over by the cancellation
  const double t = 1.0 / __dadd_rn(1.0, __dmul_rn(p, v));
  double q = __dadd_rn(__dmul_rn(a5, t), a4);
  q = __dadd_rn(__dmul_rn(q, t), a3);
  q = __dadd_rn(__dmul_rn(q, t), a2);
  q = __dadd_rn(__dmul_rn(q, t), a1);
  q = __dmul_rn(__dmul_rn(q, t), exp(-__dmul_rn(v, v)));
  return (float)__dmul_rn(sign, __dadd_rn(1.0, -q));
}
__device__ __forceinline__ float js_erf_short(float x, bool& slow) {
  const double p = 0.3275911, a1 = 0.254829592, a2 = -0.284496736,
               a3 = 1.421413741, a4 = -1.453152027, a5 = 1.061405429;
  const float ax = fabsf(x);
  slow |= !(ax >= 0x1p-13f && ax <= 26.0f);
  const double v = (double)fminf(ax, 26.0f);  // keeps -v^2 inside exp_fast's short range
  const double d = fma(p, v, 1.0);
  double t;
  asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(t) : "d"(d));  // good to ~2^-23
  t = fma(fma(-d, t, 1.0), t, t);
  double q = fma(a5, t, a4);
  q = fma(q, t, a3);
  q = fma(q, t, a2);
  q = fma(q, t, a1);
  q *= t;
  return copysignf((float)fma(-q, exp_fast(-v * v), 1.0), x);
}
// V values at once: the short form for all, the exact one again if any asked for it.
template <int V>
__device__ __forceinline__ void js_erf_vec(const float* a, float* r) {
  bool slow = false;
#pragma unroll
  for (int t = 0; t < V; ++t) r[t] = js_erf_short(a[t], slow);
  if (slow) {
#pragma unroll  // (a rolled loop would index a[] and r[] and push them out of registers)
    for (int t = 0; t < V; ++t) r[t] = js_erf_exact(a[t]);
  }
}
__device__ __forceinline__ float js_erf(float x) {
  float r;
  js_erf_vec<1>(&x, &r);
  return r;
}

// ---- fp32 forms of the transcendental kernels (default math mode) -------------------
// The reference evaluates exp / erf / tanh in JavaScript doubles and stores fp32; the
// sequences above reproduce that to the last bit or so, at the price of the double-precision
// pipe.  The contract for floating-point kernels is a tolerance (2e-3 * max|ref| per layer
// with TF32 tensor-core inputs), so in the TF32 math mode these kernels evaluate in fp32:
// the CUDA library's expf / tanhf / expm1f (at most 2 ulp) and the reference's own erf
// polynomial (tfjs-core/src/ops/erf_util.ts:18-23) with fp32 coefficients, its reciprocal
// and exponential on the special-function unit (rcp.approx, ex2.approx: a branch-free
// sequence of about 17 instructions that a GEMM epilogue can afford), whose result is
// within 8e-7 absolute of the double evaluation.  TFJS_CUDA_MATH_FP32 keeps the double
// sequences.  The op numbers below are internal (the launchers substitute them for the
// public ones); every kernel that evaluates such an op, alone or inside a chain, calls the
// same device function, so fused and separate launches still agree bit for bit.
enum {
  TFJS_CUDA_EXP_F32 = 15,
  TFJS_CUDA_ERF_F32 = 16,
  TFJS_CUDA_SIGMOID_F32 = 17,
  TFJS_CUDA_TANH_F32 = 18,
  TFJS_CUDA_ELU_F32 = 19,
  TFJS_CUDA_UNARY_OPS_END = 20
};
static inline int fast_unary_op(int op) {
  switch (op) {
    case TFJS_CUDA_EXP: return TFJS_CUDA_EXP_F32;
    case TFJS_CUDA_ERF: return TFJS_CUDA_ERF_F32;
    case TFJS_CUDA_SIGMOID: return TFJS_CUDA_SIGMOID_F32;
    case TFJS_CUDA_TANH: return TFJS_CUDA_TANH_F32;
    case TFJS_CUDA_ELU: return TFJS_CUDA_ELU_F32;
    default: return op;
  }
}
__device__ __forceinline__ float exp2_approx(float a) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}
__device__ __forceinline__ float rcp_approx(float a) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}
__device__ __forceinline__ float erf_f32(float x) {
  const float ax = fabsf(x);
  const float t = rcp_approx(__fmaf_rn(0.3275911f, ax, 1.0f));   // argument in [1, inf]
  float q = __fmaf_rn(1.061405429f, t, -1.453152027f);
  q = __fmaf_rn(q, t, 1.421413741f);
  q = __fmaf_rn(q, t, -0.284496736f);
  q = __fmaf_rn(q, t, 0.254829592f);
  q = __fmul_rn(q, t);
  // exp(-x^2) = 2^(-x^2 * log2(e)); beyond |x| = 4 the term is below fp32 resolution of 1
  const float e = exp2_approx(__fmul_rn(__fmul_rn(ax, ax), -1.4426950408889634f));
  const float r = __fmaf_rn(-q, e, 1.0f);
  return x == 0.0f ? x : copysignf(r, x);   // sign(0) * anything = 0 in the reference
}
// Two fp32 values in one 64-bit register for the packed arithmetic of sm_100
// (fma / mul / add .rn.f32x2: the same IEEE operation on each half, one instruction).
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a,
                                                        unsigned long long b,
                                                        unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a,
                                                        unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a,
                                                        unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// erf_f32 of two values: the same operations with the same roundings, the multiplications
// and fused multiply-adds two at a time.  The polynomial runs with negated coefficients
// (exactly -q), which saves negating q for the last step.
__device__ __forceinline__ unsigned long long erf_f32x2(unsigned long long x) {
  float x0, x1;
  unpack_f32x2(x, x0, x1);
  const unsigned long long ax = pack_f32x2(fabsf(x0), fabsf(x1));
#define TFJS_K2(c) pack_f32x2(c, c)
  float d0, d1;
  unpack_f32x2(fma_f32x2(TFJS_K2(0.3275911f), ax, TFJS_K2(1.0f)), d0, d1);
  const unsigned long long t = pack_f32x2(rcp_approx(d0), rcp_approx(d1));
  unsigned long long q = fma_f32x2(TFJS_K2(-1.061405429f), t, TFJS_K2(1.453152027f));
  q = fma_f32x2(q, t, TFJS_K2(-1.421413741f));
  q = fma_f32x2(q, t, TFJS_K2(0.284496736f));
  q = fma_f32x2(q, t, TFJS_K2(-0.254829592f));
  q = mul_f32x2(q, t);
  float g0, g1;
  unpack_f32x2(mul_f32x2(mul_f32x2(ax, ax), TFJS_K2(-1.4426950408889634f)), g0, g1);
  const unsigned long long e = pack_f32x2(exp2_approx(g0), exp2_approx(g1));
  float r0, r1;
  unpack_f32x2(fma_f32x2(q, e, TFJS_K2(1.0f)), r0, r1);
#undef TFJS_K2
  return pack_f32x2(x0 == 0.0f ? x0 : copysignf(r0, x0), x1 == 0.0f ? x1 : copysignf(r1, x1));
}
__device__ __forceinline__ float sigmoid_f32(float x) {
  return __frcp_rn(__fadd_rn(1.0f, expf(-x)));
}
__device__ __forceinline__ float elu_f32(float x) { return x >= 0.0f ? x : expm1f(x); }

__device__ __forceinline__ float js_relu(float v) {
  return v > 0.0f ? v : (v != v ? v : 0.0f);
}
__device__ __forceinline__ float js_relu6(float v) {
  if (v != v) return v;
  return v > 6.0f ? 6.0f : (v > 0.0f ? v : 0.0f);
}
__device__ __forceinline__ float js_elu(float v) {
  return v >= 0.0f ? v : (float)(exp((double)v) - 1.0);
}
__device__ __forceinline__ float js_sigmoid(float v) {
  return (float)(1.0 / (1.0 + exp_fast(-(double)v)));
}
__device__ __forceinline__ float js_leakyrelu(float v, double alpha) {
  return v < 0.0f ? (float)(alpha * (double)v) : v;
}

// (h * half) * (erf(h * scale) + one) with every step rounded to fp32: the five
// elementwise kernels a converted graph runs after a dense layer for the erf GELU.
__device__ __forceinline__ float js_gelu_erf(float h, const ActParams& ap) {
  const float a = ap.gelu_divide ? __fdiv_rn(h, ap.gelu_scale) : __fmul_rn(h, ap.gelu_scale);
  return __fmul_rn(__fmul_rn(h, ap.gelu_half), __fadd_rn(js_erf(a), ap.gelu_one));
}

__device__ __forceinline__ float apply_act(float v, const ActParams& ap,
                                           int channel) {
  switch (ap.act) {
    case TFJS_CUDA_ACT_RELU: return js_relu(v);
    case TFJS_CUDA_ACT_RELU6: return js_relu6(v);
    case TFJS_CUDA_ACT_PRELU: {
      const float a = ap.prelu[ap.prelu_len == 1 ? 0 : channel];
      return v < 0.0f ? a * v : v;
    }
    case TFJS_CUDA_ACT_LEAKYRELU: return js_leakyrelu(v, ap.alpha);
    case TFJS_CUDA_ACT_SIGMOID: return js_sigmoid(v);
    case TFJS_CUDA_ACT_ELU: return js_elu(v);
    case TFJS_CUDA_ACT_GELU_ERF: return js_gelu_erf(v, ap);
    default: return v;
  }
}

