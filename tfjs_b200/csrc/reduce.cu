// Softmax, Sum/Mean/Max and ArgMax.  Bandwidth-bound SIMT kernels: each row is
// read once (softmax keeps it in registers), reductions use warp shuffles.
//
// Accumulation is in double, as in the reference where the running sum is a JS
// number (tfjs-backend-cpu/src/kernels/Sum.ts:67-74); with a double accumulator
// the order of additions only matters far below fp32 resolution.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Max with the reference's NaN rule (Max_impl.ts:26-36): NaN is sticky.
__device__ __forceinline__ float nan_max(float a, float b) {
  if (a != a) return a;
  if (b != b) return b;
  return a > b ? a : b;
}

__device__ __forceinline__ float warp_nan_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- softmax: tfjs-backend-cpu/src/kernels/Softmax.ts:50-67 -----------------
// max -> a = fl32(x - max) -> e = fl32(exp(a)) -> s = fl32(sum_double(e)) ->
// out = fl32(e / s).  One warp per row.
// REGS values per lane stay in registers (rows up to 32*REGS wide); REGS == 0 is
// the wide-row variant that re-reads its own output instead.
// Optional prologue (the scaled, masked scores of an attention layer): logit =
// fl32(fl32(x * scale) + mask[row / rows_per_mask][col]), the Multiply.ts and Add.ts
// kernels in front of the softmax, formed on the way in.
struct SoftmaxPrologue {
  int has_scale;
  float scale;
  const float* mask;        // null: none
  uint64_t rows_per_mask;   // consecutive rows that share one mask row
};
__device__ __forceinline__ float softmax_logit(const SoftmaxPrologue& pg, const float* mrow,
                                               float v, uint32_t c) {
  if (pg.has_scale) v = __fmul_rn(v, pg.scale);
  if (mrow) v = __fadd_rn(v, __ldg(mrow + c));
  return v;
}

// FAST (the TF32 math mode): e = expf(a), the sum in fp32 (lanes, then a shuffle tree) and
// a multiplication by its reciprocal; relative error of a result below 1e-6.
__device__ __forceinline__ float warp_sum_f32(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int REGS, bool FAST>
__global__ void softmax_kernel(const float* __restrict__ x, float* __restrict__ y,
                               uint64_t rows, uint32_t cols, SoftmaxPrologue pg) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  if (REGS > 0) {
    // The row a warp handles next is fetched while it works on the current one: a row is a
    // chain of load -> max -> exp -> sum -> divide -> store, and without the prefetch the
    // warps sit in the load at the head of every row.
    constexpr int R = REGS > 0 ? REGS : 1;
    float nx[R], nm[R];
    auto fetch = [&](uint64_t row) {
      const float* xr = x + row * cols;
      // (a 64-bit division costs more than the rest of the row's bookkeeping)
      const uint64_t mrow_idx = (row | pg.rows_per_mask) >> 32
                                    ? row / pg.rows_per_mask
                                    : (uint64_t)((uint32_t)row / (uint32_t)pg.rows_per_mask);
      const float* mr = pg.mask ? pg.mask + mrow_idx * cols : nullptr;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const uint32_t c = lane + 32 * j;
        nx[j] = c < cols ? xr[c] : 0.0f;
        nm[j] = (mr != nullptr && c < cols) ? __ldg(mr + c) : 0.0f;
      }
    };
    if (warp < rows) fetch(warp);
    for (uint64_t r = warp; r < rows; r += nwarps) {
      float* yr = y + r * cols;
      float v[R];
#pragma unroll
      for (int j = 0; j < R; ++j) {
        float t = nx[j];
        if (pg.has_scale) t = __fmul_rn(t, pg.scale);
        if (pg.mask) t = __fadd_rn(t, nm[j]);
        v[j] = lane + 32 * j < cols ? t : -INFINITY;
      }
      if (r + nwarps < rows) fetch(r + nwarps);
      float m = __shfl_sync(0xffffffffu, v[0], 0);  // column 0 exists in every row
#pragma unroll
      for (int j = 0; j < R; ++j)
        if (lane + 32 * j < cols) m = nan_max(m, v[j]);
      m = warp_nan_max(m);
      if (FAST) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < R; ++j) {
          if (lane + 32 * j < cols) {
            v[j] = expf(__fsub_rn(v[j], m));
            s = __fadd_rn(s, v[j]);
          }
        }
        const float inv = __frcp_rn(warp_sum_f32(s));
#pragma unroll
        for (int j = 0; j < R; ++j) {
          const uint32_t c = lane + 32 * j;
          if (c < cols) yr[c] = __fmul_rn(v[j], inv);
        }
        continue;
      }
      double s = 0.0;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        if (lane + 32 * j < cols) {
          v[j] = (float)exp_fast((double)__fsub_rn(v[j], m));
          s += (double)v[j];
        }
      }
      const float sf = (float)warp_sum(s);
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const uint32_t c = lane + 32 * j;
        if (c < cols) yr[c] = __fdiv_rn(v[j], sf);
      }
    }
    return;
  }
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const float* xr = x + r * cols;
    float* yr = y + r * cols;
    const float* mrow = pg.mask ? pg.mask + (r / pg.rows_per_mask) * cols : nullptr;
    float m = softmax_logit(pg, mrow, xr[0], 0);
    {
      for (uint32_t c = lane; c < cols; c += 32) m = nan_max(m, softmax_logit(pg, mrow, xr[c], c));
      m = warp_nan_max(m);
      if (FAST) {
        float s = 0.0f;
        for (uint32_t c = lane; c < cols; c += 32) {
          const float e = expf(__fsub_rn(softmax_logit(pg, mrow, xr[c], c), m));
          yr[c] = e;
          s = __fadd_rn(s, e);
        }
        const float inv = __frcp_rn(warp_sum_f32(s));
        for (uint32_t c = lane; c < cols; c += 32) yr[c] = __fmul_rn(yr[c], inv);
        continue;
      }
      double s = 0.0;
      for (uint32_t c = lane; c < cols; c += 32) {
        const float e = (float)exp_fast((double)__fsub_rn(softmax_logit(pg, mrow, xr[c], c), m));
        yr[c] = e;
        s += (double)e;
      }
      const float sf = (float)warp_sum(s);
      for (uint32_t c = lane; c < cols; c += 32) yr[c] = __fdiv_rn(yr[c], sf);
    }
  }
}

// FAST for rows of a multiple of four floats at 16-byte aligned addresses: a lane holds
// 16-byte pieces of its row (R4 of them: rows up to 128 * R4 floats), so a row of 128 is one
// load, one mask load and one store per lane.  Pieces beyond the row hold -inf, whose
// exponential is 0: the reductions need no predicates.  max.NaN keeps a NaN as the
// reference's Math.max does; e = 2^((x - max) * log2(e)) on the special-function unit
// (two units in the last place; the argument's rounding adds |x - max| * 2^-24 relative, at
// most 2e-8 of the largest term).
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
template <int R4>
__global__ void __launch_bounds__(kThreads, R4 == 1 ? 8 : 1)
softmax_vec_kernel(const float* __restrict__ x, float* __restrict__ y, uint64_t rows,
                   uint32_t cols, SoftmaxPrologue pg) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const uint32_t n4 = cols >> 2;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 nx[R4], nm[R4];
  auto fetch = [&](uint64_t row) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
    const uint64_t mrow_idx = (row | pg.rows_per_mask) >> 32
                                  ? row / pg.rows_per_mask
                                  : (uint64_t)((uint32_t)row / (uint32_t)pg.rows_per_mask);
    const float4* mr =
        pg.mask ? reinterpret_cast<const float4*>(pg.mask + mrow_idx * cols) : nullptr;
#pragma unroll
    for (int j = 0; j < R4; ++j) {
      const uint32_t c = lane + 32 * j;
      nx[j] = c < n4 ? xr[c] : zero;
      nm[j] = (mr != nullptr && c < n4) ? __ldg(mr + c) : zero;
    }
  };
  if (warp < rows) fetch(warp);
  for (uint64_t r = warp; r < rows; r += nwarps) {
    float4* yr = reinterpret_cast<float4*>(y + r * cols);
    float v[R4][4];
#pragma unroll
    for (int j = 0; j < R4; ++j) {
      const float q[4] = {nx[j].x, nx[j].y, nx[j].z, nx[j].w};
      const float mk[4] = {nm[j].x, nm[j].y, nm[j].z, nm[j].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float t = q[k];
        if (pg.has_scale) t = __fmul_rn(t, pg.scale);
        if (pg.mask) t = __fadd_rn(t, mk[k]);
        v[j][k] = lane + 32 * j < n4 ? t : -INFINITY;
      }
    }
    if (r + nwarps < rows) fetch(r + nwarps);
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < R4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) m = max_nan(m, v[j][k]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < R4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[j][k] = exp2_approx(__fmul_rn(__fsub_rn(v[j][k], m), 1.4426950408889634f));
        s = __fadd_rn(s, v[j][k]);
      }
    const float inv = __frcp_rn(warp_sum_f32(s));
#pragma unroll
    for (int j = 0; j < R4; ++j) {
      const uint32_t c = lane + 32 * j;
      if (c < n4)
        yr[c] = make_float4(__fmul_rn(v[j][0], inv), __fmul_rn(v[j][1], inv),
                            __fmul_rn(v[j][2], inv), __fmul_rn(v[j][3], inv));
    }
  }
}

// ---- layer normalisation over the last axis, as the converter leaves it in a graph:
//   mean = Mean(x); var = Mean(SquaredDifference(x, mean)); rs = Rsqrt(var + eps);
//   y = ((x - mean) * rs) * gamma + beta
// Nine kernels of the reference (Mean.ts, SquaredDifference.ts, Add.ts, Rsqrt.ts, Sub.ts,
// Multiply.ts) in one pass: a warp keeps its row in registers and performs the same
// fp32 operations in the same order (every intermediate rounded to fp32, the two sums
// accumulated in double over fl32(element / n), lanes striding 16-byte pieces as the
// Mean kernel does), so the result carries the bits of the separate kernels.
// NV = 16-byte pieces per lane (rows up to 128 * NV floats).  With `res` the normalised
// tensor is Add(x, res) (the residual connection in front of the normalisation), formed
// in registers.
// FAST (the TF32 math mode, whose contract is a tolerance): the two sums in fp32 - mean =
// sum(x) * (1 / n), var = sum((x - mean)^2) * (1 / n) with fused multiply-adds - and the
// reciprocal square root in fp32; the normalisation itself keeps the reference's four
// roundings.  About a quarter of the instructions: the double-precision form is bound by
// its conversions, IEEE divisions and fp64 adds, this one by HBM.
template <int NV, bool FAST>
__global__ void layer_norm_rows_kernel(const float* __restrict__ x,
                                       const float* __restrict__ res,
                                       const float* __restrict__ gamma,
                                       const float* __restrict__ beta, float* __restrict__ y,
                                       uint64_t rows, uint32_t cols, float nf, float eps) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  const uint32_t n4 = cols >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  const float4* b4 = reinterpret_cast<const float4*>(beta);
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const float4* x4 = reinterpret_cast<const float4*>(x + r * cols);
    float4* y4 = reinterpret_cast<float4*>(y + r * cols);
    float v[NV][4];
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const uint32_t j = u * 32 + lane;
      const float4 q = j < n4 ? __ldg(x4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[u][0] = q.x; v[u][1] = q.y; v[u][2] = q.z; v[u][3] = q.w;
      if (res != nullptr && j < n4) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(res + r * cols) + j);
        v[u][0] = __fadd_rn(v[u][0], t.x); v[u][1] = __fadd_rn(v[u][1], t.y);
        v[u][2] = __fadd_rn(v[u][2], t.z); v[u][3] = __fadd_rn(v[u][3], t.w);
      }
    }
    float mean, rs;
    if (FAST) {
      const float rn = __frcp_rn(nf);
      float s = 0.0f;
#pragma unroll
      for (int u = 0; u < NV; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k) s = __fadd_rn(s, v[u][k]);     // pieces beyond the row hold 0
      mean = __fmul_rn(warp_sum_f32(s), rn);
      s = 0.0f;
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        if (u * 32 + lane >= n4) continue;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float d = __fsub_rn(v[u][k], mean);
          s = __fmaf_rn(d, d, s);
        }
      }
      const float var = __fmul_rn(warp_sum_f32(s), rn);
      rs = __frsqrt_rn(__fadd_rn(var, eps));
    } else {
      double acc = 0.0;
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        if (u * 32 + lane >= n4) continue;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc += (double)__fdiv_rn(v[u][k], nf);
      }
      mean = (float)warp_sum(acc);
      acc = 0.0;
#pragma unroll
      for (int u = 0; u < NV; ++u) {
        if (u * 32 + lane >= n4) continue;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // SquaredDifference.ts: the difference and its square in double, stored as fp32
          const double d = (double)v[u][k] - (double)mean;
          acc += (double)__fdiv_rn((float)(d * d), nf);
        }
      }
      const float var = (float)warp_sum(acc);
      rs = (float)(1.0 / sqrt((double)__fadd_rn(var, eps)));
    }
#pragma unroll
    for (int u = 0; u < NV; ++u) {
      const uint32_t j = u * 32 + lane;
      if (j >= n4) continue;
      const float4 g = __ldg(g4 + j), b = __ldg(b4 + j);
      const float gg[4] = {g.x, g.y, g.z, g.w}, bb[4] = {b.x, b.y, b.z, b.w};
      float o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v[u][k], mean), rs), gg[k]), bb[k]);
      y4[j] = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---- reductions over the middle axis of [outer, reduce, inner] ----------------
// OP 0 sum, 1 mean (each element divided by n in fp32 first, Mean.ts:37-48),
// 2 max.
// inner == 1: one warp per output row, lanes stride the reduced axis.
template <int OP>
__global__ void reduce_rows_kernel(const float* __restrict__ x,
                                   float* __restrict__ y, uint64_t rows,
                                   uint64_t reduce, float nf) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const float* xr = x + r * reduce;
    double acc = 0.0;
    float mx = xr[0];
    if ((reduce & 3) == 0 && ((uintptr_t)x & 15) == 0) {
      const float4* x4 = reinterpret_cast<const float4*>(xr);
      const uint32_t n4 = (uint32_t)(reduce >> 2);
      // eight 16-byte loads in flight per lane (1024 floats of the row per round)
      for (uint32_t j0 = 0; j0 < n4; j0 += 256) {
        float4 q[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint32_t j = j0 + u * 32 + lane;
          q[u] = j < n4 ? __ldg(x4 + j) : make_float4(xr[0], xr[0], xr[0], xr[0]);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (j0 + u * 32 + lane >= n4) continue;
          const float e[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (OP == 0) acc += (double)e[k];
            else if (OP == 1) acc += (double)__fdiv_rn(e[k], nf);
            else mx = nan_max(mx, e[k]);
          }
        }
      }
    } else {
      for (uint64_t j = lane; j < reduce; j += 32) {
        const float v = xr[j];
        if (OP == 0) acc += (double)v;
        else if (OP == 1) acc += (double)__fdiv_rn(v, nf);
        else mx = nan_max(mx, v);
      }
    }
    if (OP == 2) {
      mx = warp_nan_max(mx);
      if (lane == 0) y[r] = mx;
    } else {
      acc = warp_sum(acc);
      if (lane == 0) y[r] = (float)acc;
    }
  }
}

// inner > 1: one thread per (outer, inner) output, coalesced across inner.
template <int OP>
__global__ void reduce_mid_kernel(const float* __restrict__ x,
                                  float* __restrict__ y, uint64_t outer,
                                  uint64_t reduce, uint64_t inner, float nf) {
  const uint64_t n = outer * inner;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const uint64_t o = i / inner, in = i % inner;
    const float* xp = x + o * reduce * inner + in;
    double acc = 0.0;
    float mx = xp[0];
    // eight independent loads in flight per thread; the accumulation order stays j = 0, 1, ...
    uint64_t j = 0;
    for (; j + 8 <= reduce; j += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(xp + (j + u) * inner);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (OP == 0) acc += (double)v[u];
        else if (OP == 1) acc += (double)__fdiv_rn(v[u], nf);
        else mx = nan_max(mx, v[u]);
      }
    }
    for (; j < reduce; ++j) {
      const float v = xp[j * inner];
      if (OP == 0) acc += (double)v;
      else if (OP == 1) acc += (double)__fdiv_rn(v, nf);
      else mx = nan_max(mx, v);
    }
    y[i] = OP == 2 ? mx : (float)acc;
  }
}

// ---- argmax: tfjs-backend-cpu/src/kernels/ArgMax.ts:55-66 ---------------------
// Sequential semantics: max starts at element 0 and moves on `value > max`, so
// the answer is 0 when element 0 is NaN, else the first index of the largest
// non-NaN value.
struct Best {
  float v;
  int32_t i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // NaN entries never win; ties go to the smaller index.
  if (b.v != b.v) return a;
  if (a.v != a.v) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__global__ void argmax_rows_kernel(const float* __restrict__ x,
                                   int32_t* __restrict__ y, uint64_t rows,
                                   uint64_t reduce) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint64_t nwarps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const float* xr = x + r * reduce;
    const float first = xr[0];
    Best b;
    b.v = NAN;
    b.i = 0x7fffffff;
    for (uint64_t j = lane; j < reduce; j += 32) {
      Best c;
      c.v = xr[j];
      c.i = (int32_t)j;
      b = better(b, c);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best c;
      c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, c);
    }
    if (lane == 0) y[r] = (first != first || b.v != b.v) ? 0 : b.i;
  }
}

__global__ void argmax_mid_kernel(const float* __restrict__ x,
                                  int32_t* __restrict__ y, uint64_t outer,
                                  uint64_t reduce, uint64_t inner) {
  const uint64_t n = outer * inner;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const uint64_t o = i / inner, in = i % inner;
    const float* xp = x + o * reduce * inner + in;
    float mx = xp[0];
    int32_t mi = 0;
    for (uint64_t j = 0; j < reduce; ++j) {
      const float v = xp[j * inner];
      if (v > mx) { mx = v; mi = (int32_t)j; }
    }
    y[i] = mi;
  }
}

}  // namespace

extern "C" {

static int softmax_impl(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows, uint64_t cols,
                        int32_t has_scale, float scale, int32_t mask_id,
                        uint64_t rows_per_mask, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *x, *y, *mask = nullptr;
  int rc;
  if ((rc = ctx_get(ctx, x_id, rows * cols * 4, "softmax x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, rows * cols * 4, "softmax out", &y))) return rc;
  if (mask_id != 0) {
    if (rows_per_mask == 0)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "softmax: rows_per_mask must be positive");
    const uint64_t mask_rows = rows ? (rows - 1) / rows_per_mask + 1 : 0;
    if ((rc = ctx_get(ctx, mask_id, mask_rows * cols * 4, "softmax mask", &mask))) return rc;
  }
  SoftmaxPrologue pg;
  pg.has_scale = has_scale;
  pg.scale = scale;
  pg.mask = mask ? (const float*)mask->ptr : nullptr;
  pg.rows_per_mask = rows_per_mask ? rows_per_mask : 1;
  if (rows * cols == 0) return TFJS_CUDA_OK;
  if (cols > 0xffffffffu)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "softmax: row too wide");
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for(rows * 32, kThreads, ctx->sm_count);
  const float* xp = (const float*)x->ptr;
  float* yp = (float*)y->ptr;
  const uint32_t c32 = (uint32_t)cols;
  const bool fast = ctx->math_mode == TFJS_CUDA_MATH_TF32;
#define SOFTMAX(R)                                                                          \
  do {                                                                                      \
    if (fast) softmax_kernel<R, true><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, rows, c32, pg); \
    else softmax_kernel<R, false><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, rows, c32, pg);     \
  } while (0)
  const bool vec = fast && (cols & 3) == 0 && cols > 64 && cols <= 1024 &&
                   (((uintptr_t)xp | (uintptr_t)yp | (uintptr_t)pg.mask) & 15) == 0;
#define SOFTMAX_VEC(R4) \
  softmax_vec_kernel<R4><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, rows, c32, pg)
  if (vec && cols <= 128) SOFTMAX_VEC(1);
  else if (vec && cols <= 256) SOFTMAX_VEC(2);
  else if (vec && cols <= 512) SOFTMAX_VEC(4);
  else if (vec) SOFTMAX_VEC(8);
#undef SOFTMAX_VEC
  else if (cols <= 32) SOFTMAX(1);
  else if (cols <= 64) SOFTMAX(2);
  else if (cols <= 128) SOFTMAX(4);
  else if (cols <= 256) SOFTMAX(8);
  else if (cols <= 512) SOFTMAX(16);
  else if (cols <= 1024) SOFTMAX(32);
  else SOFTMAX(0);
#undef SOFTMAX
  LAUNCH_CHECK(ctx, "softmax_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_softmax(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows,
                      uint64_t cols, int32_t out_id) {
  return softmax_impl(ctx, x_id, rows, cols, 0, 1.0f, 0, 1, out_id);
}

int tfjs_cuda_softmax_scaled_masked(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows,
                                    uint64_t cols, int32_t has_scale, float scale,
                                    int32_t mask_id, uint64_t rows_per_mask, int32_t out_id) {
  return softmax_impl(ctx, x_id, rows, cols, has_scale, scale, mask_id, rows_per_mask, out_id);
}

int tfjs_cuda_layer_norm(tfjs_cuda_ctx* ctx, int32_t x_id, int32_t residual_id, int32_t gamma_id,
                         int32_t beta_id, uint64_t rows, uint64_t cols, float epsilon,
                         int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *x, *g, *b, *y, *res = nullptr;
  int rc;
  if ((rc = ctx_get(ctx, x_id, rows * cols * 4, "layer norm x", &x))) return rc;
  if (residual_id != 0 &&
      (rc = ctx_get(ctx, residual_id, rows * cols * 4, "layer norm residual", &res)))
    return rc;
  if ((rc = ctx_get(ctx, gamma_id, cols * 4, "layer norm gamma", &g))) return rc;
  if ((rc = ctx_get(ctx, beta_id, cols * 4, "layer norm beta", &b))) return rc;
  if ((rc = ctx_get(ctx, out_id, rows * cols * 4, "layer norm out", &y))) return rc;
  if (rows * cols == 0) return TFJS_CUDA_OK;
  if ((cols & 3) || cols > 1024 ||
      (((uintptr_t)x->ptr | (uintptr_t)g->ptr | (uintptr_t)b->ptr | (uintptr_t)y->ptr |
        (uintptr_t)(res ? res->ptr : nullptr)) & 15))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "layer norm: rows of a multiple of 4 up to 1024 floats, 16-byte aligned");
  cudaSetDevice(ctx->device);
  const unsigned grid = grid_for(rows * 32, kThreads, ctx->sm_count);
  const bool fast = ctx->math_mode == TFJS_CUDA_MATH_TF32;
#define LNORM(NV)                                                                          \
  do {                                                                                     \
    if (fast)                                                                              \
      layer_norm_rows_kernel<NV, true><<<grid, kThreads, 0, ctx->stream>>>(                \
          (const float*)x->ptr, res ? (const float*)res->ptr : nullptr, (const float*)g->ptr, \
          (const float*)b->ptr, (float*)y->ptr, rows, (uint32_t)cols, (float)cols, epsilon); \
    else                                                                                   \
      layer_norm_rows_kernel<NV, false><<<grid, kThreads, 0, ctx->stream>>>(               \
          (const float*)x->ptr, res ? (const float*)res->ptr : nullptr, (const float*)g->ptr, \
          (const float*)b->ptr, (float*)y->ptr, rows, (uint32_t)cols, (float)cols, epsilon); \
  } while (0)
  if (cols <= 128) LNORM(1);
  else if (cols <= 256) LNORM(2);
  else if (cols <= 512) LNORM(4);
  else if (cols <= 768) LNORM(6);
  else LNORM(8);
#undef LNORM
  LAUNCH_CHECK(ctx, "layer_norm_rows_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_reduce(tfjs_cuda_ctx* ctx, int32_t op, int32_t x_id,
                     uint64_t outer, uint64_t reduce, uint64_t inner,
                     int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (op < 0 || op > 2) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "reduce: op %d", op);
  Buffer *x, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, outer * reduce * inner * 4, "reduce x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, outer * inner * 4, "reduce out", &y))) return rc;
  if (outer * inner == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  if (reduce == 0) {
    // Sum/Mean over nothing is 0; Max over nothing is not defined by the reference.
    CUDA_TRY(ctx, cudaMemsetAsync(y->ptr, 0, outer * inner * 4, ctx->stream));
    ctx_mark_written(ctx, out_id);
    return TFJS_CUDA_OK;
  }
  const float nf = (float)reduce;
  const float* xp = (const float*)x->ptr;
  float* yp = (float*)y->ptr;
  if (inner == 1) {
    const unsigned grid = grid_for(outer * 32, kThreads, ctx->sm_count);
    if (op == 0) reduce_rows_kernel<0><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, outer, reduce, nf);
    else if (op == 1) reduce_rows_kernel<1><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, outer, reduce, nf);
    else reduce_rows_kernel<2><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, outer, reduce, nf);
  } else {
    const unsigned grid = grid_for(outer * inner, 128, ctx->sm_count);
    if (op == 0) reduce_mid_kernel<0><<<grid, 128, 0, ctx->stream>>>(xp, yp, outer, reduce, inner, nf);
    else if (op == 1) reduce_mid_kernel<1><<<grid, 128, 0, ctx->stream>>>(xp, yp, outer, reduce, inner, nf);
    else reduce_mid_kernel<2><<<grid, 128, 0, ctx->stream>>>(xp, yp, outer, reduce, inner, nf);
  }
  LAUNCH_CHECK(ctx, "reduce_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_argmax(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t outer,
                     uint64_t reduce, uint64_t inner, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *x, *y;
  int rc;
  if ((rc = ctx_get(ctx, x_id, outer * reduce * inner * 4, "argmax x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, outer * inner * 4, "argmax out", &y))) return rc;
  if (outer * inner == 0) return TFJS_CUDA_OK;
  if (reduce == 0 || reduce > 0x7fffffffu)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "argmax: bad reduce size");
  cudaSetDevice(ctx->device);
  if (inner == 1)
    argmax_rows_kernel<<<grid_for(outer * 32, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (int32_t*)y->ptr, outer, reduce);
  else
    argmax_mid_kernel<<<grid_for(outer * inner, 128, ctx->sm_count), 128, 0, ctx->stream>>>(
        (const float*)x->ptr, (int32_t*)y->ptr, outer, reduce, inner);
  LAUNCH_CHECK(ctx, "argmax_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

}  // extern "C"
