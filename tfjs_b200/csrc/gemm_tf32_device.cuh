// Device-side pieces shared by the tcgen05 TF32 GEMM kernels: the argument block,
// TMA / tcgen05 PTX wrappers, shared-memory descriptors, the bias + activation step of
// the epilogue and the persistent work iterator.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "common.cuh"
#include "gemm.h"
#include "ptx.cuh"

constexpr int BM = 128;
constexpr int BK = 32;          // floats per K step = one 128-byte swizzle row
constexpr int UMMA_K = 8;       // K of one tcgen05.mma.kind::tf32
constexpr int A_STAGE_BYTES = BM * BK * 4;

struct Tf32Args {
  float* c;
  const float* bias;
  int bias_len;
  ActParams ap;
  int M, N;
  int batch_a, batch_b;
  int tiles_m, tiles_n, total_tiles;
  int k_steps;
  int* flag;
  int c_tma;  // 1: the epilogue stores through the C tensor map (N % 4 == 0)
  const float* residual;  // optional: out = post_act(act(acc + bias) + residual)
  int post_act;
  int out_perm, perm_p, perm_d;  // heads-permuted store through a 4-D C map (GemmProblem)
  // K-split of the last, partial wave (SK instantiations): the last sk_tiles tiles are cut
  // along K into one contiguous share per CTA; partial accumulators travel through sk_ws
  int sk_tiles;
  float* sk_ws;         // [CTA][epilogue warp][chunk][32 columns][32 rows] fp32
  unsigned* sk_flags;   // [CTA][epilogue warp]: 1 while that warp's partial waits to be read
  int patch_cap;          // staged-row gather: bytes per patch buffer, 0 = off
  int patch_pitch;        // floats between patch rows (left margin + image row + right margin)
  int patch_ml;           // floats of left margin
  int patch_rows;         // image rows a buffer holds; row `patch_rows` stays zero
  int patch_bufs;         // patch buffers (2 to 8); tiles are staged patch_bufs - 1 ahead
  uint32_t ow_mul, ow_shr, oh_mul, oh_shr;  // division by out_w / out_h as multiply-shift
  // gathered convolution
  const float* x;
  ConvGeo conv;
  int chunks_per_tap;  // 32-channel chunks per filter tap
};

// CTA-pair form (tcgen05.mma.cta_group::2, gemm_tf32_pair_sm100.cu): 256 x 256 output tiles
// over two SMs.  tm_a: 128-row boxes of A (or the im2col map), tm_b: 128-row boxes of the
// K-major B operand, tm_c: 32 x 32 store boxes.  g.tiles_m counts 256-row tiles.
int launch_gemm_tf32_pair(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                          const CUtensorMap& tm_c, Tf32Args& g, bool im2col);
// 256 x 384 tiles (two N = 192 MMAs per K slice, one accumulator stage): tm_b holds 96-row
// boxes.  For outputs whose 256 x 384 tiles all run at once.
int launch_gemm_tf32_pair_wide(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a,
                               const CUtensorMap& tm_b, const CUtensorMap& tm_c, Tf32Args& g);
// The same for a group of products that share A (GemmGroup): the tile index runs over the
// members' column tiles side by side.
struct PairGroupMaps {
  CUtensorMap b[kMaxGemmGroup];
  CUtensorMap c[kMaxGemmGroup];
  const float* bias[kMaxGemmGroup];
  int count;
};
int launch_gemm_tf32_pair_group(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a,
                                const PairGroupMaps& maps, Tf32Args& g);

namespace {

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm,
                                            uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tm), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col(uint32_t dst, const CUtensorMap* tm,
                                                uint32_t bar, int c, int w, int h, int n,
                                                uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(tm), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
// Starts the fetch of a tensor map (a kernel parameter) into the TMA unit's descriptor
// cache, so that the first load or store through it does not wait for it.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t adesc,
                                            uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
      "[%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
        "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
        "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptors (128-byte swizzle, descriptor version 1).
// K-major: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3fff) | (1ull << 16) | (64ull << 32) |
         (1ull << 46) | (2ull << 61);
}
// MN-major 32-bit operands use the "128-byte swizzle, 32-byte atom" layout
// (layout type 1; TMA swizzle mode 128B_ATOM_32B): rows of 32 contiguous floats
// along N, 4-row K groups 512 bytes apart (stride offset), 32-float column
// blocks 4096 bytes apart (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3fff) | (256ull << 16) | (32ull << 32) |
         (1ull << 46) | (1ull << 61);
}

// Bias + activation on the 32 accumulator columns a thread holds, with the
// activation resolved at compile time so the unrolled loop has no per-element
// dispatch.
// The bias of column n0 + lane, fetched by each lane ahead of the accumulator (0 when the
// kernel has no bias or the column lies beyond N).
__device__ __forceinline__ float chunk_bias(const Tf32Args& g, int n0, int lane,
                                            const float* bias) {
  if (g.bias_len == 0) return 0.0f;
  if (g.bias_len == 1) return __ldg(bias);
  return n0 + lane < g.N ? __ldg(bias + n0 + lane) : 0.0f;
}
__device__ __forceinline__ float chunk_bias(const Tf32Args& g, int n0, int lane) {
  return chunk_bias(g, n0, lane, g.bias);
}

template <int ACT>
__device__ __forceinline__ void chunk_math(float* v, const Tf32Args& g, int n0, float bj,
                                           bool skip_bias = false, const float* bias = nullptr) {
  if (bias == nullptr) bias = g.bias;
  if (g.bias_len != 0 && !skip_bias) {
    if (g.bias_len > 1 && n0 + 32 <= g.N) {
      // every thread owns a row of 32 columns: eight 16-byte loads at a warp-uniform
      // address (served as broadcasts) instead of 32 shuffles
      const float4* b4 = reinterpret_cast<const float4*>(bias + n0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 b = __ldg(b4 + j);
        v[4 * j] = __fadd_rn(v[4 * j], b.x);
        v[4 * j + 1] = __fadd_rn(v[4 * j + 1], b.y);
        v[4 * j + 2] = __fadd_rn(v[4 * j + 2], b.z);
        v[4 * j + 3] = __fadd_rn(v[4 * j + 3], b.w);
      }
    } else {
      // lane j holds the bias of column n0 + j
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], __shfl_sync(0xffffffffu, bj, j));
    }
  }
  if constexpr (ACT == TFJS_CUDA_ACT_LINEAR) {
    return;
  } else if constexpr (ACT == TFJS_CUDA_ACT_GELU_ERF) {
    // the tensor-core kernels run in the TF32 math mode only, where erf is the fp32 form
    // (the same device function as the separate Erf kernel and the chain kernels)
    // two columns at a time (packed fp32 arithmetic): an epilogue warp has one issue slot
    // in two, and the MMA of a 768-deep product leaves it about 12 cycles per element
    const unsigned long long scale2 = pack_f32x2(g.ap.gelu_scale, g.ap.gelu_scale);
    const unsigned long long half2 = pack_f32x2(g.ap.gelu_half, g.ap.gelu_half);
    const unsigned long long one2 = pack_f32x2(g.ap.gelu_one, g.ap.gelu_one);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const unsigned long long x = pack_f32x2(v[j], v[j + 1]);
      const unsigned long long a =
          g.ap.gelu_divide ? pack_f32x2(__fdiv_rn(v[j], g.ap.gelu_scale),
                                        __fdiv_rn(v[j + 1], g.ap.gelu_scale))
                           : mul_f32x2(x, scale2);
      unpack_f32x2(mul_f32x2(mul_f32x2(x, half2), add_f32x2(erf_f32x2(a), one2)), v[j],
                   v[j + 1]);
    }
  } else {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float t = v[j];
    if (ACT == TFJS_CUDA_ACT_RELU) {
      // max.NaN / min.NaN keep a NaN input, as Math.max / Math.min do
      asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(v[j]) : "f"(t));
    } else if (ACT == TFJS_CUDA_ACT_RELU6) {
      float r;
      asm("max.NaN.f32 %0, %1, 0f00000000;" : "=f"(r) : "f"(t));
      asm("min.NaN.f32 %0, %1, 0f40C00000;" : "=f"(v[j]) : "f"(r));
    } else if (ACT == TFJS_CUDA_ACT_PRELU) {
      const float a = __ldg(g.ap.prelu + (g.ap.prelu_len == 1 ? 0 : (n0 + j < g.N ? n0 + j : 0)));
      v[j] = t < 0.0f ? __fmul_rn(a, t) : t;
    } else if (ACT == TFJS_CUDA_ACT_LEAKYRELU) {
      v[j] = js_leakyrelu(t, g.ap.alpha);
    } else if (ACT == TFJS_CUDA_ACT_SIGMOID) {
      v[j] = sigmoid_f32(t);
    } else if (ACT == TFJS_CUDA_ACT_ELU) {
      v[j] = elu_f32(t);
    }
  }
  }
}

__device__ __forceinline__ void chunk_math_dispatch(float* v, const Tf32Args& g, int n0,
                                                    float bj, bool skip_bias = false,
                                                    const float* bias = nullptr) {
  switch (g.ap.act) {
    case TFJS_CUDA_ACT_RELU: chunk_math<TFJS_CUDA_ACT_RELU>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_RELU6: chunk_math<TFJS_CUDA_ACT_RELU6>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_PRELU: chunk_math<TFJS_CUDA_ACT_PRELU>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_LEAKYRELU: chunk_math<TFJS_CUDA_ACT_LEAKYRELU>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_SIGMOID: chunk_math<TFJS_CUDA_ACT_SIGMOID>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_ELU: chunk_math<TFJS_CUDA_ACT_ELU>(v, g, n0, bj, skip_bias, bias); break;
    case TFJS_CUDA_ACT_GELU_ERF: chunk_math<TFJS_CUDA_ACT_GELU_ERF>(v, g, n0, bj, skip_bias, bias); break;
    default: chunk_math<TFJS_CUDA_ACT_LINEAR>(v, g, n0, bj, skip_bias, bias); break;
  }
}

// n / d for 0 <= n < 2^31 as umulhi(n, mul) >> shr (mul = ceil(2^(32+shr) / d)).
__device__ __forceinline__ int fast_div(int n, uint32_t mul, uint32_t shr) {
  return mul ? (int)(__umulhi((uint32_t)n, mul) >> shr) : n;
}
inline void fast_div_setup(int d, uint32_t* mul, uint32_t* shr) {
  if (d <= 1) { *mul = 0; *shr = 0; return; }
  int lg = 0;
  while ((1ll << lg) < d) ++lg;
  const int p = 31 + lg;
  *mul = (uint32_t)(((1ull << p) + (uint64_t)d - 1) / (uint64_t)d);
  *shr = (uint32_t)(p - 32);
}

constexpr int kTapTableEntries = 512;  // scalar-gather K limit (after padding to 32)

constexpr int kMaxSmemBytes = 232448;  // 227 KB per CTA
constexpr int kBarrierBytes = 640;  // pipeline barriers, TMEM slot, residual barriers

// The work items of a CTA, in the order every warp role walks them.  Plain: the tiles
// blockIdx.x, + gridDim.x, ... each over all K steps.  With a K-split tail: the tiles of
// the full waves first, then this CTA's contiguous share [u, u1) of the K steps of the
// last sk_tiles tiles (units = sk_tiles * k_steps, split evenly over the CTAs), which
// touches one to a few tiles: possibly the tail of a tile another CTA started, whole
// tiles, and the head of a tile that later CTAs finish.
struct WorkIter {
  int idx, n_dp, stride, first, k_steps, sk_base;
  long long u, u1;
  __device__ __forceinline__ void init(const Tf32Args& g, bool sk) {
    idx = 0;
    stride = (int)gridDim.x;
    first = (int)blockIdx.x;
    k_steps = g.k_steps;
    u = u1 = 0;
    sk_base = 0;
    if (!sk || g.sk_tiles == 0) {
      const int t = g.total_tiles - first;
      n_dp = t > 0 ? (t + stride - 1) / stride : 0;
    } else {
      sk_base = g.total_tiles - g.sk_tiles;  // a multiple of the grid
      n_dp = sk_base / stride;
      const long long T = (long long)g.sk_tiles * k_steps;
      u = T * first / stride;
      u1 = T * (first + 1) / stride;
    }
  }
  // false when the CTA has no more work; `it` of the item is idx - 1 afterwards
  __device__ __forceinline__ bool next(int& tile, int& ks0, int& ks1) {
    if (idx < n_dp) {
      tile = first + idx * stride;
      ks0 = 0;
      ks1 = k_steps;
      ++idx;
      return true;
    }
    if (u < u1) {
      const int sk = (int)(u / k_steps);
      ks0 = (int)(u - (long long)sk * k_steps);
      const long long left = u1 - u;
      ks1 = left < (long long)(k_steps - ks0) ? ks0 + (int)left : k_steps;
      tile = sk_base + sk;
      u += ks1 - ks0;
      ++idx;
      return true;
    }
    return false;
  }
};

}  // namespace
