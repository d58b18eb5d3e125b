// FusedConv2D of a 3-channel image with a 3 x 3 stride-2 filter and 32 output channels (the
// stem of MobileNetV2; tfjs-backend-cpu/src/kernels/FusedConv2D.ts:26-95 over
// Conv2D_impl's loops) as a direct fp32 kernel.
//
// K is 27: as a GEMM the layer is one padded K step per 128-pixel tile, whose per-tile
// hand-offs (gather warps, barriers, tensor memory, epilogue) cost more than its
// arithmetic, 0.30 ms at batch 256 against 87 us of compulsory traffic.  Here a persistent
// CTA takes four output rows of one image at a time: one thread copies the nine input rows
// they need into shared memory with bulk copies (four buffers, the next units' rows arrive
// while this one is computed); eight lanes own eight neighbouring output pixels, each lane
// four output channels, with the filter in shared memory.  5.5 GFLOP of fp32 FMAs in the
// reference's own accumulation order (filter row, filter column, input channel), so the
// result is the fp32 convolution: at least as close to the reference as the TF32 product it
// replaces.  Every wait is bounded.
#include "common.cuh"
#include "gemm.h"
#include "ptx.cuh"

namespace {

constexpr int kStemRows = 4;                       // output rows per unit
constexpr int kStemInRows = 2 * kStemRows + 1;     // input rows they read
constexpr int kStemWarps = 14;                     // compute warps (one more produces)
constexpr int kStemThreads = (kStemWarps + 1) * 32;
constexpr int kStemMaxSmem = 227 * 1024;
constexpr int kStemBufs = 4;                       // units whose input rows are in flight or in use

struct StemArgs {
  const float* x;      // [batch, in_h, in_w, 3]
  const float* w;      // [3, 3, 3, 32]
  const float* bias;   // 32 values, one value or null
  int bias_len;
  float* y;            // [batch, out_h, out_w, 32]
  const float* residual;   // optional, shaped like y: y = post_act(act(conv + bias) + residual)
  int post_act;
  int batch, in_h, in_w, out_h, out_w, pad_t;
  int groups;          // 8-pixel groups per output row
  int pitch;           // floats between staged input rows (row, then zeros)
  int units_per_image, units;
  int* flag;
};

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
      "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

template <int ACT>
__global__ void __launch_bounds__(kStemThreads, 1) stem_conv3x3s2_kernel(const StemArgs g) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  float* rows = reinterpret_cast<float*>(smem_raw);            // [kStemBufs][kStemInRows][pitch]
  const uint32_t rows_u32 = smem_u32(smem_raw);
  const uint32_t buf_bytes = (uint32_t)(kStemInRows * g.pitch) * 4u;
  float* wts = rows + kStemBufs * kStemInRows * g.pitch;       // the filter: [27][32]
  const uint32_t bar_base = rows_u32 + (uint32_t)kStemBufs * buf_bytes + 27u * 32u * 4u;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * kStemBufs + 8u * s; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // the columns behind a row's end stay zero for the whole kernel (right-hand padding)
  for (uint32_t i = threadIdx.x; i < kStemBufs * buf_bytes / 4u; i += blockDim.x) rows[i] = 0.0f;
  for (int k = threadIdx.x; k < 27 * 32; k += blockDim.x) wts[k] = __ldg(g.w + k);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStemBufs; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kStemWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the zeros (generic proxy) must be in place before the bulk copies (async proxy) land
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  const int first = (int)blockIdx.x, step = (int)gridDim.x;
  const uint32_t row_bytes = (uint32_t)g.in_w * 12u;

  if (warp == kStemWarps) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      int i = 0;
      for (int u = first; u < g.units; u += step, ++i) {
        const int s = i % kStemBufs;
        const uint32_t ph = (uint32_t)(i / kStemBufs) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1)) {
          atomicExch(g.flag, 1);
          break;
        }
        const int b = u / g.units_per_image;
        const int iy0 = (u - b * g.units_per_image) * kStemRows * 2 - g.pad_t;
        int lo = iy0 < 0 ? -iy0 : 0;
        int hi = g.in_h - iy0 < kStemInRows ? g.in_h - iy0 : kStemInRows;   // rows lo .. hi-1 exist
        if (hi < lo) hi = lo;
        mbar_expect_tx(full_bar(s), (uint32_t)(hi - lo) * row_bytes);
        for (int j = lo; j < hi; ++j)
          bulk_copy_g2s(rows_u32 + (uint32_t)s * buf_bytes + (uint32_t)(j * g.pitch) * 4u,
                        g.x + ((size_t)b * g.in_h + (size_t)(iy0 + j)) * g.in_w * 3, row_bytes,
                        full_bar(s));
      }
    }
    return;
  }

  // ------------------------------------------------------------- compute --
  // A lane owns four output channels (lane % 8) of one 8-pixel group (lane / 8 picks one of
  // the warp's four groups): a 16-byte shared load then fills the registers of a quarter of
  // the warp with distinct data instead of 32 copies of one value, which is what bounds a
  // one-channel-per-lane layout (512 bytes of register fill per load, 128 per cycle and SM).
  const int cq = lane & 7, sub = lane >> 3;
  const float4* wsm = reinterpret_cast<const float4*>(wts);      // [27][8] quads of channels
  float bias4[4] = {0.f, 0.f, 0.f, 0.f};
  if (g.bias_len != 0) {
#pragma unroll
    for (int c = 0; c < 4; ++c) bias4[c] = __ldg(g.bias + (g.bias_len == 1 ? 0 : 4 * cq + c));
  }
  const int items = kStemRows * g.groups;   // (output row, pixel group) pairs of a unit
  int i = 0;
  for (int u = first; u < g.units; u += step, ++i) {
    const int s = i % kStemBufs;
    const uint32_t ph = (uint32_t)(i / kStemBufs) & 1u;
    if (!mbar_wait(full_bar(s), ph)) {
      if (lane == 0) atomicExch(g.flag, 2);
      break;
    }
    const int b = u / g.units_per_image;
    const int oy0 = (u - b * g.units_per_image) * kStemRows;
    const int iy0 = oy0 * 2 - g.pad_t;
    const float* buf = rows + (size_t)s * kStemInRows * g.pitch;
    for (int q0 = 4 * warp; q0 < items; q0 += 4 * kStemWarps) {
      const int q = q0 + sub;
      const bool live = q < items;
      const int t = live ? q / g.groups : 0;
      const int grp = live ? q - t * g.groups : 0;
      const int oy = oy0 + t;
      // two channels per 64-bit register: fma.rn.f32x2 performs the same two fp32 FMAs
      unsigned long long acc[8][2];
#pragma unroll
      for (int p = 0; p < 8; ++p) acc[p][0] = acc[p][1] = 0ull;
#pragma unroll 1
      for (int kh = 0; kh < 3; ++kh) {
        const int j = 2 * t + kh;
        const int iy = iy0 + j;
        if (iy < 0 || iy >= g.in_h) continue;       // a padding row contributes nothing
        unsigned long long wk[9][2];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const float4 v = wsm[(kh * 9 + k) * 8 + cq];
          wk[k][0] = pack_f32x2(v.x, v.y);
          wk[k][1] = pack_f32x2(v.z, v.w);
        }
        // 17 input columns x 3 channels from column 16 * grp on (52 floats, 51 used)
        const float4* src =
            reinterpret_cast<const float4*>(buf + (size_t)j * g.pitch + (size_t)grp * 48);
        unsigned long long xr[52];   // each input value in both halves
#pragma unroll
        for (int k = 0; k < 13; ++k) {
          const float4 v = src[k];
          xr[4 * k] = pack_f32x2(v.x, v.x); xr[4 * k + 1] = pack_f32x2(v.y, v.y);
          xr[4 * k + 2] = pack_f32x2(v.z, v.z); xr[4 * k + 3] = pack_f32x2(v.w, v.w);
        }
#pragma unroll
        for (int p = 0; p < 8; ++p)
#pragma unroll
          for (int k = 0; k < 9; ++k) {      // k = kw * 3 + ci: the reference's order
            acc[p][0] = fma_f32x2(xr[2 * p * 3 + k], wk[k][0], acc[p][0]);
            acc[p][1] = fma_f32x2(xr[2 * p * 3 + k], wk[k][1], acc[p][1]);
          }
      }
      if (!live || oy >= g.out_h) continue;
      float* out = g.y + (((size_t)b * g.out_h + oy) * g.out_w + (size_t)grp * 8) * 32 + 4 * cq;
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        if (grp * 8 + p >= g.out_w) break;
        float v[4];
        unpack_f32x2(acc[p][0], v[0], v[1]);
        unpack_f32x2(acc[p][1], v[2], v[3]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          v[c] = __fadd_rn(v[c], bias4[c]);
          // max.NaN / min.NaN keep a NaN, as Math.max / Math.min do
          if (ACT != TFJS_CUDA_ACT_LINEAR)
            asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v[c]));
          if (ACT == TFJS_CUDA_ACT_RELU6) asm("min.NaN.f32 %0, %0, 0f40C00000;" : "+f"(v[c]));
        }
        if (g.residual != nullptr) {
          const float4 r4 = __ldg(reinterpret_cast<const float4*>(g.residual + (out - g.y) + p * 32));
          const float rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            v[c] = __fadd_rn(v[c], rr[c]);
            if (g.post_act != TFJS_CUDA_ACT_LINEAR)
              asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v[c]));
            if (g.post_act == TFJS_CUDA_ACT_RELU6)
              asm("min.NaN.f32 %0, %0, 0f40C00000;" : "+f"(v[c]));
          }
        }
        *reinterpret_cast<float4*>(out + p * 32) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));
  }
}

}  // namespace

// True when the direct kernel takes this convolution (TF32 math mode is the caller's check).
bool stem_conv_supported(const GemmProblem& pr) {
  const ConvGeo& cv = pr.conv;
  const int act = pr.ap.act;
  return pr.is_conv && cv.in_c == 3 && pr.N == 32 && cv.f_h == 3 && cv.f_w == 3 && cv.s_h == 2 &&
         cv.s_w == 2 && cv.d_h == 1 && cv.d_w == 1 && cv.pad_l == 0 && cv.pad_t >= 0 &&
         cv.pad_t <= 2 && (cv.in_w % 4) == 0 && cv.out_w > 0 && cv.out_h > 0 &&
         2 * (cv.out_w - 1) + 2 <= cv.in_w &&
         (!pr.residual || (((uintptr_t)pr.residual & 15) == 0 &&
                           (pr.post_act == TFJS_CUDA_ACT_LINEAR || pr.post_act == TFJS_CUDA_ACT_RELU ||
                            pr.post_act == TFJS_CUDA_ACT_RELU6))) &&
         (act == TFJS_CUDA_ACT_LINEAR || act == TFJS_CUDA_ACT_RELU || act == TFJS_CUDA_ACT_RELU6) &&
         (pr.bias_len == 0 || pr.bias_len == 1 || pr.bias_len == 32) &&
         (((uintptr_t)pr.a | (uintptr_t)pr.c) & 15) == 0 &&
         (uint64_t)cv.batch * cv.in_h * cv.in_w * 3 < (1ull << 40);
}

int launch_stem_conv(tfjs_cuda_ctx* ctx, const GemmProblem& pr) {
  const ConvGeo& cv = pr.conv;
  StemArgs g;
  g.x = pr.a;
  g.w = pr.b;
  g.bias = pr.bias;
  g.bias_len = pr.bias ? pr.bias_len : 0;
  g.y = pr.c;
  g.residual = pr.residual;
  g.post_act = pr.post_act;
  g.batch = cv.batch; g.in_h = cv.in_h; g.in_w = cv.in_w; g.out_h = cv.out_h; g.out_w = cv.out_w;
  g.pad_t = cv.pad_t;
  g.groups = (cv.out_w + 7) / 8;
  // a group reads 52 floats from column 16 * group on; the row itself is in_w * 3 floats
  const int reach = (g.groups - 1) * 48 + 52;
  const int need = reach > cv.in_w * 3 + 4 ? reach : cv.in_w * 3 + 4;
  g.pitch = (need + 3) / 4 * 4;
  g.units_per_image = (cv.out_h + kStemRows - 1) / kStemRows;
  g.units = cv.batch * g.units_per_image;
  g.flag = ctx->d_flag;
  const size_t smem = (size_t)kStemBufs * kStemInRows * g.pitch * 4 + 27 * 32 * 4 + 16 * kStemBufs;
  if (smem > (size_t)kStemMaxSmem)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "stem convolution: image row too wide");
  auto launch = [&](auto kern, bool* configured) -> int {
    if (ctx->device >= 64 || !configured[ctx->device]) {   // per device ordinal
      CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kStemMaxSmem));
      if (ctx->device < 64) configured[ctx->device] = true;
    }
    const int grid = g.units < ctx->sm_count ? g.units : ctx->sm_count;
    kern<<<grid, kStemThreads, smem, ctx->stream>>>(g);
    return TFJS_CUDA_OK;
  };
  static bool configured[3][64] = {};
  int rc;
  switch (pr.ap.act) {
    case TFJS_CUDA_ACT_RELU: rc = launch(stem_conv3x3s2_kernel<TFJS_CUDA_ACT_RELU>, configured[0]); break;
    case TFJS_CUDA_ACT_RELU6: rc = launch(stem_conv3x3s2_kernel<TFJS_CUDA_ACT_RELU6>, configured[1]); break;
    default: rc = launch(stem_conv3x3s2_kernel<TFJS_CUDA_ACT_LINEAR>, configured[2]); break;
  }
  if (rc != TFJS_CUDA_OK) return rc;
  LAUNCH_CHECK(ctx, "stem_conv3x3s2_kernel");
  return TFJS_CUDA_OK;
}
