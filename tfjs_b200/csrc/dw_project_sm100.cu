// FusedDepthwiseConv2D (3x3, stride 1 or 2, bias, activation) followed by a 1x1 FusedConv2D, as one
// kernel: the depthwise result never reaches memory.
//
// An inverted-residual block ends with a depthwise convolution over the expanded
// activation (6x the block's channels) and a 1x1 "projection" convolution that reads it
// back.  Here the depthwise warps of a CTA produce the projection's A operand directly in
// shared memory: per K step (32 expanded channels) a 4-D TMA tile load brings the input
// patch of the CTA's spatial tile with its halo (out-of-image pixels read as zero, which is
// what skipping those taps amounts to), eight SIMT warps run the 3x3 taps with the
// arithmetic of the stand-alone depthwise kernel (fmaf per tap in (row, column) order, fp32
// bias add, activation) - a thread walks a strip of one or two columns down the tile so that
// each input row is read from shared memory once, and groups of warps work on different K
// steps at the same time - round each value to TF32 the way the TMA unit rounds the operand
// of the stand-alone projection (nearest even) and store it in the 128-byte-swizzled K-major
// layout; one elected thread issues tcgen05.mma.kind::tf32 against the projection filter
// (streamed per K step by TMA) into a TMEM accumulator; four epilogue warps add the bias,
// apply the activation, add the block's shortcut (optional) and store NHWC rows.
//
// Warps: 0 patch producer, 1 MMA issuer (+ TMEM), 2 filter producer, 3 idle, 4-7 epilogue
// (TMEM lane quarter = warp & 3), 8-15 depthwise.  Every mbarrier wait is bounded and
// reports through the context's error word.  No cluster launch, no multicast.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <string>

#include "gemm_tf32_device.cuh"

int packed_pointwise_filter(tfjs_cuda_ctx* ctx, int32_t filter_id, Buffer* w, int out_c, int in_c,
                            const float** out);

namespace {

constexpr int kDwThreads = 512;
constexpr int kDwWarp0 = 8;          // first depthwise warp
constexpr int kDwWarps = 8;
constexpr int kEpiWarp0 = 4;
constexpr int kDpBarrierBytes = 512;

// Spatial tile of one work item: TN images x TH rows x TW columns of output pixels
// (row-major in that order = rows of the MMA's A operand, at most 128).  A depthwise thread
// owns four channels of a "unit": S adjacent output columns of one image, over RH = TH / RS
// consecutive output rows, which it walks top to bottom so that every input row is loaded
// once and feeds the (up to three) output rows it belongs to from registers.  The units of
// a tile keep WG warps busy; the eight depthwise warps form G = 8 / WG groups that work on
// G consecutive K steps at the same time, each on its own input patch and A stage.
template <int STRIDE_, int TW_, int TH_, int TN_, int S_, int RS_>
struct DpTile {
  static constexpr int STRIDE = STRIDE_, TW = TW_, TH = TH_, TN = TN_, S = S_, RS = RS_;
  static constexpr int PIX = TW * TH * TN;
  static constexpr int IW = (TW - 1) * STRIDE + 3;
  static constexpr int IH = (TH - 1) * STRIDE + 3;
  static constexpr int PATCH_BYTES = IW * IH * TN * 128;
  static constexpr int CB = TW / S;                   // column blocks per tile row
  static constexpr int RH = TH / RS;                  // output rows per unit
  static constexpr int UNITS = CB * RS * TN;
  static constexpr int WG = (UNITS * 8 + 31) / 32;    // warps per group
  static constexpr int G = kDwWarps / WG;             // K steps in flight
  static constexpr int NC = (S - 1) * STRIDE + 3;     // input columns a unit reads
  static constexpr int JN = (RH - 1) * STRIDE + 3;    // input rows a unit reads
  static_assert(PIX <= 128 && TW % S == 0 && TH % RS == 0, "tile shape");
  static_assert(kDwWarps % WG == 0 && G >= 1, "units must split the depthwise warps evenly");
  static_assert(PATCH_BYTES % 128 == 0, "patch size");
};

struct DpArgs {
  const float* dw_w;      // [3][3][C]
  const float* dw_bias;   // [C], one value, or null
  int dw_bias_len;
  ActParams dw_ap;        // relu / relu6 / linear resolved at compile time; others by apply_act
  const float* pw_bias;
  int pw_bias_len;
  ActParams pw_ap;
  const float* residual;  // optional, shaped like the output
  int post_act;
  float* out;
  int batch, in_h, in_w, c, out_h, out_w, pad_t, pad_l;
  int n;                  // projection output channels
  int n_pad, n_mma, n_blk;  // accumulator columns, columns per MMA, MMAs per K sub-step
  int k_steps;
  int tiles_w, tiles_h, tiles_n, total_tiles;
  int patch_stages, a_stages, b_stages, acc_stages;
  int* flag;
};

template <class T, int DW_ACT>
__global__ void __launch_bounds__(kDwThreads, 1)
dw_project_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_b,
                  const DpArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int PS = g.patch_stages, AS = g.a_stages, BS = g.b_stages, ACC = g.acc_stages;
  const uint32_t b_stage_bytes = (uint32_t)g.n_pad * 128u;
  const uint32_t a_base = smem_base;                                   // AS x 16 KB
  const uint32_t b_base = a_base + (uint32_t)AS * A_STAGE_BYTES;       // BS x n_pad x 128
  const uint32_t p_base = b_base + (uint32_t)BS * b_stage_bytes;       // PS x patch
  const uint32_t epi_base = p_base + (uint32_t)PS * T::PATCH_BYTES;    // 4 x 4 KB staging
  // depthwise filter and bias of every channel chunk: [k step][9 taps + bias][32 channels]
  const uint32_t w_base = epi_base + 4u * 4096u;
  const uint32_t bar_base = w_base + (uint32_t)g.k_steps * 1280u;
  // barriers: patch_full[8], patch_empty[8], a_full[8], a_empty[8], b_full[4], b_empty[4],
  // tfull[2], tempty[2], TMEM slot
  auto patch_full = [&](int s) { return bar_base + 8u * s; };
  auto patch_empty = [&](int s) { return bar_base + 8u * (8 + s); };
  auto a_full = [&](int s) { return bar_base + 8u * (16 + s); };
  auto a_empty = [&](int s) { return bar_base + 8u * (24 + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (32 + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (36 + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (40 + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (42 + a); };
  const uint32_t tmem_slot = bar_base + 8u * 44;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 96) {
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_b);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(patch_full(s), 1);
      mbar_init(patch_empty(s), T::WG);   // the warps of the group that read the patch
      mbar_init(a_full(s), T::WG);        // the warps of the group that wrote the A stage
      mbar_init(a_empty(s), 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(b_full(s), 1);
      mbar_init(b_empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
        "r"(512u)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int k_steps = g.k_steps;
  // tile -> (first image, first output row, first output column)
  auto tile_origin = [&](int tile, int& n0, int& oh0, int& ow0) {
    const int tw = tile % g.tiles_w;
    const int rest = tile / g.tiles_w;
    const int th = rest % g.tiles_h;
    n0 = (rest / g.tiles_h) * T::TN;
    oh0 = th * T::TH;
    ow0 = tw * T::TW;
  };

  if (warp == 0) {
    // ------------------------------------------------------ patch producer --
    if (lane == 0) {
      int ps = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < g.total_tiles; tile += gridDim.x) {
        int n0, oh0, ow0;
        tile_origin(tile, n0, oh0, ow0);
        const int ix = ow0 * T::STRIDE - g.pad_l, iy = oh0 * T::STRIDE - g.pad_t;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(patch_empty(ps), phase ^ 1)) {
            atomicExch(g.flag, 1);
            alive = false;
            break;
          }
          mbar_expect_tx(patch_full(ps), T::PATCH_BYTES);
          asm volatile(
              "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
              "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(p_base + (uint32_t)ps * T::PATCH_BYTES),
              "l"(&tm_x), "r"(patch_full(ps)), "r"(ks * 32), "r"(ix), "r"(iy), "r"(n0)
              : "memory");
          if (++ps == PS) { ps = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 2) {
    // ----------------------------------------------------- filter producer --
    if (lane == 0) {
      int bs = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; alive && tile < g.total_tiles; tile += gridDim.x) {
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(b_empty(bs), phase ^ 1)) {
            atomicExch(g.flag, 9);
            alive = false;
            break;
          }
          mbar_expect_tx(b_full(bs), b_stage_bytes);
          for (int j = 0; j < g.n_blk; ++j)
            tma_load_3d(b_base + (uint32_t)bs * b_stage_bytes + (uint32_t)(j * g.n_mma) * 128u,
                        &tm_b, b_full(bs), ks * BK, j * g.n_mma, 0);
          if (++bs == BS) { bs = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer --
    // One thread, a chain of dependent scalar instructions per K step, and only four short
    // MMAs (N <= 256) to hide it behind: the loop is kept to the waits, one add per
    // descriptor, the MMAs and the commits.  The descriptors of all stages and K sub-steps
    // differ only in the start-address field (16-byte units, bits 0-13) of the low word.
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) |
                             ((uint32_t)(g.n_mma >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      const uint64_t proto = desc_k_major(0);
      const uint32_t d_hi = (uint32_t)(proto >> 32);
      const uint32_t a_lo0 = (uint32_t)proto | ((a_base >> 4) & 0x3fffu);
      const uint32_t b_lo0 = (uint32_t)proto | ((b_base >> 4) & 0x3fffu);
      const uint32_t a_inc = A_STAGE_BYTES >> 4, b_inc = b_stage_bytes >> 4;
      const uint32_t kk = (UMMA_K * 4) >> 4;                     // one K sub-step
      const uint32_t j_inc = ((uint32_t)g.n_mma * 128u) >> 4;    // the second MMA's filter rows
      const int n_blk = g.n_blk, n_mma = g.n_mma;
      auto mk = [&](uint32_t lo) { return ((uint64_t)d_hi << 32) | lo; };
      int as = 0, bs = 0;
      uint32_t aph = 0, bph = 0, a_lo = a_lo0, b_lo = b_lo0;
      uint32_t a_full_bar = a_full(0), a_empty_bar = a_empty(0);
      uint32_t b_full_bar = b_full(0), b_empty_bar = b_empty(0);
      bool alive = true;
      int it = 0;
      for (int tile = blockIdx.x; alive && tile < g.total_tiles; tile += gridDim.x, ++it) {
        const int acc = it % ACC;
        const uint32_t aphase = (it / ACC) & 1;
        if (!mbar_wait(tempty_bar(acc), aphase ^ 1)) {
          atomicExch(g.flag, 2);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * g.n_pad);
#pragma unroll 1
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(b_full_bar, bph) || !mbar_wait(a_full_bar, aph)) {
            atomicExch(g.flag, 3);
            alive = false;
            break;
          }
          tc_fence_after();
          if (n_blk == 1) {
            tc_mma_tf32(d_tmem, mk(a_lo), mk(b_lo), idesc, ks != 0 ? 1u : 0u);
            tc_mma_tf32(d_tmem, mk(a_lo + kk), mk(b_lo + kk), idesc, 1u);
            tc_mma_tf32(d_tmem, mk(a_lo + 2 * kk), mk(b_lo + 2 * kk), idesc, 1u);
            tc_mma_tf32(d_tmem, mk(a_lo + 3 * kk), mk(b_lo + 3 * kk), idesc, 1u);
          } else {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc_mma_tf32(d_tmem, mk(a_lo + k * kk), mk(b_lo + k * kk), idesc, (ks | k) != 0 ? 1u : 0u);
              tc_mma_tf32(d_tmem + (uint32_t)n_mma, mk(a_lo + k * kk), mk(b_lo + j_inc + k * kk), idesc,
                          (ks | k) != 0 ? 1u : 0u);
            }
          }
          tc_commit(a_empty_bar);
          tc_commit(b_empty_bar);
          a_lo += a_inc; a_full_bar += 8; a_empty_bar += 8;
          if (++as == AS) { as = 0; aph ^= 1; a_lo = a_lo0; a_full_bar = a_full(0); a_empty_bar = a_empty(0); }
          b_lo += b_inc; b_full_bar += 8; b_empty_bar += 8;
          if (++bs == BS) { bs = 0; bph ^= 1; b_lo = b_lo0; b_full_bar = b_full(0); b_empty_bar = b_empty(0); }
        }
        if (alive) tc_commit(tfull_bar(acc));
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
    // ----------------------------------------------------------- epilogue --
    // Lane = tile row (a pixel).  A 32-column chunk is staged through a swizzled 4 KB tile
    // so that the global accesses run along the channels of a pixel: eight lanes cover one
    // pixel's 128 bytes.
    const int q = warp & 3;
    const uint32_t stage_buf = epi_base + (uint32_t)q * 4096u;
    const uint32_t my_row = stage_buf + (uint32_t)lane * 128u;
    const uint32_t sw = (uint32_t)(lane & 7);
    Tf32Args ea;  // the fields chunk_bias / chunk_math read
    ea.bias = g.pw_bias;
    ea.bias_len = g.pw_bias ? g.pw_bias_len : 0;
    ea.ap = g.pw_ap;
    ea.N = g.n;
    int it = 0;
    for (int tile = blockIdx.x; tile < g.total_tiles; tile += gridDim.x, ++it) {
      int n0, oh0, ow0;
      tile_origin(tile, n0, oh0, ow0);
      const int acc = it % ACC;
      const uint32_t aphase = (it / ACC) & 1;
      // this lane's pixel
      const int r = q * 32 + lane;
      const int tn = r / (T::TH * T::TW);
      const int rr = r - tn * (T::TH * T::TW);
      const int th = rr / T::TW, tw = rr - th * T::TW;
      const int n = n0 + tn, oh = oh0 + th, ow = ow0 + tw;
      const bool ok = r < T::PIX && n < g.batch && oh < g.out_h && ow < g.out_w;
      const int my_off = ok ? ((n * g.out_h + oh) * g.out_w + ow) * g.n : -1;  // < 2^31, checked by the host
      float bj = chunk_bias(ea, 0, lane);
      if (!mbar_wait(tfull_bar(acc), aphase)) {
        if (lane == 0) atomicExch(g.flag, 4);
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < g.n_pad; c0 += 32) {
        if (c0 >= g.n) break;
        const int w = g.n - c0 < 32 ? g.n - c0 : 32;   // valid columns, a multiple of 4
        const int qv = w >> 2;
        // the shortcut's values for this chunk travel while the accumulator is read
        float4 rs[8];
        int offs[8];
        if (qv == 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            offs[j] = __shfl_sync(0xffffffffu, my_off, j * 4 + (lane >> 3));
            rs[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g.residual && offs[j] >= 0)
              rs[j] = __ldg(reinterpret_cast<const float4*>(g.residual + offs[j] + c0 + (lane & 7) * 4));
          }
        }
        float v[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * g.n_pad + c0), v);
        if (c0 + 32 >= g.n) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        chunk_math_dispatch(v, ea, c0, bj);
        if (c0 + 32 < g.n) bj = chunk_bias(ea, c0 + 32, lane);
        __syncwarp();  // the previous chunk's reads of the staging tile are done
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                           my_row + (((uint32_t)j ^ sw) << 4)),
                       "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                       : "memory");
        __syncwarp();
        auto finish = [&](float4 val, float4 res, int o) {
          if (g.residual) {
            // shortcut + branch in the order of the reference's Add, then the trailing
            // activation
            val.x = __fadd_rn(res.x, val.x);
            val.y = __fadd_rn(res.y, val.y);
            val.z = __fadd_rn(res.z, val.z);
            val.w = __fadd_rn(res.w, val.w);
          }
          if (g.post_act == TFJS_CUDA_ACT_RELU) {
            val.x = js_relu(val.x); val.y = js_relu(val.y);
            val.z = js_relu(val.z); val.w = js_relu(val.w);
          } else if (g.post_act == TFJS_CUDA_ACT_RELU6) {
            val.x = js_relu6(val.x); val.y = js_relu6(val.y);
            val.z = js_relu6(val.z); val.w = js_relu6(val.w);
          }
          *reinterpret_cast<float4*>(g.out + o) = val;
        };
        if (qv == 8) {
          // eight lanes cover one pixel's 128 bytes; four pixels per pass
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (offs[j] < 0) continue;
            const uint32_t row = (uint32_t)(j * 4 + (lane >> 3)), vv = (uint32_t)(lane & 7);
            float4 val;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(val.x), "=f"(val.y), "=f"(val.z), "=f"(val.w)
                         : "r"(stage_buf + row * 128u + ((vv ^ (row & 7u)) << 4)));
            finish(val, rs[j], offs[j] + c0 + vv * 4);
          }
        } else {
#pragma unroll 1
          for (int idx = lane; idx < 32 * qv; idx += 32) {
            const int row = idx / qv, vv = idx - row * qv;
            const int off = __shfl_sync(0xffffffffu, my_off, row);
            if (off < 0) continue;
            float4 val;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(val.x), "=f"(val.y), "=f"(val.z), "=f"(val.w)
                         : "r"(stage_buf + (uint32_t)row * 128u +
                               (((uint32_t)vv ^ (uint32_t)(row & 7)) << 4)));
            const int o = off + c0 + vv * 4;
            float4 res = make_float4(0.f, 0.f, 0.f, 0.f);
            if (g.residual) res = __ldg(reinterpret_cast<const float4*>(g.residual + o));
            finish(val, res, o);
          }
        }
      }
    }
  } else if (warp >= kDwWarp0) {
    // ---------------------------------------------------------- depthwise --
    const int dt = threadIdx.x - kDwWarp0 * 32;   // 0 .. 255
    // The filter taps and the bias of all channel chunks go to shared memory once; a K step
    // then reads its ten 16-byte pieces from there instead of waiting on global loads.
    for (int idx = dt; idx < k_steps * 80; idx += kDwWarps * 32) {
      const int ks = idx / 80;
      const int rem = idx - ks * 80;
      const int tap = rem >> 3;
      const int c = ks * 32 + (rem & 7) * 4;
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < g.c) {
        if (tap < 9) {
          t = __ldg(reinterpret_cast<const float4*>(g.dw_w + tap * g.c + c));
        } else if (g.dw_bias_len == 1) {
          const float b0 = __ldg(g.dw_bias);
          t = make_float4(b0, b0, b0, b0);
        } else if (g.dw_bias_len > 1) {
          t = __ldg(reinterpret_cast<const float4*>(g.dw_bias + c));
        }
      }
      asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(w_base + (uint32_t)idx * 16u),
                   "f"(t.x), "f"(t.y), "f"(t.z), "f"(t.w)
                   : "memory");
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");

    const uint32_t smem0 = smem_u32(smem_raw);
    const int gi = dt / (T::WG * 32);             // this thread's group
    const int u = dt - gi * (T::WG * 32);
    const int unit = u >> 3;
    const int c4 = u & 7;
    const bool active = unit < T::UNITS;
    const int cb = unit % T::CB;
    const int rseg = (unit / T::CB) % T::RS;
    const int tn = unit / (T::CB * T::RS);
    const int th0 = rseg * T::RH;
    // this thread's window inside a patch and the A row of its first output
    const uint32_t patch_off =
        (uint32_t)(((tn * T::IH + th0 * T::STRIDE) * T::IW + cb * T::S * T::STRIDE)) * 128u +
        (uint32_t)c4 * 16u;
    const uint32_t arow0 = (uint32_t)((tn * T::TH + th0) * T::TW + cb * T::S);
    // where this thread's outputs go inside an A stage (row r = pixel, 16-byte chunk c4
    // under the 128-byte swizzle): the same for every K step, computed once
    uint32_t a_off[T::RH][T::S];
#pragma unroll
    for (int t = 0; t < T::RH; ++t)
#pragma unroll
      for (int s2 = 0; s2 < T::S; ++s2) {
        const uint32_t r = arow0 + (uint32_t)(t * T::TW + s2);
        a_off[t][s2] = r * 128u + ((((uint32_t)c4) ^ (r & 7u)) << 4);
      }
    // the CTA's K steps in issue order, dealt to the groups in turn
    const int my_tiles = g.total_tiles > (int)blockIdx.x
                             ? (g.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x
                             : 0;
    const long long total_steps = (long long)my_tiles * k_steps;
    int ks = gi % k_steps;
    int ps = gi % PS, as = gi % AS;
    uint32_t pphase = (uint32_t)(gi / PS) & 1u, aphase = (uint32_t)(gi / AS) & 1u;
    bool alive = true;
    for (long long step = gi; alive && step < total_steps; step += T::G) {
      // filter taps and bias of this thread's four channels, as packed pairs for
      // fma.rn.f32x2 (two independent fp32 FMAs per instruction); channels beyond C read
      // zeros here and in the patch, and the projection filter is zero there too
      unsigned long long wv[9][2];
      ulonglong2 bv;
      {
        // plain loads (not asm) so the compiler may schedule them among the arithmetic
        const uint8_t* wk = smem_raw + (w_base - smem0) + (uint32_t)(ks * 80 + c4) * 16u;
        __builtin_assume(__isShared(wk));
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(wk + k * 128);
          wv[k][0] = t.x;
          wv[k][1] = t.y;
        }
        bv = *reinterpret_cast<const ulonglong2*>(wk + 9 * 128);
      }
      if (!mbar_wait(patch_full(ps), pphase)) {
        if (lane == 0) atomicExch(g.flag, 7);
        alive = false;
        break;
      }
      if (!mbar_wait(a_empty(as), aphase ^ 1)) {
        if (lane == 0) atomicExch(g.flag, 8);
        alive = false;
        break;
      }
      if (active) {
        const uint8_t* patch = smem_raw + (p_base - smem0) + (uint32_t)ps * T::PATCH_BYTES + patch_off;
        uint8_t* a_tile = smem_raw + (a_base - smem0) + (uint32_t)as * A_STAGE_BYTES;
        // these are shared-memory addresses: ld.shared / st.shared, not generic accesses
        __builtin_assume(__isShared(patch));
        __builtin_assume(__isShared(a_tile));
        unsigned long long a2[3][T::S][2];
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
          for (int s = 0; s < T::S; ++s) a2[a][s][0] = a2[a][s][1] = 0ull;
#pragma unroll
        for (int j = 0; j < T::JN; ++j) {
          // input row j of the unit's window, loaded once
          unsigned long long xin[T::NC][2];
#pragma unroll
          for (int i = 0; i < T::NC; ++i) {
            const ulonglong2 t =
                *reinterpret_cast<const ulonglong2*>(patch + (j * T::IW + i) * 128);
            xin[i][0] = t.x;
            xin[i][1] = t.y;
          }
          // it is filter row fr of output row t = (j - fr) / STRIDE; an output row receives
          // its filter rows in the order 0, 1, 2 and, within one, the taps left to right:
          // the accumulation order of the reference
#pragma unroll
          for (int fr = 0; fr < 3; ++fr) {
            if (j - fr < 0 || (j - fr) % T::STRIDE != 0 || (j - fr) / T::STRIDE >= T::RH) continue;
            const int t = (j - fr) / T::STRIDE;
            const int a = t % 3;
#pragma unroll
            for (int s = 0; s < T::S; ++s) {
#pragma unroll
              for (int fc = 0; fc < 3; ++fc) {
                asm("fma.rn.f32x2 %0, %1, %2, %0;"
                    : "+l"(a2[a][s][0]) : "l"(xin[s * T::STRIDE + fc][0]), "l"(wv[fr * 3 + fc][0]));
                asm("fma.rn.f32x2 %0, %1, %2, %0;"
                    : "+l"(a2[a][s][1]) : "l"(xin[s * T::STRIDE + fc][1]), "l"(wv[fr * 3 + fc][1]));
              }
            }
            if (fr != 2) continue;
            // output row t is complete: bias, activation, TF32 rounding, A tile
#pragma unroll
            for (int s = 0; s < T::S; ++s) {
              if (g.dw_bias_len) {
                // fp32 bias add, two channels per instruction (rounded like add.rn.f32)
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(a2[a][s][0]) : "l"(bv.x));
                asm("add.rn.f32x2 %0, %0, %1;" : "+l"(a2[a][s][1]) : "l"(bv.y));
              }
              float o[4];
              asm("mov.b64 {%0, %1}, %2;" : "=f"(o[0]), "=f"(o[1]) : "l"(a2[a][s][0]));
              asm("mov.b64 {%0, %1}, %2;" : "=f"(o[2]), "=f"(o[3]) : "l"(a2[a][s][1]));
              a2[a][s][0] = a2[a][s][1] = 0ull;
              uint32_t t32[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                float v = o[k];
                // max.NaN / min.NaN keep a NaN input, as Math.max / Math.min do
                if (DW_ACT == TFJS_CUDA_ACT_RELU) {
                  asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v));
                } else if (DW_ACT == TFJS_CUDA_ACT_RELU6) {
                  asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v));
                  asm("min.NaN.f32 %0, %0, 0f40C00000;" : "+f"(v));
                } else if (DW_ACT != TFJS_CUDA_ACT_LINEAR) {
                  v = apply_act(v, g.dw_ap, ks * 32 + c4 * 4 + k);
                }
                asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(t32[k]) : "f"(v));
              }
              *reinterpret_cast<uint4*>(a_tile + a_off[t][s]) =
                  make_uint4(t32[0], t32[1], t32[2], t32[3]);
            }
          }
        }
      }
      // make the generic-proxy stores visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(a_full(as));
        mbar_arrive(patch_empty(ps));
      }
      // the group's next K step lies G steps ahead (G <= PS, G <= AS)
      ks += T::G;
      while (ks >= k_steps) ks -= k_steps;
      ps += T::G;
      if (ps >= PS) { ps -= PS; pphase ^= 1; }
      as += T::G;
      if (as >= AS) { as -= AS; aphase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(512u)
                 : "memory");
  }
}

template <class T>
int launch_tile(tfjs_cuda_ctx* ctx, const float* x, const float* packed_b, DpArgs& g) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return ctx_fail(ctx, TFJS_CUDA_DRIVER_ERROR, "cuTensorMapEncodeTiled not found");
  CUtensorMap tm_x, tm_b;
  {
    cuuint64_t dims[4] = {(cuuint64_t)g.c, (cuuint64_t)g.in_w, (cuuint64_t)g.in_h,
                          (cuuint64_t)g.batch};
    cuuint64_t strides[3] = {(cuuint64_t)g.c * 4, (cuuint64_t)g.in_w * g.c * 4,
                             (cuuint64_t)g.in_h * g.in_w * g.c * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)T::IW, (cuuint32_t)T::IH, (cuuint32_t)T::TN};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)x, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "depthwise + projection: input map refused");
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)g.c, (cuuint64_t)g.n, 1};
    cuuint64_t strides[2] = {(cuuint64_t)g.c * 4, (cuuint64_t)g.c * g.n * 4};
    cuuint32_t box[3] = {BK, (cuuint32_t)g.n_mma, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    // the packed filter is already rounded to TF32
    if (enc(&tm_b, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3, (void*)packed_b, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "depthwise + projection: filter map refused");
  }
  g.tiles_w = (g.out_w + T::TW - 1) / T::TW;
  g.tiles_h = (g.out_h + T::TH - 1) / T::TH;
  g.tiles_n = (g.batch + T::TN - 1) / T::TN;
  const long long total = (long long)g.tiles_w * g.tiles_h * g.tiles_n;
  if (total > 0x7fffffffLL) return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "depthwise + projection: too large");
  g.total_tiles = (int)total;
  // The kernel spreads a layer over the SMs by spatial tiles only (the two separate kernels
  // also split the channels), so with few tiles (small batches of small maps) most SMs would
  // idle: MobileNetV2 at batch 1 ran 0.51 ms per step this way against 0.32 ms.
  {
    const char* all = getenv("TFJS_CUDA_DW_PROJECT_ALL");
    if ((!all || all[0] == '0') && 4 * total < 3ll * ctx->sm_count)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                      "depthwise + projection: too few tiles to fill the GPU, run as two launches");
  }
  // Shared memory: every group needs a patch and an A stage of its own; what is left goes,
  // in turn, to one more patch (the next K step's input travels while all groups compute),
  // one more A stage, one more filter stage.
  const int b_stage = g.n_pad * 128;
  const int fixed = 1024 + 4 * 4096 + kDpBarrierBytes + g.k_steps * 1280;
  g.patch_stages = T::G;
  g.a_stages = T::G;
  g.b_stages = 2;
  auto need = [&]() {
    return fixed + g.a_stages * A_STAGE_BYTES + g.b_stages * b_stage +
           g.patch_stages * T::PATCH_BYTES;
  };
  if (need() > kMaxSmemBytes)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "depthwise + projection: tile does not fit");
  // (more patches in flight change nothing: with up to six beyond the groups' own the
  // stride-1 layers of MobileNetV2 ran within 1%)
  for (int round = 0; round < 2; ++round) {
    if (g.patch_stages < 8 && need() + T::PATCH_BYTES <= kMaxSmemBytes) g.patch_stages++;
    if (g.a_stages < 8 && need() + A_STAGE_BYTES <= kMaxSmemBytes) g.a_stages++;
    if (g.b_stages < 4 && need() + b_stage <= kMaxSmemBytes) g.b_stages++;
  }
  const int smem = need();
  g.acc_stages = 2 * g.n_pad <= 512 ? 2 : 1;
  const int grid = g.total_tiles < ctx->sm_count ? g.total_tiles : ctx->sm_count;
#define DP_LAUNCH(ACT)                                                                        \
  {                                                                                           \
    auto kern = dw_project_kernel<T, ACT>;                                                    \
    CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                       kMaxSmemBytes));                                       \
    kern<<<grid, kDwThreads, smem, ctx->stream>>>(tm_x, tm_b, g);                             \
  }
  switch (g.dw_ap.act) {
    case TFJS_CUDA_ACT_LINEAR: DP_LAUNCH(TFJS_CUDA_ACT_LINEAR) break;
    case TFJS_CUDA_ACT_RELU: DP_LAUNCH(TFJS_CUDA_ACT_RELU) break;
    case TFJS_CUDA_ACT_RELU6: DP_LAUNCH(TFJS_CUDA_ACT_RELU6) break;
    default: DP_LAUNCH(TFJS_CUDA_ACT_ELU) break;   // resolved per element by apply_act
  }
#undef DP_LAUNCH
  static const std::string name = "dw_project_kernel<stride=" + std::to_string(T::STRIDE) +
                                  ",tile=" + std::to_string(T::TW) + "x" + std::to_string(T::TH) +
                                  "x" + std::to_string(T::TN) + ">";
  LAUNCH_CHECK(ctx, name.c_str());
  return TFJS_CUDA_OK;
}

int fill_simple_act(tfjs_cuda_ctx* ctx, int activation, double alpha, ActParams* ap,
                    const char* who) {
  if (activation < TFJS_CUDA_ACT_LINEAR || activation > TFJS_CUDA_ACT_ELU ||
      activation == TFJS_CUDA_ACT_PRELU)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: activation %d is not supported here", who,
                    activation);
  ap->act = activation;
  ap->gelu_scale = ap->gelu_half = ap->gelu_one = 0.0f;
  ap->gelu_divide = 0;
  ap->prelu_len = 0;
  ap->prelu = nullptr;
  ap->alpha = alpha;
  return TFJS_CUDA_OK;
}

}  // namespace

extern "C" {

int tfjs_cuda_fused_depthwise_project(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* dw,
                                      const tfjs_cuda_conv2d_params* pw, int32_t x_id,
                                      int32_t dw_filter_id, int32_t dw_bias_id,
                                      int32_t pw_filter_id, int32_t pw_bias_id,
                                      int32_t residual_id, int32_t post_activation,
                                      int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (!dw || !pw) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "depthwise + projection: null params");
  const char* who = "depthwise + projection";
  // shapes this kernel takes; everything else is reported as unsupported and the caller
  // launches the two kernels separately
  const bool dw_ok = dw->filter_h == 3 && dw->filter_w == 3 && dw->stride_h == dw->stride_w &&
                     (dw->stride_h == 1 || dw->stride_h == 2) && dw->dilation_h == 1 && dw->dilation_w == 1 &&
                     dw->out_c == dw->in_c && (dw->in_c % 4) == 0 && dw->batch > 0 &&
                     dw->out_h > 0 && dw->out_w > 0 &&
                     (dw->bias_len == 0 || dw->bias_len == 1 || dw->bias_len == dw->in_c);
  const bool pw_ok = pw->filter_h == 1 && pw->filter_w == 1 && pw->stride_h == 1 &&
                     pw->stride_w == 1 && pw->pad_top == 0 && pw->pad_left == 0 &&
                     pw->batch == dw->batch && pw->in_h == dw->out_h && pw->in_w == dw->out_w &&
                     pw->out_h == pw->in_h && pw->out_w == pw->in_w && pw->in_c == dw->out_c &&
                     (pw->out_c % 4) == 0 && pw->out_c >= 8 && pw->out_c <= 512 &&
                     (pw->bias_len == 0 || pw->bias_len == 1 || pw->bias_len == pw->out_c);
  if (!dw_ok || !pw_ok || ctx->math_mode != TFJS_CUDA_MATH_TF32)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: shape or math mode not taken by the fused kernel", who);
  if (post_activation != TFJS_CUDA_ACT_LINEAR && post_activation != TFJS_CUDA_ACT_RELU &&
      post_activation != TFJS_CUDA_ACT_RELU6)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: post activation must be linear, relu or relu6", who);
  // Measured on B200 (MobileNetV2 blocks, batch 256): the fused kernel wins for strided
  // depthwise convolutions (12-44%) and for maps up to 28 x 28 (27-43%); on 56 x 56 and
  // 112 x 112 maps at stride 1 a tile has one to five K steps and its epilogue bounds the
  // kernel (0.27 against 0.25 ms, 0.32 against 0.25 ms), so those stay two launches.
  // TFJS_CUDA_DW_PROJECT_ALL=1 takes every shape the kernel can run.
  if (dw->stride_h == 1 && (dw->out_w > 28 || dw->out_h > 28)) {
    const char* all = getenv("TFJS_CUDA_DW_PROJECT_ALL");
    if (!all || all[0] == '0')
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: large stride-1 maps run as two launches", who);
  }
  const uint64_t nx = (uint64_t)dw->batch * dw->in_h * dw->in_w * dw->in_c;
  const uint64_t ny = (uint64_t)pw->batch * pw->out_h * pw->out_w * pw->out_c;
  if (ny > 0x7fffffffull || nx > 0x7fffffffull)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "depthwise + projection: tensor too large for 32-bit offsets");
  Buffer *x, *wd, *wp, *bd = nullptr, *bp = nullptr, *res = nullptr, *out;
  int rc;
  if ((rc = ctx_get(ctx, x_id, nx * 4, "depthwise + projection x", &x))) return rc;
  if ((rc = ctx_get(ctx, dw_filter_id, (uint64_t)9 * dw->in_c * 4, "depthwise filter", &wd))) return rc;
  if (dw->bias_len && (rc = ctx_get(ctx, dw_bias_id, (uint64_t)dw->bias_len * 4, "depthwise bias", &bd))) return rc;
  if ((rc = ctx_get(ctx, pw_filter_id, (uint64_t)pw->in_c * pw->out_c * 4, "projection filter", &wp))) return rc;
  if (pw->bias_len && (rc = ctx_get(ctx, pw_bias_id, (uint64_t)pw->bias_len * 4, "projection bias", &bp))) return rc;
  if (residual_id && (rc = ctx_get(ctx, residual_id, ny * 4, "depthwise + projection residual", &res))) return rc;
  if ((rc = ctx_get(ctx, out_id, ny * 4, "depthwise + projection out", &out))) return rc;
  if (((uintptr_t)x->ptr & 15) || ((uintptr_t)out->ptr & 15) || (res && ((uintptr_t)res->ptr & 15)))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: unaligned tensor", who);
  DpArgs g;
  if ((rc = fill_simple_act(ctx, dw->activation, dw->leakyrelu_alpha, &g.dw_ap, who))) return rc;
  if ((rc = fill_simple_act(ctx, pw->activation, pw->leakyrelu_alpha, &g.pw_ap, who))) return rc;
  cudaSetDevice(ctx->device);
  const float* packed;
  if ((rc = packed_pointwise_filter(ctx, pw_filter_id, wp, pw->out_c, pw->in_c, &packed))) return rc;
  g.dw_w = (const float*)wd->ptr;
  g.dw_bias = bd ? (const float*)bd->ptr : nullptr;
  g.dw_bias_len = bd ? dw->bias_len : 0;
  g.pw_bias = bp ? (const float*)bp->ptr : nullptr;
  g.pw_bias_len = bp ? pw->bias_len : 0;
  g.residual = res ? (const float*)res->ptr : nullptr;
  g.post_act = post_activation;
  g.out = (float*)out->ptr;
  g.batch = dw->batch; g.in_h = dw->in_h; g.in_w = dw->in_w; g.c = dw->in_c;
  g.out_h = dw->out_h; g.out_w = dw->out_w; g.pad_t = dw->pad_top; g.pad_l = dw->pad_left;
  g.n = pw->out_c;
  g.n_pad = (g.n + 15) / 16 * 16;
  g.n_blk = (g.n_pad + 255) / 256;
  if (g.n_pad % (16 * g.n_blk)) g.n_pad = (g.n_pad + 16 * g.n_blk - 1) / (16 * g.n_blk) * (16 * g.n_blk);
  g.n_mma = g.n_pad / g.n_blk;
  if (g.n_pad > 512) return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: too many output channels", who);
  g.k_steps = (g.c + 31) / 32;
  g.flag = ctx->d_flag;
  const float* xp = (const float*)x->ptr;
  // spatial tile by the width of the output map
  // Depthwise units at stride 1 are one output column wide (four warps per K step, two K
  // steps in flight): MobileNetV2 b256 2.709 ms per step against 2.730 with two-column units
  // (two warps per K step, four in flight), which TFJS_CUDA_DP_TWO_COLUMN_UNITS=1 selects.
  static int two_col = -1;
  if (two_col < 0) {
    const char* e = getenv("TFJS_CUDA_DP_TWO_COLUMN_UNITS");
    two_col = (e && e[0] != '0') ? 1 : 0;
  }
  if (dw->stride_h == 1) {
    if (g.out_w <= 7 && g.out_h <= 7)
      rc = launch_tile<DpTile<1, 7, 7, 2, 1, 1>>(ctx, xp, packed, g);
    else if (g.out_w % 16 == 0 || g.out_w > 56)
      rc = two_col ? launch_tile<DpTile<1, 16, 8, 1, 2, 1>>(ctx, xp, packed, g)
                   : launch_tile<DpTile<1, 16, 8, 1, 1, 1>>(ctx, xp, packed, g);
    else if (g.out_h % 8 == 0 || g.out_h > 28)
      rc = two_col ? launch_tile<DpTile<1, 14, 8, 1, 2, 1>>(ctx, xp, packed, g)
                   : launch_tile<DpTile<1, 14, 8, 1, 1, 1>>(ctx, xp, packed, g);
    else
      rc = two_col ? launch_tile<DpTile<1, 14, 7, 1, 2, 1>>(ctx, xp, packed, g)
                   : launch_tile<DpTile<1, 14, 7, 1, 1, 1>>(ctx, xp, packed, g);
  } else {
    if (g.out_w <= 7 && g.out_h <= 7)
      rc = launch_tile<DpTile<2, 7, 7, 2, 1, 1>>(ctx, xp, packed, g);
    else
      rc = launch_tile<DpTile<2, 14, 8, 1, 2, 2>>(ctx, xp, packed, g);
  }
  if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
  return rc;
}

}  // extern "C"
