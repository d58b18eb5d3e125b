// TF32 GEMM and implicit-GEMM convolution on CTA pairs (tcgen05.mma.cta_group::2).
//
// Two CTAs on neighbouring SMs (a cluster of two) share one 256 x 256 output tile.  Each
// CTA loads its own 128 rows of A and one half (128 rows) of the K-major B tile; the
// tensor cores of both SMs read both halves of B, so a K step pulls 32 KB per SM from L2
// instead of the 48 KB a single CTA needs for a 128 x 256 tile, and the shared-memory
// write traffic of the TMA unit drops by the same third.  The accumulator of CTA r (rows
// 128 r .. 128 r + 127 of the tile, all 256 columns) lives in that CTA's tensor memory.
//
// Roles per CTA (320 threads):
//   warp 0      TMA producer: loads this CTA's A rows and B half into its own shared
//               memory; the bytes are counted on the full-barrier of the LEADER CTA (rank
//               0 of the pair), which is what the MMA issuer waits on.  No multicast.
//   warp 1      leader only: one lane issues the cta_group::2 MMAs and commits them to
//               the empty / accumulator-full barriers of both CTAs; in both CTAs this warp
//               owns the tensor-memory allocation.
//   warps 2-9   epilogue: tcgen05.ld of the CTA's own accumulator, bias + activation,
//               swizzled staging tile, bulk tensor store; the accumulator is handed back
//               with an arrive on the leader's barrier (a remote arrive for the peer).
// Every wait is bounded; on giving up a role records a code in the context's error word
// and drains, and both CTAs meet at a cluster barrier before either releases tensor
// memory or exits, so no signal ever targets shared memory of a CTA that has left.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <string>

#include "gemm_tf32_device.cuh"

namespace {

// BN = 256: two accumulator stages of 256 columns, so the epilogue of one tile runs under the
// main loop of the next.  BN = 384 (256 x 384 tiles, two N = 192 MMAs per K slice, one
// accumulator of 384 columns): for outputs whose tiles all run at once, where the wider tile
// turns 1.3 waves of 256 x 256 tiles into one wave and pulls 20% less from L2 per flop.
// EW epilogue warps (8 or 16: two or four per TMEM lane quarter), one 4 KB staging tile
// each; the pipeline gets the stages that fit beside them (6 or 5; 4 at BN = 384)
template <int EW, int BN>
struct PairCfg {
  static constexpr int B_STAGE_BYTES = (BN / 2) * BK * 4;   // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int ACC = BN == 256 ? 2 : 1;              // accumulator stages
  static constexpr int STAGES =
      (kMaxSmemBytes - 1024 - kBarrierBytes - EW * 4096) / STAGE_BYTES;
  static constexpr int THREADS = 64 + EW * 32;
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EW * 4096 + kBarrierBytes;
  static_assert(BN == 256 || BN == 384, "pair kernel tile width");
  static_assert(STAGES >= 4 && 2 * STAGES + 2 * ACC + 1 <= kBarrierBytes / 8, "pair kernel layout");
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// Loads whose completion is counted on a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* tm,
                                                 uint32_t bar_cluster, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(tm), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_pair(uint32_t dst, const CUtensorMap* tm,
                                                     uint32_t bar_cluster, int c, int w, int h,
                                                     int n, uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.im2col.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(tm), "r"(bar_cluster), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ void tc_mma_tf32_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the
// MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}

// A_MODE 0: A tiles by tiled TMA ([batch][M][K] map, 128-row boxes); 2: TMA im2col over NHWC x.
// GROUP: several products share A (PairGroupMaps); g.tiles_n counts the column tiles of all
// members side by side and tiles_n_each those of one member.
template <int A_MODE, int EW, int GROUP, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((PairCfg<EW, BN>::THREADS), 1)
gemm_tf32_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                      const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_c,
                      const __grid_constant__ PairGroupMaps grp, const Tf32Args g,
                      const int tiles_n_each) {
  using Cfg = PairCfg<EW, BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC = Cfg::ACC;
  constexpr int kPairBStageBytes = Cfg::B_STAGE_BYTES;
  constexpr int kPairStageBytes = Cfg::STAGE_BYTES;
  constexpr int EPI_STEP = (EW / 4) * 32;   // columns between the chunks one warp takes
  constexpr int MMA_N = BN == 256 ? 256 : 192;   // BN = 384: two MMAs side by side
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + STAGES * A_STAGE_BYTES;
  const uint32_t epi_base = b_base + STAGES * kPairBStageBytes;
  const uint32_t bar_base = epi_base + (uint32_t)EW * 4096u;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + ACC + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 2 * ACC);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();      // 0 = leader
  const int pair = (int)(blockIdx.x >> 1);
  const int npairs = (int)(gridDim.x >> 1);

  if (threadIdx.x == 32) {
    prefetch_tensormap(&tm_a);
    if (GROUP) {
      for (int i = 0; i < grp.count; ++i) {
        prefetch_tensormap(&grp.b[i]);
        prefetch_tensormap(&grp.c[i]);
      }
    } else {
      prefetch_tensormap(&tm_b);
      prefetch_tensormap(&tm_c);
    }
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);    // the leader's expect_tx arrival (used in the leader only)
      mbar_init(empty_bar(s), 1);   // one multicast commit per phase
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * EW);  // every epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile(
        "tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
        "r"(512u)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // barriers of both CTAs initialised, tensor memory allocated
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int k_steps = g.k_steps;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer --
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = pair; alive && tile < g.total_tiles; tile += npairs) {
        int nt = tile % g.tiles_n;
        const int rest = tile / g.tiles_n;
        const int mt = rest % g.tiles_m;
        const int bz = rest / g.tiles_m;
        const CUtensorMap* map_b = &tm_b;
        if (GROUP) {
          const int member = nt / tiles_n_each;
          nt -= member * tiles_n_each;
          map_b = &grp.b[member];
        }
        const int m0 = mt * 256 + (int)rank * 128;
        // this CTA's rows of the B tile: half of each MMA's N
        const int n0 = nt * BN + (int)rank * (MMA_N / 2);
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if (A_MODE == 2) {
          const int ow = m0 % g.conv.out_w;
          const int t = m0 / g.conv.out_w;
          pix_w = ow * g.conv.s_w - g.conv.pad_l;
          pix_h = (t % g.conv.out_h) * g.conv.s_h - g.conv.pad_t;
          pix_n = t / g.conv.out_h;
        }
        // (filter row, filter column, channel chunk) of the im2col walk, stepped per K step
        int cc = 0, fr = 0, fc = 0;
        const int cc_end = g.chunks_per_tap * BK;
        const int bz_a = bz % g.batch_a, bz_b = bz % g.batch_b;
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1)) {
            atomicExch(g.flag, 1);
            alive = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2u * (uint32_t)kPairStageBytes);
          const uint32_t fb = map_to_rank(full_bar(stage), 0);
          if (A_MODE == 0) {
            tma_load_3d_pair(a_base + stage * A_STAGE_BYTES, &tm_a, fb, ks * BK, m0, bz_a);
          } else {
            tma_load_im2col_pair(a_base + stage * A_STAGE_BYTES, &tm_a, fb, cc, pix_w, pix_h,
                                 pix_n, (uint16_t)(fc * g.conv.d_w), (uint16_t)(fr * g.conv.d_h));
            cc += BK;
            if (cc >= cc_end) { cc = 0; if (++fc == g.conv.f_w) { fc = 0; ++fr; } }
          }
          tma_load_3d_pair(b_base + stage * kPairBStageBytes, map_b, fb, ks * BK, n0, bz_b);
          if (BN == 384)
            tma_load_3d_pair(b_base + stage * kPairBStageBytes + (MMA_N / 2) * BK * 4, map_b, fb,
                             ks * BK, n0 + MMA_N, bz_b);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (leader CTA) --
    if (rank == 0 && lane == 0) {
      // instruction descriptor: D = f32, A = B = tf32, both K-major, N = MMA_N, M = 256
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(MMA_N >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      // the descriptors of all stages and K sub-steps differ only in the start-address
      // field of the low word (16-byte units): running values, one add per MMA
      const uint64_t a_proto = desc_k_major(a_base), b_proto = desc_k_major(b_base);
      const uint32_t a_hi = (uint32_t)(a_proto >> 32), a_lo0 = (uint32_t)a_proto;
      const uint32_t b_hi = (uint32_t)(b_proto >> 32), b_lo0 = (uint32_t)b_proto;
      auto mk = [](uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | lo; };
      constexpr uint32_t kk = (UMMA_K * 4) >> 4;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      int it = 0;
      for (int tile = pair; alive && tile < g.total_tiles; tile += npairs, ++it) {
        const int acc = it % ACC;
        const uint32_t aphase = (it / ACC) & 1;
        if (!mbar_wait(tempty_bar(acc), aphase ^ 1)) {
          atomicExch(g.flag, 2);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(full_bar(stage), phase)) {
            atomicExch(g.flag, 3);
            alive = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            tc_mma_tf32_pair(d_tmem, mk(a_hi, a_lo + k * kk), mk(b_hi, b_lo + k * kk), idesc,
                             (ks | k) != 0 ? 1u : 0u);
            if (BN == 384)
              tc_mma_tf32_pair(d_tmem + MMA_N, mk(a_hi, a_lo + k * kk),
                               mk(b_hi, b_lo + (((MMA_N / 2) * BK * 4) >> 4) + k * kk), idesc,
                               (ks | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(stage));
          a_lo += A_STAGE_BYTES >> 4;
          b_lo += kPairBStageBytes >> 4;
          if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
        }
        if (alive) tc_commit_pair(tfull_bar(acc));
      }
    }
  } else {
    // ----------------------------------------------------------- epilogue --
    // Warp w reads TMEM lane quarter w & 3 (32 rows of this CTA's 128) and every second
    // (EW = 8) or fourth (EW = 16) 32-column chunk of the tile; a chunk goes through a swizzled 4 KB staging tile and
    // leaves as one bulk tensor store, clipped at the tensor's edge by the TMA unit.
    const int q = warp & 3;
    const int part = (warp - 2) >> 2;
    const uint32_t stage_buf = epi_base + (uint32_t)(warp - 2) * 4096u;
    const uint32_t my_row = stage_buf + (uint32_t)lane * 128u;
    const uint32_t sw = (uint32_t)(lane & 7);
    uint32_t leader_tempty[ACC];
#pragma unroll
    for (int a = 0; a < ACC; ++a) leader_tempty[a] = map_to_rank(tempty_bar(a), 0);
    int it = 0;
    for (int tile = pair; tile < g.total_tiles; tile += npairs, ++it) {
      int nt = tile % g.tiles_n;
      const int rest = tile / g.tiles_n;
      const int mt = rest % g.tiles_m;
      const int bz = rest / g.tiles_m;
      const CUtensorMap* map_c = &tm_c;
      const float* bias = g.bias;
      if (GROUP) {
        const int member = nt / tiles_n_each;
        nt -= member * tiles_n_each;
        map_c = &grp.c[member];
        bias = grp.bias[member];
      }
      const int acc = it % ACC;
      const uint32_t aphase = (it / ACC) & 1;
      float bj = chunk_bias(g, nt * BN + part * 32, lane, bias);
      if (!mbar_wait(tfull_bar(acc), aphase)) {
        if (lane == 0) atomicExch(g.flag, 4);
        break;
      }
      tc_fence_after();
      const int m_base = mt * 256 + (int)rank * 128 + q * 32;
      const bool rows_ok = m_base < g.M;
      bool released = false;
#pragma unroll 1
      for (int c0 = part * 32; c0 < BN; c0 += EPI_STEP) {
        const int n0 = nt * BN + c0;
        if (n0 >= g.N) break;
        float v[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), v);
        if (c0 + EPI_STEP >= BN || n0 + EPI_STEP >= g.N) {
          // last read of this accumulator by this warp: hand it back early
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_tempty[acc]);
          released = true;
        }
        chunk_math_dispatch(v, g, n0, bj, false, bias);
        if (c0 + EPI_STEP < BN) bj = chunk_bias(g, n0 + EPI_STEP, lane, bias);
        // the bulk store that last used the staging tile must have finished reading it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                           my_row + (((uint32_t)j ^ sw) << 4)),
                       "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0 && rows_ok) {
          if (g.out_perm == 0) {
            asm volatile(
                "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                ::"l"(map_c), "r"(stage_buf), "r"(n0), "r"(m_base), "r"(bz)
                : "memory");
          } else {
            // 4-D map over the permuted result: (d, s, h, b) for the heads split,
            // (d, h, s, b) for the merge; the 32 x 32 tile is a box of it either way
            int c0p, c1, c2, c3;
            if (g.out_perm == 1) {
              c2 = n0 / g.perm_d; c0p = n0 - c2 * g.perm_d;
              c3 = m_base / g.perm_p; c1 = m_base - c3 * g.perm_p;
            } else {
              c0p = n0; c2 = m_base;
              c3 = bz / g.perm_p; c1 = bz - c3 * g.perm_p;
            }
            asm volatile(
                "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                ::"l"(map_c), "r"(stage_buf), "r"(c0p), "r"(c1), "r"(c2), "r"(c3)
                : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tempty[acc]);
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // Neither CTA may release tensor memory or leave while its partner can still signal
  // its barriers or while MMAs that write its tensor memory are in flight.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(512u)
                 : "memory");
  }
}

template <int A_MODE, int EW, int GROUP, int BN = 256>
int launch_pair(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                const CUtensorMap& tm_c, const PairGroupMaps* maps, Tf32Args& g) {
  auto kern = gemm_tf32_pair_kernel<A_MODE, EW, GROUP, BN>;
  using C = PairCfg<EW, BN>;
  static bool configured[64] = {false};  // per device ordinal
  if (ctx->device >= 64 || !configured[ctx->device]) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       C::SMEM_BYTES));
    if (ctx->device < 64) configured[ctx->device] = true;
  }
  const int tiles_n_each = (g.N + BN - 1) / BN;
  g.tiles_n = tiles_n_each * (GROUP ? maps->count : 1);
  g.total_tiles = g.tiles_m * g.tiles_n * g.total_tiles;  // total_tiles held the batch
  const int pairs_max = ctx->sm_count / 2;
  const int pairs = g.total_tiles < pairs_max ? g.total_tiles : pairs_max;
  static const PairGroupMaps no_group = {};
  kern<<<2 * pairs, C::THREADS, C::SMEM_BYTES, ctx->stream>>>(tm_a, tm_b, tm_c,
                                                             GROUP ? *maps : no_group, g,
                                                             tiles_n_each);
  static const std::string name =
      "gemm_tf32_pair_kernel<A_MODE=" + std::to_string(A_MODE) + ",EW=" + std::to_string(EW) +
      ",GROUP=" + std::to_string(GROUP) + (BN == 256 ? "" : ",BN=" + std::to_string(BN)) + ">";
  LAUNCH_CHECK(ctx, name.c_str());
  return TFJS_CUDA_OK;
}

}  // namespace

int launch_gemm_tf32_pair(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
                          const CUtensorMap& tm_c, Tf32Args& g, bool im2col) {
  static int ew = -1;  // epilogue warps per CTA (tuning knob)
  if (ew < 0) ew = getenv("TFJS_CUDA_PAIR_EPILOGUE_WARPS") ? atoi(getenv("TFJS_CUDA_PAIR_EPILOGUE_WARPS")) : 8;
  // The erf GELU epilogue is some 24 instructions per element with chains through the
  // special-function unit: four warps per TMEM lane quarter hide them better than two
  // ([8192, 768] x [768, 3072]: 71.2 against 73.7 us; the plain epilogue prefers two: 61.9
  // against 63.2).
  if (ew == 16 || g.ap.act == TFJS_CUDA_ACT_GELU_ERF) {
    if (im2col) return launch_pair<2, 16, 0>(ctx, tm_a, tm_b, tm_c, nullptr, g);
    return launch_pair<0, 16, 0>(ctx, tm_a, tm_b, tm_c, nullptr, g);
  }
  if (im2col) return launch_pair<2, 8, 0>(ctx, tm_a, tm_b, tm_c, nullptr, g);
  return launch_pair<0, 8, 0>(ctx, tm_a, tm_b, tm_c, nullptr, g);
}

int launch_gemm_tf32_pair_wide(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a,
                               const CUtensorMap& tm_b, const CUtensorMap& tm_c, Tf32Args& g) {
  return launch_pair<0, 16, 0, 384>(ctx, tm_a, tm_b, tm_c, nullptr, g);
}

int launch_gemm_tf32_pair_group(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a,
                                const PairGroupMaps& maps, Tf32Args& g) {
  return launch_pair<0, 8, 1>(ctx, tm_a, maps.b[0], maps.c[0], &maps, g);
}
