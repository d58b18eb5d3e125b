// TF32 GEMM and implicit-GEMM convolution on the sm_100a tensor cores.
//
// One persistent CTA per SM walks 128 x BN output tiles.  Warp roles:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A and B tiles
//               into 128-byte-swizzled shared-memory stages (no multicast).
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma.kind::tf32 from
//               shared-memory descriptors into a TMEM accumulator; owns the TMEM
//               allocation.
//   warps 2-9   epilogue: tcgen05.ld the accumulator (32 lanes x 32 columns per
//               load), add the bias, apply the activation, stage through shared
//               memory and store whole rows (NHWC / row-major).
//   warps 10-13 (convolution only) A gatherers: 16-byte loads of the im2col rows
//               straight from the NHWC input (zeros for taps outside the image),
//               rounded to TF32 and stored in the same swizzled layout TMA would
//               produce.
// Convolutions with at most 128 output channels and a long K run with the operands
// swapped (A_MODE 4 / 5): the packed filter is the MMA's 128-row operand and 256
// output pixels its N axis, because a tcgen05.mma takes the same time at N = 64 as
// at N = 256; the epilogue transposes the [channel][pixel] accumulator while staging.
// Two TMEM accumulators alternate so the epilogue of tile i overlaps the main
// loop of tile i+1.  Every mbarrier wait is bounded: when it gives up the kernel
// records a code in the context's error word and drains.
//
// Operand formats.  A is K-major (rows of K contiguous floats).  B is either
// K-major ([N][K]: transposed operands and packed weights) or MN-major ([K][N]
// row-major, consumed directly through the MN-major shared-memory descriptor).
// The tensor core reads the upper 19 bits of each fp32 word, so every operand
// is rounded to TF32 before it reaches shared memory: by the TMA unit (TFLOAT32
// tensor maps), by the gather warps, or when weights are packed.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include "gemm_tf32_device.cuh"

namespace {

// Input patches of the staged-row gather that may be in flight (a tile's rows are fetched
// this many tiles ahead, less one): the copies come from DRAM, and with 13-30 KB per patch
// it takes several of them to cover its latency.
constexpr int kMaxPatchBufs = 8;

// RES: the epilogue adds a residual tile that the TMA unit prefetches into the
// staging tile of the next chunk (two staging tiles per warp, and at BN = 256 one
// pipeline stage fewer to make room for them).
template <int BN, int A_MODE = 0, int RES = 0, int EW = 8>
struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 4;
  // staging tiles per epilogue warp: two (a warp fills one while the TMA unit still
  // drains the other, and the residual epilogue prefetches into the other one), one at
  // BN = 256 without residual, in the scalar-gather mode and with sixteen warps
  static constexpr int EPI_BUFS =
      RES ? 2 : (((BN >= 256 || A_MODE == 3) || EW == 16) ? 1 : 2);
  // pipeline stages: as many as fit beside the staging tiles, up to 4 / 5 / 6 / 8 by tile
  // width; the scalar-gather mode keeps room for its tables and the staged input rows
  static constexpr int STAGES_WANTED = BN >= 256 ? 4 : (BN >= 128 ? 5 : (BN >= 64 ? 6 : 8));
  static constexpr int STAGES_FIT =
      (kMaxSmemBytes - 1024 - kBarrierBytes - EW * EPI_BUFS * 4096) /
      (A_STAGE_BYTES + B_STAGE_BYTES);
  static constexpr int STAGES =
      A_MODE == 3 ? (BN <= 64 ? 3 : 2)
                  : (STAGES_FIT < STAGES_WANTED ? STAGES_FIT : STAGES_WANTED);
  // TMEM accumulator stages.  A tile's accumulator is handed back and forth through
  // two barriers whose wake-ups cost more than a short tile's MMAs, so narrow tiles
  // (few K steps in practice) keep more tiles in flight: 256 columns at BN <= 128.
  static constexpr int ACC_STAGES = BN >= 256 ? 2 : 256 / BN;
  static constexpr int TMEM_COLS = ACC_STAGES * BN;
  // epilogue work split: P warps per TMEM lane quarter, C 32-column chunks per tile
  static constexpr int EPI_P = EW / 4, EPI_C = BN / 32;
  static constexpr int EPI_G = EPI_C >= EPI_P ? 1 : EPI_P / EPI_C;  // tiles alternate over G groups
  static constexpr int EPI_STEP = (EPI_C >= EPI_P ? EPI_P : EPI_C) * 32;
  static constexpr int EPI_ARRIVALS = 4 * (EPI_C >= EPI_P ? EPI_P : EPI_C);
  static constexpr int THREADS = 64 + EW * 32 + ((A_MODE == 1 || A_MODE == 3) ? 128 : 0);
  static constexpr int SMEM_BYTES =
      1024 + STAGES * (A_STAGE_BYTES + B_STAGE_BYTES) + kBarrierBytes + EW * EPI_BUFS * 4096 +
      (A_MODE == 3 ? kTapTableEntries * 4 + 4 * 512 : 0);  // tap table + 4 row tables
};

template <int BN, int B_MN, int A_MODE, int RES, int EW = 8, int SK = 0>
__global__ void __launch_bounds__((Cfg<BN, A_MODE, RES, EW>::THREADS), 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap tm_a,
                 const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c,
                 const __grid_constant__ CUtensorMap tm_r, const Tf32Args g) {
  using C = Cfg<BN, A_MODE, RES, EW>;
  constexpr int STAGES = C::STAGES;
  // A_MODE 4 / 5: operands swapped for narrow outputs (N <= 128).  A tcgen05.mma takes the
  // same time whatever its N, so the weights become the 128-row operand and 256 output
  // pixels the N axis: half the MMAs per pixel.  The accumulator is then [channel][pixel]
  // and the epilogue transposes it back while staging.  LOAD is how the pixel operand is
  // fetched (0 tiled TMA, 2 TMA im2col), as in modes 0 and 2.
  constexpr bool SWAP = A_MODE >= 4;
  constexpr int LOAD = SWAP ? (A_MODE == 4 ? 0 : 2) : A_MODE;
  constexpr int kTileRows = SWAP ? 256 : BM;    // output pixels (GEMM rows) per tile
  static_assert(!SWAP || (BN == 256 && !RES && !B_MN), "swapped operands: 256-pixel tiles only");
  static_assert(!SK || (BN == 256 && !RES && !SWAP && EW == 8 && (A_MODE == 0 || A_MODE == 2)),
                "K-split tail: plain 128 x 256 tiles only");
  constexpr int kGatherWarp0 = 2 + EW;          // first gather warp (A_MODE 1 and 3)
  constexpr int kGatherThread0 = 64 + EW * 32;  // its first thread
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = smem_base;
  const uint32_t b_base = smem_base + STAGES * A_STAGE_BYTES;
  const uint32_t epi_base = b_base + STAGES * C::B_STAGE_BYTES;  // 4 KB staging tiles
  const uint32_t bar_base = epi_base + (uint32_t)EW * C::EPI_BUFS * 4096u;
  // barrier layout: full[STAGES], empty[STAGES], tfull[ACC], tempty[ACC], tmem slot
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  constexpr int ACC = C::ACC_STAGES;
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + ACC + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 2 * ACC);
  // residual prefetch barriers: one per epilogue warp and staging tile
  auto res_bar = [&](int w, uint32_t b) { return bar_base + 320u + 8u * (2u * w + b); };  // up to 32

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 32) {
    if (A_MODE == 0 || A_MODE == 2 || SWAP) prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
    if (g.c_tma) prefetch_tensormap(&tm_c);
    if (RES && g.residual) prefetch_tensormap(&tm_r);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), (A_MODE == 1 || A_MODE == 3) ? 1 + 4 : 1);  // producer + 4 gather warps
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < ACC; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), C::EPI_ARRIVALS);  // one arrival per epilogue warp of a tile
    }
    if (RES)
      for (int w = 0; w < EW; ++w) {
        mbar_init(res_bar(w, 0), 1);
        mbar_init(res_bar(w, 1), 1);
      }
    if (A_MODE == 3) {  // "patch landed" barriers (this mode has no residual epilogue)
      for (int b = 0; b < kMaxPatchBufs; ++b) mbar_init(res_bar(b >> 1, b & 1), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile(
        "tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
        "r"((uint32_t)C::TMEM_COLS)
        : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  const uint32_t tap_table = bar_base + (uint32_t)kBarrierBytes;  // A_MODE 3 only
  if (A_MODE == 3 && warp >= kGatherWarp0) {
    // entry k: filter row and column of the tap in the top byte (4 bits each, 0xff =
    // padding beyond K), element offset of (tap, channel) from the tile pixel's top-left
    // input element in the low 24 bits
    for (int k = threadIdx.x - kGatherThread0; k < g.k_steps * BK; k += 128) {
      uint32_t e = 0xff000000u;  // padding beyond K, always zero
      if (g.patch_cap > 0) {
        // staged-row mode: filter row in the top byte (31 = padding), offset of the
        // element from the row's window start inside the patch in the low 24 bits
        const int fwc = g.conv.f_w * g.conv.in_c;
        e = 31u << 24;
        if (k < g.conv.f_h * fwc) {
          const int fr = k / fwc;
          e = ((uint32_t)fr << 24) | (uint32_t)(fr * g.conv.d_h * g.patch_pitch + (k - fr * fwc));
        }
      } else if (k < g.conv.f_h * g.conv.f_w * g.conv.in_c) {
        const int tap = k / g.conv.in_c, c = k - tap * g.conv.in_c;
        const int fr = tap / g.conv.f_w, fc = tap - fr * g.conv.f_w;
        e = ((uint32_t)fr << 28) | ((uint32_t)fc << 24) |
            (uint32_t)((fr * g.conv.d_h * g.conv.in_w + fc * g.conv.d_w) * g.conv.in_c + c);
      }
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(tap_table + 4u * k), "r"(e) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
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
      WorkIter wi;
      wi.init(g, SK != 0);
      int tile, ks0, ks1;
      while (alive && wi.next(tile, ks0, ks1)) {
        const int nt = tile % g.tiles_n;
        const int rest = tile / g.tiles_n;
        const int mt = rest % g.tiles_m;
        const int bz = rest / g.tiles_m;
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if (LOAD == 2) {
          const int m0 = mt * kTileRows;
          const int ow = m0 % g.conv.out_w;
          const int t = m0 / g.conv.out_w;
          pix_w = ow * g.conv.s_w - g.conv.pad_l;
          pix_h = (t % g.conv.out_h) * g.conv.s_h - g.conv.pad_t;
          pix_n = t / g.conv.out_h;
        }
        // im2col walk over (filter row, filter column, channel chunk): divided once per
        // item, stepped per K step (this thread's instructions are the producer's latency)
        int cc = 0, fr = 0, fc = 0;
        if (LOAD == 2) {
          const int tap = ks0 / g.chunks_per_tap;
          cc = (ks0 - tap * g.chunks_per_tap) * BK;
          fr = tap / g.conv.f_w;
          fc = tap - fr * g.conv.f_w;
        }
        const int cc_end = g.chunks_per_tap * BK;
        const int bz_a = bz % g.batch_a, bz_b = bz % g.batch_b;
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1)) {
            atomicExch(g.flag, 1);
            alive = false;
            break;
          }
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, ((A_MODE == 1 || A_MODE == 3) ? 0 : A_STAGE_BYTES) + C::B_STAGE_BYTES);
          if (SWAP) {
            // weights (all N <= 128 rows, zero-filled beyond) into the 128-row operand
            // slot, 256 pixels into the wide one
            tma_load_3d(a_base + stage * A_STAGE_BYTES, &tm_b, fb, ks * BK, 0, bz_b);
            const uint32_t pdst = b_base + stage * C::B_STAGE_BYTES;
            if (LOAD == 0) {
              tma_load_3d(pdst, &tm_a, fb, ks * BK, mt * kTileRows, bz_a);
            } else {
              tma_load_im2col(pdst, &tm_a, fb, cc, pix_w, pix_h, pix_n,
                              (uint16_t)(fc * g.conv.d_w), (uint16_t)(fr * g.conv.d_h));
              cc += BK;
              if (cc >= cc_end) { cc = 0; if (++fc == g.conv.f_w) { fc = 0; ++fr; } }
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
            continue;
          }
          if (A_MODE == 0) {
            tma_load_3d(a_base + stage * A_STAGE_BYTES, &tm_a, fb, ks * BK, mt * BM, bz_a);
          } else if (A_MODE == 2) {
            // im2col load: 128 consecutive output pixels starting at the tile's
            // first one, 32 channels of filter tap (fr, fc)
            tma_load_im2col(a_base + stage * A_STAGE_BYTES, &tm_a, fb, cc, pix_w, pix_h, pix_n,
                            (uint16_t)(fc * g.conv.d_w), (uint16_t)(fr * g.conv.d_h));
            cc += BK;
            if (cc >= cc_end) { cc = 0; if (++fc == g.conv.f_w) { fc = 0; ++fr; } }
          }
          const uint32_t bdst = b_base + stage * C::B_STAGE_BYTES;
          if (!B_MN) {
            tma_load_3d(bdst, &tm_b, fb, ks * BK, nt * BN, bz_b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_3d(bdst + j * 4096, &tm_b, fb, nt * BN + j * 32, ks * BK, bz_b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=tf32, A K-major, B per template,
      // N = BN, M = 128.
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) |
                             ((uint32_t)B_MN << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      const uint64_t a_proto = desc_k_major(a_base);
      const uint64_t b_proto = B_MN ? desc_mn_major(b_base) : desc_k_major(b_base);
      const uint32_t a_hi = (uint32_t)(a_proto >> 32), a_lo0 = (uint32_t)a_proto;
      const uint32_t b_hi = (uint32_t)(b_proto >> 32), b_lo0 = (uint32_t)b_proto;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      WorkIter wi;
      wi.init(g, SK != 0);
      int tile, ks0, ks1;
      while (alive && wi.next(tile, ks0, ks1)) {
        const int it = wi.idx - 1;
        const int acc = it % ACC;
        const uint32_t aphase = (it / ACC) & 1;
        if (!mbar_wait(tempty_bar(acc), aphase ^ 1)) {
          atomicExch(g.flag, 2);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int ks = ks0; ks < ks1; ++ks) {
          if (!mbar_wait(full_bar(stage), phase)) {
            atomicExch(g.flag, 3);
            alive = false;
            break;
          }
          tc_fence_after();
          // the descriptors of all stages and K sub-steps differ only in the start-address
          // field of the low word (16-byte units): one add each
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = ((uint64_t)a_hi << 32) | (a_lo + (uint32_t)(k * ((UMMA_K * 4) >> 4)));
            const uint64_t bd = ((uint64_t)b_hi << 32) |
                                (b_lo + (uint32_t)(k * (B_MN ? (1024 >> 4) : ((UMMA_K * 4) >> 4))));
            tc_mma_tf32(d_tmem, ad, bd, idesc, ((ks - ks0) | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          a_lo += A_STAGE_BYTES >> 4;
          b_lo += C::B_STAGE_BYTES >> 4;
          if (++stage == STAGES) { stage = 0; phase ^= 1; a_lo = a_lo0; b_lo = b_lo0; }
        }
        if (alive) tc_commit(tfull_bar(acc));
      }
    }
  } else if (warp < kGatherWarp0) {
    // ----------------------------------------------------------- epilogue --
    // Each warp owns 32 rows of the tile.  A 32-column chunk comes out of TMEM
    // with one row per lane; it is staged through a swizzled 4 KB shared-memory
    // tile so that the global stores run along rows: full 128-byte lines, or one
    // contiguous run when the tile spans the whole row.
    // EW / 4 warps share each TMEM lane quarter and take the chunks of a tile in turn
    // (tiles in turn when a tile has fewer chunks than that).
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;  // which of the quarter's warps this is
    if (SWAP) {
      // Accumulator rows are output channels (lane = channel 32 q + lane), columns are
      // the tile's 256 pixels.  A chunk is 32 pixels x 32 channels: the lane adds its
      // channel's bias, applies the activation and writes its 32 values down a column of
      // the staging tile, which is then a [pixel][channel] box for the bulk store.
      const int ch0 = q * 32;
      const bool ch_ok = ch0 < g.N;
      float bch = 0.0f;
      if (ch_ok && g.bias_len == 1) bch = __ldg(g.bias);
      else if (ch_ok && g.bias_len > 1 && ch0 + lane < g.N) bch = __ldg(g.bias + ch0 + lane);
      const uint32_t stage_buf = epi_base + (uint32_t)(warp - 2) * (C::EPI_BUFS * 4096u);
      const uint32_t col = (((uint32_t)lane >> 2)), word = ((uint32_t)lane & 3u) * 4u;
      int it = 0;
      for (int tile = blockIdx.x; tile < g.total_tiles; tile += gridDim.x, ++it) {
        const int rest = tile / g.tiles_n;
        const int mt = rest % g.tiles_m;
        const int bz = rest / g.tiles_m;
        const int acc = it % ACC;
        const uint32_t aphase = (it / ACC) & 1;
        if (!mbar_wait(tfull_bar(acc), aphase)) {
          if (lane == 0) atomicExch(g.flag, 4);
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c0 = part * 32; c0 < 256; c0 += C::EPI_P * 32) {
          const int m0 = mt * 256 + c0;
          if (!ch_ok || m0 >= g.M) continue;
          float v[32];
          tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), v);
          if (g.bias_len != 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], bch);
          }
          chunk_math_dispatch(v, g, 0, 0.0f, true);
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            asm volatile("st.shared.f32 [%0], %1;" ::"r"(
                             stage_buf + (uint32_t)j * 128u + ((col ^ (uint32_t)(j & 7)) << 4) + word),
                         "f"(v[j])
                         : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile(
                "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                ::"l"(&tm_c), "r"(stage_buf), "r"(ch0), "r"(m0), "r"(bz)
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        // every chunk of this tile has left TMEM
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
    constexpr int kChunk0Mod = C::EPI_C >= C::EPI_P ? C::EPI_P : C::EPI_C;
    const int my_c0 = (part % kChunk0Mod) * 32;       // first chunk this warp takes
    const int my_group = part / kChunk0Mod;           // tiles with it % EPI_G == my_group
    const uint32_t stage_base = epi_base + (uint32_t)(warp - 2) * (C::EPI_BUFS * 4096u);
    uint32_t ebuf = 0;
    const uint32_t sw = (uint32_t)(lane & 7);
    const bool vec4 = (g.N & 3) == 0;
    // Residual prefetch (RES): a cursor runs one chunk ahead of the loop below over
    // the same (tile, chunk) sequence; lane 0 asks the TMA unit for the residual
    // 32 x 32 tile of that chunk, into the staging tile the chunk will use.
    const int first_c0 = my_c0;
    int p_tile = blockIdx.x, p_it = 0, p_c0 = first_c0;
    uint32_t rphase = 0;       // bit b: parity the next wait on res_bar(b) uses
    bool res_issued = false;   // a load into the current staging tile is in flight
    auto prefetch_residual = [&](uint32_t b) -> bool {
      if (!g.residual) return false;  // this instantiation also serves as the two-buffer epilogue
      while (p_tile < g.total_tiles) {
        const int n0 = (p_tile % g.tiles_n) * BN + p_c0;
        if (!(C::EPI_G > 1 && (p_it % C::EPI_G) != my_group) && p_c0 < BN && n0 < g.N) {
          const int rest = p_tile / g.tiles_n;
          const int m_base = (rest % g.tiles_m) * BM + q * 32;
          p_c0 += C::EPI_STEP;
          if (m_base >= g.M) return false;  // rows beyond the tensor: nothing to add
          if (lane == 0) {
            const uint32_t bar = res_bar(warp - 2, b);
            mbar_expect_tx(bar, 4096u);
            tma_load_3d(stage_base + b * 4096u, &tm_r, bar, n0, m_base, rest / g.tiles_m);
          }
          return true;
        }
        p_tile += gridDim.x;
        ++p_it;
        p_c0 = first_c0;
      }
      return false;
    };
    if (RES) res_issued = prefetch_residual(0);
    WorkIter wi;
    wi.init(g, SK != 0);
    int tile, ks0, ks1;
    while (wi.next(tile, ks0, ks1)) {
      const int it = wi.idx - 1;
      // K-split tail: `sk_tail` items hold the later K steps of a tile another CTA
      // started: the raw accumulator goes to the workspace.  `sk_head` items hold the
      // first K steps of a tile that the following CTAs finish: their partial sums are
      // added, in CTA order, before bias and activation.
      const bool sk_tail = SK && ks0 > 0;
      const bool sk_head = SK && ks0 == 0 && ks1 < g.k_steps;
      constexpr int kSkChunks = C::EPI_C / C::EPI_P;  // chunks a warp handles per tile
      int peer0 = 0, peer1 = 0;                        // CTAs [peer0, peer1) finish this tile
      if (sk_head) {
        const long long T = (long long)g.sk_tiles * g.k_steps;
        const long long tile_end = (long long)(tile - wi.sk_base + 1) * g.k_steps;
        peer0 = (int)blockIdx.x + 1;
        peer1 = peer0;
        while (peer1 < (int)gridDim.x && T * peer1 / (long long)gridDim.x < tile_end) ++peer1;
      }
      const int nt = tile % g.tiles_n;
      const int rest = tile / g.tiles_n;
      const int mt = rest % g.tiles_m;
      const int bz = rest / g.tiles_m;
      const int acc = it % ACC;
      const uint32_t aphase = (it / ACC) & 1;
      if (C::EPI_G > 1 && (it % C::EPI_G) != my_group) continue;  // another warp's tile
      // the first chunk's bias travels while the tile's MMAs finish
      float bj = chunk_bias(g, nt * BN + my_c0, lane);
      if (!mbar_wait(tfull_bar(acc), aphase)) {
        if (lane == 0) atomicExch(g.flag, 4);
        // let the residual load in flight land before this CTA's shared memory goes
        if (RES && res_issued) mbar_wait(res_bar(warp - 2, ebuf), (rphase >> ebuf) & 1u);
        res_issued = false;
        break;
      }
      tc_fence_after();
      if (SK && sk_head) {
        // the part of each peer's partial tile that the same warp of that CTA wrote is
        // complete once its flag is up (bounded wait; code 7 on giving up)
        if (lane == 0) {
          for (int p = peer0; p < peer1; ++p) {
            const unsigned* f = g.sk_flags + p * EW + (warp - 2);
            const long long t0 = clock64();
            unsigned seen, n = 0;
            for (;;) {
              asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
              if (seen != 0) break;
              if ((++n & 0xff) == 0 && clock64() - t0 > kWaitCycles) {
                atomicExch(g.flag, 7);
                break;
              }
            }
          }
        }
        __syncwarp();
      }
      const int m_base = mt * BM + q * 32;
      const int rows_valid = g.M - m_base < 32 ? g.M - m_base : 32;
      float* cbase = g.c + ((long long)bz * g.M + m_base) * g.N;
      const float* rbase = g.residual + ((long long)bz * g.M + m_base) * g.N;
      bool released = false;
#pragma unroll 1
      for (int c0 = my_c0; c0 < BN; c0 += C::EPI_STEP) {
        const int n0 = nt * BN + c0;
        if (n0 >= g.N) break;
        const int w = g.N - n0 < 32 ? g.N - n0 : 32;
        float v[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), v);
        if (c0 + C::EPI_STEP >= BN || n0 + C::EPI_STEP >= g.N) {
          // last read of this accumulator by this warp: hand it back early
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
          released = true;
        }
        if (SK && (sk_tail || sk_head)) {
          const int ci = (c0 - my_c0) / C::EPI_STEP;
          if (sk_tail) {
            float* dst = g.sk_ws +
                         (((size_t)blockIdx.x * EW + (warp - 2)) * kSkChunks + ci) * 1024 + lane;
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(dst + j * 32, v[j]);
            continue;
          }
          for (int p = peer0; p < peer1; ++p) {
            const float* src =
                g.sk_ws + (((size_t)p * EW + (warp - 2)) * kSkChunks + ci) * 1024 + lane;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(v[j], __ldcg(src + j * 32));
          }
        }
        chunk_math_dispatch(v, g, n0, bj);
        if (c0 + C::EPI_STEP < BN) bj = chunk_bias(g, n0 + C::EPI_STEP, lane);  // next chunk's
        const uint32_t stage_buf = stage_base + ebuf * 4096u;
        const uint32_t my_row = stage_buf + (uint32_t)lane * 128u;
        if (RES) {
          // out = post(residual + act(acc + bias)): the residual tile sits in this
          // chunk's staging tile in the layout the result is staged in, so each lane
          // reads the 16-byte pieces it is about to overwrite.
          if (res_issued) {
            const bool ok = mbar_wait(res_bar(warp - 2, ebuf), (rphase >> ebuf) & 1u);
            rphase ^= 1u << ebuf;
            if (!ok && lane == 0) atomicExch(g.flag, 5);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 rs;
              asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(rs.x), "=f"(rs.y), "=f"(rs.z), "=f"(rs.w)
                           : "r"(my_row + (((uint32_t)j ^ sw) << 4)));
              v[4 * j] = __fadd_rn(rs.x, v[4 * j]);
              v[4 * j + 1] = __fadd_rn(rs.y, v[4 * j + 1]);
              v[4 * j + 2] = __fadd_rn(rs.z, v[4 * j + 2]);
              v[4 * j + 3] = __fadd_rn(rs.w, v[4 * j + 3]);
            }
            if (g.post_act == TFJS_CUDA_ACT_RELU) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = js_relu(v[j]);
            } else if (g.post_act == TFJS_CUDA_ACT_RELU6) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = js_relu6(v[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                             my_row + (((uint32_t)j ^ sw) << 4)),
                         "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                         : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (rows_valid > 0) {
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                  ::"l"(&tm_c), "r"(stage_buf), "r"(n0), "r"(m_base), "r"(bz)
                  : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            // the other staging tile is free once the store before this one has read it
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          }
          __syncwarp();  // no lane writes that tile before lane 0 has seen it free
          ebuf ^= 1;
          res_issued = prefetch_residual(ebuf);
          continue;
        }
        if (C::EPI_BUFS == 2) ebuf ^= 1;
        if (g.c_tma) {
          // the bulk store that last used this staging tile must have finished reading it
          if (lane == 0) {
            if (C::EPI_BUFS == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                           my_row + (((uint32_t)j ^ sw) << 4)),
                       "f"(v[4 * j]), "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                       : "memory");
        if (g.c_tma) {
          // one bulk tensor store per 32 x 32 chunk; rows / columns beyond the
          // tensor are clipped by the TMA unit
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0 && rows_valid > 0) {
            if (g.out_perm == 0) {
              asm volatile(
                  "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                  ::"l"(&tm_c), "r"(stage_buf), "r"(n0), "r"(m_base), "r"(bz)
                  : "memory");
            } else {
              // 4-D map over the permuted result: (d, s, h, b) for the heads split,
              // (d, h, s, b) for the merge; the 32 x 32 tile is a box of it either way
              int c0, c1, c2, c3;
              if (g.out_perm == 1) {
                c2 = n0 / g.perm_d; c0 = n0 - c2 * g.perm_d;
                c3 = m_base / g.perm_p; c1 = m_base - c3 * g.perm_p;
              } else {
                c0 = n0; c2 = m_base;
                c3 = bz / g.perm_p; c1 = bz - c3 * g.perm_p;
              }
              asm volatile(
                  "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                  ::"l"(&tm_c), "r"(stage_buf), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                  : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          continue;
        }
        __syncwarp();
        if (rows_valid > 0) {
          if (vec4) {
            const int qv = w >> 2;
            const int total = rows_valid * qv;
            for (int idx = lane; idx < total; idx += 32) {
              int row, vv;
              if (qv == 8) { row = idx >> 3; vv = idx & 7; }
              else { row = idx / qv; vv = idx - row * qv; }
              float4 val;
              asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(val.x), "=f"(val.y), "=f"(val.z), "=f"(val.w)
                           : "r"(stage_buf + (uint32_t)row * 128u +
                                 (((uint32_t)vv ^ (uint32_t)(row & 7)) << 4)));
              const long long off = (long long)row * g.N + n0 + vv * 4;
              if (g.residual) {
                // residual tile read along rows, like the stores: a + b in the order
                // of the reference's Add(shortcut, branch), then the trailing Relu
                const float4 rs = __ldg(reinterpret_cast<const float4*>(rbase + off));
                val.x = __fadd_rn(rs.x, val.x);
                val.y = __fadd_rn(rs.y, val.y);
                val.z = __fadd_rn(rs.z, val.z);
                val.w = __fadd_rn(rs.w, val.w);
                if (g.post_act == TFJS_CUDA_ACT_RELU) {
                  val.x = js_relu(val.x); val.y = js_relu(val.y);
                  val.z = js_relu(val.z); val.w = js_relu(val.w);
                } else if (g.post_act == TFJS_CUDA_ACT_RELU6) {
                  val.x = js_relu6(val.x); val.y = js_relu6(val.y);
                  val.z = js_relu6(val.z); val.w = js_relu6(val.w);
                }
              }
              *reinterpret_cast<float4*>(cbase + off) = val;
            }
          } else {
            const int total = rows_valid * w;
            for (int idx = lane; idx < total; idx += 32) {
              const int row = idx / w, col = idx - row * w;
              float val;
              asm volatile("ld.shared.f32 %0, [%1];"
                           : "=f"(val)
                           : "r"(stage_buf + (uint32_t)row * 128u +
                                 ((((uint32_t)col >> 2) ^ (uint32_t)(row & 7)) << 4) +
                                 ((uint32_t)col & 3u) * 4u));
              const long long off = (long long)row * g.N + n0 + col;
              if (g.residual) {
                val = __fadd_rn(__ldg(rbase + off), val);
                if (g.post_act == TFJS_CUDA_ACT_RELU) val = js_relu(val);
                else if (g.post_act == TFJS_CUDA_ACT_RELU6) val = js_relu6(val);
              }
              cbase[off] = val;
            }
          }
        }
      }
      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      if (SK && sk_tail) {
        // publish this warp's part of the partial tile
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          unsigned* f = g.sk_flags + (size_t)blockIdx.x * EW + (warp - 2);
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(f), "r"(1u) : "memory");
        }
      }
      if (SK && sk_head) {
        // every chunk of the peers' partials has been read: lower their flags for the
        // next launch
        __syncwarp();
        if (lane == 0)
          for (int p = peer0; p < peer1; ++p) g.sk_flags[p * EW + (warp - 2)] = 0u;
      }
    }
    if (g.c_tma && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }  // !SWAP
  } else if (A_MODE == 1) {
    // ----------------------------------------------------- im2col gatherers --
    // Thread r owns row r of every A tile.  Each K step it reads 32 channels of
    // one filter tap (8 x 16 bytes) into registers, rounds them to TF32
    // (nearest-even, the rounding the TMA unit applies to the other operands) and
    // stores them in the 128-byte-swizzled layout.  The loads of step i+1 are
    // issued before the stores of step i, so two steps are in flight per thread.
    const int r = threadIdx.x - kGatherThread0;
    const ConvGeo& cv = g.conv;
    const uint32_t row_off = (uint32_t)r * 128u;
    const uint32_t sw = (uint32_t)(r & 7);
    // iterator over (tile, k step) in issue order
    int tile = blockIdx.x, ks = 0;
    bool row_ok = false;
    int b = 0, r_base = 0, c_base = 0;
    auto enter_tile = [&]() {
      const int mt = (tile / g.tiles_n) % g.tiles_m;
      const int m = mt * BM + r;
      row_ok = tile < g.total_tiles && m < g.M;
      if (row_ok) {
        const int t = fast_div(m, g.ow_mul, g.ow_shr);
        const int ow = m - t * cv.out_w;
        b = fast_div(t, g.oh_mul, g.oh_shr);
        const int oh = t - b * cv.out_h;
        r_base = oh * cv.s_h - cv.pad_t;
        c_base = ow * cv.s_w - cv.pad_l;
      }
    };
    auto load_step = [&](float4* v) {
      const int tap = ks / g.chunks_per_tap;
      const int cc = (ks - tap * g.chunks_per_tap) * BK;
      const int fr = tap / cv.f_w, fc = tap - fr * cv.f_w;
      const int ri = r_base + fr * cv.d_h;
      const int ci = c_base + fc * cv.d_w;
      const bool ok = row_ok && ri >= 0 && ri < cv.in_h && ci >= 0 && ci < cv.in_w;
      const float* src = g.x + (((long long)b * cv.in_h + ri) * cv.in_w + ci) * cv.in_c + cc;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        v[j] = (ok && cc + j * 4 < cv.in_c) ? __ldg(reinterpret_cast<const float4*>(src) + j)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto advance = [&]() {
      if (++ks == k_steps) {
        ks = 0;
        tile += gridDim.x;
        enter_tile();
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    float4 cur[8], nxt[8];
    enter_tile();
    if (tile < g.total_tiles) load_step(nxt);
    while (tile < g.total_tiles) {
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
      advance();
      if (tile < g.total_tiles) load_step(nxt);
      if (!mbar_wait(empty_bar(stage), phase ^ 1)) {
        atomicExch(g.flag, 5);
        break;
      }
      const uint32_t dst = a_base + stage * A_STAGE_BYTES + row_off;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t w0, w1, w2, w3;
        asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w0) : "f"(cur[j].x));
        asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w1) : "f"(cur[j].y));
        asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w2) : "f"(cur[j].z));
        asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w3) : "f"(cur[j].w));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                         dst + (((uint32_t)j ^ sw) << 4)),
                     "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                     : "memory");
      }
      // make the generic-proxy stores visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();  // every lane fenced its stores
      if (lane == 0) mbar_arrive(full_bar(stage));
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  }

  else if (A_MODE == 3 && warp >= kGatherWarp0) {
    // ------------------------------------------- scalar im2col gatherers --
    // For inputs whose channel count is not a multiple of 4 (the 3-channel stems).
    // Warp gw builds rows 32 gw .. 32 gw + 31 of the A tile.  Within a K step lane l
    // owns column l: consecutive lanes read consecutive (tap, channel) elements of one
    // pixel's patch, which are contiguous in memory along a filter row, and write one
    // 128-byte row of the tile without bank conflicts.  k -> (tap, channel, offset)
    // comes from the tap table, the geometry of the warp's 32 rows from a small
    // per-warp table rebuilt at every tile; taps outside the image read as zero and
    // values are rounded to TF32.
    const int gw = warp - kGatherWarp0;
    const ConvGeo& cv = g.conv;
    const uint32_t row_tab = tap_table + (uint32_t)kTapTableEntries * 4u + (uint32_t)gw * 512u;
    const uint32_t kpos = ((uint32_t)lane & 3u) * 4u;
    const uint32_t kchunk = (uint32_t)lane >> 2;
    int tile = blockIdx.x, ks = 0;
    auto enter_tile = [&]() {
      long long base = 0;
      int r0 = -(1 << 28), c0 = 0;  // rows beyond M fail every bounds test
      if (tile < g.total_tiles) {
        const int mt = (tile / g.tiles_n) % g.tiles_m;
        const int m = mt * BM + gw * 32 + lane;
        if (m < g.M) {
          const int t = fast_div(m, g.ow_mul, g.ow_shr);
          const int ow = m - t * cv.out_w;
          const int b = fast_div(t, g.oh_mul, g.oh_shr);
          const int oh = t - b * cv.out_h;
          r0 = oh * cv.s_h - cv.pad_t;
          c0 = ow * cv.s_w - cv.pad_l;
          base = (((long long)b * cv.in_h + r0) * cv.in_w + c0) * cv.in_c;
        }
      }
      __syncwarp();  // every lane is done with the previous tile's table
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_tab + (uint32_t)lane * 16u),
                   "r"((uint32_t)(unsigned long long)base),
                   "r"((uint32_t)((unsigned long long)base >> 32)), "r"(r0), "r"(c0)
                   : "memory");
      __syncwarp();
    };
    if (g.patch_cap > 0) {
      // Staged rows.  The input rows a tile touches are whole image rows; bulk copies
      // bring them into a shared-memory patch (two buffers: the rows of the next tile
      // travel while this tile is expanded) whose rows carry zeroed margins for the
      // horizontal padding, plus one all-zero row that stands in for rows above or
      // below the image.  K is the filter in storage order (row, column, channel), so a
      // thread (one tile row) copies runs of filter_w * in_c contiguous floats: one
      // scalar load per element, one 16-byte store per four, no per-element bounds
      // test.
      const uint32_t patch_base = tap_table + (uint32_t)kTapTableEntries * 4u + 4u * 512u;
      const int rowlen = cv.in_w * cv.in_c;  // floats per image row
      const int pitch = g.patch_pitch;
      const int fwc = cv.f_w * cv.in_c;
      const int nb = g.patch_bufs;
      const int total_rows = cv.batch * cv.in_h;
      const int zero_off = g.patch_rows * pitch;
      {
        const uint32_t z = 0u;
        for (uint32_t o = (uint32_t)(threadIdx.x - kGatherThread0) * 16u;
             o < (uint32_t)nb * (uint32_t)g.patch_cap;
             o += 128u * 16u)
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(patch_base + o), "r"(z)
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      // first global image row (b * in_h + r) and row count of a tile's patch
      auto patch_rows = [&](int t, int* r_lo) -> int {
        const int mt = (t / g.tiles_n) % g.tiles_m;
        const int m0 = mt * BM;
        const int m1 = (m0 + BM - 1 < g.M ? m0 + BM - 1 : g.M - 1);
        const int t0 = fast_div(m0, g.ow_mul, g.ow_shr);  // (b, oh) flattened
        const int t1 = fast_div(m1, g.ow_mul, g.ow_shr);
        const int b0 = fast_div(t0, g.oh_mul, g.oh_shr), b1 = fast_div(t1, g.oh_mul, g.oh_shr);
        const int lo = b0 * cv.in_h + (t0 - b0 * cv.out_h) * cv.s_h - cv.pad_t;
        const int hi = b1 * cv.in_h + (t1 - b1 * cv.out_h) * cv.s_h - cv.pad_t +
                       (cv.f_h - 1) * cv.d_h;
        const int a = lo < 0 ? 0 : lo;
        const int b = hi > total_rows - 1 ? total_rows - 1 : hi;
        *r_lo = a;
        int n = b - a + 1;
        if (n < 0) n = 0;
        if (n > g.patch_rows) {  // the host's sizing guarantees this never holds
          atomicExch(g.flag, 7);
          n = g.patch_rows;
        }
        return n;
      };
      auto issue_patch = [&](int t, uint32_t buf) {  // the first gather warp, all lanes
        const uint32_t bar = res_bar(buf >> 1, buf & 1u);
        int r_lo;
        const int n = patch_rows(t, &r_lo);
        if (lane == 0) {
          if (n <= 0) mbar_arrive(bar);
          else mbar_expect_tx(bar, (uint32_t)n * (uint32_t)rowlen * 4u);
        }
        __syncwarp();
        // one bulk copy per image row, spread over the lanes
        const uint32_t dst0 = patch_base + buf * (uint32_t)g.patch_cap + (uint32_t)g.patch_ml * 4u;
        for (int r = lane; r < n; r += 32)
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(dst0 + (uint32_t)(r * pitch) * 4u),
              "l"(g.x + (long long)(r_lo + r) * rowlen), "r"((uint32_t)rowlen * 4u), "r"(bar)
              : "memory");
      };
      const bool leader = gw == 0;
      if (leader)
        for (int j = 0; j < nb - 1; ++j)
          if (tile + j * (int)gridDim.x < g.total_tiles) issue_patch(tile + j * gridDim.x, j);
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      const uint32_t smem0 = smem_u32(smem_raw);
      const uint32_t my_row = (uint32_t)(gw * 32 + lane) * 128u;
      const uint32_t sw = (uint32_t)lane & 7u;
      for (int t = 0; tile < g.total_tiles && alive; tile += gridDim.x, ++t) {
        const uint32_t buf = (uint32_t)(t % nb);
        // every gather thread is done with the buffer of tile t - 1: refill it with the
        // patch of tile t + nb - 1
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (leader && tile + (nb - 1) * (int)gridDim.x < g.total_tiles)
          issue_patch(tile + (nb - 1) * gridDim.x, (uint32_t)((t + nb - 1) % nb));
        // this thread's tile row: where its window starts inside the patch
        int pbase = 0, r0 = -(1 << 28);
        {
          int r_lo;
          patch_rows(tile, &r_lo);
          const int mt = (tile / g.tiles_n) % g.tiles_m;
          const int m = mt * BM + gw * 32 + lane;
          if (m < g.M) {
            const int tt = fast_div(m, g.ow_mul, g.ow_shr);
            const int ow = m - tt * cv.out_w;
            const int b = fast_div(tt, g.oh_mul, g.oh_shr);
            const int oh = tt - b * cv.out_h;
            r0 = oh * cv.s_h - cv.pad_t;
            pbase = (b * cv.in_h + r0 - r_lo) * pitch + g.patch_ml +
                    (ow * cv.s_w - cv.pad_l) * cv.in_c;
          }
        }
        if (!mbar_wait(res_bar(buf >> 1, buf & 1u), (uint32_t)(t / nb) & 1u)) {
          atomicExch(g.flag, 8);
          alive = false;
          break;
        }
        // plain shared-memory loads (not asm) so the compiler may batch them
        const float* pf = reinterpret_cast<const float*>(
            smem_raw + (patch_base + buf * (uint32_t)g.patch_cap - smem0));
        // filter rows of this thread's window that lie inside the image
        uint32_t vmask = 0;
        for (int fr = 0; fr < cv.f_h; ++fr)
          if ((unsigned)(r0 + fr * cv.d_h) < (unsigned)cv.in_h) vmask |= 1u << fr;
        const bool interior = __all_sync(0xffffffffu, vmask == (1u << cv.f_h) - 1u);
        const uint4* tp = reinterpret_cast<const uint4*>(smem_raw + (tap_table - smem0));
        const int k_real = cv.f_h * fwc;
        for (ks = 0; ks < k_steps; ++ks) {
          float v[32];
          if (interior && (ks + 1) * BK <= k_real) {
            // every element of this step exists for every row of the warp
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const uint4 t4 = tp[ks * 8 + q4];
              v[4 * q4] = pf[pbase + (int)(t4.x & 0xffffffu)];
              v[4 * q4 + 1] = pf[pbase + (int)(t4.y & 0xffffffu)];
              v[4 * q4 + 2] = pf[pbase + (int)(t4.z & 0xffffffu)];
              v[4 * q4 + 3] = pf[pbase + (int)(t4.w & 0xffffffu)];
            }
          } else {
            // rows above / below the image and the padding beyond K read the zero row
            auto pick = [&](uint32_t e) -> float {
              const bool ok = (vmask >> (e >> 24)) & 1u;
              return pf[ok ? pbase + (int)(e & 0xffffffu) : zero_off];
            };
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4) {
              const uint4 t4 = tp[ks * 8 + q4];
              v[4 * q4] = pick(t4.x);
              v[4 * q4 + 1] = pick(t4.y);
              v[4 * q4 + 2] = pick(t4.z);
              v[4 * q4 + 3] = pick(t4.w);
            }
          }
          if (!mbar_wait(empty_bar(stage), phase ^ 1)) {
            atomicExch(g.flag, 6);
            alive = false;
            break;
          }
          const uint32_t dst = a_base + stage * A_STAGE_BYTES + my_row;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t w0, w1, w2, w3;
            asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w0) : "f"(v[4 * c8]));
            asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w1) : "f"(v[4 * c8 + 1]));
            asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w2) : "f"(v[4 * c8 + 2]));
            asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w3) : "f"(v[4 * c8 + 3]));
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(
                             dst + (((uint32_t)c8 ^ sw) << 4)),
                         "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                         : "memory");
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();  // every lane fenced its stores
          if (lane == 0) mbar_arrive(full_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // patches may still be in flight after an early exit: let them land
      if (!alive && leader && lane == 0)
        for (int b = 0; b < nb; ++b) mbar_wait(res_bar(b >> 1, b & 1), 0);
    } else {
    auto load_step = [&](float* v) {
      uint32_t e;
      asm volatile("ld.shared.b32 %0, [%1];" : "=r"(e) : "r"(tap_table + 4u * (ks * BK + lane)));
      const bool kval = (e >> 24) != 0xffu;
      const int dr = (int)(e >> 28) * cv.d_h, dc = (int)((e >> 24) & 15u) * cv.d_w;
      const float* src = g.x + (e & 0xffffffu);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        uint32_t lo, hi;
        int r0, c0;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(lo), "=r"(hi), "=r"(r0), "=r"(c0)
                     : "r"(row_tab + (uint32_t)i * 16u));
        const long long base = (long long)(((unsigned long long)hi << 32) | lo);
        const bool ok = kval && (unsigned)(r0 + dr) < (unsigned)cv.in_h &&
                        (unsigned)(c0 + dc) < (unsigned)cv.in_w;
        v[i] = ok ? __ldg(src + base) : 0.0f;
      }
    };
    auto advance = [&]() {
      if (++ks == k_steps) {
        ks = 0;
        tile += gridDim.x;
        enter_tile();
      }
    };
    int stage = 0;
    uint32_t phase = 0;
    float cur[32], nxt[32];
    enter_tile();
    if (tile < g.total_tiles) load_step(nxt);
    while (tile < g.total_tiles) {
#pragma unroll
      for (int j = 0; j < 32; ++j) cur[j] = nxt[j];
      advance();
      // the loads of step i+1 are issued before the stores of step i
      if (tile < g.total_tiles) load_step(nxt);
      if (!mbar_wait(empty_bar(stage), phase ^ 1)) {
        atomicExch(g.flag, 6);
        break;
      }
      const uint32_t dst = a_base + stage * A_STAGE_BYTES + (uint32_t)gw * 4096u + kpos;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        uint32_t w;
        asm("cvt.rn.tf32.f32 %0, %1;" : "=r"(w) : "f"(cur[i]));
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(
                         dst + (uint32_t)i * 128u + ((kchunk ^ (uint32_t)(i & 7)) << 4)),
                     "r"(w)
                     : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();  // every lane fenced its stores
      if (lane == 0) mbar_arrive(full_bar(stage));
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    }  // register-held gather
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)C::TMEM_COLS)
                 : "memory");
  }
}

// ---- host side ---------------------------------------------------------------
// 3-D map over [batch][rows][inner] floats; box = [1][box_rows][32].
int make_map(tfjs_cuda_ctx* ctx, CUtensorMap* tm, const float* base, uint64_t inner,
             uint64_t rows, uint64_t batch, uint64_t row_stride_elems,
             uint64_t batch_stride_elems, uint32_t box_rows,
             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return ctx_fail(ctx, TFJS_CUDA_DRIVER_ERROR, "cuTensorMapEncodeTiled not found");
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {row_stride_elems * 4, batch_stride_elems * 4};
  if (batch == 1) strides[1] = rows * row_stride_elems * 4;
  cuuint32_t box[3] = {BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  // TFLOAT32 element type: the TMA unit rounds each fp32 word to TF32 (nearest
  // even) on its way into shared memory.  With the plain FLOAT32 type the tensor
  // core would truncate the low 13 mantissa bits, a bias toward zero that
  // compounds layer after layer.
  static int plain = -1;
  if (plain < 0) plain = getenv("TFJS_CUDA_TMA_FLOAT32") ? 1 : 0;  // debugging knob
  CUresult r = enc(tm, plain ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32,
                   3, (void*)base, dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return ctx_fail(ctx, TFJS_CUDA_DRIVER_ERROR,
                    "cuTensorMapEncodeTiled failed (%d): inner=%llu rows=%llu batch=%llu "
                    "row_stride=%llu",
                    (int)r, (unsigned long long)inner, (unsigned long long)rows,
                    (unsigned long long)batch, (unsigned long long)row_stride_elems);
  return TFJS_CUDA_OK;
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// im2col map over NHWC x: dims (C, W, H, N); 32 channels x 128 pixels per load;
// the pixel bounding box starts at -pad and ends where the last filter tap still
// fits, and pixels are traversed with the convolution stride.
bool make_im2col_map(CUtensorMap* tm, const float* x, const ConvGeo& cv, int pixels = BM) {
  static EncodeIm2colFn enc = nullptr;
  if (!enc) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
      return false;
    enc = (EncodeIm2colFn)p;
  }
  const int eff_w = (cv.f_w - 1) * cv.d_w, eff_h = (cv.f_h - 1) * cv.d_h;
  // right/bottom padding implied by the output size
  const int pad_r = (cv.out_w - 1) * cv.s_w + eff_w + 1 - cv.in_w - cv.pad_l;
  const int pad_b = (cv.out_h - 1) * cv.s_h + eff_h + 1 - cv.in_h - cv.pad_t;
  int lower[2] = {-cv.pad_l, -cv.pad_t};
  int upper[2] = {pad_r - eff_w, pad_b - eff_h};
  // the box must yield exactly out_w x out_h base pixels
  if ((cv.in_w + upper[0] - lower[0] - 1) / cv.s_w + 1 != cv.out_w ||
      (cv.in_h + upper[1] - lower[1] - 1) / cv.s_h + 1 != cv.out_h)
    return false;
  for (int i = 0; i < 2; ++i)
    if (lower[i] < -128 || lower[i] > 127 || upper[i] < -128 || upper[i] > 127) return false;
  if (eff_w > 255 || eff_h > 255 || cv.s_w > 8 || cv.s_h > 8 || (cv.in_c & 3)) return false;
  cuuint64_t dims[4] = {(cuuint64_t)cv.in_c, (cuuint64_t)cv.in_w, (cuuint64_t)cv.in_h,
                        (cuuint64_t)cv.batch};
  cuuint64_t strides[3] = {(cuuint64_t)cv.in_c * 4, (cuuint64_t)cv.in_w * cv.in_c * 4,
                           (cuuint64_t)cv.in_h * cv.in_w * cv.in_c * 4};
  cuuint32_t estr[4] = {1, (cuuint32_t)cv.s_w, (cuuint32_t)cv.s_h, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 4, (void*)x, dims, strides, lower,
                   upper, BK, (cuuint32_t)pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, int B_MN, int A_MODE, int RES = 0, int EW = 8, int SK = 0>
int launch_cfg(tfjs_cuda_ctx* ctx, const CUtensorMap& tm_a, const CUtensorMap& tm_b,
               const CUtensorMap& tm_c, const CUtensorMap& tm_r, Tf32Args& g) {
  using C = Cfg<BN, A_MODE, RES, EW>;
  auto kern = gemm_tf32_kernel<BN, B_MN, A_MODE, RES, EW, SK>;
  static bool configured[64] = {false};  // per device ordinal
  // the scalar-gather mode adds its two input patches to the fixed layout
  int smem = C::SMEM_BYTES;
  if (A_MODE == 3) {
    smem += g.patch_bufs * g.patch_cap;
  }
  if (ctx->device >= 64 || !configured[ctx->device]) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       A_MODE == 3 ? kMaxSmemBytes : C::SMEM_BYTES));
    if (ctx->device < 64) configured[ctx->device] = true;
  }
  g.tiles_n = (g.N + BN - 1) / BN;
  g.total_tiles = g.tiles_m * g.tiles_n * g.total_tiles;  // total_tiles held the batch
  int grid = g.total_tiles < ctx->sm_count ? g.total_tiles : ctx->sm_count;
  if (SK) {
    // the caller has checked that the split pays and that the workspace exists
    grid = ctx->sm_count;
    g.sk_tiles = g.total_tiles % grid;
    g.sk_ws = (float*)ctx->sk_ws;
    g.sk_flags = ctx->sk_flags;
  }
  kern<<<grid, C::THREADS, smem, ctx->stream>>>(tm_a, tm_b, tm_c, tm_r, g);
  // the instantiation's name, for the launch log behind tf.profile's extra information
  static const std::string name =
      "gemm_tf32_kernel<BN=" + std::to_string(BN) + ",B_MN=" + std::to_string(B_MN) +
      ",A_MODE=" + std::to_string(A_MODE) + ",RES=" + std::to_string(RES) +
      ",EW=" + std::to_string(EW) + ",SK=" + std::to_string(SK) + ">";
  LAUNCH_CHECK(ctx, name.c_str());
  return TFJS_CUDA_OK;
}

template <int B_MN, int A_MODE, int RES = 0, int EW = 8>
int launch_bn(tfjs_cuda_ctx* ctx, int bn, const CUtensorMap& a, const CUtensorMap& b,
              const CUtensorMap& c, const CUtensorMap& r, Tf32Args& g) {
  switch (bn) {
    case 32: return launch_cfg<32, B_MN, A_MODE, RES, EW>(ctx, a, b, c, r, g);
    case 64: return launch_cfg<64, B_MN, A_MODE, RES, EW>(ctx, a, b, c, r, g);
    case 128: return launch_cfg<128, B_MN, A_MODE, RES, EW>(ctx, a, b, c, r, g);
    default: return launch_cfg<256, B_MN, A_MODE, RES, EW>(ctx, a, b, c, r, g);
  }
}

int pick_bn(int M, int N, int batch, int sm_count, int k_steps = 0) {
  // Smallest tile that covers N, but do not starve the machine: when the tile
  // count is below the SM count a narrower tile gives more CTAs.
  int bn = N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256));
  const long long tiles_m = (M + BM - 1) / BM;
  if (k_steps >= 16 && bn > 64) {
    // Long K: a K step costs nearly the same whatever the tile's width (measured 0.41 /
    // 0.45 / 0.49 us at 64 / 128 / 256 columns), so halving the tile to fill idle SMs
    // only pays if it saves a wave.  Cost = waves x main loop of a tile + one exposed
    // epilogue (1.3 us per 32-column chunk, two warps per TMEM lane quarter).
    int best = bn;
    double best_cost = 1e30;
    for (int c = bn; c >= 64; c >>= 1) {
      const long long tiles = tiles_m * ((N + c - 1) / c) * batch;
      const long long waves = (tiles + sm_count - 1) / sm_count;
      const double step = c >= 256 ? 0.49 : (c >= 128 ? 0.45 : 0.41);
      const double epi = 1.3 * (c / 64);
      const double main_loop = k_steps * step > epi ? k_steps * step : epi;
      const double cost = waves * main_loop + epi;
      if (cost < best_cost) { best_cost = cost; best = c; }
    }
    return best;
  }
  while (bn > 64 && tiles_m * ((N + bn - 1) / bn) * batch < sm_count) bn >>= 1;
  return bn;
}

// K-split of the last wave: worth it when the partial wave leaves most SMs idle for a long
// main loop.  Costs in K steps: plain = waves x k_steps; split = full waves x k_steps + the
// even share of the rest + the exchange of partial tiles through L2 (`overhead`, measured).
// Also makes sure the workspace exists (never allocated while a step is being captured).
bool use_k_split(tfjs_cuda_ctx* ctx, int total_tiles, int k_steps) {
  // Measured: the exchange costs about as much as 20 K steps (peers store 128 KB each after
  // their last MMA, the owner then reads up to four of them before its ordinary epilogue), so
  // only long main loops gain: [8192, 3072] x [3072, 768] 82 -> 74 us, 3x3 256ch @14x14 b128
  // 66 -> 61 us, 3x3 512ch @7x7 63 -> 57 us; with K = 768 the split loses and stays off.
  static int overhead = -2;  // K steps; negative switches the split off
  if (overhead == -2)
    overhead = getenv("TFJS_CUDA_KSPLIT_OVERHEAD") ? atoi(getenv("TFJS_CUDA_KSPLIT_OVERHEAD")) : 24;
  const int grid = ctx->sm_count;
  const int rest = total_tiles % grid;
  if (overhead < 0 || rest == 0 || grid > 512) return false;
  const long long full = total_tiles / grid;
  const long long share = ((long long)rest * k_steps + grid - 1) / grid;
  if (share < 4) return false;
  const long long plain = (full + 1) * k_steps;
  const long long split = full * k_steps + share + overhead;
  if (split * 10 > plain * 9) return false;
  if (!ctx->sk_ws) {
    if (ctx->capturing) return false;
    const size_t ws = (size_t)grid * 8 * 4 * 4096;  // CTA x warp x chunk x 32 x 32 floats
    if (cudaMalloc(&ctx->sk_ws, ws) != cudaSuccess) { ctx->sk_ws = nullptr; cudaGetLastError(); return false; }
    if (cudaMalloc((void**)&ctx->sk_flags, 4096 * sizeof(unsigned)) != cudaSuccess) {
      cudaFree(ctx->sk_ws);
      ctx->sk_ws = nullptr;
      ctx->sk_flags = nullptr;
      cudaGetLastError();
      return false;
    }
    cudaMemsetAsync(ctx->sk_flags, 0, 4096 * sizeof(unsigned), ctx->stream);
  }
  return true;
}

constexpr int smem_base_mode3(int bn) {
  return bn == 32 ? Cfg<32, 3>::SMEM_BYTES
                  : (bn == 64 ? Cfg<64, 3>::SMEM_BYTES
                              : (bn == 128 ? Cfg<128, 3>::SMEM_BYTES : Cfg<256, 3>::SMEM_BYTES));
}

}  // namespace

bool tf32_patch_plan(const ConvGeo& cv, int M, int N, int sm_count, PatchPlan* plan) {
  static int off = -1;
  if (off < 0) off = getenv("TFJS_CUDA_NO_PATCH_GATHER") ? 1 : 0;  // debugging knob
  const long long rowlen = (long long)cv.in_w * cv.in_c;
  if (off || cv.d_w != 1 || cv.f_h > 15 || (rowlen & 3) || rowlen * 4 > (1 << 20)) return false;
  // margins: the window of the first / last output column reaches this far outside
  const int ml = (cv.pad_l * cv.in_c + 3) & ~3;
  long long over = (long long)(cv.out_w - 1) * cv.s_w - cv.pad_l + cv.f_w - cv.in_w;
  if (over < 0) over = 0;
  const long long mr = (over * cv.in_c + 3) & ~3ll;
  const long long pitch = ml + rowlen + mr;
  // upper bound of the image rows one 128-pixel tile touches: q output rows, at most
  // `step` global rows apart (the stride, or the jump to the next image)
  const long long q = (BM - 1) / cv.out_w + 2;
  const long long jump = (long long)cv.in_h - (long long)(cv.out_h - 1) * cv.s_h;
  const long long step = jump > cv.s_h ? jump : cv.s_h;
  long long rows = (q - 1) * step + (long long)(cv.f_h - 1) * cv.d_h + 1;
  if (rows > (long long)cv.batch * cv.in_h) rows = (long long)cv.batch * cv.in_h;
  const long long bytes = (((rows + 1) * pitch * 4) + 127) & ~127ll;
  const int bn = pick_bn(M, N, 1, sm_count);
  long long bufs = (kMaxSmemBytes - smem_base_mode3(bn)) / bytes;
  if (bufs < 2) return false;
  plan->bufs = bufs > kMaxPatchBufs ? kMaxPatchBufs : (int)bufs;
  plan->bytes = (int)bytes;
  plan->pitch = (int)pitch;
  plan->ml = ml;
  plan->rows = (int)rows;
  return true;
}

// Output map of the heads-permuted store: every 32 x 32 store tile is one box of the
// permuted tensor ((d, s, h, b) for the split, (d, h, s, b) for the merge).
static int make_heads_c_map(tfjs_cuda_ctx* ctx, const GemmProblem& pr, const float* c,
                            CUtensorMap* tm) {
  const int S = pr.out_perm == 1 ? pr.perm_p : pr.M, D = pr.perm_d;
  const bool shape_ok =
      pr.out_perm == 1 ? (pr.batch == 1 && pr.perm_p > 0 && D > 0 && pr.M % pr.perm_p == 0 &&
                          pr.N % D == 0)
                       : (pr.out_perm == 2 && pr.perm_p > 0 && pr.batch % pr.perm_p == 0 &&
                          D == pr.N);
  if (!shape_ok || (S & 31) || (D & 31) || ((uintptr_t)c & 15) || pr.residual)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "heads-permuted store: sequence and head sizes must be multiples of 32");
  EncodeTiledFn enc = get_encode();
  const cuuint64_t B = pr.out_perm == 1 ? pr.M / pr.perm_p : pr.batch / pr.perm_p;
  const cuuint64_t H = pr.out_perm == 1 ? pr.N / D : pr.perm_p;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
  dims[0] = D; dims[3] = B;
  if (pr.out_perm == 1) {  // physical [B, H, S, D]
    dims[1] = S; dims[2] = H;
    strides[0] = (cuuint64_t)D * 4; strides[1] = (cuuint64_t)S * D * 4;
    box[0] = 32; box[1] = 32; box[2] = 1; box[3] = 1;
  } else {                 // physical [B, S, H, D]
    dims[1] = H; dims[2] = S;
    strides[0] = (cuuint64_t)D * 4; strides[1] = (cuuint64_t)H * D * 4;
    box[0] = 32; box[1] = 1; box[2] = 32; box[3] = 1;
  }
  strides[2] = (cuuint64_t)H * S * D * 4;
  if (!enc || enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)c, dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "heads-permuted store: tensor map refused");
  return TFJS_CUDA_OK;
}

// Map over a row-major [batch][M][N] tensor for the epilogue's bulk stores (or the prefetch
// of the residual): dims (N, M, batch), 32 x 32 boxes.
static bool make_plain_c_map(const GemmProblem& pr, const float* base, CUtensorMap* tm,
                             CUtensorMapL2promotion l2) {
  EncodeTiledFn enc = get_encode();
  cuuint64_t dims[3] = {(cuuint64_t)pr.N, (cuuint64_t)pr.M, (cuuint64_t)pr.batch};
  cuuint64_t strides[2] = {(cuuint64_t)pr.N * 4, (cuuint64_t)pr.M * pr.N * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc && enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void*)base, dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, l2,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_gemm_tf32(tfjs_cuda_ctx* ctx, const GemmProblem& pr, const Tf32Operands& op,
                     const GemmGroup* group) {
  Tf32Args g;
  g.c = pr.c;
  g.bias = pr.bias;
  g.bias_len = pr.bias ? pr.bias_len : 0;
  g.ap = pr.ap;
  g.M = pr.M;
  g.N = pr.N;
  g.batch_a = pr.batch_a;
  g.batch_b = pr.batch_b;
  g.tiles_m = (pr.M + BM - 1) / BM;
  g.total_tiles = pr.batch;  // multiplied out in launch_cfg
  g.k_steps = op.k_steps;
  g.flag = ctx->d_flag;
  g.x = op.a;
  g.conv = pr.conv;
  g.chunks_per_tap = op.cin_pad / BK;
  const int bn = pick_bn(pr.M, pr.N, pr.batch, ctx->sm_count, op.k_steps);
  CUtensorMap tm_a, tm_b, tm_c, tm_r;
  int rc;
  // output map for the epilogue's bulk stores, and the same view of the residual for
  // its prefetches: dims (N, M, batch), 32 x 32 boxes
  memset(&tm_c, 0, sizeof tm_c);
  memset(&tm_r, 0, sizeof tm_r);
  g.c_tma = 0;
  g.residual = pr.residual;
  g.post_act = pr.post_act;
  g.patch_cap = g.patch_pitch = g.patch_ml = g.patch_rows = g.patch_bufs = 0;
  fast_div_setup(op.a_gather ? pr.conv.out_w : 1, &g.ow_mul, &g.ow_shr);
  fast_div_setup(op.a_gather ? pr.conv.out_h : 1, &g.oh_mul, &g.oh_shr);
  if (op.a_gather == 3) {
    PatchPlan plan;
    if (!tf32_patch_plan(pr.conv, pr.M, pr.N, ctx->sm_count, &plan) || ((uintptr_t)op.a & 15))
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "staged-row gather planned for a shape it cannot take");
    g.patch_cap = plan.bytes;
    g.patch_pitch = plan.pitch;
    g.patch_ml = plan.ml;
    g.patch_rows = plan.rows;
    g.patch_bufs = plan.bufs;
  }
  bool res_tma = false;
  g.sk_tiles = 0;
  g.sk_ws = nullptr;
  g.sk_flags = nullptr;
  g.out_perm = pr.out_perm;
  g.perm_p = pr.perm_p;
  g.perm_d = pr.perm_d;
  if (pr.out_perm != 0) {
    if ((rc = make_heads_c_map(ctx, pr, pr.c, &tm_c))) return rc;
    g.c_tma = 1;
  } else
  if ((pr.N & 3) == 0 && ((uintptr_t)pr.c & 15) == 0 && ((uintptr_t)pr.residual & 15) == 0) {
    static int no_tma_store = -1;
    if (no_tma_store < 0) no_tma_store = getenv("TFJS_CUDA_NO_TMA_STORE") ? 1 : 0;  // debugging knob
    const bool ok = !no_tma_store &&
                    make_plain_c_map(pr, pr.c, &tm_c, CU_TENSOR_MAP_L2_PROMOTION_NONE);
    if (!pr.residual) {
      g.c_tma = ok ? 1 : 0;
    } else if (ok && op.b_layout == B_K_MAJOR && (op.a_gather == 0 || op.a_gather == 1) &&
               make_plain_c_map(pr, pr.residual, &tm_r, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) {
      // the residual epilogue exists for the TMA-fed A operand modes
      res_tma = true;
    }
  }
  bool im2col = false;
  static int no_im2col = -1;
  if (no_im2col < 0) no_im2col = getenv("TFJS_CUDA_NO_IM2COL_TMA") ? 1 : 0;  // debugging knob
  // Narrow outputs with a long K: a tcgen05.mma takes the same time for 64 output
  // columns as for 256, so put the pixels on the instruction's N axis (256 per tile)
  // and the <= 128 output channels on its 128 rows.
  // Measured on 3x3 convolutions at batch 128: 64 -> 64 at 56x56 153 -> 95 us, 128 -> 128 at
  // 28x28 88 -> 56 us; with fewer than about 12 K steps the epilogue dominates and the two
  // forms tie.
  static int swap_k = -1;  // fewest K steps that take the swapped form; 0 switches it off
  if (swap_k < 0)
    swap_k = getenv("TFJS_CUDA_SWAP_AB_KSTEPS") ? atoi(getenv("TFJS_CUDA_SWAP_AB_KSTEPS")) : 12;
  if (swap_k > 0 && op.k_steps >= swap_k && op.b_layout == B_K_MAJOR && pr.N <= 128 &&
      g.c_tma && !pr.residual && pr.out_perm == 0 && pr.ap.act != TFJS_CUDA_ACT_PRELU &&
      (op.a_gather == 0 || (op.a_gather == 1 && !no_im2col))) {
    memset(&tm_a, 0, sizeof tm_a);
    bool ok;
    if (op.a_gather == 1) {
      ok = make_im2col_map(&tm_a, op.a, pr.conv, 256);
    } else {
      ok = make_map(ctx, &tm_a, op.a, (uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.batch_a,
                    (uint64_t)op.lda, (uint64_t)pr.M * op.lda, 256) == TFJS_CUDA_OK;
    }
    if (ok) {
      const uint64_t kk = (uint64_t)op.k_steps * BK < (uint64_t)op.ldb
                              ? (uint64_t)op.k_steps * BK : (uint64_t)op.ldb;
      if ((rc = make_map(ctx, &tm_b, op.b, kk, (uint64_t)pr.N, (uint64_t)pr.batch_b,
                         (uint64_t)op.ldb, (uint64_t)pr.N * op.ldb, (uint32_t)BM)))
        return rc;
      g.tiles_m = (pr.M + 255) / 256;
      if (op.a_gather == 1) return launch_cfg<256, 0, 5>(ctx, tm_a, tm_b, tm_c, tm_r, g);
      return launch_cfg<256, 0, 4>(ctx, tm_a, tm_b, tm_c, tm_r, g);
    }
  }
  // Wide outputs with a long enough main loop run on CTA pairs: 256 x 256 tiles over two
  // SMs that share the B tile (gemm_tf32_pair_sm100.cu).
  static int pair_k = -1;  // fewest K steps that take the pair form; 0 switches it off
  if (pair_k < 0)
    pair_k = getenv("TFJS_CUDA_PAIR_KSTEPS") ? atoi(getenv("TFJS_CUDA_PAIR_KSTEPS")) : 8;
  // Measured (device time, B200): 4096 x 1024 x 4096 58.3 -> 55.5 us, [8192, 768] x [768, 3072]
  // 67.8 -> 62.8 us; with at most two waves of pair tiles the two forms tie, and where the
  // single-CTA form splits the K loop of its last wave ([8192, 3072] x [3072, 768], the 3x3
  // convolutions at 14 x 14 and 7 x 7) that form is 5-20% faster, so those keep it.
  const long long pair_tiles = (long long)((pr.M + 255) / 256) * ((pr.N + 255) / 256) * pr.batch *
                               (group ? group->count : 1);
  const bool pair_shape = op.b_layout == B_K_MAJOR && pr.N > 128 && g.c_tma && !pr.residual &&
                          ctx->sm_count >= 2 &&
                          (op.a_gather == 0 || (op.a_gather == 1 && !no_im2col));
  if (group) {
    // a group exists in the pair kernel only
    if (!pair_shape || op.a_gather != 0 || group->count < 2 || group->count > kMaxGemmGroup)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "grouped matMul: shape not taken by the pair kernel");
    PairGroupMaps maps;
    memset(&maps, 0, sizeof maps);
    maps.count = group->count;
    if ((rc = make_map(ctx, &tm_a, op.a, (uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.batch_a,
                       (uint64_t)op.lda, (uint64_t)pr.M * op.lda, BM)))
      return rc;
    const uint64_t kk = (uint64_t)op.k_steps * BK < (uint64_t)op.ldb
                            ? (uint64_t)op.k_steps * BK : (uint64_t)op.ldb;
    for (int i = 0; i < group->count; ++i) {
      if ((rc = make_map(ctx, &maps.b[i], group->b[i], kk, (uint64_t)pr.N, (uint64_t)pr.batch_b,
                         (uint64_t)op.ldb, (uint64_t)pr.N * op.ldb, 128u)))
        return rc;
      if (pr.out_perm != 0) {
        if ((rc = make_heads_c_map(ctx, pr, group->c[i], &maps.c[i]))) return rc;
      } else if (((uintptr_t)group->c[i] & 15) ||
                 !make_plain_c_map(pr, group->c[i], &maps.c[i], CU_TENSOR_MAP_L2_PROMOTION_NONE)) {
        return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "grouped matMul: output map refused");
      }
      maps.bias[i] = group->bias[i];
    }
    g.tiles_m = (pr.M + 255) / 256;
    return launch_gemm_tf32_pair_group(ctx, tm_a, maps, g);
  }
  // Between one and 1.5 waves of 256 x 256 pair tiles: 256 x 384 tiles run as a single wave
  // ([8192, 3072] x [3072, 768] and [8192, 768] x [768, 768]: 96 tiles -> 64 on 74 pairs).
  static int pair_wide = -1;
  if (pair_wide < 0) pair_wide = getenv("TFJS_CUDA_NO_PAIR_WIDE") ? 0 : 1;
  const long long wide_tiles = (long long)((pr.M + 255) / 256) * ((pr.N + 383) / 384) * pr.batch;
  if (pair_wide && pair_k > 0 && op.k_steps >= pair_k && pair_shape && op.a_gather == 0 &&
      pr.N > 256 && pair_tiles > ctx->sm_count / 2 && wide_tiles <= ctx->sm_count / 2) {
    memset(&tm_a, 0, sizeof tm_a);
    if (make_map(ctx, &tm_a, op.a, (uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.batch_a,
                 (uint64_t)op.lda, (uint64_t)pr.M * op.lda, BM) == TFJS_CUDA_OK) {
      const uint64_t kk = (uint64_t)op.k_steps * BK < (uint64_t)op.ldb
                              ? (uint64_t)op.k_steps * BK : (uint64_t)op.ldb;
      if ((rc = make_map(ctx, &tm_b, op.b, kk, (uint64_t)pr.N, (uint64_t)pr.batch_b,
                         (uint64_t)op.ldb, (uint64_t)pr.N * op.ldb, 96u)))
        return rc;
      g.tiles_m = (pr.M + 255) / 256;
      return launch_gemm_tf32_pair_wide(ctx, tm_a, tm_b, tm_c, g);
    }
  }
  if (pair_k > 0 && op.k_steps >= pair_k && pair_shape &&
      pair_tiles > 2ll * (ctx->sm_count / 2) &&
      !(bn == 256 && use_k_split(ctx, g.tiles_m * ((pr.N + 255) / 256) * pr.batch, op.k_steps))) {
    memset(&tm_a, 0, sizeof tm_a);
    bool ok;
    if (op.a_gather == 1) {
      ok = make_im2col_map(&tm_a, op.a, pr.conv);
    } else {
      ok = make_map(ctx, &tm_a, op.a, (uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.batch_a,
                    (uint64_t)op.lda, (uint64_t)pr.M * op.lda, BM) == TFJS_CUDA_OK;
    }
    if (ok) {
      const uint64_t kk = (uint64_t)op.k_steps * BK < (uint64_t)op.ldb
                              ? (uint64_t)op.k_steps * BK : (uint64_t)op.ldb;
      if ((rc = make_map(ctx, &tm_b, op.b, kk, (uint64_t)pr.N, (uint64_t)pr.batch_b,
                         (uint64_t)op.ldb, (uint64_t)pr.N * op.ldb, 128u)))
        return rc;
      g.tiles_m = (pr.M + 255) / 256;
      return launch_gemm_tf32_pair(ctx, tm_a, tm_b, tm_c, g, op.a_gather == 1);
    }
  }
  if (op.a_gather == 1) {
    memset(&tm_a, 0, sizeof tm_a);
    im2col = !no_im2col && make_im2col_map(&tm_a, op.a, pr.conv);
  } else if (op.a_gather >= 2) {
    memset(&tm_a, 0, sizeof tm_a);
  } else {
    if ((rc = make_map(ctx, &tm_a, op.a, (uint64_t)pr.K, (uint64_t)pr.M,
                       (uint64_t)pr.batch_a, (uint64_t)op.lda,
                       (uint64_t)pr.M * op.lda, BM)))
      return rc;
  }
  if (op.b_layout == B_K_MAJOR) {
    const uint64_t kk = (uint64_t)op.k_steps * BK < (uint64_t)op.ldb
                            ? (uint64_t)op.k_steps * BK : (uint64_t)op.ldb;
    if ((rc = make_map(ctx, &tm_b, op.b, kk, (uint64_t)pr.N, (uint64_t)pr.batch_b,
                       (uint64_t)op.ldb, (uint64_t)pr.N * op.ldb, (uint32_t)bn)))
      return rc;
    if (op.a_gather >= 2) {
      tm_a = tm_b;  // unused by the gather kernel
      return launch_bn<0, 3>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
    }
    // Few K steps per tile: the kernel is a stream of epilogues, whose per-chunk chain
    // (TMEM load, bias / activation, staging, bulk store) is latency-bound with two warps
    // per TMEM lane quarter; these launches run four.
    static int wide_k = -1;  // widest K (in 32-float steps) that takes the 16-warp epilogue
    if (wide_k < 0)
      wide_k = getenv("TFJS_CUDA_WIDE_EPILOGUE_KSTEPS") ? atoi(getenv("TFJS_CUDA_WIDE_EPILOGUE_KSTEPS"))
                                                        : 8;  // tuning knob, 0 switches it off
    const bool wide = !pr.residual && op.k_steps <= wide_k;
    static int wide_res_k = -1;  // the same bound for the residual epilogue
    if (wide_res_k < 0)
      wide_res_k = getenv("TFJS_CUDA_WIDE_RESIDUAL_KSTEPS")
                       ? atoi(getenv("TFJS_CUDA_WIDE_RESIDUAL_KSTEPS")) : 8;  // tuning knob
    if (im2col) {
      if (res_tma) {
        g.c_tma = 1;
        if (op.k_steps <= wide_res_k)
          return launch_bn<0, 2, 1, 16>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
        return launch_bn<0, 2, 1>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
      }
      if (wide) return launch_bn<0, 2, 0, 16>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
      if (bn == 256 && use_k_split(ctx, g.tiles_m * ((pr.N + 255) / 256) * pr.batch, op.k_steps))
        return launch_cfg<256, 0, 2, 0, 8, 1>(ctx, tm_a, tm_b, tm_c, tm_r, g);
      return launch_bn<0, 2>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
    }
    if (op.a_gather) {
      tm_a = tm_b;  // unused by the gather kernel
      return launch_bn<0, 1>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
    }
    if (res_tma) {
      g.c_tma = 1;
      if (op.k_steps <= wide_res_k)
        return launch_bn<0, 0, 1, 16>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
      return launch_bn<0, 0, 1>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
    }
    if (wide) return launch_bn<0, 0, 0, 16>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
    if (bn == 256 && use_k_split(ctx, g.tiles_m * ((pr.N + 255) / 256) * pr.batch, op.k_steps))
      return launch_cfg<256, 0, 0, 0, 8, 1>(ctx, tm_a, tm_b, tm_c, tm_r, g);
    return launch_bn<0, 0>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
  }
  if ((rc = make_map(ctx, &tm_b, op.b, (uint64_t)pr.N, (uint64_t)pr.K,
                     (uint64_t)pr.batch_b, (uint64_t)op.ldb, (uint64_t)pr.K * op.ldb, 32,
                     CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)))
    return rc;
  if (op.a_gather)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "convolution filters are always packed K-major");
  return launch_bn<1, 0>(ctx, bn, tm_a, tm_b, tm_c, tm_r, g);
}
