// Attention of one layer as one launch: out = softmax(Q K^T * scale + mask) V for heads of
// 128 positions x 64 features, Q / K / V stored [B, H, 128, 64] (the heads-split store of the
// projections) and the result stored [B, 128, H, 64] (heads merged), as four kernels of the
// reference leave it: BatchMatMul (tfjs-backend-cpu/src/kernels/BatchMatMul.ts:29-113),
// Multiply, Add, Softmax (Softmax.ts:50-67), BatchMatMul + Transpose.  The [B, H, 128, 128]
// scores and probabilities never leave the SM: 200 MB of the 300 MB those four launches move
// for BERT-base at batch 64.
//
// One persistent CTA per SM takes (batch, head) units in turn:
//   warp 0     TMA producer: Q and K tiles (K-major, 128-byte swizzle) and the V tile (its 64
//              features contiguous: the MN-major B layout) of the next units, two units deep
//   warp 1     tensor memory allocation; one thread issues the MMAs: S = Q K^T (M = N = 128,
//              K = 64) into tensor memory, and O = P V (M = 128, N = 64, K = 128) with P read
//              from tensor memory as the A operand
//   warps 2-9  two groups of four; a group takes every second unit: each thread owns one
//              row of S (tcgen05.ld), forms x * scale + mask (the mask row staged in shared
//              memory by the group, fetched one unit ahead), the row maximum, e = 2^((x -
//              max) log2 e), the sum and p = e * (1 / sum) in registers (the arithmetic of the
//              stand-alone softmax kernel; the sum runs along the row instead of across
//              lanes), rounds p to TF32 (nearest) as the TMA load of the stand-alone product would, and
//              writes it over S (tcgen05.st); later it takes O out of tensor memory and
//              stores it through a swizzled staging tile with bulk tensor stores
// Every wait is bounded; a wait that gives up records where in the context's error word.
#include "gemm_tf32_device.cuh"

namespace {

constexpr int kS = 128;                    // positions (queries = keys)
constexpr int kD = 64;                     // features per head
constexpr int kQKBytes = 2 * kS * kD * 4;  // Q then K: each two K-step tiles of [128][128 B]
constexpr int kVBytes = kS * kD * 4;       // [4 K steps][2 column blocks][32 rows][128 B]
constexpr int kSlots = 2;
constexpr int kGroupWarps = 4;
constexpr int kAttnThreads = 64 + kSlots * kGroupWarps * 32;
constexpr int kAttnBarriers = 7 * kSlots;
constexpr int kMaskBytes = kSlots * kS * 4;   // one mask row per group
constexpr int kAttnSmem = 1024 + kSlots * (kQKBytes + kVBytes) + kSlots * kGroupWarps * 4096 +
                          kMaskBytes + kAttnBarriers * 8 + 16 + 8;
static_assert(kAttnSmem <= kMaxSmemBytes, "attention kernel: shared memory");

struct AttnArgs {
  const float* mask;     // null: none; else [units / units_per_mask][128]
  int has_scale;
  float scale;
  int units;             // batch * heads
  int heads;
  int units_per_mask;
  int* flag;
};

__device__ __forceinline__ void tc_mma_tf32_tmem_a(uint32_t d_tmem, uint32_t a_tmem,
                                                   uint64_t bdesc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 columns of this thread's TMEM lane, without waiting for them.
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t* r) {
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
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::
      "r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ float attn_max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                 const AttnArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto qk_base = [&](int s) { return smem_base + (uint32_t)s * kQKBytes; };
  auto v_base = [&](int s) { return smem_base + kSlots * kQKBytes + (uint32_t)s * kVBytes; };
  const uint32_t epi_base = smem_base + kSlots * (kQKBytes + kVBytes);
  const uint32_t mask_base = epi_base + kSlots * kGroupWarps * 4096u;
  const uint32_t bar_base = mask_base + kMaskBytes;
  auto bar = [&](int kind, int s) { return bar_base + 8u * (uint32_t)(kind * kSlots + s); };
  enum { QK_FULL = 0, QK_EMPTY, V_FULL, V_EMPTY, S_FULL, P_FULL, O_FULL };
  const uint32_t tmem_slot = bar_base + 8u * kAttnBarriers;
  const uint32_t dead_word = tmem_slot + 4u;   // + 4 * group: that group gave up on a wait

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 32) {
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_o);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(bar(QK_FULL, s), 1);
      mbar_init(bar(QK_EMPTY, s), 1);
      mbar_init(bar(V_FULL, s), 1);
      mbar_init(bar(V_EMPTY, s), 1);
      mbar_init(bar(S_FULL, s), 1);
      mbar_init(bar(P_FULL, s), kGroupWarps);
      mbar_init(bar(O_FULL, s), 1);
    }
    for (int s = 0; s < kSlots; ++s)
      asm volatile("st.shared.u32 [%0], %1;" ::"r"(dead_word + 4u * s), "r"(0u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));
  // scores / probabilities: 128 columns per slot; outputs: 64 columns per slot
  auto s_tmem = [&](int s) { return tmem_base + (uint32_t)(s * kS); };
  auto o_tmem = [&](int s) { return tmem_base + (uint32_t)(kSlots * kS + s * kD); };

  const int first = (int)blockIdx.x, step = (int)gridDim.x;
  const int n_local = first < g.units ? (g.units - first + step - 1) / step : 0;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer --
    if (lane == 0) {
      for (int i = 0; i < n_local; ++i) {
        const int u = first + i * step;
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!mbar_wait(bar(QK_EMPTY, s), ph ^ 1)) {
          atomicExch(g.flag, 1);
          break;
        }
        mbar_expect_tx(bar(QK_FULL, s), (uint32_t)kQKBytes);
        tma_load_3d(qk_base(s), &tm_q, bar(QK_FULL, s), 0, 0, u);
        tma_load_3d(qk_base(s) + 16384u, &tm_q, bar(QK_FULL, s), 32, 0, u);
        tma_load_3d(qk_base(s) + 32768u, &tm_k, bar(QK_FULL, s), 0, 0, u);
        tma_load_3d(qk_base(s) + 49152u, &tm_k, bar(QK_FULL, s), 32, 0, u);
        if (!mbar_wait(bar(V_EMPTY, s), ph ^ 1)) {
          atomicExch(g.flag, 1);
          break;
        }
        mbar_expect_tx(bar(V_FULL, s), (uint32_t)kVBytes);
#pragma unroll
        for (int ks = 0; ks < kS / 32; ++ks)
#pragma unroll
          for (int j = 0; j < kD / 32; ++j)
            tma_load_3d(v_base(s) + (uint32_t)(ks * (kD / 32) + j) * 4096u, &tm_v, bar(V_FULL, s),
                        j * 32, ks * 32, u);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      // instruction descriptors: D = f32, A = B = tf32, M = 128; scores: N = 128, B K-major;
      // output: N = 64, B MN-major
      const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kS >> 3) << 17) |
                               ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) |
                               ((uint32_t)(kD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      // Descriptors per slot, built once: the MMAs of a unit differ from them only in the
      // start-address field of the low word (16-byte units), so issuing one costs an add.
      // (This thread's scalar instructions are what separates P_FULL from O_FULL.)
      static_assert(kSlots == 2, "the low words below are selected by the slot's parity");
      const uint32_t k_hi = (uint32_t)(desc_k_major(0) >> 32);
      const uint32_t v_hi = (uint32_t)(desc_mn_major(0) >> 32);
      const uint32_t q_lo0 = (uint32_t)desc_k_major(qk_base(0));
      const uint32_t q_lo1 = (uint32_t)desc_k_major(qk_base(1));
      const uint32_t v_lo0 = (uint32_t)desc_mn_major(v_base(0));
      const uint32_t v_lo1 = (uint32_t)desc_mn_major(v_base(1));
      auto mk = [](uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | lo; };
      bool alive = true;
      auto issue_pv = [&](int i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!mbar_wait(bar(V_FULL, s), ph) || !mbar_wait(bar(P_FULL, s), ph)) {
          atomicExch(g.flag, 3);
          alive = false;
          return;
        }
        tc_fence_after();
        const uint32_t v_lo = s ? v_lo1 : v_lo0;
#pragma unroll
        for (int kk = 0; kk < kS / UMMA_K; ++kk)
          tc_mma_tf32_tmem_a(o_tmem(s), s_tmem(s) + (uint32_t)(kk * UMMA_K),
                             mk(v_hi, v_lo + (((uint32_t)(kk >> 2) * (kD / 32) * 4096u +
                                                  (uint32_t)(kk & 3) * 1024u) >> 4)),
                             idesc_o, kk != 0 ? 1u : 0u);
        tc_commit(bar(V_EMPTY, s));
        tc_commit(bar(O_FULL, s));
      };
      for (int i = 0; alive && i < n_local; ++i) {
        const int s = i & 1;
        const uint32_t ph = (uint32_t)(i >> 1) & 1u;
        if (!mbar_wait(bar(QK_FULL, s), ph)) {
          atomicExch(g.flag, 2);
          alive = false;
          break;
        }
        tc_fence_after();
        const uint32_t q_lo = s ? q_lo1 : q_lo0;
#pragma unroll
        for (int kk = 0; kk < kD / UMMA_K; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * 16384u + (uint32_t)(kk & 3) * (UMMA_K * 4);
          tc_mma_tf32(s_tmem(s), mk(k_hi, q_lo + (off >> 4)),
                      mk(k_hi, q_lo + ((32768u + off) >> 4)), idesc_s, kk != 0 ? 1u : 0u);
        }
        tc_commit(bar(QK_EMPTY, s));
        tc_commit(bar(S_FULL, s));
        if (i >= 1) issue_pv(i - 1);
      }
      if (alive && n_local > 0) issue_pv(n_local - 1);
    }
  } else {
    // ------------------------------------------- softmax and output groups --
    const int grp = (warp - 2) / kGroupWarps;   // the slot this group serves
    const int q = warp & 3;                     // TMEM lane quarter this warp may access
    const uint32_t lane_sel = (uint32_t)(q * 32) << 16;
    const uint32_t stage_buf = epi_base + (uint32_t)(warp - 2) * 4096u;
    const uint32_t my_row = stage_buf + (uint32_t)lane * 128u;
    const uint32_t sw = (uint32_t)(lane & 7);
    // The unit's mask row goes through shared memory: every thread needs all 128 values,
    // and 32 dependent global loads per thread cost more than the rest of the softmax.
    // Thread t of the group fetches value t one unit ahead.
    const int tg = (int)threadIdx.x - 64 - grp * (kGroupWarps * 32);
    const uint32_t mask_buf = mask_base + (uint32_t)grp * (kS * 4);
    auto mask_value = [&](int unit) {
      return g.mask ? __ldg(g.mask + (size_t)(unit / g.units_per_mask) * kS + tg) : 0.0f;
    };
    float mask_next = grp < n_local ? mask_value(first + grp * step) : 0.0f;
    for (int i = grp; i < n_local; i += kSlots) {
      const int u = first + i * step;
      const uint32_t ph = (uint32_t)(i >> 1) & 1u;
      // (first barrier: the group has finished reading the previous unit's row.  A warp
      // whose wait ran out does not leave on its own, which would strand the others at
      // this barrier: it marks the group and all four leave together here.)
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kGroupWarps * 32) : "memory");
      uint32_t dead;
      asm volatile("ld.shared.u32 %0, [%1];" : "=r"(dead) : "r"(dead_word + 4u * grp) : "memory");
      if (dead) break;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(mask_buf + (uint32_t)tg * 4u), "f"(mask_next)
                   : "memory");
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kGroupWarps * 32) : "memory");
      if (i + kSlots < n_local) mask_next = mask_value(first + (i + kSlots) * step);
      if (!mbar_wait(bar(S_FULL, grp), ph)) {
        if (lane == 0) {
          atomicExch(g.flag, 4);
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(dead_word + 4u * grp), "r"(1u) : "memory");
        }
        continue;
      }
      tc_fence_after();
      uint32_t raw[kS];
#pragma unroll
      for (int c = 0; c < kS / 32; ++c)
        tc_ld32_nowait(s_tmem(grp) + lane_sel + (uint32_t)(c * 32), raw + c * 32);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float v[kS];
      const bool masked = g.mask != nullptr;
      // (plain loads, so that the compiler may schedule them among the arithmetic)
      const float4* mrow = reinterpret_cast<const float4*>(smem_raw + (mask_buf - smem_u32(smem_raw)));
      __builtin_assume(__isShared(mrow));
#pragma unroll
      for (int j = 0; j < kS / 4; ++j) {
        float mv[4] = {0.f, 0.f, 0.f, 0.f};
        if (masked) {
          const float4 mk = mrow[j];
          mv[0] = mk.x; mv[1] = mk.y; mv[2] = mk.z; mv[3] = mk.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float t = __uint_as_float(raw[4 * j + k]);
          if (g.has_scale) t = __fmul_rn(t, g.scale);
          if (masked) t = __fadd_rn(t, mv[k]);
          v[4 * j + k] = t;
        }
      }
      float m4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
      for (int j = 4; j < kS; ++j) m4[j & 3] = attn_max_nan(m4[j & 3], v[j]);
      const float m = attn_max_nan(attn_max_nan(m4[0], m4[1]), attn_max_nan(m4[2], m4[3]));
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < kS; ++j) {
        v[j] = exp2_approx(__fmul_rn(__fsub_rn(v[j], m), 1.4426950408889634f));
        s4[j & 3] = __fadd_rn(s4[j & 3], v[j]);
      }
      const float inv = __frcp_rn(__fadd_rn(__fadd_rn(s4[0], s4[1]), __fadd_rn(s4[2], s4[3])));
      // p = e * inv rounded to TF32 (11 significant bits) with three fp32 operations
      // (Veltkamp's splitting by 2^13 + 1: the nearest 11-bit value; exact for p in [0, 1]
      // and for NaN) - the conversion instruction shares the special-function unit with
      // the exponentials, which already bound this phase
#pragma unroll
      for (int j = 0; j < kS; ++j) {
        const float p = __fmul_rn(v[j], inv);
        const float c = __fmul_rn(p, 8193.0f);
        raw[j] = __float_as_uint(__fsub_rn(c, __fsub_rn(c, p)));
      }
#pragma unroll
      for (int c = 0; c < kS / 32; ++c)
        tc_st32(s_tmem(grp) + lane_sel + (uint32_t)(c * 32), raw + c * 32);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL, grp));

      // the unit's output: 128 x 64, this warp's 32 rows as two 32 x 32 boxes
      if (!mbar_wait(bar(O_FULL, grp), ph)) {
        if (lane == 0) {
          atomicExch(g.flag, 5);
          asm volatile("st.shared.u32 [%0], %1;" ::"r"(dead_word + 4u * grp), "r"(1u) : "memory");
        }
        continue;
      }
      tc_fence_after();
      const int b = u / g.heads, h = u - b * g.heads;
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        float o[32];
        tc_ld32(o_tmem(grp) + lane_sel + (uint32_t)(c * 32), o);
        // the bulk store that last used the staging tile must have finished reading it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(
                           my_row + (((uint32_t)j ^ sw) << 4)),
                       "f"(o[4 * j]), "f"(o[4 * j + 1]), "f"(o[4 * j + 2]), "f"(o[4 * j + 3])
                       : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          // map over [B, 128, H, 64]: coordinates (feature, head, position, batch)
          asm volatile(
              "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
              ::"l"(&tm_o), "r"(stage_buf), "r"(c * 32), "r"(h), "r"(q * 32), "r"(b)
              : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
      // O of this slot is rewritten only after this group has handed over its next P
      tc_fence_before();
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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

// 3-D map over [units][128][64] floats, TF32 rounding on the way in.
bool make_head_map(CUtensorMap* tm, const float* base, uint64_t units, uint32_t box_rows,
                   CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode();
  cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)kS, units};
  cuuint64_t strides[2] = {(cuuint64_t)kD * 4, (cuuint64_t)kS * kD * 4};
  cuuint32_t box[3] = {32, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc && enc(tm, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 3, (void*)base, dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" {

int tfjs_cuda_fused_attention(tfjs_cuda_ctx* ctx, int32_t q_id, int32_t k_id, int32_t v_id,
                              int32_t mask_id, int32_t has_scale, float scale, int32_t batch,
                              int32_t heads, int32_t seq, int32_t head_dim,
                              int32_t units_per_mask, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  const char* who = "fused attention";
  if (batch <= 0 || heads <= 0 || seq <= 0 || head_dim <= 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: dimensions must be positive", who);
  if (mask_id != 0 && units_per_mask <= 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: units_per_mask must be positive", who);
  if (seq != kS || head_dim != kD || ctx->math_mode != TFJS_CUDA_MATH_TF32 ||
      (uint64_t)batch * heads > 0x7fffffffull / (kS * kD))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "%s: heads of 128 positions x 64 features in the TF32 math mode only", who);
  const uint64_t units = (uint64_t)batch * heads;
  const uint64_t n = units * kS * kD;
  Buffer *q, *k, *v, *mask = nullptr, *out;
  int rc;
  if ((rc = ctx_get(ctx, q_id, n * 4, "fused attention q", &q))) return rc;
  if ((rc = ctx_get(ctx, k_id, n * 4, "fused attention k", &k))) return rc;
  if ((rc = ctx_get(ctx, v_id, n * 4, "fused attention v", &v))) return rc;
  if (mask_id != 0) {
    const uint64_t mask_rows = (units - 1) / (uint64_t)units_per_mask + 1;
    if ((rc = ctx_get(ctx, mask_id, mask_rows * kS * 4, "fused attention mask", &mask))) return rc;
  }
  if ((rc = ctx_get(ctx, out_id, n * 4, "fused attention out", &out))) return rc;
  if (((uintptr_t)q->ptr | (uintptr_t)k->ptr | (uintptr_t)v->ptr | (uintptr_t)out->ptr |
       (uintptr_t)(mask ? mask->ptr : nullptr)) & 15)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: unaligned tensor", who);
  cudaSetDevice(ctx->device);
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  memset(&tm_o, 0, sizeof tm_o);
  bool ok = make_head_map(&tm_q, (const float*)q->ptr, units, kS, CU_TENSOR_MAP_SWIZZLE_128B) &&
            make_head_map(&tm_k, (const float*)k->ptr, units, kS, CU_TENSOR_MAP_SWIZZLE_128B) &&
            make_head_map(&tm_v, (const float*)v->ptr, units, 32,
                          CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
  if (ok) {
    // [B, 128, H, 64] result: dims (feature, head, position, batch), 32 x 1 x 32 x 1 boxes
    EncodeTiledFn enc = get_encode();
    cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)kS, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)kD * 4, (cuuint64_t)heads * kD * 4,
                             (cuuint64_t)kS * heads * kD * 4};
    cuuint32_t box[4] = {32, 1, 32, 1}, estr[4] = {1, 1, 1, 1};
    ok = enc(&tm_o, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, out->ptr, dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  if (!ok) return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: tensor map refused", who);
  static bool configured[64] = {false};  // per device ordinal
  if (ctx->device >= 64 || !configured[ctx->device]) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(attention_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
    if (ctx->device < 64) configured[ctx->device] = true;
  }
  AttnArgs g;
  g.mask = mask ? (const float*)mask->ptr : nullptr;
  g.has_scale = has_scale;
  g.scale = scale;
  g.units = (int)units;
  g.heads = heads;
  g.units_per_mask = mask ? units_per_mask : 1;
  g.flag = ctx->d_flag;
  const int grid = units < (uint64_t)ctx->sm_count ? (int)units : ctx->sm_count;
  attention_kernel<<<grid, kAttnThreads, kAttnSmem, ctx->stream>>>(tm_q, tm_k, tm_v, tm_o, g);
  LAUNCH_CHECK(ctx, "attention_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

}  // extern "C"
