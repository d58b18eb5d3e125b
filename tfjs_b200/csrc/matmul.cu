// Front end of FusedConv2D and _FusedMatMul / BatchMatMul: validates the call,
// picks the tensor-core (TF32) or the fp32 SIMT back end, and owns the packed
// weight cache.
//
// Weights are constants, so the first use of a filter (a buffer last filled by
// write() or dequantize()) repacks it once into the K-contiguous layout the
// tensor-core kernel streams with TMA, rounding to TF32 (nearest) on the way;
// the packed copy is dropped when the tensor is freed or rewritten.  The idea of
// a per-filter cache comes from the reference's WASM backend, which transposes
// HWIO -> OHWI once per filter id (tfjs-backend-wasm/src/cc/conv2d_impl.cc:224-257).
#include "common.cuh"
#include "gemm.h"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float round_tf32(float v) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
  return __uint_as_float(r);
}

// out[b][n][t][c] = tf32(in[b][(t*cin + c)][n]) for c < cin, else 0.
// `in` is [batch][taps*cin][N] when !in_is_nk, or [batch][N][taps*cin] when
// in_is_nk (already K-contiguous: only rounding and padding happen).
__global__ void pack_weight_kernel(const float* __restrict__ in, float* __restrict__ out,
                                   uint64_t total, int N, int taps, int cin, int cin_pad,
                                   int in_is_nk) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  const uint64_t per_b = (uint64_t)N * taps * cin_pad;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint64_t b = i / per_b;
    uint64_t rem = i % per_b;
    const int c = (int)(rem % cin_pad);
    rem /= cin_pad;
    const int t = (int)(rem % taps);
    const int n = (int)(rem / taps);
    float v = 0.0f;
    if (c < cin) {
      const uint64_t k = (uint64_t)t * cin + c;
      const uint64_t K = (uint64_t)taps * cin;
      v = in_is_nk ? in[(b * N + n) * K + k] : in[(b * K + k) * N + n];
      v = round_tf32(v);
    }
    out[i] = v;
  }
}

// Explicit im2col for inputs whose channel count is not a multiple of 4 (the
// 3-channel stem): col[m][k] with k = (fr*f_w + fc)*in_c + d1, rows padded to ld.
__global__ void im2col_kernel(const float* __restrict__ x, float* __restrict__ col,
                              uint64_t total, int K, int ld, ConvGeo cv) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int k = (int)(i % ld);
    const uint64_t m = i / ld;
    float v = 0.0f;
    if (k < K) {
      const int ow = (int)(m % cv.out_w);
      const uint64_t t = m / cv.out_w;
      const int oh = (int)(t % cv.out_h);
      const int b = (int)(t / cv.out_h);
      const int d1 = k % cv.in_c;
      const int tap = k / cv.in_c;
      const int fc = tap % cv.f_w, fr = tap / cv.f_w;
      const int r = oh * cv.s_h - cv.pad_t + fr * cv.d_h;
      const int c = ow * cv.s_w - cv.pad_l + fc * cv.d_w;
      if (r >= 0 && r < cv.in_h && c >= 0 && c < cv.in_w)
        v = x[(((uint64_t)b * cv.in_h + r) * cv.in_w + c) * cv.in_c + d1];
    }
    col[i] = v;
  }
}

// Returns the packed copy of weight `id`, building it if needed.
int get_packed(tfjs_cuda_ctx* ctx, int32_t id, Buffer* src, int batch, int N, int taps,
               int cin, int cin_pad, int in_is_nk, const float** out) {
  const int layout = (taps << 20) ^ (cin_pad << 4) ^ (in_is_nk << 1) ^ (batch << 28) ^ 1;
  auto it = ctx->packed.find(id);
  if (it != ctx->packed.end() && it->second.version == src->version &&
      it->second.layout == layout && it->second.rows == N) {
    if (ctx->capturing) ctx->capture_packed.push_back(id);
    *out = it->second.ptr;
    return TFJS_CUDA_OK;
  }
  NOT_WHILE_CAPTURING(ctx, "packing a weight tensor");
  ctx_drop_packed(ctx, id);
  PackedWeight pw;
  const uint64_t total = (uint64_t)batch * N * taps * cin_pad;
  pw.bytes = total * 4;
  CUDA_TRY(ctx, cudaMallocAsync((void**)&pw.ptr, pw.bytes ? pw.bytes : 16, ctx->stream));
  pw.version = src->version;
  pw.rows = N;
  pw.k_pad = taps * cin_pad;
  pw.layout = layout;
  if (total) {
    pack_weight_kernel<<<grid_for(total, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)src->ptr, pw.ptr, total, N, taps, cin, cin_pad, in_is_nk);
    ctx->launches++;
    if (ctx->log_launches) ctx->launch_log.push_back("pack_weight_kernel");
    int rc = ctx_check(ctx, cudaGetLastError(), "pack_weight_kernel");
    if (rc) {
      cudaFreeAsync(pw.ptr, ctx->stream);
      return rc;
    }
  }
  ctx->packed[id] = pw;
  *out = pw.ptr;
  return TFJS_CUDA_OK;
}

int fill_act(tfjs_cuda_ctx* ctx, int activation, int prelu_len, int32_t prelu_id,
             double alpha, int channels, const char* who, ActParams* ap) {
  if (activation < TFJS_CUDA_ACT_LINEAR || activation > TFJS_CUDA_ACT_ELU)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: unknown activation %d", who, activation);
  ap->act = activation;
  ap->gelu_scale = ap->gelu_half = ap->gelu_one = 0.0f;
  ap->gelu_divide = 0;
  ap->prelu_len = 0;
  ap->prelu = nullptr;
  ap->alpha = alpha;
  if (activation == TFJS_CUDA_ACT_PRELU) {
    if (!prelu_id || (prelu_len != 1 && prelu_len != channels))
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                      "%s: prelu weights must be a scalar or one per output channel", who);
    Buffer* pb;
    int rc = ctx_get(ctx, prelu_id, (uint64_t)prelu_len * 4, who, &pb);
    if (rc) return rc;
    ap->prelu = (const float*)pb->ptr;
    ap->prelu_len = prelu_len;
  }
  return TFJS_CUDA_OK;
}

}  // namespace

// The packed copy of a 1x1 convolution's filter, as conv2d_impl builds it (shared cache
// entry), for kernels outside this file.
int packed_pointwise_filter(tfjs_cuda_ctx* ctx, int32_t filter_id, Buffer* w, int out_c, int in_c,
                            const float** out) {
  return get_packed(ctx, filter_id, w, 1, out_c, 1, in_c, in_c, 0, out);
}

extern "C" {

static int matmul_impl(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p, int32_t a_id,
                       int32_t b_id, int32_t bias_id, int32_t prelu_id, int32_t out_perm,
                       int32_t perm_p, int32_t perm_d, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (!p) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_matmul: null params");
  if (p->batch_a <= 0 || p->batch_b <= 0 || p->m < 0 || p->n < 0 || p->k < 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_matmul: bad dimensions");
  const int batch = p->batch_a > p->batch_b ? p->batch_a : p->batch_b;
  if (batch % p->batch_a != 0 || batch % p->batch_b != 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                    "fused_matmul: batch dims %d and %d do not broadcast", p->batch_a,
                    p->batch_b);
  if (p->bias_len != 0 && p->bias_len != 1 && p->bias_len != p->n)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "fused_matmul: bias must be a scalar or have N elements");
  Buffer *a, *b, *bias = nullptr, *out;
  int rc;
  if ((rc = ctx_get(ctx, a_id, (uint64_t)p->batch_a * p->m * p->k * 4, "fused_matmul a", &a))) return rc;
  if ((rc = ctx_get(ctx, b_id, (uint64_t)p->batch_b * p->k * p->n * 4, "fused_matmul b", &b))) return rc;
  if (p->bias_len && (rc = ctx_get(ctx, bias_id, (uint64_t)p->bias_len * 4, "fused_matmul bias", &bias))) return rc;
  if ((rc = ctx_get(ctx, out_id, (uint64_t)batch * p->m * p->n * 4, "fused_matmul out", &out))) return rc;
  GemmProblem pr;
  const bool gelu = p->activation == TFJS_CUDA_ACT_GELU_ERF;
  if ((rc = fill_act(ctx, gelu ? TFJS_CUDA_ACT_LINEAR : p->activation, p->prelu_len, prelu_id,
                     p->leakyrelu_alpha, p->n, "fused_matmul", &pr.ap)))
    return rc;
  if (gelu) {
    pr.ap.act = TFJS_CUDA_ACT_GELU_ERF;
    pr.ap.gelu_scale = p->gelu_scale;
    pr.ap.gelu_half = p->gelu_half;
    pr.ap.gelu_one = p->gelu_one;
    pr.ap.gelu_divide = p->gelu_divide != 0;
  }
  if ((uint64_t)batch * p->m * p->n == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  pr.a = (const float*)a->ptr;
  pr.b = (const float*)b->ptr;
  pr.c = (float*)out->ptr;
  pr.bias = bias ? (const float*)bias->ptr : nullptr;
  pr.bias_len = bias ? p->bias_len : 0;
  pr.M = p->m; pr.N = p->n; pr.K = p->k;
  pr.batch = batch; pr.batch_a = p->batch_a; pr.batch_b = p->batch_b;
  pr.trans_a = p->transpose_a != 0;
  pr.trans_b = p->transpose_b != 0;
  pr.is_conv = false;
  pr.out_perm = out_perm;
  pr.perm_p = perm_p;
  pr.perm_d = perm_d;

  const bool tc_ok = ctx->math_mode == TFJS_CUDA_MATH_TF32 && p->k > 0 && (p->k % 4) == 0 &&
                     !pr.trans_a;
  if (tc_ok) {
    Tf32Operands op;
    op.a = pr.a;
    op.lda = p->k;
    op.k_steps = (p->k + 31) / 32;
    bool ready = false;
    if (b->from_host) {
      const float* packed;
      if ((rc = get_packed(ctx, b_id, b, p->batch_b, p->n, 1, p->k, p->k, pr.trans_b ? 1 : 0,
                           &packed)))
        return rc;
      op.b = packed;
      op.ldb = p->k;
      op.b_layout = B_K_MAJOR;
      ready = true;
    } else if (pr.trans_b) {
      op.b = pr.b;
      op.ldb = p->k;
      op.b_layout = B_K_MAJOR;
      ready = true;
    } else if ((p->n % 4) == 0) {
      op.b = pr.b;
      op.ldb = p->n;
      op.b_layout = B_MN_MAJOR;
      ready = true;
    }
    if (ready) {
      rc = launch_gemm_tf32(ctx, pr, op);
      if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
      return rc;
    }
  }
  if (out_perm != 0)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "fused_matmul_heads: only the tensor-core path stores permuted results");
  rc = launch_gemm_simt(ctx, pr);
  if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
  return rc;
}

int tfjs_cuda_fused_matmul(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                           int32_t a_id, int32_t b_id, int32_t bias_id,
                           int32_t prelu_id, int32_t out_id) {
  return matmul_impl(ctx, p, a_id, b_id, bias_id, prelu_id, 0, 0, 0, out_id);
}

int tfjs_cuda_fused_matmul_heads(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                                 int32_t a_id, int32_t b_id, int32_t bias_id, int32_t prelu_id,
                                 int32_t layout, int32_t rows_or_heads, int32_t head_dim,
                                 int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (layout != TFJS_CUDA_HEADS_SPLIT && layout != TFJS_CUDA_HEADS_MERGE)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_matmul_heads: unknown layout %d", layout);
  if (rows_or_heads <= 0 || head_dim <= 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_matmul_heads: bad sizes");
  return matmul_impl(ctx, p, a_id, b_id, bias_id, prelu_id, layout, rows_or_heads, head_dim,
                     out_id);
}

int tfjs_cuda_fused_matmul_group(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                                 int32_t a_id, int32_t count, const int32_t* b_ids,
                                 const int32_t* bias_ids, int32_t layout, int32_t rows_or_heads,
                                 int32_t head_dim, const int32_t* out_ids) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  const char* who = "fused_matmul_group";
  if (!p || !b_ids || !out_ids || count < 2 || count > kMaxGemmGroup)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: bad arguments", who);
  if (p->batch_a != 1 || p->batch_b != 1 || p->m <= 0 || p->n <= 0 || p->k <= 0 ||
      p->transpose_a || (p->k % 4) != 0 || p->activation == TFJS_CUDA_ACT_PRELU ||
      p->activation == TFJS_CUDA_ACT_GELU_ERF || ctx->math_mode != TFJS_CUDA_MATH_TF32 ||
      (p->bias_len != 0 && p->bias_len != p->n))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: problem not taken by the grouped kernel", who);
  if (layout != 0 && layout != TFJS_CUDA_HEADS_SPLIT)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: layout %d", who, layout);
  Buffer* a;
  int rc;
  if ((rc = ctx_get(ctx, a_id, (uint64_t)p->m * p->k * 4, "fused_matmul_group a", &a))) return rc;
  GemmProblem pr;
  if ((rc = fill_act(ctx, p->activation, 0, 0, p->leakyrelu_alpha, p->n, who, &pr.ap))) return rc;
  cudaSetDevice(ctx->device);
  GemmGroup grp;
  grp.count = count;
  for (int i = 0; i < count; ++i) {
    Buffer *b, *bias = nullptr, *out;
    if ((rc = ctx_get(ctx, b_ids[i], (uint64_t)p->k * p->n * 4, "fused_matmul_group b", &b))) return rc;
    if (p->bias_len &&
        (rc = ctx_get(ctx, bias_ids ? bias_ids[i] : 0, (uint64_t)p->bias_len * 4, "fused_matmul_group bias", &bias)))
      return rc;
    if ((rc = ctx_get(ctx, out_ids[i], (uint64_t)p->m * p->n * 4, "fused_matmul_group out", &out))) return rc;
    for (int j = 0; j < i; ++j)
      if (out_ids[j] == out_ids[i])
        return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: two members share an output", who);
    if (b->from_host) {
      const float* packed;
      if ((rc = get_packed(ctx, b_ids[i], b, 1, p->n, 1, p->k, p->k, p->transpose_b ? 1 : 0, &packed)))
        return rc;
      grp.b[i] = packed;
    } else if (p->transpose_b) {
      grp.b[i] = (const float*)b->ptr;
    } else {
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "%s: the members' B operands must be weights", who);
    }
    grp.bias[i] = bias ? (const float*)bias->ptr : nullptr;
    grp.c[i] = (float*)out->ptr;
  }
  pr.a = (const float*)a->ptr;
  pr.b = grp.b[0];
  pr.c = grp.c[0];
  pr.bias = grp.bias[0];
  pr.bias_len = p->bias_len;
  pr.M = p->m; pr.N = p->n; pr.K = p->k;
  pr.batch = pr.batch_a = pr.batch_b = 1;
  pr.trans_b = p->transpose_b != 0;
  pr.out_perm = layout;
  pr.perm_p = rows_or_heads;
  pr.perm_d = head_dim;
  Tf32Operands op;
  op.a = pr.a;
  op.lda = p->k;
  op.k_steps = (p->k + 31) / 32;
  op.b = grp.b[0];
  op.ldb = p->k;
  op.b_layout = B_K_MAJOR;
  rc = launch_gemm_tf32(ctx, pr, op, &grp);
  if (rc == TFJS_CUDA_OK)
    for (int i = 0; i < count; ++i) ctx_mark_written(ctx, out_ids[i]);
  return rc;
}

static int conv2d_impl(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p, int32_t x_id,
                       int32_t filter_id, int32_t bias_id, int32_t prelu_id,
                       int32_t residual_id, int32_t post_activation, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (!p) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_conv2d: null params");
  if (p->batch < 0 || p->in_h < 0 || p->in_w < 0 || p->in_c < 0 || p->out_h < 0 ||
      p->out_w < 0 || p->out_c < 0 || p->filter_h <= 0 || p->filter_w <= 0 ||
      p->stride_h <= 0 || p->stride_w <= 0 || p->dilation_h <= 0 || p->dilation_w <= 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_conv2d: bad geometry");
  if (p->bias_len != 0 && p->bias_len != 1 && p->bias_len != p->out_c)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "fused_conv2d: bias must be a scalar or one per output channel");
  const uint64_t nx = (uint64_t)p->batch * p->in_h * p->in_w * p->in_c;
  const uint64_t M64 = (uint64_t)p->batch * p->out_h * p->out_w;
  const int taps = p->filter_h * p->filter_w;
  const uint64_t K64 = (uint64_t)taps * p->in_c;
  if (M64 > 0x7fffffffull || K64 > 0x7fffffffull)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "fused_conv2d: problem too large");
  Buffer *x, *w, *bias = nullptr, *out;
  int rc;
  if ((rc = ctx_get(ctx, x_id, nx * 4, "fused_conv2d x", &x))) return rc;
  if ((rc = ctx_get(ctx, filter_id, K64 * p->out_c * 4, "fused_conv2d filter", &w))) return rc;
  if (p->bias_len && (rc = ctx_get(ctx, bias_id, (uint64_t)p->bias_len * 4, "fused_conv2d bias", &bias))) return rc;
  if ((rc = ctx_get(ctx, out_id, M64 * p->out_c * 4, "fused_conv2d out", &out))) return rc;
  GemmProblem pr;
  if (residual_id) {
    Buffer* res;
    if ((rc = ctx_get(ctx, residual_id, M64 * p->out_c * 4, "fused_conv2d residual", &res)))
      return rc;
    if (post_activation != TFJS_CUDA_ACT_LINEAR && post_activation != TFJS_CUDA_ACT_RELU &&
        post_activation != TFJS_CUDA_ACT_RELU6)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                      "fused_conv2d_residual: post activation must be linear, relu or relu6");
    pr.residual = (const float*)res->ptr;
    pr.post_act = post_activation;
  }
  if ((rc = fill_act(ctx, p->activation, p->prelu_len, prelu_id, p->leakyrelu_alpha,
                     p->out_c, "fused_conv2d", &pr.ap)))
    return rc;
  if (M64 * p->out_c == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  pr.a = (const float*)x->ptr;
  pr.b = (const float*)w->ptr;
  pr.c = (float*)out->ptr;
  pr.bias = bias ? (const float*)bias->ptr : nullptr;
  pr.bias_len = bias ? p->bias_len : 0;
  pr.M = (int)M64; pr.N = p->out_c; pr.K = (int)K64;
  pr.batch = pr.batch_a = pr.batch_b = 1;
  pr.is_conv = true;
  ConvGeo& cv = pr.conv;
  cv.batch = p->batch; cv.in_h = p->in_h; cv.in_w = p->in_w; cv.in_c = p->in_c;
  cv.out_h = p->out_h; cv.out_w = p->out_w; cv.f_h = p->filter_h; cv.f_w = p->filter_w;
  cv.s_h = p->stride_h; cv.s_w = p->stride_w; cv.d_h = p->dilation_h; cv.d_w = p->dilation_w;
  cv.pad_t = p->pad_top; cv.pad_l = p->pad_left;

  if (ctx->math_mode == TFJS_CUDA_MATH_TF32 && K64 > 0 && stem_conv_supported(pr)) {
    // 3-channel image, 3 x 3 stride 2, 32 output channels: 27 multiply-adds per output, too
    // few to feed a tensor-core tile; a direct fp32 kernel (TFJS_CUDA_NO_DIRECT_STEM=1: the
    // staged-row GEMM below)
    static int off = -1;
    if (off < 0) off = getenv("TFJS_CUDA_NO_DIRECT_STEM") ? 1 : 0;
    if (!off) {
      rc = launch_stem_conv(ctx, pr);
      if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
      return rc;
    }
  }
  if (ctx->math_mode == TFJS_CUDA_MATH_TF32 && K64 > 0) {
    Tf32Operands op;
    const float* packed;
    const bool pointwise = taps == 1 && p->stride_h == 1 && p->stride_w == 1 &&
                           p->pad_top == 0 && p->pad_left == 0 && p->out_h == p->in_h &&
                           p->out_w == p->in_w;
    if (pointwise && (p->in_c % 4) == 0) {
      // 1x1 stride-1: the NHWC input already is the [M, K] operand.
      if ((rc = get_packed(ctx, filter_id, w, 1, p->out_c, 1, p->in_c, p->in_c, 0, &packed)))
        return rc;
      op.a = pr.a; op.lda = p->in_c; op.a_gather = 0;
      op.b = packed; op.ldb = p->in_c; op.b_layout = B_K_MAJOR;
      op.k_steps = (p->in_c + 31) / 32;
      pr.is_conv = false;
    } else if ((p->in_c % 4) == 0) {
      const int cin_pad = ((p->in_c + 31) / 32) * 32;
      if ((rc = get_packed(ctx, filter_id, w, 1, p->out_c, taps, p->in_c, cin_pad, 0, &packed)))
        return rc;
      op.a = pr.a; op.a_gather = 1; op.cin_pad = cin_pad;
      op.b = packed; op.ldb = (long long)taps * cin_pad; op.b_layout = B_K_MAJOR;
      op.k_steps = taps * (cin_pad / 32);
    } else if (PatchPlan plan; ((int)K64 + 31) / 32 * 32 <= 512 &&
                               tf32_patch_plan(cv, pr.M, pr.N, ctx->sm_count, &plan)) {
      // few input channels (image stems), image rows staged in shared memory; K is
      // padded to a multiple of 32 in the packed filter
      const int k_pad = ((int)K64 + 31) / 32 * 32;
      if ((rc = get_packed(ctx, filter_id, w, 1, p->out_c, 1, (int)K64, k_pad, 0, &packed)))
        return rc;
      op.a = pr.a; op.a_gather = 3;
      op.b = packed; op.ldb = k_pad; op.b_layout = B_K_MAJOR;
      op.k_steps = k_pad / 32;
    } else if (p->filter_h <= 15 && p->filter_w <= 15 && ((int)K64 + 31) / 32 * 32 <= 512 &&
               (uint64_t)((p->filter_h - 1) * p->dilation_h * p->in_w +
                          (p->filter_w - 1) * p->dilation_w + 1) * p->in_c < (1u << 24)) {
      // few input channels (image stems): the gather warps assemble the im2col rows
      // element by element; K is padded to a multiple of 32 in the packed filter
      const int k_pad = ((int)K64 + 31) / 32 * 32;
      if ((rc = get_packed(ctx, filter_id, w, 1, p->out_c, 1, (int)K64, k_pad, 0, &packed)))
        return rc;
      op.a = pr.a; op.a_gather = 2;
      op.b = packed; op.ldb = k_pad; op.b_layout = B_K_MAJOR;
      op.k_steps = k_pad / 32;
    } else {
      const int ld = (((int)K64 + 3) / 4) * 4;
      void* col;
      if ((rc = ctx_scratch(ctx, M64 * ld * 4, &col))) return rc;
      const uint64_t total = M64 * ld;
      im2col_kernel<<<grid_for(total, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
          pr.a, (float*)col, total, (int)K64, ld, cv);
      LAUNCH_CHECK(ctx, "im2col_kernel");
      // Weights: [K][Cout] -> [Cout][ld], K-contiguous, zero padded.
      if ((rc = get_packed(ctx, filter_id, w, 1, p->out_c, 1, (int)K64, ld, 0, &packed)))
        return rc;
      op.a = (const float*)col; op.lda = ld; op.a_gather = 0;
      op.b = packed; op.ldb = ld; op.b_layout = B_K_MAJOR;
      op.k_steps = ((int)K64 + 31) / 32;
      pr.is_conv = false;
    }
    rc = launch_gemm_tf32(ctx, pr, op);
    if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
    return rc;
  }
  rc = launch_gemm_simt(ctx, pr);
  if (rc == TFJS_CUDA_OK) ctx_mark_written(ctx, out_id);
  return rc;
}

int tfjs_cuda_fused_conv2d(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                           int32_t x_id, int32_t filter_id, int32_t bias_id,
                           int32_t prelu_id, int32_t out_id) {
  return conv2d_impl(ctx, p, x_id, filter_id, bias_id, prelu_id, 0, TFJS_CUDA_ACT_LINEAR, out_id);
}

int tfjs_cuda_fused_conv2d_residual(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                                    int32_t x_id, int32_t filter_id, int32_t bias_id,
                                    int32_t prelu_id, int32_t residual_id,
                                    int32_t post_activation, int32_t out_id) {
  if (ctx && !residual_id)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_conv2d_residual: residual tensor missing");
  return conv2d_impl(ctx, p, x_id, filter_id, bias_id, prelu_id, residual_id, post_activation,
                     out_id);
}

}  // extern "C"
