// Problem description shared by the GEMM front end (matmul.cu) and its two
// back ends: the tcgen05 TF32 kernels and the fp32 SIMT kernels.
#pragma once
#include "common.cuh"

struct ConvGeo {
  int batch, in_h, in_w, in_c;
  int out_h, out_w;
  int f_h, f_w;
  int s_h, s_w, d_h, d_w, pad_t, pad_l;
};

struct GemmProblem {
  // C[batch][M][N] = act(A . B + bias).  For a convolution A is the implicit
  // im2col matrix of x (M = batch*out_h*out_w rows, K = f_h*f_w*in_c) and the
  // GEMM batch is 1.
  const float* a = nullptr;
  const float* b = nullptr;
  float* c = nullptr;
  const float* bias = nullptr;
  int bias_len = 0;
  ActParams ap;
  int M = 0, N = 0, K = 0;
  int batch = 1, batch_a = 1, batch_b = 1;
  bool trans_a = false, trans_b = false;
  bool is_conv = false;
  ConvGeo conv;
  // optional second stage of the epilogue: out = post_act(act(A.B + bias) + residual),
  // residual shaped like the output (the bottleneck shortcut of a residual network)
  const float* residual = nullptr;
  int post_act = 0;  // TFJS_CUDA_ACT_LINEAR or TFJS_CUDA_ACT_RELU / RELU6
  // optional permuted store for attention heads (tensor-core kernels only):
  //   1  batch == 1, M = B*perm_p, N = H*perm_d: the [B, S, H, D] view of the result is
  //      written as [B, H, S, D] (the heads split of a projection, S = perm_p, D = perm_d)
  //   2  batch = B*perm_p, N = perm_d: the [B, H, S, D] result is written as [B, S, H, D]
  //      (the heads merged back, H = perm_p, S = M, D = perm_d)
  int out_perm = 0;
  int perm_p = 0, perm_d = 0;
};

// B operand layouts understood by the tensor-core kernel.
enum BLayout {
  B_K_MAJOR = 0,   // [batch][N][ldb] with K contiguous (transposed / packed weights)
  B_MN_MAJOR = 1   // [batch][K][ldb] with N contiguous (plain row-major [K, N])
};

struct Tf32Operands {
  const float* a = nullptr;  // K-major A: [batch_a][M][lda] (or x for a gathered conv)
  long long lda = 0;         // elements between consecutive rows of A
  int a_gather = 0;          // 1: A comes from NHWC x by the conv geometry, 32-channel chunks;
                             // 2: same, one float at a time (channels not a multiple of 4)
                             // 3: same, image rows staged in shared memory
  const float* b = nullptr;
  long long ldb = 0;         // elements between consecutive rows of the B storage
  int b_layout = B_K_MAJOR;
  int k_steps = 0;           // number of 32-wide K steps
  int cin_pad = 0;           // gathered conv: per-tap channel count rounded up to 32
};

// Shared-memory plan of the staged-row gather (a_gather 3); tf32_patch_plan returns
// false when the shape cannot use it.
struct PatchPlan {
  int bytes, pitch, ml, rows;  // per buffer; floats between rows; left margin; rows held
  int bufs;                    // buffers that fit (2 to 4)
};
// Direct fp32 kernel for a 3-channel image, 3 x 3 stride-2 filter, 32 output channels
// (stem_conv.cu): whether it takes the problem, and its launch.
bool stem_conv_supported(const GemmProblem& pr);
int launch_stem_conv(tfjs_cuda_ctx* ctx, const GemmProblem& pr);
bool tf32_patch_plan(const ConvGeo& cv, int M, int N, int sm_count, PatchPlan* plan);

int launch_gemm_simt(tfjs_cuda_ctx* ctx, const GemmProblem& pr);
// Products that share A and every dimension of the problem (the query, key and value
// projections of an attention layer): member i reads b[i] (K-major, packed) and bias[i] and
// writes c[i].  One launch walks the tiles of all members, so three products of 1.3 waves
// each become one of 3.9.  Only the CTA-pair kernel takes a group; for anything else
// launch_gemm_tf32 returns TFJS_CUDA_UNSUPPORTED and the caller launches the members one
// by one.
constexpr int kMaxGemmGroup = 4;
struct GemmGroup {
  int count = 0;
  const float* b[kMaxGemmGroup];
  const float* bias[kMaxGemmGroup];
  float* c[kMaxGemmGroup];
};

int launch_gemm_tf32(tfjs_cuda_ctx* ctx, const GemmProblem& pr, const Tf32Operands& op,
                     const GemmGroup* group = nullptr);
