// fp32 SIMT GEMM / implicit-GEMM convolution.
//
// Used when the math mode is TFJS_CUDA_MATH_FP32 and for shapes the tensor-core
// kernels do not take (K or N not a multiple of 4, transposed A).  Each output
// element is accumulated with fmaf in increasing k, which for a convolution is
// the reference's (wR, wC, d1) order (tfjs-backend-cpu/src/kernels/Conv2D.ts:64-100),
// so this path agrees with the CPU backend to within double-rounding ties.
#include "common.cuh"
#include "gemm.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int kThreads = 256;

struct SimtGemmArgs {
  const float* a;
  const float* b;
  float* c;
  const float* bias;
  int bias_len;
  ActParams ap;
  int M, N, K;
  int batch, batch_a, batch_b;
  long long a_batch_stride, b_batch_stride;
  long long a_row_stride, a_k_stride;  // matmul A addressing
  long long b_k_stride, b_n_stride;
  ConvGeo conv;                        // used when IS_CONV
  const float* residual;
  int post_act;
};

template <bool IS_CONV>
__device__ __forceinline__ float load_a(const SimtGemmArgs& g, const float* a,
                                        int m, int k) {
  if (m >= g.M || k >= g.K) return 0.0f;
  if (!IS_CONV) return a[m * g.a_row_stride + k * g.a_k_stride];
  const ConvGeo& cv = g.conv;
  const int ow = m % cv.out_w;
  const int t = m / cv.out_w;
  const int oh = t % cv.out_h;
  const int b = t / cv.out_h;
  const int d1 = k % cv.in_c;
  const int tap = k / cv.in_c;
  const int fc = tap % cv.f_w, fr = tap / cv.f_w;
  const int r = oh * cv.s_h - cv.pad_t + fr * cv.d_h;
  const int c = ow * cv.s_w - cv.pad_l + fc * cv.d_w;
  if (r < 0 || r >= cv.in_h || c < 0 || c >= cv.in_w) return 0.0f;
  return a[(((long long)b * cv.in_h + r) * cv.in_w + c) * cv.in_c + d1];
}

template <bool IS_CONV>
__global__ void __launch_bounds__(kThreads)
gemm_simt_kernel(SimtGemmArgs g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int bz = blockIdx.z;
  const float* a = g.a + (long long)(bz % g.batch_a) * g.a_batch_stride;
  const float* b = g.b + (long long)(bz % g.batch_b) * g.b_batch_stride;
  float* c = g.c + (long long)bz * g.M * g.N;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int k0 = 0; k0 < g.K; k0 += BK) {
    // A tile: 64 x 16 elements, 4 per thread.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * kThreads;
      const int kk = idx % BK, mm = idx / BK;
      As[kk][mm] = load_a<IS_CONV>(g, a, m0 + mm, k0 + kk);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = threadIdx.x + e * kThreads;
      const int nn = idx % BN, kk = idx / BN;
      const int k = k0 + kk, n = n0 + nn;
      Bs[kk][nn] = (k < g.K && n < g.N) ? b[k * g.b_k_stride + n * g.b_n_stride] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.bias_len) v = __fadd_rn(v, g.bias[g.bias_len == 1 ? 0 : n]);
      v = apply_act(v, g.ap, n);
      if (g.residual) {
        v = __fadd_rn(g.residual[(long long)bz * g.M * g.N + (long long)m * g.N + n], v);
        if (g.post_act == TFJS_CUDA_ACT_RELU) v = js_relu(v);
        else if (g.post_act == TFJS_CUDA_ACT_RELU6) v = js_relu6(v);
      }
      c[(long long)m * g.N + n] = v;
    }
  }
}

}  // namespace

int launch_gemm_simt(tfjs_cuda_ctx* ctx, const GemmProblem& pr) {
  SimtGemmArgs g;
  g.a = pr.a; g.b = pr.b; g.c = pr.c;
  g.bias = pr.bias; g.bias_len = pr.bias ? pr.bias_len : 0;
  g.ap = pr.ap;
  g.M = pr.M; g.N = pr.N; g.K = pr.K;
  g.batch = pr.batch; g.batch_a = pr.batch_a; g.batch_b = pr.batch_b;
  g.a_batch_stride = (long long)pr.M * pr.K;
  g.b_batch_stride = (long long)pr.K * pr.N;
  g.a_row_stride = pr.trans_a ? 1 : pr.K;
  g.a_k_stride = pr.trans_a ? pr.M : 1;
  g.b_k_stride = pr.trans_b ? 1 : pr.N;
  g.b_n_stride = pr.trans_b ? pr.K : 1;
  g.conv = pr.conv;
  g.residual = pr.residual;
  g.post_act = pr.post_act;
  if (pr.batch > 65535)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "matmul: batch %d too large for the fp32 path", pr.batch);
  dim3 grid((pr.M + BM - 1) / BM, (pr.N + BN - 1) / BN, pr.batch);
  if (grid.y > 65535)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "matmul: N too large for the fp32 path");
  if (pr.is_conv) gemm_simt_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(g);
  else gemm_simt_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(g);
  LAUNCH_CHECK(ctx, "gemm_simt_kernel");
  return TFJS_CUDA_OK;
}
