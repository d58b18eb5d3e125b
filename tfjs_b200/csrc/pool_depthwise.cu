// MaxPool / AvgPool and FusedDepthwiseConv2D: NHWC, bandwidth-bound SIMT kernels.
// A thread owns four adjacent channels of one output pixel and moves them with
// 128-bit loads/stores, so a warp reads and writes 512 contiguous bytes per
// tap; overlapping taps of neighbouring pixels are served by L1/L2.
#include <stdlib.h>

#include "common.cuh"
#include "ptx.cuh"

namespace {

constexpr int kThreads = 256;

struct Geo {
  int batch, in_h, in_w, c;     // c = input channels
  int out_h, out_w;
  int f_h, f_w;                 // pool: effective window; conv: filter taps
  int s_h, s_w, d_h, d_w, pad_t, pad_l;
  int ch_mul;
};

// ---- pooling: tfjs-backend-cpu/src/utils/pool_utils.ts:43-84 -----------------
// The window is clipped to the image; max starts at -inf and moves on
// `pixel > max` (NaN is never selected); avg divides the double sum by the
// number of in-bounds taps.
template <bool IS_MAX, int VEC>
__global__ void pool2d_kernel(const float* __restrict__ x, float* __restrict__ y,
                              Geo g) {
  const int cv = g.c / VEC;
  const uint64_t n = (uint64_t)g.batch * g.out_h * g.out_w * cv;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const int c = (int)(i % cv) * VEC;
    uint64_t rem = i / cv;
    const int ow = (int)(rem % g.out_w);
    rem /= g.out_w;
    const int oh = (int)(rem % g.out_h);
    const int b = (int)(rem / g.out_h);
    const int r0 = oh * g.s_h - g.pad_t, c0 = ow * g.s_w - g.pad_l;
    // First in-bounds tap on the dilation grid, as `xR = xRMin; xR += dilation`
    // does in the reference (it starts at max(0, corner), not at a grid point).
    const int r_min = r0 > 0 ? r0 : 0, c_min = c0 > 0 ? c0 : 0;
    const int r_max = min(g.in_h, g.f_h + r0), c_max = min(g.in_w, g.f_w + c0);
    float mx[VEC];
    double sum[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) { mx[v] = -INFINITY; sum[v] = 0.0; }
    int count = 0;
    for (int r = r_min; r < r_max; r += g.d_h) {
      for (int cc = c_min; cc < c_max; cc += g.d_w) {
        const float* p = x + (((uint64_t)b * g.in_h + r) * g.in_w + cc) * g.c + c;
        float px[VEC];
        if (VEC == 4) {
          const float4 t = *reinterpret_cast<const float4*>(p);
          px[0] = t.x; px[1 % VEC] = t.y; px[2 % VEC] = t.z; px[3 % VEC] = t.w;
        } else {
          px[0] = p[0];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          if (IS_MAX) { if (px[v] > mx[v]) mx[v] = px[v]; }
          else sum[v] += (double)px[v];
        }
        ++count;
      }
    }
    float out[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v)
      out[v] = IS_MAX ? mx[v] : (float)(sum[v] / (double)count);
    float* q = y + (((uint64_t)b * g.out_h + oh) * g.out_w + ow) * g.c + c;
    if (VEC == 4)
      *reinterpret_cast<float4*>(q) = make_float4(out[0], out[1 % VEC], out[2 % VEC], out[3 % VEC]);
    else
      q[0] = out[0];
  }
}

// 3x3 stride-2 max pooling (the pool behind a residual network's stem): a thread owns 4
// channels of ROWS x 4 outputs, so the input rows and the nine input columns its windows
// share are loaded once (6.75 loads per output at ROWS = 1 instead of 9: the gather form is
// bound by the L1 data path, not by HBM), with every loop bound known at compile time.  Same
// rule as above: -inf start, a NaN tap is never selected (fmaxf returns the other operand),
// taps outside the image are skipped.  Measured on [128, 112, 112, 64]: gather form 124 us,
// ROWS = 1 110 us, ROWS = 2 127 us (half the threads, twice the registers).
template <int ROWS>
__global__ void maxpool3x3s2_kernel(const float* __restrict__ x, float* __restrict__ y, Geo g) {
  const int cv = g.c >> 2;
  const int wq = (g.out_w + 3) >> 2;                       // groups of four output columns
  const int hq = (g.out_h + ROWS - 1) / ROWS;              // groups of ROWS output rows
  const uint64_t n = (uint64_t)g.batch * hq * wq * cv;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int c = (int)(i % cv) * 4;
    uint64_t rem = i / cv;
    const int ow0 = (int)(rem % wq) * 4;
    rem /= wq;
    const int oh0 = (int)(rem % hq) * ROWS;
    const int b = (int)(rem / hq);
    const int r0 = oh0 * 2 - g.pad_t, c0 = ow0 * 2 - g.pad_l;
    float mx[ROWS][4][4];
#pragma unroll
    for (int t = 0; t < ROWS; ++t)
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int v = 0; v < 4; ++v) mx[t][s][v] = -INFINITY;
#pragma unroll
    for (int fr = 0; fr < 2 * ROWS + 1; ++fr) {
      const int r = r0 + fr;
      if (r < 0 || r >= g.in_h) continue;
      const float* row = x + (((uint64_t)b * g.in_h + r) * g.in_w) * g.c + c;
#pragma unroll
      for (int j = 0; j < 9; ++j) {
        const int cc = c0 + j;
        if (cc < 0 || cc >= g.in_w) continue;
        const float4 q4 = __ldg(reinterpret_cast<const float4*>(row + (uint64_t)cc * g.c));
        const float px[4] = {q4.x, q4.y, q4.z, q4.w};
        // input row fr belongs to the output rows t with 2 t <= fr <= 2 t + 2, input column
        // j to the windows s with 2 s <= j <= 2 s + 2
#pragma unroll
        for (int t = 0; t < ROWS; ++t) {
          if (fr < 2 * t || fr > 2 * t + 2) continue;
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            if (j < 2 * s || j > 2 * s + 2) continue;
#pragma unroll
            for (int v = 0; v < 4; ++v) mx[t][s][v] = fmaxf(mx[t][s][v], px[v]);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < ROWS; ++t) {
      if (oh0 + t >= g.out_h) break;
      float* q = y + (((uint64_t)b * g.out_h + oh0 + t) * g.out_w + ow0) * g.c + c;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        if (ow0 + s >= g.out_w) break;
        *reinterpret_cast<float4*>(q + (uint64_t)s * g.c) =
            make_float4(mx[t][s][0], mx[t][s][1], mx[t][s][2], mx[t][s][3]);
      }
    }
  }
}

// ---- depthwise conv: tfjs-backend-cpu/src/kernels/DepthwiseConv2dNative.ts:62-99
// Per output element the taps arrive in (wR, wC) order and every MAC rounds the
// running value to fp32; fmaf reproduces that up to double-rounding ties.
// Then bias (fp32 add) and the activation, as FusedDepthwiseConv2D.ts:42-60.
template <int VEC>  // channel multiplier 1, VEC channels per thread
__global__ void depthwise_kernel(const float* __restrict__ x,
                                 const float* __restrict__ w,
                                 const float* __restrict__ bias, int bias_len,
                                 ActParams ap, float* __restrict__ y, Geo g) {
  const int cv = g.c / VEC;
  const uint64_t n = (uint64_t)g.batch * g.out_h * g.out_w * cv;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const int c = (int)(i % cv) * VEC;
    uint64_t rem = i / cv;
    const int ow = (int)(rem % g.out_w);
    rem /= g.out_w;
    const int oh = (int)(rem % g.out_h);
    const int b = (int)(rem / g.out_h);
    const int r0 = oh * g.s_h - g.pad_t, c0 = ow * g.s_w - g.pad_l;
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.0f;
    for (int fr = 0; fr < g.f_h; ++fr) {
      const int r = r0 + fr * g.d_h;
      if (r < 0 || r >= g.in_h) continue;
      for (int fc = 0; fc < g.f_w; ++fc) {
        const int cc = c0 + fc * g.d_w;
        if (cc < 0 || cc >= g.in_w) continue;
        const float* p = x + (((uint64_t)b * g.in_h + r) * g.in_w + cc) * g.c + c;
        const float* q = w + ((uint64_t)fr * g.f_w + fc) * g.c + c;
        if (VEC == 4) {
          const float4 xv = *reinterpret_cast<const float4*>(p);
          const float4 wv = __ldg(reinterpret_cast<const float4*>(q));
          acc[0] = fmaf(xv.x, wv.x, acc[0]);
          acc[1 % VEC] = fmaf(xv.y, wv.y, acc[1 % VEC]);
          acc[2 % VEC] = fmaf(xv.z, wv.z, acc[2 % VEC]);
          acc[3 % VEC] = fmaf(xv.w, wv.w, acc[3 % VEC]);
        } else {
          acc[0] = fmaf(p[0], __ldg(q), acc[0]);
        }
      }
    }
    float* o = y + (((uint64_t)b * g.out_h + oh) * g.out_w + ow) * g.c + c;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float t = acc[v];
      if (bias_len) t = __fadd_rn(t, bias[bias_len == 1 ? 0 : c + v]);
      acc[v] = apply_act(t, ap, c + v);
    }
    if (VEC == 4)
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
    else
      o[0] = acc[0];
  }
}

// 3x3, dilation 1, channel multiplier 1, C % 4 == 0 (every MobileNet layer).
// blockIdx.y is the output row (b, oh); a thread owns 4 channels of S adjacent
// output columns, so each input row segment is loaded once into registers and
// reused by the S outputs, and all index arithmetic is 32-bit and per thread,
// not per tap.  Filter taps and accumulation order are those of
// DepthwiseConv2dNative.ts:62-99 ((wR, wC) per output element).
template <int STRIDE, int S, int ACT>
__global__ void __launch_bounds__(128)
depthwise3x3_kernel(const float* __restrict__ x, const float* __restrict__ w,
                    const float* __restrict__ bias, int bias_len, ActParams ap,
                    float* __restrict__ y, Geo g, int rows_total) {
  constexpr int NC = (S - 1) * STRIDE + 3;  // input columns a strip touches
  const int c4n = g.c >> 2;
  const int strips = (g.out_w + S - 1) / S;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= strips * c4n) return;
  const int c4 = t % c4n;
  const int ow0 = (t / c4n) * S;
  const float4* w4 = reinterpret_cast<const float4*>(w) + c4;
  float4 wv[9];
#pragma unroll
  for (int k = 0; k < 9; ++k) wv[k] = __ldg(w4 + k * c4n);
  float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (bias_len == 1) {
    const float b0 = __ldg(bias);
    bv = make_float4(b0, b0, b0, b0);
  } else if (bias_len > 1) {
    bv = __ldg(reinterpret_cast<const float4*>(bias) + c4);
  }
  const int c_lo = ow0 * STRIDE - g.pad_l;
  for (int row = blockIdx.y; row < rows_total; row += gridDim.y) {
    const int oh = row % g.out_h;
    const int b = row / g.out_h;
    float4 acc[S];
#pragma unroll
    for (int s = 0; s < S; ++s) acc[s] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int fr = 0; fr < 3; ++fr) {
      const int r = oh * STRIDE - g.pad_t + fr;
      if (r < 0 || r >= g.in_h) continue;
      const float4* xrow =
          reinterpret_cast<const float4*>(x) + ((size_t)b * g.in_h + r) * g.in_w * c4n + c4;
      float4 xin[NC];
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int cc = c_lo + i;
        xin[i] = (cc >= 0 && cc < g.in_w) ? __ldg(xrow + (size_t)cc * c4n)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int s = 0; s < S; ++s) {
#pragma unroll
        for (int fc = 0; fc < 3; ++fc) {
          // a tap outside the image is skipped by the reference; it adds 0 here
          const float4 xv = xin[s * STRIDE + fc];
          const float4 wk = wv[fr * 3 + fc];
          acc[s].x = fmaf(xv.x, wk.x, acc[s].x);
          acc[s].y = fmaf(xv.y, wk.y, acc[s].y);
          acc[s].z = fmaf(xv.z, wk.z, acc[s].z);
          acc[s].w = fmaf(xv.w, wk.w, acc[s].w);
        }
      }
    }
    float4* yrow = reinterpret_cast<float4*>(y) + ((size_t)row * g.out_w) * c4n + c4;
#pragma unroll
    for (int s = 0; s < S; ++s) {
      if (ow0 + s >= g.out_w) break;
      float o[4] = {acc[s].x, acc[s].y, acc[s].z, acc[s].w};
      const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float v = bias_len ? __fadd_rn(o[k], bb[k]) : o[k];
        if (ACT == TFJS_CUDA_ACT_RELU) v = v != v ? v : fmaxf(v, 0.0f);
        else if (ACT == TFJS_CUDA_ACT_RELU6) v = v != v ? v : fminf(fmaxf(v, 0.0f), 6.0f);
        else if (ACT != TFJS_CUDA_ACT_LINEAR) v = apply_act(v, ap, c4 * 4 + k);
        o[k] = v;
      }
      yrow[(size_t)(ow0 + s) * c4n] = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
}

template <int STRIDE, int S>
void launch_depthwise3x3(tfjs_cuda_ctx* ctx, const float* x, const float* w, const float* bias,
                         int bias_len, const ActParams& ap, float* y, const Geo& g) {
  const int c4n = g.c >> 2;
  const int strips = (g.out_w + S - 1) / S;
  const int rows_total = g.batch * g.out_h;
  dim3 grid((strips * c4n + 127) / 128, rows_total < 65535 ? rows_total : 65535);
  switch (ap.act) {
    case TFJS_CUDA_ACT_LINEAR:
      depthwise3x3_kernel<STRIDE, S, TFJS_CUDA_ACT_LINEAR><<<grid, 128, 0, ctx->stream>>>(
          x, w, bias, bias_len, ap, y, g, rows_total);
      break;
    case TFJS_CUDA_ACT_RELU:
      depthwise3x3_kernel<STRIDE, S, TFJS_CUDA_ACT_RELU><<<grid, 128, 0, ctx->stream>>>(
          x, w, bias, bias_len, ap, y, g, rows_total);
      break;
    case TFJS_CUDA_ACT_RELU6:
      depthwise3x3_kernel<STRIDE, S, TFJS_CUDA_ACT_RELU6><<<grid, 128, 0, ctx->stream>>>(
          x, w, bias, bias_len, ap, y, g, rows_total);
      break;
    default:  // resolved per element by apply_act
      depthwise3x3_kernel<STRIDE, S, TFJS_CUDA_ACT_ELU><<<grid, 128, 0, ctx->stream>>>(
          x, w, bias, bias_len, ap, y, g, rows_total);
      break;
  }
}

// ---- 3x3 depthwise through TMA-staged input tiles -------------------------------
// A CTA walks (image, output tile, 32-channel chunk) work items.  The input patch
// of a tile (with its one-pixel halo; zero outside the image, which is what
// skipping those taps amounts to) arrives in shared memory by one 4-D TMA load;
// two buffers alternate so the load of the next tile overlaps the arithmetic of
// the current one.  A thread owns 4 channels of S adjacent output columns.
template <int STRIDE, int TW_>
struct DwTile {
  static constexpr int TW = TW_;                      // output tile width (16, 14 or 28)
  static constexpr int TH = STRIDE == 1 ? 8 : 4;      // output tile height
  // outputs per strip; 28-wide tiles take 7, so that a tile is exactly 32 strips (one pass)
  static constexpr int S = TW_ == 28 ? 7 : (STRIDE == 1 && TW_ == 16) ? 4 : 2;
  static constexpr int NSTRIPS = (TW / S) * TH;       // strips per tile, 32 per pass
  static constexpr int IW = (TW - 1) * STRIDE + 3;    // input patch
  static constexpr int IH = (TH - 1) * STRIDE + 3;
  static constexpr int BUF_BYTES = IW * IH * 128;
  static constexpr int SMEM_BYTES = 2 * BUF_BYTES + 128 + 64;
};

struct DwTiles {
  int tiles_w, tiles_h, chunks, total;
};

template <int STRIDE, int TW_, int ACT>
__global__ void __launch_bounds__(256, 2)
depthwise3x3_tma_kernel(const __grid_constant__ CUtensorMap tm_x, const float* __restrict__ w,
                        const float* __restrict__ bias, int bias_len, ActParams ap,
                        float* __restrict__ y, Geo g, DwTiles tl, int* flag) {
  using T = DwTile<STRIDE, TW_>;
  constexpr int NC = (T::S - 1) * STRIDE + 3;
  extern __shared__ uint8_t dw_smem_raw[];
  const uint32_t base = (smem_u32(dw_smem_raw) + 127u) & ~127u;
  const uint32_t bar0 = base + 2 * T::BUF_BYTES;
  const int tid = threadIdx.x;
  const int c4 = tid & 7;
  constexpr int strips_per_row = T::TW / T::S;

  if (tid == 0) {
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto decode = [&](int item, int& n, int& th, int& tw, int& cc) {
    cc = item % tl.chunks;
    int rest = item / tl.chunks;
    tw = rest % tl.tiles_w;
    rest /= tl.tiles_w;
    th = rest % tl.tiles_h;
    n = rest / tl.tiles_h;
  };
  auto issue = [&](int item, int buf) {
    int n, th, tw, cc;
    decode(item, n, th, tw, cc);
    const uint32_t bar = bar0 + 8 * buf;
    mbar_expect_tx(bar, T::BUF_BYTES);
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(base + buf * T::BUF_BYTES),
        "l"(&tm_x), "r"(bar), "r"(cc * 32), "r"(tw * T::TW * STRIDE - g.pad_l),
        "r"(th * T::TH * STRIDE - g.pad_t), "r"(n)
        : "memory");
  };

  int item = blockIdx.x;
  if (tid == 0 && item < tl.total) issue(item, 0);
  uint32_t phase[2] = {0, 0};
  int buf = 0;
  for (; item < tl.total; item += gridDim.x, buf ^= 1) {
    const int next = item + gridDim.x;
    // every thread finished reading buffer buf^1 at the barrier that ended the
    // previous iteration, so it can be refilled now
    if (tid == 0 && next < tl.total) issue(next, buf ^ 1);
    int n, th, tw, cc;
    decode(item, n, th, tw, cc);
    const int c = cc * 32 + c4 * 4;
    const bool c_ok = c < g.c;
    // Arithmetic on packed pairs (fma.rn.f32x2: two independent fp32 FMAs per
    // instruction, each rounded like the scalar one): a float4 of channels is two
    // 64-bit registers.
    unsigned long long wv[9][2];
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c_ok) {
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(w + k * g.c + c));
        asm("mov.b64 %0, {%1, %2};" : "=l"(wv[k][0]) : "f"(t.x), "f"(t.y));
        asm("mov.b64 %0, {%1, %2};" : "=l"(wv[k][1]) : "f"(t.z), "f"(t.w));
      }
      if (bias_len == 1) {
        const float b0 = __ldg(bias);
        bv = make_float4(b0, b0, b0, b0);
      } else if (bias_len > 1) {
        bv = __ldg(reinterpret_cast<const float4*>(bias + c));
      }
    }
    if (!mbar_wait(bar0 + 8 * buf, phase[buf])) {
      if (tid == 0) atomicExch(flag, 7);
      break;
    }
    phase[buf] ^= 1;
    for (int strip = tid >> 3; strip < T::NSTRIPS; strip += 32) {
    const int sr = strip / strips_per_row;        // row inside the tile
    const int sc = (strip % strips_per_row) * T::S;
    const int oh = th * T::TH + sr;
    const int ow0 = tw * T::TW + sc;
    if (c_ok && oh < g.out_h && ow0 < g.out_w) {
      unsigned long long acc[T::S][2];
#pragma unroll
      for (int s = 0; s < T::S; ++s) acc[s][0] = acc[s][1] = 0ull;
      const uint32_t tile = base + buf * T::BUF_BYTES + (uint32_t)c4 * 16u;
#pragma unroll
      for (int fr = 0; fr < 3; ++fr) {
        const uint32_t row = tile + (uint32_t)((sr * STRIDE + fr) * T::IW + sc * STRIDE) * 128u;
        unsigned long long xin[NC][2];
#pragma unroll
        for (int i = 0; i < NC; ++i)
          asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];"
                       : "=l"(xin[i][0]), "=l"(xin[i][1])
                       : "r"(row + (uint32_t)i * 128u));
#pragma unroll
        for (int s = 0; s < T::S; ++s) {
#pragma unroll
          for (int fc = 0; fc < 3; ++fc) {
            asm("fma.rn.f32x2 %0, %1, %2, %0;"
                : "+l"(acc[s][0]) : "l"(xin[s * STRIDE + fc][0]), "l"(wv[fr * 3 + fc][0]));
            asm("fma.rn.f32x2 %0, %1, %2, %0;"
                : "+l"(acc[s][1]) : "l"(xin[s * STRIDE + fc][1]), "l"(wv[fr * 3 + fc][1]));
          }
        }
      }
      float* yrow = y + (((size_t)n * g.out_h + oh) * g.out_w + ow0) * g.c + c;
#pragma unroll
      for (int s = 0; s < T::S; ++s) {
        if (ow0 + s >= g.out_w) break;
        float o[4];
        asm("mov.b64 {%0, %1}, %2;" : "=f"(o[0]), "=f"(o[1]) : "l"(acc[s][0]));
        asm("mov.b64 {%0, %1}, %2;" : "=f"(o[2]), "=f"(o[3]) : "l"(acc[s][1]));
        const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float v = bias_len ? __fadd_rn(o[k], bb[k]) : o[k];
          // max.NaN / min.NaN keep a NaN input, as Math.max / Math.min do
          if (ACT == TFJS_CUDA_ACT_RELU) {
            asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v));
          } else if (ACT == TFJS_CUDA_ACT_RELU6) {
            asm("max.NaN.f32 %0, %0, 0f00000000;" : "+f"(v));
            asm("min.NaN.f32 %0, %0, 0f40C00000;" : "+f"(v));
          } else if (ACT != TFJS_CUDA_ACT_LINEAR) {
            v = apply_act(v, ap, c + k);
          }
          o[k] = v;
        }
        *reinterpret_cast<float4*>(yrow + (size_t)s * g.c) = make_float4(o[0], o[1], o[2], o[3]);
      }
    }
    }
    __syncthreads();
  }
}

template <int STRIDE, int TW_>
int launch_depthwise3x3_tma(tfjs_cuda_ctx* ctx, const float* x, const float* w, const float* bias,
                            int bias_len, const ActParams& ap, float* y, const Geo& g) {
  using T = DwTile<STRIDE, TW_>;
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  CUtensorMap tm;
  cuuint64_t dims[4] = {(cuuint64_t)g.c, (cuuint64_t)g.in_w, (cuuint64_t)g.in_h, (cuuint64_t)g.batch};
  cuuint64_t strides[3] = {(cuuint64_t)g.c * 4, (cuuint64_t)g.in_w * g.c * 4,
                           (cuuint64_t)g.in_h * g.in_w * g.c * 4};
  cuuint32_t box[4] = {32, T::IW, T::IH, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void*)x, dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -1;
  DwTiles tl;
  tl.tiles_w = (g.out_w + T::TW - 1) / T::TW;
  tl.tiles_h = (g.out_h + T::TH - 1) / T::TH;
  tl.chunks = (g.c + 31) / 32;
  const long long total = (long long)g.batch * tl.tiles_h * tl.tiles_w * tl.chunks;
  if (total > 0x7fffffffLL) return -1;
  tl.total = (int)total;
  const int grid = tl.total < ctx->sm_count * 2 ? tl.total : ctx->sm_count * 2;
#define DW_TMA(ACT)                                                                          \
  {                                                                                          \
    auto kern = depthwise3x3_tma_kernel<STRIDE, TW_, ACT>;                                        \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);  \
    kern<<<grid, 256, T::SMEM_BYTES, ctx->stream>>>(tm, w, bias, bias_len, ap, y, g, tl,     \
                                                    ctx->d_flag);                            \
  }
  switch (ap.act) {
    case TFJS_CUDA_ACT_LINEAR: DW_TMA(TFJS_CUDA_ACT_LINEAR) break;
    case TFJS_CUDA_ACT_RELU: DW_TMA(TFJS_CUDA_ACT_RELU) break;
    case TFJS_CUDA_ACT_RELU6: DW_TMA(TFJS_CUDA_ACT_RELU6) break;
    default: DW_TMA(TFJS_CUDA_ACT_ELU) break;
  }
#undef DW_TMA
  return 0;
}

// General channel multiplier: one thread per output element.
__global__ void depthwise_chmul_kernel(const float* __restrict__ x,
                                       const float* __restrict__ w,
                                       const float* __restrict__ bias,
                                       int bias_len, ActParams ap,
                                       float* __restrict__ y, Geo g) {
  const int out_c = g.c * g.ch_mul;
  const uint64_t n = (uint64_t)g.batch * g.out_h * g.out_w * out_c;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const int oc = (int)(i % out_c);
    const int d1 = oc / g.ch_mul, q = oc % g.ch_mul;
    uint64_t rem = i / out_c;
    const int ow = (int)(rem % g.out_w);
    rem /= g.out_w;
    const int oh = (int)(rem % g.out_h);
    const int b = (int)(rem / g.out_h);
    const int r0 = oh * g.s_h - g.pad_t, c0 = ow * g.s_w - g.pad_l;
    float acc = 0.0f;
    for (int fr = 0; fr < g.f_h; ++fr) {
      const int r = r0 + fr * g.d_h;
      if (r < 0 || r >= g.in_h) continue;
      for (int fc = 0; fc < g.f_w; ++fc) {
        const int cc = c0 + fc * g.d_w;
        if (cc < 0 || cc >= g.in_w) continue;
        acc = fmaf(x[(((uint64_t)b * g.in_h + r) * g.in_w + cc) * g.c + d1],
                   w[(((uint64_t)fr * g.f_w + fc) * g.c + d1) * g.ch_mul + q], acc);
      }
    }
    if (bias_len) acc = __fadd_rn(acc, bias[bias_len == 1 ? 0 : oc]);
    y[i] = apply_act(acc, ap, oc);
  }
}

int check_geo(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p, const char* who) {
  if (!p) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: null params", who);
  if (p->batch < 0 || p->in_h < 0 || p->in_w < 0 || p->in_c < 0 || p->out_h < 0 ||
      p->out_w < 0 || p->out_c < 0 || p->filter_h <= 0 || p->filter_w <= 0 ||
      p->stride_h <= 0 || p->stride_w <= 0 || p->dilation_h <= 0 || p->dilation_w <= 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "%s: bad geometry", who);
  return TFJS_CUDA_OK;
}

Geo make_geo(const tfjs_cuda_conv2d_params* p) {
  Geo g;
  g.batch = p->batch; g.in_h = p->in_h; g.in_w = p->in_w; g.c = p->in_c;
  g.out_h = p->out_h; g.out_w = p->out_w; g.f_h = p->filter_h; g.f_w = p->filter_w;
  g.s_h = p->stride_h; g.s_w = p->stride_w; g.d_h = p->dilation_h; g.d_w = p->dilation_w;
  g.pad_t = p->pad_top; g.pad_l = p->pad_left; g.ch_mul = 1;
  return g;
}

}  // namespace

extern "C" {

int tfjs_cuda_pool2d(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                     int32_t is_max, int32_t x_id, int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  int rc;
  if ((rc = check_geo(ctx, p, "pool2d"))) return rc;
  const uint64_t nx = (uint64_t)p->batch * p->in_h * p->in_w * p->in_c;
  const uint64_t ny = (uint64_t)p->batch * p->out_h * p->out_w * p->in_c;
  Buffer *x, *y;
  if ((rc = ctx_get(ctx, x_id, nx * 4, "pool2d x", &x))) return rc;
  if ((rc = ctx_get(ctx, out_id, ny * 4, "pool2d out", &y))) return rc;
  if (ny == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  Geo g = make_geo(p);
  const float* xp = (const float*)x->ptr;
  float* yp = (float*)y->ptr;
  if (is_max && g.c % 4 == 0 && g.f_h == 3 && g.f_w == 3 && g.s_h == 2 && g.s_w == 2 &&
      g.d_h == 1 && g.d_w == 1 && ((uintptr_t)xp & 15) == 0 && ((uintptr_t)yp & 15) == 0) {
    const uint64_t items = (uint64_t)g.batch * g.out_h * ((g.out_w + 3) / 4) * (g.c / 4);
    maxpool3x3s2_kernel<1><<<grid_for(items, kThreads, ctx->sm_count, 16), kThreads, 0, ctx->stream>>>(
        xp, yp, g);
    LAUNCH_CHECK(ctx, "maxpool3x3s2_kernel");
    ctx_mark_written(ctx, out_id);
    return TFJS_CUDA_OK;
  }
  if (g.c % 4 == 0) {
    const unsigned grid = grid_for(ny / 4, kThreads, ctx->sm_count);
    if (is_max) pool2d_kernel<true, 4><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, g);
    else pool2d_kernel<false, 4><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, g);
  } else {
    const unsigned grid = grid_for(ny, kThreads, ctx->sm_count);
    if (is_max) pool2d_kernel<true, 1><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, g);
    else pool2d_kernel<false, 1><<<grid, kThreads, 0, ctx->stream>>>(xp, yp, g);
  }
  LAUNCH_CHECK(ctx, "pool2d_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_fused_depthwise_conv2d(tfjs_cuda_ctx* ctx,
                                     const tfjs_cuda_conv2d_params* p,
                                     int32_t x_id, int32_t filter_id,
                                     int32_t bias_id, int32_t prelu_id,
                                     int32_t out_id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  int rc;
  if ((rc = check_geo(ctx, p, "fused_depthwise_conv2d"))) return rc;
  if (p->in_c <= 0 || p->out_c % p->in_c != 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                    "fused_depthwise_conv2d: out_c %d is not a multiple of in_c %d",
                    p->out_c, p->in_c);
  if ((p->bias_len != 0 && p->bias_len != 1 && p->bias_len != p->out_c) ||
      (p->prelu_len != 0 && p->prelu_len != 1 && p->prelu_len != p->out_c))
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "fused_depthwise_conv2d: bias/prelu must be scalar or per channel");
  if (p->activation == TFJS_CUDA_ACT_PRELU && (!prelu_id || !p->prelu_len))
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "fused_depthwise_conv2d: prelu weights missing");
  const int ch_mul = p->out_c / p->in_c;
  const uint64_t nx = (uint64_t)p->batch * p->in_h * p->in_w * p->in_c;
  const uint64_t nw = (uint64_t)p->filter_h * p->filter_w * p->out_c;
  const uint64_t ny = (uint64_t)p->batch * p->out_h * p->out_w * p->out_c;
  Buffer *x, *w, *bias = nullptr, *prelu = nullptr, *y;
  if ((rc = ctx_get(ctx, x_id, nx * 4, "fused_depthwise_conv2d x", &x))) return rc;
  if ((rc = ctx_get(ctx, filter_id, nw * 4, "fused_depthwise_conv2d filter", &w))) return rc;
  if (p->bias_len && (rc = ctx_get(ctx, bias_id, (uint64_t)p->bias_len * 4, "fused_depthwise_conv2d bias", &bias))) return rc;
  if (p->activation == TFJS_CUDA_ACT_PRELU &&
      (rc = ctx_get(ctx, prelu_id, (uint64_t)p->prelu_len * 4, "fused_depthwise_conv2d prelu", &prelu))) return rc;
  if ((rc = ctx_get(ctx, out_id, ny * 4, "fused_depthwise_conv2d out", &y))) return rc;
  if (ny == 0) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  Geo g = make_geo(p);
  g.ch_mul = ch_mul;
  ActParams ap;
  ap.act = p->activation;
  ap.prelu_len = p->prelu_len;
  ap.prelu = prelu ? (const float*)prelu->ptr : nullptr;
  ap.alpha = p->leakyrelu_alpha;
  const float* bp = bias ? (const float*)bias->ptr : nullptr;
  const int bl = bias ? p->bias_len : 0;
  const bool fast3x3 = ch_mul == 1 && g.c % 4 == 0 && g.f_h == 3 && g.f_w == 3 && g.d_h == 1 &&
                       g.d_w == 1 && g.s_h == g.s_w && (g.s_h == 1 || g.s_h == 2);
  static int no_tma = -1;
  if (no_tma < 0) no_tma = getenv("TFJS_CUDA_NO_DW_TMA") ? 1 : 0;  // debugging knob
  // 16-wide tiles measured faster than 14-wide ones even on 56 / 28 / 14 wide maps;
  // maps narrower than 12 keep the register-strip kernel
  // Stride-1 maps whose width is a multiple of 28 (56, 28, 84) take 28-wide tiles with seven
  // outputs per thread: 16-wide tiles leave an eighth of the last tile column empty there and
  // fetch a wider halo (56 x 56 x 144 at batch 256: 197 -> 148 us, 0.97 of the measured copy
  // bandwidth; 28 x 28 x 192: 67 -> 51 us).  112-wide maps are 16 x 7 and stay (142 against
  // 148 us).  TFJS_CUDA_NO_DW_TILE28=1: 16-wide tiles everywhere.
  static int wide28 = -1;
  if (wide28 < 0) wide28 = getenv("TFJS_CUDA_NO_DW_TILE28") ? 0 : 1;
  const int tw = g.out_w >= 12
                     ? ((wide28 && g.s_h == 1 && g.out_w % 28 == 0 && g.out_w % 112 != 0) ? 28 : 16)
                     : 0;
  int launched = -1;
  if (fast3x3 && !no_tma && tw) {
    const float* xp = (const float*)x->ptr;
    const float* wp = (const float*)w->ptr;
    float* yp = (float*)y->ptr;
    if (g.s_h == 1 && tw == 28) launched = launch_depthwise3x3_tma<1, 28>(ctx, xp, wp, bp, bl, ap, yp, g);
    else if (g.s_h == 1 && tw == 16) launched = launch_depthwise3x3_tma<1, 16>(ctx, xp, wp, bp, bl, ap, yp, g);
    else if (g.s_h == 1) launched = launch_depthwise3x3_tma<1, 14>(ctx, xp, wp, bp, bl, ap, yp, g);
    else if (tw == 16) launched = launch_depthwise3x3_tma<2, 16>(ctx, xp, wp, bp, bl, ap, yp, g);
    else launched = launch_depthwise3x3_tma<2, 14>(ctx, xp, wp, bp, bl, ap, yp, g);
  }
  if (launched == 0) {
    // launched
  } else if (fast3x3 && g.s_h == 1)
    launch_depthwise3x3<1, 4>(ctx, (const float*)x->ptr, (const float*)w->ptr, bp, bl, ap,
                              (float*)y->ptr, g);
  else if (fast3x3)
    launch_depthwise3x3<2, 2>(ctx, (const float*)x->ptr, (const float*)w->ptr, bp, bl, ap,
                              (float*)y->ptr, g);
  else if (ch_mul == 1 && g.c % 4 == 0)
    depthwise_kernel<4><<<grid_for(ny / 4, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (const float*)w->ptr, bp, bl, ap, (float*)y->ptr, g);
  else if (ch_mul == 1)
    depthwise_kernel<1><<<grid_for(ny, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (const float*)w->ptr, bp, bl, ap, (float*)y->ptr, g);
  else
    depthwise_chmul_kernel<<<grid_for(ny, kThreads, ctx->sm_count), kThreads, 0, ctx->stream>>>(
        (const float*)x->ptr, (const float*)w->ptr, bp, bl, ap, (float*)y->ptr, g);
  LAUNCH_CHECK(ctx, "depthwise_kernel");
  ctx_mark_written(ctx, out_id);
  return TFJS_CUDA_OK;
}

}  // extern "C"
