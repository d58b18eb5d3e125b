/*
 * tfjs_cuda.h -- C ABI of the B200 (sm_100a) backend for TensorFlow.js.
 *
 * This is the boundary a `tfjs-backend-cuda` package binds: the N-API addon
 * (and the ctypes host layer used by the tests) call exactly these entry
 * points.  The split follows the reference's WASM backend, where TypeScript
 * computes shapes/padding and passes scalars plus tensor ids to a C function
 * (tfjs-backend-wasm/src/kernels/FusedConv2D.ts:79-147 ->
 * tfjs-backend-wasm/src/cc/kernels/FusedConv2D.cc:33-52), with two changes:
 * an explicit context handle (one per GPU) instead of a process-wide singleton
 * (tfjs-backend-wasm/src/cc/backend.cc:124-152), and a status code returned by
 * every call instead of void.
 *
 * Conventions
 *   - Every function returns TFJS_CUDA_OK (0) or an error code; the message is
 *     available from tfjs_cuda_last_error() until the next failing call.
 *   - Tensors are named by int32 ids > 0 handed out by tfjs_cuda_alloc(); id 0
 *     means "absent optional input" (tfjs-backend-wasm/src/backend_wasm.ts:51).
 *   - All tensors are dense row-major; activations NHWC, filters HWIO.
 *   - Kernel launches are asynchronous on the context's single in-order stream;
 *     only read, sync, time_end and destroy block the host.
 *   - Enum values for activations and dtypes follow
 *     tfjs-backend-wasm/src/cc/backend.h:23-40.
 */
#ifndef TFJS_CUDA_H_
#define TFJS_CUDA_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tfjs_cuda_ctx tfjs_cuda_ctx;

enum tfjs_cuda_status {
  TFJS_CUDA_OK = 0,
  TFJS_CUDA_INVALID_ARG = 1,
  TFJS_CUDA_OUT_OF_MEMORY = 2,
  TFJS_CUDA_DRIVER_ERROR = 3,
  TFJS_CUDA_UNKNOWN_ID = 4,
  TFJS_CUDA_UNSUPPORTED = 5,
  TFJS_CUDA_DEVICE_TIMEOUT = 6 /* a bounded device-side wait gave up */
};

/* tfjs-backend-wasm/src/cc/backend.h:23-31 (FusableActivation). */
enum tfjs_cuda_activation {
  TFJS_CUDA_ACT_LINEAR = 0,
  TFJS_CUDA_ACT_RELU = 1,
  TFJS_CUDA_ACT_RELU6 = 2,
  TFJS_CUDA_ACT_PRELU = 3,
  TFJS_CUDA_ACT_LEAKYRELU = 4,
  TFJS_CUDA_ACT_SIGMOID = 5,
  TFJS_CUDA_ACT_ELU = 6,
  /* tfjs_cuda_fused_matmul only: the erf form of GELU as a converted graph spells it,
   * out = (h * gelu_half) * (erf(h * gelu_scale) + gelu_one)  (or erf(h / gelu_scale)
   * when gelu_divide), each product and sum rounded to fp32 as the separate Multiply.ts /
   * RealDiv.ts / Erf.ts / Add.ts kernels round them.  The graph executor substitutes it for
   * the five nodes after a dense layer. */
  TFJS_CUDA_ACT_GELU_ERF = 7
};

/* tfjs-backend-wasm/src/cc/backend.h:33-40 (DType); bool is one byte. */
enum tfjs_cuda_dtype {
  TFJS_CUDA_FLOAT32 = 0,
  TFJS_CUDA_INT32 = 1,
  TFJS_CUDA_BOOL = 2
};

/* How FusedConv2D / _FusedMatMul / BatchMatMul do their arithmetic. */
enum tfjs_cuda_math_mode {
  TFJS_CUDA_MATH_TF32 = 0, /* tcgen05 tensor cores, TF32 inputs, fp32 accumulate */
  TFJS_CUDA_MATH_FP32 = 1  /* SIMT fp32 FMA; for running fp32-tolerance suites   */
};

/* ---- context and storage: the device half of the KernelBackend contract
 * (tfjs-core/src/backends/backend.ts:100-156; reference implementation
 * tfjs-backend-cpu/src/backend_cpu.ts:52-204). ------------------------------ */

int tfjs_cuda_device_count(int* out_count);
int tfjs_cuda_create(int device_ordinal, tfjs_cuda_ctx** out_ctx);
void tfjs_cuda_destroy(tfjs_cuda_ctx* ctx);
const char* tfjs_cuda_last_error(tfjs_cuda_ctx* ctx);

/* Pool allocation (cudaMallocAsync on the context stream).  nbytes may be 0. */
int tfjs_cuda_alloc(tfjs_cuda_ctx* ctx, uint64_t nbytes, int32_t* out_id);
/* Stream-ordered free; also drops any packed-weight cache entry of the id
 * (the disposal-callback idea of tfjs-backend-wasm/src/cc/backend.cc:58-67). */
int tfjs_cuda_free(tfjs_cuda_ctx* ctx, int32_t id);
/* backend.write(): async H2D on the stream.  If `host` is pinned memory from
 * tfjs_cuda_host_alloc the copy overlaps the host; the caller must leave the
 * bytes untouched until the next blocking call. */
int tfjs_cuda_write(tfjs_cuda_ctx* ctx, int32_t id, const void* host,
                    uint64_t nbytes);
/* alloc + write in one call, on a separate copy stream: the transfer overlaps kernels
 * already queued on the compute stream, and the first kernel that consumes the new
 * tensor waits for it.  `host` should be pinned and must stay untouched until the
 * tensor has been consumed or a blocking call returns. */
int tfjs_cuda_upload(tfjs_cuda_ctx* ctx, const void* host, uint64_t nbytes, int32_t* out_id);
/* backend.readSync(): D2H then stream sync; reports a pending device timeout. */
int tfjs_cuda_read(tfjs_cuda_ctx* ctx, int32_t id, void* host, uint64_t nbytes);
/* Queue a D2H copy without waiting (pair with tfjs_cuda_sync). */
int tfjs_cuda_read_async(tfjs_cuda_ctx* ctx, int32_t id, void* host,
                         uint64_t nbytes);
/* backend.read(dataId): Promise (tfjs-core/src/backends/backend.ts:104): read_begin queues
 * the D2H copy behind the kernels already launched and returns a ticket at once;
 * read_wait blocks until that copy has landed (and reports a pending device timeout).
 * The caller keeps `host` (ideally pinned) alive and untouched in between; a ticket is
 * collected exactly once.  The tensor itself may be freed or overwritten as soon as
 * read_begin returns (stream-ordered).  Downloads of 4 MB and more leave the device through
 * a staging copy on a stream of their own, so kernels launched after read_begin run while
 * the bytes travel; tfjs_cuda_sync covers them as well. */
int tfjs_cuda_read_begin(tfjs_cuda_ctx* ctx, int32_t id, void* host, uint64_t nbytes,
                         int32_t* out_ticket);
int tfjs_cuda_read_wait(tfjs_cuda_ctx* ctx, int32_t ticket);
int tfjs_cuda_sync(tfjs_cuda_ctx* ctx);
int tfjs_cuda_size_of(tfjs_cuda_ctx* ctx, int32_t id, uint64_t* out_nbytes);
/* Raw device address of a tensor, for interop (profilers, other libraries). */
int tfjs_cuda_device_ptr(tfjs_cuda_ctx* ctx, int32_t id, void** out_ptr);
/* backend.memory() (tfjs-core/src/engine.ts:959-974). */
int tfjs_cuda_memory(tfjs_cuda_ctx* ctx, uint64_t* bytes_in_use,
                     uint64_t* bytes_reserved, uint64_t* high_water,
                     uint64_t* num_buffers);
/* Returns cached and pooled free blocks to the driver (blocks until the stream is idle). */
int tfjs_cuda_trim(tfjs_cuda_ctx* ctx);
/* Pinned host buffers for write/read staging. */
int tfjs_cuda_host_alloc(tfjs_cuda_ctx* ctx, uint64_t nbytes, void** out_ptr);
int tfjs_cuda_host_free(tfjs_cuda_ctx* ctx, void* ptr);
/* backend.time() (tfjs-core/src/engine.ts:1235-1240): CUDA events on the stream. */
int tfjs_cuda_time_begin(tfjs_cuda_ctx* ctx);
int tfjs_cuda_time_end(tfjs_cuda_ctx* ctx, float* out_kernel_ms);
/* Per-kernel timing for tf.profile (tfjs-core/src/profiler.ts:39-79 wraps every
 * kernel in backend.time): record numbered events on the stream, then ask for the
 * elapsed time between two of them (blocks until the later one has happened). */
int tfjs_cuda_event_record(tfjs_cuda_ctx* ctx, int32_t slot);
int tfjs_cuda_event_elapsed(tfjs_cuda_ctx* ctx, int32_t slot_begin, int32_t slot_end,
                            float* out_ms);
int tfjs_cuda_set_math_mode(tfjs_cuda_ctx* ctx, int mode);
/* Number of this library's kernels launched on the context so far. */
int tfjs_cuda_launch_count(tfjs_cuda_ctx* ctx, uint64_t* out_launches);
/* BackendTimingInfo.getExtraProfileInfo (tfjs-core/src/backends/backend.ts:26-30, printed
 * per kernel by tfjs-core/src/profiler.ts:74-76): while the log is on, the library notes
 * the name of every kernel instantiation it launches; launch_log_take writes them to `buf`
 * as text ("pack_weight_kernel, gemm_tf32_kernel<BN=256,...> x2", cut to cap - 1
 * characters), reports how many there were and empties the log. */
int tfjs_cuda_launch_log(tfjs_cuda_ctx* ctx, int32_t enable);
int tfjs_cuda_launch_log_take(tfjs_cuda_ctx* ctx, char* buf, uint64_t cap,
                              uint32_t* out_launches);
/* Clears L2 by overwriting a scratch buffer larger than it (benchmark hygiene). */
int tfjs_cuda_flush_l2(tfjs_cuda_ctx* ctx);

/* ---- FusedConv2D / Conv2D: tfjs-backend-cpu/src/kernels/FusedConv2D.ts:26-95,
 * Conv2D.ts:23-103; attrs tfjs-core/src/kernel_names.ts:1016-1031.  The caller
 * computes the geometry with computeConv2DInfo (tfjs-core/src/ops/conv_util.ts:
 * 177-236).  bias_len / prelu_len are 0 (absent), 1 (scalar) or out_c. -------- */
typedef struct tfjs_cuda_conv2d_params {
  int32_t batch, in_h, in_w, in_c;
  int32_t out_h, out_w, out_c;
  int32_t filter_h, filter_w;
  int32_t stride_h, stride_w;
  int32_t dilation_h, dilation_w;
  int32_t pad_top, pad_left;
  int32_t activation; /* tfjs_cuda_activation */
  int32_t bias_len, prelu_len;
  double leakyrelu_alpha;
} tfjs_cuda_conv2d_params;

int tfjs_cuda_fused_conv2d(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                           int32_t x_id, int32_t filter_id, int32_t bias_id,
                           int32_t prelu_id, int32_t out_id);

/* FusedConv2D whose epilogue also absorbs the two kernels that follow it in a residual
 * block, Add (tfjs-backend-cpu/src/kernels/Add.ts:23-30) and Relu / Relu6 (Relu.ts:22):
 *   out = post_activation(residual + act(conv(x, filter) + bias))
 * with each step rounded to fp32 as the separate kernels would.  The host layer uses it
 * when a FusedConv2D result is consumed only by such an Add (+ Relu); `residual` has the
 * output's shape; post_activation is LINEAR, RELU or RELU6. */
int tfjs_cuda_fused_conv2d_residual(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                                    int32_t x_id, int32_t filter_id, int32_t bias_id,
                                    int32_t prelu_id, int32_t residual_id,
                                    int32_t post_activation, int32_t out_id);

/* FusedDepthwiseConv2D (3x3, stride 1 or 2, bias, activation) and the 1x1 FusedConv2D that
 * consumes its result, as one launch: the depthwise result (the widest tensor of an
 * inverted-residual block) is produced tile by tile in shared memory as the projection's
 * operand and never written.  Each value goes through the roundings of the two separate
 * kernels (tfjs-backend-cpu/src/kernels/FusedDepthwiseConv2D.ts:25-61 then
 * FusedConv2D.ts:26-95): fp32 per-tap accumulation, bias, activation, then the TF32
 * rounding the projection applies to its input.  Optionally
 *   out = post_activation(residual + act(conv1x1(depthwise(x)) + bias))
 * as in tfjs_cuda_fused_conv2d_residual (residual_id 0 = none).  `dw` describes the
 * depthwise convolution, `pw` the 1x1 convolution over its output.  Returns
 * TFJS_CUDA_UNSUPPORTED for shapes the kernel does not take (other filter sizes, strides,
 * dilations, channel multipliers, the fp32 math mode); the host layer then launches the two
 * kernels separately. */
int tfjs_cuda_fused_depthwise_project(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* dw,
                                      const tfjs_cuda_conv2d_params* pw, int32_t x_id,
                                      int32_t dw_filter_id, int32_t dw_bias_id,
                                      int32_t pw_filter_id, int32_t pw_bias_id,
                                      int32_t residual_id, int32_t post_activation,
                                      int32_t out_id);

/* ---- whole-step capture and replay ----------------------------------------------------
 * The graph executor launches the same kernels with the same shapes at every
 * GraphModel.execute (tfjs-converter/src/executor/graph_executor.ts:228-310).  Between
 * capture_begin and capture_end every kernel call on this context is recorded into a
 * CUDA graph instead of being run, and tensors allocated in between live in an arena of
 * `arena_bytes` that belongs to the graph; graph_launch then replays the whole step with
 * one call.  Tensors that exist before the capture (weights, the step's input buffers)
 * are referenced by address, so a replay reads whatever they hold at that time
 * (tfjs_cuda_copy refills the input buffers).  Calls that move data to or from the host,
 * wait, or need new pool memory are refused during a capture (TFJS_CUDA_UNSUPPORTED) and
 * make capture_end discard it; the host layer then keeps running that model eagerly.
 * Tensors created during a capture that are still alive at capture_end (the step's
 * outputs) stay valid until graph_destroy and are rewritten by every replay.
 * Two kinds of memory outside the arena are also referenced by address: the library's
 * repacked copy of each weight the step reads, and its scratch buffer (explicit im2col of
 * unusual convolutions).  If, after the capture, such a weight is freed or rewritten, or an
 * eager call makes the scratch buffer grow, the graph is stale: graph_launch returns
 * TFJS_CUDA_UNSUPPORTED without launching anything and the host captures the step again
 * (or runs it eagerly). */
int tfjs_cuda_capture_begin(tfjs_cuda_ctx* ctx, uint64_t arena_bytes);
int tfjs_cuda_capture_end(tfjs_cuda_ctx* ctx, int abandon, int32_t* out_graph);
int tfjs_cuda_graph_launch(tfjs_cuda_ctx* ctx, int32_t graph);
int tfjs_cuda_graph_destroy(tfjs_cuda_ctx* ctx, int32_t graph);
/* Device-to-device copy of the first nbytes of src into dst, in stream order. */
int tfjs_cuda_copy(tfjs_cuda_ctx* ctx, int32_t src_id, int32_t dst_id, uint64_t nbytes);
/* Restart the high-water mark of tfjs_cuda_memory at the bytes in use now (sizes the arena
 * of a capture from an eager step). */
int tfjs_cuda_high_water_reset(tfjs_cuda_ctx* ctx);

/* ---- FusedDepthwiseConv2D / DepthwiseConv2dNative:
 * tfjs-backend-cpu/src/kernels/FusedDepthwiseConv2D.ts:25-61,
 * DepthwiseConv2dNative.ts:23-102; attrs kernel_names.ts:1033-1048.  out_c is
 * in_c * channel_multiplier; filter is [fh, fw, in_c, channel_multiplier]. ---- */
int tfjs_cuda_fused_depthwise_conv2d(tfjs_cuda_ctx* ctx,
                                     const tfjs_cuda_conv2d_params* p,
                                     int32_t x_id, int32_t filter_id,
                                     int32_t bias_id, int32_t prelu_id,
                                     int32_t out_id);

/* ---- _FusedMatMul / BatchMatMul: tfjs-backend-cpu/src/kernels/_FusedMatMul.ts:
 * 26-62, BatchMatMul.ts:25-133; attrs kernel_names.ts:1000-1014, :119-124.
 * a is [batch_a, M, K] (or [batch_a, K, M] when transpose_a), b is
 * [batch_b, K, N] (or [batch_b, N, K] when transpose_b); the output batch is
 * max(batch_a, batch_b) and operand batches wrap (BatchMatMul.ts:96-97).
 * bias_len is 0, 1, N, or M*N-compatible lengths are rejected (the host adds
 * those with the Add kernel). ------------------------------------------------ */
typedef struct tfjs_cuda_matmul_params {
  int32_t batch_a, batch_b;
  int32_t m, n, k;
  int32_t transpose_a, transpose_b;
  int32_t activation;
  int32_t bias_len, prelu_len;
  double leakyrelu_alpha;
  /* constants of TFJS_CUDA_ACT_GELU_ERF (ignored otherwise) */
  float gelu_scale, gelu_half, gelu_one;
  int32_t gelu_divide;
} tfjs_cuda_matmul_params;

int tfjs_cuda_fused_matmul(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                           int32_t a_id, int32_t b_id, int32_t bias_id,
                           int32_t prelu_id, int32_t out_id);

/* The same product stored through the permutation that splits or merges attention heads, so
 * that the Reshape + Transpose([0, 2, 1, 3]) around a multi-head attention
 * (tfjs-backend-cpu/src/kernels/Transpose.ts, one pass over the tensor each) cost nothing:
 *   TFJS_CUDA_HEADS_SPLIT  batch 1, M = B*S, N = H*D: the [B, S, H, D] view of the result is
 *                          written as [B, H, S, D]; rows_or_heads = S, head_dim = D.
 *   TFJS_CUDA_HEADS_MERGE  batch B*H, M = S, N = D: the [B, H, S, D] result is written as
 *                          [B, S, H, D]; rows_or_heads = H, head_dim = D.
 * The values are those of tfjs_cuda_fused_matmul; only their places differ.  S and D must
 * be multiples of 32 and the tensor-core path must apply (TF32 math mode, K % 4 == 0, a not
 * transposed); otherwise TFJS_CUDA_UNSUPPORTED, nothing is written, and the host runs the
 * plain product and the Transpose kernel. */
enum tfjs_cuda_heads_layout { TFJS_CUDA_HEADS_SPLIT = 1, TFJS_CUDA_HEADS_MERGE = 2 };
int tfjs_cuda_fused_matmul_heads(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                                 int32_t a_id, int32_t b_id, int32_t bias_id, int32_t prelu_id,
                                 int32_t layout, int32_t rows_or_heads, int32_t head_dim,
                                 int32_t out_id);

/* Several _FusedMatMul products that share their `a` operand and every dimension, as one
 * launch: the query, key and value projections of an attention layer read the same
 * activations, and three products of 1.3 waves of tiles each leave a third of the GPU idle
 * where one product of 3.9 waves does not.  Member i multiplies by b_ids[i] (a weight
 * tensor), adds bias_ids[i] (all members carry a bias of N elements, or none) and writes
 * out_ids[i]; each result is the one tfjs_cuda_fused_matmul (layout 0) or
 * tfjs_cuda_fused_matmul_heads (layout TFJS_CUDA_HEADS_SPLIT) gives for that member
 * (tfjs-backend-cpu/src/kernels/_FusedMatMul.ts:26-62).  2 <= count <= 4.  Returns
 * TFJS_CUDA_UNSUPPORTED for problems the grouped kernel does not take (batched operands,
 * transpose_a, PReLU, narrow outputs, the fp32 math mode); the caller then launches the
 * members one by one. */
int tfjs_cuda_fused_matmul_group(tfjs_cuda_ctx* ctx, const tfjs_cuda_matmul_params* p,
                                 int32_t a_id, int32_t count, const int32_t* b_ids,
                                 const int32_t* bias_ids, int32_t layout, int32_t rows_or_heads,
                                 int32_t head_dim, const int32_t* out_ids);

/* ---- MaxPool / AvgPool: tfjs-backend-cpu/src/kernels/MaxPool.ts:24-55,
 * AvgPool.ts:24-55, utils/pool_utils.ts:20-87; attrs kernel_names.ts:83-90,
 * :517-524.  Geometry from computePool2DInfo (conv_util.ts:119-140); filter_h/w
 * are the effective (dilated) window extents. --------------------------------- */
int tfjs_cuda_pool2d(tfjs_cuda_ctx* ctx, const tfjs_cuda_conv2d_params* p,
                     int32_t is_max, int32_t x_id, int32_t out_id);

/* ---- broadcasting binary kernels: tfjs-backend-cpu/src/utils/binary_impl.ts:
 * 25-69 (Add.ts, Sub.ts, Multiply.ts, RealDiv.ts, Maximum.ts, Minimum.ts, Pow.ts,
 * SquaredDifference.ts, Prelu.ts).  Shapes are given right-aligned with the same
 * rank (<= 6), padded with leading 1s. ---------------------------------------- */
enum tfjs_cuda_binary_op {
  TFJS_CUDA_ADD = 0,
  TFJS_CUDA_SUB = 1,
  TFJS_CUDA_MUL = 2,
  TFJS_CUDA_DIV = 3,
  TFJS_CUDA_MAXIMUM = 4,
  TFJS_CUDA_MINIMUM = 5,
  TFJS_CUDA_POW = 6,
  TFJS_CUDA_SQUARED_DIFFERENCE = 7,
  TFJS_CUDA_PRELU = 8
};

int tfjs_cuda_binary(tfjs_cuda_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                     int32_t a_id, const int64_t* a_shape, int32_t b_id,
                     const int64_t* b_shape, int32_t out_id,
                     const int64_t* out_shape);

/* Add of two equal-shape float32 tensors fused with a following Relu / Relu6 (or none):
 * out = activation(a + b).  Add.ts:23-30 then Relu.ts:22 / Relu6.ts:22-23. */
int tfjs_cuda_add_activation(tfjs_cuda_ctx* ctx, int32_t activation, int32_t a_id,
                             int32_t b_id, uint64_t n, int32_t out_id);

/* ---- unary kernels: tfjs-backend-cpu/src/utils/unary_impl.ts:25-36 with Relu.ts,
 * Relu6.ts, Elu.ts, Sigmoid.ts, LeakyRelu.ts, Exp.ts, Sqrt.ts, Rsqrt.ts, Square.ts,
 * Tanh.ts, Neg.ts, ClipByValue.ts, Erf.ts, Abs.ts, Log.ts.  p0/p1: leakyrelu alpha,
 * or clip min/max. -------------------------------------------------------------- */
enum tfjs_cuda_unary_op {
  TFJS_CUDA_RELU = 0,
  TFJS_CUDA_RELU6 = 1,
  TFJS_CUDA_ELU = 2,
  TFJS_CUDA_SIGMOID = 3,
  TFJS_CUDA_LEAKYRELU = 4,
  TFJS_CUDA_EXP = 5,
  TFJS_CUDA_SQRT = 6,
  TFJS_CUDA_RSQRT = 7,
  TFJS_CUDA_SQUARE = 8,
  TFJS_CUDA_TANH = 9,
  TFJS_CUDA_NEG = 10,
  TFJS_CUDA_CLIP = 11,
  TFJS_CUDA_ERF = 12,
  TFJS_CUDA_ABS = 13,
  TFJS_CUDA_LOG = 14
};

int tfjs_cuda_unary(tfjs_cuda_ctx* ctx, int32_t op, double p0, double p1,
                    int32_t x_id, uint64_t n, int32_t out_id);

/* ---- chains of elementwise kernels in one pass ---------------------------------------
 * A program is a short list of the unary / binary kernels above applied to float32 values:
 * the graph models decompose LayerNorm, GELU and scaling into such chains (e.g.
 * Mul, Erf, Add, Mul, Mul), each of which the reference runs as one pass over memory
 * (unary_impl.ts:25-36, binary_impl.ts:25-69).  The fused kernel reads every input once,
 * evaluates the ops per element in order, rounding every intermediate result to fp32
 * exactly like the separate kernels, and writes the last result: same bits, one pass.
 *
 * Value slots: 0 .. n_inputs-1 are the inputs, n_inputs + j is the result of op j.  Each
 * input is addressed relative to the OUTPUT's flat index i (cols = the output's innermost
 * extent): FULL in[i]; PERIODIC in[i % period] (a trailing-axes broadcast such as a bias);
 * ROW in[i / cols] (shape = output shape with the last axis 1); SCALAR in[0]; BATCHED
 * in[(i / aux) * period + i % period] (equal to the output on leading and trailing axes, 1 in
 * between: period = product of the trailing axes, aux = period * product of the middle ones).
 * binary ops use opcode = tfjs_cuda_binary_op, unary ops opcode = 32 + tfjs_cuda_unary_op
 * with operand a only and parameters p0, p1. */
enum tfjs_cuda_ew_input_mode {
  TFJS_CUDA_EW_FULL = 0,
  TFJS_CUDA_EW_PERIODIC = 1,
  TFJS_CUDA_EW_ROW = 2,
  TFJS_CUDA_EW_SCALAR = 3,
  TFJS_CUDA_EW_BATCHED = 4
};
#define TFJS_CUDA_EW_MAX_INPUTS 8
#define TFJS_CUDA_EW_MAX_OPS 24
#define TFJS_CUDA_EW_UNARY 32
typedef struct tfjs_cuda_ew_op {
  int16_t opcode;
  uint8_t a, b; /* value slots */
  float p0, p1;
} tfjs_cuda_ew_op;
typedef struct tfjs_cuda_ew_program {
  int32_t n_inputs, n_ops;
  uint64_t n;    /* output elements */
  uint32_t cols; /* output's innermost extent (ROW inputs), >= 1 */
  uint32_t reserved;
  int32_t input_id[TFJS_CUDA_EW_MAX_INPUTS];
  int32_t input_mode[TFJS_CUDA_EW_MAX_INPUTS];
  uint32_t input_period[TFJS_CUDA_EW_MAX_INPUTS]; /* PERIODIC: elements of the input */
  uint32_t input_aux[TFJS_CUDA_EW_MAX_INPUTS];    /* BATCHED: see above */
  tfjs_cuda_ew_op ops[TFJS_CUDA_EW_MAX_OPS];
} tfjs_cuda_ew_program;
int tfjs_cuda_fused_elementwise(tfjs_cuda_ctx* ctx, const tfjs_cuda_ew_program* prog,
                                int32_t out_id);
/* The library carries straight-line kernels for the chains graph models contain (LayerNorm
 * tail in its two usual decompositions, erf-GELU, x * a + b, a + b + c); any other program
 * runs through an interpreter kernel that is slower than the separate kernels for short
 * chains.  *out_yes = 1 when `prog` (ops and operand slots; sizes and ids are ignored)
 * matches a catalogued chain, so a host layer can keep launching the separate kernels
 * otherwise. */
int tfjs_cuda_fused_elementwise_catalogued(tfjs_cuda_ctx* ctx, const tfjs_cuda_ew_program* prog,
                                           int32_t* out_yes);

/* ---- Softmax over the last axis: tfjs-backend-cpu/src/kernels/Softmax.ts:29-77. */
int tfjs_cuda_softmax(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows,
                      uint64_t cols, int32_t out_id);

/* Softmax of fl32(fl32(x * scale) + mask): the Multiply.ts (by a scalar) and Add.ts kernels
 * that scale and mask attention scores, applied on the way into the softmax with the same
 * fp32 roundings.  has_scale = 0 skips the product; mask_id = 0 the sum.  The mask holds
 * ceil(rows / rows_per_mask) rows of cols floats; row r of x uses mask row r / rows_per_mask
 * (rows_per_mask = heads * queries for a [batch, 1, 1, keys] mask, 1 for a mask shaped like
 * x, rows for a single row). */
int tfjs_cuda_softmax_scaled_masked(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows,
                                    uint64_t cols, int32_t has_scale, float scale,
                                    int32_t mask_id, uint64_t rows_per_mask, int32_t out_id);

/* ---- One attention layer as one launch: out = softmax(fl32(fl32(q k^T * scale) + mask)) v
 * for q, k, v of shape [batch, heads, seq, head_dim] (the heads-split store of
 * tfjs_cuda_fused_matmul_heads) and out stored [batch, seq, heads, head_dim] (heads merged).
 * It stands for four kernels of the reference and the transposes around them: BatchMatMul
 * with adj_y (tfjs-backend-cpu/src/kernels/BatchMatMul.ts:29-113), Multiply by a scalar
 * (Multiply.ts), Add of the mask (Add.ts), Softmax (Softmax.ts:50-67), BatchMatMul, Transpose
 * [0, 2, 1, 3]; the [batch, heads, seq, seq] scores and probabilities are never stored.
 * has_scale = 0 skips the product, mask_id = 0 the sum.  The mask holds ceil(batch * heads /
 * units_per_mask) rows of seq floats; head u = b * heads + h uses mask row u / units_per_mask
 * (units_per_mask = heads for a [batch, 1, 1, seq] mask).  TF32 products with fp32
 * accumulation and the fp32 softmax of the TF32 math mode; the probabilities are rounded to
 * TF32 as the operand load of the separate product rounds them.  Only seq = 128 and
 * head_dim = 64 in the TF32 math mode are taken: anything else returns
 * TFJS_CUDA_UNSUPPORTED and launches nothing (the caller issues the separate kernels). */
int tfjs_cuda_fused_attention(tfjs_cuda_ctx* ctx, int32_t q_id, int32_t k_id, int32_t v_id,
                              int32_t mask_id, int32_t has_scale, float scale, int32_t batch,
                              int32_t heads, int32_t seq, int32_t head_dim,
                              int32_t units_per_mask, int32_t out_id);

/* ---- Layer normalisation over the last axis of a [rows, cols] view, in the decomposed
 * form a converted graph holds: y = ((x - mean) * rsqrt(var + epsilon)) * gamma + beta with
 * mean = Mean(x), var = Mean(SquaredDifference(x, mean)).  One launch for the nine (ten with the residual Add) kernels
 * (tfjs-backend-cpu/src/kernels/Mean.ts:25-53, SquaredDifference.ts, Add.ts, Rsqrt.ts,
 * Sub.ts, Multiply.ts) with every intermediate rounded as those kernels round it.  gamma and
 * beta hold cols floats.  residual_id != 0: the normalised tensor is Add(x, residual) (the
 * residual connection in front of the normalisation; Add.ts), never written to memory.
 * cols must be a multiple of 4 and at most 1024 (UNSUPPORTED
 * otherwise: the host then runs the separate kernels).  No counterpart in the reference's
 * kernel set; the graph executor substitutes it for the matched subgraph. */
int tfjs_cuda_layer_norm(tfjs_cuda_ctx* ctx, int32_t x_id, int32_t residual_id, int32_t gamma_id,
                         int32_t beta_id, uint64_t rows, uint64_t cols, float epsilon,
                         int32_t out_id);

/* ---- Sum / Mean / Max over the middle axis of an [outer, reduce, inner] view:
 * tfjs-backend-cpu/src/kernels/Sum.ts:28-90, Mean.ts:25-53, Max.ts:28-72.  The
 * host collapses the (contiguous) reduced axes; non-contiguous axes are first
 * transposed, as the reference does (Sum.ts:46-54). ----------------------------- */
enum tfjs_cuda_reduce_op {
  TFJS_CUDA_REDUCE_SUM = 0,
  TFJS_CUDA_REDUCE_MEAN = 1,
  TFJS_CUDA_REDUCE_MAX = 2
};

int tfjs_cuda_reduce(tfjs_cuda_ctx* ctx, int32_t op, int32_t x_id,
                     uint64_t outer, uint64_t reduce, uint64_t inner,
                     int32_t out_id);

/* ---- ArgMax over the middle axis of [outer, reduce, inner], int32 output:
 * tfjs-backend-cpu/src/kernels/ArgMax.ts:24-71. --------------------------------- */
int tfjs_cuda_argmax(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t outer,
                     uint64_t reduce, uint64_t inner, int32_t out_id);

/* ---- Transpose (rank <= 6, 4-byte or 1-byte elements):
 * tfjs-backend-cpu/src/kernels/Transpose.ts:25-48, Transpose_impl.ts:21-45. ------ */
int tfjs_cuda_transpose(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t rank,
                        int32_t x_id, const int64_t* x_shape,
                        const int32_t* perm, int32_t out_id);

/* ---- GatherV2 on a [batch, outer, dim, slice] view of x and [batch, n_idx]
 * indices: tfjs-backend-cpu/src/kernels/GatherV2.ts:25-90, GatherV2_impl.ts:20-41.
 * An index outside [0, dim-1] makes the call fail (GatherV2.ts:36-46); the range
 * check runs on the device and is reported through out_bad_index (first bad
 * value, or -1), which the caller reads after the launch. ------------------------ */
int tfjs_cuda_gather(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t x_id,
                     int32_t indices_id, uint64_t batch, uint64_t outer,
                     uint64_t dim, uint64_t slice, uint64_t n_idx,
                     int32_t out_id, int32_t check_indices,
                     int64_t* out_bad_index);

/* ---- Cast: tfjs-backend-cpu/src/kernels/Cast.ts:27-95 (float32->int32 is JS
 * ToInt32; anything->bool is x != 0; widening copies the values). --------------- */
int tfjs_cuda_cast(tfjs_cuda_ctx* ctx, int32_t from_dtype, int32_t to_dtype,
                   int32_t x_id, uint64_t n, int32_t out_id);

/* ---- strided copy glue used by Concat / Slice / PadV2 / Tile
 * (tfjs-backend-cpu/src/kernels/Concat.ts:29-103, Slice.ts, PadV2.ts, Tile.ts):
 * out[o_off + idx(loc, o_strides)] = x[x_off + idx(loc mod x_shape, x_strides)]
 * for every loc in `extent`.  rank <= 6, elem_bytes 1 or 4. --------------------- */
int tfjs_cuda_copy_strided(tfjs_cuda_ctx* ctx, int32_t elem_bytes, int32_t rank,
                           const int64_t* extent, int32_t x_id, int64_t x_off,
                           const int64_t* x_strides, const int64_t* x_wrap,
                           int32_t out_id, int64_t o_off,
                           const int64_t* o_strides);
int tfjs_cuda_fill(tfjs_cuda_ctx* ctx, int32_t elem_bytes, uint32_t bits,
                   int32_t out_id, uint64_t n);

/* ---- FusedBatchNorm: tfjs-backend-cpu/src/kernels/BatchNorm.ts:23-90; parameter
 * tensors are indexed modulo their own length (:69-87). ------------------------- */
int tfjs_cuda_batchnorm(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t n,
                        int32_t mean_id, uint64_t n_mean, int32_t var_id,
                        uint64_t n_var, int32_t scale_id, uint64_t n_scale,
                        int32_t offset_id, uint64_t n_offset, double epsilon,
                        int32_t out_id);

/* FusedBatchNorm on a [rows, cols] view of x whose parameters are rows or columns of that
 * view and need not be tiled to its shape first: tfjs-layers' LayerNormalization computes
 * the moments per row, tiles them and gamma / beta to the input's shape and calls batchNorm
 * on the tiles (tfjs-layers/src/layers/normalization.ts:578-622); the host layer keeps those
 * Tile results unmaterialised and passes the untiled tensors here.  Same arithmetic as
 * tfjs_cuda_batchnorm (BatchNorm.ts:69-87).  Modes: 0 absent (scale and offset only), 1 one
 * value per column (cols values), 2 one per row (rows values), 3 one per element, 4 one
 * value in all. */
int tfjs_cuda_batchnorm_rows(tfjs_cuda_ctx* ctx, int32_t x_id, uint64_t rows, uint64_t cols,
                             int32_t mean_id, int32_t mean_mode, int32_t var_id,
                             int32_t var_mode, int32_t scale_id, int32_t scale_mode,
                             int32_t offset_id, int32_t offset_mode, double epsilon,
                             int32_t out_id);

/* ---- weight dequantisation at load: tfjs-core/src/io/io_utils.ts:221-227
 * (float32 target) and :243-247 (int32 target).  q_dtype_bytes is 1 (uint8) or 2
 * (uint16).  The 256/65536-entry table fl32(v*scale+min) is built on the host in
 * double and looked up on the device, which makes the result bit-exact. -------- */
int tfjs_cuda_dequantize(tfjs_cuda_ctx* ctx, int32_t q_dtype_bytes,
                         int32_t to_dtype, int32_t q_id, double scale,
                         double min, uint64_t n, int32_t out_id);

/* Weights stored as float16 ('float16' quantization of a float32 weight,
 * tfjs-core/src/io/io_utils.ts:228-231, decoder :720-741): exact widening of n half-precision
 * values (raw uint16 bits in q) to float32, on the device, so such weights cross PCIe at two
 * bytes per value. */
int tfjs_cuda_decode_float16(tfjs_cuda_ctx* ctx, int32_t q_id, uint64_t n, int32_t out_id);

/* ---- weight loading: decodeWeights / decodeWeight (tfjs-core/src/io/io_utils.ts:119-135,
 * :185-292), decodeWeightsStream (:316-353) and the shard fetching of
 * tfjs-core/src/io/weights_loader.ts:38-131, behind the C ABI.  The caller lists the
 * manifest entries in order (WeightsManifestEntry, tfjs-core/src/io/types.ts:76-110) and
 * pushes the concatenated weight bytes in pieces of any size, cut anywhere: whole shards,
 * shard files by path, or the chunks of a stream.  Pieces are staged through a ring of
 * pinned host slots and copied with one cudaMemcpyAsync each on the copy stream while the
 * next slot is being filled (straight from the file for push_file); quantised and
 * float16-stored tensors are decoded on the device as soon as their bytes have been queued
 * (same kernels and results, bit for bit, as tfjs_cuda_dequantize / tfjs_cuda_decode_float16).
 *   storage RAW      the bytes are the tensor's own dtype (float32 / int32: 4 bytes per
 *                    element, bool: 1)
 *   storage UINT8 / UINT16  affine quantisation: value = q * scale + min, rounded as
 *                    io_utils.ts:221-227 (float32) or :243-247 (int32)
 *   storage FLOAT16  half-precision bits widened exactly (io_utils.ts:228-231)
 *   skip != 0        the entry's bytes are passed over and no tensor is made (its id is 0):
 *                    for entries the host keeps itself, such as the small shape / axis
 *                    constants a graph executor reads on the host
 * weights_end checks that exactly the bytes of all entries were pushed, waits for the
 * copies and returns one tensor id per entry, in manifest order (the decode kernels may
 * still be running; stream order covers their consumers).  out_ids == NULL abandons the
 * load and frees what it made; so does any failing push followed by weights_end. */
enum tfjs_cuda_weight_storage {
  TFJS_CUDA_STORED_RAW = 0,
  TFJS_CUDA_STORED_UINT8 = 1,
  TFJS_CUDA_STORED_UINT16 = 2,
  TFJS_CUDA_STORED_FLOAT16 = 3
};
typedef struct tfjs_cuda_weight_spec {
  uint64_t n;        /* elements */
  int32_t storage;   /* tfjs_cuda_weight_storage */
  int32_t dtype;     /* tfjs_cuda_dtype of the decoded tensor */
  double scale, min; /* UINT8 / UINT16 storage */
  int32_t skip;
  int32_t reserved;
} tfjs_cuda_weight_spec;
int tfjs_cuda_weights_begin(tfjs_cuda_ctx* ctx, const tfjs_cuda_weight_spec* specs,
                            int32_t n_specs, int32_t* out_loader);
int tfjs_cuda_weights_push(tfjs_cuda_ctx* ctx, int32_t loader, const void* bytes,
                           uint64_t nbytes);
/* The whole file at `path` (one shard of weightsManifest[].paths), read with pread
 * directly into the pinned ring. */
int tfjs_cuda_weights_push_file(tfjs_cuda_ctx* ctx, int32_t loader, const char* path);
int tfjs_cuda_weights_end(tfjs_cuda_ctx* ctx, int32_t loader, int32_t* out_ids,
                          uint64_t* out_bytes);

/* ---- tfjs_cuda_dequantize for callers that must not allocate device memory.
 * No counterpart in the reference; it exists for hosts that load weights while
 * device allocation is off limits -- for example an embedding application that
 * has handed the whole GPU heap to its own arena, or a loader running while another
 * component holds the allocator -- yet still need quantised weights expanded on the
 * GPU.  Same arguments, same result, bit for bit, as tfjs_cuda_dequantize; `q_id`
 * and `out_id` are the caller's existing tensors.  The one piece of scratch the
 * kernel needs, the value lookup table, is a fixed 65536-entry (256 KiB) array
 * compiled into the library; each GPU that loads the library carries it until the
 * process ends.  The call performs no cudaMalloc / cudaFree and uses no pool.
 *   - Limit: quantised types up to 2 bytes (uint8, uint16).  Anything wider would
 *     overflow the table and is refused with TFJS_CUDA_UNSUPPORTED and a message.
 *   - The first call on each device looks up the table's device address; make that
 *     first call outside any stream capture.
 *   - All calls on a GPU share the one table.  Each call rewrites every entry it
 *     will read, so nothing carries over from earlier calls; but two calls whose
 *     GPU work overlaps (two contexts on one device, each with its own stream) would
 *     overwrite each other's table.  Serialise them, e.g. sync the first context
 *     before the second one calls.
 *   - The table is built on the host in one fixed array shared by the whole process
 *     (all GPUs).  The library takes a lock around filling it and handing it to the
 *     driver, so host threads may call concurrently for different GPUs; they simply
 *     take turns for those few microseconds. */
int tfjs_cuda_dequantize_static(tfjs_cuda_ctx* ctx, int32_t q_dtype_bytes,
                                int32_t to_dtype, int32_t q_id, double scale,
                                double min, uint64_t n, int32_t out_id);

#ifdef __cplusplus
}
#endif
#endif /* TFJS_CUDA_H_ */
