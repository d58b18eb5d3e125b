// N-API shim over the C ABI of libtfjs_cuda.so (include/tfjs_cuda.h).
//
// One exported function per C entry point, forwarding arguments one to one; a
// non-zero status becomes a JavaScript exception carrying tfjs_cuda_last_error().
// The shape follows tfjs-node's addon (tfjs-node/binding/tfjs_binding.cc), but
// with typed per-kernel calls instead of a generic op executor.
//
// Calling convention used by the TypeScript side:
//   ctx        napi external holding tfjs_cuda_ctx*
//   ids        JS numbers (int32); 0 = absent optional tensor
//   params     ArrayBuffer laid out exactly like the C struct (built with DataView)
//   shapes     BigInt64Array
#include <node_api.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "tfjs_cuda.h"

namespace {

struct Args {
  napi_env env;
  std::vector<napi_value> v;
  Args(napi_env e, napi_callback_info info) : env(e), v(16) {
    size_t n = v.size();
    napi_get_cb_info(env, info, &n, v.data(), nullptr, nullptr);
    v.resize(n);
  }
  tfjs_cuda_ctx* ctx(size_t i) const {
    void* p = nullptr;
    napi_get_value_external(env, v[i], &p);
    return static_cast<tfjs_cuda_ctx*>(p);
  }
  int32_t i32(size_t i) const { int32_t x = 0; napi_get_value_int32(env, v[i], &x); return x; }
  double f64(size_t i) const { double x = 0; napi_get_value_double(env, v[i], &x); return x; }
  uint64_t u64(size_t i) const { return static_cast<uint64_t>(f64(i)); }
  void* buffer(size_t i, size_t* len = nullptr) const {
    void* p = nullptr; size_t n = 0;
    bool is_ta = false;
    napi_is_typedarray(env, v[i], &is_ta);
    if (is_ta) {
      napi_typedarray_type t; napi_value ab; size_t off;
      napi_get_typedarray_info(env, v[i], &t, &n, &p, &ab, &off);
    } else {
      napi_get_arraybuffer_info(env, v[i], &p, &n);
    }
    if (len) *len = n;
    return p;
  }
  // An Int32Array argument (element count in *count), or nullptr for null / undefined.
  const int32_t* i32array(size_t i, size_t* count) const {
    bool is_ta = false;
    if (i < v.size()) napi_is_typedarray(env, v[i], &is_ta);
    if (!is_ta) {
      if (count) *count = 0;
      return nullptr;
    }
    size_t n = 0;   // typed arrays report their length in elements
    void* p = buffer(i, &n);
    if (count) *count = n;
    return static_cast<const int32_t*>(p);
  }
};

napi_value undefined(napi_env env) { napi_value u; napi_get_undefined(env, &u); return u; }

napi_value check(napi_env env, tfjs_cuda_ctx* ctx, int rc) {
  if (rc != TFJS_CUDA_OK) napi_throw_error(env, nullptr, tfjs_cuda_last_error(ctx));
  return undefined(env);
}

napi_value num(napi_env env, double x) { napi_value r; napi_create_double(env, x, &r); return r; }

// ---- context and storage -----------------------------------------------------
napi_value Create(napi_env env, napi_callback_info info) {
  Args a(env, info);
  tfjs_cuda_ctx* ctx = nullptr;
  if (tfjs_cuda_create(a.i32(0), &ctx) != TFJS_CUDA_OK) {
    napi_throw_error(env, nullptr, "tfjs_cuda_create failed: no usable sm_100a GPU");
    return undefined(env);
  }
  napi_value ext;
  napi_create_external(env, ctx, [](napi_env, void* p, void*) {
    tfjs_cuda_destroy(static_cast<tfjs_cuda_ctx*>(p)); }, nullptr, &ext);
  return ext;
}
napi_value Alloc(napi_env env, napi_callback_info info) {
  Args a(env, info); int32_t id = 0;
  check(env, a.ctx(0), tfjs_cuda_alloc(a.ctx(0), a.u64(1), &id));
  return num(env, id);
}
napi_value Free(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_free(a.ctx(0), a.i32(1)));
}
napi_value Write(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_write(a.ctx(0), a.i32(1), a.buffer(2), a.u64(3)));
}
napi_value Read(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_read(a.ctx(0), a.i32(1), a.buffer(2), a.u64(3)));
}
napi_value Sync(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_sync(a.ctx(0)));
}
napi_value Memory(napi_env env, napi_callback_info info) {
  Args a(env, info); uint64_t u[4] = {0, 0, 0, 0};
  check(env, a.ctx(0), tfjs_cuda_memory(a.ctx(0), &u[0], &u[1], &u[2], &u[3]));
  napi_value o; napi_create_object(env, &o);
  const char* names[4] = {"numBytesInGPU", "numBytesInGPUAllocated", "poolHighWater", "numDeviceBuffers"};
  for (int i = 0; i < 4; ++i) napi_set_named_property(env, o, names[i], num(env, (double)u[i]));
  return o;
}
napi_value TimeBegin(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_time_begin(a.ctx(0)));
}
napi_value TimeEnd(napi_env env, napi_callback_info info) {
  Args a(env, info); float ms = 0;
  check(env, a.ctx(0), tfjs_cuda_time_end(a.ctx(0), &ms));
  return num(env, ms);
}
napi_value ReadBegin(napi_env env, napi_callback_info info) {
  Args a(env, info);
  int32_t ticket = 0;
  napi_value bad = check(env, a.ctx(0), tfjs_cuda_read_begin(a.ctx(0), a.i32(1), a.buffer(2), a.u64(3), &ticket));
  (void)bad;
  return num(env, ticket);
}
napi_value ReadWait(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_read_wait(a.ctx(0), a.i32(1)));
}
napi_value FusedElementwise(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_ew_program*>(a.buffer(1));   // packed program struct
  return check(env, a.ctx(0), tfjs_cuda_fused_elementwise(a.ctx(0), p, a.i32(2)));
}
napi_value FusedElementwiseCatalogued(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_ew_program*>(a.buffer(1));
  int32_t yes = 0;
  check(env, a.ctx(0), tfjs_cuda_fused_elementwise_catalogued(a.ctx(0), p, &yes));
  return num(env, yes);
}
napi_value DecodeFloat16(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_decode_float16(a.ctx(0), a.i32(1), a.u64(2), a.i32(3)));
}
napi_value CaptureBegin(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_capture_begin(a.ctx(0), a.u64(1)));
}
napi_value CaptureEnd(napi_env env, napi_callback_info info) {
  Args a(env, info);
  int32_t graph = 0;
  check(env, a.ctx(0), tfjs_cuda_capture_end(a.ctx(0), a.i32(1), &graph));
  return num(env, graph);
}
napi_value GraphLaunch(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_graph_launch(a.ctx(0), a.i32(1)));
}
napi_value GraphDestroy(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_graph_destroy(a.ctx(0), a.i32(1)));
}
napi_value Copy(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_copy(a.ctx(0), a.i32(1), a.i32(2), a.u64(3)));
}
napi_value HighWaterReset(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_high_water_reset(a.ctx(0)));
}
napi_value SetMathMode(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_set_math_mode(a.ctx(0), a.i32(1)));
}

// ---- kernels -----------------------------------------------------------------
napi_value FusedConv2D(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_fused_conv2d(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4), a.i32(5), a.i32(6)));
}
napi_value FusedConv2DResidual(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_fused_conv2d_residual(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4), a.i32(5), a.i32(6), a.i32(7), a.i32(8)));
}
// Returns false when the library does not take the shapes (the caller then launches the two
// kernels separately); other errors throw.
napi_value FusedDepthwiseProject(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, dwParams, pwParams, x, dwFilter, dwBias, pwFilter, pwBias, residual, postAct, out
  auto* dw = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(1));
  auto* pw = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(2));
  const int rc = tfjs_cuda_fused_depthwise_project(a.ctx(0), dw, pw, a.i32(3), a.i32(4), a.i32(5), a.i32(6),
                                                   a.i32(7), a.i32(8), a.i32(9), a.i32(10));
  napi_value r;
  napi_get_boolean(env, rc == TFJS_CUDA_OK, &r);
  if (rc != TFJS_CUDA_OK && rc != TFJS_CUDA_UNSUPPORTED) napi_throw_error(env, nullptr, tfjs_cuda_last_error(a.ctx(0)));
  return r;
}
napi_value AddActivation(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_add_activation(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.u64(4), a.i32(5)));
}
napi_value FusedDepthwiseConv2D(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_fused_depthwise_conv2d(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4), a.i32(5), a.i32(6)));
}
napi_value FusedMatMul(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_matmul_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_fused_matmul(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4), a.i32(5), a.i32(6)));
}
napi_value FusedMatMulHeads(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, params, aId, bId, biasId, preluId, layout, rowsOrHeads, headDim, outId
  auto* p = static_cast<tfjs_cuda_matmul_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_fused_matmul_heads(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4), a.i32(5),
                                                           a.i32(6), a.i32(7), a.i32(8), a.i32(9)));
}
// ctx, params, aId, bIds (Int32Array), biasIds (Int32Array or null), layout, rowsOrHeads, headDim,
// outIds (Int32Array).  Returns false when the library does not take the group (the caller
// then launches the members one by one); other errors throw.
napi_value FusedMatMulGroup(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_matmul_params*>(a.buffer(1));
  size_t count = 0;
  const int32_t* b_ids = a.i32array(3, &count);
  const int32_t* bias_ids = a.i32array(4, nullptr);
  const int32_t* out_ids = a.i32array(8, nullptr);
  const int rc = tfjs_cuda_fused_matmul_group(a.ctx(0), p, a.i32(2), (int32_t)count, b_ids, bias_ids,
                                              a.i32(5), a.i32(6), a.i32(7), out_ids);
  napi_value r;
  napi_get_boolean(env, rc == TFJS_CUDA_OK, &r);
  if (rc != TFJS_CUDA_OK && rc != TFJS_CUDA_UNSUPPORTED) napi_throw_error(env, nullptr, tfjs_cuda_last_error(a.ctx(0)));
  return r;
}
napi_value Pool2D(napi_env env, napi_callback_info info) {
  Args a(env, info);
  auto* p = static_cast<tfjs_cuda_conv2d_params*>(a.buffer(1));
  return check(env, a.ctx(0), tfjs_cuda_pool2d(a.ctx(0), p, a.i32(2), a.i32(3), a.i32(4)));
}
napi_value Binary(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, op, dtype, rank, aId, aShape, bId, bShape, outId, outShape
  return check(env, a.ctx(0), tfjs_cuda_binary(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.i32(4),
      static_cast<int64_t*>(a.buffer(5)), a.i32(6), static_cast<int64_t*>(a.buffer(7)), a.i32(8),
      static_cast<int64_t*>(a.buffer(9))));
}
napi_value Unary(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, op, p0, p1, xId, n, outId
  return check(env, a.ctx(0), tfjs_cuda_unary(a.ctx(0), a.i32(1), a.f64(2), a.f64(3), a.i32(4), a.u64(5), a.i32(6)));
}
napi_value Softmax(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_softmax(a.ctx(0), a.i32(1), a.u64(2), a.u64(3), a.i32(4)));
}
napi_value SoftmaxScaledMasked(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, xId, rows, cols, hasScale, scale, maskId, rowsPerMask, outId
  return check(env, a.ctx(0), tfjs_cuda_softmax_scaled_masked(a.ctx(0), a.i32(1), a.u64(2), a.u64(3), a.i32(4),
                                                              static_cast<float>(a.f64(5)), a.i32(6), a.u64(7), a.i32(8)));
}
napi_value FusedAttention(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, qId, kId, vId, maskId (0: none), hasScale, scale, batch, heads, seq, headDim,
                      // unitsPerMask, outId; false when the library does not take the shape
  const int rc = tfjs_cuda_fused_attention(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.i32(4), a.i32(5),
                                           static_cast<float>(a.f64(6)), a.i32(7), a.i32(8), a.i32(9),
                                           a.i32(10), a.i32(11), a.i32(12));
  napi_value r;
  napi_get_boolean(env, rc == TFJS_CUDA_OK, &r);
  if (rc != TFJS_CUDA_OK && rc != TFJS_CUDA_UNSUPPORTED) napi_throw_error(env, nullptr, tfjs_cuda_last_error(a.ctx(0)));
  return r;
}
napi_value LayerNorm(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, xId, residualId (0: none), gammaId, betaId, rows, cols, epsilon, outId
  return check(env, a.ctx(0), tfjs_cuda_layer_norm(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.i32(4), a.u64(5),
                                                   a.u64(6), static_cast<float>(a.f64(7)), a.i32(8)));
}
napi_value Reduce(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_reduce(a.ctx(0), a.i32(1), a.i32(2), a.u64(3), a.u64(4), a.u64(5), a.i32(6)));
}
napi_value ArgMax(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_argmax(a.ctx(0), a.i32(1), a.u64(2), a.u64(3), a.u64(4), a.i32(5)));
}
napi_value Transpose(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, elemBytes, rank, xId, xShape(BigInt64Array), perm(Int32Array), outId
  return check(env, a.ctx(0), tfjs_cuda_transpose(a.ctx(0), a.i32(1), a.i32(2), a.i32(3),
      static_cast<int64_t*>(a.buffer(4)), static_cast<int32_t*>(a.buffer(5)), a.i32(6)));
}
napi_value Gather(napi_env env, napi_callback_info info) {
  Args a(env, info); int64_t bad = -1;
  check(env, a.ctx(0), tfjs_cuda_gather(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.u64(4), a.u64(5),
                                          a.u64(6), a.u64(7), a.u64(8), a.i32(9), a.i32(10), &bad));
  return num(env, (double)bad);
}
napi_value Cast(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_cast(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.u64(4), a.i32(5)));
}
napi_value CopyStrided(napi_env env, napi_callback_info info) {
  Args a(env, info);  // ctx, elemBytes, rank, extent, xId, xOff, xStrides, xWrap, outId, oOff, oStrides
  return check(env, a.ctx(0), tfjs_cuda_copy_strided(a.ctx(0), a.i32(1), a.i32(2),
      static_cast<int64_t*>(a.buffer(3)), a.i32(4), (int64_t)a.f64(5), static_cast<int64_t*>(a.buffer(6)),
      static_cast<int64_t*>(a.buffer(7)), a.i32(8), (int64_t)a.f64(9), static_cast<int64_t*>(a.buffer(10))));
}
napi_value Fill(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_fill(a.ctx(0), a.i32(1), (uint32_t)a.u64(2), a.i32(3), a.u64(4)));
}
napi_value BatchNorm(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_batchnorm(a.ctx(0), a.i32(1), a.u64(2), a.i32(3), a.u64(4), a.i32(5),
      a.u64(6), a.i32(7), a.u64(8), a.i32(9), a.u64(10), a.f64(11), a.i32(12)));
}
napi_value Dequantize(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_dequantize(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.f64(4), a.f64(5), a.u64(6), a.i32(7)));
}
napi_value DequantizeStatic(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_dequantize_static(a.ctx(0), a.i32(1), a.i32(2), a.i32(3), a.f64(4), a.f64(5), a.u64(6), a.i32(7)));
}

napi_value BatchNormRows(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_batchnorm_rows(a.ctx(0), a.i32(1), a.u64(2), a.u64(3), a.i32(4), a.i32(5),
      a.i32(6), a.i32(7), a.i32(8), a.i32(9), a.i32(10), a.i32(11), a.f64(12), a.i32(13)));
}

// ---- the rest of the storage contract ------------------------------------------
napi_value DeviceCount(napi_env env, napi_callback_info info) {
  int n = 0; tfjs_cuda_device_count(&n); return num(env, n);
}
napi_value Upload(napi_env env, napi_callback_info info) {
  Args a(env, info); int32_t id = 0;
  check(env, a.ctx(0), tfjs_cuda_upload(a.ctx(0), a.buffer(1), a.u64(2), &id));
  return num(env, id);
}
napi_value ReadAsync(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_read_async(a.ctx(0), a.i32(1), a.buffer(2), a.u64(3)));
}
napi_value SizeOf(napi_env env, napi_callback_info info) {
  Args a(env, info); uint64_t n = 0;
  check(env, a.ctx(0), tfjs_cuda_size_of(a.ctx(0), a.i32(1), &n));
  return num(env, (double)n);
}
napi_value DevicePtr(napi_env env, napi_callback_info info) {
  Args a(env, info); void* p = nullptr;
  check(env, a.ctx(0), tfjs_cuda_device_ptr(a.ctx(0), a.i32(1), &p));
  napi_value r; napi_create_bigint_uint64(env, (uint64_t)(uintptr_t)p, &r); return r;
}
napi_value Trim(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_trim(a.ctx(0)));
}
// Pinned staging memory as an ArrayBuffer; released with hostFree (the finaliser does
// nothing, so a buffer that is merely dropped stays pinned until the context goes).
napi_value HostAlloc(napi_env env, napi_callback_info info) {
  Args a(env, info); void* p = nullptr;
  const uint64_t n = a.u64(1);
  check(env, a.ctx(0), tfjs_cuda_host_alloc(a.ctx(0), n, &p));
  napi_value ab;
  napi_create_external_arraybuffer(env, p, (size_t)n, nullptr, nullptr, &ab);
  return ab;
}
napi_value HostFree(napi_env env, napi_callback_info info) {
  Args a(env, info);
  return check(env, a.ctx(0), tfjs_cuda_host_free(a.ctx(0), a.buffer(1)));
}
napi_value EventRecord(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_event_record(a.ctx(0), a.i32(1)));
}
napi_value EventElapsed(napi_env env, napi_callback_info info) {
  Args a(env, info); float ms = 0;
  check(env, a.ctx(0), tfjs_cuda_event_elapsed(a.ctx(0), a.i32(1), a.i32(2), &ms));
  return num(env, ms);
}
napi_value LaunchCount(napi_env env, napi_callback_info info) {
  Args a(env, info); uint64_t n = 0;
  check(env, a.ctx(0), tfjs_cuda_launch_count(a.ctx(0), &n));
  return num(env, (double)n);
}
napi_value LaunchLog(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_launch_log(a.ctx(0), a.i32(1)));
}
napi_value LaunchLogTake(napi_env env, napi_callback_info info) {
  Args a(env, info);
  char text[4096]; uint32_t n = 0;
  check(env, a.ctx(0), tfjs_cuda_launch_log_take(a.ctx(0), text, sizeof text, &n));
  napi_value r; napi_create_string_utf8(env, text, NAPI_AUTO_LENGTH, &r); return r;
}
napi_value FlushL2(napi_env env, napi_callback_info info) {
  Args a(env, info); return check(env, a.ctx(0), tfjs_cuda_flush_l2(a.ctx(0)));
}

// ---- weight loader: the entry list is an ArrayBuffer of packed tfjs_cuda_weight_spec ---
napi_value WeightsBegin(napi_env env, napi_callback_info info) {
  Args a(env, info); size_t len = 0; int32_t loader = 0;
  auto* specs = static_cast<tfjs_cuda_weight_spec*>(a.buffer(1, &len));
  check(env, a.ctx(0), tfjs_cuda_weights_begin(a.ctx(0), specs, (int32_t)(len / sizeof(tfjs_cuda_weight_spec)), &loader));
  return num(env, loader);
}
napi_value WeightsPush(napi_env env, napi_callback_info info) {
  Args a(env, info); size_t len = 0;
  void* p = a.buffer(2, &len);
  return check(env, a.ctx(0), tfjs_cuda_weights_push(a.ctx(0), a.i32(1), p, (uint64_t)len));
}
napi_value WeightsPushFile(napi_env env, napi_callback_info info) {
  Args a(env, info); char path[4096]; size_t n = 0;
  napi_get_value_string_utf8(env, a.v[2], path, sizeof path, &n);
  return check(env, a.ctx(0), tfjs_cuda_weights_push_file(a.ctx(0), a.i32(1), path));
}
// weightsEnd(ctx, loader, ids: Int32Array | null): null abandons the load
napi_value WeightsEnd(napi_env env, napi_callback_info info) {
  Args a(env, info);
  napi_valuetype t; napi_typeof(env, a.v[2], &t);
  int32_t* ids = t == napi_null || t == napi_undefined ? nullptr : static_cast<int32_t*>(a.buffer(2));
  uint64_t bytes = 0;
  check(env, a.ctx(0), tfjs_cuda_weights_end(a.ctx(0), a.i32(1), ids, &bytes));
  return num(env, (double)bytes);
}

napi_value Init(napi_env env, napi_value exports) {
  struct { const char* name; napi_callback fn; } table[] = {
      {"create", Create}, {"alloc", Alloc}, {"free", Free}, {"write", Write}, {"read", Read},
      {"fusedElementwise", FusedElementwise},
      {"fusedElementwiseCatalogued", FusedElementwiseCatalogued}, {"decodeFloat16", DecodeFloat16}, {"captureBegin", CaptureBegin}, {"captureEnd", CaptureEnd}, {"graphLaunch", GraphLaunch},
      {"graphDestroy", GraphDestroy}, {"copy", Copy}, {"highWaterReset", HighWaterReset},
      {"readBegin", ReadBegin}, {"readWait", ReadWait}, {"sync", Sync}, {"memory", Memory}, {"timeBegin", TimeBegin}, {"timeEnd", TimeEnd},
      {"setMathMode", SetMathMode}, {"fusedConv2d", FusedConv2D},
      {"fusedConv2dResidual", FusedConv2DResidual}, {"fusedDepthwiseProject", FusedDepthwiseProject},
      {"addActivation", AddActivation},
      {"fusedDepthwiseConv2d", FusedDepthwiseConv2D}, {"fusedMatMul", FusedMatMul}, {"fusedMatMulHeads", FusedMatMulHeads}, {"fusedMatMulGroup", FusedMatMulGroup},
      {"pool2d", Pool2D}, {"binary", Binary}, {"unary", Unary}, {"softmax", Softmax}, {"layerNorm", LayerNorm}, {"softmaxScaledMasked", SoftmaxScaledMasked}, {"fusedAttention", FusedAttention},
      {"reduce", Reduce}, {"argMax", ArgMax}, {"transpose", Transpose}, {"gather", Gather},
      {"cast", Cast}, {"copyStrided", CopyStrided}, {"fill", Fill}, {"batchNorm", BatchNorm},
      {"dequantize", Dequantize}, {"dequantizeStatic", DequantizeStatic},
      {"batchNormRows", BatchNormRows}, {"deviceCount", DeviceCount}, {"upload", Upload},
      {"readAsync", ReadAsync}, {"sizeOf", SizeOf}, {"devicePtr", DevicePtr}, {"trim", Trim},
      {"hostAlloc", HostAlloc}, {"hostFree", HostFree}, {"eventRecord", EventRecord},
      {"eventElapsed", EventElapsed}, {"launchCount", LaunchCount}, {"launchLog", LaunchLog},
      {"launchLogTake", LaunchLogTake}, {"flushL2", FlushL2}, {"weightsBegin", WeightsBegin},
      {"weightsPush", WeightsPush}, {"weightsPushFile", WeightsPushFile},
      {"weightsEnd", WeightsEnd}};
  for (auto& e : table) {
    napi_value fn;
    napi_create_function(env, e.name, NAPI_AUTO_LENGTH, e.fn, nullptr, &fn);
    napi_set_named_property(env, exports, e.name, fn);
  }
  return exports;
}

}  // namespace

NAPI_MODULE(NODE_GYP_MODULE_NAME, Init)
