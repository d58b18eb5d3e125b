// Context, device-memory pool, id -> buffer table, host<->device transfer.
//
// The device half of the KernelBackend storage contract
// (tfjs-core/src/backends/backend.ts:100-156).  Ref-counting stays with the
// host-side DataStorage, as in the reference's WASM backend where the C++ side
// only maps tensor ids to memory (tfjs-backend-wasm/src/cc/backend.cc:124-152).
//
// Kernels, small transfers and frees run on ONE in-order stream (overlapped uploads and
// large downloads have a copy stream and a read stream of their own, ordered against it by
// events).  The
// graph executor disposes an intermediate as soon as its last consumer has
// been *enqueued* (tfjs-converter/src/executor/graph_executor.ts:382-409), so
// frees are stream-ordered (cudaFreeAsync) and a block can be handed to a later
// kernel without any host-side wait.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

int ctx_fail(tfjs_cuda_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return code;
}

int ctx_check(tfjs_cuda_ctx* ctx, cudaError_t e, const char* what) {
  if (e == cudaSuccess) return TFJS_CUDA_OK;
  int code = e == cudaErrorMemoryAllocation ? TFJS_CUDA_OUT_OF_MEMORY
                                            : TFJS_CUDA_DRIVER_ERROR;
  return ctx_fail(ctx, code, "%s: %s", what, cudaGetErrorString(e));
}

Buffer* ctx_buf(tfjs_cuda_ctx* ctx, int32_t id) {
  if (id <= 0 || (size_t)id >= ctx->bufs.size()) return nullptr;
  Buffer* b = &ctx->bufs[id];
  return b->live ? b : nullptr;
}

int ctx_get(tfjs_cuda_ctx* ctx, int32_t id, uint64_t need, const char* name,
            Buffer** out) {
  Buffer* b = ctx_buf(ctx, id);
  if (!b) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "%s: unknown tensor id %d",
                          name, id);
  if (b->bytes < need)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                    "%s: tensor id %d holds %llu bytes, kernel needs %llu", name,
                    id, (unsigned long long)b->bytes, (unsigned long long)need);
  if (b->ready) {
    NOT_WHILE_CAPTURING(ctx, "a tensor whose upload is still pending");
    // first use after an overlapped upload: order the compute stream behind the copy
    cudaStreamWaitEvent(ctx->stream, b->ready, 0);
    ctx->event_pool.push_back(b->ready);
    b->ready = nullptr;
  }
  *out = b;
  return TFJS_CUDA_OK;
}

int ctx_scratch(tfjs_cuda_ctx* ctx, uint64_t bytes, void** out) {
  if (bytes > ctx->scratch_bytes) {
    NOT_WHILE_CAPTURING(ctx, "growing the scratch buffer");
    // captured steps that use the scratch buffer carry its old address
    for (ReplayGraph& g : ctx->graphs)
      if (g.exec && g.uses_scratch) g.stale = true;
    if (ctx->scratch) CUDA_TRY(ctx, cudaFreeAsync(ctx->scratch, ctx->stream));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    uint64_t want = bytes + (bytes >> 2);
    CUDA_TRY(ctx, cudaMallocAsync(&ctx->scratch, want, ctx->stream));
    ctx->scratch_bytes = want;
  }
  if (ctx->capturing) ctx->capture_scratch = true;
  *out = ctx->scratch;
  return TFJS_CUDA_OK;
}

void ctx_mark_written(tfjs_cuda_ctx* ctx, int32_t id) {
  Buffer* b = ctx_buf(ctx, id);
  if (b) {
    b->version++;
    b->from_host = false;
  }
}

void ctx_packed_contents_changed(tfjs_cuda_ctx* ctx, int32_t id) {
  for (ReplayGraph& g : ctx->graphs)
    if (g.exec)
      for (int32_t w : g.packed_ids)
        if (w == id) g.stale = true;
}

void ctx_drop_packed(tfjs_cuda_ctx* ctx, int32_t id) {
  auto it = ctx->packed.find(id);
  if (it == ctx->packed.end()) return;
  // captured steps that read this packed copy carry its address
  ctx_packed_contents_changed(ctx, id);
  if (it->second.ptr) cudaFreeAsync(it->second.ptr, ctx->stream);
  ctx->packed.erase(it);
}

static void cache_flush(tfjs_cuda_ctx* ctx) {
  for (auto& kv : ctx->block_cache)
    for (void* p : kv.second) cudaFreeAsync(p, ctx->stream);
  ctx->block_cache.clear();
  for (UploadBlock& u : ctx->upload_cache) {
    cudaStreamWaitEvent(ctx->stream, u.released, 0);
    cudaFreeAsync(u.ptr, ctx->stream);
    ctx->event_pool.push_back(u.released);
  }
  ctx->upload_cache.clear();
  ctx->cached_bytes = 0;
}

// Pool allocation for tensors: exact-size cache first, then the stream-ordered pool;
// on failure the cache is returned to the pool and the request retried once.
// Best-fit allocator over the arena of the step being captured.  The captured step is
// one chain of graph nodes in launch order, so a span freed by the host may be handed
// to a later node straight away, exactly like the stream-ordered blocks outside capture.
static bool arena_alloc(tfjs_cuda_ctx* ctx, uint64_t padded, void** out) {
  // best fit: the smallest free span that holds the request (a model's steps ask for a few
  // distinct sizes over and over, so an exact-size hole is usually there to be found)
  int best = -1;
  for (size_t i = 0; i < ctx->arena_free.size(); ++i) {
    const ArenaSpan& f = ctx->arena_free[i];
    if (f.size < padded) continue;
    if (best < 0 || f.size < ctx->arena_free[best].size) best = (int)i;
    if (f.size == padded) break;
  }
  if (best < 0) return false;
  ArenaSpan& f = ctx->arena_free[best];
  *out = (char*)ctx->arena + f.off;
  f.off += padded;
  f.size -= padded;
  if (f.size == 0) ctx->arena_free.erase(ctx->arena_free.begin() + best);
  return true;
}

static void arena_release(tfjs_cuda_ctx* ctx, void* p, uint64_t padded) {
  const uint64_t off = (uint64_t)((char*)p - (char*)ctx->arena);
  size_t i = 0;
  while (i < ctx->arena_free.size() && ctx->arena_free[i].off < off) ++i;
  ctx->arena_free.insert(ctx->arena_free.begin() + i, ArenaSpan{off, padded});
  if (i + 1 < ctx->arena_free.size() &&
      ctx->arena_free[i].off + ctx->arena_free[i].size == ctx->arena_free[i + 1].off) {
    ctx->arena_free[i].size += ctx->arena_free[i + 1].size;
    ctx->arena_free.erase(ctx->arena_free.begin() + i + 1);
  }
  if (i > 0 && ctx->arena_free[i - 1].off + ctx->arena_free[i - 1].size == ctx->arena_free[i].off) {
    ctx->arena_free[i - 1].size += ctx->arena_free[i].size;
    ctx->arena_free.erase(ctx->arena_free.begin() + i);
  }
}

static cudaError_t block_alloc(tfjs_cuda_ctx* ctx, uint64_t padded, void** out) {
  auto it = ctx->block_cache.find(padded);
  if (it != ctx->block_cache.end() && !it->second.empty()) {
    *out = it->second.back();
    it->second.pop_back();
    ctx->cached_bytes -= padded;
    return cudaSuccess;
  }
  cudaError_t e = cudaMallocAsync(out, padded, ctx->stream);
  if (e == cudaErrorMemoryAllocation && ctx->cached_bytes) {
    cudaGetLastError();
    cache_flush(ctx);
    cudaStreamSynchronize(ctx->stream);
    e = cudaMallocAsync(out, padded, ctx->stream);
  }
  return e;
}

static void block_free(tfjs_cuda_ctx* ctx, void* p, uint64_t padded) {
  ctx->block_cache[padded].push_back(p);
  ctx->cached_bytes += padded;
}

extern "C" {

int tfjs_cuda_device_count(int* out_count) {
  if (!out_count) return TFJS_CUDA_INVALID_ARG;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  *out_count = e == cudaSuccess ? n : 0;
  return e == cudaSuccess ? TFJS_CUDA_OK : TFJS_CUDA_DRIVER_ERROR;
}

int tfjs_cuda_create(int device_ordinal, tfjs_cuda_ctx** out_ctx) {
  if (!out_ctx) return TFJS_CUDA_INVALID_ARG;
  *out_ctx = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device_ordinal < 0 ||
      device_ordinal >= n)
    return TFJS_CUDA_INVALID_ARG;
  if (cudaSetDevice(device_ordinal) != cudaSuccess)
    return TFJS_CUDA_DRIVER_ERROR;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess)
    return TFJS_CUDA_DRIVER_ERROR;
  if (prop.major != 10) {
    fprintf(stderr,
            "tfjs_cuda: device %d is sm_%d%d; this library carries sm_100a "
            "code only\n",
            device_ordinal, prop.major, prop.minor);
    return TFJS_CUDA_UNSUPPORTED;
  }
  tfjs_cuda_ctx* ctx = new tfjs_cuda_ctx();
  ctx->device = device_ordinal;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->bufs.resize(1);
  bool ok = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) ==
            cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaStreamCreateWithFlags(&ctx->read_stream, cudaStreamNonBlocking) == cudaSuccess;
  ok = ok && cudaDeviceGetDefaultMemPool(&ctx->pool, device_ordinal) ==
                 cudaSuccess;
  if (ok) {
    // Keep freed blocks in the pool instead of returning them to the driver.
    uint64_t threshold = UINT64_MAX;
    ok = cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold,
                                 &threshold) == cudaSuccess;
  }
  ok = ok && cudaMalloc(&ctx->d_flag, sizeof(int)) == cudaSuccess;
  ok = ok && cudaMemset(ctx->d_flag, 0, sizeof(int)) == cudaSuccess;
  ok = ok && cudaMallocHost(&ctx->h_flag, sizeof(int)) == cudaSuccess;
  ok = ok && cudaMalloc(&ctx->d_bad_index, sizeof(long long)) == cudaSuccess;
  ok = ok && cudaMallocHost(&ctx->h_bad_index, sizeof(long long)) == cudaSuccess;
  ok = ok && cudaEventCreate(&ctx->ev0) == cudaSuccess;
  ok = ok && cudaEventCreate(&ctx->ev1) == cudaSuccess;
  if (!ok) {
    fprintf(stderr, "tfjs_cuda: context setup failed: %s\n",
            cudaGetErrorString(cudaGetLastError()));
    tfjs_cuda_destroy(ctx);
    return TFJS_CUDA_DRIVER_ERROR;
  }
  *ctx->h_flag = 0;
  *out_ctx = ctx;
  return TFJS_CUDA_OK;
}

void tfjs_cuda_destroy(tfjs_cuda_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  loaders_drop(ctx);
  for (auto& kv : ctx->packed)
    if (kv.second.ptr) cudaFreeAsync(kv.second.ptr, ctx->stream);
  for (auto& b : ctx->bufs)
    if (b.live && b.ptr) cudaFreeAsync(b.ptr, ctx->stream);
  cache_flush(ctx);
  if (ctx->scratch) cudaFreeAsync(ctx->scratch, ctx->stream);
  if (ctx->l2_scratch) cudaFreeAsync(ctx->l2_scratch, ctx->stream);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  if (ctx->sk_ws) cudaFree(ctx->sk_ws);
  if (ctx->sk_flags) cudaFree(ctx->sk_flags);
  if (ctx->d_flag) cudaFree(ctx->d_flag);
  if (ctx->h_flag) cudaFreeHost(ctx->h_flag);
  if (ctx->d_bad_index) cudaFree(ctx->d_bad_index);
  if (ctx->h_bad_index) cudaFreeHost(ctx->h_bad_index);
  for (cudaEvent_t e : ctx->prof_events)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : ctx->event_pool) cudaEventDestroy(e);
  if (ctx->read_stream) {
    cudaStreamSynchronize(ctx->read_stream);
    cudaStreamDestroy(ctx->read_stream);
  }
  for (cudaEvent_t e : ctx->read_events) cudaEventDestroy(e);
  for (cudaEvent_t e : ctx->read_order) cudaEventDestroy(e);
  for (int* w : ctx->read_flags) cudaFreeHost(w);
  for (ReplayGraph& g : ctx->graphs)
    if (g.exec) {
      cudaGraphExecDestroy(g.exec);
      cudaFree(g.arena);
    }
  for (auto& b : ctx->bufs)
    if (b.ready) cudaEventDestroy(b.ready);
  if (ctx->copy_stream) {
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
  }
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

const char* tfjs_cuda_last_error(tfjs_cuda_ctx* ctx) {
  return ctx ? ctx->err.c_str() : "null context";
}

int tfjs_cuda_alloc(tfjs_cuda_ctx* ctx, uint64_t nbytes, int32_t* out_id) {
  if (!ctx || !out_id) return TFJS_CUDA_INVALID_ARG;
  cudaSetDevice(ctx->device);
  void* p = nullptr;
  // Round up so vectorised kernels may read a full 16-byte tail.
  uint64_t padded = ((nbytes + 255) / 256) * 256;
  if (padded == 0) padded = 256;
  const bool in_arena = ctx->capturing;
  if (in_arena) {
    if (!arena_alloc(ctx, padded, &p)) {
      ctx->capture_failed = true;
      return ctx_fail(ctx, TFJS_CUDA_OUT_OF_MEMORY,
                      "the arena of the step being captured is full (%llu bytes)",
                      (unsigned long long)ctx->arena_bytes);
    }
  } else {
    CUDA_TRY(ctx, block_alloc(ctx, padded, &p));
  }
  int32_t id;
  if (!ctx->free_ids.empty()) {
    id = ctx->free_ids.back();
    ctx->free_ids.pop_back();
  } else {
    id = (int32_t)ctx->bufs.size();
    ctx->bufs.emplace_back();
  }
  Buffer& b = ctx->bufs[id];
  b.ptr = p;
  b.bytes = nbytes;
  b.live = true;
  b.from_host = false;
  b.in_arena = in_arena;
  b.version++;
  ctx->in_use += padded;
  ctx->n_live++;
  if (ctx->in_use > ctx->high_water) ctx->high_water = ctx->in_use;
  *out_id = id;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_free(tfjs_cuda_ctx* ctx, int32_t id) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer* b = ctx_buf(ctx, id);
  if (!b) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "free: unknown tensor id %d", id);
  cudaSetDevice(ctx->device);
  if (ctx->capturing && (b->ready || ctx->packed.count(id)))
    NOT_WHILE_CAPTURING(ctx, "freeing a weight or a tensor whose upload is pending");
  ctx_drop_packed(ctx, id);
  if (b->ready) {  // never used since its upload: still order the free behind the copy
    cudaStreamWaitEvent(ctx->stream, b->ready, 0);
    ctx->event_pool.push_back(b->ready);
    b->ready = nullptr;
  }
  uint64_t padded = ((b->bytes + 255) / 256) * 256;
  if (padded == 0) padded = 256;
  cudaEvent_t rel = nullptr;
  if (b->in_arena) {
    // inside the capture the span goes back to the arena; afterwards (an output of a
    // captured step) the memory belongs to the graph and only the id is retired
    if (ctx->capturing) arena_release(ctx, b->ptr, padded);
    b->in_arena = false;
    b->ptr = nullptr;
    b->live = false;
    b->bytes = 0;
    ctx->in_use -= padded;
    ctx->n_live--;
    ctx->free_ids.push_back(id);
    return TFJS_CUDA_OK;
  }
  if (b->uploaded && !ctx->capturing) {
    if (!ctx->event_pool.empty()) {
      rel = ctx->event_pool.back();
      ctx->event_pool.pop_back();
    } else if (cudaEventCreateWithFlags(&rel, cudaEventDisableTiming) != cudaSuccess) {
      rel = nullptr;
    }
  }
  if (rel && cudaEventRecord(rel, ctx->stream) == cudaSuccess) {
    // every kernel that reads the tensor has been launched: the block may be refilled by
    // the copy stream once the compute stream gets here
    ctx->upload_cache.push_back(UploadBlock{b->ptr, padded, rel});
    ctx->cached_bytes += padded;
  } else {
    if (rel) ctx->event_pool.push_back(rel);
    block_free(ctx, b->ptr, padded);
  }
  b->uploaded = false;
  b->ptr = nullptr;
  b->live = false;
  b->bytes = 0;
  ctx->in_use -= padded;
  ctx->n_live--;
  ctx->free_ids.push_back(id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_write(tfjs_cuda_ctx* ctx, int32_t id, const void* host,
                    uint64_t nbytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "a host-to-device write");
  Buffer* b;
  int rc = ctx_get(ctx, id, nbytes, "write", &b);
  if (rc) return rc;
  if (nbytes == 0) return TFJS_CUDA_OK;
  if (!host) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "write: null host pointer");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaMemcpyAsync(b->ptr, host, nbytes, cudaMemcpyHostToDevice,
                                ctx->stream));
  b->version++;
  b->from_host = true;
  ctx_drop_packed(ctx, id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_upload(tfjs_cuda_ctx* ctx, const void* host, uint64_t nbytes, int32_t* out_id) {
  if (!ctx || !out_id) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "a host-to-device upload");
  if (nbytes && !host) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "upload: null host pointer");
  cudaSetDevice(ctx->device);
  void* p = nullptr;
  uint64_t padded = ((nbytes + 255) / 256) * 256;
  if (padded == 0) padded = 256;
  // Filled on the copy stream, so the transfer does not queue behind kernels already
  // launched on the compute stream.  The block is the one an earlier upload of this size
  // released longest ago, else a fresh one.
  // Prefer a block whose last reader has already finished; while fewer than two blocks of
  // this size wait for their readers, take a fresh one rather than stall the transfer.
  int same = 0, pick = -1;
  for (size_t i = 0; i < ctx->upload_cache.size(); ++i) {
    if (ctx->upload_cache[i].bytes != padded) continue;
    ++same;
    if (cudaEventQuery(ctx->upload_cache[i].released) == cudaSuccess) {
      pick = (int)i;
      break;
    }
    if (pick < 0) pick = (int)i;  // oldest, if nothing has finished
  }
  cudaGetLastError();  // cudaErrorNotReady from the queries is not an error
  if (pick >= 0 && (same >= 2 || cudaEventQuery(ctx->upload_cache[pick].released) == cudaSuccess)) {
    UploadBlock u = ctx->upload_cache[pick];
    ctx->upload_cache.erase(ctx->upload_cache.begin() + pick);
    ctx->cached_bytes -= padded;
    CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->copy_stream, u.released, 0));
    ctx->event_pool.push_back(u.released);
    p = u.ptr;
  }
  cudaGetLastError();
  if (!p) {
    cudaError_t e = cudaMallocAsync(&p, padded, ctx->copy_stream);
    if (e == cudaErrorMemoryAllocation && ctx->cached_bytes) {
      // the context itself may hold the memory: hand the cached blocks back and retry once
      cudaGetLastError();
      cache_flush(ctx);
      cudaStreamSynchronize(ctx->stream);
      e = cudaMallocAsync(&p, padded, ctx->copy_stream);
    }
    CUDA_TRY(ctx, e);
  }
  if (nbytes)
    CUDA_TRY(ctx, cudaMemcpyAsync(p, host, nbytes, cudaMemcpyHostToDevice, ctx->copy_stream));
  cudaEvent_t ev = nullptr;
  if (!ctx->event_pool.empty()) {
    ev = ctx->event_pool.back();
    ctx->event_pool.pop_back();
  } else {
    CUDA_TRY(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  }
  CUDA_TRY(ctx, cudaEventRecord(ev, ctx->copy_stream));
  int32_t id;
  if (!ctx->free_ids.empty()) {
    id = ctx->free_ids.back();
    ctx->free_ids.pop_back();
  } else {
    id = (int32_t)ctx->bufs.size();
    ctx->bufs.emplace_back();
  }
  Buffer& b = ctx->bufs[id];
  b.ptr = p;
  b.bytes = nbytes;
  b.live = true;
  b.from_host = true;
  b.version++;
  b.ready = ev;
  b.uploaded = true;
  ctx->in_use += padded;
  ctx->n_live++;
  if (ctx->in_use > ctx->high_water) ctx->high_water = ctx->in_use;
  *out_id = id;
  return TFJS_CUDA_OK;
}

// The device error word is copied to a pinned word of the caller's (the context's for a
// blocking sync, the ticket's for an asynchronous read) and cleared right behind the copy
// in stream order, so each device-side timeout is seen by exactly one copy and reported
// exactly once, by the wait that collects that copy.
static int fetch_flag(tfjs_cuda_ctx* ctx, int* host_word) {
  CUDA_TRY(ctx, cudaMemcpyAsync(host_word, ctx->d_flag, sizeof(int), cudaMemcpyDeviceToHost,
                                ctx->stream));
  CUDA_TRY(ctx, cudaMemsetAsync(ctx->d_flag, 0, sizeof(int), ctx->stream));
  return TFJS_CUDA_OK;
}

static int report_flag(tfjs_cuda_ctx* ctx, int* host_word) {
  if (*host_word != 0) {
    int v = *host_word;
    *host_word = 0;
    // a K-split GEMM that gave up may have left partial-tile flags raised
    if (ctx->sk_flags) cudaMemsetAsync(ctx->sk_flags, 0, 4096 * sizeof(unsigned), ctx->stream);
    return ctx_fail(ctx, TFJS_CUDA_DEVICE_TIMEOUT,
                    "a device-side wait gave up (code %d); results of the "
                    "affected kernel are invalid", v);
  }
  return TFJS_CUDA_OK;
}

int tfjs_cuda_sync(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "a stream synchronisation");
  cudaSetDevice(ctx->device);
  int rc = fetch_flag(ctx, ctx->h_flag);
  if (rc) return rc;
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->read_stream));   // staged downloads (read_begin)
  return report_flag(ctx, ctx->h_flag);
}

int tfjs_cuda_read_async(tfjs_cuda_ctx* ctx, int32_t id, void* host,
                         uint64_t nbytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "a device-to-host read");
  Buffer* b;
  int rc = ctx_get(ctx, id, nbytes, "read", &b);
  if (rc) return rc;
  if (nbytes == 0) return TFJS_CUDA_OK;
  if (!host) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "read: null host pointer");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaMemcpyAsync(host, b->ptr, nbytes, cudaMemcpyDeviceToHost,
                                ctx->stream));
  return TFJS_CUDA_OK;
}

// backend.read(): the D2H copy and an event are queued behind the kernels already on
// the stream; the host keeps launching and collects the bytes with read_wait.
// A large download (megabytes: a hundred microseconds and more of PCIe time) does not
// hold up the kernels launched after it: the tensor is copied to a staging block on the
// compute stream (device to device: microseconds) and travels to the host on the read
// stream, so the next step runs meanwhile and the tensor itself - which may be freed, or
// belong to the arena of a captured step that the next replay overwrites - is not touched
// after the compute stream has passed this point.
constexpr uint64_t kStagedReadBytes = 4ull << 20;

int tfjs_cuda_read_begin(tfjs_cuda_ctx* ctx, int32_t id, void* host, uint64_t nbytes,
                         int32_t* out_ticket) {
  if (!ctx || !out_ticket) return TFJS_CUDA_INVALID_ARG;
  *out_ticket = 0;
  void* staged = nullptr;
  int rc;
  if (nbytes >= kStagedReadBytes && host != nullptr && !ctx->capturing) {
    Buffer* b;
    if ((rc = ctx_get(ctx, id, nbytes, "read", &b))) return rc;
    cudaSetDevice(ctx->device);
    if (cudaMallocAsync(&staged, nbytes, ctx->stream) != cudaSuccess) {
      cudaGetLastError();        // no room for the staging block: the direct copy below
      staged = nullptr;
    } else {
      cudaError_t e = cudaMemcpyAsync(staged, b->ptr, nbytes, cudaMemcpyDeviceToDevice, ctx->stream);
      if (e != cudaSuccess) {
        cudaFreeAsync(staged, ctx->stream);
        return ctx_check(ctx, e, "cudaMemcpyAsync");
      }
    }
  }
  if (staged == nullptr) {
    rc = tfjs_cuda_read_async(ctx, id, host, nbytes);
    if (rc) return rc;
  }
  int slot;
  if (!ctx->read_free.empty()) {
    slot = ctx->read_free.back();
    ctx->read_free.pop_back();
  } else {
    cudaEvent_t ev;
    int* word = nullptr;
    CUDA_TRY(ctx, cudaMallocHost((void**)&word, sizeof(int)));
    *word = 0;
    cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e != cudaSuccess) {
      cudaFreeHost(word);
      return ctx_check(ctx, e, "cudaEventCreateWithFlags");
    }
    cudaEvent_t order;
    e = cudaEventCreateWithFlags(&order, cudaEventDisableTiming);
    if (e != cudaSuccess) {
      cudaFreeHost(word);
      cudaEventDestroy(ev);
      if (staged) cudaFreeAsync(staged, ctx->stream);
      return ctx_check(ctx, e, "cudaEventCreateWithFlags");
    }
    ctx->read_events.push_back(ev);
    ctx->read_order.push_back(order);
    ctx->read_flags.push_back(word);
    slot = (int)ctx->read_events.size() - 1;
  }
  // the device error word travels with every read, as it does with a blocking one, into
  // a pinned word that belongs to this ticket
  rc = fetch_flag(ctx, ctx->read_flags[slot]);
  if (rc == TFJS_CUDA_OK && staged != nullptr) {
    // read stream: behind the staging copy and the flag word, then host copy, release of the
    // staging block (stream-ordered) and the ticket's event
    cudaError_t e = cudaEventRecord(ctx->read_order[slot], ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->read_stream, ctx->read_order[slot], 0);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(host, staged, nbytes, cudaMemcpyDeviceToHost, ctx->read_stream);
    if (e == cudaSuccess) {
      cudaFreeAsync(staged, ctx->read_stream);
      staged = nullptr;
      e = cudaEventRecord(ctx->read_events[slot], ctx->read_stream);
    }
    rc = ctx_check(ctx, e, "staged read");
  } else if (rc == TFJS_CUDA_OK) {
    rc = ctx_check(ctx, cudaEventRecord(ctx->read_events[slot], ctx->stream), "cudaEventRecord");
  }
  if (rc) {
    if (staged) cudaFreeAsync(staged, ctx->stream);
    ctx->read_free.push_back(slot);
    return rc;
  }
  *out_ticket = slot + 1;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_read_wait(tfjs_cuda_ctx* ctx, int32_t ticket) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  const int slot = ticket - 1;
  if (slot < 0 || (size_t)slot >= ctx->read_events.size())
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "read_wait: unknown ticket %d", ticket);
  for (int f : ctx->read_free)
    if (f == slot) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "read_wait: ticket %d already collected", ticket);
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaEventSynchronize(ctx->read_events[slot]));
  ctx->read_free.push_back(slot);
  return report_flag(ctx, ctx->read_flags[slot]);
}

int tfjs_cuda_read(tfjs_cuda_ctx* ctx, int32_t id, void* host, uint64_t nbytes) {
  int rc = tfjs_cuda_read_async(ctx, id, host, nbytes);
  if (rc) return rc;
  return tfjs_cuda_sync(ctx);
}

int tfjs_cuda_size_of(tfjs_cuda_ctx* ctx, int32_t id, uint64_t* out_nbytes) {
  if (!ctx || !out_nbytes) return TFJS_CUDA_INVALID_ARG;
  Buffer* b = ctx_buf(ctx, id);
  if (!b) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "size_of: unknown tensor id %d", id);
  *out_nbytes = b->bytes;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_device_ptr(tfjs_cuda_ctx* ctx, int32_t id, void** out_ptr) {
  if (!ctx || !out_ptr) return TFJS_CUDA_INVALID_ARG;
  Buffer* b = ctx_buf(ctx, id);
  if (!b) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "device_ptr: unknown tensor id %d", id);
  *out_ptr = b->ptr;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_memory(tfjs_cuda_ctx* ctx, uint64_t* bytes_in_use,
                     uint64_t* bytes_reserved, uint64_t* high_water,
                     uint64_t* num_buffers) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (bytes_in_use) *bytes_in_use = ctx->in_use;
  if (high_water) *high_water = ctx->high_water;
  if (num_buffers) *num_buffers = ctx->n_live;
  if (bytes_reserved) {
    uint64_t r = 0;
    cudaSetDevice(ctx->device);
    CUDA_TRY(ctx, cudaMemPoolGetAttribute(ctx->pool,
                                          cudaMemPoolAttrReservedMemCurrent, &r));
    *bytes_reserved = r;
  }
  return TFJS_CUDA_OK;
}

int tfjs_cuda_trim(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "trimming the pool");
  cudaSetDevice(ctx->device);
  cache_flush(ctx);
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  CUDA_TRY(ctx, cudaMemPoolTrimTo(ctx->pool, 0));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_host_alloc(tfjs_cuda_ctx* ctx, uint64_t nbytes, void** out_ptr) {
  if (!ctx || !out_ptr) return TFJS_CUDA_INVALID_ARG;
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaMallocHost(out_ptr, nbytes ? nbytes : 1));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_host_free(tfjs_cuda_ctx* ctx, void* ptr) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaFreeHost(ptr));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_time_begin(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "timing");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_time_end(tfjs_cuda_ctx* ctx, float* out_kernel_ms) {
  if (!ctx || !out_kernel_ms) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "timing");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
  CUDA_TRY(ctx, cudaEventSynchronize(ctx->ev1));
  CUDA_TRY(ctx, cudaEventElapsedTime(out_kernel_ms, ctx->ev0, ctx->ev1));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_event_record(tfjs_cuda_ctx* ctx, int32_t slot) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "recording a timing event");
  if (slot < 0 || slot > (1 << 20))
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "event_record: bad slot %d", slot);
  cudaSetDevice(ctx->device);
  if ((size_t)slot >= ctx->prof_events.size()) ctx->prof_events.resize(slot + 1, nullptr);
  if (!ctx->prof_events[slot]) CUDA_TRY(ctx, cudaEventCreate(&ctx->prof_events[slot]));
  CUDA_TRY(ctx, cudaEventRecord(ctx->prof_events[slot], ctx->stream));
  return TFJS_CUDA_OK;
}

int tfjs_cuda_event_elapsed(tfjs_cuda_ctx* ctx, int32_t slot_begin, int32_t slot_end,
                            float* out_ms) {
  if (!ctx || !out_ms) return TFJS_CUDA_INVALID_ARG;
  const size_t n = ctx->prof_events.size();
  if (slot_begin < 0 || slot_end < 0 || (size_t)slot_begin >= n || (size_t)slot_end >= n ||
      !ctx->prof_events[slot_begin] || !ctx->prof_events[slot_end])
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "event_elapsed: slot was never recorded");
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaEventSynchronize(ctx->prof_events[slot_end]));
  CUDA_TRY(ctx, cudaEventElapsedTime(out_ms, ctx->prof_events[slot_begin],
                                     ctx->prof_events[slot_end]));
  return TFJS_CUDA_OK;
}

// ---- whole-step capture and replay -----------------------------------------------------
int tfjs_cuda_high_water_reset(tfjs_cuda_ctx* ctx) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  ctx->high_water = ctx->in_use;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_copy(tfjs_cuda_ctx* ctx, int32_t src_id, int32_t dst_id, uint64_t nbytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  Buffer *src, *dst;
  int rc;
  if ((rc = ctx_get(ctx, src_id, nbytes, "copy src", &src))) return rc;
  if ((rc = ctx_get(ctx, dst_id, nbytes, "copy dst", &dst))) return rc;
  if (nbytes == 0 || src->ptr == dst->ptr) return TFJS_CUDA_OK;
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaMemcpyAsync(dst->ptr, src->ptr, nbytes, cudaMemcpyDeviceToDevice, ctx->stream));
  dst->version++;
  dst->from_host = false;
  ctx_drop_packed(ctx, dst_id);
  return TFJS_CUDA_OK;
}

int tfjs_cuda_capture_begin(tfjs_cuda_ctx* ctx, uint64_t arena_bytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (ctx->capturing) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "capture_begin: already capturing");
  cudaSetDevice(ctx->device);
  arena_bytes = ((arena_bytes + 255) / 256) * 256;
  if (arena_bytes == 0) arena_bytes = 256;
  void* arena = nullptr;
  CUDA_TRY(ctx, cudaMallocAsync(&arena, arena_bytes, ctx->stream));
  // nothing of the capture may depend on work that is still in flight
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
  CUDA_TRY(ctx, cudaStreamSynchronize(ctx->copy_stream));
  cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    cudaFreeAsync(arena, ctx->stream);
    return ctx_check(ctx, e, "cudaStreamBeginCapture");
  }
  ctx->arena = arena;
  ctx->arena_bytes = arena_bytes;
  ctx->arena_free.assign(1, ArenaSpan{0, arena_bytes});
  ctx->capturing = true;
  ctx->capture_failed = false;
  ctx->capture_launches0 = ctx->launches;
  ctx->capture_packed.clear();
  ctx->capture_scratch = false;
  return TFJS_CUDA_OK;
}

// Ends the capture.  abandon != 0, a refused call during the capture or a failed
// instantiation discard it (TFJS_CUDA_UNSUPPORTED); the tensors created during the
// capture are then invalid and must only be freed.
int tfjs_cuda_capture_end(tfjs_cuda_ctx* ctx, int abandon, int32_t* out_graph) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (out_graph) *out_graph = 0;
  if (!ctx->capturing) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "capture_end: not capturing");
  cudaSetDevice(ctx->device);
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  ctx->capturing = false;
  const uint64_t launches = ctx->launches - ctx->capture_launches0;
  ctx->launches = ctx->capture_launches0;  // nothing ran yet
  cudaGraphExec_t exec = nullptr;
  const bool keep = e == cudaSuccess && graph && !abandon && !ctx->capture_failed && out_graph;
  if (keep) e = cudaGraphInstantiate(&exec, graph, 0);
  if (graph) cudaGraphDestroy(graph);
  if (!keep || e != cudaSuccess || !exec) {
    cudaGetLastError();
    cudaFreeAsync(ctx->arena, ctx->stream);
    ctx->arena = nullptr;
    ctx->arena_free.clear();
    if (e != cudaSuccess) return ctx_check(ctx, e, "ending the capture");
    std::string why = ctx->err;
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED, "capture discarded%s%s",
                    ctx->capture_failed ? ": " : "", ctx->capture_failed ? why.c_str() : "");
  }
  ReplayGraph g;
  g.exec = exec;
  g.arena = ctx->arena;
  g.arena_bytes = ctx->arena_bytes;
  g.launches = launches;
  g.packed_ids.swap(ctx->capture_packed);
  g.uses_scratch = ctx->capture_scratch;
  ctx->arena = nullptr;
  ctx->arena_free.clear();
  int slot = -1;
  for (size_t i = 0; i < ctx->graphs.size(); ++i)
    if (!ctx->graphs[i].exec) { slot = (int)i; break; }
  if (slot < 0) {
    ctx->graphs.emplace_back();
    slot = (int)ctx->graphs.size() - 1;
  }
  ctx->graphs[slot] = g;
  *out_graph = slot + 1;
  return TFJS_CUDA_OK;
}

static ReplayGraph* graph_of(tfjs_cuda_ctx* ctx, int32_t id) {
  if (id <= 0 || (size_t)id > ctx->graphs.size() || !ctx->graphs[id - 1].exec) return nullptr;
  return &ctx->graphs[id - 1];
}

int tfjs_cuda_graph_launch(tfjs_cuda_ctx* ctx, int32_t graph) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  NOT_WHILE_CAPTURING(ctx, "launching a captured step");
  ReplayGraph* g = graph_of(ctx, graph);
  if (!g) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "graph_launch: unknown graph %d", graph);
  if (g->stale)
    return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                    "graph_launch: graph %d is stale (a packed weight or the scratch buffer its "
                    "kernels address was freed or re-allocated after the capture); capture the "
                    "step again", graph);
  cudaSetDevice(ctx->device);
  CUDA_TRY(ctx, cudaGraphLaunch(g->exec, ctx->stream));
  ctx->launches += g->launches;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_graph_destroy(tfjs_cuda_ctx* ctx, int32_t graph) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  ReplayGraph* g = graph_of(ctx, graph);
  if (!g) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "graph_destroy: unknown graph %d", graph);
  cudaSetDevice(ctx->device);
  // the arena goes back to the pool behind the replays already queued
  cudaFreeAsync(g->arena, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  cudaGraphExecDestroy(g->exec);
  *g = ReplayGraph();
  return TFJS_CUDA_OK;
}

int tfjs_cuda_set_math_mode(tfjs_cuda_ctx* ctx, int mode) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  if (mode != TFJS_CUDA_MATH_TF32 && mode != TFJS_CUDA_MATH_FP32)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "unknown math mode %d", mode);
  ctx->math_mode = mode;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_launch_log(tfjs_cuda_ctx* ctx, int32_t enable) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  ctx->log_launches = enable != 0;
  ctx->launch_log.clear();
  return TFJS_CUDA_OK;
}

int tfjs_cuda_launch_log_take(tfjs_cuda_ctx* ctx, char* buf, uint64_t cap,
                              uint32_t* out_launches) {
  if (!ctx || (cap && !buf)) return TFJS_CUDA_INVALID_ARG;
  if (out_launches) *out_launches = (uint32_t)ctx->launch_log.size();
  std::string text;
  for (size_t i = 0; i < ctx->launch_log.size();) {
    size_t j = i;
    while (j < ctx->launch_log.size() && !strcmp(ctx->launch_log[j], ctx->launch_log[i])) ++j;
    if (!text.empty()) text += ", ";
    text += ctx->launch_log[i];
    if (j - i > 1) text += " x" + std::to_string(j - i);
    i = j;
  }
  ctx->launch_log.clear();
  if (cap) {
    const size_t n = text.size() < cap - 1 ? text.size() : cap - 1;
    memcpy(buf, text.data(), n);
    buf[n] = 0;
  }
  return TFJS_CUDA_OK;
}

int tfjs_cuda_launch_count(tfjs_cuda_ctx* ctx, uint64_t* out_launches) {
  if (!ctx || !out_launches) return TFJS_CUDA_INVALID_ARG;
  *out_launches = ctx->launches;
  return TFJS_CUDA_OK;
}

}  // extern "C"
