// Weight loader: the bytes of a model's weight shards go from the host (memory chunks or
// shard files) to decoded device tensors without a detour through the host language.
//
// It replaces, behind the C ABI, the loop of decodeWeights / decodeWeight
// (tfjs-core/src/io/io_utils.ts:119-135, :185-292), the chunk-by-chunk decodeWeightsStream
// (:316-353) and the shard fetching of weights_loader.ts:38-131: the caller describes the
// manifest entries in order (tfjs-core/src/io/types.ts:76-110) and pushes the concatenated
// bytes in pieces of any size, cut anywhere (a shard boundary may fall inside a tensor).
//
// Data path: bytes are staged through a small ring of pinned host slots; each piece leaves
// with its own cudaMemcpyAsync on the context's copy stream while the host fills the next
// slot (from the caller's chunk, or straight from a shard file with pread).  A tensor's
// stored bytes land in a device buffer allocated on the copy stream.  When its last byte
// has been queued, a tensor stored in its own dtype becomes a tensor at once (its first
// consumer waits for the copy's event, as after tfjs_cuda_upload); a quantised (uint8 /
// uint16 affine) or float16-stored tensor gets its decode kernel queued on the compute
// stream behind that event, so the copy of tensor k+1 overlaps the decode of tensor k, and
// the stored bytes are freed in stream order.
#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <unistd.h>

#include "common.cuh"

namespace {

constexpr int kSlots = 4;
constexpr uint64_t kSlotBytes = 8ull << 20;

struct WeightLoader {
  bool live = false;
  std::vector<tfjs_cuda_weight_spec> specs;
  std::vector<int32_t> ids;
  size_t cur = 0;            // entry being filled
  uint64_t cur_off = 0;      // of its stored bytes, how many are queued
  void* cur_dst = nullptr;   // device buffer of the current entry's stored bytes
  uint64_t cur_padded = 0;
  uint64_t expected = 0, pushed = 0;
  void* slot[kSlots] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t slot_ev[kSlots] = {nullptr, nullptr, nullptr, nullptr};
  bool slot_busy[kSlots] = {false, false, false, false};
  int s = 0;                 // slot being filled
  uint64_t fill = 0;         // bytes of it in use
  bool slot_open = false;    // pieces were queued from slot s since its last event
};

std::vector<WeightLoader>& loaders_of(tfjs_cuda_ctx* ctx) {
  // one table per context, created on first use and kept until the process ends (a context
  // has at most a handful of loaders in its life)
  static std::unordered_map<tfjs_cuda_ctx*, std::vector<WeightLoader>> all;
  return all[ctx];
}

uint64_t stored_bytes(const tfjs_cuda_weight_spec& sp) {
  switch (sp.storage) {
    case TFJS_CUDA_STORED_UINT8: return sp.n;
    case TFJS_CUDA_STORED_UINT16:
    case TFJS_CUDA_STORED_FLOAT16: return sp.n * 2;
    default: return sp.n * (sp.dtype == TFJS_CUDA_BOOL ? 1 : 4);
  }
}

uint64_t pad256(uint64_t n) {
  uint64_t p = ((n + 255) / 256) * 256;
  return p ? p : 256;
}

int32_t register_buffer(tfjs_cuda_ctx* ctx, void* p, uint64_t nbytes, cudaEvent_t ready) {
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
  b.from_host = true;   // weights: constants, packed once on first use
  b.in_arena = false;
  b.uploaded = false;
  b.version++;
  b.ready = ready;
  ctx->in_use += pad256(nbytes);
  ctx->n_live++;
  if (ctx->in_use > ctx->high_water) ctx->high_water = ctx->in_use;
  return id;
}

int take_event(tfjs_cuda_ctx* ctx, cudaEvent_t* ev) {
  if (!ctx->event_pool.empty()) {
    *ev = ctx->event_pool.back();
    ctx->event_pool.pop_back();
    return TFJS_CUDA_OK;
  }
  CUDA_TRY(ctx, cudaEventCreateWithFlags(ev, cudaEventDisableTiming));
  return TFJS_CUDA_OK;
}

// Closes the slot being filled: an event behind its last piece says when it may be refilled.
int close_slot(tfjs_cuda_ctx* ctx, WeightLoader& w) {
  if (w.slot_open) {
    CUDA_TRY(ctx, cudaEventRecord(w.slot_ev[w.s], ctx->copy_stream));
    w.slot_busy[w.s] = true;
    w.slot_open = false;
  }
  w.s = (w.s + 1) % kSlots;
  w.fill = 0;
  if (w.slot_busy[w.s]) {
    CUDA_TRY(ctx, cudaEventSynchronize(w.slot_ev[w.s]));
    w.slot_busy[w.s] = false;
  }
  return TFJS_CUDA_OK;
}

// The current entry's stored bytes are all queued: turn them into a tensor.
int finish_entry(tfjs_cuda_ctx* ctx, WeightLoader& w) {
  const tfjs_cuda_weight_spec& sp = w.specs[w.cur];
  int rc;
  if (sp.skip) {
    w.ids[w.cur] = 0;
  } else if (sp.storage == TFJS_CUDA_STORED_RAW) {
    cudaEvent_t ev;
    if ((rc = take_event(ctx, &ev))) return rc;
    CUDA_TRY(ctx, cudaEventRecord(ev, ctx->copy_stream));
    w.ids[w.cur] = register_buffer(ctx, w.cur_dst, stored_bytes(sp), ev);
    w.cur_dst = nullptr;
  } else {
    // decode on the compute stream, behind the copy
    cudaEvent_t ev;
    if ((rc = take_event(ctx, &ev))) return rc;
    CUDA_TRY(ctx, cudaEventRecord(ev, ctx->copy_stream));
    CUDA_TRY(ctx, cudaStreamWaitEvent(ctx->stream, ev, 0));
    ctx->event_pool.push_back(ev);
    int32_t out_id = 0;
    if ((rc = tfjs_cuda_alloc(ctx, sp.n * 4, &out_id))) return rc;
    void* out = ctx->bufs[out_id].ptr;
    if (sp.n) {
      if (sp.storage == TFJS_CUDA_STORED_FLOAT16)
        rc = decode_f16_enqueue(ctx, w.cur_dst, sp.n, out);
      else
        rc = dequant_enqueue(ctx, w.cur_dst, sp.storage == TFJS_CUDA_STORED_UINT8 ? 1 : 2, sp.dtype,
                             sp.scale, sp.min, sp.n, out);
      if (rc) {
        tfjs_cuda_free(ctx, out_id);
        return rc;
      }
    }
    ctx->bufs[out_id].from_host = true;
    // the stored bytes were allocated on the copy stream; the compute stream is ordered
    // behind their last use there, so it may release them
    CUDA_TRY(ctx, cudaFreeAsync(w.cur_dst, ctx->stream));
    w.cur_dst = nullptr;
    w.ids[w.cur] = out_id;
  }
  w.cur++;
  w.cur_off = 0;
  return TFJS_CUDA_OK;
}

// Opens entries until one needs bytes; entries without bytes are finished on the spot.
int open_entries(tfjs_cuda_ctx* ctx, WeightLoader& w) {
  while (w.cur < w.specs.size() && w.cur_off == 0 && w.cur_dst == nullptr) {
    const tfjs_cuda_weight_spec& sp = w.specs[w.cur];
    const uint64_t nb = stored_bytes(sp);
    if (!sp.skip) {
      w.cur_padded = pad256(nb);
      CUDA_TRY(ctx, cudaMallocAsync(&w.cur_dst, w.cur_padded, ctx->copy_stream));
    }
    if (nb != 0) return TFJS_CUDA_OK;
    int rc = finish_entry(ctx, w);
    if (rc) return rc;
  }
  return TFJS_CUDA_OK;
}

// A source of bytes: copies the next `len` bytes to dst (pinned), or passes over them.
struct Source {
  const uint8_t* mem = nullptr;  // memory chunk ...
  int fd = -1;                   // ... or a file read with pread
  uint64_t pos = 0;
  int read(void* dst, uint64_t len) {
    if (fd < 0) {
      memcpy(dst, mem + pos, len);
      pos += len;
      return 0;
    }
    uint64_t done = 0;
    while (done < len) {
      const ssize_t r = pread(fd, (char*)dst + done, len - done, (off_t)(pos + done));
      if (r < 0 && errno == EINTR) continue;
      if (r <= 0) return -1;
      done += (uint64_t)r;
    }
    pos += len;
    return 0;
  }
};

int feed(tfjs_cuda_ctx* ctx, WeightLoader& w, Source& src, uint64_t nbytes) {
  int rc;
  while (nbytes > 0) {
    if ((rc = open_entries(ctx, w))) return rc;
    if (w.cur >= w.specs.size())
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                      "weights: %llu bytes beyond what the manifest entries hold",
                      (unsigned long long)nbytes);
    const tfjs_cuda_weight_spec& sp = w.specs[w.cur];
    const uint64_t left = stored_bytes(sp) - w.cur_off;
    uint64_t take = nbytes < left ? nbytes : left;
    nbytes -= take;
    w.pushed += take;
    if (sp.skip) {
      src.pos += take;
      w.cur_off += take;
    }
    while (take > 0 && !sp.skip) {
      if (kSlotBytes - w.fill < 16 || (kSlotBytes - w.fill < take && w.fill > kSlotBytes / 2))
        if ((rc = close_slot(ctx, w))) return rc;
      const uint64_t room = kSlotBytes - w.fill;
      const uint64_t piece = take < room ? take : room;
      char* stage = (char*)w.slot[w.s] + w.fill;
      if (src.read(stage, piece) != 0)
        return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights: reading the shard failed: %s",
                        strerror(errno));
      CUDA_TRY(ctx, cudaMemcpyAsync((char*)w.cur_dst + w.cur_off, stage, piece,
                                    cudaMemcpyHostToDevice, ctx->copy_stream));
      w.slot_open = true;
      w.fill += (piece + 15) & ~15ull;
      w.cur_off += piece;
      take -= piece;
    }
    if (w.cur_off == stored_bytes(sp))
      if ((rc = finish_entry(ctx, w))) return rc;
  }
  return TFJS_CUDA_OK;
}

void release_all(tfjs_cuda_ctx* ctx, WeightLoader& w, bool free_tensors) {
  cudaStreamSynchronize(ctx->copy_stream);
  if (w.cur_dst) cudaFreeAsync(w.cur_dst, ctx->copy_stream);
  if (free_tensors)
    for (int32_t id : w.ids)
      if (id > 0) tfjs_cuda_free(ctx, id);
  for (int i = 0; i < kSlots; ++i) {
    if (w.slot[i]) cudaFreeHost(w.slot[i]);
    if (w.slot_ev[i]) cudaEventDestroy(w.slot_ev[i]);
  }
  w = WeightLoader();
}

WeightLoader* loader_of(tfjs_cuda_ctx* ctx, int32_t id) {
  std::vector<WeightLoader>& v = loaders_of(ctx);
  if (id <= 0 || (size_t)id > v.size() || !v[id - 1].live) return nullptr;
  return &v[id - 1];
}

}  // namespace

void loaders_drop(tfjs_cuda_ctx* ctx) {
  std::vector<WeightLoader>& v = loaders_of(ctx);
  for (WeightLoader& w : v)
    if (w.live) release_all(ctx, w, true);
  v.clear();
}

extern "C" {

int tfjs_cuda_weights_begin(tfjs_cuda_ctx* ctx, const tfjs_cuda_weight_spec* specs,
                            int32_t n_specs, int32_t* out_loader) {
  if (!ctx || !out_loader) return TFJS_CUDA_INVALID_ARG;
  *out_loader = 0;
  NOT_WHILE_CAPTURING(ctx, "loading weights");
  if (n_specs < 0 || (n_specs > 0 && !specs))
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_begin: bad entry list");
  WeightLoader w;
  for (int32_t i = 0; i < n_specs; ++i) {
    const tfjs_cuda_weight_spec& sp = specs[i];
    const bool quant = sp.storage == TFJS_CUDA_STORED_UINT8 || sp.storage == TFJS_CUDA_STORED_UINT16;
    if (sp.storage < TFJS_CUDA_STORED_RAW || sp.storage > TFJS_CUDA_STORED_FLOAT16 ||
        sp.dtype < TFJS_CUDA_FLOAT32 || sp.dtype > TFJS_CUDA_BOOL)
      return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_begin: entry %d: storage %d, dtype %d",
                      i, sp.storage, sp.dtype);
    // io_utils.ts:203-218: affine quantisation decodes to float32 or int32, float16 to float32
    if (quant && sp.dtype == TFJS_CUDA_BOOL)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                      "weights_begin: entry %d: quantised storage decodes to float32 or int32", i);
    if (sp.storage == TFJS_CUDA_STORED_FLOAT16 && sp.dtype != TFJS_CUDA_FLOAT32)
      return ctx_fail(ctx, TFJS_CUDA_UNSUPPORTED,
                      "weights_begin: entry %d: float16 storage decodes to float32 only", i);
    w.expected += stored_bytes(sp);
  }
  cudaSetDevice(ctx->device);
  w.specs.assign(specs, specs + n_specs);
  w.ids.assign(n_specs, 0);
  for (int i = 0; i < kSlots; ++i) {
    if (cudaMallocHost(&w.slot[i], kSlotBytes) != cudaSuccess ||
        cudaEventCreateWithFlags(&w.slot_ev[i], cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      release_all(ctx, w, false);
      return ctx_fail(ctx, TFJS_CUDA_OUT_OF_MEMORY, "weights_begin: pinned staging ring");
    }
  }
  w.live = true;
  std::vector<WeightLoader>& v = loaders_of(ctx);
  size_t slot = v.size();
  for (size_t i = 0; i < v.size(); ++i)
    if (!v[i].live) { slot = i; break; }
  if (slot == v.size()) v.emplace_back();
  v[slot] = w;
  *out_loader = (int32_t)slot + 1;
  return TFJS_CUDA_OK;
}

int tfjs_cuda_weights_push(tfjs_cuda_ctx* ctx, int32_t loader, const void* bytes,
                           uint64_t nbytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  WeightLoader* w = loader_of(ctx, loader);
  if (!w) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "weights_push: unknown loader %d", loader);
  NOT_WHILE_CAPTURING(ctx, "loading weights");
  if (nbytes && !bytes) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_push: null chunk");
  cudaSetDevice(ctx->device);
  Source src;
  src.mem = (const uint8_t*)bytes;
  return feed(ctx, *w, src, nbytes);
}

int tfjs_cuda_weights_push_file(tfjs_cuda_ctx* ctx, int32_t loader, const char* path) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  WeightLoader* w = loader_of(ctx, loader);
  if (!w) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "weights_push_file: unknown loader %d", loader);
  NOT_WHILE_CAPTURING(ctx, "loading weights");
  if (!path) return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_push_file: null path");
  const int fd = open(path, O_RDONLY);
  if (fd < 0)
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_push_file: %s: %s", path, strerror(errno));
  const off_t size = lseek(fd, 0, SEEK_END);
  if (size < 0) {
    close(fd);
    return ctx_fail(ctx, TFJS_CUDA_INVALID_ARG, "weights_push_file: %s: %s", path, strerror(errno));
  }
  cudaSetDevice(ctx->device);
  Source src;
  src.fd = fd;
  const int rc = feed(ctx, *w, src, (uint64_t)size);
  close(fd);
  return rc;
}

int tfjs_cuda_weights_end(tfjs_cuda_ctx* ctx, int32_t loader, int32_t* out_ids,
                          uint64_t* out_bytes) {
  if (!ctx) return TFJS_CUDA_INVALID_ARG;
  WeightLoader* w = loader_of(ctx, loader);
  if (!w) return ctx_fail(ctx, TFJS_CUDA_UNKNOWN_ID, "weights_end: unknown loader %d", loader);
  cudaSetDevice(ctx->device);
  int rc = out_ids ? open_entries(ctx, *w) : TFJS_CUDA_OK;   // trailing entries without bytes
  if (rc == TFJS_CUDA_OK && out_ids && (w->cur != w->specs.size() || w->pushed != w->expected))
    rc = ctx_fail(ctx, TFJS_CUDA_INVALID_ARG,
                  "weights_end: the manifest entries hold %llu bytes, %llu were pushed",
                  (unsigned long long)w->expected, (unsigned long long)w->pushed);
  if (out_bytes) *out_bytes = w->pushed;
  if (rc != TFJS_CUDA_OK || !out_ids) {
    // out_ids == NULL abandons the load
    release_all(ctx, *w, true);
    return rc;
  }
  for (size_t i = 0; i < w->ids.size(); ++i) out_ids[i] = w->ids[i];
  release_all(ctx, *w, false);   // waits for the copy stream: the ring is about to go
  return TFJS_CUDA_OK;
}

}  // extern "C"
