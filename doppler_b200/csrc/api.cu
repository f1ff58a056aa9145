// Context, buffer pool, recorder and CUDA-graph plumbing behind the C ABI.
//
// Mirrors the mechanics of the reference's src/gpu/device.js (device),
// src/memory/buffer-pool.js (size-bucketed pool) and
// src/gpu/command-recorder.js (batched recording with temporaries), with a
// CUDA stream in place of the WebGPU queue and stream capture in place of a
// command encoder.
#include "common.h"

#include <cstring>

dp_status dp_fail(dp_ctx *ctx, dp_status st, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return st;
}

extern "C" const char *dp_version(void) { return "doppler_b200 0.1 (sm_100a)"; }

extern "C" dp_status dp_ctx_create(int device, dp_ctx **out) {
  if (!out) return DP_ERR_INVALID;
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0 || device < 0 || device >= n) return DP_ERR_CUDA;
  if (cudaSetDevice(device) != cudaSuccess) return DP_ERR_CUDA;
  dp_ctx *ctx = new dp_ctx();
  ctx->device = device;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { delete ctx; return DP_ERR_CUDA; }
  ctx->sm_count = prop.multiProcessorCount;
  ctx->smem_optin = prop.sharedMemPerBlockOptin;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
    delete ctx;
    return DP_ERR_CUDA;
  }
  if (cudaMalloc(&ctx->dev_status, 256) != cudaSuccess || cudaMemset(ctx->dev_status, 0, 256) != cudaSuccess) {
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return DP_ERR_CUDA;
  }
  *out = ctx;
  return DP_OK;
}

extern "C" dp_status dp_tp_destroy(dp_ctx *ctx);

extern "C" void dp_ctx_destroy(dp_ctx *ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  dp_tp_destroy(ctx);
  for (dp_buf_s *b : ctx->all) {
    if (b->dptr) cudaFree(b->dptr);
    delete b;
  }
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  cudaStreamDestroy(ctx->stream);
  delete ctx;
}

extern "C" dp_status dp_ctx_set_wait_limit(dp_ctx *ctx, unsigned polls) {
  if (!ctx) return DP_ERR_INVALID;
  DP_CHECK(ctx, polls >= 16, "set_wait_limit: %u polls is too few", polls);
  ctx->wait_limit = polls;
  return DP_OK;
}

extern "C" const char *dp_last_error(dp_ctx *ctx) { return ctx ? ctx->err.c_str() : "null context"; }
extern "C" void *dp_ctx_stream(dp_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }
extern "C" int dp_ctx_device(dp_ctx *ctx) { return ctx ? ctx->device : -1; }
extern "C" uint64_t dp_ctx_launch_count(dp_ctx *ctx) { return ctx ? ctx->launches : 0; }

void dp_tp_reset_barrier(dp_ctx *ctx);

// Reads (and clears) the status word kernels raise when a bounded device-side wait gave up.  The stream
// must be idle.
dp_status dp_take_dev_status(dp_ctx *ctx) {
  int flag = 0;
  DP_CUDA(ctx, cudaMemcpy(&flag, ctx->dev_status, 4, cudaMemcpyDeviceToHost));
  if (flag) {
    cudaMemset(ctx->dev_status, 0, 4);
    dp_tp_reset_barrier(ctx);
    cudaStreamSynchronize(ctx->stream);
    return dp_fail(ctx, DP_ERR_TIMEOUT, "a kernel gave up on a bounded device-side wait (status %d); its output is invalid", flag);
  }
  return DP_OK;
}

extern "C" dp_status dp_ctx_sync(dp_ctx *ctx) {
  if (!ctx) return DP_ERR_INVALID;
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return dp_take_dev_status(ctx);
}

// ---- pool ------------------------------------------------------------------
// Bucket rule of src/memory/buffer-pool.js:73-118: 256-byte alignment, a minimum
// bucket, powers of two up to a threshold, then a linear step so that a large
// weight matrix is not doubled.
static const size_t kMinBucket = 256;
static const size_t kLargeThreshold = 64ull << 20;
static const size_t kLargeStep = 16ull << 20;

extern "C" size_t dp_pool_bucket_size(size_t bytes) {
  size_t aligned = dp_cdiv(bytes ? bytes : 1, DP_BUFFER_ALIGN) * DP_BUFFER_ALIGN;
  if (aligned <= kMinBucket) return kMinBucket;
  if (aligned >= kLargeThreshold) return dp_cdiv(aligned, kLargeStep) * kLargeStep;
  size_t b = kMinBucket;
  while (b < aligned) b <<= 1;
  return b;
}

extern "C" dp_status dp_buf_acquire(dp_ctx *ctx, size_t bytes, const char *label, dp_buf *out) {
  if (!ctx || !out) return DP_ERR_INVALID;
  *out = nullptr;
  size_t bucket = dp_pool_bucket_size(bytes);
  auto it = ctx->idle.find(bucket);
  dp_buf_s *b = nullptr;
  if (it != ctx->idle.end()) {
    b = it->second;
    ctx->idle.erase(it);
    ctx->stats.reuses++;
    ctx->stats.bytes_pooled -= bucket;
  } else {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bucket);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return dp_fail(ctx, DP_ERR_OOM, "buffer pool: cudaMalloc(%zu) for '%s' failed: %s", bucket,
                     label ? label : "", cudaGetErrorString(e));
    }
    b = new dp_buf_s();
    b->dptr = p;
    b->capacity = bucket;
    b->ctx = ctx;
    ctx->all.push_back(b);
    ctx->stats.allocations++;
    ctx->stats.bytes_allocated += bucket;
    if (ctx->stats.bytes_allocated > ctx->stats.peak_bytes_allocated)
      ctx->stats.peak_bytes_allocated = ctx->stats.bytes_allocated;
  }
  b->bytes = bytes;
  b->active = true;
  b->label = label ? label : "pooled_buffer";
  ctx->stats.bytes_in_use += bucket;
  *out = b;
  return DP_OK;
}

extern "C" dp_status dp_buf_release(dp_ctx *ctx, dp_buf buf) {
  if (!ctx || !buf) return DP_ERR_INVALID;
  if (buf->ctx != ctx) return dp_fail(ctx, DP_ERR_STATE, "releaseBuffer: buffer belongs to another context");
  if (!buf->active) return dp_fail(ctx, DP_ERR_STATE, "releaseBuffer: buffer '%s' is not active", buf->label.c_str());
  buf->active = false;
  ctx->idle.emplace(buf->capacity, buf);
  ctx->stats.releases++;
  ctx->stats.bytes_in_use -= buf->capacity;
  ctx->stats.bytes_pooled += buf->capacity;
  return DP_OK;
}

static dp_status check_range(dp_ctx *ctx, dp_buf buf, size_t offset, size_t bytes, const char *what) {
  if (!ctx || !buf) return DP_ERR_INVALID;
  if (!buf->active) return dp_fail(ctx, DP_ERR_STATE, "%s: buffer '%s' was released", what, buf->label.c_str());
  if (offset > buf->bytes || bytes > buf->bytes - offset)
    return dp_fail(ctx, DP_ERR_INVALID, "%s: range [%zu, %zu) exceeds buffer '%s' of %zu bytes", what, offset,
                   offset + bytes, buf->label.c_str(), buf->bytes);
  return DP_OK;
}

extern "C" dp_status dp_buf_upload(dp_ctx *ctx, dp_buf buf, const void *host, size_t offset, size_t bytes) {
  DP_TRY(check_range(ctx, buf, offset, bytes, "uploadData"));
  if (!host && bytes) return dp_fail(ctx, DP_ERR_INVALID, "uploadData: null host pointer");
  DP_CUDA(ctx, cudaMemcpyAsync((char *)buf->dptr + offset, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  // pageable sources are staged before the call returns; pinned ones need the sync
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return DP_OK;
}

extern "C" dp_status dp_buf_read(dp_ctx *ctx, dp_buf buf, void *host, size_t offset, size_t bytes) {
  DP_TRY(check_range(ctx, buf, offset, bytes, "readBuffer"));
  if (!host && bytes) return dp_fail(ctx, DP_ERR_INVALID, "readBuffer: null host pointer");
  DP_CUDA(ctx, cudaMemcpyAsync(host, (char *)buf->dptr + offset, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return DP_OK;
}

extern "C" dp_status dp_buf_fill(dp_ctx *ctx, dp_buf buf, int byte_value, size_t offset, size_t bytes) {
  DP_TRY(check_range(ctx, buf, offset, bytes, "fill"));
  DP_CUDA(ctx, cudaMemsetAsync((char *)buf->dptr + offset, byte_value, bytes, ctx->stream));
  return DP_OK;
}

extern "C" void *dp_buf_device_ptr(dp_buf buf) { return buf ? buf->dptr : nullptr; }
extern "C" size_t dp_buf_size(dp_buf buf) { return buf ? buf->bytes : 0; }
extern "C" size_t dp_buf_capacity(dp_buf buf) { return buf ? buf->capacity : 0; }

extern "C" dp_status dp_pool_get_stats(dp_ctx *ctx, dp_pool_stats *out) {
  if (!ctx || !out) return DP_ERR_INVALID;
  *out = ctx->stats;
  return DP_OK;
}

extern "C" dp_status dp_pool_trim(dp_ctx *ctx) {
  if (!ctx) return DP_ERR_INVALID;
  DP_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto &kv : ctx->idle) {
    dp_buf_s *b = kv.second;
    cudaFree(b->dptr);
    b->dptr = nullptr;
    ctx->stats.bytes_allocated -= b->capacity;
    ctx->stats.bytes_pooled -= b->capacity;
    for (size_t i = 0; i < ctx->all.size(); i++)
      if (ctx->all[i] == b) { ctx->all.erase(ctx->all.begin() + (long)i); break; }
    delete b;
  }
  ctx->idle.clear();
  return DP_OK;
}

dp_status dp_out_buffer(dp_ctx *ctx, dp_buf out_buf, size_t offset, size_t bytes, const char *label,
                        dp_buf *result) {
  if (out_buf) {
    if (!out_buf->active) return dp_fail(ctx, DP_ERR_STATE, "%s: outputBuffer was released", label);
    if (offset % DP_BUFFER_ALIGN) return dp_fail(ctx, DP_ERR_INVALID, "%s: output offset %zu is not 256-byte aligned", label, offset);
    if (offset > out_buf->bytes || bytes > out_buf->bytes - offset)
      return dp_fail(ctx, DP_ERR_INVALID, "%s: outputBuffer too small: need %zu bytes at offset %zu, have %zu", label,
                     bytes, offset, out_buf->bytes);
    *result = out_buf;
    return DP_OK;
  }
  if (offset) return dp_fail(ctx, DP_ERR_INVALID, "%s: an output offset needs an outputBuffer", label);
  return dp_buf_acquire(ctx, bytes, label, result);
}

dp_status dp_scratch(dp_ctx *ctx, dp_buf *slot, size_t bytes, const char *label) {
  if (*slot && (*slot)->capacity >= bytes) return DP_OK;
  if (*slot) {
    const bool capturing = ctx->active_recorder && ctx->active_recorder->capture;
    if (capturing || ctx->live_graphs > 0) ctx->retired_scratch.push_back(*slot);  // a graph may still point at it
    else DP_TRY(dp_buf_release(ctx, *slot));
    *slot = nullptr;
  }
  return dp_buf_acquire(ctx, bytes, label, slot);
}

// ---- recorder --------------------------------------------------------------
dp_status dp_check_rec(dp_ctx *ctx, dp_recorder *rec) {
  if (!ctx) return DP_ERR_INVALID;
  if (rec) {
    if (rec->ctx != ctx) return dp_fail(ctx, DP_ERR_STATE, "recorder belongs to another context");
    if (!rec->open) return dp_fail(ctx, DP_ERR_STATE, "recorder '%s' was already submitted", rec->label.c_str());
  }
  return DP_OK;
}

void dp_note_op(dp_ctx *, dp_recorder *rec) {
  if (rec) rec->ops++;
}

extern "C" dp_status dp_recorder_begin(dp_ctx *ctx, const char *label, int capture_graph, dp_recorder **out) {
  if (!ctx || !out) return DP_ERR_INVALID;
  if (ctx->active_recorder) return dp_fail(ctx, DP_ERR_STATE, "a recorder ('%s') is already open", ctx->active_recorder->label.c_str());
  dp_recorder *r = new dp_recorder();
  r->ctx = ctx;
  r->label = label ? label : "recorder";
  r->capture = capture_graph != 0;
  r->open = true;
  r->launches_at_begin = ctx->launches;
  if (r->capture) {
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) {
      delete r;
      return dp_fail(ctx, DP_ERR_CUDA, "cudaStreamBeginCapture failed: %s", cudaGetErrorString(e));
    }
  }
  ctx->active_recorder = r;
  *out = r;
  return DP_OK;
}

extern "C" dp_status dp_recorder_track_temporary(dp_recorder *rec, dp_buf buf) {
  if (!rec || !buf) return DP_ERR_INVALID;
  if (!rec->open) return dp_fail(rec->ctx, DP_ERR_STATE, "recorder '%s' is closed", rec->label.c_str());
  rec->temporaries.push_back(buf);
  return DP_OK;
}

extern "C" uint32_t dp_recorder_op_count(dp_recorder *rec) { return rec ? rec->ops : 0; }

static dp_status release_temporaries(dp_recorder *rec) {
  dp_status st = DP_OK;
  // all work is ordered on one stream, so a released buffer can only be reused
  // by work enqueued after the recording's kernels
  for (dp_buf b : rec->temporaries) {
    dp_status s = dp_buf_release(rec->ctx, b);
    if (s != DP_OK) st = s;
  }
  rec->temporaries.clear();
  return st;
}

static dp_status end_capture(dp_recorder *rec, dp_graph **out) {
  dp_ctx *ctx = rec->ctx;
  cudaGraph_t g = nullptr;
  DP_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
  dp_graph *gr = new dp_graph();
  gr->ctx = ctx;
  gr->graph = g;
  gr->kernels = ctx->launches - rec->launches_at_begin;
  cudaError_t e = cudaGraphInstantiate(&gr->exec, g, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(g);
    delete gr;
    return dp_fail(ctx, DP_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  // kernels recorded during capture did not run yet; they are counted per launch
  ctx->launches = rec->launches_at_begin;
  // the graph's kernels keep pointing at the recording's temporaries: they live as long as the graph
  gr->owned.swap(rec->temporaries);
  ctx->live_graphs++;
  *out = gr;
  return DP_OK;
}

static dp_status finish(dp_recorder *rec, bool wait, bool launch, dp_graph **graph_out) {
  if (!rec) return DP_ERR_INVALID;
  dp_ctx *ctx = rec->ctx;
  if (!rec->open) return dp_fail(ctx, DP_ERR_STATE, "recorder '%s' was already submitted", rec->label.c_str());
  rec->open = false;
  ctx->active_recorder = nullptr;
  dp_status st = DP_OK;
  if (rec->capture) {
    dp_graph *g = nullptr;
    st = end_capture(rec, &g);
    if (st == DP_OK && launch) st = dp_graph_launch(g);
    if (graph_out && st == DP_OK) *graph_out = g;
    else if (g) {
      if (wait || true) cudaStreamSynchronize(ctx->stream);
      dp_graph_destroy(g);
    }
  }
  dp_status st2 = release_temporaries(rec);
  if (st == DP_OK) st = st2;
  if (st == DP_OK && wait) {
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) st = dp_fail(ctx, DP_ERR_CUDA, "submitAndWait: %s", cudaGetErrorString(e));
  }
  delete rec;
  return st;
}

extern "C" dp_status dp_recorder_submit(dp_recorder *rec) { return finish(rec, false, true, nullptr); }
extern "C" dp_status dp_recorder_submit_and_wait(dp_recorder *rec) { return finish(rec, true, true, nullptr); }

extern "C" dp_status dp_recorder_finish_graph(dp_recorder *rec, dp_graph **out) {
  if (!rec || !out) return DP_ERR_INVALID;
  if (!rec->capture) return dp_fail(rec->ctx, DP_ERR_STATE, "recorder '%s' is not capturing a graph", rec->label.c_str());
  return finish(rec, false, false, out);
}

extern "C" dp_status dp_recorder_abort(dp_recorder *rec) {
  if (!rec) return DP_ERR_INVALID;
  dp_ctx *ctx = rec->ctx;
  if (rec->open && rec->capture) {
    cudaGraph_t g = nullptr;
    cudaStreamEndCapture(ctx->stream, &g);
    if (g) cudaGraphDestroy(g);
    cudaGetLastError();
    ctx->launches = rec->launches_at_begin;
  }
  rec->open = false;
  ctx->active_recorder = nullptr;
  cudaStreamSynchronize(ctx->stream);
  dp_status st = release_temporaries(rec);
  delete rec;
  return st;
}

extern "C" dp_status dp_graph_launch(dp_graph *g) {
  if (!g) return DP_ERR_INVALID;
  DP_CUDA(g->ctx, cudaGraphLaunch(g->exec, g->ctx->stream));
  g->ctx->launches += g->kernels;
  return DP_OK;
}

// `reps` replays between two CUDA events on the context's stream; *ms receives the device time of all of them
extern "C" dp_status dp_graph_launch_timed(dp_graph *g, int reps, double *ms) {
  if (!g || !ms || reps < 1) return DP_ERR_INVALID;
  dp_ctx *ctx = g->ctx;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  DP_CUDA(ctx, cudaEventCreate(&e0));
  cudaError_t e = cudaEventCreate(&e1);
  if (e == cudaSuccess) e = cudaEventRecord(e0, ctx->stream);
  for (int i = 0; i < reps && e == cudaSuccess; i++) {
    e = cudaGraphLaunch(g->exec, ctx->stream);
    ctx->launches += g->kernels;
  }
  if (e == cudaSuccess) e = cudaEventRecord(e1, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
  float t = 0.0f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
  cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (e != cudaSuccess) return dp_fail(ctx, DP_ERR_CUDA, "timed graph launch: %s", cudaGetErrorString(e));
  *ms = t;
  return DP_OK;
}

extern "C" void dp_graph_destroy(dp_graph *g) {
  if (!g) return;
  dp_ctx *ctx = g->ctx;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  // launches of the graph are ordered on the context's stream, so are later users of these buffers
  for (dp_buf b : g->owned) dp_buf_release(ctx, b);
  if (ctx && --ctx->live_graphs <= 0) {
    ctx->live_graphs = 0;
    for (dp_buf b : ctx->retired_scratch) dp_buf_release(ctx, b);
    ctx->retired_scratch.clear();
  }
  delete g;
}
