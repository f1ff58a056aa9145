// Tensor-parallel group: NCCL (loaded at run time) for allreduce / allgather on
// the context's stream.  One process per GPU; the 128-byte NCCL unique id is
// created on rank 0 and handed to every rank by the host program.
//
// The reference has no collective backend (src/config/schema/emulation.schema.js
// :108-143 only names TP degrees for an external simulator); this is the
// data-path exchange of the column/row-parallel split: one sum over ranks after
// o_proj and one after down_proj.
#include "common.h"
#include "tp_exchange.h"

#include <dlfcn.h>

#include <cstring>

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclInt8 = 0, ncclChar = 0, ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId *) = nullptr;
  int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
};

static NcclApi g_nccl;

static bool load_nccl(std::string *why) {
  if (g_nccl.handle) return true;
  const char *names[] = {"libnccl.so.2", "libnccl.so"};
  void *h = nullptr;
  for (const char *n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) { *why = std::string("cannot load libnccl: ") + dlerror(); return false; }
  NcclApi a;
  a.handle = h;
#define SYM(field, name) *(void **)(&a.field) = dlsym(h, name); if (!a.field) { *why = std::string("libnccl lacks ") + name; return false; }
  SYM(GetUniqueId, "ncclGetUniqueId");
  SYM(CommInitRank, "ncclCommInitRank");
  SYM(CommDestroy, "ncclCommDestroy");
  SYM(CommAbort, "ncclCommAbort");
  SYM(AllReduce, "ncclAllReduce");
  SYM(AllGather, "ncclAllGather");
  SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
  g_nccl = a;
  return true;
}

struct dp_tp_state {
  int rank = 0, size = 1;
  ncclComm_t comm = nullptr;
  // peer-memory exchange area (one per rank, mapped into every rank with CUDA IPC)
  void *xbuf = nullptr;             // this rank's area
  void *peer[DP_TP_MAX_RANKS] = {}; // every rank's area as seen from this process (peer[rank] == xbuf)
  bool attached = false;
  bool loopback = false;               // dp_tp_init_loopback: no communicator, every area is local memory
  dp_tp_exchange *dev_desc = nullptr;  // device copy of the descriptor handed to kernels
};

bool dp_tp_ready(dp_ctx *ctx) { return ctx && ctx->tp && (ctx->tp->comm || ctx->tp->loopback); }

extern "C" dp_status dp_tp_unique_id(void *out128) {
  if (!out128) return DP_ERR_INVALID;
  std::string why;
  if (!load_nccl(&why)) return DP_ERR_COMM;
  ncclUniqueId id;
  if (g_nccl.GetUniqueId(&id) != ncclSuccess) return DP_ERR_COMM;
  memcpy(out128, &id, 128);
  return DP_OK;
}

extern "C" dp_status dp_tp_init(dp_ctx *ctx, int rank, int size, const void *id128) {
  if (!ctx || !id128) return DP_ERR_INVALID;
  DP_CHECK(ctx, size >= 1 && rank >= 0 && rank < size, "tp_init: rank %d outside [0,%d)", rank, size);
  DP_CHECK(ctx, size <= DP_TP_MAX_RANKS, "tp_init: %d ranks requested, groups hold up to %d (one NVSwitch domain)", size, DP_TP_MAX_RANKS);
  if (ctx->tp) return dp_fail(ctx, DP_ERR_STATE, "tp_init: the context already has a group");
  std::string why;
  if (!load_nccl(&why)) return dp_fail(ctx, DP_ERR_COMM, "tp_init: %s", why.c_str());
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  DP_CUDA(ctx, cudaSetDevice(ctx->device));
  dp_tp_state *tp = new dp_tp_state();
  tp->rank = rank; tp->size = size;
  int rc = g_nccl.CommInitRank(&tp->comm, size, id, rank);
  if (rc != ncclSuccess) {
    delete tp;
    return dp_fail(ctx, DP_ERR_COMM, "tp_init: ncclCommInitRank failed: %s", g_nccl.GetErrorString(rc));
  }
  ctx->tp = tp;
  return DP_OK;
}

// A group without a communicator whose `size` exchange areas all live on THIS GPU and are written by
// nobody else.  It exists so that the bounded waits of the decode kernels can be exercised on one
// GPU: rank `rank` pushes into every area and then waits for flags that the absent ranks never raise,
// gives up after the context's poll limit and reports DP_ERR_TIMEOUT.  Collectives that need a
// communicator (prefill under tensor parallelism) return DP_ERR_STATE on such a group.
extern "C" dp_status dp_tp_init_loopback(dp_ctx *ctx, int rank, int size) {
  if (!ctx) return DP_ERR_INVALID;
  DP_CHECK(ctx, size >= 1 && size <= DP_TP_MAX_RANKS && rank >= 0 && rank < size, "tp_init_loopback: rank %d / size %d", rank, size);
  if (ctx->tp) return dp_fail(ctx, DP_ERR_STATE, "tp_init_loopback: the context already has a group");
  DP_CUDA(ctx, cudaSetDevice(ctx->device));
  dp_tp_state *tp = new dp_tp_state();
  tp->rank = rank; tp->size = size; tp->loopback = true;
  dp_tp_exchange d;
  memset(&d, 0, sizeof d);
  d.rank = rank; d.size = size;
  cudaError_t e = cudaSuccess;
  for (int r = 0; r < size && e == cudaSuccess; r++) {
    e = cudaMalloc(&tp->peer[r], dp_tp_area_bytes());
    if (e == cudaSuccess) e = cudaMemset(tp->peer[r], 0, dp_tp_area_bytes());
    d.area[r] = (uint2 *)tp->peer[r];
  }
  if (e == cudaSuccess) e = cudaMalloc(&tp->dev_desc, sizeof d + 64);
  if (e == cudaSuccess) e = cudaMemcpy(tp->dev_desc, &d, sizeof d, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    for (int r = 0; r < size; r++) if (tp->peer[r]) cudaFree(tp->peer[r]);
    if (tp->dev_desc) cudaFree(tp->dev_desc);
    delete tp;
    return dp_fail(ctx, DP_ERR_CUDA, "tp_init_loopback: %s", cudaGetErrorString(e));
  }
  tp->xbuf = tp->peer[rank];
  tp->attached = true;
  ctx->tp = tp;
  return DP_OK;
}

extern "C" dp_status dp_tp_destroy(dp_ctx *ctx) {
  if (!ctx || !ctx->tp) return DP_OK;
  if (ctx->tp->comm) g_nccl.CommDestroy(ctx->tp->comm);
  if (ctx->tp->loopback) {
    for (int r = 0; r < ctx->tp->size; r++) if (r != ctx->tp->rank && ctx->tp->peer[r]) cudaFree(ctx->tp->peer[r]);
  } else
  for (int r = 0; r < ctx->tp->size; r++)
    if (ctx->tp->attached && r != ctx->tp->rank && ctx->tp->peer[r]) cudaIpcCloseMemHandle(ctx->tp->peer[r]);
  if (ctx->tp->dev_desc) cudaFree(ctx->tp->dev_desc);
  if (ctx->tp->xbuf) cudaFree(ctx->tp->xbuf);
  delete ctx->tp;
  ctx->tp = nullptr;
  return DP_OK;
}

dp_status dp_tp_allreduce_ptr(dp_ctx *ctx, float *ptr, size_t count) {
  if (!dp_tp_ready(ctx) || !ctx->tp->comm) return dp_fail(ctx, DP_ERR_STATE, "allreduce: no tensor-parallel communicator on this context");
  int rc = g_nccl.AllReduce(ptr, ptr, count, ncclFloat32, ncclSum, ctx->tp->comm, ctx->stream);
  if (rc != ncclSuccess) return dp_fail(ctx, DP_ERR_COMM, "ncclAllReduce failed: %s", g_nccl.GetErrorString(rc));
  return DP_OK;
}

dp_status dp_tp_allgather_ptr(dp_ctx *ctx, const void *send, void *recv, size_t bytes_per_rank) {
  if (!dp_tp_ready(ctx) || !ctx->tp->comm) return dp_fail(ctx, DP_ERR_STATE, "allgather: no tensor-parallel communicator on this context");
  int rc = g_nccl.AllGather(send, recv, bytes_per_rank, ncclChar, ctx->tp->comm, ctx->stream);
  if (rc != ncclSuccess) return dp_fail(ctx, DP_ERR_COMM, "ncclAllGather failed: %s", g_nccl.GetErrorString(rc));
  return DP_OK;
}

extern "C" dp_status dp_tp_allreduce_f32(dp_ctx *ctx, dp_recorder *rec, dp_buf buf, size_t offset, size_t count) {
  DP_TRY(dp_check_rec(ctx, rec));
  DP_CHECK(ctx, buf && buf->active, "allreduce: null or released buffer");
  DP_CHECK(ctx, offset % 4 == 0 && offset + count * 4 <= buf->bytes, "allreduce: range exceeds the buffer");
  DP_TRY(dp_tp_allreduce_ptr(ctx, (float *)((char *)buf->dptr + offset), count));
  dp_note_op(ctx, rec);
  return DP_OK;
}

// ---- peer-memory exchange area ------------------------------------------------------------
// Each rank owns one area (layout: tp_exchange.h).  A rank PUSHES its partial vector into its slot of
// every rank's area with ordinary stores over NVLink and then raises its flag there; the consumer
// re-reads slots in its OWN memory only (gemv_q4k_fast.cu, model.cu).  All ranks must barrier (on the host)
// between the last decode call and dp_tp_destroy / dp_ctx_destroy: a slower peer may still be pushing
// into this rank's area.
extern "C" dp_status dp_tp_ipc_export(dp_ctx *ctx, void *out64) {
  if (!ctx || !out64) return DP_ERR_INVALID;
  if (!dp_tp_ready(ctx) || ctx->tp->loopback) return dp_fail(ctx, DP_ERR_STATE, "tp_ipc_export: call dp_tp_init first");
  dp_tp_state *tp = ctx->tp;
  DP_CHECK(ctx, tp->size <= DP_TP_MAX_RANKS, "tp_ipc_export: the exchange area holds %d ranks", DP_TP_MAX_RANKS);
  DP_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!tp->xbuf) {
    DP_CUDA(ctx, cudaMalloc(&tp->xbuf, dp_tp_area_bytes()));
    DP_CUDA(ctx, cudaMemset(tp->xbuf, 0, dp_tp_area_bytes()));
    DP_CUDA(ctx, cudaDeviceSynchronize());
  }
  cudaIpcMemHandle_t h;
  DP_CUDA(ctx, cudaIpcGetMemHandle(&h, tp->xbuf));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return DP_OK;
}

extern "C" dp_status dp_tp_ipc_attach(dp_ctx *ctx, const void *handles64_by_rank) {
  if (!ctx || !handles64_by_rank) return DP_ERR_INVALID;
  if (!dp_tp_ready(ctx) || !ctx->tp->xbuf) return dp_fail(ctx, DP_ERR_STATE, "tp_ipc_attach: export this rank's area first");
  dp_tp_state *tp = ctx->tp;
  if (tp->attached) return dp_fail(ctx, DP_ERR_STATE, "tp_ipc_attach: already attached");
  DP_CHECK(ctx, tp->size <= DP_TP_MAX_RANKS, "tp_ipc_attach: the exchange area holds %d ranks", DP_TP_MAX_RANKS);
  DP_CUDA(ctx, cudaSetDevice(ctx->device));
  for (int r = 0; r < tp->size; r++) {
    if (r == tp->rank) { tp->peer[r] = tp->xbuf; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char *)handles64_by_rank + 64 * r, 64);
    cudaError_t e = cudaIpcOpenMemHandle(&tp->peer[r], h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return dp_fail(ctx, DP_ERR_COMM, "tp_ipc_attach: cannot map rank %d's exchange area: %s", r, cudaGetErrorString(e));
    }
  }
  dp_tp_exchange d;
  memset(&d, 0, sizeof d);
  d.rank = tp->rank; d.size = tp->size;
  for (int r = 0; r < tp->size; r++) d.area[r] = (uint2 *)tp->peer[r];
  DP_CUDA(ctx, cudaMalloc(&tp->dev_desc, sizeof d + 64));
  DP_CUDA(ctx, cudaMemset(tp->dev_desc, 0, sizeof d + 64));
  DP_CUDA(ctx, cudaMemcpy(tp->dev_desc, &d, sizeof d, cudaMemcpyHostToDevice));
  tp->attached = true;
  return DP_OK;
}

// descriptor for the fused kernels, or nullptr when the exchange area is not attached
dp_tp_exchange *dp_tp_exchange_desc(dp_ctx *ctx) {
  return (ctx && ctx->tp && ctx->tp->attached) ? ctx->tp->dev_desc : nullptr;
}

// the attached group's areas by value (kernels take them as parameters); false when there is none
bool dp_tp_exchange_view(dp_ctx *ctx, int *rank, int *size, uint2 **areas) {
  if (!ctx || !ctx->tp || !ctx->tp->attached) return false;
  *rank = ctx->tp->rank; *size = ctx->tp->size;
  for (int r = 0; r < ctx->tp->size; r++) areas[r] = (uint2 *)ctx->tp->peer[r];
  return true;
}

// (kept for the status path: nothing to reset, tickets only ever grow)
void dp_tp_reset_barrier(dp_ctx *) {}
