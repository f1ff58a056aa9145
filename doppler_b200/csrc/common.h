// Internal definitions shared by the translation units of libdoppler_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <atomic>
#include <map>
#include <string>
#include <vector>

#include "../../include/doppler_b200.h"

struct dp_buf_s {
  void *dptr = nullptr;
  size_t bytes = 0;     // requested
  size_t capacity = 0;  // bucket
  dp_ctx *ctx = nullptr;
  bool active = false;
  std::string label;
};

// A function attribute (the opt-in shared-memory size) is set per device: a kernel that sets it only on its first
// launch keeps one of these, so that a second device used by the same process gets the attribute too.
struct dp_per_device_once {
  std::atomic<uint64_t> mask{0};
  bool pending(int dev) const { return ((mask.load(std::memory_order_acquire) >> (dev & 63)) & 1ull) == 0; }
  void done(int dev) { mask.fetch_or(1ull << (dev & 63), std::memory_order_release); }
};

struct dp_tp_state;     // tp.cu
struct dp_tp_exchange;  // tp_exchange.h

struct dp_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  int sm_count = 148;
  size_t smem_optin = 0;
  std::string err;
  uint64_t launches = 0;
  // buffer pool: bucket size -> idle allocations
  std::multimap<size_t, dp_buf_s *> idle;
  std::vector<dp_buf_s *> all;
  dp_pool_stats stats{};
  // lazily grown scratch for split-K attention partials (stream ordered)
  dp_buf attn_scratch = nullptr;
  dp_buf argmax_scratch = nullptr;
  dp_buf gemv_scratch = nullptr;  // quantised activation digits of the fast GEMV (stream ordered)
  dp_buf gemm_scratch = nullptr;  // f16 activations (halves, residues, row scales) of the tensor-core GEMM (stream ordered)
  dp_buf gemm_split_scratch = nullptr;  // partial output tiles of a K-split tensor-core GEMM (stream ordered)
  bool pdl = false;  // launch with programmatic dependent launch (set while the decode step is recorded)
  int *dev_status = nullptr;  // device word raised by a kernel whose bounded wait gave up
  dp_recorder *active_recorder = nullptr;
  dp_tp_state *tp = nullptr;
  unsigned wait_limit = 1u << 22;      // polls before a device-side wait on another CTA / rank gives up
  // Captured graphs keep device pointers.  While a capture is open or a graph of this context is alive,
  // a context scratch that has to grow is not handed back to the pool (a later acquire could give it to
  // somebody else while a graph replay still writes it): it waits here until the last graph is destroyed.
  int live_graphs = 0;
  std::vector<dp_buf> retired_scratch;
};

struct dp_recorder {
  dp_ctx *ctx = nullptr;
  std::string label;
  bool capture = false;
  bool open = false;
  std::vector<dp_buf> temporaries;
  uint32_t ops = 0;
  uint64_t launches_at_begin = 0;
};

struct dp_graph {
  dp_ctx *ctx = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t kernels = 0;
  std::vector<dp_buf> owned;  // the recording's temporaries: the graph's kernels point at them until it is destroyed
};

dp_status dp_fail(dp_ctx *ctx, dp_status st, const char *fmt, ...);

#define DP_CUDA(ctx, expr)                                                                  \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess)                                                                  \
      return dp_fail((ctx), _e == cudaErrorMemoryAllocation ? DP_ERR_OOM : DP_ERR_CUDA,     \
                     "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

#define DP_CHECK(ctx, cond, ...)                                   \
  do {                                                             \
    if (!(cond)) return dp_fail((ctx), DP_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define DP_TRY(expr)                 \
  do {                               \
    dp_status _s = (expr);           \
    if (_s != DP_OK) return _s;      \
  } while (0)

// Every kernel launch of this library goes through here so launches are counted
// and launch errors surface as a status.  With ctx->pdl the launch carries the
// programmatic-stream-serialization attribute: the kernel may start while its
// predecessor drains, and must execute pdl_wait() before it touches anything the
// predecessor wrote (every kernel on the decode path does, see pdl.cuh).
template <typename... KArgs, typename... Args>
static inline cudaError_t dp_launch_impl(dp_ctx *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define DP_LAUNCH(ctx, kernel, grid, block, smem, ...)                                   \
  do {                                                                                   \
    cudaError_t _e = dp_launch_impl((ctx), kernel, dim3(grid), dim3(block), (smem), __VA_ARGS__); \
    (ctx)->launches++;                                                                   \
    if (_e == cudaSuccess) _e = cudaGetLastError();                                      \
    if (_e != cudaSuccess)                                                               \
      return dp_fail((ctx), DP_ERR_CUDA, "launch of %s failed: %s", #kernel,             \
                     cudaGetErrorString(_e));                                            \
  } while (0)

static inline size_t dp_dtype_size(dp_dtype t) {
  switch (t) {
    case DP_F32: return 4;
    case DP_F16: return 2;
    case DP_I32: return 4;
    default: return 0;
  }
}

static inline const char *dp_dtype_name(dp_dtype t) {
  switch (t) {
    case DP_F32: return "f32";
    case DP_F16: return "f16";
    case DP_Q4K: return "q4k";
    case DP_I32: return "i32";
  }
  return "?";
}

static inline size_t dp_cdiv(size_t a, size_t b) { return (a + b - 1) / b; }

// Pointer of a tensor/weight (buffer base + offset), or nullptr
static inline char *dp_tptr(const dp_tensor *t) {
  return (t && t->buf) ? (char *)t->buf->dptr + t->offset : nullptr;
}
static inline size_t dp_tavail(const dp_tensor *t) {
  return (t && t->buf && t->offset <= t->buf->bytes) ? t->buf->bytes - t->offset : 0;
}

// output helper: use out_buf when given (checked for size), else acquire from the pool
dp_status dp_out_buffer(dp_ctx *ctx, dp_buf out_buf, size_t offset, size_t bytes, const char *label,
                        dp_buf *result);
void dp_note_op(dp_ctx *ctx, dp_recorder *rec);
dp_status dp_check_rec(dp_ctx *ctx, dp_recorder *rec);
dp_status dp_scratch(dp_ctx *ctx, dp_buf *slot, size_t bytes, const char *label);

// ---- kernel launchers (one per .cu) --------------------------------------
dp_status dpk_dequant_q4k(dp_ctx *ctx, const uint8_t *packed, size_t rows, size_t bpr, size_t K,
                          void *out, dp_dtype out_dtype);
dp_status dpk_gemv_q4k(dp_ctx *ctx, const uint8_t *W, const float *x, void *y, dp_dtype y_dtype,
                       int N, int K, float alpha, const float *residual);
dp_status dpk_gemm_q4k_simt(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, void *C,
                            dp_dtype c_dtype, int M, int N, int K, float alpha);
enum { DPK_ROWS_PRE_NONE = 0, DPK_ROWS_PRE_RMSNORM = 1, DPK_ROWS_PRE_SILU = 2 };
struct dpk_rows_fuse {
  int pre = 0;                      // operation on the input rows folded into the pre-pass
  const float *norm_w = nullptr;    // DPK_ROWS_PRE_RMSNORM
  float eps = 0.0f;
  const float *residual = nullptr;  // added to the output [M, N] (may be the output buffer itself)
};
// Optional fusions of the row-scaled tensor-core GEMM (f32 in, f32 out).  The caller asks by filling the pointers;
// the *_done flags say what the launch took over, the rest stays with the caller.
struct dpk_tc_fuse {
  float *silu_dst = nullptr;        // [M, N / 2]: silu(gate) * up of gate|up column pairs, stored by the epilogue instead of C
  const float *residual = nullptr;  // added by the fixed-order reduction of a K-split launch ...
  float *residual_out = nullptr;    // ... which then writes here (may be the residual itself) instead of C
  const float *norm_w = nullptr;    // RMSNorm weights: A holds the un-normalised rows and the norm is folded into their conversion to f16
  float eps = 0.0f;                 //   (the call is left unhandled, nothing launched, where that conversion cannot take it)
  bool silu_done = false, residual_done = false;
};
dp_status dpk_gemm_q4k_tc_rowscaled(dp_ctx *ctx, const uint8_t *W, const float *A, float *C, int M, int N, int K, float alpha, int passes,
                                    bool *handled, dpk_tc_fuse *fuse = nullptr);

dp_status dpk_gemm_q4k_tc_rows(dp_ctx *ctx, const uint8_t *W, const void *A, dp_dtype a_dtype, float *C, int M, int N, int K, float alpha,
                               bool *handled, const dpk_rows_fuse *fuse = nullptr);
dp_status dpk_scale_cast_rows(dp_ctx *ctx, const float *A, __half *hi, __half *lo, float *row_scale, int M, int K);
// f16 weights times 2..64+ activation rows, the weights streamed once (gemm_f16w_rows.cu)
dp_status dpk_gemm_f16w_rows(dp_ctx *ctx, const __half *W, const void *A, dp_dtype a_dtype, void *C, dp_dtype c_dtype, int M, int N, int K,
                             float alpha, bool *handled);
dp_status dpk_gemv_f16w(dp_ctx *ctx, const __half *W, const void *A, dp_dtype a_dtype, void *C,
                        dp_dtype c_dtype, int M, int N, int K, float alpha);
dp_status dpk_gemv_f32w(dp_ctx *ctx, const float *W, const float *A, float *C, int M, int N, int K,
                        float alpha);
// Optional fusion of the decode step's per-head QK RMSNorm + RoPE + KV append into the attention
// kernel (tensor-core kernel, one new token per sequence).  qkv holds the raw projections
// [sequence][nh q heads | nkv k heads | nkv v heads][head_dim]; the kernel normalises and rotates its
// own q heads, and the CTA whose key range ends at the new position builds the new K/V row, uses it
// and appends it to the cache (kc / vc, same layout and batch stride as k / v).
struct dpk_attn_fuse {
  const float *qkv = nullptr;
  const float *q_norm = nullptr, *k_norm = nullptr, *cos_t = nullptr, *sin_t = nullptr;
  const int *pos = nullptr;  // position of the new token of each sequence
  __half *kc = nullptr, *vc = nullptr;
  float eps = 0.0f;
  int nh = 0, nkv = 0;
};
struct dpk_attn_params {
  dpk_attn_fuse fuse;
  const float *q;
  const __half *k, *v;
  float *out;
  int batch, seq_len, kv_len, num_heads, num_kv_heads, head_dim;
  float scale, softcap;
  int causal, start_pos, sliding_window, kv_start;
  size_t kv_batch_stride;
  const int *kv_lens;
};
dp_status dpk_attention(dp_ctx *ctx, const dpk_attn_params &p);
bool dpk_attention_uses_tc(dp_ctx *ctx, const dpk_attn_params &p);
// variant with caller-provided scratch (no allocation); scratch_bytes must cover dpk_attention_scratch_bytes
size_t dpk_attention_scratch_bytes(dp_ctx *ctx, const dpk_attn_params &p, int *splits_out);
dp_status dpk_attention_with_scratch(dp_ctx *ctx, const dpk_attn_params &p, float *scratch, int splits);

dp_status dpk_rmsnorm(dp_ctx *ctx, const float *x, const void *w, bool w_f16, const float *residual,
                      bool pre_residual, float *residual_sum_out, float *y, int rows, int size,
                      float eps, bool weight_offset, float output_scale);
dp_status dpk_rmsnorm_qk(dp_ctx *ctx, float *q, const float *qw, float *k, const float *kw, int q_rows,
                         int k_rows, int head_dim, float eps, bool weight_offset);
dp_status dpk_rope(dp_ctx *ctx, float *x, const float *cos_t, const float *sin_t, int seq_len,
                   int num_heads, int head_dim, int rotary_dim, int pair_span, bool interleaved,
                   int start_pos);
dp_status dpk_silu_mul(dp_ctx *ctx, const float *up, const float *gate, float *out, size_t n, float clamp_max);
dp_status dpk_residual_add(dp_ctx *ctx, const float *a, const float *b, float *out, size_t n, float scale);
dp_status dpk_gather_f16(dp_ctx *ctx, const int *ids, const __half *table, float *out, int n_ids, int hidden);
dp_status dpk_kv_write(dp_ctx *ctx, const float *src, __half *dst, size_t n);
dp_status dpk_argmax_rows(dp_ctx *ctx, const float *logits, int n, size_t row_stride, int rows, int *out, float *scratch_vals,
                          int *scratch_idx, int index_base, float *best_vals);
dp_status dpk_argmax(dp_ctx *ctx, const float *logits, int n, int pad_id, int *out, int out_index,
                     float *scratch_vals, int *scratch_idx, int index_base, float *best_val_out);
