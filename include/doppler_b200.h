/*
 * doppler_b200 -- C ABI of the B200 (sm_100a) implementation of Doppler's
 * Q4_K quantized-inference hot path.
 *
 * The reference (clocksmith/doppler) has no FFI layer: its seam is the
 * JavaScript op module src/gpu/kernels/index.js plus three data types
 * (Tensor, WeightBuffer, pooled GPUBuffer) and the CommandRecorder.  Each entry
 * point below replaces one of those JavaScript functions and cites it.  A host
 * binding (N-API, ctypes, cgo ...) maps the reference call 1:1 onto these.
 *
 * Conventions
 *  - plain pointers, sizes and POD structs only; no C++ or torch types;
 *  - every call returns a dp_status; on failure dp_last_error(ctx) holds a
 *    message with shape/dtype context (the reference throws Error objects);
 *  - one host thread per context; work is ordered on the context's stream
 *    (the reference is single-threaded JS with queue order);
 *  - an op given `rec == NULL` is enqueued at once (reference runX); with a
 *    recorder it is appended to that recording (reference recordX);
 *  - an op returns a dp_tensor wrapping a pooled buffer the CALLER owns, unless
 *    the caller supplied `out_buf` (reference outputBuffer option);
 *  - there is no CPU fallback anywhere: without a CUDA device dp_ctx_create
 *    fails with DP_ERR_CUDA.
 */
#ifndef DOPPLER_B200_H
#define DOPPLER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DP_QK_K 256            /* src/config/schema/quantization.schema.js:5 */
#define DP_Q4K_BLOCK_BYTES 144 /* src/config/schema/quantization.schema.js:8 */
#define DP_BUFFER_ALIGN 256    /* src/gpu/kernels/constants.js:90-102 */

typedef enum {
  DP_OK = 0,
  DP_ERR_INVALID = 1,     /* bad argument / shape / dtype / alignment */
  DP_ERR_CUDA = 2,        /* a CUDA runtime call failed */
  DP_ERR_OOM = 3,
  DP_ERR_UNSUPPORTED = 4, /* valid in the reference, outside this path */
  DP_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
  DP_ERR_STATE = 6,       /* stale handle, wrong recorder state */
  DP_ERR_COMM = 7         /* NCCL / peer-memory failure */
} dp_status;

typedef enum { DP_F32 = 0, DP_F16 = 1, DP_Q4K = 2, DP_I32 = 3 } dp_dtype;

typedef struct dp_ctx dp_ctx;
typedef struct dp_buf_s *dp_buf; /* pooled device allocation (reference: GPUBuffer) */
typedef struct dp_recorder dp_recorder;
typedef struct dp_graph dp_graph;
typedef struct dp_kv_cache dp_kv_cache;
typedef struct dp_model dp_model;

/* reference: Tensor {buffer,dtype,shape,label}  src/gpu/tensor.js:7-19 */
typedef struct {
  dp_buf buf;
  size_t offset; /* bytes, multiple of 256 (matmul-selection.js:197-213) */
  dp_dtype dtype;
  int ndim;
  int64_t shape[4];
} dp_tensor;

/* reference: WeightBuffer {buffer,dtype,layout,shape:[N,K]}  src/gpu/weight-buffer.js:78-115 */
typedef struct {
  dp_buf buf;
  size_t offset;
  dp_dtype dtype;   /* DP_Q4K, DP_F16 or DP_F32 */
  int layout;       /* 0 = 'row' ([N,K], K contiguous); 'column' is rejected */
  int64_t shape[2]; /* [N, K] */
} dp_weight;

/* ---- context ------------------------------------------------------------ */
/* reference: initDevice / getDevice  src/gpu/device.js */
dp_status dp_ctx_create(int device, dp_ctx **out);
void dp_ctx_destroy(dp_ctx *ctx);
const char *dp_last_error(dp_ctx *ctx);
dp_status dp_ctx_sync(dp_ctx *ctx);
/* Device-side waits on another CTA or another rank (the hand-offs between the phases of the decode
 * kernels, within a GPU and across ranks) poll at most `polls` times (default 4,194,304, a few seconds) before the kernel gives up,
 * raises the status word and returns; the next dp_ctx_sync / dp_model_decode / dp_model_prefill then
 * reports DP_ERR_TIMEOUT and the context stays usable.  No counterpart in the reference (WebGPU has
 * no cross-workgroup waits); it plays the role of its device-lost detection, src/gpu/device.js:280-318. */
dp_status dp_ctx_set_wait_limit(dp_ctx *ctx, unsigned polls);
void *dp_ctx_stream(dp_ctx *ctx); /* the cudaStream_t all work is ordered on */
int dp_ctx_device(dp_ctx *ctx);
/* number of kernels this library launched on the context so far */
uint64_t dp_ctx_launch_count(dp_ctx *ctx);
const char *dp_version(void);

/* ---- buffer pool -------------------------------------------------------- */
/* reference: acquireBuffer / releaseBuffer / uploadData / readBuffer
 * src/memory/buffer-pool.js:815-869; size buckets :73-118 */
dp_status dp_buf_acquire(dp_ctx *ctx, size_t bytes, const char *label, dp_buf *out);
dp_status dp_buf_release(dp_ctx *ctx, dp_buf buf);
dp_status dp_buf_upload(dp_ctx *ctx, dp_buf buf, const void *host, size_t offset, size_t bytes);
dp_status dp_buf_read(dp_ctx *ctx, dp_buf buf, void *host, size_t offset, size_t bytes); /* synchronises */
dp_status dp_buf_fill(dp_ctx *ctx, dp_buf buf, int byte_value, size_t offset, size_t bytes);
void *dp_buf_device_ptr(dp_buf buf);
size_t dp_buf_size(dp_buf buf);     /* requested size */
size_t dp_buf_capacity(dp_buf buf); /* bucket size */
size_t dp_pool_bucket_size(size_t bytes);
typedef struct {
  uint64_t allocations, reuses, releases;
  uint64_t bytes_allocated, bytes_in_use, bytes_pooled, peak_bytes_allocated;
} dp_pool_stats;
/* reference: BufferPool.getStats  src/memory/buffer-pool.js:205-214 */
dp_status dp_pool_get_stats(dp_ctx *ctx, dp_pool_stats *out);
dp_status dp_pool_trim(dp_ctx *ctx); /* free every pooled (inactive) allocation */

/* ---- recorder ----------------------------------------------------------- */
/* reference: CommandRecorder  src/gpu/command-recorder.js:14 (begin), :419
 * (trackTemporaryBuffer), :560 (submitAndWait).  With capture_graph != 0 the
 * recording is captured into a CUDA graph that can be replayed. */
dp_status dp_recorder_begin(dp_ctx *ctx, const char *label, int capture_graph, dp_recorder **out);
dp_status dp_recorder_track_temporary(dp_recorder *rec, dp_buf buf);
dp_status dp_recorder_submit(dp_recorder *rec);          /* launches; temporaries go back to the pool */
dp_status dp_recorder_submit_and_wait(dp_recorder *rec); /* + stream synchronise */
dp_status dp_recorder_abort(dp_recorder *rec);
/* Ends a capturing recorder without launching and hands out the graph.
 * Lifetimes: a graph's kernels hold device pointers.  The graph takes over the recording's tracked
 * temporaries and returns them to the pool in dp_graph_destroy; the context's internal scratch
 * areas that recorded ops used stay allocated while any graph of the context is alive (one that a
 * later, larger call has to regrow is parked, not recycled).  Buffers the CALLER passed to recorded
 * ops (inputs, weights, output buffers) are the caller's to keep alive until dp_graph_destroy;
 * releasing one earlier lets the pool hand it to another owner that a replay then overwrites.
 * Destroy a context's graphs before the context. */
dp_status dp_recorder_finish_graph(dp_recorder *rec, dp_graph **out);
dp_status dp_graph_launch(dp_graph *g);
/* reference: recorder timestamp profiling  src/gpu/command-recorder.js:123-181,622 (resolveProfileTimings).
 * `reps` replays bracketed by two CUDA events on the context's stream, then a synchronise;
 * *ms = device time of all replays. */
dp_status dp_graph_launch_timed(dp_graph *g, int reps, double *ms);
void dp_graph_destroy(dp_graph *g);
/* reference: recorder op-label statistics  src/gpu/command-recorder.js:123-181 */
uint32_t dp_recorder_op_count(dp_recorder *rec);

/* ---- matmul ------------------------------------------------------------- */
/* reference: runMatmul / recordMatmul  src/gpu/kernels/matmul.js:659,664
 * (options: src/gpu/kernels/matmul.d.ts:20-87).
 * C[M,N] = alpha * A[M,K] . B[N,K]^T.  B.dtype DP_Q4K selects the fused
 * dequant kernels (M==1: decode GEMV, fused_matmul_q4.wgsl:279; M>1: prefill
 * GEMM, fused_matmul_q4_batched*.wgsl / _prefill_tiled_f16.wgsl); DP_F16 is the
 * f16-weight GEMV/GEMM used for the LM head (matmul_gemv_subgroup.wgsl).
 * M>1 with Q4_K weights follows the reference's rule (matmul.rules.json:15-22):
 * the dequantised weights enter the product with f32 accuracy and the sum is
 * kept in f32 (f16 outputs are rounded once, at the store:
 * fused_matmul_q4_batched_f16a.wgsl:107,151).  On the tensor cores that is the
 * f16 halves AND the f16 rounding residues of the weights (and, for f32
 * activations from 32 rows on, of the activations) multiplied into one f32
 * accumulator; smaller or untiled f32 problems run on CUDA cores.
 * opts.f16_weights = 1 selects the numerics of the reference's opt-in tiled
 * prefill kernel instead (fused_matmul_q4_prefill_tiled_f16.wgsl:201: every
 * dequantised weight rounded to f16 first), one tensor-core product. */
typedef struct {
  float alpha;        /* default 1 */
  dp_dtype out_dtype; /* DP_F32 or DP_F16 (reference: outputDtype, required) */
  size_t a_off, b_off, c_off; /* extra byte offsets, multiples of 256 */
  dp_buf out_buf;     /* optional caller-owned output */
  int transpose_b;    /* must be 1 (weights are [N,K]); 0 is DP_ERR_UNSUPPORTED */
  int exact_weights;  /* M>1 only: 1 = always the CUDA-core kernel with f32-exact weights */
  int f16_weights;    /* M>1, f16 activations: 1 = weights rounded to f16 before the product (opt-in, see above) */
} dp_matmul_opts;
void dp_matmul_opts_default(dp_matmul_opts *o);
dp_status dp_matmul(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *A, const dp_weight *B, int M,
                    int N, int K, const dp_matmul_opts *opts, dp_tensor *out);

/* ---- dequant ------------------------------------------------------------ */
/* reference: dequantize / recordDequantize  src/gpu/kernels/dequant.js:90,455
 * (dequant_shared.wgsl:86-145): numBlocks*256 values, flat. */
dp_status dp_dequant_q4k(dp_ctx *ctx, dp_recorder *rec, dp_buf packed, size_t packed_off,
                         uint32_t num_blocks, dp_dtype out_dtype, size_t out_off, dp_buf out_buf,
                         dp_tensor *out);
/* reference: dequantizeRowwise  src/gpu/kernels/dequant.js:162: [rows,K], K tail stripped */
dp_status dp_dequant_q4k_rowwise(dp_ctx *ctx, dp_recorder *rec, dp_buf packed, size_t packed_off,
                                 int rows, int K, dp_dtype out_dtype, dp_buf out_buf, dp_tensor *out);

/* ---- attention ---------------------------------------------------------- */
/* reference: runAttention / recordAttention  src/gpu/kernels/attention.js:2007,2019
 * (options attention.d.ts:18-50; kernel attention_decode_online_f16kv.wgsl:85).
 * Q f32 [seq_len, num_heads, head_dim]; K,V f16 [kv positions, num_kv_heads,
 * head_dim]; out f32 [seq_len, num_heads, head_dim].  seq_len==1 takes the
 * split-K flash-decode kernel; seq_len>1 the causal prefill kernel.
 * `batch` > 1 is an extension (the reference is batch 1): Q and out gain a
 * leading batch dimension, K/V of sequence b start at b*kv_batch_stride
 * elements, and kv_lens (device i32[batch], optional) overrides kv_len. */
typedef struct {
  int seq_len, kv_len, num_kv_heads;
  float scale;         /* <= 0 selects 1/sqrt(head_dim) */
  int causal;          /* default 1 */
  int start_pos;       /* absolute position of query row 0 */
  int sliding_window;  /* 0 = off */
  float attn_softcap;  /* 0 = off */
  int kv_start;        /* absolute position of cache row 0 */
  int batch;           /* default 1 */
  size_t kv_batch_stride; /* elements */
  dp_buf kv_lens;      /* optional device i32[batch] (reference: kvLenBuffer) */
  dp_buf out_buf;
} dp_attn_opts;
void dp_attn_opts_default(dp_attn_opts *o);
dp_status dp_attention(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *Q, const dp_tensor *K,
                       const dp_tensor *V, int num_heads, int head_dim, const dp_attn_opts *opts,
                       dp_tensor *out);

/* Decode attention (seq_len 1, no mask) for hosts that must not allocate device memory while
 * they run (a plugin called under someone else's stream capture, a worker that is only handed
 * buffers and a stream, a process with a fixed allocator budget).  No counterpart in the
 * reference.  Raw device pointers, a cudaStream_t, no context: the split-K scratch is a fixed
 * device array inside the library (dp_attention_decode_static_max_scratch() bytes on every GPU
 * that loads it).  Calls needing more scratch return DP_ERR_UNSUPPORTED; overlapping calls race on
 * the array; the first call on a device resolves the array's address and should happen outside
 * stream capture.  The message of the last failure on this thread: ..._error(). */
dp_status dp_attention_decode_static(void *stream, const float *q, const void *k_f16, const void *v_f16, float *out,
                                     int batch, int num_heads, int num_kv_heads, int head_dim, int kv_len,
                                     size_t kv_batch_stride, float scale);
const char *dp_attention_decode_static_error(void);
size_t dp_attention_decode_static_max_scratch(void);

/* ---- small ops ---------------------------------------------------------- */
/* reference: runRMSNorm / recordRMSNorm  src/gpu/kernels/rmsnorm.js:146,224 (rmsnorm.wgsl:119-187) */
typedef struct {
  int batch_size, hidden_size;
  const dp_tensor *residual; /* added AFTER the norm (rmsnorm.wgsl has_residual) */
  int pre_residual;          /* 1: norm(input + residual) instead (PRE_RESIDUAL) */
  dp_buf residual_sum_output;/* with pre_residual: receives input + residual (OUTPUT_PRENORM) */
  int weight_offset;         /* 1: use (1 + w)  (RMS_NORM_OFFSET) */
  float output_scale;        /* default 1 */
  dp_buf out_buf;
} dp_rmsnorm_opts;
void dp_rmsnorm_opts_default(dp_rmsnorm_opts *o);
dp_status dp_rmsnorm(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_tensor *weight,
                     float eps, const dp_rmsnorm_opts *opts, dp_tensor *out);
/* reference: runRMSNormQK  src/gpu/kernels/rmsnorm-qk.js (rmsnorm_qk.wgsl:75-118): in place */
dp_status dp_rmsnorm_qk(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *q, const dp_tensor *q_weight,
                        const dp_tensor *k, const dp_tensor *k_weight, int q_rows, int k_rows,
                        int head_dim, float eps, int weight_offset);
/* reference: runRoPE / recordRoPE  src/gpu/kernels/rope.js:108,112 (rope.wgsl:62-106): in place */
typedef struct {
  int num_heads, head_dim, rotary_dim, pair_span_dim, interleaved, start_pos;
} dp_rope_opts;
dp_status dp_rope(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_tensor *freqs_cos,
                  const dp_tensor *freqs_sin, int seq_len, const dp_rope_opts *opts);
/* reference: computeRoPEFreqsForTheta  src/inference/pipelines/text/init-rope.js:11-134
 * (no scaling): host-side table build into caller memory [max_seq, rotary_dim/2] */
dp_status dp_rope_tables(double theta, int rotary_dim, int max_seq, float *cos_out, float *sin_out);
/* reference: runSiLU with gate  src/gpu/kernels/silu.wgsl:98-104: out = silu(gate)*up */
dp_status dp_silu_mul(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *up, const dp_tensor *gate,
                      size_t n, float clamp_max, dp_buf out_buf, dp_tensor *out);
/* reference: runResidualAdd  src/gpu/kernels/residual.wgsl:25-32: out = (a+b)*scale */
dp_status dp_residual_add(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *a, const dp_tensor *b,
                          size_t n, float scale, dp_buf out_buf, dp_tensor *out);
/* reference: runGather  src/gpu/kernels/gather_f16.wgsl:35-66: f16 rows -> f32 */
dp_status dp_gather_f16(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *ids_i32,
                        const dp_tensor *table_f16, int n_ids, int hidden, dp_buf out_buf,
                        dp_tensor *out);
/* reference: runKVCacheWriteF32ToF16  src/gpu/kernels/kv_cache_write_f32_to_f16.wgsl:19 */
dp_status dp_kv_write_f32_to_f16(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *src_f32,
                                 dp_buf dst_f16, size_t dst_offset_elems, size_t n);
/* reference: runArgmax  src/gpu/kernels/sample.wgsl:311-408; ties -> lower index (:45-53) */
dp_status dp_argmax(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *logits, int n, int pad_id,
                    dp_buf out_tokens_i32, int output_index);

/* ---- quantizer ---------------------------------------------------------- */
/* reference: quantizeToQ4KMRowWise  src/converter/quantizer.js:253-288 (full_pad = 0: the tail of a
 * row's last block is left out of the ranges) and quantizeToQ4KM :223-251 (rows = 1, full_pad = 1:
 * the tail is zero padded and quantised as a full block).  Bit-exact with the reference's
 * double-precision arithmetic.  src f32 [rows, cols]; out: packed blocks, dtype q4k, layout row. */
dp_status dp_quantize_q4k(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *src_f32, int64_t rows, int64_t cols,
                          int full_pad, dp_buf out_buf, dp_weight *out);

/* ---- fused decode ops ---------------------------------------------------
 * The reference exposes these as ops of their own (src/gpu/kernels/index.js:300-330); they keep
 * the reference's argument meaning so that a pipeline that records them needs no other change. */
/* reference: runFusedFFN / recordFusedFFN  src/gpu/kernels/fused_ffn.js:501,605 (fused_ffn_q4k.wgsl:
 * 115-117,241-246): out[b,i] = clamp(silu(Wgate.x_b)_i * (Wup.x_b)_i * alpha, +-swiglu_limit),
 * silu(x) = x / (1 + exp(-x)); f32 input [batch, hidden], f32 output [batch, inter]. */
typedef struct {
  int batch_size;       /* default 1 */
  float alpha;          /* default 1 */
  float swiglu_limit;   /* 0 = no clamp */
  dp_buf out_buf;
} dp_ffn_opts;
void dp_ffn_opts_default(dp_ffn_opts *o);
dp_status dp_fused_ffn(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *w_gate,
                       const dp_weight *w_up, int hidden_size, int intermediate_size,
                       const dp_ffn_opts *opts, dp_tensor *out);
/* reference: runMatmulResidualFused  src/gpu/kernels/fused_matmul_residual.js:27 (M = 1):
 * out[N] = alpha * (W.x) + residual */
dp_status dp_matmul_residual(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *weight,
                             const dp_tensor *residual, int N, int K, float alpha, dp_buf out_buf,
                             dp_tensor *out);
/* reference: runMatmulRMSNormFused  src/gpu/kernels/fused_matmul_rmsnorm.js:52
 * (fused_matmul_rmsnorm.wgsl:1-12,161): out[N] = rmsnorm(W.x, norm_weight, eps) + residual (M = 1) */
dp_status dp_matmul_rmsnorm(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *weight,
                            const dp_tensor *norm_weight, int N, int K, float eps,
                            const dp_tensor *residual, int weight_offset, dp_buf out_buf, dp_tensor *out);
/* reference: recordLmHeadArgmax  src/gpu/kernels/lm-head-argmax.js:292 (lm_head_argmax_q4k.wgsl):
 * token = argmax_v (lm_head[v,:] . x), pad_token_id excluded, ties to the lower index; the id is
 * written to out_tokens_i32[output_index].  lm_head is f16 or Q4_K [vocab, hidden]. */
dp_status dp_lm_head_argmax(dp_ctx *ctx, dp_recorder *rec, const dp_tensor *input, const dp_weight *lm_head,
                            int vocab_size, int hidden_size, int pad_token_id, dp_buf out_tokens_i32,
                            int output_index);

/* ---- KV cache ----------------------------------------------------------- */
/* reference: KVCache (contiguous f16)  src/inference/kv-cache/base.js:18,99-153;
 * truncate :962; clone :829.  Per layer two buffers [batch][max_seq, n_kv_heads, head_dim] f16. */
dp_status dp_kv_cache_create(dp_ctx *ctx, int layers, int max_seq, int n_kv_heads, int head_dim,
                             int batch, dp_kv_cache **out);
void dp_kv_cache_destroy(dp_kv_cache *kv);
dp_status dp_kv_layer(dp_kv_cache *kv, int layer, dp_buf *keys, dp_buf *values);
int dp_kv_seq_len(dp_kv_cache *kv);
dp_status dp_kv_set_seq_len(dp_kv_cache *kv, int len);
dp_status dp_kv_truncate(dp_kv_cache *kv, int len);
dp_status dp_kv_clone(dp_kv_cache *kv, dp_kv_cache **out);
size_t dp_kv_bytes(dp_kv_cache *kv);

/* ---- decoder runner (scheduling + weight upload) ------------------------ */
/* reference: decodeStep  src/inference/pipelines/text/generator-steps.js:588,
 * processLayerGPU layer.js:682, loadQ4KFused src/loader/tensors/tensor-loader.js:540-558.
 * Dense Qwen3-shaped decoder: f32 activations, per-head QK RMSNorm, rotate-half
 * RoPE, f16 KV, Q4_K linear weights kept packed in HBM, f16 embedding/LM head.
 * Under tensor parallelism (tp_size > 1) q/k/v/gate/up are split by output rows,
 * o/down by 256-element super-block columns, the LM head by vocabulary rows. */
typedef struct {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, inter, vocab, max_seq;
  float eps, rope_theta;
  int max_batch; /* sequences decoded side by side (extension; reference = 1) */
  int tp_rank, tp_size;
} dp_model_cfg;
typedef enum {
  DP_W_Q = 0, DP_W_K, DP_W_V, DP_W_O, DP_W_GATE, DP_W_UP, DP_W_DOWN,      /* Q4_K */
  DP_W_IN_NORM, DP_W_POST_NORM, DP_W_Q_NORM, DP_W_K_NORM                  /* f32 */
} dp_weight_id;
dp_status dp_model_create(dp_ctx *ctx, const dp_model_cfg *cfg, dp_model **out);
void dp_model_destroy(dp_model *m);
/* host_bytes hold the FULL matrix; the runner keeps only this rank's slice */
dp_status dp_model_load_q4k(dp_model *m, int layer, dp_weight_id which, const void *host_bytes,
                            int N, int K);
dp_status dp_model_load_norm(dp_model *m, int layer, dp_weight_id which, const float *host, int n);
dp_status dp_model_load_final_norm(dp_model *m, const float *host, int n);
/* rows [row0,row0+rows) of the f16 [vocab,hidden] tables, so a caller can stream them */
dp_status dp_model_load_embed(dp_model *m, const void *host_f16, int row0, int rows);
dp_status dp_model_load_lm_head(dp_model *m, const void *host_f16, int row0, int rows);
dp_status dp_model_reset(dp_model *m);
/* prompt of n tokens for sequence `seq`; next_token receives the greedy token */
dp_status dp_model_prefill(dp_model *m, int seq, const int32_t *tokens, int n, int32_t *next_token);
/* `steps` greedy decode steps for `batch` sequences; out_tokens is [steps][batch] */
dp_status dp_model_decode(dp_model *m, int batch, const int32_t *first_tokens, int steps,
                          int32_t *out_tokens);
/* timing of the last dp_model_decode (device time between events) and logits probe */
double dp_model_last_decode_ms(dp_model *m);
dp_status dp_model_read_logits(dp_model *m, float *host, int n);
dp_status dp_model_read_hidden(dp_model *m, float *host, int n);
size_t dp_model_weight_bytes(dp_model *m);
int dp_model_seq_len(dp_model *m, int seq);
/* Kernel-level timing of the dominant kernel (reference: CommandRecorder timestamp profiling,
 * src/gpu/command-recorder.js:123-181): launches every Q4_K decode GEMV of the loaded model
 * (qkv, o, gate|up, down of every layer) back to back, `reps` passes, between two CUDA events
 * on the context's stream.  bytes = algorithmic bytes of those launches
 * (N*ceil(K/256)*144 + 4K + 4N each). */
dp_status dp_model_bench_gemv(dp_model *m, int reps, double *ms_total, uint64_t *launches,
                              uint64_t *algorithmic_bytes);
/* 0: NCCL allreduce; 1: one-shot peer-memory allreduce fused into the consumer kernels */
dp_status dp_model_set_allreduce_mode(dp_model *m, int mode);

/* ---- tensor parallel group --------------------------------------------- */
/* No counterpart in the reference (it has no collective backend; only the
 * emulation schema src/config/schema/emulation.schema.js:108-143 names TP). */
dp_status dp_tp_unique_id(void *out128);                               /* ncclGetUniqueId */
dp_status dp_tp_init(dp_ctx *ctx, int rank, int size, const void *id128);
/* A group WITHOUT a communicator whose `size` exchange areas all live on this GPU and are written by
 * nobody else: for exercising the bounded waits on one GPU (rank `rank` waits for flags the absent
 * ranks never raise and gives up with DP_ERR_TIMEOUT).  Ops that need a communicator return DP_ERR_STATE. */
dp_status dp_tp_init_loopback(dp_ctx *ctx, int rank, int size);
dp_status dp_tp_allreduce_f32(dp_ctx *ctx, dp_recorder *rec, dp_buf buf, size_t offset, size_t count);
/* peer-memory exchange area: export this rank's handle, attach every rank's */
dp_status dp_tp_ipc_export(dp_ctx *ctx, void *out64);
dp_status dp_tp_ipc_attach(dp_ctx *ctx, const void *handles64_by_rank);
dp_status dp_tp_destroy(dp_ctx *ctx);

/* ---- seeded synthetic inputs (host side) --------------------------------
 * No counterpart in the reference: stand-ins for real checkpoints, which are not
 * available offline.  Counter based, so any shard can be generated on its own. */
uint64_t dp_synth_key(uint64_t seed, uint64_t tensor_id);
void dp_synth_normal_f32(uint64_t key, uint64_t first, size_t n, float sigma, float mean, float *out);
void dp_synth_normal_f16(uint64_t key, uint64_t first, size_t n, float sigma, void *out_f16);
/* Q4_K blocks: d, dmin = f16(|N(0,0.02)|), uniform 6-bit codes, uniform nibbles */
void dp_synth_q4k_blocks(uint64_t key, uint64_t first_block, size_t n_blocks, void *out);
void dp_synth_tokens(uint64_t key, size_t n, int vocab, int32_t *out);

#ifdef __cplusplus
}
#endif
#endif
