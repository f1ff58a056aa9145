/*
 * CPU oracle for the Doppler Q4_K quantized-inference hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in plain C, the CPU math the
 * reference project (clocksmith/doppler, JavaScript) uses to check its own GPU
 * kernels.  Nothing in the shipped CUDA library calls into it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg load it.
 *
 * Parity pin: the reference holds no literal numeric golden vectors for this
 * path and its JavaScript cannot be executed where this is built (no JS
 * runtime), so the oracle is pinned by re-running the reference's own
 * procedural unit tests (same seeded inputs, same assertions) against these
 * functions; see tests/test_oracle_pins.py.  Every function cites the reference
 * file:line it follows.  JavaScript numbers are IEEE doubles and Float32Array
 * stores round to nearest-even, so each expression below uses double arithmetic
 * with an explicit (float) cast wherever the reference stores into a
 * Float32Array.  Build with -ffp-contract=off and without -ffast-math.
 */
#ifndef DOPPLER_ORACLE_H
#define DOPPLER_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_QK_K 256            /* src/config/schema/quantization.schema.js:5  */
#define ORC_Q4K_BLOCK_BYTES 144 /* src/config/schema/quantization.schema.js:8  */
#define ORC_K_SCALE_SIZE 12     /* src/config/schema/quantization.schema.js:20 */

/* ---- f16 <-> f32 ------------------------------------------------------- */
/* src/converter/quantizer.js:15-46 (mantissa truncation, f32 subnormals -> 0) */
uint16_t orc_f32_to_f16_trunc(double value);
/* src/converter/quantizer.js:48-65 */
float orc_f16_to_f32(uint16_t h);
/* src/inference/kv-cache/types.js:25-43 (round half up on the mantissa) */
uint16_t orc_f32_to_f16_kvhost(float value);
/* IEEE round-to-nearest-even, what a device-side f16() conversion does */
uint16_t orc_f32_to_f16_rne(float value);

/* ---- seeded test data of the reference's test harness ------------------- */
/* tests/kernels/harness/tolerance.js:110-141 (generateTestData, float32) */
void orc_lcg_test_data(float *out, size_t n, uint32_t seed, double lo, double hi);
/* tests/kernels/fused-matmul-q4-widetile-f16a-parity.test.js:28-34 (makePrng) */
void orc_prng1664525(double *out, size_t n, uint32_t seed);

/* ---- Q4_K ---------------------------------------------------------------- */
/* src/converter/quantizer.js:78-166 */
void orc_q4k_quantize_block(const float *data, int valid_len, uint8_t *block144);
/* src/converter/quantizer.js:223-251 (flat: pad to blocks of 256) */
size_t orc_q4k_quantize_flat(const float *data, size_t n, uint8_t *out);
/* src/converter/quantizer.js:253-288 (row-wise: each row padded on its own) */
size_t orc_q4k_quantize_rowwise(const float *data, size_t rows, size_t cols, uint8_t *out);
/* src/converter/quantizer.js:172-221 == tools/lib/q4k-projection-reference.js:21-58 */
void orc_q4k_dequant_block(const uint8_t *block144, float *out256);
/* src/converter/quantizer.js:425-443 */
void orc_q4k_dequant_flat(const uint8_t *q, size_t num_blocks, size_t n, float *out);
/* src/converter/quantizer.js:445-463 */
void orc_q4k_dequant_rowwise(const uint8_t *q, size_t rows, size_t cols, float *out);
/* header decode only: 8 scale codes, 8 min codes, d, dmin
 * (tools/lib/q4k-projection-reference.js:26-42) */
void orc_q4k_decode_header(const uint8_t *block144, uint8_t sc[8], uint8_t mn[8], float *d, float *dmin);

/* ---- matmul -------------------------------------------------------------- */
/* tools/lib/q4k-projection-reference.js:84-181: double accumulate in k order */
void orc_q4k_gemv(const uint8_t *w, size_t rows, size_t cols, const float *x, float alpha, float *y);
/* same math for M rows of A (f32, row-major [M,K]); C is f32 [M,N].
 * tests/kernels/fused-matmul-q4-widetile-f16a-parity.test.js:59-74 */
void orc_q4k_gemm(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c);
/* same with every dequantised weight rounded to f16 first: the reference's opt-in tiled prefill kernel,
 * src/gpu/kernels/fused_matmul_q4_prefill_tiled_f16.wgsl:196-201,226-229 */
void orc_q4k_gemm_f16_weights(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c);
/* f16-weight GEMV, tools/lib/q4k-projection-reference.js:183-209 */
void orc_f16_gemv(const uint16_t *w, size_t rows, size_t cols, const float *x, float *y);

/* ---- attention ----------------------------------------------------------- */
/* tests/kernels/reference/attention.js:4-63.  mask may be NULL; when non-NULL
 * it is additive [seq_len, kv_len].  scale < 0 selects 1/sqrt(head_dim). */
void orc_attention(const float *q, const float *k, const float *v, int seq_len, int kv_len,
                   int num_heads, int num_kv_heads, int head_dim, const float *mask,
                   double scale, float *out);
/* same with K/V held as f16 (widened exactly) and the causal rule of
 * src/gpu/kernels/attention_decode_online_f16kv.wgsl:59-66: key j is masked
 * for query i when j > start_pos + i. */
void orc_attention_f16kv(const float *q, const uint16_t *k, const uint16_t *v, int seq_len,
                         int kv_len, int num_heads, int num_kv_heads, int head_dim,
                         int causal, int start_pos, double scale, float *out);

/* ---- small ops ----------------------------------------------------------- */
/* tests/kernels/reference/rmsnorm.js:4-28 */
void orc_rmsnorm(const float *x, const float *w, int rows, int size, double eps, float *y);
/* src/inference/pipelines/text/init-rope.js:11-134 (no scaling, scale 1) */
void orc_rope_tables(double theta, int rotary_dim, int max_seq, float *cos_out, float *sin_out);
/* tests/kernels/reference/rope.js:22-49 (rotate-half, in the given span) */
void orc_rope(float *x, const float *cos_t, const float *sin_t, int seq_len, int num_heads,
              int head_dim, int start_pos);
/* tests/kernels/reference/silu.js:21-29 */
void orc_silu_gated(const float *gate, const float *up, size_t n, float *out);
/* src/gpu/kernels/silu.wgsl:30-37,98-104: sigmoid argument clamped to +-15 */
void orc_silu_gated_clamped(const float *gate, const float *up, size_t n, float *out);
/* src/gpu/kernels/residual.wgsl:25-32 */
void orc_residual_add(const float *a, const float *b, size_t n, float scale, float *out);
/* src/gpu/kernels/gather_f16.wgsl:57-66 */
void orc_gather_f16(const uint16_t *table, const int32_t *ids, int n_ids, int hidden, float *out);
/* src/gpu/kernels/sample.wgsl:45-53,311-408: lower index wins ties; pad_id < 0 = none */
int orc_argmax(const float *logits, int n, int pad_id);

/* ---- whole-model oracle (dense Qwen3-shaped decoder) ---------------------- */
typedef struct {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, inter, vocab, max_seq;
  float eps;
  float rope_theta;
} orc_model_cfg;

typedef struct {
  const uint8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown; /* packed Q4_K, row-major [N,K] */
  const float *in_norm, *post_norm, *q_norm, *k_norm;
} orc_layer_weights;

typedef struct orc_model orc_model;

orc_model *orc_model_create(const orc_model_cfg *cfg, const orc_layer_weights *layers,
                            const uint16_t *embed_f16, const uint16_t *lm_head_f16,
                            const float *final_norm);
void orc_model_destroy(orc_model *m);
void orc_model_reset(orc_model *m);
/* Run n tokens at positions [cur, cur+n); returns greedy token for the last
 * position.  margin (may be NULL) receives top1 - top2 of the logits.
 * logits_out (may be NULL) receives the vocab-sized logits row.  */
int orc_model_forward(orc_model *m, const int32_t *tokens, int n, float *margin, float *logits_out);
int orc_model_seq_len(const orc_model *m);
/* hidden state [n, hidden] after the last forward (last n tokens), for layer probes */
const float *orc_model_last_hidden(const orc_model *m);

int orc_num_threads(void);
void orc_set_num_threads(int n);

/* ---- seeded synthetic inputs (restatement of the library's dp_synth_* host generators) ---- */
uint64_t orc_synth_key(uint64_t seed, uint64_t tensor_id);
void orc_synth_normal_f32(uint64_t key, uint64_t first, size_t n, float sigma, float mean, float *out);
void orc_synth_normal_f16(uint64_t key, uint64_t first, size_t n, float sigma, uint16_t *out);
void orc_synth_q4k_blocks(uint64_t key, uint64_t first_block, size_t n_blocks, uint8_t *out);
void orc_synth_tokens(uint64_t key, size_t n, int vocab, int32_t *out);
/* benchmark helper: n positions of synthetic f16 K/V in every layer, sequence position = n */
int orc_model_fill_kv(orc_model *m, int n, uint64_t key);

#ifdef __cplusplus
}
#endif
#endif
