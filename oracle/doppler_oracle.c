/*
 * CPU oracle for the Doppler Q4_K quantized-inference hot path (see the header
 * for what this is and is not).  TEST INFRASTRUCTURE ONLY.
 *
 * Every function follows a named piece of the reference's own CPU code and
 * keeps its evaluation order: JavaScript numbers are doubles, Float32Array
 * stores round to f32, Math.round is round-half-up.
 */
#include "doppler_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* helpers                                                                   */
/* ------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* JavaScript Math.round: nearest integer, halves toward +infinity. */
static inline double js_round(double x) {
  double r = floor(x);
  if (x - r >= 0.5) r += 1.0;
  return r;
}

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; a timed baseline sets the
 * team size itself. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------ */
/* f16 <-> f32                                                               */
/* ------------------------------------------------------------------------ */

/* src/converter/quantizer.js:15-46 */
uint16_t orc_f32_to_f16_trunc(double value) {
  uint32_t f = f32_bits((float)value);
  uint32_t sign = (f >> 31) & 1u;
  int exp = (int)((f >> 23) & 0xffu);
  uint32_t frac = f & 0x7fffffu;
  if (exp == 0xff) return (uint16_t)((sign << 15) | 0x7c00u | (frac ? 0x200u : 0u));
  if (exp == 0) return (uint16_t)(sign << 15);
  exp = exp - 127 + 15;
  if (exp >= 31) return (uint16_t)((sign << 15) | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)(sign << 15);
    frac = (frac | 0x800000u) >> (1 - exp);
    return (uint16_t)((sign << 15) | (frac >> 13));
  }
  return (uint16_t)((sign << 15) | ((uint32_t)exp << 10) | (frac >> 13));
}

/* src/converter/quantizer.js:48-65 */
float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t frac = h & 0x3ffu;
  double v;
  if (exp == 0) {
    if (frac == 0) return sign ? -0.0f : 0.0f;
    v = ldexp((double)frac / 1024.0, -14);
  } else if (exp == 31) {
    if (frac) return NAN;
    return sign ? -INFINITY : INFINITY;
  } else {
    v = ldexp(1.0 + (double)frac / 1024.0, (int)exp - 15);
  }
  return (float)(sign ? -v : v);
}

/* src/inference/kv-cache/types.js:25-43 */
uint16_t orc_f32_to_f16_kvhost(float value) {
  uint32_t x = f32_bits(value);
  uint32_t sign = (x >> 16) & 0x8000u;
  int exp = (int)((x >> 23) & 0xffu) - 127 + 15;
  uint32_t mant = x & 0x7fffffu;
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    mant = (mant | 0x800000u) >> (1 - exp);
    return (uint16_t)(sign | ((mant + 0x1000u) >> 13));
  }
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0u));
  return (uint16_t)(sign | ((uint32_t)exp << 10) | ((mant + 0x1000u) >> 13));
}

/* IEEE-754 binary32 -> binary16, round to nearest even. */
uint16_t orc_f32_to_f16_rne(float value) {
  uint32_t x = f32_bits(value);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0u));
  if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to >= 65520 -> inf */
  if (ax < 0x33000001u) return (uint16_t)sign;               /* <= 2^-25 -> 0 */
  int e = (int)(ax >> 23) - 127;
  uint32_t m = (ax & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t hexp;
  if (e < -14) { shift = 13 + (-14 - e); hexp = 0; }
  else { shift = 13; hexp = (uint32_t)(e + 15); }
  uint32_t q = m >> shift;
  uint32_t rem = m & ((1u << shift) - 1u);
  uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) q++;
  uint32_t out;
  if (hexp == 0) out = q;                 /* subnormal; carry into exponent is natural */
  else out = ((hexp - 1u) << 10) + q;     /* q holds the implicit bit at 0x400 */
  return (uint16_t)(sign | out);
}

/* ------------------------------------------------------------------------ */
/* seeded data of the reference's test harness                               */
/* ------------------------------------------------------------------------ */

/* tests/kernels/harness/tolerance.js:110-141.  The product state*1103515245 is
 * a double product in JavaScript (it exceeds 2^53 and rounds), then & converts
 * through ToInt32; both are reproduced. */
void orc_lcg_test_data(float *out, size_t n, uint32_t seed, double lo, double hi) {
  double state = (double)seed;
  double range = hi - lo;
  for (size_t i = 0; i < n; i++) {
    double p = state * 1103515245.0;
    p = p + 12345.0;
    uint64_t t = (uint64_t)p; /* p is a non-negative integer-valued double < 2^63 */
    state = (double)(uint32_t)(t & 0x7fffffffu);
    double normalized = state / 2147483647.0;
    out[i] = (float)(lo + normalized * range);
  }
}

/* tests/kernels/fused-matmul-q4-widetile-f16a-parity.test.js:28-34 */
void orc_prng1664525(double *out, size_t n, uint32_t seed) {
  uint32_t s = seed;
  for (size_t i = 0; i < n; i++) {
    s = s * 1664525u + 1013904223u;
    out[i] = (double)s / 4294967296.0;
  }
}

/* ------------------------------------------------------------------------ */
/* Q4_K quantize / dequantize                                                */
/* ------------------------------------------------------------------------ */

/* src/converter/quantizer.js:78-166 */
void orc_q4k_quantize_block(const float *data, int valid_len, uint8_t *block) {
  float scales[8], min_offsets[8];
  uint8_t quantized[256];
  memset(block, 0, ORC_Q4K_BLOCK_BYTES);
  memset(quantized, 0, sizeof quantized);
  if (valid_len < 0) valid_len = 0;
  if (valid_len > ORC_QK_K) valid_len = ORC_QK_K;

  for (int sb = 0; sb < 8; sb++) {
    int start = sb * 32;
    int valid = valid_len - start;
    if (valid > 32) valid = 32;
    if (valid <= 0) { scales[sb] = 0; min_offsets[sb] = 0; continue; }
    double mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < valid; i++) {
      double v = data[start + i];
      if (v < mn) mn = v;
      if (v > mx) mx = v;
    }
    min_offsets[sb] = (float)(-mn);
    double range = mx - mn;
    scales[sb] = (float)(range > 0 ? range / 15.0 : 0.0);
    double inv_scale = scales[sb] > 0 ? 1.0 / (double)scales[sb] : 0.0;
    for (int i = 0; i < valid; i++) {
      double v = data[start + i];
      double q = js_round((v - mn) * inv_scale);
      if (q < 0) q = 0;
      if (q > 15) q = 15;
      quantized[start + i] = (uint8_t)q;
    }
  }

  double max_scale = 0, max_min = 0;
  for (int i = 0; i < 8; i++) {
    if (scales[i] > max_scale) max_scale = scales[i];
    if (min_offsets[i] > max_min) max_min = min_offsets[i];
    if (min_offsets[i] < 0) min_offsets[i] = 0;
  }
  double d = max_scale / 63.0;
  double dmin = max_min / 63.0;
  uint16_t dh = orc_f32_to_f16_trunc(d), dmh = orc_f32_to_f16_trunc(dmin);
  block[0] = (uint8_t)(dh & 0xff); block[1] = (uint8_t)(dh >> 8);
  block[2] = (uint8_t)(dmh & 0xff); block[3] = (uint8_t)(dmh >> 8);
  double inv_d = d > 0 ? 1.0 / d : 0.0;
  double inv_dmin = dmin > 0 ? 1.0 / dmin : 0.0;

  uint8_t sc[8], mb[8];
  for (int i = 0; i < 8; i++) {
    double s = js_round((double)scales[i] * inv_d);
    double mo = min_offsets[i] > 0 ? (double)min_offsets[i] : 0.0;
    double m = js_round(mo * inv_dmin);
    sc[i] = (uint8_t)(s < 63 ? s : 63);
    mb[i] = (uint8_t)(m < 63 ? m : 63);
  }
  for (int i = 0; i < 4; i++) {
    block[4 + i] = (uint8_t)((sc[i] & 0x3f) | (((sc[i + 4] >> 4) & 3) << 6));
    block[8 + i] = (uint8_t)((mb[i] & 0x3f) | (((mb[i + 4] >> 4) & 3) << 6));
    block[12 + i] = (uint8_t)((sc[i + 4] & 0x0f) | ((mb[i + 4] & 0x0f) << 4));
  }
  for (int chunk = 0; chunk < 4; chunk++)
    for (int i = 0; i < 32; i++)
      block[16 + chunk * 32 + i] =
          (uint8_t)((quantized[chunk * 64 + i] & 0x0f) | ((quantized[chunk * 64 + 32 + i] & 0x0f) << 4));
}

/* src/converter/quantizer.js:223-251 */
size_t orc_q4k_quantize_flat(const float *data, size_t n, uint8_t *out) {
  size_t nb = (n + ORC_QK_K - 1) / ORC_QK_K;
  float pad[ORC_QK_K];
  for (size_t b = 0; b < nb; b++) {
    size_t off = b * ORC_QK_K;
    size_t have = n - off < ORC_QK_K ? n - off : ORC_QK_K;
    if (have == ORC_QK_K) {
      orc_q4k_quantize_block(data + off, ORC_QK_K, out + b * ORC_Q4K_BLOCK_BYTES);
    } else { /* zero-padded copy, quantized as a full block */
      memset(pad, 0, sizeof pad);
      memcpy(pad, data + off, have * sizeof(float));
      orc_q4k_quantize_block(pad, ORC_QK_K, out + b * ORC_Q4K_BLOCK_BYTES);
    }
  }
  return nb;
}

/* src/converter/quantizer.js:253-288 */
size_t orc_q4k_quantize_rowwise(const float *data, size_t rows, size_t cols, uint8_t *out) {
  size_t bpr = (cols + ORC_QK_K - 1) / ORC_QK_K;
  float pad[ORC_QK_K];
  for (size_t r = 0; r < rows; r++)
    for (size_t b = 0; b < bpr; b++) {
      size_t rem = cols - b * ORC_QK_K;
      int valid = (int)(rem < ORC_QK_K ? rem : ORC_QK_K);
      /* the reference reads past the row for the invalid tail but never uses it */
      memset(pad, 0, sizeof pad);
      memcpy(pad, data + r * cols + b * ORC_QK_K, (size_t)valid * sizeof(float));
      orc_q4k_quantize_block(pad, valid, out + (r * bpr + b) * ORC_Q4K_BLOCK_BYTES);
    }
  return rows * bpr;
}

/* tools/lib/q4k-projection-reference.js:26-37 */
void orc_q4k_decode_header(const uint8_t *b, uint8_t sc[8], uint8_t mn[8], float *d, float *dmin) {
  *d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
  *dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
  for (int i = 0; i < 4; i++) {
    sc[i] = b[4 + i] & 0x3f;
    sc[i + 4] = (uint8_t)(((b[4 + i] >> 6) & 3) << 4);
    mn[i] = b[8 + i] & 0x3f;
    mn[i + 4] = (uint8_t)(((b[8 + i] >> 6) & 3) << 4);
  }
  for (int i = 0; i < 4; i++) {
    sc[i + 4] |= b[12 + i] & 0x0f;
    mn[i + 4] |= (b[12 + i] >> 4) & 0x0f;
  }
}

/* src/converter/quantizer.js:172-221 */
void orc_q4k_dequant_block(const uint8_t *b, float *out) {
  uint8_t sc[8], mn[8];
  float d, dmin, scales[8], mins[8];
  orc_q4k_decode_header(b, sc, mn, &d, &dmin);
  for (int i = 0; i < 8; i++) {
    scales[i] = (float)((double)d * (double)sc[i]);
    mins[i] = (float)((double)dmin * (double)mn[i]);
  }
  for (int chunk = 0; chunk < 4; chunk++) {
    const uint8_t *qs = b + 16 + chunk * 32;
    int s0 = chunk * 2, s1 = s0 + 1;
    for (int i = 0; i < 32; i++) {
      uint8_t byte = qs[i];
      out[chunk * 64 + i] = (float)((double)scales[s0] * (double)(byte & 0x0f) - (double)mins[s0]);
      out[chunk * 64 + 32 + i] = (float)((double)scales[s1] * (double)(byte >> 4) - (double)mins[s1]);
    }
  }
}

/* src/converter/quantizer.js:425-443 */
void orc_q4k_dequant_flat(const uint8_t *q, size_t num_blocks, size_t n, float *out) {
  float tmp[ORC_QK_K];
  for (size_t b = 0; b < num_blocks; b++) {
    size_t start = b * ORC_QK_K;
    if (start >= n) break;
    size_t len = n - start < ORC_QK_K ? n - start : ORC_QK_K;
    orc_q4k_dequant_block(q + b * ORC_Q4K_BLOCK_BYTES, tmp);
    memcpy(out + start, tmp, len * sizeof(float));
  }
}

/* src/converter/quantizer.js:445-463 */
void orc_q4k_dequant_rowwise(const uint8_t *q, size_t rows, size_t cols, float *out) {
  size_t bpr = (cols + ORC_QK_K - 1) / ORC_QK_K;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; r++)
    orc_q4k_dequant_flat(q + (size_t)r * bpr * ORC_Q4K_BLOCK_BYTES, bpr, cols, out + (size_t)r * cols);
}

/* ------------------------------------------------------------------------ */
/* matmul                                                                    */
/* ------------------------------------------------------------------------ */

/* tools/lib/q4k-projection-reference.js:84-181 */
void orc_q4k_gemv(const uint8_t *w, size_t rows, size_t cols, const float *x, float alpha, float *y) {
  size_t bpr = (cols + ORC_QK_K - 1) / ORC_QK_K;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; r++) {
    float vals[ORC_QK_K];
    double sum = 0;
    size_t off = 0;
    for (size_t b = 0; b < bpr; b++) {
      orc_q4k_dequant_block(w + ((size_t)r * bpr + b) * ORC_Q4K_BLOCK_BYTES, vals);
      size_t cnt = cols - off < ORC_QK_K ? cols - off : ORC_QK_K;
      for (size_t i = 0; i < cnt; i++) sum += (double)x[off + i] * (double)vals[i];
      off += cnt;
    }
    y[r] = (float)(alpha == 1.0f ? sum : sum * (double)alpha);
  }
}

#define ORC_MB 16
/* tests/kernels/fused-matmul-q4-widetile-f16a-parity.test.js:59-74: each
 * C[m,n] is a double sum over k in order.  Sums for different m are
 * independent, so they are carried side by side (same result, vectorisable). */
static void q4k_gemm_impl(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c, int f16_weights);

void orc_q4k_gemm(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c) {
  if (m == 1) { orc_q4k_gemv(w, n, k, a, alpha, c); return; } /* same sum, same order */
  q4k_gemm_impl(w, n, k, a, m, alpha, c, 0);
}

/* The reference's opt-in tiled prefill kernel, src/gpu/kernels/fused_matmul_q4_prefill_tiled_f16.wgsl:
 * every dequantised weight is rounded to f16 when it is staged (:196-201, tileB[slot] = f16(w)) and widened
 * again for the multiply (:226-229); sums as above. */
void orc_q4k_gemm_f16_weights(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c) {
  q4k_gemm_impl(w, n, k, a, m, alpha, c, 1);
}

static void q4k_gemm_impl(const uint8_t *w, size_t n, size_t k, const float *a, size_t m, float alpha, float *c, int f16_weights) {
  size_t bpr = (k + ORC_QK_K - 1) / ORC_QK_K;
  size_t mp = (m + ORC_MB - 1) / ORC_MB * ORC_MB;
  /* A transposed to [k][mp] so that the m-lanes are contiguous */
  float *at = (float *)calloc(k * mp, sizeof(float));
  for (size_t i = 0; i < m; i++)
    for (size_t j = 0; j < k; j++) at[j * mp + i] = a[i * k + j];
#pragma omp parallel
  {
    float *row = (float *)malloc(bpr * ORC_QK_K * sizeof(float));
#pragma omp for schedule(dynamic, 8)
    for (long r = 0; r < (long)n; r++) {
      for (size_t b = 0; b < bpr; b++)
        orc_q4k_dequant_block(w + ((size_t)r * bpr + b) * ORC_Q4K_BLOCK_BYTES, row + b * ORC_QK_K);
      if (f16_weights)
        for (size_t kk = 0; kk < bpr * ORC_QK_K; kk++) row[kk] = orc_f16_to_f32(orc_f32_to_f16_rne(row[kk]));
      for (size_t m0 = 0; m0 < mp; m0 += ORC_MB) {
        double acc[ORC_MB];
        for (int j = 0; j < ORC_MB; j++) acc[j] = 0;
        for (size_t kk = 0; kk < k; kk++) {
          double wv = row[kk];
          const float *ap = at + kk * mp + m0;
          for (int j = 0; j < ORC_MB; j++) acc[j] += (double)ap[j] * wv;
        }
        for (int j = 0; j < ORC_MB && m0 + j < m; j++)
          c[(m0 + j) * n + r] = (float)(alpha == 1.0f ? acc[j] : acc[j] * (double)alpha);
      }
    }
    free(row);
  }
  free(at);
}

/* all 65536 f16 codes decoded once with orc_f16_to_f32 (same values, faster inner loops) */
static float *f16_table(void) {
  static float *tbl = NULL;
#pragma omp critical(orc_f16_table)
  {
    if (!tbl) {
      float *t = (float *)malloc(65536 * sizeof(float));
      for (uint32_t i = 0; i < 65536; i++) t[i] = orc_f16_to_f32((uint16_t)i);
      tbl = t;
    }
  }
  return tbl;
}

/* tools/lib/q4k-projection-reference.js:183-209 */
void orc_f16_gemv(const uint16_t *w, size_t rows, size_t cols, const float *x, float *y) {
  const float *tbl = f16_table();
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; r++) {
    double sum = 0;
    const uint16_t *wr = w + (size_t)r * cols;
    for (size_t c = 0; c < cols; c++) sum += (double)x[c] * (double)tbl[wr[c]];
    y[r] = (float)sum;
  }
}

/* ------------------------------------------------------------------------ */
/* attention                                                                 */
/* ------------------------------------------------------------------------ */

/* tests/kernels/reference/attention.js:4-63 (one head, one query row) */
static void attention_row(const float *qrow, const float *kf, const uint16_t *kh, const float *vf,
                          const uint16_t *vh, int kv_len, int kv_stride, int head_dim,
                          const float *mask_row, int causal_limit, double scale, float *scores,
                          float *out) {
  const float *tbl = f16_table();
  for (int k = 0; k < kv_len; k++) {
    double score = 0;
    if (kf) {
      const float *kr = kf + (size_t)k * kv_stride;
      for (int d = 0; d < head_dim; d++) score += (double)qrow[d] * (double)kr[d];
    } else {
      const uint16_t *kr = kh + (size_t)k * kv_stride;
      for (int d = 0; d < head_dim; d++) score += (double)qrow[d] * (double)tbl[kr[d]];
    }
    scores[k] = (float)(score * scale);
    if (mask_row) scores[k] = (float)((double)scores[k] + (double)mask_row[k]);
    if (causal_limit >= 0 && k > causal_limit) scores[k] = -INFINITY;
  }
  double max_score = -INFINITY;
  for (int k = 0; k < kv_len; k++) max_score = fmax(max_score, (double)scores[k]);
  double sum_exp = 0;
  for (int k = 0; k < kv_len; k++) {
    scores[k] = (float)exp((double)scores[k] - max_score);
    sum_exp += (double)scores[k];
  }
  for (int k = 0; k < kv_len; k++) scores[k] = (float)((double)scores[k] / sum_exp);
  for (int d = 0; d < head_dim; d++) {
    double val = 0;
    if (vf) for (int k = 0; k < kv_len; k++) val += (double)scores[k] * (double)vf[(size_t)k * kv_stride + d];
    else for (int k = 0; k < kv_len; k++) val += (double)scores[k] * (double)tbl[vh[(size_t)k * kv_stride + d]];
    out[d] = (float)val;
  }
}

void orc_attention(const float *q, const float *k, const float *v, int seq_len, int kv_len,
                   int num_heads, int num_kv_heads, int head_dim, const float *mask,
                   double scale, float *out) {
  if (scale < 0) scale = 1.0 / sqrt((double)head_dim);
  int hpk = num_heads / num_kv_heads;
#pragma omp parallel
  {
    float *scores = (float *)malloc((size_t)(kv_len > 0 ? kv_len : 1) * sizeof(float));
#pragma omp for collapse(2) schedule(static)
    for (int h = 0; h < num_heads; h++)
      for (int s = 0; s < seq_len; s++) {
        int kvh = h / hpk;
        size_t qo = ((size_t)s * num_heads + h) * head_dim;
        attention_row(q + qo, k + (size_t)kvh * head_dim, NULL, v + (size_t)kvh * head_dim, NULL,
                      kv_len, num_kv_heads * head_dim, head_dim,
                      mask ? mask + (size_t)s * kv_len : NULL, -1, scale, scores, out + qo);
      }
    free(scores);
  }
}

void orc_attention_f16kv(const float *q, const uint16_t *k, const uint16_t *v, int seq_len,
                         int kv_len, int num_heads, int num_kv_heads, int head_dim,
                         int causal, int start_pos, double scale, float *out) {
  if (scale < 0) scale = 1.0 / sqrt((double)head_dim);
  int hpk = num_heads / num_kv_heads;
#pragma omp parallel
  {
    float *scores = (float *)malloc((size_t)(kv_len > 0 ? kv_len : 1) * sizeof(float));
#pragma omp for collapse(2) schedule(static)
    for (int h = 0; h < num_heads; h++)
      for (int s = 0; s < seq_len; s++) {
        int kvh = h / hpk;
        size_t qo = ((size_t)s * num_heads + h) * head_dim;
        int limit = causal ? start_pos + s : -1;
        attention_row(q + qo, NULL, k + (size_t)kvh * head_dim, NULL, v + (size_t)kvh * head_dim,
                      kv_len, num_kv_heads * head_dim, head_dim, NULL, limit, scale, scores, out + qo);
      }
    free(scores);
  }
}

/* ------------------------------------------------------------------------ */
/* small ops                                                                 */
/* ------------------------------------------------------------------------ */

/* tests/kernels/reference/rmsnorm.js:4-28 */
void orc_rmsnorm(const float *x, const float *w, int rows, int size, double eps, float *y) {
  for (int b = 0; b < rows; b++) {
    const float *xr = x + (size_t)b * size;
    float *yr = y + (size_t)b * size;
    double sum_sq = 0;
    for (int i = 0; i < size; i++) sum_sq += (double)xr[i] * (double)xr[i];
    double mean_sq = sum_sq / (double)size;
    double scale = 1.0 / sqrt(mean_sq + eps);
    for (int i = 0; i < size; i++) yr[i] = (float)((double)xr[i] * scale * (double)w[i]);
  }
}

/* src/inference/pipelines/text/init-rope.js:22-25,121-131 with ropeScale = 1 */
void orc_rope_tables(double theta, int rotary_dim, int max_seq, float *cos_out, float *sin_out) {
  int half = rotary_dim / 2;
  float *freqs = (float *)malloc((size_t)half * sizeof(float));
  for (int i = 0; i < half; i++) freqs[i] = (float)(1.0 / pow(theta, (double)(2 * i) / (double)rotary_dim));
  for (int pos = 0; pos < max_seq; pos++)
    for (int i = 0; i < half; i++) {
      double scaled_pos = (double)pos / 1.0;
      double angle = scaled_pos * (double)freqs[i];
      cos_out[(size_t)pos * half + i] = (float)(cos(angle) * 1.0);
      sin_out[(size_t)pos * half + i] = (float)(sin(angle) * 1.0);
    }
  free(freqs);
}

/* tests/kernels/reference/rope.js:22-49, rotaryDim = pairSpanDim = headDim */
void orc_rope(float *x, const float *cos_t, const float *sin_t, int seq_len, int num_heads,
              int head_dim, int start_pos) {
  int half = head_dim / 2;
  for (int s = 0; s < seq_len; s++) {
    int pos = s + start_pos;
    for (int h = 0; h < num_heads; h++) {
      float *xr = x + ((size_t)s * num_heads + h) * head_dim;
      for (int i = 0; i < half; i++) {
        double x0 = xr[i], x1 = xr[i + half];
        double c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
        xr[i] = (float)(x0 * c - x1 * sn);
        xr[i + half] = (float)(x0 * sn + x1 * c);
      }
    }
  }
}

/* tests/kernels/reference/silu.js:3-5,21-29 */
void orc_silu_gated(const float *gate, const float *up, size_t n, float *out) {
  for (size_t i = 0; i < n; i++) {
    double g = gate[i];
    out[i] = (float)((g / (1.0 + exp(-g))) * (double)up[i]);
  }
}

/* src/gpu/kernels/silu.wgsl:30-37,98-104 */
void orc_silu_gated_clamped(const float *gate, const float *up, size_t n, float *out) {
  for (size_t i = 0; i < n; i++) {
    double g = gate[i];
    double cl = g < -15.0 ? -15.0 : (g > 15.0 ? 15.0 : g);
    double sig = 1.0 / (1.0 + exp(-cl));
    out[i] = (float)((g * sig) * (double)up[i]);
  }
}

/* src/gpu/kernels/residual.wgsl:25-32 */
void orc_residual_add(const float *a, const float *b, size_t n, float scale, float *out) {
  for (size_t i = 0; i < n; i++) {
    float s = a[i] + b[i];
    out[i] = scale == 1.0f ? s : s * scale;
  }
}

/* src/gpu/kernels/gather_f16.wgsl:57-66 */
void orc_gather_f16(const uint16_t *table, const int32_t *ids, int n_ids, int hidden, float *out) {
  for (int t = 0; t < n_ids; t++)
    for (int i = 0; i < hidden; i++)
      out[(size_t)t * hidden + i] = orc_f16_to_f32(table[(size_t)ids[t] * hidden + i]);
}

/* src/gpu/kernels/sample.wgsl:45-53,311-408 */
int orc_argmax(const float *logits, int n, int pad_id) {
  float best = -3.402823e+38f;
  int best_i = 0;
  for (int i = 0; i < n; i++) {
    if (i == pad_id) continue;
    float v = logits[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  return best_i;
}


/* ------------------------------------------------------------------------ */
/* seeded synthetic inputs                                                   */
/* ------------------------------------------------------------------------ */
/*
 * Restatement of the library's host-side input generators (dp_synth_* in
 * doppler_b200/csrc/synth.cu), so that the CPU baseline can build the benchmark's
 * model without loading the CUDA library.  Counter based: element i of stream
 * `key` is a function of (key, i) only.  tests/test_oracle_synth.py checks that
 * both produce the same bytes.
 */
static inline uint64_t synth_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
static inline uint64_t synth_word(uint64_t key, uint64_t i) { return synth_mix64(key + i * 0x9E3779B97F4A7C15ULL); }
static inline float synth_normal(uint64_t h) { /* Box-Muller on two 24-bit uniforms, f32 arithmetic */
  const float u1 = (float)((h >> 40) + 1u) * (1.0f / 16777216.0f);
  const float u2 = (float)((h >> 16) & 0xFFFFFFu) * (1.0f / 16777216.0f);
  return sqrtf(-2.0f * logf(u1)) * cosf(6.2831853071795864f * u2);
}

uint64_t orc_synth_key(uint64_t seed, uint64_t tensor_id) { return synth_mix64(seed * 0x100000001B3ULL + tensor_id); }

void orc_synth_normal_f32(uint64_t key, uint64_t first, size_t n, float sigma, float mean, float *out) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) out[i] = mean + sigma * synth_normal(synth_word(key, first + i));
}

void orc_synth_normal_f16(uint64_t key, uint64_t first, size_t n, float sigma, uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_f16_rne(sigma * synth_normal(synth_word(key, first + i)));
}

/* d, dmin = f16(|N(0, 0.02)|); scale bytes and quants = 140 uniformly random bytes */
void orc_synth_q4k_blocks(uint64_t key, uint64_t first_block, size_t n_blocks, uint8_t *out) {
#pragma omp parallel for schedule(static)
  for (size_t b = 0; b < n_blocks; b++) {
    const uint64_t base = (first_block + b) * 20u;
    uint8_t *blk = out + b * 144u;
    const uint16_t d = orc_f32_to_f16_rne(fabsf(0.02f * synth_normal(synth_word(key, base))));
    const uint16_t dm = orc_f32_to_f16_rne(fabsf(0.02f * synth_normal(synth_word(key, base + 1))));
    memcpy(blk, &d, 2);
    memcpy(blk + 2, &dm, 2);
    uint8_t bytes[144];
    for (int j = 0; j < 18; j++) {
      const uint64_t w = synth_word(key, base + 2 + (uint64_t)j);
      memcpy(bytes + j * 8, &w, 8);
    }
    memcpy(blk + 4, bytes, 140);
  }
}

void orc_synth_tokens(uint64_t key, size_t n, int vocab, int32_t *out) {
  for (size_t i = 0; i < n; i++) out[i] = (int32_t)(synth_word(key, i) % (uint64_t)vocab);
}

/* ------------------------------------------------------------------------ */
/* whole-model oracle                                                        */
/* ------------------------------------------------------------------------ */
/*
 * Op order and rounding points of the reference's dense Qwen3-shaped text
 * pipeline (src/config/conversion/qwen3/qwen-3-embedding-0-6b-q4k-ehf16-af32.json
 * execution.decode/prefill; src/inference/pipelines/text/attention/interpreter.js
 * :340,550-568,629-657,705-717,1141-1148; ffn/standard.js:110-165,310;
 * ffn/dense.js:1459-1466): f32 activations, per-head QK RMSNorm, rotate-half
 * RoPE, K and V rounded to f16 when appended to the cache, attention reads the
 * f16 cache including the tokens just written, greedy argmax with the lower
 * index winning ties.
 */
struct orc_model {
  orc_model_cfg cfg;
  orc_layer_weights *layers;
  const uint16_t *embed, *lm_head;
  const float *final_norm;
  uint16_t **kc, **vc; /* per layer [max_seq, n_kv_heads, head_dim] f16 */
  float *rope_cos, *rope_sin;
  int cur;
  float *last_hidden;
  int last_n;
};

orc_model *orc_model_create(const orc_model_cfg *cfg, const orc_layer_weights *layers,
                            const uint16_t *embed_f16, const uint16_t *lm_head_f16,
                            const float *final_norm) {
  orc_model *m = (orc_model *)calloc(1, sizeof *m);
  m->cfg = *cfg;
  m->layers = (orc_layer_weights *)malloc((size_t)cfg->n_layers * sizeof *layers);
  memcpy(m->layers, layers, (size_t)cfg->n_layers * sizeof *layers);
  m->embed = embed_f16; m->lm_head = lm_head_f16; m->final_norm = final_norm;
  size_t kv = (size_t)cfg->max_seq * cfg->n_kv_heads * cfg->head_dim;
  m->kc = (uint16_t **)malloc((size_t)cfg->n_layers * sizeof(void *));
  m->vc = (uint16_t **)malloc((size_t)cfg->n_layers * sizeof(void *));
  for (int l = 0; l < cfg->n_layers; l++) {
    m->kc[l] = (uint16_t *)calloc(kv, 2);
    m->vc[l] = (uint16_t *)calloc(kv, 2);
  }
  size_t half = (size_t)cfg->head_dim / 2;
  m->rope_cos = (float *)malloc((size_t)cfg->max_seq * half * sizeof(float));
  m->rope_sin = (float *)malloc((size_t)cfg->max_seq * half * sizeof(float));
  orc_rope_tables((double)cfg->rope_theta, cfg->head_dim, cfg->max_seq, m->rope_cos, m->rope_sin);
  return m;
}

void orc_model_destroy(orc_model *m) {
  if (!m) return;
  for (int l = 0; l < m->cfg.n_layers; l++) { free(m->kc[l]); free(m->vc[l]); }
  free(m->kc); free(m->vc); free(m->layers); free(m->rope_cos); free(m->rope_sin);
  free(m->last_hidden); free(m);
}

void orc_model_reset(orc_model *m) { m->cur = 0; }
int orc_model_seq_len(const orc_model *m) { return m->cur; }
const float *orc_model_last_hidden(const orc_model *m) { return m->last_hidden; }

int orc_model_forward(orc_model *m, const int32_t *tokens, int n, float *margin, float *logits_out) {
  const orc_model_cfg *c = &m->cfg;
  int H = c->hidden, D = c->head_dim, NH = c->n_heads, NKV = c->n_kv_heads, I = c->inter;
  int qdim = NH * D, kvdim = NKV * D;
  if (m->cur + n > c->max_seq) return -1;
  float *h = (float *)malloc((size_t)n * H * 4), *nrm = (float *)malloc((size_t)n * H * 4);
  float *q = (float *)malloc((size_t)n * qdim * 4), *k = (float *)malloc((size_t)n * kvdim * 4);
  float *v = (float *)malloc((size_t)n * kvdim * 4), *att = (float *)malloc((size_t)n * qdim * 4);
  float *proj = (float *)malloc((size_t)n * H * 4);
  float *g = (float *)malloc((size_t)n * I * 4), *u = (float *)malloc((size_t)n * I * 4);
  float *act = (float *)malloc((size_t)n * I * 4);

  orc_gather_f16(m->embed, tokens, n, H, h);
  for (int l = 0; l < c->n_layers; l++) {
    const orc_layer_weights *w = &m->layers[l];
    orc_rmsnorm(h, w->in_norm, n, H, (double)c->eps, nrm);
    orc_q4k_gemm(w->wq, (size_t)qdim, (size_t)H, nrm, (size_t)n, 1.0f, q);
    orc_q4k_gemm(w->wk, (size_t)kvdim, (size_t)H, nrm, (size_t)n, 1.0f, k);
    orc_q4k_gemm(w->wv, (size_t)kvdim, (size_t)H, nrm, (size_t)n, 1.0f, v);
    orc_rmsnorm(q, w->q_norm, n * NH, D, (double)c->eps, q);
    orc_rmsnorm(k, w->k_norm, n * NKV, D, (double)c->eps, k);
    orc_rope(q, m->rope_cos, m->rope_sin, n, NH, D, m->cur);
    orc_rope(k, m->rope_cos, m->rope_sin, n, NKV, D, m->cur);
    for (size_t i = 0; i < (size_t)n * kvdim; i++) {
      m->kc[l][(size_t)m->cur * kvdim + i] = orc_f32_to_f16_rne(k[i]);
      m->vc[l][(size_t)m->cur * kvdim + i] = orc_f32_to_f16_rne(v[i]);
    }
    orc_attention_f16kv(q, m->kc[l], m->vc[l], n, m->cur + n, NH, NKV, D, 1, m->cur, -1.0, att);
    orc_q4k_gemm(w->wo, (size_t)H, (size_t)qdim, att, (size_t)n, 1.0f, proj);
    orc_residual_add(h, proj, (size_t)n * H, 1.0f, h);
    orc_rmsnorm(h, w->post_norm, n, H, (double)c->eps, nrm);
    orc_q4k_gemm(w->wgate, (size_t)I, (size_t)H, nrm, (size_t)n, 1.0f, g);
    orc_q4k_gemm(w->wup, (size_t)I, (size_t)H, nrm, (size_t)n, 1.0f, u);
    orc_silu_gated_clamped(g, u, (size_t)n * I, act);
    orc_q4k_gemm(w->wdown, (size_t)H, (size_t)I, act, (size_t)n, 1.0f, proj);
    orc_residual_add(h, proj, (size_t)n * H, 1.0f, h);
  }
  m->cur += n;
  free(m->last_hidden);
  m->last_hidden = (float *)malloc((size_t)n * H * 4);
  memcpy(m->last_hidden, h, (size_t)n * H * 4);
  m->last_n = n;

  float *logits = (float *)malloc((size_t)c->vocab * 4);
  orc_rmsnorm(h + (size_t)(n - 1) * H, m->final_norm, 1, H, (double)c->eps, nrm);
  orc_f16_gemv(m->lm_head, (size_t)c->vocab, (size_t)H, nrm, logits);
  int tok = orc_argmax(logits, c->vocab, -1);
  if (margin) {
    float second = -3.402823e+38f;
    for (int i = 0; i < c->vocab; i++) if (i != tok && logits[i] > second) second = logits[i];
    *margin = logits[tok] - second;
  }
  if (logits_out) memcpy(logits_out, logits, (size_t)c->vocab * 4);
  free(logits); free(h); free(nrm); free(q); free(k); free(v); free(att); free(proj); free(g); free(u); free(act);
  return tok;
}

/* Benchmark helper: put `n` positions of synthetic f16 K/V (values ~N(0,1)) into every layer's
 * cache and move the sequence there, so that a timed decode step attends over a context of n
 * tokens without an n-token prefill on the CPU. */
int orc_model_fill_kv(orc_model *m, int n, uint64_t key) {
  if (n < 0 || n > m->cfg.max_seq) return -1;
  size_t per = (size_t)n * m->cfg.n_kv_heads * m->cfg.head_dim;
  for (int l = 0; l < m->cfg.n_layers; l++) {
    orc_synth_normal_f16(key + 2u * (uint64_t)l, 0, per, 1.0f, m->kc[l]);
    orc_synth_normal_f16(key + 2u * (uint64_t)l + 1u, 0, per, 1.0f, m->vc[l]);
  }
  m->cur = n;
  return 0;
}
