// The small memory-bound ops on the decode path.  Each kernel cites the WGSL it
// replaces; arithmetic is f32 like the reference's.
#include "common.h"
#include "pdl.cuh"

#include <cfloat>

__device__ __forceinline__ float block_sum(float v, float *sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? sh[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;  // every thread holds the total
}

// src/gpu/kernels/rmsnorm.wgsl:119-187: y = x * (1/sqrt(mean(x^2)+eps)) * w
// (+ optional (1+w), residual added before or after the norm, output scale)
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const void *__restrict__ w, int w_f16,
                                                      const float *__restrict__ residual, int pre_residual,
                                                      float *__restrict__ residual_sum_out, float *__restrict__ y,
                                                      int size, float eps, int weight_offset, float output_scale) {
  pdl_launch();
  pdl_wait();
  __shared__ float sh[32];
  const size_t base = (size_t)blockIdx.x * size;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    float v = x[base + i];
    if (pre_residual) v += residual[base + i];
    ss = fmaf(v, v, ss);
  }
  const float total = block_sum(ss, sh);
  const float inv_rms = 1.0f / sqrtf(total / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    float v = x[base + i];
    if (pre_residual) v += residual[base + i];
    float wv = w_f16 ? __half2float(((const __half *)w)[i]) : ((const float *)w)[i];
    if (weight_offset) wv = 1.0f + wv;
    float r = v * inv_rms * wv;
    if (residual && !pre_residual) r += residual[base + i];
    if (pre_residual && residual_sum_out) residual_sum_out[base + i] = v;
    y[base + i] = r * output_scale;
  }
}

// Same op for rows of up to 4096 values (size % 4 == 0): the row is read once with 16-byte
// loads, kept in registers across the reduction, and written with 16-byte stores.
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float *__restrict__ x, const void *__restrict__ w, int w_f16,
                                                          const float *__restrict__ residual, int pre_residual,
                                                          float *__restrict__ residual_sum_out, float *__restrict__ y,
                                                          int size, float eps, int weight_offset, float output_scale) {
  pdl_launch();
  pdl_wait();
  __shared__ float sh[32];
  const size_t base = (size_t)blockIdx.x * size;
  const int n4 = size >> 2;
  float4 v[4], r[4];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int idx = threadIdx.x + i * 256;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    r[i] = v[i];
    if (idx < n4) {
      v[i] = *reinterpret_cast<const float4 *>(x + base + 4 * idx);
      if (residual) r[i] = *reinterpret_cast<const float4 *>(residual + base + 4 * idx);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    if (pre_residual) { v[i].x += r[i].x; v[i].y += r[i].y; v[i].z += r[i].z; v[i].w += r[i].w; }
    ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
  }
  const float total = block_sum(ss, sh);
  const float inv_rms = 1.0f / sqrtf(total / (float)size + eps);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int idx = threadIdx.x + i * 256;
    if (idx >= n4) continue;
    float wv[4];
    if (w_f16) {
      const __half2 *wp = reinterpret_cast<const __half2 *>((const __half *)w + 4 * idx);
      const float2 a = __half22float2(wp[0]), b = __half22float2(wp[1]);
      wv[0] = a.x; wv[1] = a.y; wv[2] = b.x; wv[3] = b.y;
    } else {
      const float4 t = *reinterpret_cast<const float4 *>((const float *)w + 4 * idx);
      wv[0] = t.x; wv[1] = t.y; wv[2] = t.z; wv[3] = t.w;
    }
    const float xv[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, rv[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float ww = weight_offset ? 1.0f + wv[j] : wv[j];
      float t = xv[j] * inv_rms * ww;
      if (residual && !pre_residual) t += rv[j];
      o[j] = t * output_scale;
    }
    if (pre_residual && residual_sum_out) *reinterpret_cast<float4 *>(residual_sum_out + base + 4 * idx) = v[i];
    *reinterpret_cast<float4 *>(y + base + 4 * idx) = make_float4(o[0], o[1], o[2], o[3]);
  }
}

dp_status dpk_rmsnorm(dp_ctx *ctx, const float *x, const void *w, bool w_f16, const float *residual, bool pre_residual,
                      float *residual_sum_out, float *y, int rows, int size, float eps, bool weight_offset,
                      float output_scale) {
  if (rows <= 0) return DP_OK;
  if (size % 4 == 0 && size >= 1024 && size <= 4096) {
    DP_LAUNCH(ctx, rmsnorm_vec_kernel, rows, 256, 0, x, w, w_f16 ? 1 : 0, residual, pre_residual ? 1 : 0, residual_sum_out,
              y, size, eps, weight_offset ? 1 : 0, output_scale);
    return DP_OK;
  }
  int threads = size >= 1024 ? 256 : (size >= 256 ? 128 : 32);
  DP_LAUNCH(ctx, rmsnorm_kernel, rows, threads, 0, x, w, w_f16 ? 1 : 0, residual, pre_residual ? 1 : 0, residual_sum_out,
            y, size, eps, weight_offset ? 1 : 0, output_scale);
  return DP_OK;
}

// src/gpu/kernels/rmsnorm_qk.wgsl:75-118: per-head RMSNorm of the Q rows and the K rows in one
// launch, in place.  One warp per row.
__global__ void __launch_bounds__(256) rmsnorm_qk_kernel(float *__restrict__ q, const float *__restrict__ qw,
                                                         float *__restrict__ k, const float *__restrict__ kw, int q_rows,
                                                         int k_rows, int head_dim, float eps, int weight_offset) {
  pdl_launch();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= q_rows + k_rows) return;
  float *p = row < q_rows ? q + (size_t)row * head_dim : k + (size_t)(row - q_rows) * head_dim;
  const float *w = row < q_rows ? qw : kw;
  float ss = 0.0f;
  for (int i = lane; i < head_dim; i += 32) { const float v = p[i]; ss = fmaf(v, v, ss); }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv_rms = 1.0f / sqrtf(ss / (float)head_dim + eps);
  for (int i = lane; i < head_dim; i += 32) {
    float wv = w[i];
    if (weight_offset) wv = 1.0f + wv;
    p[i] = p[i] * inv_rms * wv;
  }
}

dp_status dpk_rmsnorm_qk(dp_ctx *ctx, float *q, const float *qw, float *k, const float *kw, int q_rows, int k_rows,
                         int head_dim, float eps, bool weight_offset) {
  const int rows = q_rows + k_rows;
  if (rows <= 0) return DP_OK;
  DP_LAUNCH(ctx, rmsnorm_qk_kernel, (rows + 7) / 8, 256, 0, q, qw, k, kw, q_rows, k_rows, head_dim, eps,
            weight_offset ? 1 : 0);
  return DP_OK;
}

// src/gpu/kernels/rope.wgsl:62-106: in-place rotation of pairs (i, i + span/2) (rotate-half) or
// (2i, 2i+1) (interleaved) with f32 cos/sin tables [max_seq, rotary_dim/2].
__global__ void rope_kernel(float *__restrict__ x, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                            int seq_len, int num_heads, int head_dim, int rotary_dim, int pair_span, int interleaved,
                            int start_pos) {
  pdl_launch();
  pdl_wait();
  const int half = rotary_dim / 2;
  const long total = (long)seq_len * num_heads * half;
  for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const long sh = idx / half;
    const int h = (int)(sh % num_heads), s = (int)(sh / num_heads);
    const int pos = s + start_pos;
    float *p = x + ((size_t)s * num_heads + h) * head_dim;
    const int i0 = interleaved ? 2 * i : i;
    const int i1 = interleaved ? 2 * i + 1 : i + pair_span / 2;
    const float c = cos_t[(size_t)pos * half + i], sn = sin_t[(size_t)pos * half + i];
    const float x0 = p[i0], x1 = p[i1];
    p[i0] = x0 * c - x1 * sn;
    p[i1] = x0 * sn + x1 * c;
  }
}

dp_status dpk_rope(dp_ctx *ctx, float *x, const float *cos_t, const float *sin_t, int seq_len, int num_heads,
                   int head_dim, int rotary_dim, int pair_span, bool interleaved, int start_pos) {
  const long total = (long)seq_len * num_heads * (rotary_dim / 2);
  if (total <= 0) return DP_OK;
  long grid = (total + 255) / 256;
  if (grid > ctx->sm_count * 16) grid = ctx->sm_count * 16;
  DP_LAUNCH(ctx, rope_kernel, (unsigned)grid, 256, 0, x, cos_t, sin_t, seq_len, num_heads, head_dim, rotary_dim,
            pair_span, interleaved ? 1 : 0, start_pos);
  return DP_OK;
}

// src/gpu/kernels/silu.wgsl:30-37,98-104: out = silu(gate) * up, sigmoid argument clamped to +-15,
// optional SwiGLU clamp.
__global__ void silu_mul_kernel(const float *__restrict__ up, const float *__restrict__ gate, float *__restrict__ out,
                                size_t n, float clamp_max) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float g = gate[i];
    const float cl = fminf(fmaxf(g, -15.0f), 15.0f);
    const float sig = 1.0f / (1.0f + expf(-cl));
    float v = (g * sig) * up[i];
    if (clamp_max > 0.0f) v = fminf(fmaxf(v, -clamp_max), clamp_max);
    out[i] = v;
  }
}

dp_status dpk_silu_mul(dp_ctx *ctx, const float *up, const float *gate, float *out, size_t n, float clamp_max) {
  if (!n) return DP_OK;
  size_t grid = (n + 255) / 256;
  if (grid > (size_t)ctx->sm_count * 16) grid = (size_t)ctx->sm_count * 16;
  DP_LAUNCH(ctx, silu_mul_kernel, (unsigned)grid, 256, 0, up, gate, out, n, clamp_max);
  return DP_OK;
}

// src/gpu/kernels/residual.wgsl:25-32
__global__ void residual_add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                    size_t n, float scale) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float s = a[i] + b[i];
    out[i] = scale == 1.0f ? s : s * scale;
  }
}

dp_status dpk_residual_add(dp_ctx *ctx, const float *a, const float *b, float *out, size_t n, float scale) {
  if (!n) return DP_OK;
  size_t grid = (n + 255) / 256;
  if (grid > (size_t)ctx->sm_count * 16) grid = (size_t)ctx->sm_count * 16;
  DP_LAUNCH(ctx, residual_add_kernel, (unsigned)grid, 256, 0, a, b, out, n, scale);
  return DP_OK;
}

// src/gpu/kernels/gather_f16.wgsl:35-66: embedding rows f16 -> f32
__global__ void gather_f16_kernel(const int *__restrict__ ids, const __half *__restrict__ table, float *__restrict__ out,
                                  int hidden) {
  pdl_launch();
  pdl_wait();
  const int t = blockIdx.x;
  const __half *row = table + (size_t)ids[t] * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[(size_t)t * hidden + i] = __half2float(row[i]);
}

dp_status dpk_gather_f16(dp_ctx *ctx, const int *ids, const __half *table, float *out, int n_ids, int hidden) {
  if (n_ids <= 0) return DP_OK;
  DP_LAUNCH(ctx, gather_f16_kernel, n_ids, 256, 0, ids, table, out, hidden);
  return DP_OK;
}

// src/gpu/kernels/kv_cache_write_f32_to_f16.wgsl:19 (round to nearest even, like WGSL f16())
__global__ void kv_write_kernel(const float *__restrict__ src, __half *__restrict__ dst, size_t n) {
  pdl_launch();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2half_rn(src[i]);
}

dp_status dpk_kv_write(dp_ctx *ctx, const float *src, __half *dst, size_t n) {
  if (!n) return DP_OK;
  size_t grid = (n + 255) / 256;
  if (grid > (size_t)ctx->sm_count * 16) grid = (size_t)ctx->sm_count * 16;
  DP_LAUNCH(ctx, kv_write_kernel, (unsigned)grid, 256, 0, src, dst, n);
  return DP_OK;
}

// src/gpu/kernels/sample.wgsl:311-408: two-phase greedy argmax; ties go to the lower index
// (candidate_beats :45-53); pad_id is skipped.
__device__ __forceinline__ bool beats(float cv, int ci, float bv, int bi) {
  return cv > bv || (cv == bv && ci < bi);
}

#define ARGMAX_BLOCKS 256

__global__ void __launch_bounds__(256) argmax_phase1(const float *__restrict__ logits, int n, int pad_id,
                                                     float *__restrict__ vals, int *__restrict__ idxs) {
  pdl_launch();
  pdl_wait();
  float best = -3.402823e+38f;
  int bi = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (i == pad_id) continue;
    const float v = logits[i];
    if (beats(v, i, best, bi)) { best = v; bi = i; }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  sv[threadIdx.x] = best; si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s && beats(sv[threadIdx.x + s], si[threadIdx.x + s], sv[threadIdx.x], si[threadIdx.x])) {
      sv[threadIdx.x] = sv[threadIdx.x + s]; si[threadIdx.x] = si[threadIdx.x + s];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { vals[blockIdx.x] = sv[0]; idxs[blockIdx.x] = si[0]; }
}

__global__ void __launch_bounds__(256) argmax_phase2(const float *__restrict__ vals, const int *__restrict__ idxs,
                                                     int groups, int *__restrict__ out, int out_index, int index_base,
                                                     float *__restrict__ best_val_out) {
  pdl_launch();
  pdl_wait();
  __shared__ float sv[256];
  __shared__ int si[256];
  const int t = threadIdx.x;
  sv[t] = t < groups ? vals[t] : -3.402823e+38f;
  si[t] = t < groups ? idxs[t] : 0x7fffffff;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (t < s && beats(sv[t + s], si[t + s], sv[t], si[t])) { sv[t] = sv[t + s]; si[t] = si[t + s]; }
    __syncthreads();
  }
  if (t == 0) {
    out[out_index] = si[0] + index_base;
    if (best_val_out) *best_val_out = sv[0];
  }
}

// the same two phases for `rows` independent logit rows in two launches: grid (groups, rows) and (rows);
// row r uses scratch entries [r * ARGMAX_BLOCKS, (r + 1) * ARGMAX_BLOCKS)
__global__ void __launch_bounds__(256) argmax_rows_phase1(const float *__restrict__ logits, int n, size_t row_stride,
                                                          float *__restrict__ vals, int *__restrict__ idxs) {
  pdl_launch();
  pdl_wait();
  const float *row = logits + (size_t)blockIdx.y * row_stride;
  float best = -3.402823e+38f;
  int bi = 0;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float v = row[i];
    if (beats(v, i, best, bi)) { best = v; bi = i; }
  }
  __shared__ float sv[256];
  __shared__ int si[256];
  sv[threadIdx.x] = best; si[threadIdx.x] = bi;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s && beats(sv[threadIdx.x + s], si[threadIdx.x + s], sv[threadIdx.x], si[threadIdx.x])) {
      sv[threadIdx.x] = sv[threadIdx.x + s]; si[threadIdx.x] = si[threadIdx.x + s];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) { vals[blockIdx.y * ARGMAX_BLOCKS + blockIdx.x] = sv[0]; idxs[blockIdx.y * ARGMAX_BLOCKS + blockIdx.x] = si[0]; }
}

__global__ void __launch_bounds__(256) argmax_rows_phase2(const float *__restrict__ vals, const int *__restrict__ idxs, int groups,
                                                          int *__restrict__ out, int index_base, float *__restrict__ best_vals) {
  pdl_launch();
  pdl_wait();
  __shared__ float sv[256];
  __shared__ int si[256];
  const int t = threadIdx.x, r = blockIdx.x;
  sv[t] = t < groups ? vals[r * ARGMAX_BLOCKS + t] : -3.402823e+38f;
  si[t] = t < groups ? idxs[r * ARGMAX_BLOCKS + t] : 0x7fffffff;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (t < s && beats(sv[t + s], si[t + s], sv[t], si[t])) { sv[t] = sv[t + s]; si[t] = si[t + s]; }
    __syncthreads();
  }
  if (t == 0) {
    out[r] = si[0] + index_base;
    if (best_vals) best_vals[r] = sv[0];
  }
}

dp_status dpk_argmax_rows(dp_ctx *ctx, const float *logits, int n, size_t row_stride, int rows, int *out, float *scratch_vals,
                          int *scratch_idx, int index_base, float *best_vals) {
  int groups = (n + 255) / 256;
  if (groups > 64) groups = 64;  // rows x groups blocks: enough to fill the GPU from a few rows on
  if (groups < 1) groups = 1;
  DP_LAUNCH(ctx, argmax_rows_phase1, dim3((unsigned)groups, (unsigned)rows), 256, 0, logits, n, row_stride, scratch_vals, scratch_idx);
  DP_LAUNCH(ctx, argmax_rows_phase2, (unsigned)rows, 256, 0, (const float *)scratch_vals, (const int *)scratch_idx, groups, out, index_base, best_vals);
  return DP_OK;
}

dp_status dpk_argmax(dp_ctx *ctx, const float *logits, int n, int pad_id, int *out, int out_index, float *scratch_vals,
                     int *scratch_idx, int index_base, float *best_val_out) {
  int groups = (n + 255) / 256;
  if (groups > ARGMAX_BLOCKS) groups = ARGMAX_BLOCKS;
  if (groups < 1) groups = 1;
  DP_LAUNCH(ctx, argmax_phase1, groups, 256, 0, logits, n, pad_id, scratch_vals, scratch_idx);
  DP_LAUNCH(ctx, argmax_phase2, 1, 256, 0, scratch_vals, scratch_idx, groups, out, out_index, index_base, best_val_out);
  return DP_OK;
}
