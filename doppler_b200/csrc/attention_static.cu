// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc while they run: a plugin that is invoked
// inside somebody else's CUDA-graph capture or from a real-time audio/render callback, a process
// whose memory is entirely owned by a framework allocator with a fixed budget, or a sandboxed
// worker that is handed buffers and a stream and nothing else.  The regular entry point
// (dp_attention) needs a context, whose buffer pool allocates the split-K scratch on demand.  This
// one takes raw device pointers and a stream, and keeps its scratch in a fixed device array that
// is part of the library image.
//
// Cost and limits, so nobody is surprised:
//  - the array (DP_STATIC_ATTN_SCRATCH_BYTES) occupies memory on EVERY GPU that loads the library,
//    from load until the process exits;
//  - a call whose split-K partials would not fit is refused with DP_ERR_UNSUPPORTED;
//  - all calls share the one array.  Each call rewrites every partial it later reads, so nothing
//    has to be cleared between calls, but two calls that overlap on the GPU (different streams, or
//    a second process is NOT affected, it has its own copy) race on it: serialise them;
//  - the first call on a device looks up the array's device address (cudaGetSymbolAddress with
//    that device current).  Make that first call outside any stream capture.
#include "common.h"

#include <cmath>
#include <string>

#define DP_STATIC_ATTN_SCRATCH_BYTES (2u << 20)

// Device-side storage.  In host code the NAME below is only a handle for the runtime, never a
// device address: it is turned into one with cudaGetSymbolAddress before any kernel sees it.
static __device__ __align__(256) float g_static_attn_scratch[DP_STATIC_ATTN_SCRATCH_BYTES / sizeof(float)];

static float *g_scratch_addr[64] = {};
static thread_local std::string g_static_err;

extern "C" const char *dp_attention_decode_static_error(void) { return g_static_err.c_str(); }
extern "C" size_t dp_attention_decode_static_max_scratch(void) { return DP_STATIC_ATTN_SCRATCH_BYTES; }

static dp_status static_fail(dp_status st, const std::string &msg) {
  g_static_err = msg;
  return st;
}

extern "C" dp_status dp_attention_decode_static(void *stream, const float *q, const void *k_f16, const void *v_f16, float *out,
                                                int batch, int num_heads, int num_kv_heads, int head_dim, int kv_len,
                                                size_t kv_batch_stride, float scale) {
  if (!q || !k_f16 || !v_f16 || !out) return static_fail(DP_ERR_INVALID, "attention (static scratch): null pointer");
  if (batch < 1 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads || head_dim < 8 || head_dim > 512 ||
      head_dim % 8 || kv_len < 0)
    return static_fail(DP_ERR_INVALID, "attention (static scratch): invalid batch/heads/headDim/kvLen");
  if (batch > 1 && (kv_batch_stride < (size_t)kv_len * num_kv_heads * head_dim || kv_batch_stride % 8))
    return static_fail(DP_ERR_INVALID, "attention (static scratch): kv_batch_stride too small or not a multiple of 8");
  if (((uintptr_t)q | (uintptr_t)k_f16 | (uintptr_t)v_f16 | (uintptr_t)out) & 15)
    return static_fail(DP_ERR_INVALID, "attention (static scratch): pointers must be 16-byte aligned");
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= 64)
    return static_fail(DP_ERR_CUDA, std::string("attention (static scratch): no current CUDA device: ") + cudaGetErrorString(e));
  if (!g_scratch_addr[device]) {
    // once per device, with that device current: the symbol's address on THIS device.  The table is
    // filled without a lock: two host threads that race here both look the address up and both
    // store the same pointer, which is harmless (an aligned pointer store is not torn).
    float *p = nullptr;
    e = cudaGetSymbolAddress((void **)&p, g_static_attn_scratch);
    if (e != cudaSuccess || !p)
      return static_fail(DP_ERR_CUDA, std::string("attention (static scratch): cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
    g_scratch_addr[device] = p;
  }
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return static_fail(DP_ERR_CUDA, std::string("attention (static scratch): ") + cudaGetErrorString(e));

  // a context object on the stack: it only carries the stream and the SM count to the launcher
  dp_ctx ctx;
  ctx.device = device;
  ctx.stream = (cudaStream_t)stream;
  ctx.sm_count = sms;
  dpk_attn_params p{};
  p.q = q;
  p.k = (const __half *)k_f16;
  p.v = (const __half *)v_f16;
  p.out = out;
  p.batch = batch; p.seq_len = 1; p.kv_len = kv_len;
  p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.head_dim = head_dim;
  p.scale = scale > 0.0f ? scale : 1.0f / sqrtf((float)head_dim);
  p.softcap = 0.0f;
  p.causal = 0; p.start_pos = 0; p.sliding_window = 0; p.kv_start = 0;
  p.kv_batch_stride = kv_batch_stride;
  p.kv_lens = nullptr;
  int splits = 1;
  const size_t need = dpk_attention_scratch_bytes(&ctx, p, &splits);
  if (need > DP_STATIC_ATTN_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof msg,
             "attention (static scratch): this call needs %zu bytes of split-K scratch, the built-in array holds %u; "
             "use dp_attention (pooled scratch) or a smaller batch",
             need, DP_STATIC_ATTN_SCRATCH_BYTES);
    return static_fail(DP_ERR_UNSUPPORTED, msg);
  }
  dp_status st = dpk_attention_with_scratch(&ctx, p, g_scratch_addr[device], splits);
  if (st != DP_OK) g_static_err = ctx.err;
  return st;
}
