// Embedding gather, SwiGLU and small helpers.
//
// Reference counterparts: nn.Embedding (python/lyapunov_engine/models/llama.py:172,205)
// and swiglu_kernel (csrc/kernels/fused_rmsnorm_swiglu.cu:152-179).
#include "common.cuh"

LE_API const char *le_last_error() { return le::error_buffer(); }

namespace {

// One block per token: row `ids[t]` of the table goes to row t of the
// 32-bit residual stream.  An id outside the table sets the status word and
// writes zeros instead of reading out of bounds.
template <typename T>
__global__ void embed_kernel(float *__restrict__ out, const T *__restrict__ table, const int32_t *__restrict__ ids,
                             int hidden, int vocab, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int id = ids[t];
  float *dst = out + static_cast<int64_t>(t) * hidden;
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = 0.0f;
    return;
  }
  const T *src = table + static_cast<int64_t>(id) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = le::to_f32(src[i]);
}

// out[t, i] = silu(gu[t, i]) * gu[t, I + i], in 32-bit, rounded once.
template <typename T>
__global__ void swiglu_kernel(T *__restrict__ out, const T *__restrict__ gu, int64_t total, int inter) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int64_t t = idx / inter;
  const int i = static_cast<int>(idx - t * inter);
  const float g = le::to_f32(gu[t * 2 * inter + i]);
  const float u = le::to_f32(gu[t * 2 * inter + inter + i]);
  out[idx] = le::from_f32<T>(g / (1.0f + expf(-g)) * u);
}

// The same with 16-byte accesses; `inter` is a multiple of 8.
__global__ void swiglu_bf16x8_kernel(__nv_bfloat16 *__restrict__ out, const __nv_bfloat16 *__restrict__ gu, int64_t total8,
                                     int inter8) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int64_t t = idx / inter8;
  const int i = static_cast<int>(idx - t * inter8);
  const uint4 g4 = *reinterpret_cast<const uint4 *>(gu + (t * 2 * inter8 + i) * 8);
  const uint4 u4 = *reinterpret_cast<const uint4 *>(gu + (t * 2 * inter8 + inter8 + i) * 8);
  const __nv_bfloat162 *g2 = reinterpret_cast<const __nv_bfloat162 *>(&g4);
  const __nv_bfloat162 *u2 = reinterpret_cast<const __nv_bfloat162 *>(&u4);
  uint4 o4;
  __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
    o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
  }
  *reinterpret_cast<uint4 *>(out + idx * 8) = o4;
}

template <typename TO, typename TI>
__global__ void convert_kernel(TO *__restrict__ out, const TI *__restrict__ in, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = le::from_f32<TO>(le::to_f32(in[i]));
}

// One block per request of the step: a request none of whose tokens are in the
// cache yet (ctx_before == 0) gets its row of a per-request state buffer
// zeroed.  Rows that stand for no request (slot < 0) are skipped.
__global__ void zero_fresh_state_kernel(uint32_t *__restrict__ state, int64_t row_words, int num_rows,
                                        const int32_t *__restrict__ slots, const int32_t *__restrict__ ctx_before) {
  const int b = blockIdx.x;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_rows || ctx_before[b] != 0) return;
  uint32_t *row = state + static_cast<int64_t>(slot) * row_words;
  for (int64_t i = threadIdx.x; i < row_words; i += blockDim.x) row[i] = 0u;
}

}  // namespace

// How many multiprocessors the current device has (grids are sized by it).
LE_API int le_sm_count() {
  int device = 0, count = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
  return count;
}

// state: [num_rows, row_bytes] bytes, row_bytes a multiple of 4.
LE_API int le_zero_fresh_state(void *state, int64_t row_bytes, int num_rows, const int32_t *slots,
                               const int32_t *ctx_before, int num_requests, cudaStream_t stream) {
  if (num_requests <= 0 || row_bytes <= 0) return 0;
  if (row_bytes % 4) return le::invalid("le_zero_fresh_state: rows of %lld bytes are not a multiple of 4", (long long)row_bytes);
  zero_fresh_state_kernel<<<num_requests, 256, 0, stream>>>(static_cast<uint32_t *>(state), row_bytes / 4, num_rows, slots,
                                                            ctx_before);
  return le::launched();
}

LE_API int le_embed(float *out, const void *table, int table_dtype, const int32_t *ids, int num_tokens, int hidden,
                    int vocab, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  LE_DISPATCH_DTYPE(table_dtype, T,
                    return le::launch_chained(embed_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream, out,
                                              static_cast<const T *>(table), ids, hidden, vocab, status));
}

LE_API int le_swiglu(void *out, const void *gate_up, int dtype, int num_tokens, int inter, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int64_t total = static_cast<int64_t>(num_tokens) * inter;
  const int threads = 256;
  if (dtype == LE_BF16 && inter % 8 == 0) {
    const int64_t total8 = total / 8;
    const int64_t blocks8 = (total8 + threads - 1) / threads;
    if (blocks8 > 2147483647LL) return le::invalid("le_swiglu: %lld elements are too many for one launch", (long long)total);
    swiglu_bf16x8_kernel<<<static_cast<unsigned>(blocks8), threads, 0, stream>>>(
        static_cast<__nv_bfloat16 *>(out), static_cast<const __nv_bfloat16 *>(gate_up), total8, inter / 8);
    return le::launched();
  }
  const int64_t blocks = (total + threads - 1) / threads;
  if (blocks > 2147483647LL) return le::invalid("le_swiglu: %lld elements are too many for one launch", (long long)total);
  LE_DISPATCH_DTYPE(dtype, T,
                    swiglu_kernel<T><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
                        static_cast<T *>(out), static_cast<const T *>(gate_up), total, inter));
  return le::launched();
}

// out (f32) = in (bf16) or out (bf16) = in (f32).
LE_API int le_convert(void *out, int out_dtype, const void *in, int in_dtype, int64_t n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n + threads - 1) / threads);
  if (out_dtype == LE_F32 && in_dtype == LE_BF16)
    convert_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>(static_cast<float *>(out), static_cast<const __nv_bfloat16 *>(in), n);
  else if (out_dtype == LE_BF16 && in_dtype == LE_F32)
    convert_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>(static_cast<__nv_bfloat16 *>(out), static_cast<const float *>(in), n);
  else
    return le::invalid("le_convert: unsupported pair of dtypes %d -> %d", in_dtype, out_dtype);
  return le::launched();
}
