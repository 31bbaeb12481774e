// Rotary position encoding of queries and keys, fused with the write of keys
// and values into the paged cache.
//
// For token t at absolute position p of request b, head h, pair j < rot/2:
//   o[j]         = x[j] * cos(p f_j) - x[j + rot/2] * sin(p f_j)
//   o[j + rot/2] = x[j + rot/2] * cos(p f_j) + x[j] * sin(p f_j)
// (rotate-half pairing; python/lyapunov_engine/models/llama.py:23-31).  cos and
// sin come from a 32-bit table [max_pos, rot] = cos(rot/2) || sin(rot/2), the
// rotation is 32-bit and rounded once.  Dimensions from `rot` on pass through.
// Queries are rotated in place inside the fused qkv buffer; rotated keys and
// plain values go to page block_table[b][p / page] at offset p % page of pools
// laid out [pages, kv_heads, page, head_dim].
//
// The reference's kernel of this kind (csrc/kernels/fused_rope_paged.cu:7-86)
// takes one token per request at position context_len - 1; this one takes
// every token's own position, so portions of prompts work.
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_kv_kernel(T *__restrict__ qkv, T *__restrict__ k_cache, T *__restrict__ v_cache,
                               const float *__restrict__ cos_sin, const int32_t *__restrict__ positions,
                               const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                               int max_blocks, int num_heads, int num_kv_heads, int head_dim, int rot, int max_pos,
                               int page_size, int num_pages, int write_kv, int *__restrict__ status) {
  const int t = blockIdx.x;
  const int h = blockIdx.y;  // 0..nh-1 queries, then keys, then values
  const int pos = positions[t];
  const int row = (num_heads + 2 * num_kv_heads) * head_dim;
  T *x = qkv + static_cast<int64_t>(t) * row + static_cast<int64_t>(h) * head_dim;
  const bool is_q = h < num_heads;
  const bool is_k = !is_q && h < num_heads + num_kv_heads;
  if (!is_q && !write_kv) return;
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_POSITION);
    return;
  }
  T *dst = x;
  if (!is_q) {
    const int b = request_of_token[t];
    const int page = block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
      return;
    }
    const int kvh = is_k ? h - num_heads : h - num_heads - num_kv_heads;
    T *pool = is_k ? k_cache : v_cache;
    dst = pool + ((static_cast<int64_t>(page) * num_kv_heads + kvh) * page_size + pos % page_size) * head_dim;
  }
  const int half = rot / 2;
  if (is_q || is_k) {
    const float *cs = cos_sin + static_cast<int64_t>(pos) * rot;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      const float x0 = le::to_f32(x[j]), x1 = le::to_f32(x[j + half]);
      const float c = cs[j], s = cs[half + j];
      dst[j] = le::from_f32<T>(x0 * c - x1 * s);
      dst[j + half] = le::from_f32<T>(x1 * c + x0 * s);
    }
    if (dst != x)
      for (int j = rot + threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = x[j];
  } else {
    for (int j = threadIdx.x; j < head_dim; j += blockDim.x) dst[j] = x[j];
  }
}

}  // namespace

LE_API int le_rope_kv_write(void *qkv, int dtype, void *k_cache, void *v_cache, const float *cos_sin,
                            const int32_t *positions, const int32_t *request_of_token, const int32_t *block_table,
                            int max_blocks, int num_tokens, int num_heads, int num_kv_heads, int head_dim, int rot,
                            int max_pos, int page_size, int num_pages, int write_kv, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot < 0 || rot > head_dim || rot % 2) return le::invalid("le_rope_kv_write: rotary width %d must be even and at most head_dim %d", rot, head_dim);
  if (num_heads + 2 * num_kv_heads > 65535) return le::invalid("le_rope_kv_write: too many heads for one launch");
  dim3 grid(num_tokens, num_heads + 2 * num_kv_heads);
  int threads = 32;
  while (threads < head_dim / 2 && threads < 128) threads *= 2;
  LE_DISPATCH_DTYPE(dtype, T,
                    rope_kv_kernel<T><<<grid, threads, 0, stream>>>(
                        static_cast<T *>(qkv), static_cast<T *>(k_cache), static_cast<T *>(v_cache), cos_sin, positions,
                        request_of_token, block_table, max_blocks, num_heads, num_kv_heads, head_dim, rot, max_pos,
                        page_size, num_pages, write_kv, status));
  return le::launched();
}
