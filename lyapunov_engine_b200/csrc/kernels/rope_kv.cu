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

// The same work with 16-byte accesses: one block per token walks all heads;
// a thread takes VEC consecutive dimensions of the low half together with their
// partners in the high half.  Needs rot/2 and head_dim to be multiples of VEC.
template <typename T>
struct alignas(16) Vec16 {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_vec_kernel(T *__restrict__ qkv, T *__restrict__ k_cache, T *__restrict__ v_cache,
                   const float *__restrict__ cos_sin, const int32_t *__restrict__ positions,
                   const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                   int max_blocks, int num_heads, int num_kv_heads, int head_dim, int rot, int max_pos, int page_size,
                   int num_pages, int write_kv, int *__restrict__ status) {
  constexpr int VEC = Vec16<T>::N;
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int chunks = head_dim / VEC, half_chunks = rot / 2 / VEC, rot_chunks = rot / VEC;
  const int row = (num_heads + 2 * num_kv_heads) * head_dim;
  T *x_row = qkv + static_cast<int64_t>(t) * row;
  const int half = rot / 2;
  // Work items, so that no thread idles: for every query and key head `half_chunks` pairs (a chunk of the low
  // half with its partner of the high half) and the chunks beyond the rotary width; for every value head its
  // chunks.  One pass of the block covers a token of the usual shapes.
  const int tail_chunks = chunks - rot_chunks;
  const int per_qk = half_chunks + tail_chunks;
  const int qk_items = (num_heads + (write_kv ? num_kv_heads : 0)) * per_qk;
  const int items = qk_items + (write_kv ? num_kv_heads * chunks : 0);
  // An item's one or two chunks of the token's row.  Where they lie depends on the token alone, so they are
  // asked for before the token's position, its page and its angles are known: the row's loads, the position's
  // and the request's then fly together, and the page and the angles follow as one more round, where the
  // position, the request, the page and the row used to be four rounds one after the other.
  auto fetch = [&](int item, Vec16<T> &a, Vec16<T> &b) {
    if (item < qk_items) {
      const int h = item / per_qk, j = item - h * per_qk;
      const T *x = x_row + static_cast<int64_t>(h) * head_dim;
      if (j < half_chunks) {
        a = *reinterpret_cast<const Vec16<T> *>(x + j * VEC);
        b = *reinterpret_cast<const Vec16<T> *>(x + half + j * VEC);
      } else if (h >= num_heads) {
        a = *reinterpret_cast<const Vec16<T> *>(x + (rot_chunks + j - half_chunks) * VEC);
      }
    } else {
      const int idx = item - qk_items;
      const int kvh = idx / chunks, c = idx - kvh * chunks;
      a = *reinterpret_cast<const Vec16<T> *>(x_row + static_cast<int64_t>(num_heads + num_kv_heads + kvh) * head_dim + c * VEC);
    }
  };
  int item = threadIdx.x;
  Vec16<T> a, b;
  if (item < items) fetch(item, a, b);
  const int pos = positions[t];
  const int request = write_kv ? request_of_token[t] : 0;
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_POSITION);
    return;
  }
  int64_t kv_base = -1;
  if (write_kv) {
    const int page = block_table[static_cast<int64_t>(request) * max_blocks + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
    } else {
      kv_base = (static_cast<int64_t>(page) * num_kv_heads * page_size + pos % page_size) * head_dim;
    }
  }
  const float *cs = cos_sin + static_cast<int64_t>(pos) * rot;
  while (item < items) {
    if (item < qk_items) {
      const int h = item / per_qk, j = item - h * per_qk;
      const bool is_q = h < num_heads;
      T *dst = x_row + static_cast<int64_t>(h) * head_dim;
      if (!is_q) dst = kv_base < 0 ? nullptr : k_cache + kv_base + static_cast<int64_t>(h - num_heads) * page_size * head_dim;
      if (dst != nullptr) {
        if (j < half_chunks) {
          float cc[VEC], ss[VEC];
#pragma unroll
          for (int i = 0; i < VEC; i += 4) {
            *reinterpret_cast<float4 *>(cc + i) = *reinterpret_cast<const float4 *>(cs + j * VEC + i);
            *reinterpret_cast<float4 *>(ss + i) = *reinterpret_cast<const float4 *>(cs + half + j * VEC + i);
          }
          Vec16<T> out_lo, out_hi;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float x0 = le::to_f32(a.v[i]), x1 = le::to_f32(b.v[i]);
            out_lo.v[i] = le::from_f32<T>(x0 * cc[i] - x1 * ss[i]);
            out_hi.v[i] = le::from_f32<T>(x1 * cc[i] + x0 * ss[i]);
          }
          *reinterpret_cast<Vec16<T> *>(dst + j * VEC) = out_lo;
          *reinterpret_cast<Vec16<T> *>(dst + half + j * VEC) = out_hi;
        } else if (!is_q) {
          *reinterpret_cast<Vec16<T> *>(dst + (rot_chunks + j - half_chunks) * VEC) = a;
        }
      }
    } else if (kv_base >= 0) {
      const int idx = item - qk_items;
      const int kvh = idx / chunks, c = idx - kvh * chunks;
      T *dst = v_cache + kv_base + static_cast<int64_t>(kvh) * page_size * head_dim;
      *reinterpret_cast<Vec16<T> *>(dst + c * VEC) = a;
    }
    item += blockDim.x;
    if (item < items) fetch(item, a, b);
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
  const int vec = dtype == LE_BF16 ? 8 : 4;
  if (head_dim % vec == 0 && (rot / 2) % vec == 0 && reinterpret_cast<uintptr_t>(cos_sin) % 16 == 0) {
    LE_DISPATCH_DTYPE(dtype, T,
                      return le::launch_chained(rope_kv_vec_kernel<T>, dim3(num_tokens), dim3(256), 0, stream,
                                                static_cast<T *>(qkv), static_cast<T *>(k_cache), static_cast<T *>(v_cache),
                                                cos_sin, positions, request_of_token, block_table, max_blocks, num_heads,
                                                num_kv_heads, head_dim, rot, max_pos, page_size, num_pages, write_kv, status));
  }
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
