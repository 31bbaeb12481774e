// Causal grouped-query attention over the paged cache on the FP32 pipes: the
// attention of the true 32-bit path and the plain twin of the tensor-core
// kernels.  One formula for every cut of the work: the query token at
// absolute position p of request b reads keys max(0, p - window + 1) .. p of
// that request through its block table, whether the step brings a whole
// prompt, a portion of two tokens or one decoded token.
//
// One block per (tile of 16 query tokens of one request, query head).  Keys
// are visited in tiles of 32 from position 0 (or the window's start) with a
// running maximum and sum (scores, softmax and the weighted sum of values are
// all 32-bit, expf); the output is rounded once.  Without a window the chain
// of operations for a token does not depend on which tokens share its tile,
// so logits are bit-for-bit the same under every cut.
//
// Reference: flash_attn_v2_fwd_kernel (csrc/kernels/flash_attn_v2.cu:13-212),
// whose mask is aligned top-left (key > query index, line 114) and whose keys
// are contiguous; and paged_attention_kernel (csrc/kernels/paged_attention.cu:9-109).
// Compiled once per head size (LE_HEAD_DIM).
#include "common.cuh"

#ifndef LE_HEAD_DIM
#error "compile with -DLE_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int HD = LE_HEAD_DIM;
constexpr int QT = 16;   // query rows per block
constexpr int KT = 32;   // keys per tile
constexpr int THREADS = 128;
constexpr int KPAD = HD + 1;

struct GenericSmem {
  float q[QT][HD];
  float k[KT][KPAD];
  float v[KT][HD];
  float s[QT][KT + 1];
};

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_generic_kernel(T *__restrict__ out, int64_t out_stride, const T *__restrict__ q, int64_t q_stride,
                         const T *__restrict__ k_cache, const T *__restrict__ v_cache,
                         const int32_t *__restrict__ block_table, int max_blocks, const int32_t *__restrict__ cu_q,
                         const int32_t *__restrict__ ctx_before, const int32_t *__restrict__ tile_request,
                         const int32_t *__restrict__ tile_q0, int num_heads, int num_kv_heads, int page_size,
                         int num_pages, int window, float scale, int *__restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  GenericSmem &sm = *reinterpret_cast<GenericSmem *>(smem_raw);

  const int tile = blockIdx.x, head = blockIdx.y;
  const int kvh = head / (num_heads / num_kv_heads);
  const int b = tile_request[tile];
  const int q0 = tile_q0[tile];
  const int q_len = cu_q[b + 1] - cu_q[b];
  const int rows = min(QT, q_len - q0);
  const int tok0 = cu_q[b] + q0;
  const int p0 = ctx_before[b] + q0;           // position of row 0
  const int p_last = p0 + rows - 1;
  const int tid = threadIdx.x;
  const int32_t *table = block_table + static_cast<int64_t>(b) * max_blocks;

  for (int i = tid; i < QT * HD; i += THREADS) {
    const int r = i / HD, d = i % HD;
    sm.q[r][d] = r < rows ? le::to_f32(q[(tok0 + r) * q_stride + head * HD + d]) : 0.0f;
  }

  const int row = tid / 8, sub = tid % 8;      // this thread's query row and its lane in the row's group of 8
  const int p_row = p0 + row;
  const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
  float m_run = -INFINITY, l_run = 0.0f;
  float acc[HD / 8];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) acc[j] = 0.0f;

  int k_begin = 0;
  if (window > 0) k_begin = max(0, p0 - window + 1) / KT * KT;

  for (int k0 = k_begin; k0 <= p_last; k0 += KT) {
    __syncthreads();
    // keys and values of this tile, one key row per group of 4 threads
    {
      const int kk = tid / 4, part = tid % 4;
      const int pos = k0 + kk;
      const bool live = pos <= p_last;
      int page = 0;
      if (live) {
        page = table[pos / page_size];
        if (page < 0 || page >= num_pages) {
          atomicOr(status, LE_STATUS_BAD_PAGE);
          page = -1;
        }
      }
      const int64_t base = live && page >= 0
                               ? ((static_cast<int64_t>(page) * num_kv_heads + kvh) * page_size + pos % page_size) * HD
                               : -1;
      for (int d = part; d < HD; d += 4) {
        sm.k[kk][d] = base >= 0 ? le::to_f32(k_cache[base + d]) : 0.0f;
        sm.v[kk][d] = base >= 0 ? le::to_f32(v_cache[base + d]) : 0.0f;
      }
    }
    __syncthreads();

    // scores of this thread's row against keys sub, sub + 8, sub + 16, sub + 24
    float s[KT / 8];
    float tile_max = -INFINITY;
#pragma unroll
    for (int c = 0; c < KT / 8; ++c) {
      const int kk = sub + 8 * c;
      const int pos = k0 + kk;
      float dot = 0.0f;
#pragma unroll 8
      for (int d = 0; d < HD; ++d) dot = fmaf(sm.q[row][d], sm.k[kk][d], dot);
      const bool seen = row < rows && pos <= p_row && pos >= lo_row;
      s[c] = seen ? dot * scale : -INFINITY;
      tile_max = fmaxf(tile_max, s[c]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
    const float m_new = fmaxf(m_run, tile_max);
    const float alpha = (m_new == -INFINITY) ? 1.0f : expf(m_run - m_new);
    float tile_sum = 0.0f;
#pragma unroll
    for (int c = 0; c < KT / 8; ++c) {
      const float p = (s[c] == -INFINITY) ? 0.0f : expf(s[c] - m_new);
      sm.s[row][sub + 8 * c] = p;
      tile_sum += p;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, o);
    l_run = l_run * alpha + tile_sum;
    m_run = m_new;
    __syncwarp();  // the 8 threads of a row live in one warp; their probabilities are written

    // weighted values: this thread owns dimensions sub, sub + 8, ...
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) acc[j] *= alpha;
    for (int kk = 0; kk < KT; ++kk) {
      const float p = sm.s[row][kk];
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) acc[j] = fmaf(p, sm.v[kk][sub + 8 * j], acc[j]);
    }
  }

  if (row < rows) {
    const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
    T *o = out + (tok0 + row) * out_stride + head * HD;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) o[sub + 8 * j] = le::from_f32<T>(acc[j] * inv);
  }
}

}  // namespace

LE_API int le_attention_head_dim() { return HD; }

// Each library keeps its own message of the last refused call.
LE_API const char *le_last_error() { return le::error_buffer(); }

// out: [T, num_heads * HD] with row stride out_stride; q: rows of stride
// q_stride holding num_heads * HD query values; caches [pages, kv_heads,
// page, HD].  tile_request / tile_q0 list the tiles of 16 query tokens.
LE_API int le_attention_generic(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *k_cache,
                                const void *v_cache, int dtype, const int32_t *block_table, int max_blocks,
                                const int32_t *cu_q, const int32_t *ctx_before, const int32_t *tile_request,
                                const int32_t *tile_q0, int num_tiles, int num_heads, int num_kv_heads, int page_size,
                                int num_pages, int window, float scale, int *status, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads) return le::invalid("le_attention_generic: %d heads do not divide into %d groups", num_heads, num_kv_heads);
  if (num_heads > 65535) return le::invalid("le_attention_generic: too many heads for one launch");
  dim3 grid(num_tiles, num_heads);
  const size_t smem = sizeof(GenericSmem);
#define LE_GO(T)                                                                                                       \
  do {                                                                                                                 \
    auto kernel = attention_generic_kernel<T>;                                                                         \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
      if (e != cudaSuccess) return le::invalid("le_attention_generic: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                                  \
    kernel<<<grid, THREADS, smem, stream>>>(static_cast<T *>(out), out_stride, static_cast<const T *>(q), q_stride,    \
                                            static_cast<const T *>(k_cache), static_cast<const T *>(v_cache),          \
                                            block_table, max_blocks, cu_q, ctx_before, tile_request, tile_q0,          \
                                            num_heads, num_kv_heads, page_size, num_pages, window, scale, status);     \
  } while (0)
  if (dtype == LE_F32) LE_GO(float);
  else if (dtype == LE_BF16) LE_GO(__nv_bfloat16);
  else return le::invalid("le_attention_generic: unknown dtype code %d", dtype);
#undef LE_GO
  return le::launched();
}
