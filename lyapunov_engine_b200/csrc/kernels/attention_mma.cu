// Tensor-core attention over the paged cache for bfloat16, head sizes 16..128:
//   * le_attention_prefill_bf16: portions of prompts (any number of query
//     tokens per request), FlashAttention-2 style: a block owns 128 query
//     tokens of one head, walks the keys in tiles of 64 with a running maximum
//     and sum, S = Q K^T and O += P V on mma.sync m16n8k16 with 32-bit
//     accumulators, softmax in 32 bits (exp2 with the scale folded in);
//   * le_attention_decode_bf16: single decoded tokens, the keys of a request
//     split over several blocks (flash-decoding) so that a small batch still
//     fills the GPU; the query heads of one group are the 16 rows of the MMA
//     and share every key and value that is read; partial results (32-bit
//     output, maximum, sum) go to scratch memory and le_attention_merge sums
//     them.
// Keys and values are gathered row by row through the block table with
// 16-byte cp.async copies into a swizzled shared-memory tile, several tiles in
// flight, so any page size works and a page's rows need not be adjacent.
// One formula for every cut: the query at absolute position p sees keys
// max(0, p - window + 1) .. p of its own request.
//
// Reference: flash_attn_v2.cu:13-212 (contiguous keys, scalar dot products,
// top-left mask), flash_decoding.cu:13-147 (contiguous keys, every thread
// walks the whole partition), paged_attention.cu:9-109 (one key at a time).
// Compiled once per head size (LE_HEAD_DIM).
#include "common.cuh"

#ifndef LE_HEAD_DIM
#error "compile with -DLE_HEAD_DIM=<head size>"
#endif

#if LE_HEAD_DIM <= 128

namespace {

constexpr int HD = LE_HEAD_DIM;
constexpr int CPR = HD / 8;        // 16-byte chunks per row
constexpr int KSTEPS = HD / 16;    // k-steps of S = Q K^T
constexpr int NT_O = HD / 8;       // n-tiles of the output
constexpr int BN = 64;             // keys per tile
constexpr float LOG2E = 1.4426950408889634f;

using bf16 = __nv_bfloat16;

// Element (row, 16-byte chunk) of a [rows][HD] tile lives at this chunk index:
// an XOR swizzle inside each 128-byte line so that the 8 rows one ldmatrix
// reads fall into different banks.
__device__ __forceinline__ int swizzled_chunk(int row, int chunk) {
  const int id = row * CPR + chunk;
  const int line = id >> 3, pos = id & 7;
  const int key = (CPR >= 8) ? (row & 7) : (line & 7);
  return (line << 3) | (pos ^ key);
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem, bool valid) {
  const int bytes = valid ? 16 : 0;   // zero-fill when the row is not there
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Where the rows of one kv head lie in the paged pools.
struct KvLayout {
  const bf16 *k_cache, *v_cache;
  const int32_t *table;     // this request's row of the block table
  int64_t page_stride;      // elements between pages
  int64_t head_offset;      // elements to this kv head inside a page
  int page_size, page_shift, num_pages;   // page_shift < 0: page_size is no power of two
};

// Copies keys [k0, k0 + ROWS) into a swizzled tile of ROWS rows; rows at or
// after `k_end` are zero-filled.  `threads` threads (a block or one warp) share
// the work; `tid` is the caller's index among them.
template <int ROWS>
__device__ __forceinline__ void load_kv_tile(bf16 *k_tile, bf16 *v_tile, const KvLayout &kv, int k0, int k_end, int tid,
                                             int threads, int *status) {
#pragma unroll 4
  for (int c = tid; c < ROWS * CPR; c += threads) {
    const int row = c / CPR, chunk = c % CPR;
    const int pos = k0 + row;
    bool valid = pos < k_end;
    int64_t offset = 0;
    if (valid) {
      int slot, in_page;
      if (kv.page_shift >= 0) {
        slot = pos >> kv.page_shift;
        in_page = pos & (kv.page_size - 1);
      } else {
        slot = pos / kv.page_size;
        in_page = pos - slot * kv.page_size;
      }
      const int page = kv.table[slot];
      if (page < 0 || page >= kv.num_pages) {
        atomicOr(status, LE_STATUS_BAD_PAGE);
        valid = false;
      } else {
        offset = page * kv.page_stride + kv.head_offset + in_page * HD + chunk * 8;
      }
    }
    const int dst = swizzled_chunk(row, chunk) * 8;
    cp_async16(k_tile + dst, kv.k_cache + offset, valid);
    cp_async16(v_tile + dst, kv.v_cache + offset, valid);
  }
}

// One warp copies ROWS (16 or 32) keys whose first key starts a page (pages of 1..ROWS keys,
// a power of two): each lane looks one page of the tile up and the others get
// it by shuffle, so a tile costs one block-table read per lane.
template <int ROWS>
__device__ __forceinline__ void load_kv_tile_warp(bf16 *k_tile, bf16 *v_tile, const KvLayout &kv, int k0, int k_end,
                                                  int lane, int *status) {
  const int pages_in_tile = ROWS >> kv.page_shift;
  int my_page = -1;
  if (lane < pages_in_tile && k0 + (lane << kv.page_shift) < k_end) {
    my_page = kv.table[(k0 >> kv.page_shift) + lane];
    if (my_page < 0 || my_page >= kv.num_pages) {
      atomicOr(status, LE_STATUS_BAD_PAGE);
      my_page = -1;
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS * CPR / 32; ++i) {
    const int c = lane + 32 * i;
    const int row = c / CPR, chunk = c % CPR;
    const int page = __shfl_sync(0xffffffffu, my_page, row >> kv.page_shift);
    const bool valid = page >= 0 && k0 + row < k_end;
    const int64_t offset = valid ? page * kv.page_stride + kv.head_offset + (row & (kv.page_size - 1)) * HD + chunk * 8 : 0;
    const int dst = swizzled_chunk(row, chunk) * 8;
    cp_async16(k_tile + dst, kv.k_cache + offset, valid);
    cp_async16(v_tile + dst, kv.v_cache + offset, valid);
  }
}

__device__ __forceinline__ KvLayout make_kv_layout(const bf16 *k_cache, const bf16 *v_cache, const int32_t *table, int kvh,
                                                   int num_kv_heads, int page_size, int page_shift, int num_pages) {
  KvLayout kv;
  kv.k_cache = k_cache; kv.v_cache = v_cache; kv.table = table;
  kv.page_stride = static_cast<int64_t>(num_kv_heads) * page_size * HD;
  kv.head_offset = static_cast<int64_t>(kvh) * page_size * HD;
  kv.page_size = page_size; kv.page_shift = page_shift; kv.num_pages = num_pages;
  return kv;
}

// Where each lane's ldmatrix rows lie in a swizzled tile does not change from
// tile to tile: the element offsets are computed once per kernel.
// S = Q K^T reads, per k-step and pair of 8-key n-tiles, one x4 of K.
template <int NT>
struct ScoreOffsets {
  int off[KSTEPS][NT / 2];
  __device__ __forceinline__ void init(int lane) {
    const int j = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        const int row = np * 16 + (j >> 1) * 8 + (lane & 7);
        off[ks][np] = swizzled_chunk(row, ks * 2 + (j & 1)) * 8;
      }
  }
};
// O += P V reads, per 16 keys and pair of 8-dim n-tiles, one transposed x4 of V.
template <int KK>
struct ValueOffsets {
  int off[KK][NT_O / 2];
  __device__ __forceinline__ void init(int lane) {
    const int j = lane >> 3;
#pragma unroll
    for (int kk = 0; kk < KK; ++kk)
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        const int row = kk * 16 + (j & 1) * 8 + (lane & 7);
        off[kk][np] = swizzled_chunk(row, np * 2 + (j >> 1)) * 8;
      }
  }
};

// S[16 x 8 NT] += Q[16 x HD] K^T for one warp: q fragments in registers.
template <int NT>
__device__ __forceinline__ void scores(float (&s)[NT][4], const uint32_t (&qf)[KSTEPS][4], const bf16 *k_tile,
                                       const ScoreOffsets<NT> &at) {
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, k_tile + at.off[ks][np]);
      mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
      mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
    }
  }
}

// O[16 x HD] += P[16 x 16 KK] V for one warp: probabilities as A fragments.
template <int KK>
__device__ __forceinline__ void weighted_values(float (&o)[NT_O][4], const uint32_t (&pf)[KK][4], const bf16 *v_tile,
                                                const ValueOffsets<KK> &at) {
#pragma unroll
  for (int kk = 0; kk < KK; ++kk) {
#pragma unroll
    for (int np = 0; np < NT_O / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, v_tile + at.off[kk][np]);
      mma_bf16(o[2 * np], pf[kk], b[0], b[1]);
      mma_bf16(o[2 * np + 1], pf[kk], b[2], b[3]);
    }
  }
}

// ---------------------------------------------------------------- prefill
constexpr int PF_BM = 128;          // query tokens per block
constexpr int PF_WARPS = PF_BM / 16;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_STAGES = 2;

__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(bf16 *__restrict__ out, int64_t out_stride, const bf16 *__restrict__ q, int64_t q_stride,
                         const bf16 *__restrict__ k_cache, const bf16 *__restrict__ v_cache,
                         const int32_t *__restrict__ block_table, int max_blocks, const int32_t *__restrict__ cu_q,
                         const int32_t *__restrict__ ctx_before, const int32_t *__restrict__ tile_request,
                         const int32_t *__restrict__ tile_q0, int num_heads, int num_kv_heads, int page_size,
                         int page_shift, int num_pages, int window, float scale, int *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16 *q_tile = reinterpret_cast<bf16 *>(smem_raw);
  bf16 *k_tiles = q_tile + PF_BM * HD;
  bf16 *v_tiles = k_tiles + PF_STAGES * BN * HD;

  // later tiles of a prompt see more keys and take longer: start them first
  const int tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;   // the tile is the slow index: the first wave holds the long blocks
  const int kvh = head / (num_heads / num_kv_heads);
  const int b = tile_request[tile];
  const int q0 = tile_q0[tile];
  const int q_len = cu_q[b + 1] - cu_q[b];
  const int rows = min(PF_BM, q_len - q0);
  const int tok0 = cu_q[b] + q0;
  const int p0 = ctx_before[b] + q0;
  const int p_last = p0 + rows - 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int32_t *table = block_table + static_cast<int64_t>(b) * max_blocks;

  // queries of this tile (rows beyond the request's tokens are zero and are never stored)
  for (int c = tid; c < PF_BM * CPR; c += PF_THREADS) {
    const int row = c / CPR, chunk = c % CPR;
    const bool valid = row < rows;
    const bf16 *src = q + (tok0 + (valid ? row : 0)) * q_stride + head * HD + chunk * 8;
    cp_async16(q_tile + swizzled_chunk(row, chunk) * 8, src, valid);
  }
  int k_begin = 0;
  if (window > 0) k_begin = max(0, p0 - window + 1) / BN * BN;
  const int k_end = p_last + 1;
  const int num_tiles = (k_end - k_begin + BN - 1) / BN;

  const KvLayout kv = make_kv_layout(k_cache, v_cache, table, kvh, num_kv_heads, page_size, page_shift, num_pages);
  load_kv_tile<BN>(k_tiles, v_tiles, kv, k_begin, k_end, tid, PF_THREADS, status);
  cp_async_commit();

  uint32_t qf[KSTEPS][4];
  ScoreOffsets<BN / 8> k_at;
  ValueOffsets<BN / 16> v_at;
  k_at.init(lane);
  v_at.init(lane);
  float o[NT_O][4];
#pragma unroll
  for (int nt = 0; nt < NT_O; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
  // running maximum in units of the raw score, running sum; rows g and g + 8 of this warp
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const float sl2 = scale * LOG2E;
  const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
  const int p_row[2] = {p0 + row_lo, p0 + row_hi};
  const int lo_row[2] = {window > 0 ? max(0, p_row[0] - window + 1) : 0, window > 0 ? max(0, p_row[1] - window + 1) : 0};
  // what this warp's 16 rows can see at all
  const int warp_p_first = p0 + warp * 16, warp_p_last = warp_p_first + 15;
  const int warp_lo_first = window > 0 ? max(0, warp_p_first - window + 1) : 0;
  const int warp_lo_last = window > 0 ? max(0, warp_p_last - window + 1) : 0;

  for (int it = 0; it < num_tiles; ++it) {
    const int k0 = k_begin + it * BN;
    const int stage = it % PF_STAGES;
    if (it + 1 < num_tiles) {
      const int next = (it + 1) % PF_STAGES;
      load_kv_tile<BN>(k_tiles + next * BN * HD, v_tiles + next * BN * HD, kv, k0 + BN, k_end, tid, PF_THREADS, status);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) {
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int j = lane >> 3;
        const int row = warp * 16 + (j & 1) * 8 + (lane & 7);
        ldmatrix_x4(qf[ks], q_tile + swizzled_chunk(row, ks * 2 + (j >> 1)) * 8);
      }
    }
    // a warp skips tiles none of its rows can see (all keys after its last row, or all before its window)
    const bool visible = k0 <= warp_p_last && k0 + BN - 1 >= warp_lo_first;
    if (visible) {
      const bf16 *k_tile = k_tiles + stage * BN * HD, *v_tile = v_tiles + stage * BN * HD;
      float s[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
      scores<BN / 8>(s, qf, k_tile, k_at);
      // only tiles that cross the causal diagonal or the window's edge need the mask
      const bool needs_mask = k0 + BN - 1 > warp_p_first || k0 < warp_lo_last;
      if (needs_mask) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const int pos = k0 + nt * 8 + 2 * t + (e & 1);
            if (pos > p_row[r] || pos < lo_row[r]) s[nt][e] = -INFINITY;
          }
        }
      }
      float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        tile_max[0] = fmaxf(tile_max[0], fmaxf(s[nt][0], s[nt][1]));
        tile_max[1] = fmaxf(tile_max[1], fmaxf(s[nt][2], s[nt][3]));
      }
      float alpha[2], neg_m[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float m_new = fmaxf(m_run[r], tile_max[r]);
        alpha[r] = (m_new == -INFINITY) ? 1.0f : le::fast_exp2((m_run[r] - m_new) * sl2);
        neg_m[r] = (m_new == -INFINITY) ? 0.0f : -m_new * sl2;
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = le::fast_exp2(fmaf(s[nt][e], sl2, neg_m[e >> 1]));   // exp2(-inf) = 0 for masked keys
          s[nt][e] = p;
          l_run[e >> 1] += p;
        }
      }
      uint32_t pf[BN / 16][4];
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        pf[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pf[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pf[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      }
#pragma unroll
      for (int nt = 0; nt < NT_O; ++nt) {
        o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
        o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
      }
      weighted_values<BN / 16>(o, pf, v_tile, v_at);
    }
    __syncthreads();   // everyone is done with this stage before it is filled again
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const float inv[2] = {l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if ((r ? row_hi : row_lo) >= rows) continue;
    bf16 *dst = out + (tok0 + (r ? row_hi : row_lo)) * out_stride + head * HD;
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
      *reinterpret_cast<uint32_t *>(dst + nt * 8 + 2 * t) = pack_bf16(o[nt][2 * r] * inv[r], o[nt][2 * r + 1] * inv[r]);
    }
  }
}

// ---------------------------------------------------------------- decode
constexpr int DC_MAX_CLUSTER = 16;                // the most splits a cluster of blocks merges by itself
constexpr int DC_WARPS = 4;
constexpr int DC_THREADS = DC_WARPS * 32;
// Keys per warp and pipeline stage.  16 for the large heads: a block's stages are then 96 KB whatever the head
// size, two blocks fit a multiprocessor, and every scheduler has two warps to switch between (with one, the
// dependent instructions of a tile, some thousand per warp at head 128, run at their full latency: 2.4 us a tile).
constexpr int DC_TILE_DEFAULT = HD > 64 ? 16 : 32;
constexpr int DC_STAGES = 3;                      // stages per warp
constexpr int dc_warp_smem(int tile) { return DC_STAGES * 2 * tile * HD; }   // bf16 elements per warp

// One block per (split of the keys, kv head, request).  Its four warps take
// the split's tiles of 32 keys in turn, each with a cp.async pipeline of its
// own (no block barrier inside the loop), and keep their own running maximum,
// sum and output; these are merged through shared memory at the end and
// written as the split's partial result (or, with one split, as the result).
// Scratch per (request, head, split): HD floats of unnormalised output, then
// the maximum (in log2 units) and the sum.
template <int DC_TILE>
__global__ void __launch_bounds__(DC_THREADS)
attention_decode_kernel(bf16 *__restrict__ out, int64_t out_stride, float *__restrict__ part_o, float *__restrict__ part_ml,
                        const bf16 *__restrict__ q, int64_t q_stride, const bf16 *__restrict__ k_cache,
                        const bf16 *__restrict__ v_cache, const int32_t *__restrict__ block_table, int max_blocks,
                        const int32_t *__restrict__ cu_q, const int32_t *__restrict__ ctx_before,
                        const int32_t *__restrict__ requests, int num_heads, int num_kv_heads, int page_size,
                        int page_shift, int num_pages, int window, float scale, int num_splits, int cluster_merge,
                        int *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // (the kernel before this one wrote the queries and the newest key and value of every request; what is
  // read before wait_for_predecessor() below is older than that: the step's integers and keys of earlier steps)
  const int split = blockIdx.x;
  const int group = num_heads / num_kv_heads;
  const int row_tiles = (group + 15) / 16;
  const int kvh = blockIdx.y / row_tiles;
  const int h0 = kvh * group + (blockIdx.y % row_tiles) * 16;    // first query head of this block
  const int heads_here = min(16, kvh * group + group - h0);
  const int b = requests ? requests[blockIdx.z] : blockIdx.z;
  const int tok = cu_q[b];                                        // a decode request brings one token
  const int p = ctx_before[b];                                    // its position; keys 0 .. p
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const KvLayout kv = make_kv_layout(k_cache, v_cache, block_table + static_cast<int64_t>(b) * max_blocks, kvh,
                                     num_kv_heads, page_size, page_shift, num_pages);

  // A request at position 0 whose first page is the page that nobody owns is padding of a step of fixed shape (a
  // real request's first token has a page of its own).  Its row is left zero and the block ends at once, and with
  // it its whole cluster, which is that request's: such blocks then pass through the multiprocessors beside the
  // real ones without holding a place for longer than their launch.
  if (p == 0 && kv.table[0] == num_pages - 1) {
    const int64_t first = (static_cast<int64_t>(blockIdx.z) * num_heads + h0) * num_splits + split;
    for (int i = tid; i < heads_here * HD; i += DC_THREADS) {
      const int row = i / HD, d = i % HD;
      if (num_splits == 1 || cluster_merge) {
        if (split == 0) out[tok * out_stride + (h0 + row) * HD + d] = __float2bfloat16_rn(0.0f);
      } else {
        const int64_t slot = first + static_cast<int64_t>(row) * num_splits;
        part_o[slot * HD + d] = 0.0f;
        if (d == 0) {
          part_ml[slot * 2] = -INFINITY;
          part_ml[slot * 2 + 1] = 0.0f;
        }
      }
    }
    return;
  }
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int total = p + 1 - lo;
  int per_split = (total + num_splits - 1) / num_splits;
  per_split = (per_split + DC_TILE - 1) / DC_TILE * DC_TILE;
  const int k_begin = lo + split * per_split;
  const int k_end = min(p + 1, k_begin + per_split);
  const int tiles_in_split = k_end > k_begin ? (k_end - k_begin + DC_TILE - 1) / DC_TILE : 0;
  const int my_tiles = tiles_in_split > warp ? (tiles_in_split - warp + DC_WARPS - 1) / DC_WARPS : 0;   // tiles warp, warp+4, ...

  bf16 *my_smem = reinterpret_cast<bf16 *>(smem_raw) + warp * (DC_STAGES * 2 * DC_TILE * HD);
  auto k_stage = [&](int s) { return my_smem + s * 2 * DC_TILE * HD; };
  auto v_stage = [&](int s) { return my_smem + s * 2 * DC_TILE * HD + DC_TILE * HD; };
  auto tile_start = [&](int i) { return k_begin + (warp + i * DC_WARPS) * DC_TILE; };

  ScoreOffsets<DC_TILE / 8> k_at;
  ValueOffsets<DC_TILE / 16> v_at;
  k_at.init(lane);
  v_at.init(lane);
  // pages that divide a tile and tiles that start on a page boundary take the cheap loader
  const bool paged_tiles = page_shift >= 0 && page_size <= DC_TILE && (k_begin & (page_size - 1)) == 0;
  auto load_tile = [&](int stage, int i) {
    if (paged_tiles) load_kv_tile_warp<DC_TILE>(k_stage(stage), v_stage(stage), kv, tile_start(i), k_end, lane, status);
    else load_kv_tile<DC_TILE>(k_stage(stage), v_stage(stage), kv, tile_start(i), k_end, lane, 32, status);
  };
  // The first tiles are asked for while the kernel before this one still runs, unless they hold the key at
  // position p, which that kernel writes.
  auto older_than_this_step = [&](int i) { return tile_start(i) + DC_TILE <= p; };
  bool late = false;
#pragma unroll
  for (int s = 0; s < DC_STAGES - 1; ++s) {
    if (s < my_tiles) {
      if (older_than_this_step(s)) load_tile(s, s);
      else late = true;
    }
    cp_async_commit();
  }
  le::wait_for_predecessor();
  if (late) {                                 // (only the warps at the very end of a request's keys)
#pragma unroll
    for (int s = 0; s < DC_STAGES - 1; ++s)
      if (s < my_tiles && !older_than_this_step(s)) load_tile(s, s);
    cp_async_commit();
    cp_async_wait<0>();                       // so that the order of the groups below stays what the loop expects
  }

  // query fragments straight from global memory: rows are the group's heads
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = g + (i & 1) * 8;
      const int dim = ks * 16 + 2 * t + (i >> 1) * 8;
      qf[ks][i] = row < heads_here ? *reinterpret_cast<const uint32_t *>(q + tok * q_stride + (h0 + row) * HD + dim) : 0u;
    }
  }

  float o[NT_O][4];
#pragma unroll
  for (int nt = 0; nt < NT_O; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  const float sl2 = scale * LOG2E;
  const bool upper_rows = heads_here > 8;     // rows 8..15 of the MMA are padding for small groups

  for (int it = 0; it < my_tiles; ++it) {
    cp_async_wait<DC_STAGES - 2>();
    __syncwarp();                          // tile `it` has landed for every lane; stage of it - 1 is free
    const int nxt = it + DC_STAGES - 1;
    if (nxt < my_tiles) load_tile(nxt % DC_STAGES, nxt);
    cp_async_commit();
    const bf16 *k_tile = k_stage(it % DC_STAGES), *v_tile = v_stage(it % DC_STAGES);
    const int k0 = tile_start(it);
    float s[DC_TILE / 8][4];
#pragma unroll
    for (int nt = 0; nt < DC_TILE / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
    scores<DC_TILE / 8>(s, qf, k_tile, k_at);
    const bool full = k0 + DC_TILE <= k_end;
    if (!full) {
#pragma unroll
      for (int nt = 0; nt < DC_TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (k0 + nt * 8 + 2 * t + (e & 1) >= k_end) s[nt][e] = -INFINITY;
    }
    // softmax per row in units of the raw score; rows 8..15 only when they hold heads
    float alpha[2] = {1.0f, 1.0f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r == 1 && !upper_rows) {
#pragma unroll
        for (int nt = 0; nt < DC_TILE / 8; ++nt) s[nt][2] = s[nt][3] = 0.0f;
        continue;
      }
      float tile_max = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < DC_TILE / 8; ++nt) tile_max = fmaxf(tile_max, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
      const float m_new = fmaxf(m_run[r], tile_max);
      alpha[r] = (m_new == -INFINITY) ? 1.0f : le::fast_exp2((m_run[r] - m_new) * sl2);
      const float neg_m = (m_new == -INFINITY) ? 0.0f : -m_new * sl2;
      m_run[r] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < DC_TILE / 8; ++nt) {
        const float p0 = le::fast_exp2(fmaf(s[nt][2 * r], sl2, neg_m)), p1 = le::fast_exp2(fmaf(s[nt][2 * r + 1], sl2, neg_m));
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      l_run[r] = l_run[r] * alpha[r] + sum;
    }
    uint32_t pf[DC_TILE / 16][4];
#pragma unroll
    for (int kk = 0; kk < DC_TILE / 16; ++kk) {
      pf[kk][0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pf[kk][1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pf[kk][2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pf[kk][3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
      o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
    }
    weighted_values<DC_TILE / 16>(o, pf, v_tile, v_at);
  }
  cp_async_wait<0>();
  __syncthreads();
  le::let_successor_start();   // only the merge and the stores are left

  // merge the four warps through shared memory (the tiles are no longer needed)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float *sm_o = reinterpret_cast<float *>(smem_raw);            // [warps][16 rows][HD]
  float *sm_m = sm_o + DC_WARPS * 16 * HD;                      // [warps][16]
  float *sm_l = sm_m + DC_WARPS * 16;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
#pragma unroll
    for (int nt = 0; nt < NT_O; ++nt) {
      sm_o[(warp * 16 + row) * HD + nt * 8 + 2 * t] = o[nt][2 * r];
      sm_o[(warp * 16 + row) * HD + nt * 8 + 2 * t + 1] = o[nt][2 * r + 1];
    }
    if (t == 0) {
      sm_m[warp * 16 + row] = m_run[r];
      sm_l[warp * 16 + row] = l_run[r];
    }
  }
  __syncthreads();
  // with `cluster_merge` the splits of a (request, kv head) are the blocks of one cluster: each leaves its partial
  // result in its own shared memory, and after the cluster has met the blocks share out the heads' columns and
  // add the splits up from there, so no partial result goes through global memory and no merge kernel follows
  float *cl_o = sm_l + DC_WARPS * 16;                           // [16 rows][HD]
  float *cl_m = cl_o + 16 * HD;                                 // [16]
  float *cl_l = cl_m + 16;                                      // [16]
  for (int i = tid; i < heads_here * HD; i += DC_THREADS) {
    const int row = i / HD, d = i % HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) m = fmaxf(m, sm_m[w * 16 + row]);
    float acc = 0.0f, l = 0.0f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) {
      const float mw = sm_m[w * 16 + row];
      const float f = (mw == -INFINITY) ? 0.0f : le::fast_exp2((mw - m) * sl2);
      acc += f * sm_o[(w * 16 + row) * HD + d];
      l += f * sm_l[w * 16 + row];
    }
    const int head = h0 + row;
    if (num_splits == 1) {
      out[tok * out_stride + head * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    } else if (cluster_merge) {
      cl_o[row * HD + d] = acc;
      if (d == 0) {
        cl_m[row] = m * sl2;                  // in log2 units (-inf stays -inf)
        cl_l[row] = l;
      }
    } else {
      const int64_t slot = (static_cast<int64_t>(blockIdx.z) * num_heads + head) * num_splits + split;
      part_o[slot * HD + d] = acc;
      if (d == 0) {
        part_ml[slot * 2] = m * sl2;          // in log2 units, as the merge kernel reads it (-inf stays -inf)
        part_ml[slot * 2 + 1] = l;
      }
    }
  }
  if (num_splits > 1 && cluster_merge) {
    le::cluster_sync();
    // block `split` of the cluster takes every num_splits-th column; everything a column needs of the other
    // blocks is asked for before any of it is used (one trip through the cluster's network, not one per split)
    for (int i = tid * num_splits + split; i < heads_here * HD; i += DC_THREADS * num_splits) {
      const int row = i / HD, d = i % HD;
      float ms[DC_MAX_CLUSTER], ls[DC_MAX_CLUSTER], os[DC_MAX_CLUSTER];
#pragma unroll
      for (int s2 = 0; s2 < DC_MAX_CLUSTER; ++s2) {
        if (s2 < num_splits) {
          ms[s2] = le::cluster_peer_f32(cl_m + row, s2);
          ls[s2] = le::cluster_peer_f32(cl_l + row, s2);
          os[s2] = le::cluster_peer_f32(cl_o + row * HD + d, s2);
        } else {
          ms[s2] = -INFINITY, ls[s2] = 0.0f, os[s2] = 0.0f;
        }
      }
      float m = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < DC_MAX_CLUSTER; ++s2) m = fmaxf(m, ms[s2]);
      float acc = 0.0f, l = 0.0f;
#pragma unroll
      for (int s2 = 0; s2 < DC_MAX_CLUSTER; ++s2) {
        const float f = ms[s2] == -INFINITY ? 0.0f : le::fast_exp2(ms[s2] - m);     // a split without keys counts nothing
        acc += f * os[s2];
        l += f * ls[s2];
      }
      out[tok * out_stride + (h0 + row) * HD + d] = __float2bfloat16_rn(l > 0.0f ? acc / l : 0.0f);
    }
    le::cluster_sync();                       // nobody leaves while another still reads its shared memory
  }
}

// out[request, head] = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s
// The first warp turns the splits' (m_s, l_s) into weights, lanes side by side; then every thread adds its
// column of the partial outputs with loads that do not wait for one another.
constexpr int MERGE_MAX_SPLITS = 1024;
__global__ void attention_merge_kernel(bf16 *__restrict__ out, int64_t out_stride, const float *__restrict__ part_o,
                                       const float *__restrict__ part_ml, const int32_t *__restrict__ cu_q,
                                       const int32_t *__restrict__ requests, int num_heads, int num_splits) {
  extern __shared__ float merge_weight[];          // [num_splits], then the reciprocal of the sum
  le::let_successor_start();
  le::wait_for_predecessor();
  const int head = blockIdx.x, z = blockIdx.y;
  const int b = requests ? requests[z] : z;
  const int tok = cu_q[b];
  const int64_t base = (static_cast<int64_t>(z) * num_heads + head) * num_splits;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const float2 *ml = reinterpret_cast<const float2 *>(part_ml) + base;
    float m = -INFINITY;
    for (int s = lane; s < num_splits; s += 32) m = fmaxf(m, ml[s].x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.0f;
    for (int s = lane; s < num_splits; s += 32) {
      const float2 v = ml[s];
      const float f = v.x == -INFINITY ? 0.0f : le::fast_exp2(v.x - m);
      merge_weight[s] = f;
      l += f * v.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) merge_weight[num_splits] = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
  const float inv_l = merge_weight[num_splits];
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    const float *col = part_o + base * HD + d;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int s = 0;
    for (; s + 4 <= num_splits; s += 4) {
      float v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = col[static_cast<int64_t>(s + u) * HD];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float f = merge_weight[s + u];
        acc[u] += f != 0.0f ? f * v[u] : 0.0f;     // a split without keys left its row unwritten
      }
    }
    for (; s < num_splits; ++s) {
      const float f = merge_weight[s];
      const float v = col[static_cast<int64_t>(s) * HD];
      acc[0] += f != 0.0f ? f * v : 0.0f;
    }
    out[tok * out_stride + head * HD + d] = __float2bfloat16_rn(((acc[0] + acc[1]) + (acc[2] + acc[3])) * inv_l);
  }
}

}  // namespace

LE_API int le_attention_mma_available() { return 1; }

static int page_shift_of(int page_size) {
  for (int s = 0; s < 30; ++s)
    if ((1 << s) == page_size) return s;
  return -1;
}

LE_API int le_attention_prefill_bf16(void *out, int64_t out_stride, const void *q, int64_t q_stride, const void *k_cache,
                                     const void *v_cache, const int32_t *block_table, int max_blocks, const int32_t *cu_q,
                                     const int32_t *ctx_before, const int32_t *tile_request, const int32_t *tile_q0,
                                     int num_tiles, int num_heads, int num_kv_heads, int page_size, int num_pages,
                                     int window, float scale, int *status, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads) return le::invalid("le_attention_prefill_bf16: %d heads do not divide into %d groups", num_heads, num_kv_heads);
  if (num_heads > 65535) return le::invalid("le_attention_prefill_bf16: too many heads for one launch");
  const size_t smem = static_cast<size_t>(PF_BM + 2 * PF_STAGES * BN) * HD * sizeof(bf16);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return le::invalid("le_attention_prefill_bf16: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  }
  if (num_tiles > 65535) return le::invalid("le_attention_prefill_bf16: %d tiles of queries are too many for one launch", num_tiles);
  dim3 grid(num_heads, num_tiles);
  attention_prefill_kernel<<<grid, PF_THREADS, smem, stream>>>(
      static_cast<bf16 *>(out), out_stride, static_cast<const bf16 *>(q), q_stride, static_cast<const bf16 *>(k_cache),
      static_cast<const bf16 *>(v_cache), block_table, max_blocks, cu_q, ctx_before, tile_request, tile_q0, num_heads,
      num_kv_heads, page_size, page_shift_of(page_size), num_pages, window, scale, status);
  return le::launched();
}

// Floats of scratch the decode kernel needs for `num_requests` requests.
LE_API int64_t le_attention_decode_scratch_floats(int num_requests, int num_heads, int num_splits) {
  return num_splits <= 1 ? 0 : static_cast<int64_t>(num_requests) * num_heads * num_splits * (HD + 2);
}

// Up to this many splits are merged inside the attention kernel, by the blocks of a thread-block cluster;
// beyond it the partial results go through scratch memory to a merge kernel.  By default up to 8 (clusters of
// 16 need the non-portable size and were slower than the merge kernel at batches of 1 and 2);
// LYAPUNOV_CLUSTER_MERGE=<n> sets another limit up to 16, 0 switches it off.


// LYAPUNOV_DECODE_SMALL_TILES=0: the tile of the head size in every case.
static bool small_tiles_enabled() {
  static const bool on = [] {
    const char *env = getenv("LYAPUNOV_DECODE_SMALL_TILES");
    return env == nullptr || env[0] != '0';
  }();
  return on;
}

static size_t decode_smem_bytes(int tile = DC_TILE_DEFAULT) {
  size_t smem = static_cast<size_t>(DC_WARPS) * dc_warp_smem(tile) * sizeof(bf16);
  // the warps' partial results, and behind them the block's own for the merge across a cluster
  const size_t merge = static_cast<size_t>(DC_WARPS * 16 * HD + 2 * DC_WARPS * 16 + 16 * HD + 32) * sizeof(float);
  return merge > smem ? merge : smem;
}

// The decode kernel with tiles of TILE keys: what the device holds of it and how it is launched.
template <int TILE>
struct DecodeForm {
  static size_t smem() { return decode_smem_bytes(TILE); }
  // the kernel may ask for its shared memory (done once)
  static bool ready() {
    static const bool ok = smem() <= 48 * 1024 ||
                           cudaFuncSetAttribute(attention_decode_kernel<TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                static_cast<int>(smem())) == cudaSuccess;
    if (!ok) cudaGetLastError();
    return ok;
  }
  // Clusters of `num_splits` blocks that the device holds at once; 0 if it takes none.
  static int clusters_resident(int num_splits) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(num_splits, 1, 1);
    config.blockDim = dim3(DC_THREADS);
    config.dynamicSmemBytes = smem();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(num_splits);
    attr[0].val.clusterDim.y = attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    const bool ok = cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel<TILE>, &config) == cudaSuccess;
    cudaGetLastError();                                    // a refusal is an answer, not an error of the caller
    return ok && clusters > 0 ? clusters : 0;
  }
  // Clusters the device holds at once where the splits run as one cluster that merges by itself, else 0 (asked of
  // the device once per size).
  static int cluster_count(int num_splits) {
    static const int limit = [] {
      const char *env = getenv("LYAPUNOV_CLUSTER_MERGE");
      const int n = env == nullptr ? 8 : atoi(env);
      return n < 0 ? 0 : (n > DC_MAX_CLUSTER ? DC_MAX_CLUSTER : n);
    }();
    if (num_splits < 2 || num_splits > limit || !ready()) return 0;
    static int known[DC_MAX_CLUSTER + 1] = {};            // 0: not asked yet, > 0: clusters resident, -1: does not fit
    if (known[num_splits] == 0) {
      bool fits = true;
      if (num_splits > 8)
        fits = cudaFuncSetAttribute(attention_decode_kernel<TILE>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
      const int clusters = fits ? clusters_resident(num_splits) : 0;
      cudaGetLastError();                                  // a refusal above is an answer, not an error of the caller
      known[num_splits] = clusters > 0 ? clusters : -1;
    }
    return known[num_splits] > 0 ? known[num_splits] : 0;
  }
  static bool cluster_fits(int num_splits) { return cluster_count(num_splits) > 0; }
  // Blocks the device holds at once when the keys are cut `num_splits` ways: whole clusters where the splits run
  // as a cluster (clusters stay inside one part of the chip, so fewer blocks fit than the multiprocessors' shared
  // memory alone would take), single blocks otherwise.  0 if the device could not be asked.
  static int64_t blocks_resident(int num_splits) {
    if (!ready()) return 0;
    if (const int clusters = cluster_count(num_splits)) return static_cast<int64_t>(num_splits) * clusters;
    static const int64_t single = [] {
      int device = 0, sms = 0, per_sm = 0;
      if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<TILE>, DC_THREADS, smem()) != cudaSuccess) {
        cudaGetLastError();
        return int64_t{0};
      }
      return static_cast<int64_t>(sms) * per_sm;
    }();
    return single;
  }
  static int launch(dim3 grid, cudaStream_t stream, void *out, int64_t out_stride, float *scratch, const void *q, int64_t q_stride,
                    const void *k_cache, const void *v_cache, const int32_t *block_table, int max_blocks, const int32_t *cu_q,
                    const int32_t *ctx_before, const int32_t *requests, int num_requests, int num_heads, int num_kv_heads,
                    int page_size, int num_pages, int window, float scale, int num_splits, int *status) {
    if (!ready()) return le::invalid("le_attention_decode_bf16: cannot get %zu bytes of shared memory", smem());
    if (cluster_fits(num_splits)) {
      // the splits of a (request, kv head) as one cluster: merged through shared memory, no scratch, no second kernel
      return le::launch_chained_cluster(attention_decode_kernel<TILE>, grid, dim3(DC_THREADS), smem(), stream, num_splits,
                                        static_cast<bf16 *>(out), out_stride, static_cast<float *>(nullptr),
                                        static_cast<float *>(nullptr), static_cast<const bf16 *>(q), q_stride,
                                        static_cast<const bf16 *>(k_cache), static_cast<const bf16 *>(v_cache), block_table,
                                        max_blocks, cu_q, ctx_before, requests, num_heads, num_kv_heads, page_size,
                                        page_shift_of(page_size), num_pages, window, scale, num_splits, 1, status);
    }
    if (num_splits > 1 && scratch == nullptr) return le::invalid("le_attention_decode_bf16: splitting the keys %d ways needs scratch memory", num_splits);
    if (reinterpret_cast<uintptr_t>(scratch) % 8) return le::invalid("le_attention_decode_bf16: the scratch memory must start on an 8-byte boundary");
    float *part_o = scratch;
    float *part_ml = scratch ? scratch + static_cast<int64_t>(num_requests) * num_heads * num_splits * HD : nullptr;
    int rc = le::launch_chained(attention_decode_kernel<TILE>, grid, dim3(DC_THREADS), smem(), stream, static_cast<bf16 *>(out), out_stride,
                                part_o, part_ml, static_cast<const bf16 *>(q), q_stride, static_cast<const bf16 *>(k_cache),
                                static_cast<const bf16 *>(v_cache), block_table, max_blocks, cu_q, ctx_before, requests, num_heads,
                                num_kv_heads, page_size, page_shift_of(page_size), num_pages, window, scale, num_splits, 0, status);
    if (rc != 0 || num_splits == 1) return rc;
    dim3 mgrid(num_heads, num_requests);
    return le::launch_chained(attention_merge_kernel, mgrid, dim3(HD < 32 ? 32 : (HD > 128 ? 128 : HD)),
                              (static_cast<size_t>(num_splits) + 1) * sizeof(float), stream,
                              static_cast<bf16 *>(out), out_stride, static_cast<const float *>(part_o),
                              static_cast<const float *>(part_ml), cu_q, requests, num_heads, num_splits);
  }
};

// Where even the unsplit blocks of the usual form (32-key tiles at head sizes up to 64) are more than the device
// holds at once, the form with 16-key tiles runs instead: its blocks are half as large, twice as many are resident,
// the waves are finer and the ends of some blocks overlap the streaming of others (64 requests of Llama-3.2-1B
// shapes: 2.28 -> 2.22 ms a step; 80 requests, the keys cut in three: 3.24 -> 2.82 ms).  With fewer blocks it is
// slower: a block alone takes longer per key.  (`blocks`: before splitting.)
static bool small_form(int64_t blocks) {
  if constexpr (DC_TILE_DEFAULT != 32) return false;
  if (!small_tiles_enabled()) return false;
  return blocks > DecodeForm<DC_TILE_DEFAULT>::blocks_resident(1) && DecodeForm<16>::ready();
}

// Blocks of the decode kernel that the device holds at once when the keys are cut `num_splits` ways, in the usual
// form (small = 0) or in the form with 16-key tiles that takes over where the usual one's blocks do not all fit.
LE_API int le_attention_decode_resident_blocks(int num_splits, int small) {
  if (num_splits < 1) return 0;
  if (small && DC_TILE_DEFAULT == 32 && small_tiles_enabled()) return static_cast<int>(DecodeForm<16>::blocks_resident(num_splits));
  return static_cast<int>(DecodeForm<DC_TILE_DEFAULT>::blocks_resident(num_splits));
}

// The pool's last page (num_pages - 1) is the page that nobody owns: a request at position 0 whose first page it
// is counts as padding of a step of fixed shape; its blocks end at once and its row of `out` is written as zeros.
// `requests` (optional): the indices of the batch's decode requests; without
// it requests 0 .. num_requests-1 are taken.  `scratch` holds
// le_attention_decode_scratch_floats(...) floats; it is used when the keys are
// cut into more splits than a thread-block cluster merges by itself.
// `form`: 0 lets the number of blocks decide between the usual form of the kernel and the one with 16-key tiles
// (see small_form); 1 asks for the usual form, 2 for the small one where the head size has it (a caller that pads
// the step with dummy requests knows how many of the blocks are real; the grid does not show it).
LE_API int le_attention_decode_bf16_form(void *out, int64_t out_stride, float *scratch, const void *q, int64_t q_stride,
                                         const void *k_cache, const void *v_cache, const int32_t *block_table, int max_blocks,
                                         const int32_t *cu_q, const int32_t *ctx_before, const int32_t *requests,
                                         int num_requests, int num_heads, int num_kv_heads, int page_size, int num_pages,
                                         int window, float scale, int num_splits, int form, int *status, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (num_kv_heads <= 0 || num_heads % num_kv_heads) return le::invalid("le_attention_decode_bf16: %d heads do not divide into %d groups", num_heads, num_kv_heads);
  if (num_splits < 1 || num_splits > MERGE_MAX_SPLITS) return le::invalid("le_attention_decode_bf16: %d splits (1..%d)", num_splits, MERGE_MAX_SPLITS);
  const int group = num_heads / num_kv_heads;
  const int row_tiles = (group + 15) / 16;
  if (num_kv_heads * row_tiles > 65535 || num_requests > 65535) return le::invalid("le_attention_decode_bf16: the batch is too large for one launch");
  dim3 grid(num_splits, num_kv_heads * row_tiles, num_requests);
  const bool small = form == 0 ? small_form(static_cast<int64_t>(grid.y) * grid.z)
                               : (form == 2 && DC_TILE_DEFAULT == 32 && small_tiles_enabled() && DecodeForm<16>::ready());
  if (small)
    return DecodeForm<16>::launch(grid, stream, out, out_stride, scratch, q, q_stride, k_cache, v_cache, block_table, max_blocks, cu_q,
                                  ctx_before, requests, num_requests, num_heads, num_kv_heads, page_size, num_pages, window, scale,
                                  num_splits, status);
  return DecodeForm<DC_TILE_DEFAULT>::launch(grid, stream, out, out_stride, scratch, q, q_stride, k_cache, v_cache, block_table,
                                             max_blocks, cu_q, ctx_before, requests, num_requests, num_heads, num_kv_heads, page_size,
                                             num_pages, window, scale, num_splits, status);
}

LE_API int le_attention_decode_bf16(void *out, int64_t out_stride, float *scratch, const void *q, int64_t q_stride,
                                    const void *k_cache, const void *v_cache, const int32_t *block_table, int max_blocks,
                                    const int32_t *cu_q, const int32_t *ctx_before, const int32_t *requests,
                                    int num_requests, int num_heads, int num_kv_heads, int page_size, int num_pages,
                                    int window, float scale, int num_splits, int *status, cudaStream_t stream) {
  return le_attention_decode_bf16_form(out, out_stride, scratch, q, q_stride, k_cache, v_cache, block_table, max_blocks, cu_q,
                                       ctx_before, requests, num_requests, num_heads, num_kv_heads, page_size, num_pages, window,
                                       scale, num_splits, 0, status, stream);
}

// ---------------------------------------------------------------- no allocation
// The same decode attention with its scratch inside the library, for callers
// that cannot allocate (see attention_static_scratch.h for who they are and
// what the limits are).
#include <mutex>

#include "attention_static_scratch.h"

static __device__ __align__(256) float le_static_scratch[LE_STATIC_SCRATCH_FLOATS];

namespace {

// In host code `le_static_scratch` is only a handle for the runtime, not an
// address a kernel could use; the device address is looked up once per device.
int static_scratch_address(float **address) {
  constexpr int kMaxDevices = 64;
  static std::mutex guard;
  static float *per_device[kMaxDevices] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return le::invalid("le_attention_decode_bf16_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices) return le::invalid("le_attention_decode_bf16_static: device %d is beyond the %d this library tracks", device, kMaxDevices);
  std::lock_guard<std::mutex> lock(guard);
  if (per_device[device] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, le_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return le::invalid("le_attention_decode_bf16_static: cudaGetSymbolAddress on device %d: %s", device, cudaGetErrorString(e));
    per_device[device] = static_cast<float *>(p);
  }
  *address = per_device[device];
  return 0;
}

}  // namespace

LE_API int le_attention_decode_bf16_static(void *out, int64_t out_stride, const void *q, int64_t q_stride,
                                           const void *k_cache, const void *v_cache, const int32_t *block_table,
                                           int max_blocks, const int32_t *cu_q, const int32_t *ctx_before,
                                           const int32_t *requests, int num_requests, int num_heads, int num_kv_heads,
                                           int page_size, int num_pages, int window, float scale, int num_splits,
                                           int *status, cudaStream_t stream) {
  if (num_requests <= 0) return 0;
  if (num_heads <= 0 || num_splits < 1) return le::invalid("le_attention_decode_bf16_static: %d heads, %d splits", num_heads, num_splits);
  const int64_t need = le_attention_decode_scratch_floats(num_requests, num_heads, num_splits);
  if (need > LE_STATIC_SCRATCH_FLOATS)
    return le::invalid("le_attention_decode_bf16_static: %d requests x %d heads x %d splits need %lld floats of scratch, "
                       "the built-in array holds %d; use fewer splits or le_attention_decode_bf16 with your own scratch",
                       num_requests, num_heads, num_splits, static_cast<long long>(need), LE_STATIC_SCRATCH_FLOATS);
  float *scratch = nullptr;
  if (need > 0) {
    const int rc = static_scratch_address(&scratch);
    if (rc != 0) return rc;
  }
  return le_attention_decode_bf16(out, out_stride, scratch, q, q_stride, k_cache, v_cache, block_table, max_blocks, cu_q,
                                  ctx_before, requests, num_requests, num_heads, num_kv_heads, page_size, num_pages,
                                  window, scale, num_splits, status, stream);
}

#else  // head sizes above 128 use the generic kernel

#include "attention_static_scratch.h"

LE_API int le_attention_mma_available() { return 0; }

// There is no split-key kernel for this head size: the no-allocation entry
// point exists so that a caller can link against it, and refuses every call.
LE_API int le_attention_decode_bf16_static(void *, int64_t, const void *, int64_t, const void *, const void *, const int32_t *,
                                           int, const int32_t *, const int32_t *, const int32_t *, int, int, int, int, int,
                                           int, float, int, int *, cudaStream_t) {
  return le::invalid("le_attention_decode_bf16_static: this library was built for head size %d; the split-key decode "
                     "attention exists for head sizes up to 128", LE_HEAD_DIM);
}

#endif
