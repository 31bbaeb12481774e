// Prefill attention on the fifth-generation tensor cores (tcgen05, tensor
// memory, TMA), for bfloat16 with head sizes 64 and 128 and pages of 8..128
// keys (a power of two): portions of prompts against the paged cache.
//
// One block owns 128 query tokens of one head and walks the keys in tiles of
// 128.  Roles:
//   warp 0      producer: its lanes look the tile's pages up in the block table
//               and each issues the TMA copies of one page's keys and values
//               (128-byte swizzle) into a ring of stages;
//   warp 1      tensor core: one thread issues S = Q K^T (128 x 128 x head
//               size) into one of two score buffers in tensor memory and, when
//               the probabilities are ready, O += P V (128 x head size x 128);
//   warps 2..9  softmax: two threads share query row r, each with 64 of the
//               tile's 128 keys.  A thread reads its scores from tensor memory,
//               masks what the row may not see, agrees with its partner on the
//               row's maximum, keeps the running maximum and its share of the
//               sum in 32 bits (exp2 with the scale folded in), writes the
//               probabilities as bfloat16 into shared memory in the operand
//               layout of the next product (two buffers, so this overlaps the
//               product of the tile before), and rescales its half of the
//               output accumulator in tensor memory when a row's maximum grew.
// Scores of tile j + 1 are issued before the product of tile j, so the softmax
// of one tile overlaps the tensor core's work on its neighbours.  At the end
// the softmax threads normalise their rows and store them.
//
// Every wait on an mbarrier is bounded in time; a block that gives up sets the
// status word, lets copies in flight land, frees its tensor memory and returns.
//
// Same contract as the mma.sync kernel in attention_mma.cu (query at absolute
// position p sees keys max(0, p - window + 1) .. p of its own request through
// the block table), which stays for other head and page sizes.
// Reference: flash_attn_v2.cu:13-212 (contiguous keys, scalar products).
#include "tc_common.cuh"

#ifndef LE_HEAD_DIM
#error "compile with -DLE_HEAD_DIM=<head size>"
#endif

#if LE_HEAD_DIM == 64 || LE_HEAD_DIM == 128

namespace {

using namespace tc;
using bf16 = __nv_bfloat16;
constexpr int HD = LE_HEAD_DIM;
constexpr int DB = HD / 64;                 // 64-wide blocks of the head size
constexpr int BM = 128, BN = 128;           // query rows, keys per tile
constexpr int STAGES = HD == 64 ? 3 : 2;
constexpr int THREADS = 320;               // producer warp, tensor-core warp, eight softmax warps
constexpr int Q_BYTES = BM * HD * 2, K_BYTES = BN * HD * 2, V_BYTES = BN * HD * 2, P_BYTES = BM * BN * 2;
constexpr int P_BUFFERS = HD == 64 ? 2 : 1;   // probabilities double-buffered where shared memory allows
constexpr int STAGE_BYTES = K_BYTES + V_BYTES;
constexpr uint32_t TMEM_COLS = 512;         // scores 0..127 and 128..255, output from 256
constexpr uint32_t O_COL = 256;
constexpr float LOG2E = 1.4426950408889634f;

__global__ void __launch_bounds__(THREADS)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, bf16 *__restrict__ out, int64_t out_stride,
                    const int32_t *__restrict__ block_table, int max_blocks, const int32_t *__restrict__ cu_q,
                    const int32_t *__restrict__ ctx_before, const int32_t *__restrict__ tile_request,
                    const int32_t *__restrict__ tile_q0, int num_heads, int num_kv_heads, int page_size, int page_shift,
                    int num_pages, int window, float scale, int *__restrict__ status) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  unsigned char *q_smem = smem;
  unsigned char *kv_smem = q_smem + Q_BYTES;
  unsigned char *p_smem = kv_smem + STAGES * STAGE_BYTES;
  float *pair_max = reinterpret_cast<float *>(p_smem + P_BUFFERS * P_BYTES);   // [2 tile parities][2 halves][BM]
  float *pair_sum = pair_max + 4 * BM;                                         // [2 halves][BM]
  uint64_t *q_full = reinterpret_cast<uint64_t *>(pair_sum + 2 * BM);
  uint64_t *kv_full = q_full + 1;            // [STAGES]
  uint64_t *kv_empty = kv_full + STAGES;     // [STAGES]
  uint64_t *s_full = kv_empty + STAGES;      // [2]
  uint64_t *s_free = s_full + 2;             // [2]
  uint64_t *p_full = s_free + 2;
  uint64_t *o_done = p_full + 1;
  uint64_t *p_free = o_done + 1;             // [2]
  uint64_t *pair_bar = p_free + 2;           // [4]: the two warps that share 32 rows meet here
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(pair_bar + 4);
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // later tiles of a prompt see more keys and take longer: start them first
  const int tile = gridDim.x - 1 - blockIdx.x, head = blockIdx.y;
  const int kvh = head / (num_heads / num_kv_heads);
  const int b = tile_request[tile];
  const int q0 = tile_q0[tile];
  const int q_len = cu_q[b + 1] - cu_q[b];
  const int rows = min(BM, q_len - q0);
  const int tok0 = cu_q[b] + q0;
  const int p0 = ctx_before[b] + q0;
  const int p_last = p0 + rows - 1;
  int k_begin = 0;
  if (window > 0) k_begin = max(0, p0 - window + 1) / BN * BN;
  const int num_tiles = (p_last + 1 - k_begin + BN - 1) / BN;
  const int32_t *table = block_table + static_cast<int64_t>(b) * max_blocks;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(kv_full + s, 1); mbar_init(kv_empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(s_full + a, 1); mbar_init(s_free + a, 8); mbar_init(p_free + a, 1); }
    mbar_init(p_full, 8);
    mbar_init(o_done, 1);
    for (int a = 0; a < 4; ++a) mbar_init(pair_bar + a, 64);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      for (int d = 0; d < DB; ++d) tma_load_2d(q_smem + d * BM * 128, &map_q, q_full, head * HD + d * 64, tok0);
    }
    const int pages_per_tile = BN >> page_shift;            // at most 16: one lane per page
    int issued = 0;
    bool ok = true;
    for (int j = 0; j < num_tiles && ok; ++j, ++issued) {
      const int s = j % STAGES;
      if (lane == 0) {
        ok = !*failed && mbar_wait(kv_empty + s, ((j / STAGES) & 1) ^ 1, failed);
        if (ok) mbar_expect_tx(kv_full + s, STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < pages_per_tile) {
        const int slot = ((k_begin + j * BN) >> page_shift) + lane;
        int page = slot < max_blocks ? table[slot] : num_pages - 1;
        if (page < 0 || page >= num_pages) {
          atomicOr(status, LE_STATUS_BAD_PAGE);
          page = num_pages - 1;                              // the page nobody owns: finite values, masked anyway
        }
        const int row = (page * num_kv_heads + kvh) * page_size;
        unsigned char *k_dst = kv_smem + s * STAGE_BYTES + lane * page_size * 128;
        unsigned char *v_dst = k_dst + K_BYTES;
        for (int d = 0; d < DB; ++d) {
          tma_load_2d(k_dst + d * BN * 128, &map_k, kv_full + s, d * 64, row);
          tma_load_2d(v_dst + d * BN * 128, &map_v, kv_full + s, d * 64, row);
        }
      }
    }
    if (!ok && lane == 0) {
      *failed = 1;
      atomicOr(status, LE_STATUS_WAIT_TIMEOUT);
      volatile int never = 0;
      for (int j = max(0, issued - STAGES); j < issued; ++j) mbar_wait(kv_full + j % STAGES, (j / STAGES) & 1, &never);
    }
  } else if (warp == 1) {
    // ---- tensor-core issue
    if (lane == 0) {
      // F32 accumulate, BF16 operands, M = 128; S: both K-major, N = 128; PV: B is MN-major (bit 16), N = head size
      constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
      constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(HD >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
      const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
      auto issue_scores = [&](int j) {
        const uint32_t k_addr = smem_u32(kv_smem + (j % STAGES) * STAGE_BYTES);
        const uint32_t tmem_s = tmem_base + (j & 1) * BN;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          // k-step k lies in 64-wide block k / 4 of the head size, 32 bytes per step inside it
          const uint32_t off = (k / 4) * (BM * 128) + (k % 4) * 32;
          tc_mma(tmem_s, smem_desc(q_addr + off), smem_desc(k_addr + off), idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(s_full + (j & 1));
      };
      bool ok = mbar_wait(q_full, 0, failed) && mbar_wait(kv_full, 0, failed);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int j = 0; j < num_tiles && ok; ++j) {
        if (j + 1 < num_tiles) {
          ok = mbar_wait(kv_full + (j + 1) % STAGES, ((j + 1) / STAGES) & 1, failed);
          if (ok && j + 1 >= 2) ok = mbar_wait(s_free + ((j + 1) & 1), (((j + 1) >> 1) - 1) & 1, failed);
          if (!ok) break;
          tc_fence_after();
          issue_scores(j + 1);
        }
        ok = mbar_wait(p_full, j & 1, failed);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(kv_smem + (j % STAGES) * STAGE_BYTES + K_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // P: K-major, keys in two 64-wide blocks; V: rows are keys, 16 keys = 2048 bytes, 64-wide dim blocks BN * 128 apart
          const uint64_t da = smem_desc(p_addr + (j % P_BUFFERS) * P_BYTES + (k / 4) * (BM * 128) + (k % 4) * 32);
          const uint64_t db = smem_desc_mn(v_addr + k * 16 * 128, BN * 128);
          tc_mma(tmem_base + O_COL, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(kv_empty + j % STAGES);     // the stage's keys and values have been read
        tc_commit(p_free + (j & 1));          // ... and this tile's probabilities
        tc_commit(o_done);                    // the output accumulator holds tiles 0..j
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else {
    // ---- softmax: threads (quarter, lane) of the two halves share query row r; each takes 64 of the 128 keys
    const int quarter = warp & 3;               // the tensor-memory lanes this warp may touch
    const int half = (warp - 2) >> 2;           // which 64 keys of a tile, which half of the output columns
    const int r = quarter * 32 + lane;
    const int p_row = p0 + r;
    const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const float sl2 = scale * LOG2E;
    constexpr int OC = HD / 2;                  // output columns per thread
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    uint32_t pair_phase = 0;
    // the two threads of a row exchange a value through shared memory: arrive, then a bounded wait for all 64
    auto pair_sync = [&]() {
      mbar_arrive(pair_bar + quarter);
      const bool met = mbar_wait(pair_bar + quarter, pair_phase, failed);
      pair_phase ^= 1;
      return met;
    };
    for (int j = 0; j < num_tiles; ++j) {
      const int k0 = k_begin + j * BN + half * 64;
      ok = mbar_wait(s_full + (j & 1), (j >> 1) & 1, failed);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      uint32_t v[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tc_load32_async(lane_base + (j & 1) * BN + half * 64 + c * 32, v[c]);
      tc_wait_loads();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free + (j & 1));          // the tensor core may overwrite this score buffer
      // mask what this row may not see, find the maximum of this half, then of the row
      const bool edge = k0 + 63 > p_row || k0 < lo_row;
      float tile_max = -INFINITY;
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(v[c][i]);
          if (edge) {
            const int pos = k0 + c * 32 + i;
            if (pos > p_row || pos < lo_row) x = -INFINITY;
          }
          v[c][i] = __float_as_uint(x);
          tile_max = fmaxf(tile_max, x);
        }
      float *mine = pair_max + ((j & 1) * 2 + half) * BM, *theirs = pair_max + ((j & 1) * 2 + (half ^ 1)) * BM;
      mine[r] = tile_max;
      ok = pair_sync();
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tile_max = fmaxf(tile_max, theirs[r]);
      const float m_new = fmaxf(m_run, tile_max);
      const float alpha = (m_new == -INFINITY) ? 1.0f : exp2f((m_run - m_new) * sl2);
      const float neg_m = (m_new == -INFINITY) ? 0.0f : -m_new * sl2;
      m_run = m_new;
      if (P_BUFFERS == 2) {
        if (j >= 2) {                            // the product two tiles back has read this buffer
          ok = mbar_wait(p_free + (j & 1), ((j >> 1) - 1) & 1, failed);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
        }
      } else if (j > 0) {                        // one buffer: the product of the tile before must be through
        ok = mbar_wait(o_done, (j - 1) & 1, failed);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tc_fence_after();
      }
      unsigned char *p_tile = p_smem + (j % P_BUFFERS) * P_BYTES + half * (BM * 128) + r * 128;
      float sum = 0.0f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float p[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            p[e] = exp2f(fmaf(__uint_as_float(v[c][i + e]), sl2, neg_m));
            sum += p[e];
          }
          uint4 packed;
          __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&packed);
#pragma unroll
          for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
          const int chunk = c * 4 + i / 8;                   // 16-byte chunk 0..7 of this half's 64 keys
          *reinterpret_cast<uint4 *>(p_tile + ((chunk ^ (r & 7)) << 4)) = packed;
        }
      }
      l_run = l_run * alpha + sum;
      if (P_BUFFERS == 2 && j > 0) {             // the output accumulator holds every tile before this one
        ok = mbar_wait(o_done, (j - 1) & 1, failed);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tc_fence_after();
      }
      // rescale this thread's half of the output accumulator when some row of the warp moved its maximum
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t o[32];
          tc_load32(lane_base + O_COL + half * OC + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc_store32(lane_base + O_COL + half * OC + c * 32, o);
        }
        tc_wait_stores();
      }
      fence_async_proxy();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) {
      ok = mbar_wait(o_done, (num_tiles - 1) & 1, failed);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (!ok) {
      if (lane == 0) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    } else {
      tc_fence_after();
      pair_sum[half * BM + r] = l_run;
      if (!pair_sync()) atomicOr(status, LE_STATUS_WAIT_TIMEOUT);   // the row is then stored with its own share only
      const float l = l_run + pair_sum[(half ^ 1) * BM + r];
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      bf16 *dst = out + (tok0 + r) * out_stride + head * HD + half * OC;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tc_load32(lane_base + O_COL + half * OC + c * 32, o);
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&packed);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h[e] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4 *>(dst + c * 32 + i) = packed;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

int tc_page_shift_of(int page_size) {
  for (int s = 0; s < 30; ++s)
    if ((1 << s) == page_size) return s;
  return -1;
}

}  // namespace

// 1 when this head size has the kernel and the page size suits it.
LE_API int le_attention_tc_available(int page_size) {
  const int shift = tc_page_shift_of(page_size);
  return shift >= 3 && page_size <= 128 ? 1 : 0;
}

// Same arguments as le_attention_prefill_bf16 plus the shape of the buffer q
// lives in; the tiles list 128 query tokens each.  q must be 16-byte aligned
// with q_stride a multiple of 8; out rows must be 16-byte aligned.
LE_API int le_attention_prefill_tc_bf16(void *out, int64_t out_stride, const void *q, int64_t q_stride, int num_tokens,
                                        int q_width, const void *k_cache, const void *v_cache, const int32_t *block_table,
                                        int max_blocks, const int32_t *cu_q, const int32_t *ctx_before,
                                        const int32_t *tile_request, const int32_t *tile_q0, int num_tiles, int num_heads,
                                        int num_kv_heads, int page_size, int num_pages, int window, float scale, int *status,
                                        cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (!le_attention_tc_available(page_size)) return le::invalid("le_attention_prefill_tc_bf16: pages of %d keys are not supported (8..128, a power of two)", page_size);
  if (num_kv_heads <= 0 || num_heads % num_kv_heads) return le::invalid("le_attention_prefill_tc_bf16: %d heads do not divide into %d groups", num_heads, num_kv_heads);
  if (num_heads > 65535) return le::invalid("le_attention_prefill_tc_bf16: too many heads for one launch");
  if (q_stride % 8 || out_stride % 8 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return le::invalid("le_attention_prefill_tc_bf16: q and out must be 16-byte aligned with row strides that are multiples of 8");
  CUtensorMap map_q, map_k, map_v;
  int rc = tensor_map(&map_q, q, num_tokens, q_width, q_stride, BM);
  if (rc != 0) return rc;
  const int cache_rows = num_pages * num_kv_heads * page_size;
  rc = tensor_map(&map_k, k_cache, cache_rows, HD, HD, page_size);
  if (rc != 0) return rc;
  rc = tensor_map(&map_v, v_cache, cache_rows, HD, HD, page_size);
  if (rc != 0) return rc;
  const size_t smem = Q_BYTES + STAGES * STAGE_BYTES + P_BUFFERS * P_BYTES + 6 * BM * sizeof(float) + 1024 + 256;
  cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return le::invalid("le_attention_prefill_tc_bf16: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  dim3 grid(num_tiles, num_heads);
  attention_tc_kernel<<<grid, THREADS, smem, stream>>>(map_q, map_k, map_v, static_cast<bf16 *>(out), out_stride, block_table,
                                                       max_blocks, cu_q, ctx_before, tile_request, tile_q0, num_heads,
                                                       num_kv_heads, page_size, tc_page_shift_of(page_size), num_pages, window,
                                                       scale, status);
  return le::launched();
}

#else

LE_API int le_attention_tc_available(int) { return 0; }

#endif
