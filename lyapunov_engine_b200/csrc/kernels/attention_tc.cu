// Prefill attention on the fifth-generation tensor cores (tcgen05, tensor
// memory, TMA), for bfloat16 with head sizes 64 and 128 and pages of 8..128
// keys (a power of two): portions of prompts against the paged cache.
//
// One block owns 128 query tokens of one head and walks the keys in tiles of
// 128.  Roles:
//   warp 0      producer: its lanes look the tile's pages up in the block table
//               and each issues the TMA copies of one page's keys or values
//               (128-byte swizzle) into a ring of key stages and one of value
//               stages;
//   warp 1      tensor core: one thread issues S = Q K^T (128 x 128 x head
//               size) into one of two score buffers in tensor memory and, when
//               the probabilities are ready, O += P V (128 x head size x 128);
//   warp 10     where tensor memory has room for the probabilities beside the
//               scores (head size 64), a thread of its own issues the scores
//               from tile 2 on, so that they never wait behind a product;
//   warps 2..9  softmax, in two groups of four warps.  Group g takes the tiles
//               j = g, g + 2, ... and keeps a running maximum, a sum and an
//               output accumulator of its own for them, so the two groups never
//               wait for each other: while one computes exponentials the other
//               waits for its scores.  Thread (quarter, lane) of a group owns
//               query row r with all 128 keys of the tile: it reads the scores
//               from tensor memory, masks what the row may not see, and writes the
//               probabilities as bfloat16 into the group's buffer in shared
//               memory in the operand layout of the next product.
// The running maximum only moves when the tile's maximum exceeds it by more
// than 2^8 in the exponent; until then probabilities up to 256 go into the
// product and the sum (both 32-bit accumulations), which the final division
// takes out again.  The accumulator in tensor memory is therefore rescaled
// rarely.  A group frees its score buffer as soon as the scores are in its
// registers, and the tensor core fills it with the scores of the group's next
// tile while the group still works on this one.  At the end the two groups' partial results are merged like the
// splits of a decode: each thread combines half of the columns of its row.
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
constexpr int KS = HD == 64 ? 4 : 3;        // key stages
constexpr int VS = HD == 64 ? 4 : 2;        // value stages
constexpr int THREADS = 352;                // producer warp, tensor-core warp, two softmax groups of four warps, score-issue warp
constexpr int SCORE_WARP = 10;
constexpr int Q_BYTES = BM * HD * 2, K_BYTES = BN * HD * 2, V_BYTES = BN * HD * 2;
constexpr uint32_t TMEM_COLS = 512;         // scores at 0 and 128, the groups' outputs at 256 and 256 + head size
constexpr uint32_t O_COL = 256;
// The probabilities (bfloat16, two to a column: 64 columns) have columns of their own where tensor memory has
// room (head size 64); else they take the place of the scores they were made from, and the scores of the
// group's next tile can only follow the product that reads them.
constexpr bool OWN_P_COLUMNS = 256 + 2 * HD + 2 * 64 <= 512;
__device__ __forceinline__ uint32_t p_col(int g) { return OWN_P_COLUMNS ? 256 + 2 * HD + g * 64 : g * BN; }
constexpr float LOG2E = 1.4426950408889634f;
constexpr float MAX_SLACK = 8.0f;           // the running maximum may lag the true one by this much (base-2 exponent)

// 32 scores of a row from tensor memory, masked where the row may not see the key.
__device__ __forceinline__ void mask32(uint32_t (&v)[32], int first_key, int p_row, int lo_row) {
  if (first_key + 31 > p_row || first_key < lo_row) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (first_key + i > p_row || first_key + i < lo_row) v[i] = 0xff800000u;   // -inf
  }
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, bf16 *__restrict__ out, int64_t out_stride,
                    const int32_t *__restrict__ block_table, int max_blocks, const int32_t *__restrict__ cu_q,
                    const int32_t *__restrict__ ctx_before, const int32_t *__restrict__ tile_request,
                    const int32_t *__restrict__ tile_q0, int num_heads, int num_kv_heads, int page_size, int page_shift,
                    int num_pages, int window, float scale, int *__restrict__ status) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  unsigned char *q_smem = smem;
  unsigned char *k_smem = q_smem + Q_BYTES;
  unsigned char *v_smem = k_smem + KS * K_BYTES;
  float *group_stats = reinterpret_cast<float *>(v_smem + VS * V_BYTES);      // [2 groups][maximum, sum][BM]
  uint64_t *q_full = reinterpret_cast<uint64_t *>(group_stats + 4 * BM);
  uint64_t *k_full = q_full + 1;             // [KS]
  uint64_t *k_empty = k_full + KS;           // [KS]
  uint64_t *v_full = k_empty + KS;           // [VS]
  uint64_t *v_empty = v_full + VS;           // [VS]
  uint64_t *s_full = v_empty + VS;           // [2]: scores of the group's next tile are in tensor memory
  uint64_t *s_free = s_full + 2;             // [2]: the group has the scores in registers, the buffer may be overwritten
  uint64_t *p_full = s_free + 2;             // [2]: the group's probabilities are in shared memory
  uint64_t *o_done = p_full + 2;             // [2]: the group's accumulator holds all its tiles so far
  uint64_t *merge_bar = o_done + 2;          // both groups have their final sums
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(merge_bar + 1);
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

  // ---- the producer's tools (warp 0).  Keys run one tile ahead of values, the order in which the tensor core wants them.
  const int pages_per_tile = BN >> page_shift;              // at most 16: one lane per page
  int keys_issued = 0, values_issued = 0;
  // this lane's page of tile j, looked up two tiles before it is needed: the block table is in global memory
  auto page_of = [&](int j) {
    int page = num_pages - 1;
    if (lane < pages_per_tile && j < num_tiles) {
      const int slot = ((k_begin + j * BN) >> page_shift) + lane;
      if (slot < max_blocks) page = table[slot];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, LE_STATUS_BAD_PAGE);
        page = num_pages - 1;                                // the page nobody owns: finite values, masked anyway
      }
    }
    return page;
  };
  // one tile's keys or values: lane 0 waits for the stage and announces the bytes, then one lane per page copies
  auto load_tile = [&](int j, int page, const CUtensorMap *map, unsigned char *ring, int stages, uint64_t *full, uint64_t *empty) {
    const int s = j % stages;
    bool ok = true;
    if (lane == 0) {
      ok = mbar_wait(empty + s, ((j / stages) & 1) ^ 1, failed);
      if (ok) mbar_expect_tx(full + s, K_BYTES);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) return false;
    if (lane < pages_per_tile) {
      const int row = (page * num_kv_heads + kvh) * page_size;
      unsigned char *dst = ring + s * K_BYTES + lane * page_size * 128;
      for (int d = 0; d < DB; ++d) tma_load_2d(dst + d * BN * 128, map, full + s, d * 64, row);
    }
    return true;
  };
  int page_now = 0, page_next = 0;
  bool producer_ok = true;

  if (warp == 0) {
    if (lane == 0) {
      mbar_init(q_full, 1);
      for (int s = 0; s < KS; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
      for (int s = 0; s < VS; ++s) { mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
      for (int g = 0; g < 2; ++g) { mbar_init(s_full + g, 1); mbar_init(s_free + g, 4); mbar_init(p_full + g, 4); mbar_init(o_done + g, 1); }
      mbar_init(merge_bar, 8);
      *failed = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_async_proxy();
    }
    __syncwarp();
    // The first copies need nothing but the barriers: they start before tensor memory is set up and the block
    // meets, so the scores of tile 0 can follow the block's start closely.
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      for (int d = 0; d < DB; ++d) tma_load_2d(q_smem + d * BM * 128, &map_q, q_full, head * HD + d * 64, tok0);
    }
    page_now = page_of(0);
    page_next = page_of(1);
    producer_ok = load_tile(0, page_now, &map_k, k_smem, KS, k_full, k_empty);
    if (producer_ok) keys_issued = 1;
    if (producer_ok && num_tiles > 1) {
      producer_ok = load_tile(1, page_next, &map_k, k_smem, KS, k_full, k_empty);
      if (producer_ok) keys_issued = 2;
    }
    if (producer_ok) {
      producer_ok = load_tile(0, page_now, &map_v, v_smem, VS, v_full, v_empty);
      if (producer_ok) values_issued = 1;
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // F32 accumulate, BF16 operands, M = 128; S: both K-major, N = 128; PV: B is MN-major (bit 16), N = head size
  constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
  constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | (static_cast<uint32_t>(HD >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
  // scores of tile j into the buffer of group j & 1; frees the key stage when they are through
  auto issue_scores = [&](int j) {
    if (!mbar_wait(k_full + j % KS, (j / KS) & 1, failed)) return false;
    tc_fence_after();
    const uint32_t q_addr = smem_u32(q_smem);
    const uint32_t k_addr = smem_u32(k_smem + (j % KS) * K_BYTES);
    const uint32_t tmem_s = tmem_base + (j & 1) * BN;
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      // k-step k lies in 64-wide block k / 4 of the head size, 32 bytes per step inside it
      const uint32_t off = (k / 4) * (BM * 128) + (k % 4) * 32;
      tc_mma(tmem_s, smem_desc(q_addr + off), smem_desc(k_addr + off), idesc_s, k > 0 ? 1u : 0u);
    }
    tc_commit(s_full + (j & 1));
    tc_commit(k_empty + j % KS);
    return true;
  };

  if (warp == 0) {
    // ---- producer, from where the early copies stopped
    bool ok = producer_ok;
    for (int j = 0; j < num_tiles && ok; ++j) {
      const int page_after = page_of(j + 2);                 // needed in the next round
      if (j + 1 < num_tiles && j + 1 >= keys_issued) {
        ok = load_tile(j + 1, page_next, &map_k, k_smem, KS, k_full, k_empty);
        if (!ok) break;
        ++keys_issued;
      }
      if (j >= values_issued) {
        ok = load_tile(j, page_now, &map_v, v_smem, VS, v_full, v_empty);
        if (ok) ++values_issued;
      }
      page_now = page_next;
      page_next = page_after;
    }
    if (!ok && lane == 0) {
      *failed = 1;
      atomicOr(status, LE_STATUS_WAIT_TIMEOUT);
      volatile int never = 0;                                // copies in flight must land before the block may end
      for (int j = max(0, keys_issued - KS); j < keys_issued; ++j) mbar_wait(k_full + j % KS, (j / KS) & 1, &never);
      for (int j = max(0, values_issued - VS); j < values_issued; ++j) mbar_wait(v_full + j % VS, (j / VS) & 1, &never);
    }
  } else if (warp == 1) {
    // ---- tensor-core issue: the first scores and every product O += P V
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, failed) && issue_scores(0);
      if (ok && num_tiles > 1) ok = issue_scores(1);
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int g = j & 1;
        ok = mbar_wait(p_full + g, (j >> 1) & 1, failed) && mbar_wait(v_full + j % VS, (j / VS) & 1, failed);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(v_smem + (j % VS) * V_BYTES);
#pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          // P: in tensor memory, 16 keys = 8 columns; V: rows are keys, 16 keys = 2048 bytes, 64-wide dim blocks BN * 128 apart
          const uint64_t db = smem_desc_mn(v_addr + k * 16 * 128, BN * 128);
          tc_mma_ts(tmem_base + O_COL + g * HD, tmem_base + p_col(g) + k * 8, db, idesc_o, (j >= 2 || k > 0) ? 1u : 0u);
        }
        tc_commit(v_empty + j % VS);          // the stage's values have been read
        tc_commit(o_done + g);                // the group's accumulator holds its tiles up to j; its probabilities are free
        // without columns of their own the probabilities sat where the next scores go: those follow the product
        if (!OWN_P_COLUMNS && j + 2 < num_tiles) ok = issue_scores(j + 2);
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else if (warp == SCORE_WARP) {
    // ---- tensor-core issue: the scores from tile 2 on, where they do not have to follow a product.  As soon
    // as a group has taken the scores of tile j into registers its buffer takes tile j + 2, from a thread of
    // its own so that this never waits behind the products' thread (which waits for probabilities).
    if (OWN_P_COLUMNS && lane == 0) {
      bool ok = true;
      for (int j = 2; j < num_tiles && ok; ++j) {
        ok = mbar_wait(s_free + (j & 1), ((j - 2) >> 1) & 1, failed);
        if (!ok) break;
        tc_fence_after();
        ok = issue_scores(j);
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else {
    // ---- softmax: thread (quarter, lane) of group g owns query row r for the tiles g, g + 2, ...
    const int quarter = warp & 3;               // the tensor-memory lanes this warp may touch
    const int g = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;
    const int p_row = p0 + r;
    const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_col = lane_base + g * BN, o_col = lane_base + O_COL + g * HD;
    const float sl2 = scale * LOG2E;
    const float2 sl2_2 = make_float2(sl2, sl2);
    const uint32_t p_tmem = lane_base + p_col(g);
    float m_run = -INFINITY, l_run = 0.0f;      // m_run in exponent units (score * scale * log2 e)
    bool ok = true;
    int t = 0;                                  // how many tiles this group has done
    for (int j = g; j < num_tiles; j += 2, ++t) {
      const int k0 = k_begin + j * BN;
      ok = mbar_wait(s_full + g, t & 1, failed) && ok;
      tc_fence_after();
      // the row's 128 scores stay in registers from here to the exponentials
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_load32_async(s_col + c * 32, v[c]);
      tc_wait_loads();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free + g);              // the tensor core may overwrite the score buffer
      float chunk_max[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        mask32(v[c], k0 + c * 32, p_row, lo_row);
        chunk_max[c] = -INFINITY;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) chunk_max[c] = fmaxf(chunk_max[c], __uint_as_float(v[c][i]));   // four chains side by side
      float tile_max = fmaxf(fmaxf(chunk_max[0], chunk_max[1]), fmaxf(chunk_max[2], chunk_max[3]));
      tile_max *= sl2;
      float alpha = 1.0f;
      if (tile_max > m_run + MAX_SLACK) {        // also the first keys a row sees (m_run is -inf until then)
        alpha = le::fast_exp2(m_run - tile_max);
        m_run = tile_max;
      }
      const float neg_m = (m_run == -INFINITY) ? 0.0f : -m_run;
      const float2 neg_m2 = make_float2(neg_m, neg_m);
      if (t > 0) {                               // the product of this group's tile before has read the probabilities
        ok = mbar_wait(o_done + g, (t - 1) & 1, failed) && ok;
        tc_fence_after();
      }
      // exponentials, the row's sum, probabilities as bfloat16 pairs into tensor memory (the next product's A operand)
      float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float2 x = __ffma2_rn(make_float2(__uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1])), sl2_2, neg_m2);
          x.x = le::fast_exp2(x.x);
          x.y = le::fast_exp2(x.y);
          sum2 = __fadd2_rn(sum2, x);
          const __nv_bfloat162 pair = __floats2bfloat162_rn(x.x, x.y);
          packed[i / 2] = *reinterpret_cast<const uint32_t *>(&pair);
        }
        tc_store16(p_tmem + c * 16, packed);
      }
      l_run = l_run * alpha + (sum2.x + sum2.y);
      // (rarely) some row of the warp moved its maximum: rescale the group's accumulator before the next product
      if (t > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tc_load32(o_col + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc_store32(o_col + c * 32, o);
        }
        tc_wait_stores();
      }
      tc_wait_stores();
      tc_fence_before();
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      if (lane == 0) mbar_arrive(p_full + g);
    }
    if (ok && t > 0) ok = mbar_wait(o_done + g, (t - 1) & 1, failed);
    // ---- merge the two groups: each thread takes half of the columns of its row
    float *mine = group_stats + g * 2 * BM, *theirs = group_stats + (g ^ 1) * 2 * BM;
    mine[r] = m_run;
    mine[BM + r] = l_run;
    tc_fence_before();
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) mbar_arrive(merge_bar);
    if (ok) ok = mbar_wait(merge_bar, 0, failed);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    } else {
      tc_fence_after();
      const float m0 = g == 0 ? m_run : theirs[r], m1 = g == 0 ? theirs[r] : m_run;
      const float l0 = g == 0 ? l_run : theirs[BM + r], l1 = g == 0 ? theirs[BM + r] : l_run;
      const float m = fmaxf(m0, m1);
      const float w0 = m0 == -INFINITY ? 0.0f : le::fast_exp2(m0 - m);
      const float w1 = m1 == -INFINITY ? 0.0f : le::fast_exp2(m1 - m);
      const float l = l0 * w0 + l1 * w1;
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const float f0 = w0 * inv, f1 = w1 * inv;
      constexpr int OC = HD / 2;                 // output columns per thread
      bf16 *dst = out + (tok0 + r) * out_stride + head * HD + g * OC;
      const uint32_t col = lane_base + O_COL + g * OC;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t a[32], bb[32];
        tc_load32_async(col + c * 32, a);
        if (num_tiles > 1) tc_load32_async(col + HD + c * 32, bb);     // the second group had no tile otherwise
        tc_wait_loads();
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            __nv_bfloat162 *pk = reinterpret_cast<__nv_bfloat162 *>(&packed);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x = __uint_as_float(a[i + 2 * e]) * f0, y = __uint_as_float(a[i + 2 * e + 1]) * f0;
              if (num_tiles > 1) {
                x = fmaf(__uint_as_float(bb[i + 2 * e]), f1, x);
                y = fmaf(__uint_as_float(bb[i + 2 * e + 1]), f1, y);
              }
              pk[e] = __floats2bfloat162_rn(x, y);
            }
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
  const size_t smem = Q_BYTES + KS * K_BYTES + VS * V_BYTES + 4 * BM * sizeof(float) + 1024 + 256;   // 1024 to align, 256 for the barriers
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
