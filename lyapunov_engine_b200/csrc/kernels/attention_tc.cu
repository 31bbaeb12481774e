// Prefill attention on the fifth-generation tensor cores (tcgen05, tensor
// memory, TMA), for bfloat16 with head sizes 64 and 128 and pages of 8..128
// keys (a power of two): portions of prompts against the paged cache.
//
// One block owns 128 query tokens of TWO query heads that share a key/value
// head (one head where the group has an odd one left) and walks the keys in
// tiles of 128; every tile of keys and values is fetched once for both heads.
// Roles:
//   warps 0..7  softmax, a group of four warps per head.  Thread (quarter,
//               lane) owns query row r with all 128 keys of the tile: it reads
//               the scores from tensor memory into registers, masks what the
//               row may not see, keeps the running maximum and the sum in 32
//               bits (exp2 with the scale folded in) and writes the
//               probabilities as bfloat16 pairs back into tensor memory, the A
//               operand of the next product.
//   warp 8      producer: its lanes look the tile's pages up in the block table
//               and each issues the TMA copies of one page's keys or values
//               (128-byte swizzle) into a ring of key stages and one of value
//               stages;
//   warp 9      tensor core: one thread issues the products O += P V (128 x
//               head size x 128) of both heads when their probabilities are
//               ready;
//   warp 10     tensor core: one thread issues the scores S = Q K^T (128 x 128
//               x head size) of both heads, each as soon as the head's softmax
//               group has taken the scores of the tile before into registers.
//               (Where tensor memory has no room for the probabilities beside
//               the scores - head size 128 - they overwrite the scores they
//               came from, the next scores must follow the product that reads
//               them, and warp 9 issues everything in that order.)
//   warp 11     none: it fills the third warp group.
// A softmax thread holds its row's 128 scores in registers; the other roles
// need few.  Registers are shared out by warp group (setmaxnreg): the third
// group gives up what the two softmax groups take (72 and 216 a thread where
// the launch bound gives 168 to all), which ends the softmax loop's spills.
// The running maximum only moves when the tile's maximum exceeds it by more
// than 2^8 in the exponent; until then probabilities up to 256 go into the
// product and the sum (both 32-bit accumulations), which the final division
// takes out again.  The accumulator in tensor memory is therefore rescaled
// rarely.  At the end every thread normalises its row and stores it.
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
// Warps 0..7: two softmax groups of four (a warp group each); warps 8..11: producer, products, scores, one idle.
// The roles need very different numbers of registers, and a block's registers are shared out by warp group:
// the softmax groups take what the fourth group gives up.
constexpr int THREADS = 384;
constexpr int PRODUCER_WARP = 8, PRODUCT_WARP = 9, SCORE_WARP = 10;
constexpr int SOFTMAX_REGS = 216, OTHER_REGS = 72;      // 2 x 216 + 72 = 3 x 168, what the launch bound gives each thread
constexpr int Q_BYTES = BM * HD * 2, K_BYTES = BN * HD * 2, V_BYTES = BN * HD * 2;
constexpr uint32_t TMEM_COLS = 512;         // head g: scores at g * 128, output at 256 + g * head size
constexpr uint32_t O_COL = 256;
// The probabilities (bfloat16, two to a column: 64 columns) have columns of their own where tensor memory has
// room (head size 64); else they take the place of the scores they were made from.
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
  unsigned char *q_smem = smem;                // [2 heads]
  unsigned char *k_smem = q_smem + 2 * Q_BYTES;
  unsigned char *v_smem = k_smem + KS * K_BYTES;
  uint64_t *q_full = reinterpret_cast<uint64_t *>(v_smem + VS * V_BYTES);
  uint64_t *k_full = q_full + 1;             // [KS]
  uint64_t *k_empty = k_full + KS;           // [KS]
  uint64_t *v_full = k_empty + KS;           // [VS]
  uint64_t *v_empty = v_full + VS;           // [VS]
  uint64_t *s_full = v_empty + VS;           // [2]: the head's scores of the next tile are in tensor memory
  uint64_t *s_free = s_full + 2;             // [2]: the head's group has them in registers, the buffer may be overwritten
  uint64_t *p_full = s_free + 2;             // [2]: the head's probabilities are in tensor memory
  uint64_t *o_done = p_full + 2;             // [2]: the head's accumulator holds all tiles so far
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_done + 2);
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Later tiles of a prompt see more keys and take longer: they start first.  The tile is the slow index of
  // the grid, so that the whole first wave of blocks holds the long ones, whatever the head.
  const int tile = gridDim.y - 1 - blockIdx.y;
  const int group = num_heads / num_kv_heads, pairs = (group + 1) / 2;
  const int kvh = blockIdx.x / pairs, pair = blockIdx.x % pairs;
  const int head0 = kvh * group + 2 * pair;
  const int heads_here = min(2, group - 2 * pair);
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

  if (warp == PRODUCER_WARP) {
    if (lane == 0) {
      mbar_init(q_full, 1);
      for (int s = 0; s < KS; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
      for (int s = 0; s < VS; ++s) { mbar_init(v_full + s, 1); mbar_init(v_empty + s, 1); }
      for (int g = 0; g < 2; ++g) { mbar_init(s_full + g, 1); mbar_init(s_free + g, 4); mbar_init(p_full + g, 4); mbar_init(o_done + g, 1); }
      *failed = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_async_proxy();
    }
    __syncwarp();
    // Launched as a dependent of the kernel before it (which wrote the queries and this step's keys and values):
    // up to here the block overlapped that kernel's end; nothing of its output is read before this line, and
    // every other role works on what this warp's copies bring.
    le::wait_for_predecessor();
    // The first copies need nothing but the barriers: they start before tensor memory is set up and the block
    // meets, so the scores of tile 0 can follow the block's start closely.
    if (lane == 0) {
      mbar_expect_tx(q_full, heads_here * Q_BYTES);
      for (int g = 0; g < heads_here; ++g)
        for (int d = 0; d < DB; ++d) tma_load_2d(q_smem + g * Q_BYTES + d * BM * 128, &map_q, q_full, (head0 + g) * HD + d * 64, tok0);
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
  if (warp == PRODUCT_WARP) {
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
  // head g's scores of tile j (whose keys have landed) into the head's score buffer
  auto issue_scores = [&](int j, int g) {
    const uint32_t q_addr = smem_u32(q_smem + g * Q_BYTES);
    const uint32_t k_addr = smem_u32(k_smem + (j % KS) * K_BYTES);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      // k-step k lies in 64-wide block k / 4 of the head size, 32 bytes per step inside it
      const uint32_t off = (k / 4) * (BM * 128) + (k % 4) * 32;
      tc_mma(tmem_base + g * BN, smem_desc(q_addr + off), smem_desc(k_addr + off), idesc_s, k > 0 ? 1u : 0u);
    }
    tc_commit(s_full + g);
  };
  // head g's product of tile j (whose values have landed): P from tensor memory, 16 keys = 8 columns; V: rows
  // are keys, 16 keys = 2048 bytes, 64-wide blocks of the head size BN * 128 apart
  auto issue_product = [&](int j, int g) {
    const uint32_t v_addr = smem_u32(v_smem + (j % VS) * V_BYTES);
#pragma unroll
    for (int k = 0; k < BN / 16; ++k)
      tc_mma_ts(tmem_base + O_COL + g * HD, tmem_base + p_col(g) + k * 8, smem_desc_mn(v_addr + k * 16 * 128, BN * 128), idesc_o,
                (j > 0 || k > 0) ? 1u : 0u);
    tc_commit(o_done + g);                    // the head's accumulator holds tiles 0..j; its probabilities are free
  };

  if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(OTHER_REGS));
  if (warp == PRODUCER_WARP) {
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
  } else if (warp == PRODUCT_WARP) {
    // ---- tensor-core issue: the products; and the scores too where they have to follow the products
    if (lane == 0) {
      bool ok = true;
      if (!OWN_P_COLUMNS) {
        ok = mbar_wait(q_full, 0, failed) && mbar_wait(k_full, 0, failed);
        if (ok) {
          tc_fence_after();
          for (int g = 0; g < heads_here; ++g) issue_scores(0, g);
          tc_commit(k_empty);
        }
      }
      for (int j = 0; j < num_tiles && ok; ++j) {
        ok = mbar_wait(v_full + j % VS, (j / VS) & 1, failed);
        const bool more = !OWN_P_COLUMNS && j + 1 < num_tiles;
        for (int g = 0; g < heads_here && ok; ++g) {
          ok = mbar_wait(p_full + g, j & 1, failed);
          if (!ok) break;
          tc_fence_after();
          issue_product(j, g);
          if (more) {                         // the head's next scores overwrite the probabilities just read
            if (g == 0) ok = mbar_wait(k_full + (j + 1) % KS, ((j + 1) / KS) & 1, failed);
            if (!ok) break;
            tc_fence_after();
            issue_scores(j + 1, g);
          }
        }
        if (!ok) break;
        tc_commit(v_empty + j % VS);          // the stage's values have been read
        if (more) tc_commit(k_empty + (j + 1) % KS);
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else if (warp == SCORE_WARP) {
    // ---- tensor-core issue: the scores, from a thread of their own where they need not follow a product, so
    // that they never wait behind the products' thread (which waits for probabilities)
    if (OWN_P_COLUMNS && lane == 0) {
      bool ok = mbar_wait(q_full, 0, failed);
      for (int j = 0; j < num_tiles && ok; ++j) {
        ok = mbar_wait(k_full + j % KS, (j / KS) & 1, failed);
        for (int g = 0; g < heads_here && ok; ++g) {
          if (j > 0) ok = mbar_wait(s_free + g, (j - 1) & 1, failed);   // the group has read the tile before
          if (!ok) break;
          tc_fence_after();
          issue_scores(j, g);
        }
        if (!ok) break;
        tc_commit(k_empty + j % KS);          // the stage's keys have been read
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else if (warp < 8 && (warp >> 2) < heads_here) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
    // ---- softmax: thread (quarter, lane) of group g owns query row r of head head0 + g
    const int quarter = warp & 3;               // the tensor-memory lanes this warp may touch
    const int g = warp >> 2;
    const int r = quarter * 32 + lane;
    const int p_row = p0 + r;
    const int lo_row = window > 0 ? max(0, p_row - window + 1) : 0;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_col = lane_base + g * BN, o_col = lane_base + O_COL + g * HD;
    const uint32_t p_tmem = lane_base + p_col(g);
    const float sl2 = scale * LOG2E;
    const float2 sl2_2 = make_float2(sl2, sl2);
    float m_run = -INFINITY, l_run = 0.0f;      // m_run in exponent units (score * scale * log2 e)
    bool ok = true;
    for (int j = 0; j < num_tiles; ++j) {
      const int k0 = k_begin + j * BN;
      ok = mbar_wait(s_full + g, j & 1, failed) && ok;
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
      const float tile_max = fmaxf(fmaxf(chunk_max[0], chunk_max[1]), fmaxf(chunk_max[2], chunk_max[3])) * sl2;
      float alpha = 1.0f;
      if (tile_max > m_run + MAX_SLACK) {        // also the first keys a row sees (m_run is -inf until then)
        alpha = le::fast_exp2(m_run - tile_max);
        m_run = tile_max;
      }
      const float neg_m = (m_run == -INFINITY) ? 0.0f : -m_run;
      const float2 neg_m2 = make_float2(neg_m, neg_m);
      if (j > 0) {                               // the product of the tile before has read the probabilities
        ok = mbar_wait(o_done + g, (j - 1) & 1, failed) && ok;
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
          const __nv_bfloat162 both = __floats2bfloat162_rn(x.x, x.y);
          packed[i / 2] = *reinterpret_cast<const uint32_t *>(&both);
        }
        tc_store16(p_tmem + c * 16, packed);
      }
      l_run = l_run * alpha + (sum2.x + sum2.y);
      // (rarely) some row of the warp moved its maximum: rescale the head's accumulator before the next product
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tc_load32(o_col + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc_store32(o_col + c * 32, o);
        }
      }
      tc_wait_stores();
      tc_fence_before();
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      if (lane == 0) mbar_arrive(p_full + g);
    }
    if (ok) ok = mbar_wait(o_done + g, (num_tiles - 1) & 1, failed);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    } else {
      tc_fence_after();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      bf16 *dst = out + (tok0 + r) * out_stride + (head0 + g) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        tc_load32(o_col + c * 32, o);
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            __nv_bfloat162 *pk = reinterpret_cast<__nv_bfloat162 *>(&packed);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              pk[e] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * e]) * inv, __uint_as_float(o[i + 2 * e + 1]) * inv);
            *reinterpret_cast<uint4 *>(dst + c * 32 + i) = packed;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == PRODUCT_WARP) {
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
  const size_t smem = 2 * Q_BYTES + KS * K_BYTES + VS * V_BYTES + 1024 + 256;   // 1024 to align, 256 for the barriers
  cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return le::invalid("le_attention_prefill_tc_bf16: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  const int group = num_heads / num_kv_heads;
  if (num_tiles > 65535) return le::invalid("le_attention_prefill_tc_bf16: %d tiles of queries are too many for one launch", num_tiles);
  dim3 grid(num_kv_heads * ((group + 1) / 2), num_tiles);   // two heads of a group per block
  return le::launch_chained(attention_tc_kernel, grid, dim3(THREADS), smem, stream, map_q, map_k, map_v, static_cast<bf16 *>(out),
                            out_stride, block_table, max_blocks, cu_q, ctx_before, tile_request, tile_q0, num_heads,
                            num_kv_heads, page_size, tc_page_shift_of(page_size), num_pages, window, scale, status);
}

#else

LE_API int le_attention_tc_available(int) { return 0; }

#endif
