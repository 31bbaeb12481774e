// out[M, N] = x[M, K] W[N, K]^T for a handful of rows (M <= 64): the matrix
// products of a decode step, which are bound by the bandwidth at which the
// weights stream from HBM, not by arithmetic.
//
// The weights are the 16-row operand of mma.sync m16n8k16 and the tokens its
// 8 columns, so a few tokens waste no tensor-core rows.  A block owns just 16
// weight rows (so even a 2048-row matrix gives 128 blocks, each streaming long
// contiguous rows) and its four warps split every k-tile between them; their
// partial sums meet in shared memory at the end.  Weights and the matching
// slice of x flow through a cp.async pipeline (eight stages for up to 16 rows
// of the plain forms, else four) in swizzled shared
// memory.  Three forms:
//   * plain:   out (bfloat16 or float32) = x W^T;
//   * split-K: the K range is cut into `splits` slices and slice s writes its
//     partial sums to out[s] (float32 [splits, M, N]); whoever consumes them
//     adds them in a fixed order (the next norm kernel does), so the result
//     does not depend on timing;
//   * gated:   W holds gate rows then up rows ([2 I, K]); the block computes
//     both for its columns and writes silu(gate) * up (bfloat16 [M, I]).
//   * rotary: W is the fused query/key/value projection of an attention layer
//     (plain form, bfloat16).  A block takes 8 columns of the low half of one
//     head and the 8 columns of the high half that rotate with them, so the
//     thread that holds a value also holds its partner: the epilogue rotates
//     queries and keys by the tokens' positions (32-bit table), writes the
//     queries to `out` and keys and values into the paged cache.  No kernel
//     runs between the product and the attention.
// The kernel may start before the kernel that produces x has finished: it
// fetches its first weight tiles, then waits for x.
//
// The reference's projections are nn.Linear calls into the vendor library
// (python/lyapunov_engine/models/llama.py:45-48,112-117,177).
#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int BN = 16;            // weight rows per block

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp16(void *smem, const void *gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void *p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MT: token tiles of 8 (M <= 8 MT).  GATED: gate and up rows, SiLU epilogue.
// What the rotary form needs beyond the product's arguments (rope_kv.cu has the stand-alone kernel).
struct RotaryArgs {
  const float *cos_sin;            // [max_pos, head_dim]: cosines of the head_dim / 2 angles, then sines
  const int32_t *positions;        // [M]
  const int32_t *request_of_token; // [M]
  const int32_t *block_table;      // [requests, max_blocks]
  bf16 *k_cache, *v_cache;         // [pages, kv_heads, page, head_dim]
  int *status;
  int max_blocks, num_heads, num_kv_heads, head_dim, max_pos, page_size, num_pages, write_kv;
};

// BK: k per pipeline stage.
// STAGES: depth of the cp.async pipeline.
// ROTARY: the fused qkv projection with rotation and cache write in the epilogue.
// RG: groups of 16 weight rows a block takes (of the gate rows and of the up rows each, in the gated form).  One
// for up to 16 tokens (two where K is split); with more tokens a block takes two or four groups, so that the slice
// of x it streams beside its weights (every block reads all of x) stays no larger than they are.
template <int MT, int RG, bool GATED, typename TO, int BK, int STAGES, bool ROTARY>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(TO *__restrict__ out, const bf16 *__restrict__ x, const bf16 *__restrict__ w, int M, int N, int K,
                   int64_t ldx, int64_t ldw, int64_t ldo, int k_per_split, int64_t split_stride, int early_successor,
                   RotaryArgs rotary) {
  static_assert(!ROTARY || RG == 1, "the rotary form takes one group of rows a block");
  constexpr int WSETS = GATED ? 2 : 1;
  constexpr int ROWS = BN * RG;                    // weight rows per set and block
  constexpr int CPR = BK / 8;                      // 16-byte chunks per row of a tile
  constexpr int W_STAGE = WSETS * ROWS * BK;       // elements
  constexpr int X_STAGE = MT * 8 * BK;
  constexpr int KSTEPS_PER_WARP = BK / 16 / WARPS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16 *w_smem = reinterpret_cast<bf16 *>(smem_raw);
  bf16 *x_smem = w_smem + STAGES * W_STAGE;
  // chunk c of row r: an XOR swizzle of the low chunk bits keeps the 8 rows of an ldmatrix in different banks
  auto swz = [](int r, int c) { return r * CPR + (c ^ (r & 7)); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * ROWS;                // first output column of this block
  const int split = blockIdx.y;
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int num_tiles = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;
  const int n_out = GATED ? N / 2 : N;             // output columns
  // rotary: the block's 16 weight rows are columns j0 .. j0 + 7 of a head's low half and of its high half
  const int half = ROTARY ? rotary.head_dim / 2 : 0;
  const int rot_head = ROTARY ? (blockIdx.x * 8) / half : 0;
  const int rot_j0 = ROTARY ? (blockIdx.x * 8) % half : 0;

  auto load_w = [&](int stage, int kt) {
    const int k0 = k_begin + kt * BK;
    bf16 *dst = w_smem + stage * W_STAGE;
#pragma unroll
    for (int i = 0; i < WSETS * ROWS * CPR / THREADS; ++i) {
      const int c = tid + i * THREADS;
      const int set = c / (ROWS * CPR), rc = c % (ROWS * CPR);
      const int row = rc / CPR, chunk = rc % CPR;
      const int n = n0 + row;
      const int k = k0 + chunk * 8;
      const bool valid = n < n_out && k < k_end;
      int64_t wrow = GATED ? (set == 0 ? n : n_out + n) : n;
      if constexpr (ROTARY) wrow = rot_head * rotary.head_dim + (row < 8 ? rot_j0 + row : half + rot_j0 + row - 8);
      cp16(dst + set * ROWS * BK + swz(row, chunk) * 8, w + (valid ? wrow * ldw + k : 0), valid);
    }
  };
  auto load_x = [&](int stage, int kt) {
    const int k0 = k_begin + kt * BK;
    bf16 *dst = x_smem + stage * X_STAGE;
#pragma unroll
    for (int i = 0; i < MT * 8 * CPR / THREADS; ++i) {
      const int c = tid + i * THREADS;
      const int row = c / CPR, chunk = c % CPR;
      const int k = k0 + chunk * 8;
      const bool valid = row < M && k < k_end;
      cp16(dst + swz(row, chunk) * 8, x + (valid ? row * ldx + k : 0), valid);
    }
  };

  // When all of this kernel's blocks run at once, the kernel after it may start its own preamble at once too
  // (the next product its first weight tiles, the attention kernel after the rotary form the keys of earlier
  // steps) in whatever room the multiprocessors have left or gain as blocks end; it waits for this kernel's
  // results where it needs them.  A grid of several waves keeps the room for its own blocks and lets the
  // successor start when its main loop is through.
  if (early_successor) le::let_successor_start();
  // the first weight tiles do not depend on the kernel before this one
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_w(s, s);
    cp_commit();
  }
  // rotary: what the epilogue needs to know about this lane's tokens (rows 2t and 2t + 1 of every tile of 8) is
  // asked for now, and is there long before the epilogue
  float rot_cos[MT][2], rot_sin[MT][2];
  int64_t rot_dst[MT][2];                          // where the pair goes: < 0: nowhere
  if constexpr (ROTARY) {
    if (warp == 0) {
      const int g = lane >> 2, t = lane & 3;
      const bool is_q = rot_head < rotary.num_heads;
      const bool is_k = !is_q && rot_head < rotary.num_heads + rotary.num_kv_heads;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int row = m * 8 + 2 * t + q;
          rot_dst[m][q] = -1;
          rot_cos[m][q] = 1.0f, rot_sin[m][q] = 0.0f;
          if (row >= M) continue;
          const int pos = rotary.positions[row];
          if (pos < 0 || pos >= rotary.max_pos) {
            atomicOr(rotary.status, LE_STATUS_BAD_POSITION);
            continue;
          }
          if (is_q || is_k) {
            rot_cos[m][q] = rotary.cos_sin[static_cast<int64_t>(pos) * rotary.head_dim + rot_j0 + g];
            rot_sin[m][q] = rotary.cos_sin[static_cast<int64_t>(pos) * rotary.head_dim + half + rot_j0 + g];
          }
          if (is_q) {
            rot_dst[m][q] = static_cast<int64_t>(row) * ldo + rot_head * rotary.head_dim + rot_j0 + g;
          } else if (rotary.write_kv) {
            const int b = rotary.request_of_token[row];
            const int page = rotary.block_table[static_cast<int64_t>(b) * rotary.max_blocks + pos / rotary.page_size];
            if (page < 0 || page >= rotary.num_pages) {
              atomicOr(rotary.status, LE_STATUS_BAD_PAGE);
              continue;
            }
            const int kvh = is_k ? rot_head - rotary.num_heads : rot_head - rotary.num_heads - rotary.num_kv_heads;
            rot_dst[m][q] = ((static_cast<int64_t>(page) * rotary.num_kv_heads + kvh) * rotary.page_size + pos % rotary.page_size) *
                                rotary.head_dim + rot_j0 + g;
          }
        }
    }
  }
  le::wait_for_predecessor();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_x(s, s);
    cp_commit();
  }

  float acc[WSETS][RG][MT][4];
#pragma unroll
  for (int a = 0; a < WSETS; ++a)
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[a][r][m][0] = acc[a][r][m][1] = acc[a][r][m][2] = acc[a][r][m][3] = 0.0f;

  const int j = lane >> 3;
  for (int kt = 0; kt < num_tiles; ++kt) {
    cp_wait<STAGES - 2>();
    __syncthreads();
    const int nxt = kt + STAGES - 1;
    if (nxt < num_tiles) {
      load_w(nxt % STAGES, nxt);
      load_x(nxt % STAGES, nxt);
    }
    cp_commit();
    const bf16 *ws = w_smem + (kt % STAGES) * W_STAGE;
    const bf16 *xs = x_smem + (kt % STAGES) * X_STAGE;
#pragma unroll
    for (int i = 0; i < KSTEPS_PER_WARP; ++i) {
      const int ks = warp + i * WARPS;             // this warp's k-steps of the tile
      // the tokens' fragments of this k-step once, for every group of weight rows
      uint32_t b[(MT + 1) / 2][4];
      if constexpr (MT == 1) {
        // one token tile: matrices 0 and 1 are (k low, k high) of this k-step; 2 and 3 repeat them
        ldsm4(b[0], xs + swz(lane & 7, ks * 2 + (j & 1)) * 8);
      } else {
#pragma unroll
        for (int m = 0; m < MT; m += 2) {
          const int row = m * 8 + (j >> 1) * 8 + (lane & 7);
          ldsm4(b[m / 2], xs + swz(row, ks * 2 + (j & 1)) * 8);
        }
      }
#pragma unroll
      for (int set = 0; set < WSETS; ++set) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          uint32_t a[4];
          const int row = r * BN + (j & 1) * 8 + (lane & 7);
          ldsm4(a, ws + set * ROWS * BK + swz(row, ks * 2 + (j >> 1)) * 8);
          if constexpr (MT == 1) {
            mma16816(acc[set][r][0], a, b[0][0], b[0][1]);
          } else {
#pragma unroll
            for (int m = 0; m < MT; m += 2) {
              mma16816(acc[set][r][m], a, b[m / 2][0], b[m / 2][1]);
              mma16816(acc[set][r][m + 1], a, b[m / 2][2], b[m / 2][3]);
            }
          }
        }
      }
    }
  }
  cp_wait<0>();
  __syncthreads();
  if (!early_successor) le::let_successor_start();   // only the reduction and the stores are left

  // the four warps hold partial sums over their k-steps: add them in warp order
  float *red = reinterpret_cast<float *>(smem_raw);          // [WARPS][VALUES][32]
  constexpr int VALUES = WSETS * RG * MT * 4;
  auto value_at = [](int set, int r, int m, int e) { return ((r * MT + m) * 4 + e) * WSETS + set; };
#pragma unroll
  for (int a = 0; a < WSETS; ++a)
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[(warp * VALUES + value_at(a, r, m, e)) * 32 + lane] = acc[a][r][m][e];
  __syncthreads();
  // fragment (n, m): c0, c1 at (n = g, m = 2t, 2t + 1); c2, c3 at (n = g + 8, same m)
  const int g = lane >> 2, t = lane & 3;
  if constexpr (ROTARY) {
    if (warp != 0) return;
    // c0 / c1 are the low-half values of tokens 2t / 2t + 1, c2 / c3 their partners in the high half
    const bool is_q = rot_head < rotary.num_heads;
    const bool is_k = !is_q && rot_head < rotary.num_heads + rotary.num_kv_heads;
    bf16 *target = is_q ? reinterpret_cast<bf16 *>(out) : (is_k ? rotary.k_cache : rotary.v_cache);
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        float lo = 0.0f, hi = 0.0f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) {
          lo += red[(wi * VALUES + value_at(0, 0, m, q)) * 32 + lane];
          hi += red[(wi * VALUES + value_at(0, 0, m, 2 + q)) * 32 + lane];
        }
        if (rot_dst[m][q] < 0) continue;
        // the product's output is rounded to bfloat16 as the plain form rounds it, then rotated in 32 bits
        const float x0 = __bfloat162float(__float2bfloat16_rn(lo)), x1 = __bfloat162float(__float2bfloat16_rn(hi));
        const float c = rot_cos[m][q], sn = rot_sin[m][q];
        target[rot_dst[m][q]] = __float2bfloat16_rn(x0 * c - x1 * sn);
        target[rot_dst[m][q] + half] = __float2bfloat16_rn(x1 * c + x0 * sn);
      }
    return;
  }
  // the (group of rows, tile of tokens) pieces of the block's result are shared out over the warps
  TO *dst = out + static_cast<int64_t>(split) * split_stride;
  for (int item = warp; item < RG * MT; item += WARPS) {
    const int r = item / MT, m = item % MT;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v[WSETS];
#pragma unroll
      for (int a = 0; a < WSETS; ++a) {
        v[a] = 0.0f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v[a] += red[(wi * VALUES + value_at(a, r, m, e)) * 32 + lane];
      }
      const int n = n0 + r * BN + g + (e >> 1) * 8;
      const int row = m * 8 + 2 * t + (e & 1);
      if (n < n_out && row < M) {
        float x = v[0];
        if constexpr (GATED) x = x / (1.0f + expf(-x)) * v[WSETS - 1];
        dst[row * ldo + n] = le::from_f32<TO>(x);
      }
    }
  }
}

// Which forms let their successor start at once when their blocks all run at once: bit 0 the rotary form,
// bit 1 the gated form, bit 2 split-K partial sums, bit 3 the plain form.  LYAPUNOV_EARLY_TRIGGER=<mask>;
// 0: every form lets its successor start after its main loop.
inline int early_trigger_mask() {
  static const int mask = [] {
    const char *env = getenv("LYAPUNOV_EARLY_TRIGGER");
    return env == nullptr ? 3 : atoi(env);
  }();
  return mask;
}

// Blocks of one form of the kernel that the device holds at once (asked once per form).
template <typename Kernel>
int64_t resident_blocks(Kernel kernel, size_t smem) {
  int per_sm = 0, device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return static_cast<int64_t>(per_sm) * sms;
}

template <int MT, int RG, bool GATED, typename TO, bool ROTARY, int STAGES>
struct Form {
  static constexpr int WSETS = GATED ? 2 : 1;
  static constexpr int BK = 128;
  static constexpr int ROWS = BN * RG;
  static size_t smem() {
    const size_t pipeline = static_cast<size_t>(STAGES) * (WSETS * ROWS * BK + MT * 8 * BK) * sizeof(bf16);
    const size_t reduce = static_cast<size_t>(WARPS) * WSETS * RG * MT * 4 * 32 * sizeof(float);
    return reduce > pipeline ? reduce : pipeline;
  }
  // 0 when the form cannot get its shared memory
  static int64_t resident() {
    static const int64_t n = [] {
      auto kernel = gemm_skinny_kernel<MT, RG, GATED, TO, BK, STAGES, ROTARY>;
      if (smem() >= 48 * 1024 &&
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem())) != cudaSuccess) {
        cudaGetLastError();
        return int64_t{0};
      }
      return resident_blocks(kernel, smem());
    }();
    return n;
  }
  static int go(void *out, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits,
                int64_t split_stride, cudaStream_t stream, const RotaryArgs &rotary) {
    if (resident() <= 0) return le::invalid("le_gemm_skinny: cannot get %zu bytes of shared memory", smem());
    const int n_out = GATED ? N / 2 : N;
    int k_per_split = (K + splits - 1) / splits;
    k_per_split = (k_per_split + BK - 1) / BK * BK;
    dim3 grid((n_out + ROWS - 1) / ROWS, splits);
    const int form = ROTARY ? 1 : (GATED ? 2 : (splits > 1 ? 4 : 8));
    const int early = (early_trigger_mask() & form) && static_cast<int64_t>(grid.x) * grid.y <= resident() ? 1 : 0;
    return le::launch_chained(gemm_skinny_kernel<MT, RG, GATED, TO, BK, STAGES, ROTARY>, grid, dim3(THREADS), smem(), stream,
                              static_cast<TO *>(out), static_cast<const bf16 *>(x), static_cast<const bf16 *>(w), M, N, K, ldx, ldw,
                              ldo, k_per_split, split_stride, early, rotary);
  }
};

// LYAPUNOV_SKINNY_WIDE_SPLIT_K=0: 16 weight rows a block for up to 16 tokens in every form.
bool wide_split_k_enabled() {
  static const bool on = [] {
    const char *env = getenv("LYAPUNOV_SKINNY_WIDE_SPLIT_K");
    return env == nullptr || env[0] != '0';
  }();
  return on;
}

template <int MT, bool GATED, typename TO, bool ROTARY = false>
int launch(void *out, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits,
           int64_t split_stride, cudaStream_t stream, const RotaryArgs &rotary = RotaryArgs{}) {
  if constexpr (MT <= 2 || ROTARY) {
    // Few rows leave shared memory for a deeper pipeline: more bytes in flight per block (3 % of a decode step).
    // Not for the gated form: with two weight tiles per stage its 512 blocks no longer fit the GPU all at once.
    // (17 stages for the rotary form, so that a block has asked for all of a K of 2048 before it waits for the norm
    // before it, made the step slower, 0.809 -> 0.826 ms at batch 8: the blocks' 96 KB keep the attention kernel
    // that follows from starting beside them and fetching its keys early.)
    constexpr int STAGES = (MT <= 2 && !GATED) ? 8 : 4;
    if constexpr (!GATED && !ROTARY) {
      // Where K is split there are blocks enough for 32 weight rows each: the slice of x that a block streams
      // beside its weights (from L2, every block the same rows) is then half of them (9 to 16 tokens) or a
      // quarter, not their equal or half.  Decode at 16 requests 1.10 -> 1.01 ms, at 8 0.810 -> 0.803, at 1
      // 0.683 -> 0.671.  (Not the gated form: no gain at 9 to 16 tokens, slower below; not the output head's
      // unsplit product: slower up to 8 tokens; 64 rows a block: slower.)
      if (splits > 1 && wide_split_k_enabled())
        return Form<MT, 2, GATED, TO, ROTARY, STAGES>::go(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream, rotary);
    }
    return Form<MT, 1, GATED, TO, ROTARY, STAGES>::go(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream, rotary);
  } else {
    // 17 to 64 tokens: a block takes 64 weight rows where K is split (many blocks anyway), else 32 (or 32 gate and
    // 32 up rows), with as many stages as leave two blocks a multiprocessor
    constexpr int STAGES = MT <= 4 ? 4 : 3;
    if constexpr (!GATED) {
      if (splits > 1)
        return Form<MT, 4, GATED, TO, ROTARY, STAGES>::go(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream, rotary);
    }
    return Form<MT, 2, GATED, TO, ROTARY, STAGES>::go(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream, rotary);
  }
}

template <bool GATED, typename TO>
int dispatch_m(void *out, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits,
               int64_t split_stride, cudaStream_t stream) {
  if (M <= 8) return launch<1, GATED, TO>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
  if (M <= 16) return launch<2, GATED, TO>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
  if (M <= 32) return launch<4, GATED, TO>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
  return launch<8, GATED, TO>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
}

}  // namespace

// gated = 0: out[M, N] (out_dtype bfloat16 or float32) = x W^T; with splits > 1
// out is float32 [splits, M, N] (split s at out + s * split_stride elements).
// gated = 1: W is [N = 2 I, K], out is bfloat16 [M, I]; splits must be 1.
// Needs M <= 64, K a multiple of 8, 16-byte aligned rows of x and W.
LE_API int le_gemm_skinny_bf16(void *out, int out_dtype, const void *x, const void *w, int M, int N, int K, int64_t ldx,
                               int64_t ldw, int64_t ldo, int splits, int64_t split_stride, int gated, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) return le::invalid("le_gemm_skinny_bf16: at most 64 rows, got %d", M);
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) return le::invalid("le_gemm_skinny_bf16: K (%d) and the leading dimensions must be multiples of 8", K);
  if (splits < 1 || splits > 65535) return le::invalid("le_gemm_skinny_bf16: %d splits", splits);
  if (gated) {
    if (splits != 1 || out_dtype != LE_BF16 || N % 2) return le::invalid("le_gemm_skinny_bf16: the gated form has one split, bfloat16 output and an even N");
    return dispatch_m<true, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, 1, 0, stream);
  }
  if (splits > 1 && out_dtype != LE_F32) return le::invalid("le_gemm_skinny_bf16: partial sums of a split K are float32");
  if (out_dtype == LE_F32) return dispatch_m<false, float>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
  if (out_dtype == LE_BF16) return dispatch_m<false, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, splits, split_stride, stream);
  return le::invalid("le_gemm_skinny_bf16: unknown dtype code %d", out_dtype);
}

// The fused query/key/value projection of an attention layer with the rotary
// position encoding and the cache write in its epilogue (at most 64 rows):
//   qkv[t, head h] = rotate(x[t] W_h^T, positions[t]) for the query heads,
//   keys (rotated) and values go to their place in the paged cache
//   [pages, kv_heads, page, head_dim] through the block table (write_kv = 0:
//   they are dropped, the layer reads another layer's cache).
// W is [(heads + 2 kv_heads) head_dim, K]; the whole head rotates (the table
// [max_pos, head_dim] holds head_dim / 2 cosines, then sines, per position);
// head_dim is a multiple of 16.  Same arithmetic and roundings as the plain
// product followed by le_rope_kv_write.
LE_API int le_gemm_skinny_rotary_bf16(void *qkv, const void *x, const void *w, int M, int K, int64_t ldx, int64_t ldw, int64_t ldo,
                                      void *k_cache, void *v_cache, const float *cos_sin, const int32_t *positions,
                                      const int32_t *request_of_token, const int32_t *block_table, int max_blocks,
                                      int num_heads, int num_kv_heads, int head_dim, int max_pos, int page_size, int num_pages,
                                      int write_kv, int *status, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 64) return le::invalid("le_gemm_skinny_rotary_bf16: at most 64 rows, got %d", M);
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) return le::invalid("le_gemm_skinny_rotary_bf16: K (%d) and the leading dimensions must be multiples of 8", K);
  if (head_dim < 16 || head_dim % 16) return le::invalid("le_gemm_skinny_rotary_bf16: head size %d is no multiple of 16", head_dim);
  if (num_heads < 1 || num_kv_heads < 0 || page_size < 1) return le::invalid("le_gemm_skinny_rotary_bf16: bad geometry");
  RotaryArgs r{};
  r.cos_sin = cos_sin, r.positions = positions, r.request_of_token = request_of_token, r.block_table = block_table;
  r.k_cache = static_cast<bf16 *>(k_cache), r.v_cache = static_cast<bf16 *>(v_cache), r.status = status;
  r.max_blocks = max_blocks, r.num_heads = num_heads, r.num_kv_heads = num_kv_heads, r.head_dim = head_dim;
  r.max_pos = max_pos, r.page_size = page_size, r.num_pages = num_pages, r.write_kv = write_kv;
  const int N = (num_heads + 2 * num_kv_heads) * head_dim;
  if (M <= 8) return launch<1, false, bf16, true>(qkv, x, w, M, N, K, ldx, ldw, ldo, 1, 0, stream, r);
  if (M <= 16) return launch<2, false, bf16, true>(qkv, x, w, M, N, K, ldx, ldw, ldo, 1, 0, stream, r);
  if (M <= 32) return launch<4, false, bf16, true>(qkv, x, w, M, N, K, ldx, ldw, ldo, 1, 0, stream, r);
  return launch<8, false, bf16, true>(qkv, x, w, M, N, K, ldx, ldw, ldo, 1, 0, stream, r);
}
