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
// BK: k per pipeline stage.
// STAGES: depth of the cp.async pipeline.
template <int MT, bool GATED, typename TO, int BK, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(TO *__restrict__ out, const bf16 *__restrict__ x, const bf16 *__restrict__ w, int M, int N, int K,
                   int64_t ldx, int64_t ldw, int64_t ldo, int k_per_split, int64_t split_stride) {
  constexpr int WSETS = GATED ? 2 : 1;
  constexpr int CPR = BK / 8;                      // 16-byte chunks per row of a tile
  constexpr int W_STAGE = WSETS * BN * BK;         // elements
  constexpr int X_STAGE = MT * 8 * BK;
  constexpr int KSTEPS_PER_WARP = BK / 16 / WARPS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16 *w_smem = reinterpret_cast<bf16 *>(smem_raw);
  bf16 *x_smem = w_smem + STAGES * W_STAGE;
  // chunk c of row r: an XOR swizzle of the low chunk bits keeps the 8 rows of an ldmatrix in different banks
  auto swz = [](int r, int c) { return r * CPR + (c ^ (r & 7)); };

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN;                  // first output column of this block
  const int split = blockIdx.y;
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int num_tiles = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;
  const int n_out = GATED ? N / 2 : N;             // output columns

  auto load_w = [&](int stage, int kt) {
    const int k0 = k_begin + kt * BK;
    bf16 *dst = w_smem + stage * W_STAGE;
#pragma unroll
    for (int i = 0; i < WSETS * BN * CPR / THREADS; ++i) {
      const int c = tid + i * THREADS;
      const int set = c / (BN * CPR), rc = c % (BN * CPR);
      const int row = rc / CPR, chunk = rc % CPR;
      const int n = n0 + row;
      const int k = k0 + chunk * 8;
      const bool valid = n < n_out && k < k_end;
      const int64_t wrow = GATED ? (set == 0 ? n : n_out + n) : n;
      cp16(dst + set * BN * BK + swz(row, chunk) * 8, w + (valid ? wrow * ldw + k : 0), valid);
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

  // the first weight tiles do not depend on the kernel before this one
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_w(s, s);
    cp_commit();
  }
  le::wait_for_predecessor();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_x(s, s);
    cp_commit();
  }

  float acc[WSETS][MT][4];
#pragma unroll
  for (int a = 0; a < WSETS; ++a)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[a][m][0] = acc[a][m][1] = acc[a][m][2] = acc[a][m][3] = 0.0f;

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
      uint32_t a[WSETS][4];
#pragma unroll
      for (int set = 0; set < WSETS; ++set) {
        const int row = (j & 1) * 8 + (lane & 7);
        ldsm4(a[set], ws + set * BN * BK + swz(row, ks * 2 + (j >> 1)) * 8);
      }
      if constexpr (MT == 1) {
        // one token tile: matrices 0 and 1 are (k low, k high) of this k-step; 2 and 3 repeat them
        uint32_t b[4];
        ldsm4(b, xs + swz(lane & 7, ks * 2 + (j & 1)) * 8);
#pragma unroll
        for (int set = 0; set < WSETS; ++set) mma16816(acc[set][0], a[set], b[0], b[1]);
      } else {
#pragma unroll
        for (int m = 0; m < MT; m += 2) {
          uint32_t b[4];
          const int row = m * 8 + (j >> 1) * 8 + (lane & 7);
          ldsm4(b, xs + swz(row, ks * 2 + (j & 1)) * 8);
#pragma unroll
          for (int set = 0; set < WSETS; ++set) {
            mma16816(acc[set][m], a[set], b[0], b[1]);
            mma16816(acc[set][m + 1], a[set], b[2], b[3]);
          }
        }
      }
    }
  }
  cp_wait<0>();
  __syncthreads();
  le::let_successor_start();   // only the reduction and the stores are left

  // the four warps hold partial sums over their k-steps: add them in warp order
  float *red = reinterpret_cast<float *>(smem_raw);          // [WARPS][WSETS * MT * 4][32]
  constexpr int VALUES = WSETS * MT * 4;
#pragma unroll
  for (int a = 0; a < WSETS; ++a)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) red[(warp * VALUES + (a * MT + m) * 4 + e) * 32 + lane] = acc[a][m][e];
  __syncthreads();
  if (warp != 0) return;
  // fragment (n, m): c0, c1 at (n = g, m = 2t, 2t + 1); c2, c3 at (n = g + 8, same m)
  const int g = lane >> 2, t = lane & 3;
  TO *dst = out + static_cast<int64_t>(split) * split_stride;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float v[WSETS];
#pragma unroll
      for (int a = 0; a < WSETS; ++a) {
        v[a] = 0.0f;
#pragma unroll
        for (int wi = 0; wi < WARPS; ++wi) v[a] += red[(wi * VALUES + (a * MT + m) * 4 + e) * 32 + lane];
      }
      const int n = n0 + g + (e >> 1) * 8;
      const int row = m * 8 + 2 * t + (e & 1);
      if (n < n_out && row < M) {
        float r = v[0];
        if constexpr (GATED) r = r / (1.0f + expf(-r)) * v[WSETS - 1];
        dst[row * ldo + n] = le::from_f32<TO>(r);
      }
    }
  }
}

template <int MT, bool GATED, typename TO>
int launch(void *out, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int splits,
           int64_t split_stride, cudaStream_t stream) {
  constexpr int WSETS = GATED ? 2 : 1;
  constexpr int BK = 128;
  // Few rows leave shared memory for a deeper pipeline: more bytes in flight per block (3 % of a decode step).
  // Not for the gated form: with two weight tiles per stage its 512 blocks no longer fit the GPU all at once.
  constexpr int STAGES = (MT <= 2 && !GATED) ? 8 : 4;
  size_t smem = static_cast<size_t>(STAGES) * (WSETS * BN * BK + MT * 8 * BK) * sizeof(bf16);
  const size_t reduce = static_cast<size_t>(WARPS) * WSETS * MT * 4 * 32 * sizeof(float);
  if (reduce > smem) smem = reduce;
  auto kernel = gemm_skinny_kernel<MT, GATED, TO, BK, STAGES>;
  if (smem >= 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return le::invalid("le_gemm_skinny: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  }
  const int n_out = GATED ? N / 2 : N;
  int k_per_split = (K + splits - 1) / splits;
  k_per_split = (k_per_split + BK - 1) / BK * BK;
  dim3 grid((n_out + BN - 1) / BN, splits);
  return le::launch_chained(kernel, grid, dim3(THREADS), smem, stream, static_cast<TO *>(out), static_cast<const bf16 *>(x),
                            static_cast<const bf16 *>(w), M, N, K, ldx, ldw, ldo, k_per_split, split_stride);
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
