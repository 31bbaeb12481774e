// out[M, N] = x[M, K] W[N, K]^T in bfloat16 on the fifth-generation tensor
// cores: the matrix products of prompt portions (many rows).
//
// One block computes a 128 x BN tile of the output (BN = 128 or 256).  Warp 0
// is the producer: one thread issues TMA tile loads (cp.async.bulk.tensor, 128
// byte swizzle) of x and W into a ring of shared-memory stages and arms each
// stage's mbarrier with the bytes to expect.  Warp 1 owns tensor memory: it
// allocates BN columns, and one thread issues tcgen05.mma (128 x BN x 16,
// operands straight from shared memory through matrix descriptors,
// accumulator in tensor memory) four times per stage and commits the stage's
// "empty" barrier, so the producer may refill it while the tensor core still
// works on later stages.  Warps 2-5 are the epilogue: after the last commit
// they read the accumulator with tcgen05.ld (each warp its own 32 lanes = 32
// output rows), convert and store.  Forms: plain (bfloat16 or float32 output)
// and gated (W = [gate rows; up rows]; a block loads 128 gate rows and the 128
// up rows that belong to them as one 256-row operand and writes
// silu(gate) * up), which removes the separate activation pass over 2 I
// columns.
//
// The kernel is persistent (one block per SM walks a list of tiles) and keeps
// two accumulators in tensor memory, so the epilogue of a tile overlaps the
// products of the next.
//
// PAIR form: two blocks on neighbouring SMs (a cluster of two) compute one
// 256 x 256 tile with tcgen05.mma.cta_group::2.  Each block loads its own 128
// rows of x and half of the tile's 256 rows of W (in the gated form the first
// block the gate rows, the second the up rows), so a stage is 32 KB a block
// instead of 48 and six stages fit where four did; the first block's thread
// issues every MMA, which reads W from both blocks' shared memory and writes
// each block's 128 rows of the accumulator into that block's tensor memory.
// Barriers: a stage's "full" barrier lives in the first block and counts both
// blocks' copies; "empty" and "accumulator full" are signalled in both blocks
// by one multicast commit; the epilogue warps of both blocks arrive on the
// first block's "accumulator empty".  The blocks meet at a cluster barrier
// before anything remote is touched and before either leaves.
//
// Every wait on an mbarrier is bounded: when a limit runs out the block sets
// the status word (LE_STATUS_WAIT_TIMEOUT), stops issuing work, lets what is in
// flight land (again bounded), frees its tensor memory and returns.
//
// The reference's projections are nn.Linear calls into the vendor library
// (python/lyapunov_engine/models/llama.py:45-48,112-117,177).
#include "tc_common.cuh"

namespace {

using namespace tc;
using bf16 = __nv_bfloat16;
constexpr int BM = 128;
constexpr int BK = 64;                 // 128 bytes of bfloat16: one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;           // producer warp, MMA warp, four epilogue warps

// ---- a pair of blocks on one tile
// Shared-memory addresses of a block in a cluster carry the block's rank; with this bit cleared an address names
// the same offset in the pair's first block.
constexpr uint32_t FIRST_OF_PAIR = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of both blocks arrives by itself (the roles leave their loops at different times, so warps
// are not converged here).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx_first(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(smem_u32(bar) & FIRST_OF_PAIR), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_first(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & FIRST_OF_PAIR) : "memory");
}
// A tile into this block's shared memory; the bytes count on the first block's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void *smem, const CUtensorMap *map, uint64_t *bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar) & FIRST_OF_PAIR), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, when the MMAs issued so far are done, on the barrier at this offset in both blocks of the pair.
__device__ __forceinline__ void tc_commit_pair(uint64_t *bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

// Tiles in the order the blocks take them: bands of eight tiles of rows, and within a band down the rows first.
// What runs at one time then covers about as many tiles of W as of x (it reads the fewest distinct bytes),
// however many rows x has.
constexpr int BAND = 8;
__device__ __forceinline__ void tile_position(int tile, int tiles_m, int tiles_n, int &m_idx, int &n_idx) {
  const int band_tiles = BAND * tiles_n;
  const int band = tile / band_tiles, within = tile - band * band_tiles;
  const int first_m = band * BAND;
  const int rows = min(BAND, tiles_m - first_m);
  m_idx = first_m + within % rows;
  n_idx = within / rows;
}

// BN: output columns of the MMA.  GATED: the BN-row operand is BN/2 gate rows
// and their BN/2 up rows; a tile then has BN/2 output columns.  STAGES:
// shared-memory stages.  PAIR: two blocks (a cluster) per tile.  The kernel is
// persistent: block (or pair) b takes tiles b, b + the number of blocks (or
// pairs), ...; two accumulators in tensor memory alternate, so the epilogue of
// one tile runs while the tensor core works on the next.
template <int BN, bool GATED, typename TO, int STAGES, bool PAIR>
__global__ void __launch_bounds__(THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TO *__restrict__ out,
               int M, int N, int K, int64_t ldo, int up_row_offset, int tiles_m, int tiles_n, int *__restrict__ status) {
  static_assert(!PAIR || BN == 256, "a pair of blocks computes 256 x 256 tiles");
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;         // rows of W in this block's stage
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int N_TILE = GATED ? BN / 2 : BN;        // output columns per tile
  constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;      // output rows per tile
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
  uint64_t *empty = full + STAGES;
  uint64_t *acc_full = empty + STAGES;               // [2]
  uint64_t *acc_empty = acc_full + 2;                // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_k_tiles = (K + BK - 1) / BK;
  const int num_tiles = tiles_m * tiles_n;
  const int rank = PAIR ? static_cast<int>(cluster_rank()) : 0;           // which block of the pair
  const int first_tile = PAIR ? blockIdx.x >> 1 : blockIdx.x;
  const int tile_step = PAIR ? gridDim.x >> 1 : gridDim.x;

  if (threadIdx.x == 0) {
    // pair: both blocks' producers arrive on the first block's "full"; both blocks' epilogue warps on its "accumulator empty"
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, PAIR ? 2 : 1); mbar_init(empty + s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, PAIR ? 8 : 4); }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();      // the other block's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: one thread keeps the ring of stages full across all of this block's tiles
    if (lane == 0) {
      int issued = 0;
      // launched as a dependent of the kernel before it: what came before this line (barriers, tensor memory)
      // overlapped that kernel's end; x is read only now (every other role works on what these copies bring)
      le::wait_for_predecessor();
      for (int tile = first_tile; tile < num_tiles && !*failed; tile += tile_step) {
        int m_idx, n_idx;
        tile_position(tile, tiles_m, tiles_n, m_idx, n_idx);
        const int m0 = m_idx * TILE_ROWS + rank * BM, n0 = n_idx * N_TILE;
        for (int kt = 0; kt < num_k_tiles; ++kt, ++issued) {
          const int s = issued % STAGES;
          const uint32_t phase = (issued / STAGES) & 1;
          if (*failed || !mbar_wait(empty + s, phase ^ 1, failed)) { *failed = 1; break; }
          unsigned char *a_dst = smem + s * STAGE_BYTES, *b_dst = a_dst + A_BYTES;
          if constexpr (PAIR) {
            // this block's rows of x and its half of the tile's rows of W; the bytes count in the first block
            mbar_expect_tx_first(full + s, STAGE_BYTES);
            tma_load_2d_pair(a_dst, &map_a, full + s, kt * BK, m0);
            const int w_row = GATED ? (rank == 0 ? n0 : up_row_offset + n0) : n0 + rank * B_ROWS;
            tma_load_2d_pair(b_dst, &map_b, full + s, kt * BK, w_row);
            continue;
          }
          mbar_expect_tx(full + s, STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full + s, kt * BK, m0);
          if (GATED) {
            tma_load_2d(b_dst, &map_b, full + s, kt * BK, n0);
            tma_load_2d(b_dst + B_BYTES / 2, &map_b, full + s, kt * BK, up_row_offset + n0);
          } else {
            tma_load_2d(b_dst, &map_b, full + s, kt * BK, n0);
          }
        }
      }
      if (*failed) {
        // let the copies already issued land before the block goes away (the second block of a pair cannot see
        // the barrier they count on; it has waited out its own time limit by now, far longer than a copy takes)
        atomicOr(status, LE_STATUS_WAIT_TIMEOUT);
        volatile int never = 0;
        if (rank == 0)
          for (int i = max(0, issued - STAGES); i < issued; ++i) mbar_wait(full + i % STAGES, (i / STAGES) & 1, &never);
      }
    }
  } else if (warp == 1) {
    // ---- tensor-core issue
    if (lane == 0 && rank == 0) {
      // instruction descriptor: F32 accumulate, BF16 x BF16, both K-major, N >> 3, M >> 4 (the pair's 256 rows)
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                 (static_cast<uint32_t>(TILE_ROWS >> 4) << 24);
      int consumed = 0, local = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++local) {
        const int acc = local & 1;
        // the epilogue must have drained this accumulator (two tiles ago)
        if (*failed || !mbar_wait(acc_empty + acc, ((local >> 1) & 1) ^ 1, failed)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * BN;
        for (int kt = 0; kt < num_k_tiles; ++kt, ++consumed) {
          const int s = consumed % STAGES;
          const uint32_t phase = (consumed / STAGES) & 1;
          if (*failed || !mbar_wait(full + s, phase, failed)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = smem_desc(a_addr + k * UMMA_K * 2), db = smem_desc(b_addr + k * UMMA_K * 2);
            if constexpr (PAIR) tc_mma_pair(tmem_acc, da, db, idesc, (kt > 0 || k > 0) ? 1u : 0u);
            else tc_mma(tmem_acc, da, db, idesc, (kt > 0 || k > 0) ? 1u : 0u);
          }
          // arrives when the MMAs above have read the stage (pair: in both blocks)
          if constexpr (PAIR) tc_commit_pair(empty + s);
          else tc_commit(empty + s);
        }
        if (ok) {                        // arrives when this tile's accumulator is complete
          if constexpr (PAIR) tc_commit_pair(acc_full + acc);
          else tc_commit(acc_full + acc);
        }
      }
      if (!ok) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31, i.e. those rows of the tile
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++local) {
      int m_idx, n_idx;
      tile_position(tile, tiles_m, tiles_n, m_idx, n_idx);
      const int m0 = m_idx * TILE_ROWS + rank * BM, n0 = n_idx * N_TILE;
      const int acc = local & 1;
      const int row = m0 + quarter * 32 + lane;
      bool ok = mbar_wait(acc_full + acc, (local >> 1) & 1, failed);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) { *failed = 1; atomicOr(status, LE_STATUS_WAIT_TIMEOUT); }
        break;
      }
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      TO *dst = out + static_cast<int64_t>(row) * ldo;
      const int n_limit = GATED ? N / 2 : N;
#pragma unroll 1
      for (int c = 0; c < N_TILE; c += 32) {
        uint32_t v[32], u[32];
        tc_load32(lane_addr + c, v);
        if (GATED) tc_load32(lane_addr + BN / 2 + c, u);
        if (row < M) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            const int col = n0 + c + j;
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              f[i] = __uint_as_float(v[j + i]);
              if (GATED) f[i] = f[i] / (1.0f + __expf(-f[i])) * __uint_as_float(u[j + i]);
            }
            if (col + 8 <= n_limit && (reinterpret_cast<uintptr_t>(dst + col) & 15) == 0) {
              if constexpr (sizeof(TO) == 2) {
                uint4 pack;
                __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pack);
#pragma unroll
                for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                *reinterpret_cast<uint4 *>(dst + col) = pack;
              } else {
                *reinterpret_cast<float4 *>(dst + col) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4 *>(dst + col + 4) = make_float4(f[4], f[5], f[6], f[7]);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col + i < n_limit) dst[col + i] = le::from_f32<TO>(f[i]);
            }
          }
        }
      }
      // this warp has read its part of the accumulator: hand it back to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_first(acc_empty + acc);
        else mbar_arrive(acc_empty + acc);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync();      // neither block leaves, or frees tensor memory, while the other may still use it
  if (warp == 1) {
    tc_fence_after();
    if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

int sm_count() {
  static int cached = 0;
  if (cached == 0) {
    int dev = 0, count = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && count > 0) cached = count;
    else cached = 148;
  }
  return cached;
}

// LYAPUNOV_TC_PAIR=0 keeps every product on single SMs.
bool pairs_enabled() {
  static const bool on = [] {
    const char *env = getenv("LYAPUNOV_TC_PAIR");
    return env == nullptr || env[0] != '0';
  }();
  return on;
}

template <int BN, bool GATED, typename TO, bool PAIR = false>
int launch(void *out, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw, int64_t ldo, int *status,
           cudaStream_t stream) {
  // 192 KB of stages either way: one persistent block per SM
  constexpr int STAGES = PAIR ? 6 : (BN == 256 ? 4 : 6);
  constexpr int W_ROWS = PAIR ? BN / 2 : BN;             // rows of W per block and stage
  constexpr int STAGE_BYTES = (BM + W_ROWS) * BK * 2;
  constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;
  const size_t smem = static_cast<size_t>(STAGES) * STAGE_BYTES + 1024 + 256;
  CUtensorMap map_a, map_b;
  int rc = tensor_map(&map_a, x, M, K, ldx, BM);
  if (rc != 0) return rc;
  rc = tensor_map(&map_b, w, N, K, ldw, (GATED || PAIR) ? BN / 2 : BN);
  if (rc != 0) return rc;
  auto kernel = gemm_tc_kernel<BN, GATED, TO, STAGES, PAIR>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return le::invalid("le_gemm_tc_bf16: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  const int n_out = GATED ? N / 2 : N;
  const int n_tile = GATED ? BN / 2 : BN;
  const int tiles_m = (M + TILE_ROWS - 1) / TILE_ROWS, tiles_n = (n_out + n_tile - 1) / n_tile;
  const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n;
  const int sms = sm_count();
  cudaLaunchConfig_t config = {};
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  config.attrs = attr;
  if (le::chaining_enabled()) {
    attr[config.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[config.numAttrs].val.programmaticStreamSerializationAllowed = 1;
    ++config.numAttrs;
  }
  if constexpr (PAIR) {
    attr[config.numAttrs].id = cudaLaunchAttributeClusterDimension;
    attr[config.numAttrs].val.clusterDim.x = 2;
    attr[config.numAttrs].val.clusterDim.y = 1;
    attr[config.numAttrs].val.clusterDim.z = 1;
    ++config.numAttrs;
    // as many pairs as the GPU holds at once (fewer than SMs / 2 where a pair does not fit into what is left of a GPC)
    static int resident_pairs = 0;
    if (resident_pairs == 0) {
      config.gridDim = dim3(sms / 2 * 2);
      int clusters = 0;
      e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &config);
      resident_pairs = (e == cudaSuccess && clusters > 0) ? clusters : sms / 2;
      (void)cudaGetLastError();
    }
    const int pairs = static_cast<int>(tiles < resident_pairs ? tiles : resident_pairs);
    config.gridDim = dim3(2 * pairs);
  } else {
    config.gridDim = dim3(static_cast<int>(tiles < sms ? tiles : sms));
  }
  e = cudaLaunchKernelEx(&config, kernel, map_a, map_b, static_cast<TO *>(out), M, N, K, ldo, GATED ? N / 2 : 0, tiles_m, tiles_n,
                         status);
  if (e != cudaSuccess) return le::invalid("le_gemm_tc_bf16: launch failed: %s", cudaGetErrorString(e));
  return le::launched();
}

}  // namespace

// gated = 0: out[M, N] (bfloat16 or float32) = x W^T.  gated = 1: W is
// [N = 2 I, K] (gate rows, then up rows), out is bfloat16 [M, I] =
// silu(x Wg^T) * (x Wu^T).  Needs K and the leading dimensions of x and W to
// be multiples of 8 and their base addresses 16-byte aligned (TMA).
LE_API int le_gemm_tc_bf16(void *out, int out_dtype, const void *x, const void *w, int M, int N, int K, int64_t ldx, int64_t ldw,
                           int64_t ldo, int gated, int *status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) return le::invalid("le_gemm_tc_bf16: K (%d) and the leading dimensions must be multiples of 8", K);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) return le::invalid("le_gemm_tc_bf16: x and W must be 16-byte aligned");
  // pairs of SMs on 256 x 256 tiles where those give at least half of the pairs a tile and the second block of a
  // pair has rows of its own (with up to 128 rows of x the product is bound by fetching W, which single blocks
  // on narrower tiles do faster: decode of 64 requests 2.45 -> 2.37 ms per step)
  const int64_t pair_tiles = static_cast<int64_t>((M + 2 * BM - 1) / (2 * BM)) * (((gated ? N / 2 : N) + (gated ? 127 : 255)) / (gated ? 128 : 256));
  const bool pair = pairs_enabled() && M > BM && pair_tiles >= 37;
  if (gated) {
    if (out_dtype != LE_BF16 || N % 2) return le::invalid("le_gemm_tc_bf16: the gated form has bfloat16 output and an even N");
    if (pair) return launch<256, true, bf16, true>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
    // a tile's 256 rows of W are 128 gate and 128 up rows; narrower tiles only where the wide ones would leave
    // more than half of the SMs without one (few rows of x: the product is bound by fetching W)
    const int64_t gated_tiles = static_cast<int64_t>((M + BM - 1) / BM) * ((N / 2 + 127) / 128);
    if (gated_tiles >= 74) return launch<256, true, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
    return launch<128, true, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
  }
  // 128 x 256 tiles: an MMA instruction costs about the same to issue whatever its width, so the wide tile is
  // the faster one (measured on every shape of the model, 2,048 to 8,192 rows) unless it leaves more than half
  // of the SMs without a tile
  const int64_t tiles_m = (M + BM - 1) / BM;
  const bool wide = tiles_m * ((N + 255) / 256) >= 74;
  if (pair && out_dtype == LE_BF16) return launch<256, false, bf16, true>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
  if (pair && out_dtype == LE_F32) return launch<256, false, float, true>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
  if (out_dtype == LE_BF16)
    return wide ? launch<256, false, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream)
                : launch<128, false, bf16>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
  if (out_dtype == LE_F32)
    return wide ? launch<256, false, float>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream)
                : launch<128, false, float>(out, x, w, M, N, K, ldx, ldw, ldo, status, stream);
  return le::invalid("le_gemm_tc_bf16: unknown dtype code %d", out_dtype);
}
