// Next-token choice on the device: argmax, and temperature sampling with the
// reference's top-k and top-p filters.
//
// The reference samples row by row with torch ops and one device-to-host
// transfer per row (python/lyapunov_engine/engine/sampling.py:15-72): greedy
// when temperature < 1e-4 (first maximum), else logits / T, keep values not
// below the k-th largest, drop the sorted tail whose preceding cumulative
// probability exceeds top_p, softmax, one multinomial draw from torch's global
// generator.  Here one block handles one row, nothing is sorted (the two
// thresholds are found by bisection over the ordered bit patterns of the
// logits), the softmax is 32-bit, and the draw is the inverse of the
// cumulative distribution in token order at a uniform number that depends only
// on (seed, index of the sampled token): the result does not depend on what
// else is in the batch.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t ordered_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

__device__ __forceinline__ float uniform_from(uint64_t seed, uint64_t counter) {
  const uint64_t r = splitmix64(splitmix64(seed) ^ (counter * 0xD1342543DE82EF95ull + 1));
  return static_cast<float>(r >> 40) * (1.0f / 16777216.0f);  // 24 bits, in [0, 1)
}

__device__ __forceinline__ int block_sum_int(int v, int *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int s = scratch[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}

// First index of the row's maximum.
__device__ int block_argmax(const float *row, int vocab, float *fs, int *is) {
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float x = row[i];
    if (x > best || (x == best && i < idx)) { best = x; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { fs[warp] = best; is[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    best = lane < warps ? fs[lane] : -INFINITY;
    idx = lane < warps ? is[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if (lane == 0) { is[32] = idx; fs[32] = best; }
  }
  __syncthreads();
  return is[32];
}

__global__ void __launch_bounds__(THREADS) argmax_kernel(int32_t *__restrict__ out, const float *__restrict__ logits,
                                                         int vocab, int64_t stride) {
  __shared__ float fs[33];
  __shared__ int is[33];
  const int idx = block_argmax(logits + blockIdx.x * stride, vocab, fs, is);
  if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// Two stages for wide vocabularies: blocks of a row's chunks, then one block per row.
constexpr int ARGMAX_CHUNK = 4096;

__global__ void __launch_bounds__(256) argmax_partial_kernel(float *__restrict__ part_val, int32_t *__restrict__ part_idx,
                                                             const float *__restrict__ logits, int vocab, int64_t stride,
                                                             int chunks) {
  __shared__ float fs[33];
  __shared__ int is[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int begin = chunk * ARGMAX_CHUNK;
  const int n = min(ARGMAX_CHUNK, vocab - begin);
  const int idx = block_argmax(logits + row * stride + begin, n, fs, is);
  if (threadIdx.x == 0) {
    part_val[row * chunks + chunk] = fs[32];
    part_idx[row * chunks + chunk] = begin + idx;
  }
}

__global__ void argmax_final_kernel(int32_t *__restrict__ out, const float *__restrict__ part_val,
                                    const int32_t *__restrict__ part_idx, int chunks) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int row = blockIdx.x;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int c = threadIdx.x; c < chunks; c += 32) {
    const float v = part_val[row * chunks + c];
    const int i = part_idx[row * chunks + c];
    if (v > best || (v == best && i < idx)) { best = v; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
  }
  if (threadIdx.x == 0) out[row] = idx;
}

// params per row: temperature, top_p (floats), top_k, seed_lo, seed_hi, counter (ints).
__global__ void __launch_bounds__(THREADS)
sample_kernel(int32_t *__restrict__ out, const float *__restrict__ logits, int vocab, int64_t stride,
              const float *__restrict__ temperature, const float *__restrict__ top_p, const int32_t *__restrict__ top_k,
              const int32_t *__restrict__ seeds, const float *__restrict__ uniforms, float *__restrict__ probs_out) {
  __shared__ float fs[33];
  __shared__ int is[33];
  __shared__ float chunk_sums[THREADS];
  const int r = blockIdx.x;
  const float *row = logits + r * stride;
  const float temp = temperature[r];
  const int best = block_argmax(row, vocab, fs, is);
  if (temp < 1e-4f) {
    if (threadIdx.x == 0) out[r] = best;
    if (probs_out)
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) probs_out[static_cast<int64_t>(r) * vocab + i] = i == best ? 1.0f : 0.0f;
    return;
  }
  const float row_max = fs[32];
  const float inv_t = 1.0f / temp;

  // top-k: the smallest ordered key with at most k - 1 ... no: the k-th largest value.
  uint32_t keep_key = 0;  // values whose ordered key is >= keep_key stay
  const int k = top_k[r];
  if (k > 0 && k < vocab) {
    // largest key c with count(key >= c) >= k
    uint32_t lo = 0, hi = 0xffffffffu;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1;  // upper middle
      int count = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) count += ordered_key(row[i]) >= mid;
      count = block_sum_int(count, is);
      if (count >= k) lo = mid; else hi = mid - 1;
    }
    keep_key = lo;
  }

  // normaliser over what top-k kept
  float z = 0.0f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x)
    if (ordered_key(row[i]) >= keep_key) z += expf((row[i] - row_max) * inv_t);
  z = le::block_sum(z, fs);

  // top-p: the smallest key c for which the mass of keys > c is <= top_p * z
  const float p_keep = top_p[r];
  if (p_keep < 1.0f) {
    uint32_t lo = keep_key, hi = ordered_key(row_max);
    const float limit = p_keep * z;
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      float above = 0.0f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const uint32_t key = ordered_key(row[i]);
        if (key > mid) above += expf((row[i] - row_max) * inv_t);
      }
      above = le::block_sum(above, fs);
      if (above <= limit) hi = mid; else lo = mid + 1;
    }
    keep_key = lo;
    z = 0.0f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
      if (ordered_key(row[i]) >= keep_key) z += expf((row[i] - row_max) * inv_t);
    z = le::block_sum(z, fs);
  }

  if (probs_out) {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
      probs_out[static_cast<int64_t>(r) * vocab + i] =
          ordered_key(row[i]) >= keep_key ? expf((row[i] - row_max) * inv_t) / z : 0.0f;
  }

  // inverse CDF in token order: each thread owns a contiguous chunk
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, static_cast<int>(threadIdx.x) * chunk), end = min(vocab, begin + chunk);
  float mine = 0.0f;
  for (int i = begin; i < end; ++i)
    if (ordered_key(row[i]) >= keep_key) mine += expf((row[i] - row_max) * inv_t);
  chunk_sums[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(seeds[3 * r + 1])) << 32) | static_cast<uint32_t>(seeds[3 * r]);
    const float u = uniforms ? uniforms[r] : uniform_from(seed, static_cast<uint32_t>(seeds[3 * r + 2]));
    float total = 0.0f;
    for (int t = 0; t < blockDim.x; ++t) total += chunk_sums[t];
    const float target = u * total;
    float cum = 0.0f;
    int owner = -1;
    for (int t = 0; t < blockDim.x; ++t) {
      if (chunk_sums[t] > 0.0f && cum + chunk_sums[t] > target) { owner = t; break; }
      cum += chunk_sums[t];
    }
    int choice = best;
    if (owner >= 0) {
      const int b0 = min(vocab, owner * chunk), e0 = min(vocab, b0 + chunk);
      int last_kept = -1;
      choice = -1;
      for (int i = b0; i < e0; ++i) {
        if (ordered_key(row[i]) < keep_key) continue;
        last_kept = i;
        cum += expf((row[i] - row_max) * inv_t);
        if (cum > target) { choice = i; break; }
      }
      if (choice < 0) choice = last_kept >= 0 ? last_kept : best;
    }
    out[r] = choice;
  }
}

}  // namespace

// `scratch` (optional): room for num_rows * ceil(vocab / 4096) floats and as
// many ints after them; with it a wide vocabulary is searched by many blocks.
LE_API int le_argmax(int32_t *out, const float *logits, int num_rows, int vocab, int64_t stride, float *scratch,
                     cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  const int chunks = (vocab + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
  if (scratch == nullptr || chunks < 4) {
    argmax_kernel<<<num_rows, THREADS, 0, stream>>>(out, logits, vocab, stride);
    return le::launched();
  }
  if (num_rows > 65535) return le::invalid("le_argmax: too many rows for one launch");
  float *part_val = scratch;
  int32_t *part_idx = reinterpret_cast<int32_t *>(scratch + static_cast<int64_t>(num_rows) * chunks);
  int rc = le::launch_chained(argmax_partial_kernel, dim3(chunks, num_rows), dim3(256), 0, stream, part_val, part_idx, logits,
                              vocab, stride, chunks);
  if (rc != 0) return rc;
  return le::launch_chained(argmax_final_kernel, dim3(num_rows), dim3(32), 0, stream, out, static_cast<const float *>(part_val),
                            static_cast<const int32_t *>(part_idx), chunks);
}

// seeds: [rows, 3] = seed low word, seed high word, counter.  `uniforms`
// (optional) overrides the generator; `probs_out` (optional, [rows, vocab])
// receives the filtered distribution, for tests.
LE_API int le_sample(int32_t *out, const float *logits, int num_rows, int vocab, int64_t stride,
                     const float *temperature, const float *top_p, const int32_t *top_k, const int32_t *seeds,
                     const float *uniforms, float *probs_out, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  sample_kernel<<<num_rows, THREADS, 0, stream>>>(out, logits, vocab, stride, temperature, top_p, top_k, seeds, uniforms, probs_out);
  return le::launched();
}
