// Next-token choice on the device: argmax, and temperature sampling with the
// reference's top-k and top-p filters.
//
// The reference samples row by row with torch ops and one device-to-host
// transfer per row (python/lyapunov_engine/engine/sampling.py:15-72): greedy
// when temperature < 1e-4 (first maximum), else logits / T, keep values not
// below the k-th largest, drop the sorted tail whose preceding cumulative
// probability exceeds top_p, softmax, one multinomial draw from torch's global
// generator.  Here a cluster of eight blocks handles one row from shared
// memory, nothing is sorted (the two thresholds are found by radix selection
// over the ordered bit patterns of the logits: three histogram passes each),
// the softmax is 32-bit, and the draw is the inverse of the
// cumulative distribution in token order at a uniform number that depends only
// on (seed, index of the sampled token): the result does not depend on what
// else is in the batch.
#include <cooperative_groups.h>

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

// ---- temperature / top-k / top-p sampling.
// A row belongs to a cluster of SAMPLE_BLOCKS thread blocks; each copies its slice of the row into shared
// memory once, and every later pass runs from there.  The blocks exchange what they find through distributed
// shared memory.
//
// The two thresholds need no sort: radix selection over the ordered bit patterns, 11 + 11 + 10 bits.  A level
// makes a histogram (count, and for top-p the probability mass, per digit) of the row's values whose higher
// digits are the ones chosen so far; block 0 adds the blocks' histograms up and picks the digit the threshold
// lies in.  Masses are fixed-point integers (2^-40 of the largest probability), so that sums do not depend on
// the order of the atomic additions.
namespace cg = cooperative_groups;
constexpr int SAMPLE_BLOCKS = 8;
constexpr int RADIX_BINS = 2048;
constexpr float MASS_ONE = 1099511627776.0f;   // 2^40

// The sum of the blocks' histograms, in block 0's (dynamic) shared memory; the others add to it remotely.
struct MergedHistogram {
  unsigned long long mass[RADIX_BINS];
  int count[RADIX_BINS];
};

struct SampleShared {
  unsigned int mass_lo[RADIX_BINS], mass_hi[RADIX_BINS];   // 64-bit sums kept as two words: 32-bit atomics are the fast ones
  int count[RADIX_BINS];
  unsigned long long warp_mass[33];
  int warp_count[33];
  float warp_f[33];
  int warp_i[33];
  // what block 0 decides for all (read by the others through distributed shared memory)
  int digit;
  int count_above;
  unsigned long long mass_above;
  unsigned long long mass_limit;
  // what every block tells the others
  float block_max;
  int block_argmax;
  float block_total;
  float block_z;
  int block_last_kept;
};

__device__ __forceinline__ float prob_of(float x, float row_max, float inv_t) { return expf((x - row_max) * inv_t); }

// One level's histogram of this block's slice.  Values take part when (key & prefix_mask) == prefix and
// key >= min_key.
__device__ void radix_histogram(SampleShared &h, const float *vals, int n, uint32_t prefix_mask, uint32_t prefix, int shift,
                                int bits, uint32_t min_key, bool with_mass, float row_max, float inv_t) {
  const int bins = 1 << bits;
  for (int bin = threadIdx.x; bin < bins; bin += blockDim.x) { h.count[bin] = 0; h.mass_lo[bin] = 0; h.mass_hi[bin] = 0; }
  __syncthreads();
  const int rounds = (n + blockDim.x - 1) / blockDim.x;
  for (int round = 0; round < rounds; ++round) {
    const int i = round * blockDim.x + threadIdx.x;
    bool in = false;
    uint32_t digit = 0;
    unsigned long long m = 0;
    if (i < n) {
      const float x = vals[i];
      const uint32_t key = ordered_key(x);
      in = (key & prefix_mask) == prefix && key >= min_key;
      digit = (key >> shift) & (bins - 1);
      if (in && with_mass) m = __float2ull_rd(prob_of(x, row_max, inv_t) * MASS_ONE);
    }
    // lanes of a warp that fall into the same bin add together, then one of them adds to the bin: the values
    // of a row crowd into few bins at the first level
    const unsigned active = __ballot_sync(0xffffffffu, in);
    if (in) {
      const unsigned peers = __match_any_sync(active, digit);
      const int leader = __ffs(peers) - 1;
      unsigned lo = static_cast<unsigned>(m & 0xfffffu), hi = static_cast<unsigned>(m >> 20);   // 32 sums of 20 bits fit
      if (with_mass) {
        lo = __reduce_add_sync(peers, lo);
        hi = __reduce_add_sync(peers, hi);
      }
      if ((threadIdx.x & 31) == leader) {
        atomicAdd(&h.count[digit], __popc(peers));
        if (with_mass) {
          const unsigned long long sum = (static_cast<unsigned long long>(hi) << 20) + lo;
          const unsigned int add_lo = static_cast<unsigned int>(sum), add_hi = static_cast<unsigned int>(sum >> 32);
          const unsigned int old = atomicAdd(&h.mass_lo[digit], add_lo);
          const unsigned int carry = old + add_lo < old ? 1u : 0u;      // additions with carry commute: the sum is exact
          if (add_hi + carry) atomicAdd(&h.mass_hi[digit], add_hi + carry);
        }
      }
    }
  }
}

// Block 0, on the merged histogram: for every thread the sums over the bins above its own (bins are dealt out
// in order, `per` to a thread), and the total mass.
__device__ void radix_suffix(SampleShared &h, const MergedHistogram &all, int bins, int per, int &count_above_mine,
                             unsigned long long &mass_above_mine, unsigned long long &mass_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  int lc = 0;
  unsigned long long lm = 0;
  for (int j = 0; j < per; ++j) {
    const int bin = threadIdx.x * per + j;
    if (bin < bins) { lc += all.count[bin]; lm += all.mass[bin]; }
  }
  int ic = lc;
  unsigned long long im = lm;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int oc = __shfl_down_sync(0xffffffffu, ic, o);
    const unsigned long long om = __shfl_down_sync(0xffffffffu, im, o);
    if (lane + o < 32) { ic += oc; im += om; }
  }
  if (lane == 0) { h.warp_count[warp] = ic; h.warp_mass[warp] = im; }
  __syncthreads();
  if (warp == 0) {
    const int wc = lane < warps ? h.warp_count[lane] : 0;
    const unsigned long long wm = lane < warps ? h.warp_mass[lane] : 0;
    int sc = wc;
    unsigned long long sm = wm;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int oc = __shfl_down_sync(0xffffffffu, sc, o);
      const unsigned long long om = __shfl_down_sync(0xffffffffu, sm, o);
      if (lane + o < 32) { sc += oc; sm += om; }
    }
    if (lane == 0) h.warp_mass[32] = sm;
    h.warp_count[lane] = sc - wc;          // warps above this one
    h.warp_mass[lane] = sm - wm;
  }
  __syncthreads();
  count_above_mine = (ic - lc) + h.warp_count[warp];
  mass_above_mine = (im - lm) + h.warp_mass[warp];
  mass_total = h.warp_mass[32];
}

// top-k (with_mass false): the largest key c with at least k values >= c.
// top-p (with_mass true): the smallest key c >= min_key for which the mass of the kept values with key > c is
// at most top_p times the mass of all kept values (kept: key >= min_key).
// `merged` is this block's MergedHistogram; block 0's must be all zero on entry and is left so.
__device__ uint32_t radix_select(cg::cluster_group &cluster, SampleShared &h, MergedHistogram *merged, const float *vals, int n,
                                 bool with_mass, int k, float top_p, uint32_t min_key, float row_max, float inv_t) {
  const unsigned rank = cluster.block_rank();
  SampleShared *first = cluster.map_shared_rank(&h, 0);
  MergedHistogram *all = cluster.map_shared_rank(merged, 0);
  uint32_t prefix = 0, prefix_mask = 0;
  const int level_bits[3] = {11, 11, 10};
  int shift = 32;
  for (int level = 0; level < 3; ++level) {
    const int bits = level_bits[level], bins = 1 << bits;
    shift -= bits;
    radix_histogram(h, vals, n, prefix_mask, prefix, shift, bits, min_key, with_mass, row_max, inv_t);
    __syncthreads();
    // what this block found goes to block 0's histogram: few bins are not empty
    for (int bin = threadIdx.x; bin < bins; bin += blockDim.x) {
      const int c = h.count[bin];
      if (c != 0) {
        atomicAdd(&all->count[bin], c);
        if (with_mass) atomicAdd(&all->mass[bin], (static_cast<unsigned long long>(h.mass_hi[bin]) << 32) + h.mass_lo[bin]);
      }
    }
    cluster.sync();                        // every block's share has arrived
    if (rank == 0) {
      const int per = max(1, bins / static_cast<int>(blockDim.x));
      int ca;
      unsigned long long ma, total;
      radix_suffix(h, *merged, bins, per, ca, ma, total);
      if (threadIdx.x == 0) {
        if (level == 0) {
          h.count_above = 0;
          h.mass_above = 0;
          h.mass_limit = with_mass ? __double2ull_rd(static_cast<double>(top_p) * static_cast<double>(total)) : 0;
        }
        h.digit = 0;                       // (stays when no bin crosses: a row whose masses all round to zero)
      }
      __syncthreads();
      const int count_in = h.count_above;
      const unsigned long long mass_in = h.mass_above, limit = h.mass_limit;
      __syncthreads();
      int running_c = count_in + ca;       // what lies in bins above the one looked at
      unsigned long long running_m = mass_in + ma;
      for (int j = per - 1; j >= 0; --j) {
        const int bin = threadIdx.x * per + j;
        if (bin >= bins) continue;
        if (with_mass) {
          const unsigned long long with_bin = running_m + merged->mass[bin];
          if (running_m <= limit && with_bin > limit) { h.digit = bin; h.mass_above = running_m; }
          running_m = with_bin;
        } else {
          const int with_bin = running_c + merged->count[bin];
          if (with_bin >= k && running_c < k) { h.digit = bin; h.count_above = running_c; }
          running_c = with_bin;
        }
        merged->count[bin] = 0;            // ready for the next level
        merged->mass[bin] = 0;
      }
    }
    cluster.sync();                        // block 0 has chosen, and its histogram is empty again
    prefix |= static_cast<uint32_t>(first->digit) << shift;
    prefix_mask |= static_cast<uint32_t>(bins - 1) << shift;
  }
  return prefix > min_key ? prefix : min_key;
}

// An inclusive prefix sum over the block's threads in thread order (fixed tree: the same bits every time).
__device__ float block_inclusive_scan(float v, float *warp_f, float &block_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += up;
  }
  __syncthreads();
  if (lane == 31) warp_f[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? warp_f[lane] : 0.0f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += up;
    }
    warp_f[lane] = w;                       // inclusive over warps
  }
  __syncthreads();
  block_total = warp_f[warps - 1];
  return v + (warp > 0 ? warp_f[warp - 1] : 0.0f);
}

// params per row: temperature, top_p (floats), top_k, seed_lo, seed_hi, counter (ints).
// slice: values per block (a multiple of 4); `staged`: the slice fits in shared memory and is copied there.
__global__ void __launch_bounds__(THREADS)
sample_kernel(int32_t *__restrict__ out, const float *__restrict__ logits, int vocab, int64_t stride, int slice, int staged,
              const float *__restrict__ temperature, const float *__restrict__ top_p, const int32_t *__restrict__ top_k,
              const int32_t *__restrict__ seeds, const float *__restrict__ uniforms, float *__restrict__ probs_out) {
  extern __shared__ __align__(16) unsigned char dynamic_smem[];
  MergedHistogram *merged = reinterpret_cast<MergedHistogram *>(dynamic_smem);
  float *slice_smem = reinterpret_cast<float *>(dynamic_smem + sizeof(MergedHistogram));
  __shared__ SampleShared sh;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const int r = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *row = logits + r * stride;
  const int begin = min(vocab, rank * slice);
  const int n = min(slice, vocab - begin);
  const float temp = temperature[r];

  // ---- this block's slice into shared memory; its maximum (first index on ties)
  const float *vals = row + begin;
  if (staged) {
    if ((reinterpret_cast<uintptr_t>(row + begin) & 15) == 0) {       // 16 bytes at a time, several in flight
      const float4 *src = reinterpret_cast<const float4 *>(row + begin);
      float4 *dst = reinterpret_cast<float4 *>(slice_smem);
      const int quads = n / 4;
#pragma unroll 4
      for (int i = threadIdx.x; i < quads; i += blockDim.x) dst[i] = src[i];
      for (int i = quads * 4 + threadIdx.x; i < n; i += blockDim.x) slice_smem[i] = row[begin + i];
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) slice_smem[i] = row[begin + i];
    }
    vals = slice_smem;
  }
  if (rank == 0)
    for (int bin = threadIdx.x; bin < RADIX_BINS; bin += blockDim.x) { merged->count[bin] = 0; merged->mass[bin] = 0; }
  __syncthreads();
  {
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float x = vals[i];
      if (x > best || (x == best && begin + i < idx)) { best = x; idx = begin + i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    }
    if (lane == 0) { sh.warp_f[warp] = best; sh.warp_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
      const int warps = (blockDim.x + 31) >> 5;
      best = lane < warps ? sh.warp_f[lane] : -INFINITY;
      idx = lane < warps ? sh.warp_i[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
      }
      if (lane == 0) { sh.block_max = best; sh.block_argmax = idx; }
    }
  }
  cluster.sync();
  float row_max = -INFINITY;
  int best = 0x7fffffff;
  for (int other = 0; other < SAMPLE_BLOCKS; ++other) {
    const SampleShared *theirs = cluster.map_shared_rank(&sh, other);
    const float m = theirs->block_max;
    const int i = theirs->block_argmax;
    if (m > row_max || (m == row_max && i < best)) { row_max = m; best = i; }
  }
  if (temp < 1e-4f) {
    if (rank == 0 && threadIdx.x == 0) out[r] = best;
    if (probs_out)
      for (int i = threadIdx.x; i < n; i += blockDim.x) probs_out[static_cast<int64_t>(r) * vocab + begin + i] = begin + i == best ? 1.0f : 0.0f;
    cluster.sync();                        // nobody leaves while its shared memory may still be read
    return;
  }
  const float inv_t = 1.0f / temp;

  // ---- the thresholds: values whose ordered key is >= keep_key stay
  uint32_t keep_key = 0;
  const int k = top_k[r];
  if (k > 0 && k < vocab) keep_key = radix_select(cluster, sh, merged, vals, n, false, k, 1.0f, 0u, row_max, inv_t);
  const float p_keep = top_p[r];
  if (p_keep < 1.0f) keep_key = radix_select(cluster, sh, merged, vals, n, true, 0, p_keep, keep_key, row_max, inv_t);

  // ---- the kept mass in token order: a thread takes a run of consecutive values of the slice
  const int chunk = (slice + blockDim.x - 1) / blockDim.x;
  const int c_begin = min(n, static_cast<int>(threadIdx.x) * chunk), c_end = min(n, c_begin + chunk);
  float mine = 0.0f;
  int last_kept = -1;
  for (int i = c_begin; i < c_end; ++i)
    if (ordered_key(vals[i]) >= keep_key) { mine += prob_of(vals[i], row_max, inv_t); last_kept = begin + i; }
  float mine_total;
  const float upto_me = block_inclusive_scan(mine, sh.warp_f, mine_total);   // mass of this block's threads 0 .. this one
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) last_kept = max(last_kept, __shfl_xor_sync(0xffffffffu, last_kept, o));
  if (lane == 0) sh.warp_i[warp] = last_kept;
  __syncthreads();
  if (threadIdx.x == 0) {
    sh.block_total = mine_total;
    int last = -1;
    for (int w = 0; w < (blockDim.x + 31) >> 5; ++w) last = max(last, sh.warp_i[w]);
    sh.block_last_kept = last;
    sh.digit = 0x7fffffff;                 // (reused below: the first thread past the target)
  }
  cluster.sync();
  float before = 0.0f, total = 0.0f;       // mass of the blocks before this one, and of all
  int last_of_all = best;
  bool mass_after_me = false;
  for (int other = 0; other < SAMPLE_BLOCKS; ++other) {
    const SampleShared *theirs = cluster.map_shared_rank(&sh, other);
    const float t = theirs->block_total;
    if (other == rank) before = total;
    if (other > rank && t > 0.0f) mass_after_me = true;
    total += t;
    if (theirs->block_last_kept >= 0) last_of_all = theirs->block_last_kept;
  }

  if (probs_out)
    for (int i = threadIdx.x; i < n; i += blockDim.x)
      probs_out[static_cast<int64_t>(r) * vocab + begin + i] = ordered_key(vals[i]) >= keep_key ? prob_of(vals[i], row_max, inv_t) / total : 0.0f;

  // ---- the draw: the inverse of the cumulative distribution in token order at a uniform number
  const uint64_t seed = (static_cast<uint64_t>(static_cast<uint32_t>(seeds[3 * r + 1])) << 32) | static_cast<uint32_t>(seeds[3 * r]);
  const float u = uniforms ? uniforms[r] : uniform_from(seed, static_cast<uint32_t>(seeds[3 * r + 2]));
  const float target = u * total;
  // the block the target falls into; the last block with mass also takes a target that rounding put past the end
  const bool here = mine_total > 0.0f && target >= before && (target < before + mine_total || !mass_after_me);
  if (here) {
    // the first thread whose running mass passes the target searches its run
    if (mine > 0.0f && before + upto_me > target) atomicMin(&sh.digit, static_cast<int>(threadIdx.x));
    __syncthreads();
    const int owner = sh.digit;
    if (owner == 0x7fffffff) {
      if (threadIdx.x == 0) out[r] = sh.block_last_kept >= 0 ? sh.block_last_kept : last_of_all;
    } else if (static_cast<int>(threadIdx.x) == owner) {
      float cum = before + (upto_me - mine);
      int choice = -1, seen = -1;
      for (int i = c_begin; i < c_end; ++i) {
        if (ordered_key(vals[i]) < keep_key) continue;
        seen = begin + i;
        cum += prob_of(vals[i], row_max, inv_t);
        if (cum > target) { choice = begin + i; break; }
      }
      out[r] = choice >= 0 ? choice : seen;
    }
  }
  cluster.sync();                          // nobody leaves while its shared memory may still be read
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
  if (num_rows > 65535) return le::invalid("le_sample: too many rows for one launch");
  int slice = (vocab + SAMPLE_BLOCKS - 1) / SAMPLE_BLOCKS;
  slice = (slice + 3) / 4 * 4;
  // the slice is copied into shared memory where it fits beside the histograms (vocabularies up to about 300,000)
  const size_t slice_bytes = static_cast<size_t>(slice) * sizeof(float);
  const int staged = slice_bytes <= 152 * 1024 ? 1 : 0;
  const size_t smem = sizeof(MergedHistogram) + (staged ? slice_bytes : 0);
  {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return le::invalid("le_sample: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(SAMPLE_BLOCKS, num_rows);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = SAMPLE_BLOCKS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&config, sample_kernel, out, logits, vocab, stride, slice, staged, temperature, top_p, top_k, seeds,
                                     uniforms, probs_out);
  if (e != cudaSuccess) return le::invalid("le_sample: %s", cudaGetErrorString(e));
  return le::launched();
}
