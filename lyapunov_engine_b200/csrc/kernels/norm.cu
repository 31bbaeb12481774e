// RMSNorm over the 32-bit residual stream, with the residual addition fused.
//
//   resid[r] += delta[0][r] + delta[1][r] + ...   (when delta is given)
//   out[r]    = resid[r] * rsqrt(mean(resid[r]^2) + eps) * weight
//
// delta is the output of the sub-layer before the norm: one tensor in the
// activations' type, or the float32 partial sums of a split-K product, which
// are added here in their fixed order.
//
// Sum, mean, rsqrt and the product are 32-bit; the output is rounded once.
// Rows of up to 8192 values are read once and kept in registers between the
// sum of squares and the scaling.
// With `rows` given, only those rows are normed, into consecutive rows of
// `out`, and the residual stream is left as it is (the final norm before the
// output head runs on the wanted rows alone).
//
// Reference: rmsnorm_kernel, csrc/kernels/fused_rmsnorm_swiglu.cu:15-113 (same
// arithmetic; its residual stream has the activations' type, ours is 32-bit).
#include "common.cuh"

namespace {

// VEC values at p (aligned to VEC elements) as floats, in one memory access where VEC is 4.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(float (&dst)[VEC], const T *p) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    dst[0] = a.x, dst[1] = a.y, dst[2] = b.x, dst[3] = b.y;
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) dst[v] = le::to_f32(p[v]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T *p, const float (&src)[VEC]) {
  if constexpr (VEC == 4 && sizeof(T) == 4) {
    *reinterpret_cast<float4 *>(p) = make_float4(src[0], src[1], src[2], src[3]);
  } else if constexpr (VEC == 4 && sizeof(T) == 2) {
    uint2 raw;
    *reinterpret_cast<__nv_bfloat162 *>(&raw.x) = __floats2bfloat162_rn(src[0], src[1]);
    *reinterpret_cast<__nv_bfloat162 *>(&raw.y) = __floats2bfloat162_rn(src[2], src[3]);
    *reinterpret_cast<uint2 *>(p) = raw;
  } else {
#pragma unroll
    for (int v = 0; v < VEC; ++v) p[v] = le::from_f32<T>(src[v]);
  }
}

// PER_THREAD > 0: the row fits in PER_THREAD vectors of VEC values per thread, which stay in registers
// between the sum of squares and the scaling (one pass over memory).  0: any width, two passes.
// PARTIALS > 0: `num_partials` is this number, known when compiling, so that every load of a thread is asked
// for before the first is used (a decode step's norm is one round trip to memory, not one per partial sum).
template <typename TO, typename TD, int VEC, int PER_THREAD, int PARTIALS>
__global__ void rmsnorm_kernel(TO *__restrict__ out, float *__restrict__ resid, const TD *__restrict__ delta,
                               int num_partials, int64_t partial_stride, const float *__restrict__ weight,
                               const int32_t *__restrict__ rows, float eps, int hidden) {
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int64_t src_row = rows ? rows[blockIdx.x] : blockIdx.x;
  float *x = resid + src_row * hidden;
  const TD *d = delta ? delta + src_row * hidden : nullptr;
  TO *o = out + static_cast<int64_t>(blockIdx.x) * hidden;
  const bool write_back = (d != nullptr) && (rows == nullptr);

  if constexpr (PER_THREAD > 0 && PARTIALS > 0) {
    float val[PER_THREAD][VEC], add[PER_THREAD][PARTIALS][VEC], w[PER_THREAD][VEC];
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        load_vec<float, VEC>(val[it], x + i);
        if (d) {
#pragma unroll
          for (int p = 0; p < PARTIALS; ++p) load_vec<TD, VEC>(add[it][p], d + p * partial_stride + i);
        }
        load_vec<float, VEC>(w[it], weight + i);
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        if (d) {
#pragma unroll
          for (int p = 0; p < PARTIALS; ++p)       // in the partial sums' order, as the general form adds them
#pragma unroll
            for (int v = 0; v < VEC; ++v) val[it][v] += add[it][p][v];
        }
        if (write_back) store_vec<float, VEC>(x + i, val[it]);
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss += val[it][v] * val[it][v];
      }
    }
    ss = le::block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
#pragma unroll
        for (int v = 0; v < VEC; ++v) w[it][v] = val[it][v] * inv * w[it][v];
        store_vec<TO, VEC>(o + i, w[it]);
      }
    }
    return;
  }
  if constexpr (PER_THREAD > 0) {
    float val[PER_THREAD][VEC];
    float ss = 0.0f;
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        load_vec<float, VEC>(val[it], x + i);
        if (d)
          for (int p = 0; p < num_partials; ++p) {
            float add[VEC];
            load_vec<TD, VEC>(add, d + p * partial_stride + i);
#pragma unroll
            for (int v = 0; v < VEC; ++v) val[it][v] += add[v];
          }
        if (write_back) store_vec<float, VEC>(x + i, val[it]);
#pragma unroll
        for (int v = 0; v < VEC; ++v) ss += val[it][v] * val[it][v];
      }
    }
    ss = le::block_sum(ss, scratch);
    const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
#pragma unroll
    for (int it = 0; it < PER_THREAD; ++it) {
      const int i = (it * blockDim.x + threadIdx.x) * VEC;
      if (i < hidden) {
        float w[VEC];
        load_vec<float, VEC>(w, weight + i);
#pragma unroll
        for (int v = 0; v < VEC; ++v) w[v] = val[it][v] * inv * w[v];
        store_vec<TO, VEC>(o + i, w);
      }
    }
    return;
  }

  float ss = 0.0f;
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float val = x[i + v];
      if (d)
        for (int p = 0; p < num_partials; ++p) val += le::to_f32(d[p * partial_stride + i + v]);
      if (write_back) x[i + v] = val;
      ss += val * val;
    }
  }
  ss = le::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
  for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float val = x[i + v];
      if (d && !write_back)
        for (int p = 0; p < num_partials; ++p) val += le::to_f32(d[p * partial_stride + i + v]);
      o[i + v] = le::from_f32<TO>(val * inv * weight[i + v]);
    }
  }
}

template <typename TO, typename TD>
int launch(void *out, float *resid, const void *delta, int num_partials, int64_t partial_stride, const float *weight,
           const int32_t *rows, float eps, int num_rows, int hidden, cudaStream_t stream) {
  int threads = 32;
  while (threads < 512 && threads * 8 < hidden) threads *= 2;
#define LE_NORM_P(VEC, PER, PARTIALS)                                                                                  \
  return le::launch_chained(rmsnorm_kernel<TO, TD, VEC, PER, PARTIALS>, dim3(num_rows), dim3(threads), 0, stream,      \
                            static_cast<TO *>(out), resid, static_cast<const TD *>(delta), num_partials, partial_stride, \
                            weight, rows, eps, hidden)
#define LE_NORM(VEC, PER)                                                                                               \
  do {                                                                                                                  \
    if (PER > 0 && PER <= 2) {                                                                                          \
      if (delta == nullptr || num_partials == 1) LE_NORM_P(VEC, PER, 1);                                                \
      if (num_partials == 2) LE_NORM_P(VEC, PER, 2);                                                                    \
      if (num_partials == 3) LE_NORM_P(VEC, PER, 3);                                                                    \
      if (num_partials == 4) LE_NORM_P(VEC, PER, 4);                                                                    \
    }                                                                                                                   \
    LE_NORM_P(VEC, PER, 0);                                                                                             \
  } while (0)
  const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(resid) | reinterpret_cast<uintptr_t>(delta) |
                         reinterpret_cast<uintptr_t>(weight)) & 15) == 0 && partial_stride % 4 == 0;
  if (hidden % 4 == 0 && aligned) {
    const int per_thread = (hidden / 4 + threads - 1) / threads;   // vectors of 4 a thread holds
    if (per_thread <= 2) LE_NORM(4, 2);
    if (per_thread <= 4) LE_NORM(4, 4);
    LE_NORM(4, 0);
  }
  LE_NORM(1, 0);
#undef LE_NORM
#undef LE_NORM_P
}

}  // namespace

// `out_dtype` is the type of `out`; `delta_dtype` that of `delta`, which holds
// `num_partials` tensors of the residual stream's shape, `partial_stride`
// elements apart.
LE_API int le_rmsnorm(void *out, int out_dtype, float *resid, const void *delta, int delta_dtype, int num_partials,
                      int64_t partial_stride, const float *weight, const int32_t *rows, float eps, int num_rows, int hidden,
                      cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden <= 0) return le::invalid("le_rmsnorm: hidden must be positive");
  if (delta != nullptr && num_partials < 1) return le::invalid("le_rmsnorm: num_partials must be at least 1");
#define LE_GO(TO, TD) return launch<TO, TD>(out, resid, delta, num_partials, partial_stride, weight, rows, eps, num_rows, hidden, stream)
  if (out_dtype == LE_F32 && (delta == nullptr || delta_dtype == LE_F32)) LE_GO(float, float);
  if (out_dtype == LE_BF16 && (delta == nullptr || delta_dtype == LE_BF16)) LE_GO(__nv_bfloat16, __nv_bfloat16);
  if (out_dtype == LE_BF16 && delta_dtype == LE_F32) LE_GO(__nv_bfloat16, float);
#undef LE_GO
  return le::invalid("le_rmsnorm: unsupported types: out %d, delta %d", out_dtype, delta_dtype);
}
