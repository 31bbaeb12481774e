// Shared by every kernel file: the C interface's conventions, element types,
// reductions and the device status word.
//
// Every launcher is `extern "C" int le_*(...)`: raw device pointers, sizes,
// a dtype code and the CUDA stream; it returns 0 or a cudaError_t, or
// LE_INVALID for arguments it refuses (le_last_error() then says why).  No
// launcher allocates or synchronises.
//
// The reference's helpers of the same kind are csrc/include/utils/cuda_utils.cuh
// (CUDA_CHECK, to_float/from_float, warp and block reductions).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define LE_API extern "C" __attribute__((visibility("default")))

enum : int { LE_F32 = 0, LE_BF16 = 1 };
enum : int { LE_INVALID = -1 };

// Bits of the device status word that kernels set instead of faulting.
enum : int {
  LE_STATUS_BAD_TOKEN = 1,     // a token id outside the vocabulary
  LE_STATUS_BAD_PAGE = 2,      // a block table entry outside the pool
  LE_STATUS_BAD_POSITION = 4,  // a position outside the rotary table
  LE_STATUS_WAIT_TIMEOUT = 8,  // a bounded wait inside a kernel ran out
};

namespace le {

inline char *error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int invalid(const char *fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(error_buffer(), 512, fmt, args);
  va_end(args);
  return LE_INVALID;
}

inline int launched() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
  return static_cast<int>(e);
}

// Programmatic dependent launch: a kernel launched with launch_chained() may
// start while its predecessor in the stream still runs.  It must call
// wait_for_predecessor() before it reads anything the predecessor wrote and
// before it writes anything the predecessor may still read; what it does
// before that (address arithmetic, fetching weights) overlaps the predecessor's
// tail.  let_successor_start() lets the next kernel in the stream begin its own
// preamble.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void wait_for_predecessor() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void let_successor_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool chaining_enabled() {
  static const bool on = [] {
    const char *env = getenv("LYAPUNOV_PDL");
    return env == nullptr || env[0] != '0';
  }();
  return on;
}

template <typename... KernelArgs, typename... Args>
inline int launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = chaining_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  if (e != cudaSuccess) {
    snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return launched();
}

// The same for a kernel whose blocks form thread-block clusters of `cluster_x`
// blocks along x (they are scheduled together and can read one another's shared
// memory); more than 8 to a cluster needs the kernel's non-portable attribute.
template <typename... KernelArgs, typename... Args>
inline int launch_chained_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  int cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = chaining_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
  if (e != cudaSuccess) {
    snprintf(error_buffer(), 512, "CUDA: %s", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return launched();
}

// Every thread of every block of the cluster arrives; returns when all have.
// What a block wrote to its shared memory before is visible to the others after.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// A float at the same shared-memory address in block `rank` of the cluster.
__device__ __forceinline__ float cluster_peer_f32(const float *mine, unsigned rank) {
  const uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(mine));
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// 2^x in one instruction (ex2.approx, relative error about 2^-22, results
// below the normal range flush to zero); exp2f() spends several more on them.
// For softmax numerators in the bfloat16 kernels; the 32-bit path uses expf.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread gets it.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < warps ? scratch[lane] : 0.0f;
    s = warp_sum(s);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float s = lane < warps ? scratch[lane] : -INFINITY;
    s = warp_max(s);
    if (lane == 0) scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace le

#define LE_DISPATCH_DTYPE(code, T, ...)                                  \
  do {                                                                   \
    if ((code) == LE_F32) { using T = float; __VA_ARGS__; }              \
    else if ((code) == LE_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return le::invalid("unknown dtype code %d", (code));            \
  } while (0)
