// C[M, N] = A[M, K] * W[N, K]^T on the FP32 FMA pipes: the matrix product of
// the true 32-bit path (no tensor cores, no TF32), and the plain twin of the
// tensor-core products.
//
// Every output element is one chain of fused multiply-adds over k = 0 .. K-1
// in ascending order, so a token's projections are bit-for-bit the same
// whichever rows share its step and wherever its row lies in the batch.
//
// The reference has no matrix-product kernel: its projections are nn.Linear
// (python/lyapunov_engine/models/llama.py:45-48,112-117,177).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TI, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(TC *__restrict__ C, const TI *__restrict__ A, const TI *__restrict__ W,
                                                        int M, int N, int K, int64_t lda, int64_t ldw, int64_t ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid / 4, lk = (tid % 4) * 4;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int k = k0 + lk + v;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + v][lrow] = (am < M && k < K) ? le::to_f32(A[am * lda + k]) : 0.0f;
      Ws[lk + v][lrow] = (wn < N && k < K) ? le::to_f32(W[wn * ldw + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[m * ldc + n] = le::from_f32<TC>(acc[i][j]);
    }
  }
}

}  // namespace

// Inputs of one type (f32 or bf16), 32-bit accumulation, output f32 or bf16.
// Leading dimensions are in elements.
LE_API int le_gemm_simt(void *C, int c_dtype, const void *A, const void *W, int in_dtype, int M, int N, int K,
                        int64_t lda, int64_t ldw, int64_t ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return le::invalid("le_gemm_simt: K must be positive");
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return le::invalid("le_gemm_simt: M = %d is too large for one launch", M);
#define LE_GO(TI, TC) gemm_simt_kernel<TI, TC><<<grid, 256, 0, stream>>>(static_cast<TC *>(C), static_cast<const TI *>(A), static_cast<const TI *>(W), M, N, K, lda, ldw, ldc)
  if (in_dtype == LE_F32 && c_dtype == LE_F32) LE_GO(float, float);
  else if (in_dtype == LE_BF16 && c_dtype == LE_F32) LE_GO(__nv_bfloat16, float);
  else if (in_dtype == LE_BF16 && c_dtype == LE_BF16) LE_GO(__nv_bfloat16, __nv_bfloat16);
  else return le::invalid("le_gemm_simt: unsupported dtypes in %d out %d", in_dtype, c_dtype);
#undef LE_GO
  return le::launched();
}
