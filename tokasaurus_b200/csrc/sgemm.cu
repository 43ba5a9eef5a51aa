// True 32-bit matrix product on the FP32 pipes (no tensor cores, no tf32):
//   C[M, N] = A[M, K] * W[N, K]^T        (A, W and C row-major; K contiguous in both operands)
// Every element of C is one sequential float32 FMA chain over K in index order, whatever M is,
// so a token's result does not depend on which other tokens share the batch.
// Any M, N, K >= 1; A and W may have row strides (lda, ldw) larger than K.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256) sgemm_tn_kernel(const float* __restrict__ A, const float* __restrict__ W,
                                                       float* __restrict__ C, int M, int N, int K, int lda, int ldw,
                                                       int ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = tid & 15, ty = tid >> 4;  // outputs rows ty*4.., cols tx*4..
  // loader mapping: 64 rows x 16 k per tile = 1024 elements, 4 per thread
  const int lrow = tid >> 2;       // 0..63
  const int lk = (tid & 3) * 4;    // 0,4,8,12
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + lrow;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int k = k0 + lk + u;
        As[lk + u][lrow] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
      }
      const int n = n0 + lrow;
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int k = k0 + lk + u;
        Ws[lk + u][lrow] = (n < N && k < K) ? W[(size_t)n * ldw + k] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; j++) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; i++) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; j++) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

}  // namespace

TKB_EXPORT int tkb_sgemm_tn_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw,
                                int ldc, void* st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -2;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return -3;
  sgemm_tn_kernel<<<grid, 256, 0, (cudaStream_t)st>>>(A, W, C, M, N, K, lda, ldw, ldc);
  return tkb::launch_status();
}
