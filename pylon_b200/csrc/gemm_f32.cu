// y[M, N] = x[M, K] * W[N, K]^T in true float32: plain FMA on the CUDA cores, float32
// accumulation, no tensor cores and no reduced-precision matrix mode.  This is the matrix
// product of the engine's 32-bit path (raun6k/Pylon runs its float32 model through
// nn.Linear, src/pylon/model/layers.py:17-23,95-106).
//
// Each output element sums its K products in ascending k order inside one thread, so a
// row's result does not depend on which other rows share the launch.
#include "common.cuh"

namespace pylon {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

__global__ void __launch_bounds__(256) gemm_f32_nt_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                          float* __restrict__ y, int M, int N, int K,
                                                          long long ldx, long long ldw, long long ldy) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // Loader mapping: 256 threads cover a 64 x 16 tile, 4 consecutive k per thread.
  const int lrow = tid / 4, lk = (tid % 4) * 4;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lrow, n = n0 + lrow;
      xs[lk + j][lrow] = (m < M && k < K) ? x[(size_t)m * ldx + k] : 0.f;
      ws[lk + j][lrow] = (n < N && k < K) ? w[(size_t)n * ldw + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[k][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tn + j;
      if (n < N) y[(size_t)m * ldy + n] = acc[i][j];
    }
  }
}

}  // namespace pylon

extern "C" int pylon_gemm_f32_nt(const float* x, const float* w, float* y, int M, int N, int K, long long ldx,
                                 long long ldw, long long ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) PYLON_REFUSE("gemm_f32: K = %d", K);
  if (ldx < K || ldw < K || ldy < N) PYLON_REFUSE("gemm_f32: a leading dimension is shorter than its row");
  dim3 grid((N + pylon::BN - 1) / pylon::BN, (M + pylon::BM - 1) / pylon::BM);
  if (grid.y > 65535) PYLON_REFUSE("gemm_f32: M = %d is too large", M);
  pylon::gemm_f32_nt_kernel<<<grid, 256, 0, stream>>>(x, w, y, M, N, K, ldx, ldw, ldy);
  PYLON_CHECK_LAUNCH("gemm_f32");
}
