// fp32 matrix product on the CUDA cores (IEEE fused multiply-add, no tf32): the oracle
// configuration of the model on a GPU (fp32 weights, activations and KV cache).  It stands where the
// reference calls cublasSgemm under CUBLAS_PEDANTIC_MATH (src/core/kernels.cu:11-25, 61-89); it is
// not a throughput path.  Operands are addressed through element strides, so all three transposes
// of a linear layer are one kernel:
//
//   C[m, n] = sum_k A[m * sa_m + k * sa_k] * B[k * sb_k + n * sb_n]          (C row-major, pitch ldc)
//
// 64 x 64 output tile per CTA, 16-deep K slices staged in shared memory, 4 x 4 outputs per thread.
#include "common.cuh"

namespace {
constexpr int TS = 64, TK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, long sa_m, long sa_k, const float* __restrict__ B, long sb_k, long sb_n,
                float* __restrict__ C, long ldc, int M, int N, int K) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float As[TK][TS + 1];
  __shared__ float Bs[TK][TS + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += TK) {
    // 64 x 16 elements of each operand, 4 per thread; the faster-varying index follows the smaller stride
    for (int e = threadIdx.x; e < TS * TK; e += 256) {
      int mm, kk;
      if (sa_k == 1) { kk = e % TK; mm = e / TK; } else { mm = e % TS; kk = e / TS; }
      const int m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < M && k < K) ? A[(long)m * sa_m + (long)k * sa_k] : 0.f;
      int nn, kb;
      if (sb_k == 1) { kb = e % TK; nn = e / TK; } else { nn = e % TS; kb = e / TS; }
      const int n = n0 + nn, k2 = k0 + kb;
      Bs[kb][nn] = (n < N && k2 < K) ? B[(long)k2 * sb_k + (long)n * sb_n] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(long)m * ldc + n] = acc[i][j];
    }
  }
}
}  // namespace

extern "C" int kh_gemm_f32(const void* A, long sa_m, long sa_k, const void* B, long sb_k, long sb_n, void* C, long ldc,
                           int M, int N, int K, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) { kh_set_error("gemm_f32: empty problem %dx%dx%d", M, N, K); return -1; }
  dim3 grid((N + TS - 1) / TS, (M + TS - 1) / TS);
  if (grid.y > 65535) { kh_set_error("gemm_f32: M=%d is beyond the grid limit of this oracle kernel", M); return -1; }
  KH_LAUNCH(gemm_f32_kernel, grid, 256, 0, (cudaStream_t)stream, (const float*)A, sa_m, sa_k, (const float*)B, sb_k, sb_n,
                                                          (float*)C, ldc, M, N, K);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kh_set_error("gemm_f32 launch failed: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
