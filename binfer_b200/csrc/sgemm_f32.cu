// True 32-bit matrix product for the float32 engine: C[M,N] = A[M,K] * W[N,K]^T.
//
// Plain FP32 FMAs on the CUDA cores; no tensor-core mode of any kind (TF32
// included) is used, so this path shows faults that bfloat16 rounding hides.
// The reference has no 32-bit product at all: every dense product is a cuBLAS
// bf16 call with float accumulation (cuda/kernels/gemm.cu:244-267); the operand
// layout here is the same (weights as stored, [out, in] row-major).
//
// Every output element is summed in one order that depends on K alone, whatever M,
// N or the tile variant, so a token's result does not depend on which other tokens
// share the batch: ascending runs of SG_RUN terms, one fmaf per term, and the runs'
// sums added in ascending order.  (One sequential sum has a rounding error that grows
// with sqrt(K): at the 12288 inner features of the Qwen3-8B shape it stood at 5e-6 of
// the logits' rms.  In runs of 64 it grows with sqrt(64 + K / 64).)
#include "common.cuh"

#define SG_RUN 64

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, long long lda, long long ldw, long long ldc) {
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  static_assert(SG_RUN % BK == 0, "a run is a whole number of K tiles");
  float acc[TM][TN], total[TM][TN];      // the current run's sum; the sum of the runs before
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = total[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += THREADS) {
      const int r = idx / BK, c = idx % BK;
      const int gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.f;
    }
    for (int idx = tid; idx < BN * BK; idx += THREADS) {
      const int r = idx / BK, c = idx % BK;
      const int gn = n0 + r, gk = k0 + c;
      Ws[c][r] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.f;
    }
    __syncthreads();
    // A zero-filled tail (gk >= K) adds +0 terms, which leave every sum unchanged.
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
    if ((k0 + BK) % SG_RUN == 0 || k0 + BK >= K) {      // a run ends (the last may be short)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          total[i][j] += acc[i][j];
          acc[i][j] = 0.f;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = total[i][j];
    }
  }
}

BF_EXPORT int bf_sgemm_nt(const float* A, const float* W, float* C, int M, int N, int K,
                          long long lda, long long ldw, long long ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M <= 16) {
    dim3 grid((N + 63) / 64, (M + 15) / 16);
    sgemm_nt_kernel<16, 64, 16, 1, 4><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
  } else if (M <= 64) {
    dim3 grid((N + 127) / 128, (M + 31) / 32);
    sgemm_nt_kernel<32, 128, 16, 2, 8><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw, ldc);
  } else {
    dim3 grid((N + 127) / 128, (M + 127) / 128);
    sgemm_nt_kernel<128, 128, 16, 8, 8><<<grid, 256, 0, stream>>>(A, W, C, M, N, K, lda, ldw,
                                                                 ldc);
  }
  return bf_launch_status();
}
