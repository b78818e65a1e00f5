// The true 32-bit matrix product: C[M, N] (+)= A[M, K] * W[N, K]^T (+ bias[N]), float32 in, float32 out,
// plain FMA on the CUDA cores. No tensor-core mode of any kind is involved, so nothing is rounded below float32.
//
// Every output element is accumulated by one thread with k ascending from 0 to K-1 (one fmaf per k), whatever the
// tile shape and whatever M is. A row's result therefore does not depend on how many rows run together, which is
// what lets the 32-bit path give the same logits for a whole prompt, for single tokens and for any batch.
// (The reference has no such path on the GPU: its float32 models run under bfloat16 autocast there,
// sleuth/forge/infer/generate.py:76-77.)
#include "common.cuh"

namespace slb {

constexpr int kBK = 16;

template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
  pdl_enter();
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[kBK][BM + 1];
  __shared__ float Ws[kBK][BN + 1];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += kBK) {
    for (int e = tid; e < BM * kBK; e += THREADS) {
      const int m = e / kBK, k = e % kBK;
      const int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? A[(size_t)gm * lda + gk] : 0.0f;
    }
    for (int e = tid; e < BN * kBK; e += THREADS) {
      const int n = e / kBK, k = e % kBK;
      const int gn = n0 + n, gk = k0 + k;
      Ws[k][n] = (gn < N && gk < K) ? W[(size_t)gn * ldw + gk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
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
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      float* c = C + (size_t)gm * ldc + gn;
      *c = accumulate ? *c + v : v;
    }
  }
}

}  // namespace slb

using namespace slb;

extern "C" int slb_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K, int lda,
                            int ldw, int ldc, int accumulate, void* stream) {
  SLB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_f32: M=%d N=%d K=%d", M, N, K);
  SLB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_f32: leading dimensions lda=%d ldw=%d ldc=%d for K=%d N=%d", lda,
              ldw, ldc, K, N);
  if (M == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (M <= 16) {
    constexpr int BM = 16, BN = 32;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    launch(gemm_f32_kernel<BM, BN, 1, 2>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate);
  } else {
    constexpr int BM = 64, BN = 64;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    SLB_REQUIRE(grid.y < 65536, "gemm_f32: M=%d needs more than 65535 row tiles", M);
    launch(gemm_f32_kernel<BM, BN, 4, 4>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate);
  }
  return check_launch("gemm_f32");
}
