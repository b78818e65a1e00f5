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

// The same product for up to 16 rows (single-token steps): a block takes 32 output features and all rows, a thread one
// row and two features, k in slices of 32. What bounds it is not arithmetic but the wait for each slice, so the next
// slice is fetched into registers (16-byte loads) while the current one is multiplied. Same chain per output as above.
constexpr int kRowsBK = 32;

__global__ void __launch_bounds__(256)
gemm_f32_rows_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                     float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
  pdl_enter();
  __shared__ float As[kRowsBK][16 + 1];
  __shared__ float Ws[kRowsBK][32 + 1];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;       // row ty, features 2 * tx and 2 * tx + 1
  const int n0 = blockIdx.x * 32;
  // this thread's share of a slice: four k values of one weight row; threads 0..127 also four of one token row
  const int wr = tid >> 3, wk = (tid & 7) * 4;
  float4 pw, pa;
  auto fetch = [&](int k0) {
    pw = make_float4(0.f, 0.f, 0.f, 0.f);
    pa = make_float4(0.f, 0.f, 0.f, 0.f);
    const int gk = k0 + wk;
    if (n0 + wr < N && gk < K) pw = *reinterpret_cast<const float4*>(W + (size_t)(n0 + wr) * ldw + gk);      // K is a multiple of 4 here
    if (tid < 128 && wr < M && gk < K) pa = *reinterpret_cast<const float4*>(A + (size_t)wr * lda + gk);
  };
  float acc0 = 0.0f, acc1 = 0.0f;
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += kRowsBK) {
    Ws[wk][wr] = pw.x; Ws[wk + 1][wr] = pw.y; Ws[wk + 2][wr] = pw.z; Ws[wk + 3][wr] = pw.w;
    if (tid < 128) { As[wk][wr] = pa.x; As[wk + 1][wr] = pa.y; As[wk + 2][wr] = pa.z; As[wk + 3][wr] = pa.w; }
    __syncthreads();
    if (k0 + kRowsBK < K) fetch(k0 + kRowsBK);
    const int kn = min(kRowsBK, K - k0);
    if (kn == kRowsBK) {
#pragma unroll
      for (int kk = 0; kk < kRowsBK; ++kk) {
        const float av = As[kk][ty];
        acc0 = fmaf(av, Ws[kk][2 * tx], acc0);
        acc1 = fmaf(av, Ws[kk][2 * tx + 1], acc1);
      }
    } else {
      for (int kk = 0; kk < kn; ++kk) {
        const float av = As[kk][ty];
        acc0 = fmaf(av, Ws[kk][2 * tx], acc0);
        acc1 = fmaf(av, Ws[kk][2 * tx + 1], acc1);
      }
    }
    __syncthreads();
  }
  if (ty < M) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int gn = n0 + 2 * tx + j;
      if (gn >= N) continue;
      float v = j ? acc1 : acc0;
      if (bias) v += bias[gn];
      float* c = C + (size_t)ty * ldc + gn;
      *c = accumulate ? *c + v : v;
    }
  }
}

// The same product for many rows: a 128 x 128 tile per block, 8 x 8 outputs per thread (two 4-wide groups of rows
// by two of columns, so that a warp's shared-memory reads are one or two broadcasts and one contiguous run), operands
// brought in 16 k values at a time with 16-byte global loads where the matrices allow it (the next slice is already in
// registers while the current one is multiplied), read back from shared memory as float4. Every output is still one
// thread's own chain acc = fmaf(a[k], w[k], acc) for k = 0, 1, ..., K - 1: bit for bit what the kernel above computes.
constexpr int kBigTile = 128;
constexpr int kBigPad = 4;       // floats between the k-rows of a tile in shared memory: keeps float4 alignment, spreads banks

__global__ void __launch_bounds__(256)
gemm_f32_big_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                    float* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, int accumulate, int vector_loads) {
  pdl_enter();
  __shared__ __align__(16) float As[kBK][kBigTile + kBigPad];
  __shared__ __align__(16) float Ws[kBK][kBigTile + kBigPad];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * kBigTile, n0 = blockIdx.x * kBigTile;
  // this thread's share of a slice: rows lr and lr + 64 of each operand, k values lk .. lk + 3
  const int lr = tid >> 2, lk = (tid & 3) * 4;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  float4 pa[2], pw[2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gm = m0 + lr + 64 * h, gn = n0 + lr + 64 * h, gk = k0 + lk;
      float4 va = make_float4(0.f, 0.f, 0.f, 0.f), vw = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gm < M) {
        const float* src = A + (size_t)gm * lda + gk;
        if (vector_loads && gk + 3 < K) va = *reinterpret_cast<const float4*>(src);
        else {
          if (gk < K) va.x = src[0];
          if (gk + 1 < K) va.y = src[1];
          if (gk + 2 < K) va.z = src[2];
          if (gk + 3 < K) va.w = src[3];
        }
      }
      if (gn < N) {
        const float* src = W + (size_t)gn * ldw + gk;
        if (vector_loads && gk + 3 < K) vw = *reinterpret_cast<const float4*>(src);
        else {
          if (gk < K) vw.x = src[0];
          if (gk + 1 < K) vw.y = src[1];
          if (gk + 2 < K) vw.z = src[2];
          if (gk + 3 < K) vw.w = src[3];
        }
      }
      pa[h] = va;
      pw[h] = vw;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += kBK) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = lr + 64 * h;
      As[lk][r] = pa[h].x; As[lk + 1][r] = pa[h].y; As[lk + 2][r] = pa[h].z; As[lk + 3][r] = pa[h].w;
      Ws[lk][r] = pw[h].x; Ws[lk + 1][r] = pw[h].y; Ws[lk + 2][r] = pw[h].z; Ws[lk + 3][r] = pw[h].w;
    }
    __syncthreads();
    if (k0 + kBK < K) fetch(k0 + kBK);
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Ws[kk][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Ws[kk][64 + tx * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
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
  const bool aligned = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
  if (M <= 16 && aligned) {
    launch(gemm_f32_rows_kernel, dim3((N + 31) / 32), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate);
  } else if (M <= 16) {
    constexpr int BM = 16, BN = 32;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    launch(gemm_f32_kernel<BM, BN, 1, 2>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate);
  } else if (M < 96) {
    constexpr int BM = 64, BN = 64;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    launch(gemm_f32_kernel<BM, BN, 4, 4>, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate);
  } else {
    dim3 grid((N + kBigTile - 1) / kBigTile, (M + kBigTile - 1) / kBigTile);
    SLB_REQUIRE(grid.y < 65536, "gemm_f32: M=%d needs more than 65535 row tiles", M);
    const int vector_loads = (lda % 4 == 0) && (ldw % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    launch(gemm_f32_big_kernel, dim3(grid), dim3(256), 0, s, A, W, bias, C, M, N, K, lda, ldw, ldc, accumulate, vector_loads);
  }
  return check_launch("gemm_f32");
}
