// Matrix product for a handful of rows: C[M, N] = X[M, K] * W[N, K]^T with M <= 64, bfloat16 in, float32 accumulation.
//
// A decode step multiplies a few token rows by every weight matrix, so the time is the time to stream the weights
// from memory once. The kernel is built around that: each lane fetches 16 contiguous bytes of a weight row straight
// from global memory into the register layout the tensor core wants, every weight byte is read exactly once, and a
// block asks for its whole weight tile before it computes, so that many loads are in flight on every SM.
//
// Mapping. mma.sync m16n8k16 computes D[16 x 8] += A[16 x 16] * B[16 x 8]. Rows of A are the token rows (up to 16), the
// 8 columns of B are 8 weight rows (output features), k runs over the inner dimension. In the instruction's
// register layout lane (g, t) holds the k indices {2t, 2t+1, 2t+8, 2t+9} of A rows g, g+8 and of B column g. The sum
// over k does not care about order, so for a block of 32 k values lane (g, t) may instead hold the 8 consecutive
// values 8t .. 8t+7 (one 16-byte load per row), used as two instructions' worth of operands, as long as A and B use
// the same assignment, which they do here.
//
// A block owns NF * 8 output features and all of K: its 8 warps take one eighth of K each and their partial sums are
// added through shared memory in warp order (a fixed order: the result does not depend on timing). Epilogues: store
// bfloat16, store float32, add into a float32 matrix (the residual stream), or the gated activation
// act = silu(gate) * up for a weight matrix holding the gate rows followed by the up rows
// (sleuth/forge/model/mlp.py:37-40), which a block computes from matching gate and up features.
#include "common.cuh"

namespace slb {

enum SkinnyMode : int { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSwiglu = 3 };

struct SkinnyArgs {
  const float* Xf;          // NORM: the float32 stream [M, K]; rows are normalised on the fly
  const float* gain;        // NORM: [K]
  float eps;
  const __nv_bfloat16* X;   // [M, K]
  const __nv_bfloat16* W;   // [N, K]  (kSwiglu: [2 * inter, K], gate rows then up rows)
  void* C;                  // [M, ldc]
  int M, N, K, ldc;         // kSwiglu: N = inter (features of the output)
};

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kSkinnyWarps = 8;
// Blocks of 32 k values whose weights a warp fetches before it uses any: 8 sixteen-byte loads per lane in flight.
__host__ __device__ constexpr int unroll_for(int tiles) { return tiles >= 8 ? 1 : (tiles >= 4 ? 2 : (tiles >= 2 ? 4 : 8)); }

// NORM: X is not given; instead the block reads the float32 stream and applies the RMSNorm itself,
// y = rmsnorm(x) W^T with rmsnorm(x) = x * gain / sqrt(mean(x^2) + eps) (sleuth/forge/model/norm.py:50). The row
// factor 1/sqrt(..) is a scalar per row, so it is taken out of the product: the tensor cores multiply
// bfloat16(x * gain) and the factor is applied to the float32 sums in the epilogue. The sum of squares is
// gathered from the same loads that feed the product, so the norm costs no extra pass, no extra kernel and no
// wait in front of the product.
// Two blocks per SM are asked for where a warp multiplies a single tile of weight rows (the narrow matrices, whose
// blocks are many and short): measured faster there, slower for the two-tile shapes. Three for the four-tile shape
// that serves very wide matrices (the output matrix over the vocabulary): 80 registers, no spills, 4.9 instead of
// 4.6 TB/s; four would spill.
// MT: token rows come in tiles of 16; MT = 1 serves up to 16 rows, MT = 2 up to 32, MT = 4 up to 64. With MT > 1
// the token fragments are fetched as they are needed (they sit in L1 after the first block of an SM has read them)
// while the weight loads still go out in one batch.
template <int NF, int MODE, bool NORM, int MT>
__global__ void __launch_bounds__(kSkinnyWarps * 32, (MODE != kSwiglu && NF == 1 && MT == 1) ? 2 : ((NF == 4 && MT == 1 && !NORM) ? 3 : 1)) gemm_skinny_kernel(SkinnyArgs a) {
  constexpr int TILES = MODE == kSwiglu ? 2 * NF : NF;       // weight-row tiles of 8 that a warp multiplies
  constexpr int kUnroll = unroll_for(TILES);
  static_assert(MT == 1 || !NORM, "the fused norm is built for up to 16 rows");
  __shared__ float red[kSkinnyWarps][TILES][16 * MT][8 + 1];
  __shared__ float ssq_part[kSkinnyWarps][16];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (NF * 8);
  const int kb_total = a.K / 32;
  const int per = (kb_total + kSkinnyWarps - 1) / kSkinnyWarps;
  const int kb_begin = warp * per, kb_end = min(kb_total, kb_begin + per);

  // weight row of each tile for this lane, or null beyond the matrix
  const __nv_bfloat16* wrow[TILES];
#pragma unroll
  for (int f = 0; f < TILES; ++f) {
    const int feat = n0 + (f % NF) * 8 + g;
    const int row = (MODE == kSwiglu && f >= NF) ? a.N + feat : feat;
    wrow[f] = feat < a.N ? a.W + (size_t)row * a.K + 8 * t : nullptr;
  }
  const __nv_bfloat16* xrow0 = (!NORM && g < a.M) ? a.X + (size_t)g * a.K + 8 * t : nullptr;
  const __nv_bfloat16* xrow1 = (!NORM && g + 8 < a.M) ? a.X + (size_t)(g + 8) * a.K + 8 * t : nullptr;
  const float* frow0 = (NORM && g < a.M) ? a.Xf + (size_t)g * a.K + 8 * t : nullptr;
  const float* frow1 = (NORM && g + 8 < a.M) ? a.Xf + (size_t)(g + 8) * a.K + 8 * t : nullptr;

  float acc[MT][TILES][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int f = 0; f < TILES; ++f) acc[mt][f][0] = acc[mt][f][1] = acc[mt][f][2] = acc[mt][f][3] = 0.0f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 w[kUnroll][TILES];
  auto fetch_weights = [&](int kb) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const bool live = kb + u < kb_end;
      const int off = (kb + u) * 32;
#pragma unroll
      for (int f = 0; f < TILES; ++f) w[u][f] = (live && wrow[f]) ? ldg16(wrow[f] + off) : zero;
    }
  };
  // Weights are written by no kernel, so the first batch of loads goes out before the wait for the kernel that
  // produces X: the memory system is already streaming this layer's weights while the previous kernel finishes.
  pdl_launch_dependents();
  fetch_weights(kb_begin);
  pdl_wait();
  // Adding into the stream: the old values of the outputs this thread will write are asked for now, so that the
  // epilogue does not end on a load from L2.
  constexpr int kOutPerThread = (16 * MT * NF * 8 + kSkinnyWarps * 32 - 1) / (kSkinnyWarps * 32);
  float old_out[kOutPerThread];
  if (MODE == kAddF32) {
#pragma unroll
    for (int i = 0; i < kOutPerThread; ++i) {
      const int idx = threadIdx.x + i * kSkinnyWarps * 32;
      const int r = idx / (NF * 8), feat = n0 + idx % (NF * 8);
      old_out[i] = (idx < 16 * MT * NF * 8 && r < a.M && feat < a.N)
                       ? reinterpret_cast<const float*>(a.C)[(size_t)r * a.ldc + feat] : 0.0f;
    }
  }
  float ssq0 = 0.0f, ssq1 = 0.0f;     // NORM: sums of squares of this lane's share of rows g and g + 8
  for (int kb = kb_begin; kb < kb_end; kb += kUnroll) {
    if (kb != kb_begin) fetch_weights(kb);
    if (MT > 1) {
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (kb + u >= kb_end) break;
        const int off = (kb + u) * 32 + 8 * t;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int r0 = 16 * mt + g, r1 = r0 + 8;
          const uint4 xa = r0 < a.M ? *reinterpret_cast<const uint4*>(a.X + (size_t)r0 * a.K + off) : zero;
          const uint4 xb = r1 < a.M ? *reinterpret_cast<const uint4*>(a.X + (size_t)r1 * a.K + off) : zero;
#pragma unroll
          for (int f = 0; f < TILES; ++f) {
            mma_16816(acc[mt][f], xa.x, xb.x, xa.y, xb.y, w[u][f].x, w[u][f].y);
            mma_16816(acc[mt][f], xa.z, xb.z, xa.w, xb.w, w[u][f].z, w[u][f].w);
          }
        }
      }
      continue;
    }
    uint4 x0[kUnroll], x1[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const bool live = kb + u < kb_end;
      const int off = (kb + u) * 32;
      if (NORM) {
        x0[u] = zero;
        x1[u] = zero;
        if (live) {
          const float4 g0 = *reinterpret_cast<const float4*>(a.gain + off + 8 * t);
          const float4 g1 = *reinterpret_cast<const float4*>(a.gain + off + 8 * t + 4);
          if (frow0) {
            const float4 p = *reinterpret_cast<const float4*>(frow0 + off), q = *reinterpret_cast<const float4*>(frow0 + off + 4);
            ssq0 += (p.x * p.x + p.y * p.y) + (p.z * p.z + p.w * p.w) + (q.x * q.x + q.y * q.y) + (q.z * q.z + q.w * q.w);
            x0[u].x = pack2(p.x * g0.x, p.y * g0.y);
            x0[u].y = pack2(p.z * g0.z, p.w * g0.w);
            x0[u].z = pack2(q.x * g1.x, q.y * g1.y);
            x0[u].w = pack2(q.z * g1.z, q.w * g1.w);
          }
          if (frow1) {
            const float4 p = *reinterpret_cast<const float4*>(frow1 + off), q = *reinterpret_cast<const float4*>(frow1 + off + 4);
            ssq1 += (p.x * p.x + p.y * p.y) + (p.z * p.z + p.w * p.w) + (q.x * q.x + q.y * q.y) + (q.z * q.z + q.w * q.w);
            x1[u].x = pack2(p.x * g0.x, p.y * g0.y);
            x1[u].y = pack2(p.z * g0.z, p.w * g0.w);
            x1[u].z = pack2(q.x * g1.x, q.y * g1.y);
            x1[u].w = pack2(q.z * g1.z, q.w * g1.w);
          }
        }
      } else {
        x0[u] = (live && xrow0) ? *reinterpret_cast<const uint4*>(xrow0 + off) : zero;
        x1[u] = (live && xrow1) ? *reinterpret_cast<const uint4*>(xrow1 + off) : zero;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
      for (int f = 0; f < TILES; ++f) {
        mma_16816(acc[0][f], x0[u].x, x1[u].x, x0[u].y, x1[u].y, w[u][f].x, w[u][f].y);
        mma_16816(acc[0][f], x0[u].z, x1[u].z, x0[u].w, x1[u].w, w[u][f].z, w[u][f].w);
      }
    }
  }

  // accumulator layout: c0, c1 = (row g, cols 2t, 2t+1); c2, c3 = (row g+8, same cols)
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int f = 0; f < TILES; ++f) {
      red[warp][f][16 * mt + g][2 * t] = acc[mt][f][0];
      red[warp][f][16 * mt + g][2 * t + 1] = acc[mt][f][1];
      red[warp][f][16 * mt + g + 8][2 * t] = acc[mt][f][2];
      red[warp][f][16 * mt + g + 8][2 * t + 1] = acc[mt][f][3];
    }
  if (NORM) {
    // the eight warps' slices of K cover every element of rows 0..15 exactly once, so the row sums of squares
    // come from the very loads that fed the product: lanes of a quad, then warps, added in a fixed order
    ssq0 += __shfl_xor_sync(0xffffffffu, ssq0, 1);
    ssq0 += __shfl_xor_sync(0xffffffffu, ssq0, 2);
    ssq1 += __shfl_xor_sync(0xffffffffu, ssq1, 1);
    ssq1 += __shfl_xor_sync(0xffffffffu, ssq1, 2);
    if (t == 0) { ssq_part[warp][g] = ssq0; ssq_part[warp][g + 8] = ssq1; }
  }
  __syncthreads();

#pragma unroll
  for (int i = 0; i < kOutPerThread; ++i) {
    const int idx = threadIdx.x + i * kSkinnyWarps * 32;
    if (idx >= 16 * MT * NF * 8) break;
    const int r = idx / (NF * 8), c = idx % (NF * 8);
    const int feat = n0 + c;
    if (r >= a.M || feat >= a.N) continue;
    const int f = c / 8, cc = c % 8;
    float v = 0.0f;
#pragma unroll
    for (int w8 = 0; w8 < kSkinnyWarps; ++w8) v += red[w8][f][r][cc];
    float inv = 1.0f;
    if (NORM) {
      float ss = 0.0f;
#pragma unroll
      for (int w8 = 0; w8 < kSkinnyWarps; ++w8) ss += ssq_part[w8][r];
      inv = 1.0f / sqrtf(ss / (float)a.K + a.eps);
      v *= inv;
    }
    if (MODE == kSwiglu) {
      float u = 0.0f;
#pragma unroll
      for (int w8 = 0; w8 < kSkinnyWarps; ++w8) u += red[w8][NF + f][r][cc];
      u *= inv;
      v = (v / (1.0f + expf(-v))) * u;
      reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)r * a.ldc + feat] = __float2bfloat16_rn(v);
    } else if (MODE == kStoreBf16) {
      reinterpret_cast<__nv_bfloat16*>(a.C)[(size_t)r * a.ldc + feat] = __float2bfloat16_rn(v);
    } else if (MODE == kStoreF32) {
      reinterpret_cast<float*>(a.C)[(size_t)r * a.ldc + feat] = v;
    } else {
      reinterpret_cast<float*>(a.C)[(size_t)r * a.ldc + feat] = old_out[i] + v;
    }
  }
}

template <int NF, bool NORM, int MT>
static int launch_skinny(const SkinnyArgs& a, int mode, cudaStream_t s) {
  const int blocks = (a.N + NF * 8 - 1) / (NF * 8);
  const int threads = kSkinnyWarps * 32;
  switch (mode) {
    case kStoreBf16: launch_prefetching(gemm_skinny_kernel<NF, kStoreBf16, NORM, MT>, dim3(blocks), dim3(threads), 0, s, a); break;
    case kStoreF32: launch_prefetching(gemm_skinny_kernel<NF, kStoreF32, NORM, MT>, dim3(blocks), dim3(threads), 0, s, a); break;
    case kAddF32: launch_prefetching(gemm_skinny_kernel<NF, kAddF32, NORM, MT>, dim3(blocks), dim3(threads), 0, s, a); break;
    default:
      if constexpr (2 * NF * MT <= 8) {      // gate and up tiles of every row tile must fit the partial-sum buffer
        launch_prefetching(gemm_skinny_kernel<NF, kSwiglu, NORM, MT>, dim3(blocks), dim3(threads), 0, s, a);
      } else {
        return fail(1, "gemm_skinny: the gated epilogue is not built for %d features a block with %d rows", NF * 8, 16 * MT);
      }
      break;
  }
  return check_launch("gemm_skinny");
}

template <bool NORM>
static int dispatch_skinny(const SkinnyArgs& a, int mode, cudaStream_t s) {
  if (a.M > 32) {       // up to 64 rows: 8 or 16 features per block (the partial sums of 64 rows must fit shared memory)
    if (mode == kSwiglu || a.N < 4096) return launch_skinny<1, false, 4>(a, mode, s);
    return launch_skinny<2, false, 4>(a, mode, s);
  }
  if (a.M > 16) {
    if (mode == kSwiglu || a.N < 4096) return launch_skinny<1, false, 2>(a, mode, s);
    return launch_skinny<2, false, 2>(a, mode, s);
  }
  // wide matrices: 16 or 32 features per block; narrow ones: 8, so that enough blocks exist to fill the GPU
  if (mode == kSwiglu) return a.N >= 4096 ? launch_skinny<2, NORM, 1>(a, mode, s) : launch_skinny<1, NORM, 1>(a, mode, s);
  if (a.N >= 32768) return launch_skinny<4, NORM, 1>(a, mode, s);
  if (a.N >= 4096) return launch_skinny<2, NORM, 1>(a, mode, s);
  return launch_skinny<1, NORM, 1>(a, mode, s);
}

}  // namespace slb

using namespace slb;

// 1 when the skinny kernel takes this problem (the caller otherwise uses the library product).
extern "C" int slb_gemm_skinny_supported(int M, int N, int K) {
  return M >= 1 && M <= 64 && K >= 32 && K % 32 == 0 && N >= 1;
}

// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated activation (W holds 2 * N rows, C is [M, N]).
extern "C" int slb_gemm_skinny(const void* X, const void* W, void* C, int M, int N, int K, int ldc, int mode,
                               void* stream) {
  SLB_REQUIRE(slb_gemm_skinny_supported(M, N, K),
              "gemm_skinny: M=%d N=%d K=%d is outside what the kernel takes (1 <= M <= 64, K a multiple of 32)", M, N, K);
  SLB_REQUIRE(mode >= 0 && mode <= 3 && ldc >= N, "gemm_skinny: mode=%d ldc=%d N=%d", mode, ldc, N);
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_skinny: X and W must be 16-byte aligned");
  SkinnyArgs a{};
  a.X = (const __nv_bfloat16*)X; a.W = (const __nv_bfloat16*)W; a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  return dispatch_skinny<false>(a, mode, (cudaStream_t)stream);
}

// The same with the RMSNorm of the input fused in: X is the float32 stream [M, K], rows are normalised with
// `gain` [K] and `eps` and rounded to bfloat16 on the way into the product.
extern "C" int slb_gemm_skinny_norm(const float* X, const float* gain, float eps, const void* W, void* C, int M, int N,
                                    int K, int ldc, int mode, void* stream) {
  SLB_REQUIRE(slb_gemm_skinny_supported(M, N, K) && M <= 16,
              "gemm_skinny: M=%d N=%d K=%d is outside what the kernel with the norm fused in takes (1 <= M <= 16, K a multiple of 32)", M, N, K);
  SLB_REQUIRE(mode >= 0 && mode <= 3 && ldc >= N && eps > 0.0f, "gemm_skinny: mode=%d ldc=%d N=%d eps=%g", mode, ldc, N, (double)eps);
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)gain % 16 == 0),
              "gemm_skinny: X, gain and W must be 16-byte aligned");
  SkinnyArgs a{};
  a.Xf = X; a.gain = gain; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  return dispatch_skinny<true>(a, mode, (cudaStream_t)stream);
}
