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
  NextRead next;            // what the kernel after this one reads, or nothing
  NextPages pages;          // cache pages that the attention kernel after this one reads first, or nothing
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
constexpr int kNormPad = 64;          // bytes between the normalised rows in shared memory, against bank conflicts
constexpr int kNormMaxK = 4096;      // widest stream the fused norm takes (16 rows of it fit shared memory)
// Blocks of 32 k values whose weights a warp fetches before it uses any: 8 sixteen-byte loads per lane in flight.
__host__ __device__ constexpr int unroll_for(int tiles) { return tiles >= 8 ? 1 : (tiles >= 4 ? 2 : (tiles >= 2 ? 4 : 8)); }

// NORM: X is not given; instead the block reads the float32 stream and applies the RMSNorm itself,
// rmsnorm(x) = (x / sqrt(mean(x^2) + eps)) * gain (sleuth/forge/model/norm.py:50): after the wait for the kernel in
// front, each of the eight warps takes a row (two, above eight rows), sums its squares, and writes the normalised
// row as bfloat16 into shared memory, from where all warps then take their token fragments. The weights of the
// first batch are already on their way at that time, so the norm costs no kernel of its own and hides behind
// the weight stream. Every block normalises all rows again (they come from L2): 16 rows of 1,024 are 64 KB.
// Shared memory holds the rows that exist, so that a single wide row does not cost the SM its other blocks.
// Two blocks per SM are asked for where a warp multiplies a single tile of weight rows (the narrow matrices, whose
// blocks are many and short): measured faster there, slower for the two-tile shapes. Three for the four-tile shape
// that serves very wide matrices (the output matrix over the vocabulary): 80 registers, no spills, 4.9 instead of
// 4.6 TB/s; four would spill. Three also for the gated shape with one tile pair per warp: the gate/up product of a
// single-token step has 384 blocks, which then run at once on 148 SMs instead of in two rounds (1.150 -> 1.098 ms a
// step at batch 8).
// MT: token rows come in tiles of 16; MT = 1 serves up to 16 rows, MT = 2 up to 32, MT = 4 up to 64. With MT > 1
// the token fragments are fetched as they are needed (they sit in L1 after the first block of an SM has read them)
// while the weight loads still go out in one batch.
template <int NF, int MODE, bool NORM, int MT>
__global__ void __launch_bounds__(kSkinnyWarps * 32, (MODE != kSwiglu && NF == 1 && MT == 1) ? 2 : (((NF == 4 && MT == 1 && !NORM) || (MODE == kSwiglu && NF == 1 && MT <= 2 && !NORM)) ? 3 : 1)) gemm_skinny_kernel(SkinnyArgs a) {
  Tracer trace(kTraceSkinny);
  constexpr int TILES = MODE == kSwiglu ? 2 * NF : NF;       // weight-row tiles of 8 that a warp multiplies
  constexpr int kUnroll = unroll_for(TILES);
  static_assert(MT == 1 || !NORM, "the fused norm is built for up to 16 rows");
  __shared__ float red[kSkinnyWarps][TILES][16 * MT][8 + 1];
  extern __shared__ __align__(16) unsigned char normed_rows[];      // NORM: [M][K * 2 + kNormPad] bytes
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
  const int norm_stride = a.K * 2 + kNormPad;

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
  if (threadIdx.x == 0) prefetch_share(a.next, blockIdx.x, gridDim.x);
  if (a.pages.k_pool != nullptr && warp == kSkinnyWarps - 1) {
    const int items = a.pages.n_seqs * a.pages.splits * a.pages.depth * 2;
    for (int item = blockIdx.x; item < items; item += gridDim.x) prefetch_page_item(a.pages, item, lane);
  }
  if (NORM) {      // the gains are read after the rows' sums of squares: asked into L1 now, they are there by then
    for (int line = threadIdx.x; line * 32 < a.K; line += kSkinnyWarps * 32)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(a.gain + line * 32));
  }
  pdl_wait();
  trace.mark(1);
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
  if (NORM) {
    for (int r = warp; r < a.M; r += kSkinnyWarps) {
      uint2* dst = reinterpret_cast<uint2*>(normed_rows + (size_t)r * norm_stride);
      const float4* src = reinterpret_cast<const float4*>(a.Xf + (size_t)r * a.K);
      float ss = 0.0f;
      for (int c = lane; c < a.K / 4; c += 32) {
        const float4 v = src[c];
        ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = 1.0f / sqrtf(ss / (float)a.K + a.eps);
      const float4* gn = reinterpret_cast<const float4*>(a.gain);
      for (int c = lane; c < a.K / 4; c += 32) {
        const float4 v = src[c], gv = gn[c];
        dst[c] = make_uint2(pack2((v.x * inv) * gv.x, (v.y * inv) * gv.y), pack2((v.z * inv) * gv.z, (v.w * inv) * gv.w));
      }
    }
    __syncthreads();
  }
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
        const unsigned char* base = normed_rows + (size_t)(off + 8 * t) * 2;
        x0[u] = (live && g < a.M) ? *reinterpret_cast<const uint4*>(base + (size_t)g * norm_stride) : zero;
        x1[u] = (live && g + 8 < a.M) ? *reinterpret_cast<const uint4*>(base + (size_t)(g + 8) * norm_stride) : zero;
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

  trace.mark(2);
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
    if (MODE == kSwiglu) {
      float u = 0.0f;
#pragma unroll
      for (int w8 = 0; w8 < kSkinnyWarps; ++w8) u += red[w8][NF + f][r][cc];
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

template <int NF, int MODE, bool NORM, int MT>
static int launch_skinny_mode(const SkinnyArgs& a, cudaStream_t s) {
  const int blocks = (a.N + NF * 8 - 1) / (NF * 8);
  const size_t smem = NORM ? (size_t)a.M * (a.K * 2 + kNormPad) : 0;     // rows that do not exist multiply as zeros
  if (NORM) {
    static bool configured = false;
    if (!configured) {
      const int most = 16 * (kNormMaxK * 2 + kNormPad);
      cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NF, MODE, NORM, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
      if (e != cudaSuccess) return fail(2, "gemm_skinny: cannot reserve %d bytes of shared memory: %s", most, cudaGetErrorString(e));
      configured = true;
    }
  }
  launch_prefetching(gemm_skinny_kernel<NF, MODE, NORM, MT>, dim3(blocks), dim3(kSkinnyWarps * 32), smem, s, a);
  return check_launch("gemm_skinny");
}

template <int NF, bool NORM, int MT>
static int launch_skinny(const SkinnyArgs& a, int mode, cudaStream_t s) {
  switch (mode) {
    case kStoreBf16: return launch_skinny_mode<NF, kStoreBf16, NORM, MT>(a, s);
    case kStoreF32: return launch_skinny_mode<NF, kStoreF32, NORM, MT>(a, s);
    case kAddF32: return launch_skinny_mode<NF, kAddF32, NORM, MT>(a, s);
    default:
      if constexpr (2 * NF * MT <= 8) {      // gate and up tiles of every row tile must fit the partial-sum buffer
        return launch_skinny_mode<NF, kSwiglu, NORM, MT>(a, s);
      } else {
        return fail(1, "gemm_skinny: the gated epilogue is not built for %d features a block with %d rows", NF * 8, 16 * MT);
      }
  }
}

// `features`: 0 lets the rule below choose how many output features (8, 16 or 32) a block takes; 8, 16 or 32 force it
// (the caller has measured what this matrix likes: see parts/linear.py).
template <bool NORM>
static int dispatch_skinny(const SkinnyArgs& a, int mode, int features, cudaStream_t s) {
  if (a.M > 32) {       // up to 64 rows: 8 or 16 features per block (the partial sums of 64 rows must fit shared memory)
    if (mode == kSwiglu || a.N < 4096) return launch_skinny<1, false, 4>(a, mode, s);
    return launch_skinny<2, false, 4>(a, mode, s);
  }
  if (a.M > 16) {
    if (mode == kSwiglu || a.N < 4096) return launch_skinny<1, false, 2>(a, mode, s);
    return launch_skinny<2, false, 2>(a, mode, s);
  }
  if (features == 8) return launch_skinny<1, NORM, 1>(a, mode, s);
  if (features == 16) return launch_skinny<2, NORM, 1>(a, mode, s);
  if (features == 32 && mode != kSwiglu) return launch_skinny<4, NORM, 1>(a, mode, s);
  // wide matrices: 16 or 32 features per block; narrow ones: 8, so that enough blocks exist to fill the GPU
  if (mode == kSwiglu) return a.N >= 4096 ? launch_skinny<2, NORM, 1>(a, mode, s) : launch_skinny<1, NORM, 1>(a, mode, s);
  if (a.N >= 32768) return launch_skinny<4, NORM, 1>(a, mode, s);
  if (a.N >= 4096) return launch_skinny<2, NORM, 1>(a, mode, s);
  return launch_skinny<1, NORM, 1>(a, mode, s);
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(gemm_skinny)

// 1 when the skinny kernel takes this problem (the caller otherwise uses the library product).
extern "C" int slb_gemm_skinny_supported(int M, int N, int K) {
  return M >= 1 && M <= 64 && K >= 32 && K % 32 == 0 && N >= 1;
}

// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated activation (W holds 2 * N rows, C is [M, N]).
// next / next_bytes: a read-only range (the next kernel's weights) that the blocks ask into L2, or null.
// pages: null, or what the attention kernel that follows this product will read first (see NextPages).
static int take_pages(SkinnyArgs& a, const NextPages* pages) {
  a.pages = NextPages{};
  if (pages == nullptr || pages->k_pool == nullptr) return 0;
  SLB_REQUIRE(pages->v_pool && pages->block_table && pages->past && pages->page_bytes > 0 && pages->page_bytes % 16 == 0 &&
              (uintptr_t)pages->k_pool % 16 == 0 && (uintptr_t)pages->v_pool % 16 == 0 && pages->table_stride > 0 &&
              pages->n_seqs > 0 && pages->splits > 0 && pages->depth > 0 && pages->window >= 0 &&
              pages->page_bytes <= 32 * 32768,
              "gemm_skinny: the description of the pages to prefetch is incomplete");
  a.pages = *pages;
  return 0;
}

extern "C" int slb_gemm_skinny(const void* X, const void* W, void* C, int M, int N, int K, int ldc, int mode,
                               const void* next, long long next_bytes, const NextPages* pages, int features, void* stream) {
  SLB_REQUIRE(slb_gemm_skinny_supported(M, N, K),
              "gemm_skinny: M=%d N=%d K=%d is outside what the kernel takes (1 <= M <= 64, K a multiple of 32)", M, N, K);
  SLB_REQUIRE(mode >= 0 && mode <= 3 && ldc >= N, "gemm_skinny: mode=%d ldc=%d N=%d", mode, ldc, N);
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_skinny: X and W must be 16-byte aligned");
  SkinnyArgs a{};
  a.X = (const __nv_bfloat16*)X; a.W = (const __nv_bfloat16*)W; a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  SLB_REQUIRE(next_bytes >= 0 && (uintptr_t)next % 16 == 0, "gemm_skinny: the range to prefetch must be 16-byte aligned");
  a.next.ptr = (const char*)next; a.next.bytes = next ? next_bytes : 0;
  if (int rc = take_pages(a, pages)) return rc;
  SLB_REQUIRE(features == 0 || features == 8 || features == 16 || features == 32, "gemm_skinny: features per block 0 (rule), 8, 16 or 32, got %d", features);
  return dispatch_skinny<false>(a, mode, features, (cudaStream_t)stream);
}

// The same with the RMSNorm of the input fused in: X is the float32 stream [M, K], rows are normalised with
// `gain` [K] and `eps` and rounded to bfloat16 on the way into the product.
extern "C" int slb_gemm_skinny_norm(const float* X, const float* gain, float eps, const void* W, void* C, int M, int N,
                                    int K, int ldc, int mode, const void* next, long long next_bytes,
                                    const NextPages* pages, int features, void* stream) {
  SLB_REQUIRE(slb_gemm_skinny_supported(M, N, K) && M <= 16 && K <= kNormMaxK,
              "gemm_skinny: M=%d N=%d K=%d is outside what the kernel with the norm fused in takes (1 <= M <= 16, K a multiple of 32, at most %d)",
              M, N, K, kNormMaxK);
  SLB_REQUIRE(mode >= 0 && mode <= 3 && ldc >= N && eps > 0.0f, "gemm_skinny: mode=%d ldc=%d N=%d eps=%g", mode, ldc, N, (double)eps);
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)gain % 16 == 0),
              "gemm_skinny: X, gain and W must be 16-byte aligned");
  SkinnyArgs a{};
  a.Xf = X; a.gain = gain; a.eps = eps; a.W = (const __nv_bfloat16*)W; a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc;
  SLB_REQUIRE(next_bytes >= 0 && (uintptr_t)next % 16 == 0, "gemm_skinny: the range to prefetch must be 16-byte aligned");
  a.next.ptr = (const char*)next; a.next.bytes = next ? next_bytes : 0;
  if (int rc = take_pages(a, pages)) return rc;
  SLB_REQUIRE(features == 0 || features == 8 || features == 16 || features == 32, "gemm_skinny: features per block 0 (rule), 8, 16 or 32, got %d", features);
  return dispatch_skinny<true>(a, mode, features, (cudaStream_t)stream);
}
