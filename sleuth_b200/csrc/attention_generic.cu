// Causal grouped-query attention over the paged cache: the general kernel.
//
// It serves every head size (even, up to 256), both dtypes, prompts, single decoded tokens and anything between,
// because a step first writes its keys and values to the cache and then every query reads all its keys from there.
// A query at position p of sequence s sees the keys at positions lo..p of s, lo = max(0, p - window + 1) with a
// window and 0 without (sleuth/forge/model/attention.py:160-169); query head h reads key/value head h / (H / K)
// (attention.py:197-199); scores are (q . k) * scale, softmax and the weighted sum run in float32
// (attention.py:200-206).
//
// One block of eight warps per (token, query head). Keys are taken 32 at a time, aligned to multiples of 32 positions;
// the groups of 32 go to the warps in turn (group i of the query's range to warp i % 8), so that a single token with
// thousands of keys behind it still has eight warps at work. Within a group each lane computes the whole dot product
// of its key (channels in ascending order), the warp keeps a running maximum and sum over its groups (online softmax),
// then the lanes switch to channels for the weighted sum of values; at the end the eight warps' results are merged in
// warp order. Which warp takes which keys, and so the order of every addition, depends only on the token's own
// position and window, never on the batch or on how the sequence was cut into steps: in float32 the result is the
// same bit for bit under every schedule.
#include <math.h>

#include "common.cuh"

namespace slb {

struct AttnArgs {
  const void* q;        // [tokens, H, hd]
  const void* k_pool;   // [pages, K, 64, hd]
  const void* v_pool;
  void* out;            // [tokens, H * hd]
  const int* tok_seq;
  const int* tok_pos;
  const int* block_table;
  int table_stride;
  int tokens, heads, kv_heads, head_dim, window;
  float scale;
};

template <typename T> struct RowDot;

template <> struct RowDot<float> {
  static __device__ __forceinline__ float run(const float* __restrict__ k, const float* __restrict__ q, int hd) {
    float d = 0.0f;
    if ((hd & 3) == 0) {
      const float4* k4 = reinterpret_cast<const float4*>(k);
      for (int i = 0; i < hd / 4; ++i) {
        const float4 kv = k4[i];
        d = fmaf(q[4 * i + 0], kv.x, d);
        d = fmaf(q[4 * i + 1], kv.y, d);
        d = fmaf(q[4 * i + 2], kv.z, d);
        d = fmaf(q[4 * i + 3], kv.w, d);
      }
    } else {
      for (int i = 0; i < hd; ++i) d = fmaf(q[i], k[i], d);
    }
    return d;
  }
};

template <> struct RowDot<__nv_bfloat16> {
  static __device__ __forceinline__ float run(const __nv_bfloat16* __restrict__ k, const float* __restrict__ q,
                                              int hd) {
    float d = 0.0f;
    if ((hd & 7) == 0) {
      const Bf16x8* k8 = reinterpret_cast<const Bf16x8*>(k);
      for (int i = 0; i < hd / 8; ++i) {
        float f[8];
        unpack8(k8[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(q[8 * i + e], f[e], d);
      }
    } else {
      for (int i = 0; i < hd; ++i) d = fmaf(q[i], __bfloat162float(k[i]), d);
    }
    return d;
  }
};

constexpr int kAttnWarps = 8;

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_generic_kernel(AttnArgs a) {
  pdl_enter();
  __shared__ float qs[256];
  __shared__ float part_acc[kAttnWarps][PER_LANE * 32];
  __shared__ float part_m[kAttnWarps], part_l[kAttnWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = blockIdx.x;
  const int t = (int)(item / a.heads), h = (int)(item - (long long)t * a.heads);
  const int hd = a.head_dim;
  const int kh = h / (a.heads / a.kv_heads);
  const int pos = a.tok_pos[t];
  const int* table = a.block_table + (size_t)a.tok_seq[t] * a.table_stride;
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;

  const T* qrow = (const T*)a.q + ((size_t)t * a.heads + h) * hd;
  for (int c = threadIdx.x; c < hd; c += kAttnWarps * 32) qs[c] = to_f32(qrow[c]);
  __syncthreads();

  const T* kpool = (const T*)a.k_pool;
  const T* vpool = (const T*)a.v_pool;

  float acc[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
  float m = -INFINITY, l = 0.0f;

  for (int base = (lo / 32) * 32 + 32 * warp; base <= pos; base += 32 * kAttnWarps) {
    const int j = base + lane;
    const bool valid = j >= lo && j <= pos;
    int row = 0;          // row of the pools: (page * K + kh) * 64 + j % 64
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / kPageTokens];
      row = (page * a.kv_heads + kh) * kPageTokens + (j % kPageTokens);
      s = RowDot<T>::run(kpool + (size_t)row * hd, qs, hd) * a.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.0f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] *= alpha;
    const int first = max(lo - base, 0), last = min(31, pos - base);
    for (int jj = first; jj <= last; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int rj = __shfl_sync(0xffffffffu, row, jj);
      const T* vrow = vpool + (size_t)rj * hd;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) acc[i] = fmaf(pj, to_f32(vrow[c]), acc[i]);
      }
    }
    m = m_new;
  }

  // the warps' results (a warp that had no keys brings maximum -inf and sum 0), merged in warp order
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) part_acc[warp][lane + 32 * i] = acc[i];
  if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
  __syncthreads();
  float top = -INFINITY;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) top = fmaxf(top, part_m[w]);
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < kAttnWarps; ++w) total += part_l[w] * expf(part_m[w] - top);
  T* o = (T*)a.out + ((size_t)t * a.heads + h) * hd;
  const float inv = 1.0f / total;
  for (int c = threadIdx.x; c < hd; c += kAttnWarps * 32) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) v += part_acc[w][c] * expf(part_m[w] - top);
    o[c] = from_f32<T>(v * inv);
  }
}

template <typename T>
static int launch_attn_generic(const AttnArgs& a, cudaStream_t s) {
  const long long items = (long long)a.tokens * a.heads;
  const long long blocks = items;
  SLB_REQUIRE(blocks < (1ll << 31), "attention: too many rows (%lld)", items);
  const int per_lane = (a.head_dim + 31) / 32;
  const int threads = kAttnWarps * 32;
  switch (per_lane) {
    case 1: launch(attn_generic_kernel<T, 1>, dim3((int)blocks), dim3(threads), 0, s, a); break;
    case 2: launch(attn_generic_kernel<T, 2>, dim3((int)blocks), dim3(threads), 0, s, a); break;
    case 3: launch(attn_generic_kernel<T, 3>, dim3((int)blocks), dim3(threads), 0, s, a); break;
    case 4: launch(attn_generic_kernel<T, 4>, dim3((int)blocks), dim3(threads), 0, s, a); break;
    default: launch(attn_generic_kernel<T, 8>, dim3((int)blocks), dim3(threads), 0, s, a); break;
  }
  return check_launch("attention (general kernel)");
}

}  // namespace slb

using namespace slb;

extern "C" int slb_attention_generic(const void* q, const void* k_pool, const void* v_pool, void* out,
                                     const int* tok_seq, const int* tok_pos, const int* block_table,
                                     int table_stride, int tokens, int heads, int kv_heads, int head_dim, int window,
                                     float scale, int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention: tokens=%d heads=%d kv_heads=%d", tokens, heads, kv_heads);
  SLB_REQUIRE(head_dim > 0 && head_dim <= 256 && head_dim % 2 == 0,
              "attention: head_dim %d is not supported (even, at most 256)", head_dim);
  SLB_REQUIRE(window >= 0 && table_stride > 0, "attention: window=%d table_stride=%d", window, table_stride);
  if (tokens == 0) return 0;
  AttnArgs a;
  a.q = q; a.k_pool = k_pool; a.v_pool = v_pool; a.out = out;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.block_table = block_table; a.table_stride = table_stride;
  a.tokens = tokens; a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.window = window;
  a.scale = scale;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) return launch_attn_generic<float>(a, s);
  if (dtype == kBF16) return launch_attn_generic<__nv_bfloat16>(a, s);
  return fail(1, "attention: unknown dtype %d", dtype);
}
