// After the fused q/k/v projection: bias, per-head RMSNorm of q and k, rotation, and the cache write.
//
// One warp handles one (token, head) row of the projection output [tokens, (H + 2K) * head_dim]:
//   q heads: (+bias) -> RMSNorm over head_dim with the layer's q gain -> rotation -> q_out [tokens, H, head_dim]
//   k heads: (+bias) -> RMSNorm with the k gain -> rotation -> key page of the token's sequence
//   v heads: (+bias) -> value page, unchanged
// Norm before rotation, values never normalised (sleuth/forge/model/attention.py:121-126); rotation pairs
// channel i with i + rot/2: (a, b) -> (a*cos - b*sin, b*cos + a*sin) (sleuth/forge/model/rope.py:41-55); the
// reference's own fused form is sleuth/forge/model/fused_ops.py:53-85. Everything is float32 between the load and
// the single rounding at the store. cos/sin come from tables [positions, rot/2] that the position part built in
// float32, so the angles are those of the reference's tables (rope.py:30-38).
//
// A token's key and value go to page block_table[seq, pos / 64], row pos % 64 of the pool
// [pages, kv_heads, 64, head_dim].
#include "common.cuh"

namespace slb {

struct QkvPostArgs {
  const void* qkv;
  const float* bias;        // [(H + 2K) * hd] or null
  const float* q_gain;      // [hd] or null (no QK-norm)
  const float* k_gain;
  const float* cos_table;   // [positions, rot / 2] or null (no rotation)
  const float* sin_table;
  void* q_out;              // [tokens, H, hd]
  void* k_pool;             // [pages, K, 64, hd] or null (this application only reads a shared cache)
  void* v_pool;
  const int* tok_seq;       // [tokens]
  const int* tok_pos;       // [tokens]
  const int* block_table;   // [seqs, table_stride]
  int table_stride;
  int tokens, heads, kv_heads, head_dim, rot_dim;
  float eps;
};

template <typename T, int PER_LANE>
__global__ void qkv_post_kernel(QkvPostArgs a) {
  pdl_enter();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rows_per_token = a.heads + 2 * a.kv_heads;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)a.tokens * rows_per_token) return;
  const int t = (int)(item / rows_per_token);
  const int r = (int)(item - (long long)t * rows_per_token);
  const int hd = a.head_dim, half = a.rot_dim >> 1;

  const T* src = (const T*)a.qkv + ((size_t)t * rows_per_token + r) * hd;
  const float* bias = a.bias ? a.bias + (size_t)r * hd : nullptr;

  // lane l holds channels l, l + 32, ... (PER_LANE of them, guarded by head_dim)
  float v[PER_LANE];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int c = lane + 32 * i;
    float x = 0.0f;
    if (c < hd) {
      x = to_f32(src[c]);
      if (bias) x += bias[c];
    }
    v[i] = x;
    ss = fmaf(x, x, ss);
  }

  const bool is_q = r < a.heads;
  const bool is_k = !is_q && r < a.heads + a.kv_heads;
  const float* gain = is_q ? a.q_gain : (is_k ? a.k_gain : nullptr);

  if (is_q || is_k) {
    if (gain) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) v[i] = (v[i] * inv) * gain[c];
      }
    }
    if (a.cos_table && half > 0) {
      // Channel c < half pairs with c + half. The partner lives in another lane or register, so the
      // row goes through shared memory once.
      __shared__ float stage_all[8][256];
      float* stage = stage_all[threadIdx.x >> 5];
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) stage[c] = v[i];
      }
      __syncwarp();
      const int pos = a.tok_pos[t];
      const float* cs = a.cos_table + (size_t)pos * half;
      const float* sn = a.sin_table + (size_t)pos * half;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < a.rot_dim) {
          const int j = c < half ? c : c - half;
          const float co = cs[j], si = sn[j];
          const float other = c < half ? -stage[c + half] : stage[c - half];
          v[i] = v[i] * co + other * si;
        }
      }
    }
  }

  T* dst;
  if (is_q) {
    dst = (T*)a.q_out + ((size_t)t * a.heads + r) * hd;
  } else {
    if (a.k_pool == nullptr) return;
    const int kh = is_k ? r - a.heads : r - a.heads - a.kv_heads;
    const int pos = a.tok_pos[t];
    const int page = a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens];
    T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
    dst = pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + (pos % kPageTokens)) * hd;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int c = lane + 32 * i;
    if (c < hd) dst[c] = from_f32<T>(v[i]);
  }
}

// Head sizes 64, 128 and 256 with the whole head rotated (or none of it): lane l holds the EPL = head_dim / 32
// contiguous channels l * EPL .., one vector load and store per lane, and a channel's rotation partner
// (head_dim / 2 away) sits at the same place in lane l ^ 16, so a shuffle replaces the shared-memory staging.
template <typename T, int EPL>
struct alignas(sizeof(T) * EPL) LaneVec {
  T v[EPL];
};

template <typename T, int EPL>
__global__ void qkv_post_vec_kernel(QkvPostArgs a) {
  pdl_enter();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rows_per_token = a.heads + 2 * a.kv_heads;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)a.tokens * rows_per_token) return;
  const int t = (int)(item / rows_per_token);
  const int r = (int)(item - (long long)t * rows_per_token);
  constexpr int HD = 32 * EPL;
  const int c0 = lane * EPL;

  const LaneVec<T, EPL> in = *reinterpret_cast<const LaneVec<T, EPL>*>(
      (const T*)a.qkv + ((size_t)t * rows_per_token + r) * HD + c0);
  float v[EPL];
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    float x = to_f32(in.v[e]);
    if (a.bias) x += a.bias[(size_t)r * HD + c0 + e];
    v[e] = x;
    ss = fmaf(x, x, ss);
  }
  const bool is_q = r < a.heads;
  const bool is_k = !is_q && r < a.heads + a.kv_heads;
  const float* gain = is_q ? a.q_gain : (is_k ? a.k_gain : nullptr);
  const int pos = a.tok_pos[t];
  if (is_q || is_k) {
    if (gain) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] = (v[e] * inv) * gain[c0 + e];
    }
    if (a.cos_table) {
      const float* cs = a.cos_table + (size_t)pos * (HD / 2) + (lane & 15) * EPL;
      const float* sn = a.sin_table + (size_t)pos * (HD / 2) + (lane & 15) * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[e], 16);
        const float other = lane < 16 ? -partner : partner;
        v[e] = v[e] * cs[e] + other * sn[e];
      }
    }
  }
  T* dst;
  if (is_q) {
    dst = (T*)a.q_out + ((size_t)t * a.heads + r) * HD;
  } else {
    if (a.k_pool == nullptr) return;
    const int kh = is_k ? r - a.heads : r - a.heads - a.kv_heads;
    const int page = a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens];
    T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
    dst = pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + (pos % kPageTokens)) * HD;
  }
  LaneVec<T, EPL> out;
#pragma unroll
  for (int e = 0; e < EPL; ++e) out.v[e] = from_f32<T>(v[e]);
  *reinterpret_cast<LaneVec<T, EPL>*>(dst + c0) = out;
}

template <typename T>
static int launch_qkv_post(const QkvPostArgs& a, cudaStream_t s) {
  const long long items = (long long)a.tokens * (a.heads + 2 * a.kv_heads);
  const int warps = 8;
  const long long blocks = (items + warps - 1) / warps;
  SLB_REQUIRE(blocks < (1ll << 31), "qkv_post: too many rows (%lld)", items);
  const bool whole = a.cos_table == nullptr || a.rot_dim == a.head_dim;
  if (whole && (a.head_dim == 64 || a.head_dim == 128 || a.head_dim == 256) && ((uintptr_t)a.qkv % 16 == 0)) {
    if (a.head_dim == 64) launch(qkv_post_vec_kernel<T, 2>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    else if (a.head_dim == 128) launch(qkv_post_vec_kernel<T, 4>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    else launch(qkv_post_vec_kernel<T, 8>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    return check_launch("qkv_post");
  }
  const int per_lane = (a.head_dim + 31) / 32;
  switch (per_lane) {
    case 1: launch(qkv_post_kernel<T, 1>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 2: launch(qkv_post_kernel<T, 2>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 3: launch(qkv_post_kernel<T, 3>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 4: launch(qkv_post_kernel<T, 4>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    default: launch(qkv_post_kernel<T, 8>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
  }
  return check_launch("qkv_post");
}

}  // namespace slb

using namespace slb;

extern "C" int slb_qkv_post(const void* qkv, const float* bias, const float* q_gain, const float* k_gain,
                            const float* cos_table, const float* sin_table, void* q_out, void* k_pool, void* v_pool,
                            const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride,
                            int tokens, int heads, int kv_heads, int head_dim, int rot_dim, float eps, int dtype,
                            void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads >= 0, "qkv_post: tokens=%d heads=%d kv_heads=%d", tokens, heads,
              kv_heads);
  SLB_REQUIRE(head_dim > 0 && head_dim <= 256 && head_dim % 2 == 0,
              "qkv_post: head_dim %d is not supported (even, at most 256)", head_dim);
  SLB_REQUIRE(rot_dim >= 0 && rot_dim <= head_dim && rot_dim % 2 == 0, "qkv_post: rot_dim=%d for head_dim=%d",
              rot_dim, head_dim);
  SLB_REQUIRE((q_gain == nullptr) == (k_gain == nullptr) || kv_heads == 0, "qkv_post: q and k gains go together");
  SLB_REQUIRE(kv_heads == 0 || k_pool == nullptr || (v_pool && block_table && table_stride > 0),
              "qkv_post: a cache write needs both pools and a block table");
  if (tokens == 0) return 0;
  QkvPostArgs a;
  a.qkv = qkv; a.bias = bias; a.q_gain = q_gain; a.k_gain = k_gain;
  a.cos_table = rot_dim > 0 ? cos_table : nullptr; a.sin_table = sin_table;
  a.q_out = q_out; a.k_pool = k_pool; a.v_pool = v_pool;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.block_table = block_table; a.table_stride = table_stride;
  a.tokens = tokens; a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.rot_dim = rot_dim;
  a.eps = eps;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) return launch_qkv_post<float>(a, s);
  if (dtype == kBF16) return launch_qkv_post<__nv_bfloat16>(a, s);
  return fail(1, "qkv_post: unknown dtype %d", dtype);
}
