// Attention over the paged cache for steps that bring many tokens (prompts), on the fifth-generation tensor cores.
//
// The step has already written its keys and values into the cache; every query row reads the cache
// (scores = q k^T * scale, causal mask with an optional window, softmax in float32, weighted sum of values:
// sleuth/forge/model/attention.py:131-141, mask sleuth/forge/model/attention.py:57-68). Rows of one
// (sequence, kv head) are (token, head of the group): row r is token r / G, head kv * G + r % G, so a page of keys
// serves all G heads of the group.
//
// A block takes 128 rows and walks over the pages (64 keys each) that those rows may see:
//   * warp 0, one lane: TMA producer. The 128 x HD query tile once (a 3-D box over [tokens, heads, HD]), then for
//     every page the key tile and the value tile [64, HD] straight from the pool, two stages each, all in the
//     128-byte-swizzled layout that the tensor core reads.
//   * warp 1, one lane: MMA issuer. S = Q K^T (M = 128, N = 64) into one of two score buffers in tensor memory, so
//     that the scores of page j + 1 are computed while the softmax of page j runs; then O += P V (M = 128, N = HD),
//     with P read from shared memory and V read in place as an N-major operand.
//   * warps 2 to 5: softmax, one row per thread. They read a score row from tensor memory, scale and mask it, keep
//     the running maximum and sum, write P as bfloat16 into shared memory, and when a row's maximum has grown by
//     more than 2^8 since O was last scaled, rescale O in tensor memory (otherwise the old maximum keeps serving:
//     exact in float32, since numerator and denominator carry the same factor). At the end they divide by the sum
//     and store. Value rows of the last page that lie beyond the sequence are zeroed in shared memory before the
//     product, so that leftovers of an earlier tenant of the page cannot reach the sum (0 * inf).
// Two blocks fit on an SM (112 KB of shared memory and 256 columns of tensor memory each for HD = 128); while one
// waits for its softmax the other's products keep the tensor core busy.
//
// Every wait is bounded; a wait that gives up writes a code into `status`, and the block still frees its tensor
// memory and returns. TMA loads never use cluster multicast.
#include <math.h>

#include "tcgen05.cuh"

namespace slb {

constexpr int kAtThreads = 192;
constexpr int kAtRows = 128;
constexpr float kRescaleStep = 8.0f;     // in log2 units

struct AttnTcArgs {
  __nv_bfloat16* out;           // [tokens, H * HD]
  const int* seq_start;         // [n + 1]
  const int* past;              // [n]
  const int* counts;            // [n]
  const int* block_table;       // [n, table_stride]
  int table_stride;
  int heads, kv_heads, window;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

template <int HD>
struct AttnTcLayout {
  static constexpr int Q_BYTES = kAtRows * HD * 2;
  static constexpr int KV_BYTES = 64 * HD * 2;       // one page tile
  static constexpr int P_BYTES = kAtRows * 64 * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;      // two stages
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES; // two stages
  static constexpr int P_OFF = V_OFF + 2 * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int N_BARS = 15;
  static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 16;
  static constexpr int TMEM_COLS = 256;              // S0, S1 (64 each) and O (HD <= 128)
};

template <int HD>
__global__ void __launch_bounds__(kAtThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, AttnTcArgs a) {
  using L = AttnTcLayout<HD>;
  extern __shared__ __align__(1024) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_addr(smem);
  if ((base & 1023u) != 0) {            // the swizzled tiles need 1024-byte alignment; refuse rather than compute nonsense
    if (threadIdx.x == 0) atomicExch(a.status, 20);
    return;
  }
  const uint32_t sQ = base + L::Q_OFF, sK = base + L::K_OFF, sV = base + L::V_OFF, sP = base + L::P_OFF;
  const uint32_t bars = base + L::BAR_OFF;
  const uint32_t q_full = bars, k_full = bars + 8, k_empty = bars + 24, v_full = bars + 40, v_empty = bars + 56,
                 s_full = bars + 72, s_empty = bars + 88, p_full = bars + 104, pv_done = bars + 112;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + L::N_BARS * 8);

  const int seq = blockIdx.z, kh = blockIdx.y;
  const int G = a.heads / a.kv_heads;
  const int count = a.counts[seq], past = a.past[seq], tok0 = a.seq_start[seq];
  const int rows_total = count * G;
  const int n_tiles = (rows_total + kAtRows - 1) / kAtRows;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;    // heavy (late) tiles first
  if (tile >= n_tiles) return;
  const int r0 = tile * kAtRows;
  const int t_first = r0 / G;
  const int t_last = min(rows_total - 1, r0 + kAtRows - 1) / G;
  const int key_lo = a.window > 0 ? max(0, past + t_first - a.window + 1) : 0;
  const int page_lo = key_lo / 64, page_hi = (past + t_last) / 64;
  const int n_pages = page_hi - page_lo + 1;
  const int seq_len = past + count;
  const int* table = a.block_table + (size_t)seq * a.table_stride;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(v_empty + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(s_empty + 8 * i, 4);     // one arrival per softmax warp
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tO = tmem + 128;

  pdl_launch_dependents();     // only now: a successor that also wants tensor memory must not take it before this block has its own
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h)
        tma_load_3d(sQ + h * (kAtRows * 128), &map_q, h * 64, kh * G, tok0 + t_first, q_full);
      for (int j = 0; j < n_pages; ++j) {
        const int s = j & 1;
        const int row0 = (table[page_lo + j] * a.kv_heads + kh) * 64;
        if (j >= 2 && !mbar_wait(k_empty + 8 * s, ((j >> 1) - 1) & 1)) { atomicExch(a.status, 21); break; }
        mbar_expect_tx(k_full + 8 * s, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_2d(sK + s * L::KV_BYTES + h * 8192, &map_k, h * 64, row0, k_full + 8 * s);
        if (j >= 2 && !mbar_wait(v_empty + 8 * s, ((j >> 1) - 1) & 1)) { atomicExch(a.status, 22); break; }
        mbar_expect_tx(v_full + 8 * s, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_2d(sV + s * L::KV_BYTES + h * 8192, &map_v, h * 64, row0, v_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer ----
      constexpr uint32_t idesc_s = instr_desc(kAtRows, 64);
      constexpr uint32_t idesc_o = instr_desc(kAtRows, HD, true);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(a.status, 23);
      auto issue_scores = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(k_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 24); return false; }
        if (j >= 2 && !mbar_wait(s_empty + 8 * s, ((j >> 1) - 1) & 1)) { atomicExch(a.status, 25); return false; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
          const uint64_t dq = smem_desc(sQ + h * (kAtRows * 128)), dk = smem_desc(sK + s * L::KV_BYTES + h * 8192);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_bf16_ss(tmem + (uint32_t)(s * 64), dq + (uint64_t)(k4 * 2), dk + (uint64_t)(k4 * 2), idesc_s, (h > 0 || k4 > 0) ? 1u : 0u);
        }
        mma_commit(s_full + 8 * s);
        mma_commit(k_empty + 8 * s);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < n_pages && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_pages && !issue_scores(j + 1)) break;
        if (!mbar_wait(p_full, j & 1)) { atomicExch(a.status, 26); break; }
        if (!mbar_wait(v_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 27); break; }
        tc_fence_after();
        const uint64_t dp = smem_desc(sP);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {      // 16 keys each: 32 bytes along a row of P, two 8-key groups of V
          const uint64_t dv = smem_desc_mn(sV + s * L::KV_BYTES + k4 * 2048, 8192, 1024);
          mma_bf16_ss(tO, dp + (uint64_t)(k4 * 2), dv, idesc_o, (j > 0 || k4 > 0) ? 1u : 0u);
        }
        mma_commit(pv_done);
        mma_commit(v_empty + 8 * s);
      }
    }
  } else {
    // ---- softmax: warps 2..5, tensor-memory lanes 32 * (warp % 4) .. + 31; thread = row ----
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int R = r0 + r;
    const int pos = R < rows_total ? past + R / G : -1;        // -1: a padding row sees nothing
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    float m_used = -INFINITY, l = 0.0f;
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
      bool ready = true;
      if (lane == 0) ready = mbar_wait(bar, parity);
      ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
      if (!ready && lane == 0) atomicExch(a.status, code);
      return ready;
    };
    for (int j = 0; j < n_pages; ++j) {
      const int b = j & 1, key0 = (page_lo + j) * 64;
      if (!wait_all(s_full + 8 * b, (j >> 1) & 1, 28)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld32(lane_addr + (uint32_t)(b * 64), sr[0]);
      tmem_ld32(lane_addr + (uint32_t)(b * 64 + 32), sr[1]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty + 8 * b);

      // raw scores -> masked raw scores and their maximum; the mask costs two compares and a select per score, so
      // only warps with a row that needs it (the diagonal, a window's edge, padding) run it
      float mx = -INFINITY;
      if (__any_sync(0xffffffffu, key0 + 63 > pos || key0 < lo)) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          if (key > pos || key < lo) sr[c >> 5][c & 31] = 0xff800000u;     // -inf
        }
      }
#pragma unroll
      for (int c = 0; c < 64; c += 2) mx = max3(mx, __uint_as_float(sr[c >> 5][c & 31]), __uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]));
      const float m_new = fmaxf(m_used, mx * a.scale_log2);               // the scale is positive
      const bool grow = m_new > m_used + kRescaleStep;      // also true for the first finite maximum
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        if (!wait_all(pv_done, (j - 1) & 1, 29)) { ok = false; break; }
        tc_fence_after();
        const float alpha = grow ? ex2(m_used - m_new) : 1.0f;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(lane_addr + 128 + c0, o);
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st32(lane_addr + 128 + c0, o);
        }
        l *= alpha;
        tc_fence_before();
      }
      if (grow) m_used = m_new;
      const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
      uint32_t pk[32];
      float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), a.scale_log2, neg_m));
        const float p1 = ex2(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), a.scale_log2, neg_m));
        l0 += p0;
        l1 += p1;
        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
      }
      l += l0 + l1;
      if (j > 0 && !wait_all(pv_done, (j - 1) & 1, 30)) { ok = false; break; }     // the last product has read P
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint32_t dst = sP + (uint32_t)(r * 128 + ((ch ^ (r & 7)) << 4));
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * ch]), "r"(pk[4 * ch + 1]),
                     "r"(pk[4 * ch + 2]), "r"(pk[4 * ch + 3]) : "memory");
      }
      const int valid = seq_len - key0;          // rows of this page that belong to the sequence
      if (valid < 64) {
        if (!wait_all(v_full + 8 * b, (j >> 1) & 1, 31)) { ok = false; break; }
        if (r < 64 && r >= valid) {
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              const uint32_t dst = sV + (uint32_t)(b * L::KV_BYTES + h * 8192 + r * 128 + ch * 16);
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
            }
        }
      }
      fence_smem_to_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && wait_all(pv_done, (n_pages - 1) & 1, 32)) {
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      __nv_bfloat16* dst = a.out + ((size_t)(tok0 + (R < rows_total ? R / G : 0)) * a.heads + kh * G + R % G) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(lane_addr + 128 + c0, o);
        if (R < rows_total) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 q;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            q.x = *reinterpret_cast<uint32_t*>(&h0); q.y = *reinterpret_cast<uint32_t*>(&h1);
            q.z = *reinterpret_cast<uint32_t*>(&h2); q.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + c0 + c) = q;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------------------------ host side ----
static int encode(CUtensorMap* map, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                  const cuuint32_t* box, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(2, "attention (tcgen05): the driver does not offer cuTensorMapEncodeTiled");
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(2, "attention (tcgen05): cuTensorMapEncodeTiled failed for %s with code %d", what, (int)r);
  return 0;
}

template <int HD>
static int launch_attn_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& a,
                          int n_seqs, int max_count, cudaStream_t s) {
  using L = AttnTcLayout<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return fail(2, "attention (tcgen05): cannot reserve %d bytes of shared memory: %s", L::TOTAL, cudaGetErrorString(e));
    configured = true;
  }
  const int G = a.heads / a.kv_heads;
  const int tiles = (max_count * G + kAtRows - 1) / kAtRows;
  dim3 grid(tiles, a.kv_heads, n_seqs);
  launch(attn_tc_kernel<HD>, grid, dim3(kAtThreads), (size_t)L::TOTAL, s, mq, mk, mv, a);
  return check_launch("attention (tcgen05)");
}

}  // namespace slb

using namespace slb;

// 1 when the tcgen05 kernel takes this shape: bfloat16, head size 64 or 128, a group size that divides 128.
extern "C" int slb_attention_tc_supported(int heads, int kv_heads, int head_dim) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
  const int G = heads / kv_heads;
  return (head_dim == 64 || head_dim == 128) && G <= 128 && (128 % G) == 0;
}

// q [tokens, heads, head_dim]; k_pool, v_pool [pool_pages, kv_heads, 64, head_dim]; out [tokens, heads * head_dim];
// all bfloat16. `status` is a zeroed device int that receives a code if a bounded wait inside the kernel gave up.
extern "C" int slb_attention_tc(const void* q, const void* k_pool, const void* v_pool, void* out, const int* seq_start,
                                const int* past, const int* counts, const int* block_table, int table_stride,
                                int n_seqs, int max_count, long long tokens, long long pool_pages, int heads,
                                int kv_heads, int head_dim, int window, float scale, int* status, void* stream) {
  SLB_REQUIRE(slb_attention_tc_supported(heads, kv_heads, head_dim),
              "attention (tcgen05): heads=%d kv_heads=%d head_dim=%d is not taken (head size 64 or 128, group size a divisor of 128)",
              heads, kv_heads, head_dim);
  SLB_REQUIRE(scale > 0.0f, "attention (tcgen05): the kernel takes a positive scale, got %g", (double)scale);
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && window >= 0 && table_stride > 0 && n_seqs < 65536 && kv_heads < 65536 &&
              tokens >= 0 && pool_pages > 0 && status != nullptr,
              "attention (tcgen05): seqs=%d max_count=%d window=%d table_stride=%d", n_seqs, max_count, window, table_stride);
  SLB_REQUIRE(pool_pages * kv_heads * 64 < (1ll << 31), "attention (tcgen05): the pool has too many rows for one tensor map");
  SLB_REQUIRE(((uintptr_t)q % 16 == 0) && ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) && ((uintptr_t)out % 16 == 0),
              "attention (tcgen05): q, pools and out must be 16-byte aligned");
  if (n_seqs == 0 || max_count == 0 || tokens == 0) return 0;
  const int G = heads / kv_heads;
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)heads * head_dim * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(kAtRows / G)};
    int rc = encode(&mq, 3, q, dims, strides, box, "q");
    if (rc) return rc;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)(pool_pages * kv_heads * 64)};
    cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    cuuint32_t box[2] = {64, 64};
    int rc = encode(&mk, 2, k_pool, dims, strides, box, "the key pool");
    if (rc) return rc;
    rc = encode(&mv, 2, v_pool, dims, strides, box, "the value pool");
    if (rc) return rc;
  }
  AttnTcArgs a;
  a.out = (__nv_bfloat16*)out; a.seq_start = seq_start; a.past = past; a.counts = counts; a.block_table = block_table;
  a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f; a.status = status;
  return head_dim == 64 ? launch_attn_tc<64>(mq, mk, mv, a, n_seqs, max_count, (cudaStream_t)stream)
                        : launch_attn_tc<128>(mq, mk, mv, a, n_seqs, max_count, (cudaStream_t)stream);
}
