// Attention over the paged cache for steps that bring many tokens (prompts), on the fifth-generation tensor cores.
//
// The step has already written its keys and values into the cache; every query row reads the cache
// (scores = q k^T * scale, causal mask with an optional window, softmax in float32, weighted sum of values:
// sleuth/forge/model/attention.py:131-141, mask sleuth/forge/model/attention.py:57-68). Rows of one
// (sequence, kv head) are (token, head of the group): row r is token r / G, head kv * G + r % G, so a page of keys
// serves all G heads of the group.
//
// A block takes 128 rows and walks over the pages (64 keys each) that those rows may see:
//   * warp 0, one lane: the scores. It asks TMA for the 128 x HD query tile once (a 3-D box over [tokens, heads, HD])
//     and for the key page [64, HD] of every step, two stages, straight from the pool in the 128-byte-swizzled layout
//     that the tensor core reads, and issues S = Q K^T (M = 128, N = 64) into one of two score buffers in tensor
//     memory, one page ahead of the softmax.
//   * warp 1, one lane: the values. It asks TMA for the value pages and issues O += P V (M = 128, N = HD) as soon as
//     the softmax has written P; P is read from tensor memory (the A operand), V in place from shared memory as an
//     N-major operand.
//   * warps 2 to 9: softmax, two threads per row (keys 0..31 and 32..63 of the page). They read their half of a score
//     row from tensor memory, mask it, agree on the row's maximum through shared memory (the two warps of a row
//     meet at a hardware barrier of their own, once per page), write P as bfloat16 back into tensor memory, into
//     the columns its scores came from (so P has two buffers as S has, and the softmax of a page does not wait for
//     the product of the page before; a score buffer is written again only when the product that read its P is
//     through), and when a row's maximum has grown by more than 2^8 since O was last scaled, wait for the last
//     product and rescale O in tensor memory (otherwise the old maximum keeps serving: exact, since numerator and
//     denominator carry the same factor). At the end they add their sums, divide, and store through shared memory
//     so that a warp writes whole lines. Value rows of the last page that lie beyond the sequence are zeroed in
//     shared memory before the product, so that leftovers of an earlier tenant of the page cannot reach the sum
//     (0 * inf).
// Two blocks fit on an SM (98 KB of shared memory and 256 columns of tensor memory each); while one waits for its
// softmax the other's products keep the tensor core busy. A block's own chain per page (scores -> softmax -> P ->
// product) is what bounds a single long prompt; many sequences or heads fill the GPU.
//
// Every wait on an mbarrier is bounded; a wait that gives up writes a code into `status`, the thread stops waiting
// and runs on to the end of its loop (so that it still meets its partner at their hardware barrier), and the block
// frees its tensor memory and returns. TMA loads never use cluster multicast.
#include <math.h>

#include "tcgen05.cuh"

namespace slb {

constexpr int kAtThreads = 320;      // producer warp, MMA warp, eight softmax warps
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

// The way a block's results leave (both kernels): a lane holds a row of the accumulator, so a warp's store would touch
// 32 lines at once. The normalised rows go through shared memory instead, into the query tile's place (the last score
// product has read it): rows of HD * 2 bytes, the 16-byte pieces of each 128 bytes exchanged by the row's low bits so
// that a warp's 32 rows spread over the banks. stage_row writes COLS values of row r from column col0 on;
// store_rows, after a barrier of the softmax warps, lets warp w of WARPS store 128 / WARPS rows, its lanes along a
// row: whole 128-byte lines.
template <int HD, int COLS>
__device__ __forceinline__ void stage_row(uint32_t sQ, int r, int col0, const uint32_t (&o)[COLS], float inv) {
#pragma unroll
  for (int c = 0; c < COLS; c += 8) {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
    __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
    __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
    const int piece = (col0 + c) >> 3;
    const uint32_t dst = sQ + (uint32_t)(r * (HD * 2) + (((piece & ~7) | ((piece ^ r) & 7)) << 4));
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(*reinterpret_cast<uint32_t*>(&h0)),
                 "r"(*reinterpret_cast<uint32_t*>(&h1)), "r"(*reinterpret_cast<uint32_t*>(&h2)),
                 "r"(*reinterpret_cast<uint32_t*>(&h3)) : "memory");
  }
}

template <int HD, int WARPS>
__device__ __forceinline__ void store_rows(uint32_t sQ, int w, int lane, int r0, int rows_total, bool ok, __nv_bfloat16* out,
                                           int tok0, int G, int heads, int kh) {
  constexpr int kPieces = HD / 8, kRowsAtOnce = 32 / kPieces, kRows = kAtRows / WARPS;
  const int piece = lane % kPieces;
#pragma unroll
  for (int it = 0; it < kRows / kRowsAtOnce; ++it) {
    const int rr = w * kRows + it * kRowsAtOnce + lane / kPieces;
    const int Rr = r0 + rr;
    if (ok && Rr < rows_total) {
      const uint32_t src = sQ + (uint32_t)(rr * (HD * 2) + (((piece & ~7) | ((piece ^ rr) & 7)) << 4));
      uint4 q;
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(src) : "memory");
      *reinterpret_cast<uint4*>(out + ((size_t)(tok0 + Rr / G) * heads + kh * G + Rr % G) * HD + piece * 8) = q;
    }
  }
}

template <int HD>
struct AttnTcLayout {
  static constexpr int Q_BYTES = kAtRows * HD * 2;
  static constexpr int KV_BYTES = 64 * HD * 2;       // one page tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;      // two stages
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES; // two stages
  static constexpr int SUM_OFF = V_OFF + 2 * KV_BYTES;        // the halves' row sums, float [2 halves][128 rows]
  static constexpr int BAR_OFF = SUM_OFF + 2 * kAtRows * 4;
  static constexpr int N_BARS = 12;
  static constexpr int XCH_OFF = BAR_OFF + N_BARS * 8 + 16;   // row maxima as 16-bit values, [2 pages][2 halves][128 rows]
  static constexpr int TOTAL = XCH_OFF + 4 * kAtRows * 2;
  static_assert(2 * (TOTAL + 1024) <= 228 * 1024, "two blocks must fit on an SM");
  static constexpr int TMEM_COLS = 256;              // S0, S1 (64 each; P_j takes the first 32 of S_j's) and O (HD <= 128)
};

template <int HD>
__global__ void __launch_bounds__(kAtThreads, 2)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, AttnTcArgs a) {
  using L = AttnTcLayout<HD>;
  extern __shared__ __align__(1024) unsigned char smem[];
  Tracer trace(kTraceAttnTc);      // thread 0 issues the score products: past its wait, last scores issued, exit
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_addr(smem);
  if ((base & 1023u) != 0) {            // the swizzled tiles need 1024-byte alignment; refuse rather than compute nonsense
    if (threadIdx.x == 0) atomicExch(a.status, 20);
    return;
  }
  const uint32_t sQ = base + L::Q_OFF, sK = base + L::K_OFF, sV = base + L::V_OFF;
  const uint32_t bars = base + L::BAR_OFF;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 24, s_full = bars + 40, p_full = bars + 56,
                 pv_done = bars + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + L::N_BARS * 8);

  // Blocks start in the order of their index, and a late tile of a prompt walks many more pages than an early one:
  // longest first.
  const int pairs = (int)(gridDim.y * gridDim.z);
  const int lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  const int seq = (lin % pairs) / (int)gridDim.y, kh = (lin % pairs) % (int)gridDim.y;
  const int G = a.heads / a.kv_heads;
  const int count = a.counts[seq], past = a.past[seq], tok0 = a.seq_start[seq];
  const int rows_total = count * G;
  const int n_tiles = (rows_total + kAtRows - 1) / kAtRows;
  const int tile = (int)gridDim.x - 1 - lin / pairs;
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
      mbar_init(v_full + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(pv_done + 8 * i, 1);
      mbar_init(p_full + 8 * i, 8);      // one arrival per softmax warp
    }
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
  trace.mark(1);

  if (warp == 0) {
    if (lane == 0) {
      // ---- scores: loads Q and the key pages, issues S_j = Q K_j^T one page ahead of the softmax. A page's keys are
      // asked for before the products of the page before are issued, its number a page earlier still ----
      constexpr uint32_t idesc_s = instr_desc(kAtRows, 64);
      auto page_of = [&](int i) { return i < n_pages ? table[page_lo + i] : 0; };
      auto load_keys = [&](int j, int page) {
        const int s = j & 1;
        const int row0 = (page * a.kv_heads + kh) * 64;
        mbar_expect_tx(k_full + 8 * s, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_2d(sK + s * L::KV_BYTES + h * 8192, &map_k, h * 64, row0, k_full + 8 * s);
      };
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h)
        tma_load_3d(sQ + h * (kAtRows * 128), &map_q, h * 64, kh * G, tok0 + t_first, q_full);
      load_keys(0, page_of(0));
      int next_page = page_of(1);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(a.status, 23);
      for (int j = 0; j < n_pages && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_pages) {
          // the other key stage was read by S_{j-1}, issued a whole page ago
          if (j >= 1 && !mbar_wait(s_full + 8 * (s ^ 1), ((j - 1) >> 1) & 1)) { atomicExch(a.status, 21); break; }
          load_keys(j + 1, next_page);
          next_page = page_of(j + 2);
        }
        if (!mbar_wait(k_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 24); break; }
        // S_j lands where S_{j-2} and then P_{j-2} lay: the product that read P_{j-2} must be through
        if (j >= 2 && !mbar_wait(pv_done + 8 * s, ((j >> 1) - 1) & 1)) { atomicExch(a.status, 25); break; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
          const uint64_t dq = smem_desc(sQ + h * (kAtRows * 128)), dk = smem_desc(sK + s * L::KV_BYTES + h * 8192);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_bf16_ss(tmem + (uint32_t)(s * 64), dq + (uint64_t)(k4 * 2), dk + (uint64_t)(k4 * 2), idesc_s, (h > 0 || k4 > 0) ? 1u : 0u);
        }
        mma_commit(s_full + 8 * s);          // S_j is complete: the softmax may read it, and this key stage is free again
      }
      trace.mark(2);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- values: loads the value pages, issues O += P_j V_j as soon as the softmax has written P_j ----
      constexpr uint32_t idesc_o = instr_desc(kAtRows, HD, true);
      auto page_of = [&](int i) { return i < n_pages ? table[page_lo + i] : 0; };
      auto load_values = [&](int j, int page) {
        const int s = j & 1;
        const int row0 = (page * a.kv_heads + kh) * 64;
        mbar_expect_tx(v_full + 8 * s, L::KV_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) tma_load_2d(sV + s * L::KV_BYTES + h * 8192, &map_v, h * 64, row0, v_full + 8 * s);
      };
      load_values(0, page_of(0));
      int next_page = page_of(1);
      for (int j = 0; j < n_pages; ++j) {
        const int s = j & 1;
        if (j + 1 < n_pages) {
          // the other value stage was read by the product of page j - 1
          if (j >= 1 && !mbar_wait(pv_done + 8 * (s ^ 1), ((j - 1) >> 1) & 1)) { atomicExch(a.status, 22); break; }
          load_values(j + 1, next_page);
          next_page = page_of(j + 2);
        }
        if (!mbar_wait(v_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 27); break; }
        // a barrier per score buffer: the softmax may be a page ahead of this warp, never two
        if (!mbar_wait(p_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 26); break; }
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {      // 16 keys each: 8 columns of P in tensor memory, two 8-key groups of V
          const uint64_t dv = smem_desc_mn(sV + s * L::KV_BYTES + k4 * 2048, 8192, 1024);
          mma_bf16_ts(tO, tmem + (uint32_t)(s * 64 + k4 * 8), dv, idesc_o, (j > 0 || k4 > 0) ? 1u : 0u);
        }
        mma_commit(pv_done + 8 * s);         // this score buffer and this value stage are free again when it fires
      }
    }
  } else {
    // ---- softmax: warps 2..9. Tensor-memory lanes 32 * (warp % 4) .. + 31 hold the rows; two warps share those
    // lanes, one for keys 0..31 of the page, one for keys 32..63: two threads per row ----
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int R = r0 + r;
    const int pos = R < rows_total ? past + R / G : -1;        // -1: a padding row sees nothing
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    unsigned short* xch = reinterpret_cast<unsigned short*>(smem + L::XCH_OFF);     // [2 pages][2 halves][128 rows]
    float m_used = -INFINITY, l = 0.0f;
    // A wait that gives up ends nothing here: the warp notes it, stops waiting and walks on to the end, because its
    // partner (the warp with the other half of the same rows) meets it at a hardware barrier twice per page and
    // would otherwise stay there. The result is then garbage and the status word says so.
    bool ok = true;
    auto wait_warp = [&](uint32_t bar, uint32_t parity, int code) {
      if (ok && !mbar_wait(bar, parity)) {       // every lane polls: no divergence, no shuffle
        ok = false;
        if (lane == 0) atomicExch(a.status, code);
      }
    };
    auto arrive_warp = [&](uint32_t bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory"); };
    uint32_t s_ready = 0;
    for (int j = 0; j < n_pages; ++j) {
      const int b = j & 1, key0 = (page_lo + j) * 64 + half * 32;
      if (!s_ready) wait_warp(s_full + 8 * b, (j >> 1) & 1, 28);
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(lane_addr + (uint32_t)(b * 64 + half * 32), sr);

      // raw scores -> masked raw scores and their maximum; the mask costs two compares and a select per score, so
      // only warps with a row that needs it (the diagonal, a window's edge, padding) run it
      if (__any_sync(0xffffffffu, key0 + 31 > pos || key0 < lo)) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int key = key0 + c;
          if (key > pos || key < lo) sr[c] = 0xff800000u;     // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 2) mx = max3(mx, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
      // The row's maximum is the larger of the two halves'. They are exchanged rounded up to 16 bits (any common
      // reference at or above the maximum serves a softmax), so both threads of a row take the same decisions.
      {
        const uint32_t bits = __float_as_uint(mx);
        const unsigned short up = (unsigned short)(((bits & 0x80000000u) ? bits : bits + 0xffffu) >> 16);
        // a place per page parity: when this is written again two pages on, the partner has passed the barrier of
        // the page between, which it reaches only after reading this one
        xch[b * 256 + half * 128 + r] = up;
        pair_sync();
        const unsigned short other = xch[b * 256 + (half ^ 1) * 128 + r];
        mx = fmaxf(__uint_as_float((uint32_t)up << 16), __uint_as_float((uint32_t)other << 16));
      }
      const float m_new = fmaxf(m_used, mx * a.scale_log2);               // the scale is positive
      const bool grow = m_new > m_used + kRescaleStep;      // also true for the first finite maximum
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        wait_warp(pv_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, 29);      // O must hold all of the last product
        tc_fence_after();
        const float alpha = grow ? ex2(m_used - m_new) : 1.0f;
#pragma unroll
        for (int c0 = 0; c0 < HD / 2; c0 += 16) {      // this thread's half of the accumulator row
          uint32_t o[16];
          tmem_ld16(lane_addr + 128 + half * (HD / 2) + c0, o);
#pragma unroll
          for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st16(lane_addr + 128 + half * (HD / 2) + c0, o);
        }
        l *= alpha;
      }
      if (grow) m_used = m_new;
      const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
      uint32_t pk[16];
      float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[c]), a.scale_log2, neg_m));
        const float p1 = ex2(fmaf(__uint_as_float(sr[c + 1]), a.scale_log2, neg_m));
        l0 += p0;
        l1 += p1;
        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
      }
      l += l0 + l1;
      // asked now, needed at the top of the next page: are its scores complete?
      s_ready = j + 1 < n_pages ? mbar_test(s_full + 8 * (b ^ 1), ((j + 1) >> 1) & 1) : 0u;
      // P_j goes where S_j was: both threads of the row have read their scores (they met at the barrier above), and
      // the product that read P_{j-2} from these columns finished before S_j was written
      tmem_st16(lane_addr + (uint32_t)(b * 64 + half * 16), pk);
      const int valid = seq_len - (page_lo + j) * 64;          // rows of this page that belong to the sequence
      if (valid < 64) {
        wait_warp(v_full + 8 * b, (j >> 1) & 1, 31);
        if (r < 64 && r >= valid && half < HD / 64) {          // each half clears one 64-wide slab of the row
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t dst = sV + (uint32_t)(b * L::KV_BYTES + half * 8192 + r * 128 + ch * 16);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
          }
        }
        fence_smem_to_async();
      }
      tc_fence_before();
      arrive_warp(p_full + 8 * b);
    }
    wait_warp(pv_done + 8 * ((n_pages - 1) & 1), ((n_pages - 1) >> 1) & 1, 32);
    {
      tc_fence_after();
      // the row's sum is the two halves' sums
      float* xl = reinterpret_cast<float*>(smem + L::SUM_OFF);
      xl[half * 128 + r] = l;
      pair_sync();
      l += xl[(half ^ 1) * 128 + r];
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      // this thread's half of the accumulator row: all loads under way at once, one wait
      uint32_t o[HD / 2];
#pragma unroll
      for (int c0 = 0; c0 < HD / 2; c0 += 16) tmem_ld16_nowait(lane_addr + 128 + half * (HD / 2) + c0, o + c0);
      tmem_wait_ld();
      stage_row<HD, HD / 2>(sQ, r, half * (HD / 2), o, inv);
      asm volatile("bar.sync 5, 256;" ::: "memory");      // the eight softmax warps
      store_rows<HD, 8>(sQ, warp - 2, lane, r0, rows_total, ok, a.out, tok0, G, a.heads, kh);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
}

// ------------------------------------------------------------------------------- long tiles ----
// The same walk in steps of two pages (128 keys), for steps whose tiles are long. What bounds one long tile is the
// chain of a step, not a pipe: the scores' load, the exchange of maxima, the exponentials of one thread, P's store
// and the barriers cost the same for 128 keys as for 64 when four threads share a row instead of two. So this form
// has sixteen softmax warps (keys 0..31, 32..63 of the first page, the same of the second), score buffers of 128
// columns, one block an SM (all 512 columns of tensor memory, two stages of two pages each for keys and for values)
// and about half the time per page. Its fixed costs are not hidden by a second block, so short tiles stay with the
// kernel above. A step's second page may not exist (an odd number of pages): its scores are never written and
// are masked like every key behind the row's own position, its product is not issued.
constexpr int kAwThreads = 576;      // score warp, value warp, sixteen softmax warps

template <int HD>
struct AttnWideLayout {
  static constexpr int Q_BYTES = kAtRows * HD * 2;
  static constexpr int PAGE_BYTES = 64 * HD * 2;
  static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;          // two stages
  static constexpr int V_OFF = K_OFF + 2 * STAGE_BYTES;  // two stages
  static constexpr int SUM_OFF = V_OFF + 2 * STAGE_BYTES;        // the parts' row sums, float [4 parts][128 rows]
  static constexpr int BAR_OFF = SUM_OFF + 4 * kAtRows * 4;
  static constexpr int N_BARS = 12;
  static constexpr int XCH_OFF = BAR_OFF + N_BARS * 8 + 16;      // row maxima as 16-bit values, [2 steps][4 parts][128 rows]
  static constexpr int TOTAL = XCH_OFF + 2 * 4 * kAtRows * 2;
  static_assert(TOTAL + 1024 <= 227 * 1024, "the block must fit on an SM");
  static constexpr int TMEM_COLS = 512;                  // S0, S1 (128 each; P takes the first 64 of its S) and O (HD <= 128)
};

template <int HD>
__global__ void __launch_bounds__(kAwThreads, 1)
attn_tc_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, AttnTcArgs a) {
  using L = AttnWideLayout<HD>;
  extern __shared__ __align__(1024) unsigned char smem[];
  Tracer trace(kTraceAttnTc);      // thread 0 issues the score products: past its wait, last scores issued, exit
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_addr(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(a.status, 20);
    return;
  }
  const uint32_t sQ = base + L::Q_OFF, sK = base + L::K_OFF, sV = base + L::V_OFF;
  const uint32_t bars = base + L::BAR_OFF;
  const uint32_t q_full = bars, k_full = bars + 8, v_full = bars + 24, s_full = bars + 40, p_full = bars + 56,
                 pv_done = bars + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::BAR_OFF + L::N_BARS * 8);

  const int pairs = (int)(gridDim.y * gridDim.z);
  const int lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  const int seq = (lin % pairs) / (int)gridDim.y, kh = (lin % pairs) % (int)gridDim.y;
  const int G = a.heads / a.kv_heads;
  const int count = a.counts[seq], past = a.past[seq], tok0 = a.seq_start[seq];
  const int rows_total = count * G;
  const int n_tiles = (rows_total + kAtRows - 1) / kAtRows;
  const int tile = (int)gridDim.x - 1 - lin / pairs;     // longest first
  if (tile >= n_tiles) return;
  const int r0 = tile * kAtRows;
  const int t_first = r0 / G;
  const int t_last = min(rows_total - 1, r0 + kAtRows - 1) / G;
  const int key_lo = a.window > 0 ? max(0, past + t_first - a.window + 1) : 0;
  const int page_lo = key_lo / 64, page_hi = (past + t_last) / 64;
  const int n_pages = page_hi - page_lo + 1;
  const int n_steps = (n_pages + 1) >> 1;
  const int seq_len = past + count;
  const int* table = a.block_table + (size_t)seq * a.table_stride;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(pv_done + 8 * i, 1);
      mbar_init(p_full + 8 * i, 16);     // one arrival per softmax warp
    }
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
  const uint32_t tO = tmem + 256;

  pdl_launch_dependents();     // only now: a successor that also wants tensor memory must not take it before this block has its own
  pdl_wait();
  trace.mark(1);

  if (warp == 0) {
    if (lane == 0) {
      // ---- scores: Q once, two key pages per step, S_j = Q K_j^T a step ahead of the softmax. The two pages of a
      // stage lie one behind the other in each 64-wide half of the head, so one product of N = 128 covers both (an
      // instruction costs the same time whatever its N); the page numbers of the step after next are asked for a
      // step early, and a step's keys are asked for before the products of the step before are issued ----
      constexpr uint32_t idesc_s2 = instr_desc(kAtRows, 128), idesc_s1 = instr_desc(kAtRows, 64);
      auto page_of = [&](int i) { return i < n_pages ? table[page_lo + i] : 0; };
      auto load_keys = [&](int j, int pg0, int pg1) {
        const int s = j & 1, n = min(2, n_pages - 2 * j);
        mbar_expect_tx(k_full + 8 * s, (uint32_t)(n * L::PAGE_BYTES));
        for (int pg = 0; pg < n; ++pg) {
          const int row0 = ((pg ? pg1 : pg0) * a.kv_heads + kh) * 64;
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            tma_load_2d(sK + s * L::STAGE_BYTES + h * 16384 + pg * 8192, &map_k, h * 64, row0, k_full + 8 * s);
        }
      };
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h)
        tma_load_3d(sQ + h * (kAtRows * 128), &map_q, h * 64, kh * G, tok0 + t_first, q_full);
      load_keys(0, page_of(0), page_of(1));
      int nx0 = page_of(2), nx1 = page_of(3);      // the pages of step j + 1
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(a.status, 23);
      for (int j = 0; j < n_steps && ok; ++j) {
        const int s = j & 1, n = min(2, n_pages - 2 * j);
        if (j + 1 < n_steps) {
          // the other key stage was read by S_{j-1}, issued a whole step ago
          if (j >= 1 && !mbar_wait(s_full + 8 * (s ^ 1), ((j - 1) >> 1) & 1)) { atomicExch(a.status, 21); break; }
          load_keys(j + 1, nx0, nx1);
          nx0 = page_of(2 * j + 4);
          nx1 = page_of(2 * j + 5);
        }
        if (!mbar_wait(k_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 24); break; }
        // S_j lands where S_{j-2} and then P_{j-2} lay: the product that read P_{j-2} must be through
        if (j >= 2 && !mbar_wait(pv_done + 8 * s, ((j >> 1) - 1) & 1)) { atomicExch(a.status, 25); break; }
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
          const uint64_t dq = smem_desc(sQ + h * (kAtRows * 128)), dk = smem_desc(sK + s * L::STAGE_BYTES + h * 16384);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            mma_bf16_ss(tmem + (uint32_t)(s * 128), dq + (uint64_t)(k4 * 2), dk + (uint64_t)(k4 * 2), n == 2 ? idesc_s2 : idesc_s1,
                        (h > 0 || k4 > 0) ? 1u : 0u);
        }
        mma_commit(s_full + 8 * s);          // S_j is complete: the softmax may read it, and this key stage is free again
      }
      trace.mark(2);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- values: two value pages per step, O += P_j V_j as soon as the softmax has written P_j ----
      constexpr uint32_t idesc_o = instr_desc(kAtRows, HD, true);
      auto page_of = [&](int i) { return i < n_pages ? table[page_lo + i] : 0; };
      auto load_values = [&](int j, int pg0, int pg1) {
        const int s = j & 1, n = min(2, n_pages - 2 * j);
        mbar_expect_tx(v_full + 8 * s, (uint32_t)(n * L::PAGE_BYTES));
        for (int pg = 0; pg < n; ++pg) {
          const int row0 = ((pg ? pg1 : pg0) * a.kv_heads + kh) * 64;
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            tma_load_2d(sV + s * L::STAGE_BYTES + pg * L::PAGE_BYTES + h * 8192, &map_v, h * 64, row0, v_full + 8 * s);
        }
      };
      load_values(0, page_of(0), page_of(1));
      int nx0 = page_of(2), nx1 = page_of(3);
      for (int j = 0; j < n_steps; ++j) {
        const int s = j & 1, n = min(2, n_pages - 2 * j);
        if (j + 1 < n_steps) {
          // the other value stage was read by the product of step j - 1
          if (j >= 1 && !mbar_wait(pv_done + 8 * (s ^ 1), ((j - 1) >> 1) & 1)) { atomicExch(a.status, 22); break; }
          load_values(j + 1, nx0, nx1);
          nx0 = page_of(2 * j + 4);
          nx1 = page_of(2 * j + 5);
        }
        if (!mbar_wait(v_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 27); break; }
        if (!mbar_wait(p_full + 8 * s, (j >> 1) & 1)) { atomicExch(a.status, 26); break; }
        tc_fence_after();
        for (int pg = 0; pg < n; ++pg) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {      // 16 keys each: 8 columns of P in tensor memory, two 8-key groups of V
            const uint64_t dv = smem_desc_mn(sV + s * L::STAGE_BYTES + pg * L::PAGE_BYTES + k4 * 2048, 8192, 1024);
            mma_bf16_ts(tO, tmem + (uint32_t)(s * 128 + pg * 32 + k4 * 8), dv, idesc_o, (j > 0 || pg > 0 || k4 > 0) ? 1u : 0u);
          }
        }
        mma_commit(pv_done + 8 * s);         // this score buffer and this value stage are free again when it fires
      }
    }
  } else {
    // ---- softmax: warps 2..17. Tensor-memory lanes 32 * (warp % 4) .. + 31 hold the rows; four warps share those
    // lanes, one for each 32 keys of the step: four threads per row ----
    const int quad = warp & 3, part = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int R = r0 + r;
    const int pos = R < rows_total ? past + R / G : -1;        // -1: a padding row sees nothing
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16);
    unsigned short* xch = reinterpret_cast<unsigned short*>(smem + L::XCH_OFF);     // [2 steps][4 parts][128 rows]
    float m_used = -INFINITY, l = 0.0f;
    bool ok = true;      // a wait that gives up ends nothing here, as in the kernel above
    auto wait_warp = [&](uint32_t bar, uint32_t parity, int code) {
      if (ok && !mbar_wait(bar, parity)) {
        ok = false;
        if (lane == 0) atomicExch(a.status, code);
      }
    };
    auto arrive_warp = [&](uint32_t bar) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    };
    auto row_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + quad) : "memory"); };
    uint32_t s_ready = 0;
    for (int j = 0; j < n_steps; ++j) {
      const int b = j & 1, page = page_lo + 2 * j + (part >> 1), key0 = page * 64 + (part & 1) * 32;
      if (!s_ready) wait_warp(s_full + 8 * b, (j >> 1) & 1, 28);
      tc_fence_after();
      uint32_t sr[32];
      tmem_ld32(lane_addr + (uint32_t)(b * 128 + part * 32), sr);

      // a page behind the tile's last one was never multiplied: what lies in its columns is masked like every key
      // behind the row's own position
      if (__any_sync(0xffffffffu, key0 + 31 > pos || key0 < lo)) {
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int key = key0 + c;
          if (key > pos || key < lo) sr[c] = 0xff800000u;     // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; c += 2) mx = max3(mx, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
      {
        const uint32_t bits = __float_as_uint(mx);
        const unsigned short up = (unsigned short)(((bits & 0x80000000u) ? bits : bits + 0xffffu) >> 16);
        unsigned short* x = xch + b * 512 + r;
        x[part * 128] = up;
        row_sync();
        mx = fmaxf(fmaxf(__uint_as_float((uint32_t)x[0] << 16), __uint_as_float((uint32_t)x[128] << 16)),
                   fmaxf(__uint_as_float((uint32_t)x[256] << 16), __uint_as_float((uint32_t)x[384] << 16)));
      }
      const float m_new = fmaxf(m_used, mx * a.scale_log2);               // the scale is positive
      const bool grow = m_new > m_used + kRescaleStep;      // also true for the first finite maximum
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        wait_warp(pv_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, 29);      // O must hold all of the last product
        tc_fence_after();
        const float alpha = grow ? ex2(m_used - m_new) : 1.0f;
#pragma unroll
        for (int c0 = 0; c0 < HD / 4; c0 += 16) {      // this thread's quarter of the accumulator row
          uint32_t o[16];
          tmem_ld16(lane_addr + 256 + part * (HD / 4) + c0, o);
#pragma unroll
          for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
          tmem_st16(lane_addr + 256 + part * (HD / 4) + c0, o);
        }
        l *= alpha;
      }
      if (grow) m_used = m_new;
      const float neg_m = m_used == -INFINITY ? 0.0f : -m_used;
      uint32_t pk[16];
      float l0 = 0.0f, l1 = 0.0f;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {
        const float p0 = ex2(fmaf(__uint_as_float(sr[c]), a.scale_log2, neg_m));
        const float p1 = ex2(fmaf(__uint_as_float(sr[c + 1]), a.scale_log2, neg_m));
        l0 += p0;
        l1 += p1;
        __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
        pk[c >> 1] = *reinterpret_cast<uint32_t*>(&h2);
      }
      l += l0 + l1;
      s_ready = j + 1 < n_steps ? mbar_test(s_full + 8 * (b ^ 1), ((j + 1) >> 1) & 1) : 0u;
      // P_j goes where S_j was: the four threads of the row have read their scores (they met at the barrier above)
      tmem_st16(lane_addr + (uint32_t)(b * 128 + part * 16), pk);
      const int valid = seq_len - page * 64;          // rows of this warp's page that belong to the sequence
      if (page <= page_hi && valid < 64) {
        wait_warp(v_full + 8 * b, (j >> 1) & 1, 31);
        if (r < 64 && r >= valid && (part & 1) < HD / 64) {          // each of the page's two warps-per-quad clears one 64-wide slab
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t dst = sV + (uint32_t)(b * L::STAGE_BYTES + (part >> 1) * L::PAGE_BYTES + (part & 1) * 8192 + r * 128 + ch * 16);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
          }
        }
        fence_smem_to_async();
      }
      tc_fence_before();
      arrive_warp(p_full + 8 * b);
    }
    wait_warp(pv_done + 8 * ((n_steps - 1) & 1), ((n_steps - 1) >> 1) & 1, 32);
    {
      tc_fence_after();
      float* xl = reinterpret_cast<float*>(smem + L::SUM_OFF) + r;
      xl[part * 128] = l;
      row_sync();
      l = (xl[0] + xl[128]) + (xl[256] + xl[384]);
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      uint32_t o[HD / 4];      // this thread's quarter of the accumulator row
#pragma unroll
      for (int c0 = 0; c0 < HD / 4; c0 += 16) tmem_ld16_nowait(lane_addr + 256 + part * (HD / 4) + c0, o + c0);
      tmem_wait_ld();
      stage_row<HD, HD / 4>(sQ, r, part * (HD / 4), o, inv);
      asm volatile("bar.sync 5, 512;" ::: "memory");      // the sixteen softmax warps
      store_rows<HD, 16>(sQ, warp - 2, lane, r0, rows_total, ok, a.out, tok0, G, a.heads, kh);
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

// Which kernel a step takes, from what the host knows: the longest tile's pages (a block's chain: 0.9 us a page
// with one page a step, 0.6 with two) against the pages an SM has to walk in all (0.46 us a page with two blocks of
// the first kernel on an SM, 0.6 with one of the second). `max_keys`: the most keys any sequence has after this
// step (0 = not known: taken as max_count, sequences that start here).
static bool wide_pays(int n_seqs, int max_count, int max_keys, int heads, int kv_heads, int window) {
  const int G = heads / kv_heads;
  const long long tiles = (max_count * (long long)G + kAtRows - 1) / kAtRows, blocks = tiles * kv_heads * n_seqs;
  const int sms = sm_count();
  if (blocks <= sms) return true;          // one round either way: the shorter chain wins
  if (max_keys < max_count) max_keys = max_count;
  int longest = (max_keys + 63) / 64;      // pages of the last tile
  int mean = longest - (max_count / 64) / 2;      // tiles of a prompt grow from its first page to its last
  if (window > 0) {
    const int seen = (window + kAtRows / G + 63) / 64 + 1;
    longest = min(longest, seen);
    mean = min(mean, seen);
  }
  return longest >= 16 && blocks * (long long)max(mean, 1) < (long long)sms * longest * 5 / 4;
}

template <int HD>
static int launch_attn_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcArgs& a,
                          int n_seqs, int max_count, bool wide, cudaStream_t s) {
  const int total = wide ? AttnWideLayout<HD>::TOTAL : AttnTcLayout<HD>::TOTAL;
  static bool configured[2] = {false, false};
  if (!configured[wide]) {
    cudaError_t e = wide ? cudaFuncSetAttribute(attn_tc_wide_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, total)
                         : cudaFuncSetAttribute(attn_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, total);
    if (e != cudaSuccess) return fail(2, "attention (tcgen05): cannot reserve %d bytes of shared memory: %s", total, cudaGetErrorString(e));
    configured[wide] = true;
  }
  const int G = a.heads / a.kv_heads;
  const int tiles = (max_count * G + kAtRows - 1) / kAtRows;
  dim3 grid(tiles, a.kv_heads, n_seqs);
  // its prologue (barriers, tensor memory) runs while the kernel in front drains
  if (wide) launch_prefetching(attn_tc_wide_kernel<HD>, grid, dim3(kAwThreads), (size_t)total, s, mq, mk, mv, a);
  else launch_prefetching(attn_tc_kernel<HD>, grid, dim3(kAtThreads), (size_t)total, s, mq, mk, mv, a);
  return check_launch("attention (tcgen05)");
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(attention_tc)

// 1 when the tcgen05 kernel takes this shape: bfloat16, head size 64 or 128, a group size that divides 128.
extern "C" int slb_attention_tc_supported(int heads, int kv_heads, int head_dim) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 0;
  const int G = heads / kv_heads;
  return (head_dim == 64 || head_dim == 128) && G <= 128 && (128 % G) == 0;
}

// 1 when a step of this shape would take the kernel that walks two pages a step (see wide_pays), else 0.
extern "C" int slb_attention_tc_wide_pays(int n_seqs, int max_count, int max_keys, int heads, int kv_heads, int window) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || n_seqs <= 0 || max_count <= 0) return 0;
  return wide_pays(n_seqs, max_count, max_keys, heads, kv_heads, window) ? 1 : 0;
}

// q [tokens, heads, head_dim]; k_pool, v_pool [pool_pages, kv_heads, 64, head_dim]; out [tokens, heads * head_dim];
// all bfloat16. `status` is a zeroed device int that receives a code if a bounded wait inside the kernel gave up.
// `wide`: 1 = the kernel that walks two pages a step, 0 = the one that walks one, -1 = chosen from the step's shape
// (max_keys: the most keys a sequence has after this step, 0 if not known).
extern "C" int slb_attention_tc(const void* q, const void* k_pool, const void* v_pool, void* out, const int* seq_start,
                                const int* past, const int* counts, const int* block_table, int table_stride,
                                int n_seqs, int max_count, long long tokens, long long pool_pages, int heads,
                                int kv_heads, int head_dim, int window, float scale, int* status, int wide,
                                int max_keys, void* stream) {
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
  const bool use_wide = wide < 0 ? wide_pays(n_seqs, max_count, max_keys, heads, kv_heads, window) : wide != 0;
  return head_dim == 64 ? launch_attn_tc<64>(mq, mk, mv, a, n_seqs, max_count, use_wide, (cudaStream_t)stream)
                        : launch_attn_tc<128>(mq, mk, mv, a, n_seqs, max_count, use_wide, (cudaStream_t)stream);
}
