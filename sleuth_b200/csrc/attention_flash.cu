// Causal grouped-query attention over the paged cache on the tensor cores (bfloat16, head sizes 64 and 128).
//
// Same contract as the general kernel (attention_generic.cu): a step has written its keys and values to the
// cache; a query at position p of sequence s sees keys lo..p of s (lo = max(0, p - window + 1) with a window).
// Formulas: sleuth/forge/model/attention.py:160-206 (mask, 1/sqrt(head_dim) scale, GQA head mapping, float32
// softmax); the reference itself calls a library kernel here (F.scaled_dot_product_attention, attention.py:171-193).
//
// Rows. The G = H / K query heads that share a key/value head are packed into the rows of one tile:
// row r of (sequence, kv head) is token r / G, head kv * G + r % G. A key/value page (64 keys) loaded once thus
// serves all G heads, in prefill and in decode alike.
//
// Two kernels share the inner loop (S = Q K^T by mma.sync m16n8k16, online softmax in float32 with exp2,
// O += P V):
//   * attn_prefill_kernel: a block takes 64 rows of one (sequence, kv head); its 4 warps take 16 rows each
//     and walk the same key pages, double-buffered through shared memory with cp.async.
//   * attn_decode_kernel: every sequence brings one token, so a (sequence, kv head) has only G rows. A block
//     takes one slice of the sequence's pages (split-KV); its 4 warps take 16 keys each of every page, and
//     their partial results (max, sum, weighted values) are merged through shared memory. With more than one
//     slice the block writes an unnormalised partial result to scratch memory, and the block that finishes last
//     (a ticket counter per sequence and kv head tells which) merges the slices in slice order.
// Shared-memory tiles are [64 rows][HD] bfloat16 with the 16-byte chunks of a row XOR-swizzled by the row
// number, which keeps ldmatrix free of bank conflicts.
#include <math.h>

#include "common.cuh"
#include "mma_sync.cuh"

namespace slb {

struct FlashArgs {
  const __nv_bfloat16* q;       // [tokens, H, HD]
  const __nv_bfloat16* k_pool;  // [pages, K, 64, HD]
  const __nv_bfloat16* v_pool;
  __nv_bfloat16* out;           // [tokens, H * HD]
  const int* seq_start;         // [n + 1]
  const int* past;              // [n]
  const int* counts;            // [n]
  const int* block_table;       // [n, table_stride]
  int table_stride;
  int heads, kv_heads, window;
  float scale_log2;             // scale * log2(e)
  // decode only
  NextRead next;                // what the kernel after this one reads (its weights), or nothing
  int splits;
  float* part_o;                // [n, H, splits, HD] unnormalised
  float* part_ml;               // [n, H, splits, 2]  running max (log2 units) and sum
  int* counters;                // [n, kv_heads, row_tiles] zero between launches: slices that have finished
  // decode with the q/k/v post-processing fused in (qkv != null): q is not read; instead the raw projection rows
  const __nv_bfloat16* qkv;     // [n, (H + 2 * qkv_kv_heads) * HD]
  const float* bias;            // [(H + 2 * qkv_kv_heads) * HD] or null
  const float* q_gain;          // [HD] or null
  const float* k_gain;
  const float* cos_table;       // [positions, HD / 2] or null: the whole head is rotated, or nothing
  const float* sin_table;
  float eps;
  int qkv_kv_heads;             // key/value heads present in qkv (0: this layer reads another layer's cache)
  int pages_after_wait;         // 1: no cache page is asked for before the kernel in front has completed (see the kernel)
};

// byte offset of element (row, col) in a swizzled [rows][HD] bf16 tile; col is a multiple of 8
template <int HD> __device__ __forceinline__ uint32_t swz(int row, int col) {
  return (uint32_t)(row * (HD * 2) + ((((col >> 3) ^ (row & 7))) << 4));
}

// Cooperative load of one 64-row page tile (contiguous in global memory) into a swizzled tile. Rows from
// `valid_rows` on lie beyond the sequence's length: a reused page holds another sequence's leftovers there, and
// although their weights are exactly zero, 0 * inf would still poison the sum, so they are filled with zeros.
template <int HD, int THREADS>
__device__ __forceinline__ void load_page(unsigned char* smem_base, uint32_t dst_off, const __nv_bfloat16* src,
                                          int valid_rows, int tid) {
  constexpr int CHUNKS = 64 * HD / 8;
  const uint32_t dst = smem_u32(smem_base) + dst_off;
#pragma unroll
  for (int i = tid; i < CHUNKS; i += THREADS) {
    const int row = i / (HD / 8), ch = i % (HD / 8);
    if (row < valid_rows)
      cp_async16(dst + swz<HD>(row, ch * 8), src + (size_t)row * HD + ch * 8);
    else
      *reinterpret_cast<uint4*>(smem_base + dst_off + swz<HD>(row, ch * 8)) = make_uint4(0, 0, 0, 0);
  }
}

constexpr int kFlashThreads = 128;
constexpr int kMergeBatch = 16;      // slices whose partial results the merging block asks for at once

// ------------------------------------------------------------------------------------ prefill ----
template <int HD>
__global__ void __launch_bounds__(kFlashThreads) attn_prefill_kernel(FlashArgs a) {
  pdl_enter();
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE = 64 * HD * 2;            // bytes of one [64][HD] tile
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + TILE, sV = sK + 2 * TILE;   // two stages each

  const int seq = blockIdx.z, kh = blockIdx.y;
  const int G = a.heads / a.kv_heads;
  const int count = a.counts[seq], past = a.past[seq], tok0 = a.seq_start[seq];
  const int rows_total = count * G;
  const int n_tiles = (rows_total + 63) / 64;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;    // heavy (late) tiles first
  if (tile >= n_tiles) return;
  const int r0 = tile * 64;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int t_first = r0 / G;
  const int t_last = min(rows_total - 1, r0 + 63) / G;
  const int p_hi = past + t_last;
  const int key_lo = a.window > 0 ? max(0, past + t_first - a.window + 1) : 0;
  const int page_lo = key_lo / 64, page_hi = p_hi / 64;
  const int* table = a.block_table + (size_t)seq * a.table_stride;

  // Q tile: row r <- q[tok0 + r / G, kh * G + r % G, :]
  for (int i = tid; i < 64 * (HD / 8); i += kFlashThreads) {
    const int row = i / (HD / 8), ch = i % (HD / 8);
    const int R = r0 + row;
    if (R < rows_total) {
      const __nv_bfloat16* src = a.q + ((size_t)(tok0 + R / G) * a.heads + kh * G + R % G) * HD + ch * 8;
      cp_async16(sQ + swz<HD>(row, ch * 8), src);
    } else {
      *reinterpret_cast<uint4*>(smem + swz<HD>(row, ch * 8)) = make_uint4(0, 0, 0, 0);
    }
  }
  const int seq_len = past + count;
  {
    const size_t base = ((size_t)table[page_lo] * a.kv_heads + kh) * 64 * HD;
    load_page<HD, kFlashThreads>(smem, TILE, a.k_pool + base, seq_len - page_lo * 64, tid);
    load_page<HD, kFlashThreads>(smem, 3 * TILE, a.v_pool + base, seq_len - page_lo * 64, tid);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // this warp's 16 query rows as A fragments
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kb = 0; kb < HD / 16; ++kb) {
    const int row = warp * 16 + (lane & 15), col = kb * 16 + ((lane >> 4) << 3);
    ldmatrix_x4(qf[kb], sQ + swz<HD>(row, col));
  }
  // positions of this thread's two rows (g and g + 8 of the warp's 16)
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = r0 + warp * 16 + g + 8 * h;
    const int p = R < rows_total ? past + R / G : -1;      // -1: a padding row sees nothing
    pos_r[h] = p;
    lo_r[h] = a.window > 0 ? max(0, p - a.window + 1) : 0;
  }
  const int warp_p_min = past + min(rows_total - 1, r0 + warp * 16) / G;
  const int warp_R_last = min(rows_total - 1, r0 + warp * 16 + 15);
  const bool warp_active = r0 + warp * 16 < rows_total;
  const int warp_lo_max = a.window > 0 ? max(0, past + warp_R_last / G - a.window + 1) : 0;

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};

  for (int page = page_lo; page <= page_hi; ++page) {
    const int stage = (page - page_lo) & 1;
    if (page < page_hi) {
      const size_t base = ((size_t)table[page + 1] * a.kv_heads + kh) * 64 * HD;
      load_page<HD, kFlashThreads>(smem, (1 + (stage ^ 1)) * TILE, a.k_pool + base, seq_len - (page + 1) * 64, tid);
      load_page<HD, kFlashThreads>(smem, (3 + (stage ^ 1)) * TILE, a.v_pool + base, seq_len - (page + 1) * 64, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = page * 64;
    // skip pages that lie wholly after this warp's last row or before its first row's window
    if (warp_active && key0 <= past + warp_R_last / G && key0 + 63 >= (a.window > 0 ? max(0, warp_p_min - a.window + 1) : 0)) {
      const uint32_t kS = sK + stage * TILE, vS = sV + stage * TILE;
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
      for (int kb = 0; kb < HD / 16; ++kb) {
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {     // 16 keys at a time
          uint32_t kf[4];
          const int row = jp * 16 + (lane & 7) + ((lane >> 4) << 3), col = kb * 16 + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(kf, kS + swz<HD>(row, col));
          mma_bf16(s[2 * jp], qf[kb], kf[0], kf[1]);
          mma_bf16(s[2 * jp + 1], qf[kb], kf[2], kf[3]);
        }
      }
      const bool need_mask = key0 + 63 > warp_p_min || key0 < warp_lo_max;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          float v = s[j][e] * a.scale_log2;
          if (need_mask) {
            const int key = key0 + j * 8 + 2 * t4 + (e & 1);
            if (key > pos_r[h] || key < lo_r[h]) v = -INFINITY;
          }
          s[j][e] = v;
          mx[h] = fmaxf(mx[h], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_r[h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
        alpha[h] = exp2f(m_r[h] - m_use[h]);
        m_r[h] = m_new;
      }
      float sum[2] = {0.0f, 0.0f};
      uint32_t pf[4][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
        const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
        sum[0] += p0 + p1;
        sum[1] += p2 + p3;
        pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
        pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_r[h] = l_r[h] * alpha[h] + sum[h];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
        o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {         // 16 keys at a time
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) { // 16 channels at a time
          uint32_t vf[4];
          const int row = kb * 16 + (lane & 15), col = dp * 16 + ((lane >> 4) << 3);
          ldmatrix_x4_trans(vf, vS + swz<HD>(row, col));
          mma_bf16(o[2 * dp], pf[kb], vf[0], vf[1]);
          mma_bf16(o[2 * dp + 1], pf[kb], vf[2], vf[3]);
        }
      }
    }
    __syncthreads();
  }

  // the row sums live spread over the 4 threads of a quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = r0 + warp * 16 + g + 8 * h;
    if (R >= rows_total) continue;
    const float inv = 1.0f / l_r[h];
    __nv_bfloat16* dst = a.out + ((size_t)(tok0 + R / G) * a.heads + kh * G + R % G) * HD;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      const uint32_t v = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = v;
    }
  }
}

// ------------------------------------------------------------------------------------- decode ----
// grid: (splits * row_tiles, kv_heads, sequences); every sequence has count 1.
// Three page buffers: while one page is being multiplied, the next two are already on their way, which is what
// keeps the memory system busy when a block's work per page is short compared with the latency of a load.

// One row of the raw q/k/v projection, as csrc/qkv_post.cu treats it: + bias, RMSNorm over the head with `gain`
// (when given), rotation of the whole head by the token's angles (when tables are given); float32 throughout.
// Lane l gets channels l * EPL .. l * EPL + EPL - 1; the whole warp must call.
// The lane's gains, cosines and sines come in registers: they are weights and tables, which the caller fetches before
// it waits for the kernel that writes `src`.
template <int HD>
__device__ __forceinline__ void post_row(const __nv_bfloat16* src, const float* bias, bool normalise,
                                         const float (&gain)[HD / 32], float eps, bool rotate, const float (&cs)[HD / 32],
                                         const float (&sn)[HD / 32], int lane, float (&v)[HD / 32]) {
  constexpr int EPL = HD / 32;
  const int c0 = lane * EPL;
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    float x = __bfloat162float(src[c0 + e]);
    if (bias) x += bias[c0 + e];
    v[e] = x;
    ss = fmaf(x, x, ss);
  }
  if (normalise) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = (v[e] * inv) * gain[e];
  }
  if (rotate) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float partner = __shfl_xor_sync(0xffffffffu, v[e], 16);
      const float other = lane < 16 ? -partner : partner;
      v[e] = v[e] * cs[e] + other * sn[e];
    }
  }
}

// Writes a lane's EPL channels of `row` into a swizzled [rows][HD] bfloat16 tile in shared memory.
template <int HD>
__device__ __forceinline__ void put_row(unsigned char* tile, int row, int lane, const float (&v)[HD / 32]) {
  constexpr int EPL = HD / 32;
  const int c0 = lane * EPL;
  unsigned char* dst = tile + swz<HD>(row, c0 & ~7) + (c0 & 7) * 2;
  if constexpr (EPL == 4) {
    uint2 pk;
    pk.x = pack_bf16(v[0], v[1]);
    pk.y = pack_bf16(v[2], v[3]);
    *reinterpret_cast<uint2*>(dst) = pk;
  } else {
    *reinterpret_cast<uint32_t*>(dst) = pack_bf16(v[0], v[1]);
  }
}

// S: page buffers per block. Three (two pages on their way while one is worked on) is the default; with two, three
// blocks fit an SM instead of two, which lets two slices per (sequence, kv head) run at once where one slice each
// would leave half the GPU idle (see decode_stages).
template <int HD, int S>
__global__ void __launch_bounds__(kFlashThreads) attn_decode_kernel(FlashArgs a) {
  // Fused form: the keys and values of earlier tokens, the block table and the lengths were all written before the
  // kernel that precedes this one began, so pages are requested before the wait for that kernel (which produces
  // only the raw projection of the new token). That holds when this kernel itself appends the token's key and value,
  // and only while an ordinary launch (one that does not start early: a norm, the embedding) stands somewhere
  // between this step's earlier cache writers and this kernel, which is the case when only the prefetching kernels
  // start early. The launcher sets pages_after_wait where it does not hold: the unfused form (the kernel in front
  // writes the newest cache row), an entry that another layer application of this step wrote, and the mode in which
  // every kernel starts early.
  const bool fused = a.qkv != nullptr;
  pdl_launch_dependents();
  if (a.pages_after_wait) pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int TILE = 64 * HD * 2;
  constexpr int EPL = HD / 32;
  const uint32_t sK = smem_u32(smem), sV = sK + S * TILE;
  const uint32_t sQ = sV + S * TILE;          // [16][HD]
  unsigned char* sQ_ptr = smem + 2 * S * TILE;

  Tracer trace(kTraceDecodeAttention);
  const int seq = blockIdx.z, kh = blockIdx.y;
  const int G = a.heads / a.kv_heads;
  const int row_tiles = (G + 15) / 16;
  const int split = blockIdx.x / row_tiles, rt = blockIdx.x % row_tiles;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int pos = a.past[seq], tok = a.seq_start[seq];
  const int key_lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int page_lo = key_lo / 64, page_hi = pos / 64;
  const int n_pages = page_hi - page_lo + 1;
  const int per = (n_pages + a.splits - 1) / a.splits;
  const int my_lo = page_lo + split * per, my_hi = min(page_hi, my_lo + per - 1);
  const int* table = a.block_table + (size_t)seq * a.table_stride;
  const int head0 = kh * G + rt * 16;          // first query head of this row tile
  const int rows = min(16, G - rt * 16);
  // this slice's page numbers, fetched once so that the page loop does not wait for the table
  __shared__ int my_pages[kFlashThreads];
  __shared__ int ticket;
  if (my_lo + tid <= my_hi) my_pages[tid] = table[my_lo + tid];
  auto page_of = [&](int page) { return page - my_lo < kFlashThreads ? my_pages[page - my_lo] : table[page]; };
  __syncthreads();

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};

  auto fetch = [&](int page) {      // one commit group per page, empty beyond the slice
    if (page <= my_hi) {
      const int st = (page - my_lo) % S;
      const size_t base = ((size_t)page_of(page) * a.kv_heads + kh) * 64 * HD;
      load_page<HD, kFlashThreads>(smem, st * TILE, a.k_pool + base, pos + 1 - page * 64, tid);
      load_page<HD, kFlashThreads>(smem, (S + st) * TILE, a.v_pool + base, pos + 1 - page * 64, tid);
    }
    cp_async_commit();
  };
  if (my_lo <= my_hi) {
#pragma unroll
    for (int d = 0; d < S - 1; ++d) fetch(my_lo + d);
  }
  // The fused form's gains and rotation factors for this lane: weights and tables, asked for before the wait.
  float q_gain[EPL], k_gain[EPL], cos_l[EPL], sin_l[EPL];
  const bool norm_q = fused && a.q_gain != nullptr, norm_k = fused && a.k_gain != nullptr;
  const bool rotate = fused && a.cos_table != nullptr;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    q_gain[e] = norm_q ? a.q_gain[lane * EPL + e] : 1.0f;
    k_gain[e] = norm_k ? a.k_gain[lane * EPL + e] : 1.0f;
    cos_l[e] = rotate ? a.cos_table[(size_t)pos * (HD / 2) + (lane & 15) * EPL + e] : 1.0f;
    sin_l[e] = rotate ? a.sin_table[(size_t)pos * (HD / 2) + (lane & 15) * EPL + e] : 0.0f;
  }
  // Nothing but read-only loads may come before this wait: the workspace this kernel writes to is shared with
  // kernels that may still be running.
  if (!a.pages_after_wait) pdl_wait();
  trace.mark(1);
  if (my_lo <= my_hi) {
    // the newest token's own key and value are not in the cache yet in the fused form: the block whose slice
    // holds the last page works them out itself (warp 0 the key, warp 1 the value) and patches its copy of the page
    const bool owns_last = fused && a.qkv_kv_heads > 0 && my_hi == page_hi;
    float new_kv[EPL];
    if (fused) {
      const int rows_per_token = a.heads + 2 * a.qkv_kv_heads;
      const __nv_bfloat16* raw = a.qkv + (size_t)tok * rows_per_token * HD;
      for (int row = warp; row < 16; row += kFlashThreads / 32) {
        float v[EPL];
        if (row < rows) {
          const int head = head0 + row;
          post_row<HD>(raw + (size_t)head * HD, a.bias ? a.bias + (size_t)head * HD : nullptr, norm_q, q_gain, a.eps, rotate,
                       cos_l, sin_l, lane, v);
        } else {
#pragma unroll
          for (int e = 0; e < EPL; ++e) v[e] = 0.0f;
        }
        put_row<HD>(sQ_ptr, row, lane, v);
      }
      if (owns_last && warp < 2) {
        const int r = a.heads + (warp == 0 ? 0 : a.qkv_kv_heads) + kh;
        post_row<HD>(raw + (size_t)r * HD, a.bias ? a.bias + (size_t)r * HD : nullptr, warp == 0 && norm_k, k_gain, a.eps,
                     warp == 0 && rotate, cos_l, sin_l, lane, new_kv);
        if (rt == 0) {      // one block per (sequence, kv head) stores the row for later steps
          __nv_bfloat16* pool = warp == 0 ? const_cast<__nv_bfloat16*>(a.k_pool) : const_cast<__nv_bfloat16*>(a.v_pool);
          __nv_bfloat16* dst = pool + (((size_t)page_of(page_hi) * a.kv_heads + kh) * 64 + (pos % 64)) * HD + lane * EPL;
          if constexpr (EPL == 4) {
            uint2 pk;
            pk.x = pack_bf16(new_kv[0], new_kv[1]);
            pk.y = pack_bf16(new_kv[2], new_kv[3]);
            *reinterpret_cast<uint2*>(dst) = pk;
          } else {
            *reinterpret_cast<uint32_t*>(dst) = pack_bf16(new_kv[0], new_kv[1]);
          }
        }
      }
    } else {
      for (int i = tid; i < 16 * (HD / 8); i += kFlashThreads) {
        const int row = i / (HD / 8), ch = i % (HD / 8);
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < rows) val = *reinterpret_cast<const uint4*>(a.q + ((size_t)tok * a.heads + head0 + row) * HD + ch * 8);
        *reinterpret_cast<uint4*>(sQ_ptr + swz<HD>(row, ch * 8)) = val;
      }
    }
    uint32_t qf[HD / 16][4];

    for (int page = my_lo; page <= my_hi; ++page) {
      const int stage = (page - my_lo) % S;
      fetch(page + S - 1);       // into the buffer that the page before this one has left
      cp_async_wait<S - 1>();    // all but the newest groups: this page has landed
      __syncthreads();
      if (owns_last && page == page_hi) {     // put the new token's key and value where the cache copy has a stale row
        if (warp < 2) put_row<HD>(smem + ((warp == 0 ? 0 : S) + stage) * TILE, pos % 64, lane, new_kv);
        __syncthreads();
      }
      if (page == my_lo) {
#pragma unroll
        for (int kb = 0; kb < HD / 16; ++kb) {
          const int row = lane & 15, col = kb * 16 + ((lane >> 4) << 3);
          ldmatrix_x4(qf[kb], sQ + swz<HD>(row, col));
        }
      }
      const int key0 = page * 64 + warp * 16;     // this warp's 16 keys of the page
      if (key0 <= pos && key0 + 15 >= key_lo) {
        const uint32_t kS = sK + stage * TILE, vS = sV + stage * TILE;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.0f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
#pragma unroll
        for (int kb = 0; kb < HD / 16; ++kb) {
          uint32_t kf[4];
          const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3), col = kb * 16 + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(kf, kS + swz<HD>(row, col));
          mma_bf16(s[0], qf[kb], kf[0], kf[1]);
          mma_bf16(s[1], qf[kb], kf[2], kf[3]);
        }
        // every row of the tile is the same token (different heads): one mask serves all
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + j * 8 + 2 * t4 + (e & 1);
            float v = s[j][e] * a.scale_log2;
            if (key > pos || key < key_lo) v = -INFINITY;
            s[j][e] = v;
          }
        float mxr[2];
        mxr[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mxr[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mxr[h] = fmaxf(mxr[h], __shfl_xor_sync(0xffffffffu, mxr[h], 1));
          mxr[h] = fmaxf(mxr[h], __shfl_xor_sync(0xffffffffu, mxr[h], 2));
          const float m_new = fmaxf(m_r[h], mxr[h]);
          m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
          alpha[h] = exp2f(m_r[h] - m_use[h]);
          m_r[h] = m_new;
        }
        uint32_t pf[4];
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float p0 = exp2f(s[j][0] - m_use[0]), p1 = exp2f(s[j][1] - m_use[0]);
          const float p2 = exp2f(s[j][2] - m_use[1]), p3 = exp2f(s[j][3] - m_use[1]);
          sum[0] += p0 + p1;
          sum[1] += p2 + p3;
          pf[j * 2 + 0] = pack_bf16(p0, p1);
          pf[j * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_r[h] = l_r[h] * alpha[h] + sum[h];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
          o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
          uint32_t vf[4];
          const int row = warp * 16 + (lane & 15), col = dp * 16 + ((lane >> 4) << 3);
          ldmatrix_x4_trans(vf, vS + swz<HD>(row, col));
          mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
          mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
        }
      }
      __syncthreads();
    }
    cp_async_wait<0>();
  }
  trace.mark(2);
  // this block has asked for its last page: the next kernel's weights may now use the memory system
  if (tid == 0)
    prefetch_share(a.next, blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z), gridDim.x * gridDim.y * gridDim.z);

  // merge the four warps (each saw different keys) through shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
    l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
  }
  float* mo = reinterpret_cast<float*>(smem);            // [4 warps][16 rows][HD]
  float* mm = mo + 4 * 16 * HD;                          // [4][16]
  float* ml = mm + 4 * 16;                               // [4][16]
  __syncthreads();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    if (row >= rows) continue;         // only the rows that exist are read back (two of sixteen with two heads a group)
    if (t4 == 0) { mm[warp * 16 + row] = m_r[h]; ml[warp * 16 + row] = l_r[h]; }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
      *reinterpret_cast<float2*>(mo + (warp * 16 + row) * HD + i * 8 + 2 * t4) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
  }
  __syncthreads();
  for (int idx = tid; idx < rows * HD; idx += kFlashThreads) {
    const int row = idx / HD, d = idx % HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mm[w * 16 + row]);
    const float m_use = m == -INFINITY ? 0.0f : m;
    float l = 0.0f, acc = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(mm[w * 16 + row] - m_use);
      l += ml[w * 16 + row] * f;
      acc += mo[(w * 16 + row) * HD + d] * f;
    }
    const int head = head0 + row;
    if (a.splits == 1) {
      a.out[((size_t)tok * a.heads + head) * HD + d] = __float2bfloat16_rn(acc / l);
    } else {
      const size_t pi = ((size_t)seq * a.heads + head) * a.splits + split;
      a.part_o[pi * HD + d] = acc;
      if (d == 0) { a.part_ml[pi * 2] = m; a.part_ml[pi * 2 + 1] = l; }
    }
  }
  if (a.splits == 1) return;
  trace.mark(3);

  // The slice that finishes last merges all slices of its (sequence, kv head, row tile): every block publishes
  // its partial result, then takes a ticket; the holder of the last ticket reads them all back, always in slice
  // order, so the sum does not depend on which block that is. It leaves the counter at zero for the next launch.
  // The block's stores are ordered before the barrier, the barrier before thread 0's ticket, and the ticket is one
  // release-acquire operation at device scope: what the blocks with earlier tickets stored is visible to this thread
  // after it, and through the second barrier to the whole block.
  __syncthreads();
  int* counter = a.counters + ((size_t)seq * a.kv_heads + kh) * row_tiles + rt;
  if (tid == 0) {
    int got;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(got) : "l"(counter) : "memory");
    ticket = got;
  }
  __syncthreads();
  if (ticket != a.splits - 1) return;
  for (int idx = tid; idx < rows * HD; idx += kFlashThreads) {
    const int row = idx / HD, d = idx % HD;
    const int head = head0 + row;
    const size_t base = ((size_t)seq * a.heads + head) * a.splits;
    // sixteen slices at a time, all loads issued before any is used (they come from L2, one latency per batch);
    // a running maximum rescales what has been summed, as in the attention loop itself
    float m = -INFINITY, l = 0.0f, acc = 0.0f;
    for (int s0 = 0; s0 < a.splits; s0 += kMergeBatch) {
      float pm[kMergeBatch], pl[kMergeBatch], po[kMergeBatch];
#pragma unroll
      for (int j = 0; j < kMergeBatch; ++j) {
        const bool live = s0 + j < a.splits;
        pm[j] = live ? __ldcg(a.part_ml + (base + s0 + j) * 2) : -INFINITY;
        pl[j] = live ? __ldcg(a.part_ml + (base + s0 + j) * 2 + 1) : 0.0f;
        po[j] = live ? __ldcg(a.part_o + (base + s0 + j) * HD + d) : 0.0f;
      }
      float m_new = m;
#pragma unroll
      for (int j = 0; j < kMergeBatch; ++j) m_new = fmaxf(m_new, pm[j]);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float keep = exp2f(m - m_use);
      l *= keep;
      acc *= keep;
#pragma unroll
      for (int j = 0; j < kMergeBatch; ++j) {
        const float f = exp2f(pm[j] - m_use);
        l += pl[j] * f;
        acc += po[j] * f;
      }
      m = m_new;
    }
    a.out[((size_t)tok * a.heads + head) * HD + d] = __float2bfloat16_rn(acc / l);
  }
  if (tid == 0) *counter = 0;
}

template <int HD>
static int launch_prefill(const FlashArgs& a, int n_seqs, int max_count, cudaStream_t s) {
  const int G = a.heads / a.kv_heads;
  const int tiles = (max_count * G + 63) / 64;
  const int smem = 5 * 64 * HD * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(2, "attention (prefill): cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(tiles, a.kv_heads, n_seqs);
  launch(attn_prefill_kernel<HD>, dim3(grid), dim3(kFlashThreads), smem, s, a);
  return check_launch("attention (prefill)");
}

// Two page buffers instead of three when that makes all blocks resident at once: with three buffers two blocks fit
// an SM (296 in all), with two buffers three (444).
static int decode_stages(long long blocks) {
  const int sms = sm_count();
  return (blocks > 2ll * sms && blocks <= 3ll * sms) ? 2 : 3;
}

template <int HD, int S>
static int launch_decode_staged(const FlashArgs& a, int n_seqs, cudaStream_t s) {
  const int G = a.heads / a.kv_heads;
  const int row_tiles = (G + 15) / 16;
  const int tiles_bytes = 2 * S * 64 * HD * 2 + 16 * HD * 2;
  const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * 4;
  const int smem = tiles_bytes > merge_bytes ? tiles_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(2, "attention (decode): cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid(a.splits * row_tiles, a.kv_heads, n_seqs);
  if (a.qkv != nullptr)      // the fused form asks for its pages before it waits for the kernel in front of it
    launch_prefetching(attn_decode_kernel<HD, S>, dim3(grid), dim3(kFlashThreads), smem, s, a);
  else
    launch(attn_decode_kernel<HD, S>, dim3(grid), dim3(kFlashThreads), smem, s, a);
  return check_launch("attention (decode)");
}

template <int HD>
static int launch_decode(const FlashArgs& a, int n_seqs, cudaStream_t s) {
  const int row_tiles = (a.heads / a.kv_heads + 15) / 16;
  const long long blocks = (long long)a.splits * row_tiles * a.kv_heads * n_seqs;
  return decode_stages(blocks) == 2 ? launch_decode_staged<HD, 2>(a, n_seqs, s) : launch_decode_staged<HD, 3>(a, n_seqs, s);
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(attention_flash)

// 1 when the tensor-core kernels take this shape, else 0 (the general kernel then serves it).
extern "C" int slb_attention_flash_supported(int head_dim, int dtype) {
  return dtype == kBF16 && (head_dim == 64 || head_dim == 128);
}

// Scratch floats a decode call with `splits` slices needs: partial values plus (max, sum) pairs.
extern "C" long long slb_attention_decode_scratch_floats(int n_seqs, int heads, int head_dim, int splits) {
  return splits <= 1 ? 0 : (long long)n_seqs * heads * splits * (head_dim + 2);
}

extern "C" int slb_attention_prefill(const void* q, const void* k_pool, const void* v_pool, void* out,
                                     const int* seq_start, const int* past, const int* counts, const int* block_table,
                                     int table_stride, int n_seqs, int max_count, int heads, int kv_heads, int head_dim,
                                     int window, float scale, void* stream) {
  SLB_REQUIRE(n_seqs >= 0 && max_count >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention (prefill): seqs=%d max_count=%d heads=%d kv_heads=%d", n_seqs, max_count, heads, kv_heads);
  SLB_REQUIRE(head_dim == 64 || head_dim == 128, "attention (prefill): the tensor-core kernel takes head_dim 64 or 128, got %d", head_dim);
  SLB_REQUIRE(window >= 0 && table_stride > 0 && n_seqs < 65536 && kv_heads < 65536, "attention (prefill): window=%d table_stride=%d", window, table_stride);
  if (n_seqs == 0 || max_count == 0) return 0;
  FlashArgs a{};
  a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
  a.out = (__nv_bfloat16*)out; a.seq_start = seq_start; a.past = past; a.counts = counts;
  a.block_table = block_table; a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads;
  a.window = window; a.scale_log2 = scale * 1.4426950408889634f; a.splits = 1;
  return head_dim == 64 ? launch_prefill<64>(a, n_seqs, max_count, (cudaStream_t)stream)
                        : launch_prefill<128>(a, n_seqs, max_count, (cudaStream_t)stream);
}

extern "C" int slb_attention_decode(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* seq_start, const int* past, const int* block_table, int table_stride,
                                    int n_seqs, int heads, int kv_heads, int head_dim, int window, float scale,
                                    int splits, float* scratch, long long scratch_floats, int* counters,
                                    long long n_counters, const void* qkv, int qkv_kv_heads, const float* bias,
                                    const float* q_gain, const float* k_gain, const float* cos_table,
                                    const float* sin_table, float eps, const void* next, long long next_bytes,
                                    void* stream) {
  // qkv != null: `q` is ignored; the kernel takes the new token's raw projection rows [n, (H + 2 * qkv_kv_heads) * hd],
  // applies bias, QK-norm and the rotation itself, and (qkv_kv_heads == kv_heads) writes the token's key and value
  // into the cache. cos/sin tables, if given, are [positions, hd / 2]: the whole head rotates.
  SLB_REQUIRE(qkv != nullptr || q != nullptr, "attention (decode): neither q nor the raw projection was given");
  SLB_REQUIRE(qkv == nullptr || qkv_kv_heads == 0 || qkv_kv_heads == kv_heads,
              "attention (decode): the raw projection holds %d key/value heads, the cache %d", qkv_kv_heads, kv_heads);
  SLB_REQUIRE(qkv == nullptr || ((q_gain == nullptr) == (k_gain == nullptr)) || qkv_kv_heads == 0,
              "attention (decode): q and k gains go together");
  SLB_REQUIRE(qkv == nullptr || (cos_table == nullptr) == (sin_table == nullptr), "attention (decode): cos and sin tables go together");
  SLB_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
              "attention (decode): seqs=%d heads=%d kv_heads=%d", n_seqs, heads, kv_heads);
  SLB_REQUIRE(head_dim == 64 || head_dim == 128, "attention (decode): the tensor-core kernel takes head_dim 64 or 128, got %d", head_dim);
  SLB_REQUIRE(window >= 0 && table_stride > 0 && splits >= 1 && n_seqs < 65536 && kv_heads < 65536,
              "attention (decode): window=%d table_stride=%d splits=%d", window, table_stride, splits);
  const long long need = slb_attention_decode_scratch_floats(n_seqs, heads, head_dim, splits);
  SLB_REQUIRE(need == 0 || (scratch != nullptr && scratch_floats >= need),
              "attention (decode): %d slices need %lld floats of scratch memory, %lld were given", splits, need, scratch_floats);
  SLB_REQUIRE(splits == 1 || (counters != nullptr && n_counters >= (long long)n_seqs * kv_heads * ((heads / kv_heads + 15) / 16)),
              "attention (decode): %d slices need a zeroed counter per (sequence, kv head, row tile); %lld were given", splits, n_counters);
  if (n_seqs == 0) return 0;
  FlashArgs a{};
  a.counters = counters;
  a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
  a.out = (__nv_bfloat16*)out; a.seq_start = seq_start; a.past = past; a.counts = nullptr;
  a.block_table = block_table; a.table_stride = table_stride; a.heads = heads; a.kv_heads = kv_heads;
  a.window = window; a.scale_log2 = scale * 1.4426950408889634f; a.splits = splits;
  a.part_o = scratch;
  a.part_ml = scratch ? scratch + (size_t)n_seqs * heads * splits * head_dim : nullptr;
  a.qkv = (const __nv_bfloat16*)qkv; a.qkv_kv_heads = qkv_kv_heads; a.bias = bias; a.q_gain = q_gain; a.k_gain = k_gain;
  a.cos_table = cos_table; a.sin_table = sin_table; a.eps = eps;
  a.pages_after_wait = (qkv == nullptr || qkv_kv_heads == 0 || pdl_mode() == 1) ? 1 : 0;
  SLB_REQUIRE(next_bytes >= 0 && (uintptr_t)next % 16 == 0, "attention (decode): the range to prefetch must be 16-byte aligned");
  a.next.ptr = (const char*)next; a.next.bytes = next ? next_bytes : 0;
  return head_dim == 64 ? launch_decode<64>(a, n_seqs, (cudaStream_t)stream)
                        : launch_decode<128>(a, n_seqs, (cudaStream_t)stream);
}
