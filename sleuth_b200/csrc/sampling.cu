// Choosing the next token of every row of a logits matrix [rows, vocab] (float32). The argmax cuts a row into 64
// slices; the sampler gives a row to a cluster of eight thread blocks, an eighth of the row each, which exchange
// their partial maxima, sums and histograms through distributed shared memory between cluster barriers.
//
// Order of operations, as in sleuth/forge/infer/sampling.py:110-127 and :78-107:
//   ban list and repetition penalty (slb_penalize, in place)  ->  temperature <= 0: argmax, first index on ties
//   ->  divide by the temperature  ->  top-k (keep values >= the k-th largest)  ->  top-p (a token goes when the
//   probability mass before it, in descending order, reaches p; the best token always stays)  ->  min-p (drop
//   p < min_p * p_max)  ->  draw from what is left.
//
// The draw is an inverse-CDF walk in token order with one uniform number per row supplied by the caller (a
// counter-based generator on the host keyed by seed, request and step), so a row's token does not depend on the
// batch it is in. Probability masses are kept as 64-bit fixed-point integers (exp(x - max) * 2^40): integer sums
// are exact and order-independent, which makes the thresholds and the draw reproducible although the histograms
// are built with atomics. Tokens tied with the top-p threshold value are kept together (the reference keeps those
// that its unstable sort happens to place first).
//
// Cost at a 152k vocabulary: a pass over the row with exp and division is compute-bound on one SM (~50 us), hence
// the eight blocks; top-k works on the stored values (order is all it needs) and usually leaves few enough tokens
// to finish on a short list in one block.
#include <math.h>

#include <cooperative_groups.h>

#include <atomic>

#include "common.cuh"
#include "no_alloc.h"

namespace cg = cooperative_groups;

namespace slb {

constexpr int kSampleThreads = 1024;
constexpr double kMassScale = 1099511627776.0;  // 2^40

__device__ __forceinline__ unsigned int sort_key(float v) {
  const unsigned int b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // larger float -> larger key
}

__device__ __forceinline__ unsigned long long mass_of(float x, float mx) {
  return (unsigned long long)((double)expf(x - mx) * kMassScale + 0.5);
}

// recent/banned: [rows, stride] token ids with a count per row. Positive logits of recent tokens are divided by
// the penalty, others multiplied (sampling.py:67-75); banned logits become the lowest float (sampling.py:116-120).
// The caller passes each token at most once per row.
__global__ void penalize_kernel(float* logits, long long ld, int limit, const int* recent, const int* n_recent,
                                int recent_stride, float penalty, const int* banned, const int* n_banned,
                                int banned_stride) {
  pdl_enter();
  const int r = blockIdx.x;
  float* row = logits + (size_t)r * ld;
  if (banned) {
    const int n = n_banned[r];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int tok = banned[(size_t)r * banned_stride + i];
      if (tok >= 0 && tok < limit) row[tok] = -3.4028234663852886e38f;
    }
  }
  __syncthreads();
  if (recent && penalty != 1.0f) {
    const int n = n_recent[r];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const int tok = recent[(size_t)r * recent_stride + i];
      if (tok >= 0 && tok < limit) {
        const float v = row[tok];
        row[tok] = v > 0.0f ? v / penalty : v * penalty;
      }
    }
  }
}

// Argmax in two stages so that a few rows still use the whole GPU: kArgmaxChunks blocks per row each find the
// best (value, lowest index) of their slice, then one warp per row picks among the slices. Ties go to the lowest
// index at both stages (sampling.py:104-105 with torch.argmax's first-index rule, tests/test_generate.py:96-104).
constexpr int kArgmaxChunks = 64;
constexpr int kArgmaxThreads = 256;

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_partial_kernel(const float* __restrict__ logits, long long ld, int limit, float* __restrict__ part_v,
                      int* __restrict__ part_i) {
  Tracer trace(kTraceArgmaxPart);
  pdl_enter();
  trace.mark(1);
  __shared__ float best_v[8];
  __shared__ int best_i[8];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const int per = (limit + kArgmaxChunks - 1) / kArgmaxChunks;
  const int begin = chunk * per, end = min(limit, begin + per);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += kArgmaxThreads) {
    const float v = row[i];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < kArgmaxThreads / 32 ? best_v[lane] : -INFINITY;
    bi = lane < kArgmaxThreads / 32 ? best_i[lane] : 0x7fffffff;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { part_v[r * kArgmaxChunks + chunk] = bv; part_i[r * kArgmaxChunks + chunk] = bi; }
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                    int* __restrict__ out) {
  Tracer trace(kTraceArgmaxFinal);
  pdl_enter();
  trace.mark(1);
  const int r = blockIdx.x, lane = threadIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < kArgmaxChunks; c += 32) {
    const float v = part_v[r * kArgmaxChunks + c];
    const int i = part_i[r * kArgmaxChunks + c];
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;   // a row of NaNs picks token 0
}

constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kSampleTeam = 8;        // blocks per row: a thread-block cluster, each block takes an eighth of the row
constexpr int kCandidates = 2048;     // what top-k leaves is kept in shared memory when it is at most this many tokens

// What a block shows to the other blocks of its row (read through distributed shared memory after a cluster
// barrier). Two copies, used alternately: a block may already write its next contribution while a slower block
// still reads the last one, but never the one before that, since a barrier lies between.
struct SampleExchange {
  unsigned long long hist[2][256];
  unsigned long long sum[2];
  float max[2];
  int count[2];
  unsigned long long seg[kSampleWarps];
};

struct SampleShared {
  SampleExchange x;
  unsigned long long hist[256];
  unsigned long long total;
  unsigned long long above;
  unsigned int prefix;
  int chosen;
  int count;
  int flip;
  float red[33];
};

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The blocks that work on one row. With `solo` the block is on its own (the short list after top-k lives in one
// block); otherwise reductions go over the cluster. Every block of a team takes every decision from the same
// numbers, so all of them follow the same path and meet at the same barriers.
struct Team {
  cg::cluster_group cluster;
  SampleShared* sh;
  bool solo;
  int size;
  __device__ int flip() {
    __syncthreads();
    const int f = sh->flip;
    __syncthreads();
    if (threadIdx.x == 0) sh->flip = f ^ 1;
    return f;
  }
  __device__ float max(float v) {
    v = block_max(v, sh->red);
    if (solo) return v;
    const int f = flip();
    if (threadIdx.x == 0) sh->x.max[f] = v;
    cluster.sync();
    float m = -INFINITY;
    for (int c = 0; c < size; ++c) m = fmaxf(m, cluster.map_shared_rank(&sh->x, c)->max[f]);
    return m;
  }
  __device__ unsigned long long sum(unsigned long long v) {
    v = warp_sum_u64(v);
    if (threadIdx.x == 0) sh->total = 0ull;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) atomicAdd(&sh->total, v);
    __syncthreads();
    unsigned long long t = sh->total;
    __syncthreads();
    if (solo) return t;
    const int f = flip();
    if (threadIdx.x == 0) sh->x.sum[f] = t;
    cluster.sync();
    t = 0ull;
    for (int c = 0; c < size; ++c) t += cluster.map_shared_rank(&sh->x, c)->sum[f];
    return t;
  }
  // sh->hist := sum over the team of each block's 32 warp histograms
  __device__ void histogram(const unsigned long long* warp_hist) {
    const int f = solo ? 0 : flip();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
      unsigned long long t = 0ull;
#pragma unroll 8
      for (int w = 0; w < kSampleWarps; ++w) t += warp_hist[w * 256 + b];
      if (solo) sh->hist[b] = t; else sh->x.hist[f][b] = t;
    }
    if (solo) { __syncthreads(); return; }
    cluster.sync();
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
      unsigned long long t = 0ull;
      for (int c = 0; c < size; ++c) t += cluster.map_shared_rank(&sh->x, c)->hist[f][b];
      sh->hist[b] = t;
    }
    __syncthreads();
  }
};

// The tokens a block looks at: its part of the row as stored, its part divided by the temperature on the way in,
// or the list of candidates that top-k left (already divided). `each` hands every element to f(token, value)
// exactly once, spread over the block's threads, in no particular order.
struct RawSource {
  const float* part;      // first element of this block's part
  int base, n;            // its token number, and how many
  template <typename F> __device__ __forceinline__ void each(F f) const {
    if ((reinterpret_cast<uintptr_t>(part) & 15) == 0) {
      const int n4 = n >> 2;
      const float4* r4 = reinterpret_cast<const float4*>(part);
#pragma unroll 4
      for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        const float4 v = r4[i];
        f(base + 4 * i, v.x); f(base + 4 * i + 1, v.y); f(base + 4 * i + 2, v.z); f(base + 4 * i + 3, v.w);
      }
      for (int i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x) f(base + i, part[i]);
    } else {
      for (int i = threadIdx.x; i < n; i += blockDim.x) f(base + i, part[i]);
    }
  }
};
struct RowSource {
  RawSource raw;
  float temp;
  template <typename F> __device__ __forceinline__ void each(F f) const {
    const float t = temp;
    raw.each([&](int i, float v) { f(i, v / t); });
  }
};
struct ListSource {
  const int* token;
  const float* value;
  int n;
  template <typename F> __device__ __forceinline__ void each(F f) const {
    for (int i = threadIdx.x; i < n; i += blockDim.x) f(token[i], value[i]);
  }
};

// Radix descent over the 32-bit sort keys, 8 bits a level. COUNT: each element weighs 1 (top-k), otherwise its
// fixed-point mass (top-p). Among the elements with key >= floor_key it finds the key of the element whose
// inclusion, in descending key order, first makes the accumulated weight reach `target` (>= 1).
// Every warp counts into a histogram of its own: most keys share their top byte, and thirty-two warps adding to the
// same two or three words would take turns. The warps' histograms are summed afterwards, over the whole team.
template <bool COUNT, typename SRC>
__device__ unsigned int radix_threshold(Team& team, const SRC& src, float mx, unsigned int floor_key,
                                        unsigned long long target, unsigned long long* warp_hist) {
  SampleShared& sh = *team.sh;
  unsigned long long* mine = warp_hist + (threadIdx.x >> 5) * 256;
  if (threadIdx.x == 0) { sh.prefix = 0u; sh.above = 0ull; }
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    for (int i = threadIdx.x; i < 256 * kSampleWarps; i += blockDim.x) warp_hist[i] = 0ull;
    __syncthreads();
    const unsigned int prefix = sh.prefix;
    const unsigned int mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    src.each([&](int, float x) {
      const unsigned int key = sort_key(x);
      if (key >= floor_key && (key & mask) == prefix)
        atomicAdd(&mine[(key >> shift) & 255u], COUNT ? 1ull : mass_of(x, mx));
    });
    __syncthreads();
    team.histogram(warp_hist);
    // From bin 255 downwards: the first bin at which what lies above plus the bin reaches the target (bin 0 if none
    // does). Warp 0 does it, eight bins a lane, lane 0 the highest.
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      const int hi = 255 - 8 * lane;
      unsigned long long h[8], mine_sum = 0ull;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        h[j] = (hi - j) > 0 ? sh.hist[hi - j] : 0ull;      // bin 0 is never tested, it only catches what is left
        mine_sum += h[j];
      }
      unsigned long long incl = mine_sum;
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const unsigned long long above = sh.above;
      const unsigned int reach = __ballot_sync(0xffffffffu, above + incl >= target);
      const int first = reach ? __ffs(reach) - 1 : -1;
      const unsigned long long all = __shfl_sync(0xffffffffu, incl, 31);
      __syncwarp();
      if (first < 0) {
        if (lane == 0) { sh.above = above + all; sh.prefix = prefix; }
      } else if (lane == first) {
        unsigned long long acc = above + incl - mine_sum;
        int b = hi;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (acc + h[j] >= target) { b = hi - j; break; }
          acc += h[j];
          b = hi - j - 1;
        }
        sh.above = acc;
        sh.prefix = prefix | ((unsigned int)b << shift);
      }
    }
    __syncthreads();
  }
  const unsigned int found = sh.prefix;
  __syncthreads();
  return found;
}

// Sum over the team of the masses of the elements at or above floor_key.
template <typename SRC>
__device__ unsigned long long kept_mass(Team& team, const SRC& src, float mx, unsigned int floor_key) {
  unsigned long long part = 0ull;
  src.each([&](int, float x) {
    if (sort_key(x) >= floor_key) part += mass_of(x, mx);
  });
  return team.sum(part);
}

// One warp walks `n` elements in order, 32 at a time (element j of its range is get(j) -> (token, value)), and
// returns the token at which the running sum of kept masses, started at `acc`, first exceeds `target`; -1 if none.
template <typename G>
__device__ int warp_walk(int n, G get, float mx, unsigned int floor_key, float min_p, unsigned long long acc,
                         unsigned long long target) {
  const int lane = threadIdx.x & 31;
  for (int j0 = 0; j0 < n; j0 += 32) {
    int tok = -1;
    unsigned long long m = 0ull;
    if (j0 + lane < n) {
      float x;
      get(j0 + lane, tok, x);
      if (sort_key(x) >= floor_key && expf(x - mx) >= min_p) m = mass_of(x, mx);
    }
    unsigned long long incl = m;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned int hit = __ballot_sync(0xffffffffu, m > 0ull && acc + incl > target);
    if (hit) return __shfl_sync(0xffffffffu, tok, __ffs(hit) - 1);
    acc += __shfl_sync(0xffffffffu, incl, 31);
  }
  return -1;
}

__global__ void __cluster_dims__(kSampleTeam, 1, 1) __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, long long ld, int limit, float temperature, int top_k, float top_p,
              float min_p, const float* __restrict__ uniform, int* __restrict__ out) {
  pdl_enter();
  __shared__ SampleShared sh;
  __shared__ int cand_token[kCandidates];
  __shared__ float cand_value[kCandidates];
  extern __shared__ __align__(16) unsigned long long warp_hist[];      // [warps][256]
  Team team{cg::this_cluster(), &sh, false, kSampleTeam};
  const int r = blockIdx.x / kSampleTeam, rank = (int)team.cluster.block_rank();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) sh.flip = 0;
  // this block's part of the row: a contiguous eighth, a multiple of 128 tokens so that 16-byte loads stay aligned
  const float* row = logits + (size_t)r * ld;
  const int per_block = ((limit + kSampleTeam - 1) / kSampleTeam + 127) & ~127;
  const int part_begin = min(limit, rank * per_block), part_end = min(limit, part_begin + per_block);
  const RawSource raw{row + part_begin, part_begin, part_end - part_begin};
  const RowSource whole{raw, temperature};
  __syncthreads();

  // division by a positive temperature keeps the order, so the largest quotient is the quotient of the largest value
  float mx = -INFINITY;
  raw.each([&](int, float x) { mx = fmaxf(mx, x); });
  mx = team.max(mx) / temperature;

  // ---- top-k: the key of the k-th largest value; what it leaves usually fits in shared memory, and everything
  // after works on that short list in one block (sorted by token, since the draw walks in token order) ----
  unsigned int floor_key = 0u;
  bool listed = false;
  int n_listed = 0;
  if (top_k > 0 && top_k < limit) {
    // The k-th largest quotient is the quotient of the k-th largest stored value, so the descent runs on the stored
    // values (no division). Values a little below the k-th one can still round to the same quotient and then stay
    // too (the rule keeps quotients >= the k-th): the cut moves down over them, one float at a time.
    const unsigned int kth_key = radix_threshold<true>(team, raw, 0.0f, 0u, (unsigned long long)top_k, warp_hist);
    if (threadIdx.x == 0) {
      const unsigned int b = (kth_key & 0x80000000u) ? (kth_key & 0x7fffffffu) : ~kth_key;     // back to the float
      float cut = __uint_as_float(b);
      const float q = cut / temperature;
      bool settled = false;
      for (int step = 0; step < 4096; ++step) {
        const float below = nextafterf(cut, -INFINITY);
        if (!(below / temperature == q) || below == cut) { settled = true; break; }
        cut = below;
      }
      sh.prefix = sort_key(cut);
      sh.chosen = settled ? 1 : 0;
      sh.count = 0;
      sh.above = (unsigned long long)sort_key(q);
    }
    __syncthreads();
    const unsigned int raw_floor = sh.prefix;
    const bool settled = sh.chosen != 0;
    floor_key = (unsigned int)sh.above;
    __syncthreads();
    if (settled) {
      raw.each([&](int i, float x) {
        if (sort_key(x) >= raw_floor) {
          const int at = atomicAdd(&sh.count, 1);
          if (at < kCandidates) { cand_token[at] = i; cand_value[at] = x / temperature; }
        }
      });
    } else {      // a temperature so large that thousands of floats share a quotient: compare quotients
      whole.each([&](int i, float x) {
        if (sort_key(x) >= floor_key) {
          const int at = atomicAdd(&sh.count, 1);
          if (at < kCandidates) { cand_token[at] = i; cand_value[at] = x; }
        }
      });
    }
    __syncthreads();
    // how many candidates the whole team holds; if they fit, block 0 collects them and goes on alone
    const int f = team.flip();
    if (threadIdx.x == 0) sh.x.count[f] = sh.count;
    team.cluster.sync();
    int n = 0, before = 0;
    for (int c = 0; c < kSampleTeam; ++c) {
      const int k = team.cluster.map_shared_rank(&sh.x, c)->count[f];
      if (c < rank) before += k;
      n += k;
    }
    (void)before;
    if (n <= kCandidates) {
      listed = true;
      n_listed = n;
      int* all_token = reinterpret_cast<int*>(warp_hist);
      float* all_value = reinterpret_cast<float*>(warp_hist) + kCandidates;
      if (rank == 0) {
        int at = 0;
        for (int c = 0; c < kSampleTeam; ++c) {
          const int k = team.cluster.map_shared_rank(&sh.x, c)->count[f];
          const int* their_token = team.cluster.map_shared_rank(cand_token, c);
          const float* their_value = team.cluster.map_shared_rank(cand_value, c);
          for (int i = threadIdx.x; i < k; i += blockDim.x) { all_token[at + i] = their_token[i]; all_value[at + i] = their_value[i]; }
          at += k;
        }
      }
      team.cluster.sync();           // the lists have been read: the other blocks may leave
      if (rank != 0) return;
      team.solo = true;
      // order by token: each entry counts the entries with a smaller token
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int t = all_token[i];
        int pos = 0;
        for (int j = 0; j < n; ++j) pos += all_token[j] < t ? 1 : 0;
        cand_token[pos] = t;
        cand_value[pos] = all_value[i];
      }
      __syncthreads();
    }
  }
  const ListSource list{cand_token, cand_value, n_listed};

  // ---- top-p: the key at which the descending running mass of what top-k left reaches p * total ----
  if (top_p < 1.0f) {
    const unsigned long long total = listed ? kept_mass(team, list, mx, floor_key) : kept_mass(team, whole, mx, floor_key);
    unsigned long long target = (unsigned long long)ceil((double)top_p * (double)total);
    if (target < 1ull) target = 1ull;
    if (target > total) target = total;
    floor_key = listed ? radix_threshold<false>(team, list, mx, floor_key, target, warp_hist)
                       : radix_threshold<false>(team, whole, mx, floor_key, target, warp_hist);
  }

  // ---- the draw: in token order, the token at which the running sum of kept masses passes uniform * total ----
  if (listed) {
    // a short list: warp 0 sums it and walks it
    if (warp == 0) {
      unsigned long long mine = 0ull;
      for (int i = lane; i < list.n; i += 32) {
        const float x = cand_value[i];
        if (sort_key(x) >= floor_key && expf(x - mx) >= min_p) mine += mass_of(x, mx);
      }
      const unsigned long long total = warp_sum_u64(mine);
      unsigned long long target = (unsigned long long)((double)uniform[r] * (double)total);
      if (total > 0ull && target >= total) target = total - 1ull;
      int pick = -1;
      if (total > 0ull)
        pick = warp_walk(list.n, [&](int j, int& tok, float& x) { tok = cand_token[j]; x = cand_value[j]; }, mx, floor_key,
                         min_p, 0ull, target);
      if (lane == 0) out[r] = pick >= 0 ? pick : 0;
    }
    return;
  }
  // the whole row: every warp of every block owns a contiguous stretch of tokens and sums it (coalesced loads), each
  // block finds the stretch the draw falls into, and the warp that owns it walks it
  const int stretch = ((raw.n + kSampleWarps - 1) / kSampleWarps + 31) & ~31;
  const int begin = min(raw.n, warp * stretch), end = min(raw.n, begin + stretch);
  {
    unsigned long long mine = 0ull;
    for (int i = begin + lane; i < end; i += 32) {
      const float x = raw.part[i] / temperature;
      if (sort_key(x) >= floor_key && expf(x - mx) >= min_p) mine += mass_of(x, mx);
    }
    mine = warp_sum_u64(mine);
    if (lane == 0) sh.x.seg[warp] = mine;
  }
  __syncthreads();
  // the blocks' totals go round; every block then knows the draw's target and which block it falls into
  unsigned long long block_total = 0ull;
  for (int w = 0; w < kSampleWarps; ++w) block_total += sh.x.seg[w];
  const int f = team.flip();
  if (threadIdx.x == 0) sh.x.sum[f] = block_total;
  team.cluster.sync();
  unsigned long long total = 0ull, before = 0ull;
  for (int c = 0; c < kSampleTeam; ++c) {
    const unsigned long long t = team.cluster.map_shared_rank(&sh.x, c)->sum[f];
    if (c < rank) before += t;
    total += t;
  }
  unsigned long long target = (unsigned long long)((double)uniform[r] * (double)total);
  if (total > 0ull && target >= total) target = total - 1ull;
  if (total == 0ull) {
    if (rank == 0 && threadIdx.x == 0) out[r] = 0;
  } else if (target >= before && target < before + block_total) {
    // this block's stretch: find the warp, which then walks its tokens
    unsigned long long acc = before;
    int which = -1;
    for (int w = 0; w < kSampleWarps; ++w) {
      const unsigned long long t = sh.x.seg[w];
      if (t > 0ull && target < acc + t) { which = w; break; }
      acc += t;
    }
    if (warp == which) {
      const int pick = warp_walk(end - begin,
                                 [&](int j, int& tok, float& x) { tok = raw.base + begin + j; x = raw.part[begin + j] / temperature; },
                                 mx, floor_key, min_p, acc, target);
      if (lane == 0) out[r] = pick >= 0 ? pick : 0;
    }
  }
  team.cluster.sync();             // nobody leaves while another block may still read its total
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(sampling)

extern "C" int slb_penalize(float* logits, long long ld, int rows, int limit, const int* recent, const int* n_recent,
                            int recent_stride, float penalty, const int* banned, const int* n_banned,
                            int banned_stride, void* stream) {
  SLB_REQUIRE(rows >= 0 && limit > 0 && ld >= limit, "penalize: rows=%d limit=%d ld=%lld", rows, limit, ld);
  SLB_REQUIRE(penalty > 0.0f, "penalize: repetition penalty must be positive, got %g", (double)penalty);
  if (rows == 0 || (!recent && !banned)) return 0;
  launch(penalize_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)stream, logits, ld, limit, recent, n_recent, recent_stride, penalty,
                                                          banned, n_banned, banned_stride);
  return check_launch("penalize");
}

// scratch: 2 * rows * 64 four-byte words (slb_argmax_scratch_words), written and read within the call.
extern "C" long long slb_argmax_scratch_words(int rows) { return 2ll * rows * kArgmaxChunks; }

extern "C" int slb_argmax(const float* logits, long long ld, int rows, int limit, int* out, void* scratch,
                          long long scratch_words, void* stream) {
  SLB_REQUIRE(rows >= 0 && rows < 65536 && limit > 0 && ld >= limit, "argmax: rows=%d limit=%d ld=%lld", rows, limit, ld);
  SLB_REQUIRE(rows == 0 || (logits != nullptr && out != nullptr), "argmax: logits and out must be device pointers, not null");
  SLB_REQUIRE(scratch != nullptr && scratch_words >= slb_argmax_scratch_words(rows),
              "argmax: %lld words of scratch memory are needed, %lld were given", slb_argmax_scratch_words(rows), scratch_words);
  if (rows == 0) return 0;
  float* part_v = (float*)scratch;
  int* part_i = (int*)scratch + (size_t)rows * kArgmaxChunks;
  cudaStream_t s = (cudaStream_t)stream;
  launch(argmax_partial_kernel, dim3(dim3(kArgmaxChunks, rows)), dim3(kArgmaxThreads), 0, s, logits, ld, limit, part_v, part_i);
  int rc = check_launch("argmax (slices)");
  if (rc) return rc;
  launch(argmax_final_kernel, dim3(rows), dim3(32), 0, s, part_v, part_i, out);
  return check_launch("argmax");
}

// ---------------------------------------------------------------- argmax without any allocation ----
// See no_alloc.h. The slices' partial results live in a fixed array inside the library image instead of in
// memory the caller hands over. In host code the array's name is only a handle: its device address is asked
// for once per device (cudaGetSymbolAddress, with that device current) and kept.
constexpr int kStaticArgmaxRows = SLB_ARGMAX_STATIC_MAX_ROWS;
static __device__ __align__(256) unsigned int g_argmax_scratch[2 * kStaticArgmaxRows * kArgmaxChunks];
static std::atomic<void*> g_argmax_scratch_addr[64];     // per device; host threads may race to fill a slot: all write the same address

extern "C" int slb_argmax_static(const float* logits, long long ld, int rows, int limit, int* out, void* stream) {
  SLB_REQUIRE(rows >= 0 && limit > 0 && ld >= limit, "argmax_static: rows=%d limit=%d ld=%lld", rows, limit, ld);
  SLB_REQUIRE(rows == 0 || (logits != nullptr && out != nullptr), "argmax_static: logits and out must be device pointers, not null");
  SLB_REQUIRE(rows <= kStaticArgmaxRows,
              "argmax_static: %d rows are more than the built-in scratch array holds (%d); use slb_argmax with scratch "
              "memory of your own", rows, kStaticArgmaxRows);
  if (rows == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(2, "argmax_static: no usable current device (%s)", cudaGetErrorString(e));
  void* base = g_argmax_scratch_addr[dev].load(std::memory_order_acquire);
  if (base == nullptr) {
    e = cudaGetSymbolAddress(&base, g_argmax_scratch);     // first call on this device; not during stream capture
    if (e != cudaSuccess || base == nullptr)
      return fail(2, "argmax_static: cannot find the scratch array on device %d: %s", dev, cudaGetErrorString(e));
    g_argmax_scratch_addr[dev].store(base, std::memory_order_release);
  }
  float* part_v = (float*)base;
  int* part_i = (int*)base + (size_t)kStaticArgmaxRows * kArgmaxChunks;
  cudaStream_t s = (cudaStream_t)stream;
  // every slot that the second stage reads is written by the first stage of the same call, so nothing left in
  // the array by an earlier call is ever read and nothing has to be cleared
  launch(argmax_partial_kernel, dim3(kArgmaxChunks, rows), dim3(kArgmaxThreads), 0, s, logits, ld, limit, part_v, part_i);
  int rc = check_launch("argmax_static (slices)");
  if (rc) return rc;
  launch(argmax_final_kernel, dim3(rows), dim3(32), 0, s, (const float*)part_v, (const int*)part_i, out);
  return check_launch("argmax_static");
}

extern "C" int slb_argmax_static_max_rows() { return kStaticArgmaxRows; }

extern "C" int slb_sample(const float* logits, long long ld, int rows, int limit, float temperature, int top_k,
                          float top_p, float min_p, const float* uniform, int* out, void* stream) {
  SLB_REQUIRE(rows >= 0 && limit > 0 && ld >= limit, "sample: rows=%d limit=%d ld=%lld", rows, limit, ld);
  SLB_REQUIRE(temperature > 0.0f, "sample: temperature must be positive here (argmax handles <= 0), got %g",
              (double)temperature);
  SLB_REQUIRE(top_k >= 0 && top_p > 0.0f && min_p >= 0.0f && min_p <= 1.0f, "sample: top_k=%d top_p=%g min_p=%g", top_k,
              (double)top_p, (double)min_p);
  if (rows == 0) return 0;
  const size_t hist_bytes = (size_t)(kSampleThreads / 32) * 256 * sizeof(unsigned long long);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_bytes);
    if (e != cudaSuccess) return fail(2, "sample: cannot reserve %d bytes of shared memory: %s", (int)hist_bytes, cudaGetErrorString(e));
    configured = true;
  }
  launch(sample_kernel, dim3(rows * kSampleTeam), dim3(kSampleThreads), hist_bytes, (cudaStream_t)stream, logits, ld, limit, temperature, top_k, top_p,
         min_p, uniform, out);
  return check_launch("sample");
}
