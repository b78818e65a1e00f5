// Choosing the next token of every row of a logits matrix [rows, vocab] (float32), one thread block per row.
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
#include <math.h>

#include "common.cuh"
#include "no_alloc.h"

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
  pdl_enter();
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
  pdl_enter();
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

struct SampleShared {
  unsigned long long hist[256];
  unsigned long long scan[kSampleThreads / 32 + 1];
  unsigned long long total;
  unsigned int prefix;
  unsigned long long above;
  float red[33];
  int chosen;
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

// Radix descent over the 32-bit sort keys, 8 bits a level. COUNT: each element weighs 1 (top-k), otherwise its
// fixed-point mass (top-p). Among the elements with key >= floor_key it finds the key of the element whose
// inclusion, in descending key order, first makes the accumulated weight reach `target` (>= 1).
template <bool COUNT>
__device__ unsigned int radix_threshold(const float* row, int limit, float temp, float mx, unsigned int floor_key,
                                        unsigned long long target, SampleShared& sh) {
  if (threadIdx.x == 0) { sh.prefix = 0u; sh.above = 0ull; }
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.hist[i] = 0ull;
    __syncthreads();
    const unsigned int prefix = sh.prefix;
    const unsigned int mask = level == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < limit; i += blockDim.x) {
      const float x = row[i] / temp;
      const unsigned int key = sort_key(x);
      if (key < floor_key || (key & mask) != prefix) continue;
      atomicAdd(&sh.hist[(key >> shift) & 255u], COUNT ? 1ull : mass_of(x, mx));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long acc = sh.above;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + sh.hist[b] >= target) break;
        acc += sh.hist[b];
      }
      sh.above = acc;
      sh.prefix = prefix | ((unsigned int)b << shift);
    }
    __syncthreads();
  }
  return sh.prefix;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, long long ld, int limit, float temperature, int top_k, float top_p,
              float min_p, const float* __restrict__ uniform, int* __restrict__ out) {
  pdl_enter();
  __shared__ SampleShared sh;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature;

  float mx = -INFINITY;
  for (int i = threadIdx.x; i < limit; i += blockDim.x) mx = fmaxf(mx, row[i] / temp);
  mx = block_max(mx, sh.red);

  unsigned int floor_key = 0u;
  if (top_k > 0 && top_k < limit)
    floor_key = radix_threshold<true>(row, limit, temp, mx, 0u, (unsigned long long)top_k, sh);

  if (top_p < 1.0f) {
    // total mass of what top-k left, then the key at which the descending running mass reaches p * total
    unsigned long long part = 0ull;
    for (int i = threadIdx.x; i < limit; i += blockDim.x) {
      const float x = row[i] / temp;
      if (sort_key(x) >= floor_key) part += mass_of(x, mx);
    }
    if (threadIdx.x == 0) sh.total = 0ull;
    __syncthreads();
    atomicAdd(&sh.total, part);
    __syncthreads();
    unsigned long long target = (unsigned long long)ceil((double)top_p * (double)sh.total);
    if (target < 1ull) target = 1ull;
    if (target > sh.total) target = sh.total;
    __syncthreads();
    floor_key = radix_threshold<false>(row, limit, temp, mx, floor_key, target, sh);
  }

  // Each thread owns a contiguous run of tokens; integer prefix sums of the kept masses locate the draw.
  const int chunk = (limit + blockDim.x - 1) / blockDim.x;
  const int begin = min(limit, (int)threadIdx.x * chunk), end = min(limit, begin + chunk);
  unsigned long long mine = 0ull;
  for (int i = begin; i < end; ++i) {
    const float x = row[i] / temp;
    if (sort_key(x) >= floor_key && expf(x - mx) >= min_p) mine += mass_of(x, mx);
  }
  // inclusive scan over threads: within warps by shuffles, then over the warp totals
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long incl = mine;
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) sh.scan[warp] = incl;
  if (threadIdx.x == 0) sh.chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long acc = 0ull;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      const unsigned long long t = sh.scan[w];
      sh.scan[w] = acc;
      acc += t;
    }
    sh.total = acc;
  }
  __syncthreads();
  const unsigned long long total = sh.total;
  const unsigned long long before = sh.scan[warp] + incl - mine;
  unsigned long long target = (unsigned long long)((double)uniform[r] * (double)total);
  if (target >= total) target = total - 1ull;
  if (total > 0ull && mine > 0ull && target >= before && target < before + mine) {
    unsigned long long acc = before;
    int pick = begin;
    for (int i = begin; i < end; ++i) {
      const float x = row[i] / temp;
      if (sort_key(x) >= floor_key && expf(x - mx) >= min_p) {
        const unsigned long long m = mass_of(x, mx);
        if (m > 0ull) pick = i;
        acc += m;
        if (acc > target) break;
      }
    }
    sh.chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = sh.chosen >= 0 ? sh.chosen : 0;
}

}  // namespace slb

using namespace slb;

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
static void* g_argmax_scratch_addr[64] = {nullptr};

extern "C" int slb_argmax_static(const float* logits, long long ld, int rows, int limit, int* out, void* stream) {
  SLB_REQUIRE(rows >= 0 && limit > 0 && ld >= limit, "argmax_static: rows=%d limit=%d ld=%lld", rows, limit, ld);
  SLB_REQUIRE(rows <= kStaticArgmaxRows,
              "argmax_static: %d rows are more than the built-in scratch array holds (%d); use slb_argmax with scratch "
              "memory of your own", rows, kStaticArgmaxRows);
  if (rows == 0) return 0;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(2, "argmax_static: no usable current device (%s)", cudaGetErrorString(e));
  if (g_argmax_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_argmax_scratch);     // first call on this device; not during stream capture
    if (e != cudaSuccess || p == nullptr)
      return fail(2, "argmax_static: cannot find the scratch array on device %d: %s", dev, cudaGetErrorString(e));
    g_argmax_scratch_addr[dev] = p;
  }
  float* part_v = (float*)g_argmax_scratch_addr[dev];
  int* part_i = (int*)g_argmax_scratch_addr[dev] + (size_t)kStaticArgmaxRows * kArgmaxChunks;
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
  launch(sample_kernel, dim3(rows), dim3(kSampleThreads), 0, (cudaStream_t)stream, logits, ld, limit, temperature, top_k, top_p, min_p,
                                                                  uniform, out);
  return check_launch("sample");
}
