// Shared helpers of the sleuth_b200 kernels (sm_100a).
//
// Conventions of every exported launcher:
//   * `extern "C" int slb_<name>(..., void* stream)`; returns 0, or a non-zero code after storing a
//     message that `slb_last_error()` returns. A launcher checks every size it was given and refuses
//     what its kernel cannot run; it never launches a kernel on sizes it has not checked.
//   * activations and cache entries are `float` or `__nv_bfloat16` (the launcher's `dtype` argument:
//     0 = float32, 1 = bfloat16); the residual stream, norm gains, biases, rotation tables and logits
//     are always float32; all reductions accumulate in float32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace slb {

constexpr int kPageTokens = 64;   // tokens per cache page

enum Dtype : int { kF32 = 0, kBF16 = 1 };

int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define SLB_REQUIRE(cond, ...)                    \
  do {                                            \
    if (!(cond)) return slb::fail(1, __VA_ARGS__); \
  } while (0)

// Programmatic dependent launch. Every kernel of this library is launched with the stream-serialization
// attribute (unless slb_set_pdl(0) turned it off): it may then begin while the kernel before it in the stream is
// still running. A kernel first lets its own successor start (pdl_launch_dependents), may fetch data that no
// kernel writes (weights), and must call pdl_wait() before it reads or writes anything else: the wait returns
// when the preceding kernel has completed and its writes are visible. Without the attribute both are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_launch_dependents();
  pdl_wait();
}

// A range of memory that the kernel after this one will read and that no kernel writes (the next weight matrix).
// The blocks of a kernel that is given one ask the L2 cache for it, a share each, so that the next kernel finds its
// weights on the chip: a single-token step leaves the memory system idle more than half of the time, and a kernel
// that starts early cannot fetch for itself while the blocks in front of it still hold the SM's registers.
struct NextRead {
  const char* ptr;
  long long bytes;
};

__device__ __forceinline__ void prefetch_share(const NextRead& n, int block, int blocks) {
  if (n.bytes <= 0) return;
  const long long share = (((n.bytes + blocks - 1) / blocks) + 127) & ~127LL;      // whole 128-byte lines
  long long off = (long long)block * share;
  const long long end = min(n.bytes & ~15LL, off + share);
  for (; off < end; off += 32768) {
    const uint32_t size = (uint32_t)min(32768LL, end - off);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(n.ptr + off), "r"(size) : "memory");
  }
}

// The first pages that the single-token attention kernel two launches on will read: that kernel's blocks get onto the
// SMs only when the blocks of the product in front of it leave, too late to fetch ahead for themselves, while the
// memory system idles through most of that product. So the product's blocks ask the L2 cache for them: item
// i = ((sequence * splits + slice) * depth + d) * 2 + (0 key page | 1 value page), the slices cut as
// attn_decode_kernel cuts them. A page here is a cache page of all kv heads (they lie together).
struct NextPages {
  const char* k_pool;        // null: nothing to do
  const char* v_pool;
  const int* block_table;    // [n_seqs, table_stride]
  const int* past;           // [n_seqs] position of each sequence's new token
  long long page_bytes;
  int table_stride, n_seqs, splits, depth, window;
};

// The whole warp calls; every lane works out the same page, lanes 0.. ask for 32 KB of it each.
__device__ __forceinline__ void prefetch_page_item(const NextPages& p, int item, int lane) {
  const int which = item & 1;
  int rest = item >> 1;
  const int d = rest % p.depth;
  rest /= p.depth;
  const int slice = rest % p.splits, seq = rest / p.splits;
  if (seq >= p.n_seqs) return;
  const int pos = p.past[seq];
  const int key_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int page_lo = key_lo / 64, page_hi = pos / 64;
  const int per = (page_hi - page_lo + 1 + p.splits - 1) / p.splits;
  const int my_lo = page_lo + slice * per, my_hi = min(page_hi, my_lo + per - 1);
  const int page = my_lo + d;
  if (page > my_hi || page >= p.table_stride) return;
  const int phys = p.block_table[(size_t)seq * p.table_stride + page];
  const char* base = (which ? p.v_pool : p.k_pool) + (size_t)phys * p.page_bytes;
  const long long off = (long long)lane * 32768;
  if (off < p.page_bytes) {
    const uint32_t size = (uint32_t)min(32768LL, (p.page_bytes - off) & ~15LL);
    if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(size) : "memory");
  }
}

// A timeline of the kernels, for finding where a step's time goes between and inside its launches. It exists only
// in a library compiled with -DSLB_TIMELINE (otherwise every line below is empty): thread 0 of each block reads the
// global nanosecond timer when the block enters, at up to three marks, and when it leaves, and appends one record of
// six 64-bit words [kind | block << 16 | SM << 48, enter, mark 1, mark 2, mark 3, leave] to a buffer whose first word
// counts the records. Each file with kernels keeps its own pointer to the buffer (slb_timeline_set_<file>).
enum TraceKind : int { kTraceEmbed = 1, kTraceNorm, kTraceSkinny, kTraceDecodeAttention, kTraceArgmaxPart, kTraceArgmaxFinal,
                       kTraceSample, kTraceOther, kTraceGemmTc, kTraceAttnTc };
#ifdef SLB_TIMELINE
static __device__ unsigned long long* g_timeline = nullptr;
static __device__ unsigned int g_timeline_records = 0;
#define SLB_TIMELINE_SETTER(file)                                                          \
  extern "C" int slb_timeline_set_##file(void* buffer, unsigned int records) {            \
    cudaError_t e = cudaMemcpyToSymbol(slb::g_timeline, &buffer, sizeof(buffer));          \
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(slb::g_timeline_records, &records, sizeof(records)); \
    return e == cudaSuccess ? 0 : 2;                                                       \
  }
struct Tracer {
  unsigned long long t[4];
  int kind;
  static __device__ __forceinline__ unsigned long long now() {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
  }
  __device__ __forceinline__ explicit Tracer(int k) : kind(k) {
    t[0] = now();
    t[1] = t[2] = t[3] = 0;
  }
  __device__ __forceinline__ void mark(int i) {
    if (threadIdx.x == 0 && threadIdx.y == 0) t[i] = now();
  }
  __device__ __forceinline__ ~Tracer() {
    if (threadIdx.x != 0 || threadIdx.y != 0 || g_timeline == nullptr) return;
    const unsigned long long leave = now();
    const unsigned int i = atomicAdd(reinterpret_cast<unsigned int*>(g_timeline), 1u);
    if (i >= g_timeline_records) return;
    unsigned int sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    const unsigned long long block = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    unsigned long long* r = g_timeline + 1 + 6ull * i;
    r[0] = (unsigned long long)kind | (block << 16) | ((unsigned long long)sm << 48);
    r[1] = t[0]; r[2] = t[1]; r[3] = t[2]; r[4] = t[3]; r[5] = leave;
  }
};
#else
#define SLB_TIMELINE_SETTER(file)
struct Tracer {
  __device__ __forceinline__ explicit Tracer(int) {}
  __device__ __forceinline__ void mark(int) {}
};
#endif

int sm_count();                       // streaming multiprocessors of the current device (148 on a B200)
int pdl_mode();                       // 0 off, 1 every kernel, 2 only kernels that prefetch before their wait
inline bool pdl_enabled() { return pdl_mode() != 0; }
void note_launch_error(cudaError_t e);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_with(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = early ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) note_launch_error(e);
  return e;
}

// The same for kernels whose blocks come in clusters of `cluster` along x (the grid's x must be a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_clusters(bool early, unsigned cluster, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                   size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = early ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  if (e != cudaSuccess) note_launch_error(e);
  return e;
}

// Ordinary kernels: allowed to start early only in mode 1. Kernels that fetch weights before their wait: modes 1 and 2.
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
  return launch_with(pdl_mode() == 1, kernel, grid, block, smem, stream, args...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_prefetching(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args... args) {
  return launch_with(pdl_mode() != 0, kernel, grid, block, smem, stream, args...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
// The order of additions is fixed by the thread layout, so a row's sum never depends on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// 8 bfloat16 values in one 16-byte register group.
struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const Bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

}  // namespace slb
