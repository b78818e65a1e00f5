// bfloat16 matrix product on the fifth-generation tensor cores: C[M, N] = X[M, K] * W[N, K]^T for many rows (prefill).
//
// One block per SM walks over 128 x BN tiles of C (BN = 32 to 256 columns), with two accumulators in tensor memory
// so that the epilogue of one tile overlaps the products of the next:
//   * warp 0, one lane: the producer. For every 64-wide slice of K it asks TMA (cp.async.bulk.tensor) for the
//     128 x 64 tile of X and the BN x 64 tile of W; both arrive in shared memory in the 128-byte-swizzled K-major
//     layout that the tensor core reads, and their arrival is counted on the stage's "full" mbarrier.
//   * warp 1, one lane: the MMA issuer. It waits for a full stage and issues four tcgen05.mma (K = 16 each,
//     M = 128, N = BN) that accumulate into tensor memory (TMEM), then tcgen05.commit makes the stage's "empty"
//     mbarrier fire when those MMAs have read the stage. After a tile's last slice a commit arms the accumulator's
//     "full" mbarrier; before reusing an accumulator it waits for the epilogue warps' "drained" arrivals.
//   * warps 2 to 5: the epilogue. Each reads its 32 rows of the accumulator (tcgen05.ld, 32 columns at a
//     time), applies the epilogue and stores: bfloat16, float32, float32 accumulate (residual stream), or the gated
//     activation silu(gate) * up when W holds the gate rows followed by the up rows (sleuth/forge/model/mlp.py:37-40);
//     the block then multiplies X by 128 gate rows and the 128 matching up rows in one N = 256 instruction.
// Rows, columns and K beyond the matrices are zero-filled by TMA and masked at the store, so every M, N and every K
// that is a multiple of 8 is taken. (The reference calls a library here: nn.Linear, sleuth/forge/model/attention.py:106-108.)
// A lane of an epilogue warp holds a row of the tile, so epilogues move 32 bytes a lane where alignment allows (half as
// many accesses of the load/store unit, which sets their length). With many rows (4,096 and more) two blocks of a
// cluster share tiles of 256 rows through cta_group::2: see the template parameter PAIR below.
//
// Every wait is bounded: a thread that waits longer than a few seconds' worth of polls records where in
// `status` and leaves its loop; the block then still frees its tensor memory and returns. TMA loads never use
// cluster multicast.
#include "tcgen05.cuh"

namespace slb {

constexpr int kTcBM = 128;
constexpr int kTcBK = 64;             // bf16 elements per slice: 128 bytes, one swizzle row
// TMA stages: as many as fit in 192 KB (at most 8). What is in flight per SM bounds the operand stream (latency x
// bandwidth), so narrow tiles, whose stages are small, get more of them.
__host__ __device__ constexpr int tc_stages(int bn) {
  const int n = (192 * 1024) / ((kTcBM + bn) * kTcBK * 2);
  return n > 8 ? 8 : n;
}
constexpr int kTcThreads = 192;       // producer warp, MMA warp, four epilogue warps

enum TcMode : int { kTcBf16 = 0, kTcF32 = 1, kTcAddF32 = 2, kTcSwiglu = 3, kTcQkv = 4 };

struct TcArgs {
  void* C;
  int M, N, K, ldc, mode;
  int up_row0;          // kTcSwiglu: first up row in W (= number of gate rows)
  int* status;          // 0 = fine; else a code saying which wait gave up
};

// kTcQkv: what follows the fused q/k/v projection, done on the accumulator rows (float32) before anything is
// rounded: bias, per-head RMSNorm of q and k, rotation of the whole head, and the store of q into [tokens, H, hd]
// and of k and v into the token's cache page (sleuth/forge/model/attention.py:121-130, rotation
// sleuth/forge/model/rope.py:41-55). A tile covers whole heads: BN is a multiple of head_dim.
struct TcQkv {
  const float* bias;        // [(H + 2K) * hd] or null
  const float* q_gain;      // [hd] or null (no QK-norm)
  const float* k_gain;
  const float* cos_table;   // [positions, hd / 2] or null (no rotation)
  const float* sin_table;
  __nv_bfloat16* q_out;     // [tokens, H, hd]
  __nv_bfloat16* k_pool;    // [pages, K, 64, hd]; null when the projection holds only q heads
  __nv_bfloat16* v_pool;
  const int* tok_seq;       // [tokens]
  const int* tok_pos;       // [tokens]
  const int* block_table;   // [seqs, table_stride]
  int table_stride, heads, kv_heads, head_dim;
  float eps;
};

// 32-byte accesses of one thread (addresses aligned to 32 bytes).
__device__ __forceinline__ void ld_global_256(const float* p, float (&v)[8]) {
  asm volatile("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p));
}
// (memory that this kernel also writes: not through the read-only path)
__device__ __forceinline__ void ld_global_256_rw(const float* p, float (&v)[8]) {
  asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_global_256(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

// One head of one row: `taddr` is this thread's lane at the head's first accumulator column. Two passes over the
// accumulator keep the registers few: the first sums the squares, the second takes the channels in the pairs that
// rotate together (c, c + HD / 2), 32 pairs at a time.
template <int HD>
__device__ __forceinline__ void qkv_head_epilogue(const TcQkv& q, uint32_t taddr, int row, int M, int head) {
  const bool live = row < M && head < q.heads + 2 * q.kv_heads;
  const bool is_q = head < q.heads, is_k = !is_q && head < q.heads + q.kv_heads;
  const float* gain = (is_q || is_k) ? (is_q ? q.q_gain : q.k_gain) : nullptr;
  const float* bias = q.bias ? q.bias + (size_t)head * HD : nullptr;
  float inv = 1.0f;
  if (gain) {          // uniform over the warp: every lane is in the same head
    float ss = 0.0f;
#pragma unroll
    for (int c0 = 0; c0 < HD; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(taddr + c0, r);
      if (live) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 t = bias ? *reinterpret_cast<const float4*>(bias + c0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
          const float x0 = __uint_as_float(r[j]) + t.x, x1 = __uint_as_float(r[j + 1]) + t.y;
          const float x2 = __uint_as_float(r[j + 2]) + t.z, x3 = __uint_as_float(r[j + 3]) + t.w;
          ss = fmaf(x0, x0, ss); ss = fmaf(x1, x1, ss); ss = fmaf(x2, x2, ss); ss = fmaf(x3, x3, ss);
        }
      }
    }
    inv = 1.0f / sqrtf(ss / (float)HD + q.eps);
  }
  const int pos = live ? q.tok_pos[row] : 0;
  __nv_bfloat16* dst = nullptr;
  if (live) {
    if (is_q) {
      dst = q.q_out + ((size_t)row * q.heads + head) * HD;
    } else {
      const int kh = is_k ? head - q.heads : head - q.heads - q.kv_heads;
      const int page = q.block_table[(size_t)q.tok_seq[row] * q.table_stride + pos / 64];
      dst = (is_k ? q.k_pool : q.v_pool) + (((size_t)page * q.kv_heads + kh) * 64 + (pos % 64)) * HD;
    }
  }
  const bool rotate = q.cos_table != nullptr && (is_q || is_k);
  constexpr int HALF = HD / 2;
#pragma unroll
  for (int c0 = 0; c0 < HALF; c0 += 32) {
    uint32_t ra[32], rb[32];
    __syncwarp();                 // rows beyond the matrix skipped the arithmetic; the loads need the whole warp
    tmem_ld32(taddr + c0, ra);
    tmem_ld32(taddr + HALF + c0, rb);
    if (!live) continue;
    float x[32], y[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      x[j] = __uint_as_float(ra[j]);
      y[j] = __uint_as_float(rb[j]);
    }
    if (bias) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(bias + c0 + j), u = *reinterpret_cast<const float4*>(bias + HALF + c0 + j);
        x[j] += t.x; x[j + 1] += t.y; x[j + 2] += t.z; x[j + 3] += t.w;
        y[j] += u.x; y[j + 1] += u.y; y[j + 2] += u.z; y[j + 3] += u.w;
      }
    }
    if (gain) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(gain + c0 + j), u = *reinterpret_cast<const float4*>(gain + HALF + c0 + j);
        x[j] = (x[j] * inv) * t.x; x[j + 1] = (x[j + 1] * inv) * t.y; x[j + 2] = (x[j + 2] * inv) * t.z; x[j + 3] = (x[j + 3] * inv) * t.w;
        y[j] = (y[j] * inv) * u.x; y[j + 1] = (y[j + 1] * inv) * u.y; y[j + 2] = (y[j + 2] * inv) * u.z; y[j + 3] = (y[j + 3] * inv) * u.w;
      }
    }
    // A lane holds a row, so each of its loads and stores touches a line of its own: 32 bytes at a time (the widest
    // there is) halves what the load/store unit has to do for the rotation factors and for the results.
    if (rotate) {
      const float* cs = q.cos_table + (size_t)pos * HALF + c0;
      const float* sn = q.sin_table + (size_t)pos * HALF + c0;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        float cc[8], sv[8];
        ld_global_256(cs + j, cc);
        ld_global_256(sn + j, sv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a0 = x[j + e], b0 = y[j + e];
          x[j + e] = a0 * cc[e] + (-b0) * sv[e];
          y[j + e] = b0 * cc[e] + a0 * sv[e];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 16) {
      uint32_t o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        __nv_bfloat162 p = __floats2bfloat162_rn(x[j + 2 * e], x[j + 2 * e + 1]);
        o[e] = *reinterpret_cast<uint32_t*>(&p);
      }
      st_global_256(dst + c0 + j, o);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        __nv_bfloat162 p = __floats2bfloat162_rn(y[j + 2 * e], y[j + 2 * e + 1]);
        o[e] = *reinterpret_cast<uint32_t*>(&p);
      }
      st_global_256(dst + HALF + c0 + j, o);
    }
  }
}

__device__ __forceinline__ float fast_silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Stores 32 consecutive float32 accumulator values of one row according to the mode.
__device__ __forceinline__ void store_row32(const TcArgs& a, int row, int col0, const float (&v)[32]) {
  const bool full = col0 + 32 <= a.N;
  if (a.mode == kTcBf16 || a.mode == kTcSwiglu) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)row * a.ldc + col0;
    if (full && (a.ldc % 16 == 0) && ((uintptr_t)a.C % 32 == 0)) {      // 32 bytes at a time (a lane holds a row)
#pragma unroll
      for (int j = 0; j < 32; j += 16) {
        uint32_t o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          __nv_bfloat162 p = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
          o[e] = *reinterpret_cast<uint32_t*>(&p);
        }
        st_global_256(dst + j, o);
      }
    } else if (full && (a.ldc % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 q;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        q.x = *reinterpret_cast<uint32_t*>(&p0); q.y = *reinterpret_cast<uint32_t*>(&p1);
        q.z = *reinterpret_cast<uint32_t*>(&p2); q.w = *reinterpret_cast<uint32_t*>(&p3);
        *reinterpret_cast<uint4*>(dst + j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < a.N) dst[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* dst = reinterpret_cast<float*>(a.C) + (size_t)row * a.ldc + col0;
    if (full && (a.ldc % 8 == 0) && ((uintptr_t)a.C % 32 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint32_t o[8];
        if (a.mode == kTcAddF32) {
          float old[8];
          ld_global_256_rw(dst + j, old);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(old[e] + v[j + e]);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(v[j + e]);
        }
        st_global_256(dst + j, o);
      }
    } else if (full && (a.ldc % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 q = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (a.mode == kTcAddF32) {
          const float4 o = *reinterpret_cast<const float4*>(dst + j);
          q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
        }
        *reinterpret_cast<float4*>(dst + j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < a.N) dst[j] = (a.mode == kTcAddF32 ? dst[j] : 0.0f) + v[j];
    }
  }
}

// Persistent: a block walks the output tiles blockIdx.x, blockIdx.x + gridDim.x, ... Two accumulators in tensor
// memory alternate, so the epilogue warps drain tile t while the tensor core already works on tile t + 1.
// The q/k/v form has eight epilogue warps, two per quarter of the rows, each taking half of the tile's heads: its
// epilogue is long, and what of it the next tile's products do not hide shows at the end of the kernel.
//
// PAIR: two blocks of a cluster share a tile of 256 rows (cta_group::2). Each loads its own 128 rows of X and half of
// the tile's rows of W (for the gated form: one the gate rows, the other the up rows), the even block issues one
// instruction for both, and each finds its 128 rows of the result in its own tensor memory. A block's shared
// memory then serves half as many bytes per product (what bounds the single block: 12 KB read per 128-cycle
// instruction beside TMA's writes), and a stage holds half as much, so twice as many are in flight. A stage's "full"
// barrier is the even block's and counts both blocks' loads; commits arrive at both blocks' barriers; the odd
// block's epilogue warps hand the accumulator back at the even block's barrier.
template <int BN, bool QKV, bool PAIR>
__global__ void __launch_bounds__(QKV ? kTcThreads + 128 : kTcThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, TcArgs a, TcQkv qa) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  Tracer trace(kTraceGemmTc);      // thread 0 is the producer: past its wait, all loads asked for, exit
  // tiles first (each a multiple of 1024 bytes, as the swizzle wants), barriers after
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int BROWS = PAIR ? BN / 2 : BN;          // rows of W in this block's shared memory
  constexpr int A_BYTES = kTcBM * kTcBK * 2, B_BYTES = BROWS * kTcBK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int S = tc_stages(BROWS);
  constexpr int kRows = PAIR ? 2 * kTcBM : kTcBM;    // rows of a tile
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int n_workers = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x, worker = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * STAGE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8 * S, tfull0 = empty0 + 8 * S, tempty0 = tfull0 + 16;
  const uint32_t tiles = smem_addr(smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gated = a.mode == kTcSwiglu;
  const int cols_per_tile = gated ? BN / 2 : BN;
  const int m_tiles = (a.M + kRows - 1) / kRows, n_tiles = (a.N + cols_per_tile - 1) / cols_per_tile;
  const int total = m_tiles * n_tiles;
  const int k_tiles = (a.K + kTcBK - 1) / kTcBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull0 + 8 * i, 1);
      mbar_init(tempty0 + 8 * i, (QKV ? 8 : 4) * (PAIR ? 2 : 1));        // one arrival per epilogue warp (of both blocks)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {     // one warp allocates both accumulators: 2 * BN columns of tensor memory
    __syncwarp();
    if constexpr (PAIR) {      // the same warp of each block of the pair
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(2 * BN) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(2 * BN) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (PAIR) cluster_sync_all();      // both blocks' barriers and tensor memory are there
  else __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  pdl_launch_dependents();
  pdl_wait();          // X is the previous kernel's output
  trace.mark(1);

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      int it = 0;
      bool ok = true;
      for (int tile = worker; tile < total && ok; tile += n_workers) {
        const int m0 = (tile % m_tiles) * kRows + (int)rank * kTcBM, n0 = (tile / m_tiles) * cols_per_tile;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S;
          if (it >= S && !mbar_wait(empty0 + 8 * s, ((it / S) - 1) & 1)) {
            atomicExch(a.status, 1);
            ok = false;
            break;
          }
          const uint32_t sa = tiles + s * STAGE, sb = sa + A_BYTES;
          if constexpr (PAIR) {
            // the even block's barrier counts the bytes of both; this block's half of W's rows: the gate rows or the
            // up rows of the gated form, the first or the second half of the tile's columns otherwise
            const uint32_t full = cluster_map(full0 + 8 * s, 0);
            if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE);
            const int w_row = gated ? (rank ? a.up_row0 + n0 : n0) : n0 + (int)rank * BROWS;
            tma_load_2d_pair(sa, &map_x, kt * kTcBK, m0, full);
            tma_load_2d_pair(sb, &map_w, kt * kTcBK, w_row, full);
          } else {
            mbar_expect_tx(full0 + 8 * s, STAGE);
            tma_load_2d(sa, &map_x, kt * kTcBK, m0, full0 + 8 * s);
            tma_load_2d(sb, &map_w, kt * kTcBK, n0, full0 + 8 * s);
            if (gated) tma_load_2d(sb + B_BYTES / 2, &map_w, kt * kTcBK, a.up_row0 + n0, full0 + 8 * s);
            else if (BN == 256) tma_load_2d(sb + B_BYTES / 2, &map_w, kt * kTcBK, n0 + 128, full0 + 8 * s);
          }
        }
      }
      trace.mark(2);
    }
  } else if (warp == 1 && rank == 0) {
    // ---- MMA issuer: the whole warp walks the loop (its counters and descriptors then live in uniform registers),
    // one lane issues the products and the commits; of a pair, the even block's ----
    constexpr uint32_t idesc = instr_desc(kRows, BN);
    constexpr uint32_t kAll = 0xffffffffu;
    int it = 0, t = 0;
    bool ok = true;
    bool next_ready = false;
    for (int tile = worker; tile < total && ok; tile += n_workers, ++t) {
      const int buf = t & 1;
      if (t >= 2 && !__all_sync(kAll, mbar_wait(tempty0 + 8 * buf, ((t / 2) - 1) & 1))) {   // the epilogue has drained this accumulator
        if (lane == 0) atomicExch(a.status, 4);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t acc = tmem + (uint32_t)(buf * BN);
      for (int kt = 0; kt < k_tiles; ++kt, ++it) {
        const int s = it % S;
        if (!next_ready && !__all_sync(kAll, mbar_wait(full0 + 8 * s, (it / S) & 1))) {
          if (lane == 0) atomicExch(a.status, 2);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // A look at the next stage's barrier goes out before this stage's products: its answer (a couple of
        // hundred cycles away) is back by the time they are issued, so a loaded stage costs no wait of its own.
        const int sn = (it + 1) % S;
        const uint32_t probe = mbar_test(full0 + 8 * sn, ((it + 1) / S) & 1);
        const uint32_t sa = tiles + s * STAGE, sb = sa + A_BYTES;
        const uint64_t da = smem_desc(sa), db = smem_desc(sb);
        if (lane == 0) {
#pragma unroll
          for (int k4 = 0; k4 < kTcBK / 16; ++k4) {  // 16 elements = 32 bytes further along K inside the swizzle row
            if constexpr (PAIR) mma_bf16_ss_pair(acc, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
            else mma_bf16_ss(acc, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
          }
          if constexpr (PAIR) mma_commit_pair(empty0 + 8 * s);      // both blocks' stages
          else mma_commit(empty0 + 8 * s);           // fires when these MMAs have read the stage
        }
        next_ready = __all_sync(kAll, probe != 0);
      }
      if (ok && lane == 0) {                                    // fires when the whole tile has been accumulated
        if constexpr (PAIR) mma_commit_pair(tfull0 + 8 * buf);
        else mma_commit(tfull0 + 8 * buf);
      }
      __syncwarp();
    }
  } else if (warp >= 2) {
    // ---- epilogue: warps 2..5, tensor-memory lanes 32 * (warp % 4) .. + 31 ----
    const int quad = warp & 3;
    const uint32_t tempty_at = PAIR ? cluster_map(tempty0, 0) : tempty0;      // the issuing block's barriers
    int t = 0;
    for (int tile = worker; tile < total; tile += n_workers, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % m_tiles) * kRows + (int)rank * kTcBM, n0 = (tile / m_tiles) * cols_per_tile;
      const int row = m0 + quad * 32 + lane;
      // Adding into the stream: the old values of this thread's row are fetched while the products still run, so
      // that the epilogue (which nothing hides when a block has a single tile) does not wait for them.
      constexpr bool kPreload = !QKV && BN <= 128;
      float old[kPreload ? BN : 1];
      // (the whole warp or none of it: the tensor-memory loads are collective; a warp with rows beyond the matrix
      // takes the general path)
      const bool preloaded = kPreload && __all_sync(0xffffffffu, a.mode == kTcAddF32 && row < a.M && n0 + BN <= a.N &&
                                                                    (a.ldc % 8 == 0) && ((uintptr_t)a.C % 32 == 0));
      if constexpr (kPreload) {
        if (preloaded) {
          const float* src = reinterpret_cast<const float*>(a.C) + (size_t)row * a.ldc + n0;
#pragma unroll
          for (int j = 0; j < BN; j += 8) ld_global_256_rw(src + j, *reinterpret_cast<float(*)[8]>(&old[j]));
        }
      }
      bool ready = true;
      if (lane == 0) ready = mbar_wait(tfull0 + 8 * buf, (t / 2) & 1);
      ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
      if (!ready) {
        if (lane == 0) atomicExch(a.status, 3);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
      if constexpr (kPreload) {
        if (preloaded) {
          float* dst = reinterpret_cast<float*>(a.C) + (size_t)row * a.ldc + n0;
#pragma unroll
          for (int c = 0; c < BN; c += 32) {
            uint32_t r[32];
            tmem_ld32(lane_base + c, r);
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __float_as_uint(old[c + j + e] + __uint_as_float(r[j + e]));
              st_global_256(dst + c + j, o);
            }
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(tempty_at + 8 * buf);
            else mbar_arrive(tempty0 + 8 * buf);
          }
          continue;
        }
      }
      if constexpr (QKV) {
        const int c_lo = ((warp - 2) >> 2) * (BN / 2);          // this warp group's half of the tile's columns
        if (qa.head_dim == 128) {
          for (int c = c_lo; c < c_lo + BN / 2; c += 128) qkv_head_epilogue<128>(qa, lane_base + c, row, a.M, (n0 + c) / 128);
        } else {
          for (int c = c_lo; c < c_lo + BN / 2; c += 64) qkv_head_epilogue<64>(qa, lane_base + c, row, a.M, (n0 + c) / 64);
        }
      } else
      for (int c = 0; c < cols_per_tile; c += 32) {
        uint32_t r[32];
        float v[32];
        tmem_ld32(lane_base + c, r);
        if (gated) {
          uint32_t u[32];
          tmem_ld32(lane_base + BN / 2 + c, u);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fast_silu(__uint_as_float(r[j])) * __uint_as_float(u[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        }
        if (row < a.M && n0 + c < a.N) store_row32(a, row, n0 + c, v);
      }
      // this warp has read its part of the accumulator: let the tensor core have the buffer back
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(tempty_at + 8 * buf);
        else mbar_arrive(tempty0 + 8 * buf);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if constexpr (PAIR) {
    cluster_sync_all();        // neither block frees tensor memory, or leaves, while the other may still be signalled
    if (warp == 2)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  } else {
    __syncthreads();
    if (warp == 2)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
  }
}

// What every tensor-memory kernel here does when one of its waits runs out, as a kernel of its own, so that the
// path can be exercised without anything going wrong: the block takes tensor memory, one thread waits `polls` times
// on a barrier that nothing will ever complete, records `code` in the status word, and the block gives its tensor
// memory back and returns. Nothing faults and nothing hangs; the host then finds the code.
__global__ void __launch_bounds__(64) tc_wait_probe_kernel(int* status, uint32_t polls, int code) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_slot)), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  if (threadIdx.x == 0 && !mbar_wait(smem_addr(&bar), 0, polls)) atomicExch(status, code);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32) : "memory");
}

// ------------------------------------------------------------------------------------ host side ----
// A [rows, K] bfloat16 row-major matrix seen through boxes of box_rows x 64 elements, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(2, "gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)kTcBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(2, "gemm_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

template <int BN, bool QKV = false, bool PAIR = false>
static int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, const TcArgs& a, cudaStream_t s, const TcQkv& qa = TcQkv{}) {
  constexpr int kBRows = PAIR ? BN / 2 : BN;
  constexpr int kStages = tc_stages(kBRows);
  const int smem = kStages * (kTcBM * kTcBK * 2 + kBRows * kTcBK * 2) + (2 * kStages + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, QKV, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(2, "gemm_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int cols_per_tile = a.mode == kTcSwiglu ? BN / 2 : BN;
  const int rows_per_tile = PAIR ? 2 * kTcBM : kTcBM;
  const long long total = (long long)((a.N + cols_per_tile - 1) / cols_per_tile) * ((a.M + rows_per_tile - 1) / rows_per_tile);
  const int sms = sm_count();
  const dim3 block(QKV ? kTcThreads + 128 : kTcThreads);
  if (PAIR) {
    const long long pairs = sms / 2;
    dim3 grid((unsigned)(2 * (total < pairs ? total : pairs)));
    launch_clusters(pdl_mode() != 0, 2, gemm_tc_kernel<BN, QKV, PAIR>, grid, block, (size_t)smem, s, mx, mw, a, qa);
  } else {
    dim3 grid((unsigned)(total < sms ? total : sms));
    launch_prefetching(gemm_tc_kernel<BN, QKV, PAIR>, grid, block, (size_t)smem, s, mx, mw, a, qa);
  }
  return check_launch("gemm_tc");
}

// Whether two blocks share tiles of 256 rows. SLEUTH_B200_GEMM_PAIR=0/1 decides for every product of at least 256
// rows; otherwise pairs take the products of many rows, where they were measured faster (Qwen3-0.6B shapes, one
// B200: level at 2,048 rows, 3 to 12 % faster from 4,096 on, slower below 2,048). The q/k/v form, whose epilogue
// weighs more than its products, gained nothing below 16,384 rows and stays with single blocks.
static bool pair_pays(int M) {
  static int forced = -2;
  if (forced == -2) {
    const char* e = getenv("SLEUTH_B200_GEMM_PAIR");
    forced = e ? (e[0] == '0' ? 0 : 1) : -1;
  }
  if (M < 256) return false;
  return forced >= 0 ? forced != 0 : M >= 4096;
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(gemm_tc)

// Runs the give-up path of the tensor-memory kernels on purpose, harmlessly (see tc_wait_probe_kernel): after it,
// `status` holds `code`. polls: how often the one waiting thread looks at its barrier (1 to 1,000,000).
extern "C" int slb_tc_wait_probe(int* status, int polls, int code, void* stream) {
  SLB_REQUIRE(status != nullptr && polls >= 1 && polls <= 1000000 && code != 0, "tc_wait_probe: status=%p polls=%d code=%d",
              (void*)status, polls, code);
  launch(tc_wait_probe_kernel, dim3(1), dim3(64), 0, (cudaStream_t)stream, status, (uint32_t)polls, code);
  return check_launch("tc_wait_probe");
}

extern "C" int slb_gemm_tc_supported(int M, int N, int K) { return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0; }

// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 gated activation (W holds N gate rows then N up
// rows; C is [M, N] bfloat16). `status` is a device int that the caller zeroed; the kernel writes a non-zero code
// there if one of its bounded waits gave up (the result is then invalid and the caller must say so).
extern "C" int slb_gemm_tc(const void* X, const void* W, void* C, int M, int N, int K, int ldc, int mode, int* status,
                           void* stream) {
  SLB_REQUIRE(slb_gemm_tc_supported(M, N, K), "gemm_tc: M=%d N=%d K=%d is not taken (K must be a multiple of 8)", M, N, K);
  SLB_REQUIRE(mode >= 0 && mode <= 3 && ldc >= N && status != nullptr, "gemm_tc: mode=%d ldc=%d N=%d", mode, ldc, N);
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)C % 16 == 0),
              "gemm_tc: X, W and C must be 16-byte aligned");
  const bool gated = mode == kTcSwiglu;
  // Tile width: the narrowest tile with which all tiles still run at once (one per SM). Measured with 1,024 columns:
  // within one round a narrower tile is a little faster (more SMs stream operands), while a second round costs
  // nearly twice (768 rows: 17 us with 96 tiles of 64 columns, 28 us with 192 of 32). When even the widest tile
  // needs several rounds, the widest is the most efficient.
  const bool pair = pair_pays(M);
  const long long m_tiles = pair ? (M + 255) / 256 : (M + 127) / 128;
  const int sms = sm_count(), workers = pair ? sms / 2 : sms;
  int bn = 256;
  for (int cand = pair ? 128 : (gated ? 64 : 32); cand <= 256; cand <<= 1) {
    const int cols = gated ? cand / 2 : cand;
    if (m_tiles * ((N + cols - 1) / cols) <= workers) { bn = cand; break; }
  }
  CUtensorMap mx, mw;
  int rc = make_map(&mx, X, M, K, kTcBM);
  if (rc) return rc;
  // a block of a pair loads half of the tile's rows of W in one box; a single block loads boxes of at most 128 rows
  rc = make_map(&mw, W, gated ? 2ll * N : N, K, gated || pair ? bn / 2 : (bn < 128 ? bn : 128));
  if (rc) return rc;
  TcArgs a;
  a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc; a.mode = mode; a.up_row0 = N; a.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  if (pair) return bn == 256 ? launch_tc<256, false, true>(mx, mw, a, s) : launch_tc<128, false, true>(mx, mw, a, s);
  switch (bn) {
    case 256: return launch_tc<256>(mx, mw, a, s);
    case 128: return launch_tc<128>(mx, mw, a, s);
    case 64: return launch_tc<64>(mx, mw, a, s);
    default: return launch_tc<32>(mx, mw, a, s);
  }
}

// The fused q/k/v projection of a step with many tokens: X [M, K] times W [(H + 2 * kv_heads) * head_dim, K]^T, and on
// the float32 accumulators bias, per-head RMSNorm of q and k (gains given), rotation of the whole head (tables
// [positions, head_dim / 2] given) and the stores: q into q_out [M, H, head_dim], k and v into the cache page of each
// token (block_table[tok_seq, tok_pos / 64], row tok_pos % 64). kv_heads == 0: the projection holds only q heads.
extern "C" int slb_gemm_tc_qkv(const void* X, const void* W, int M, int K, int heads, int kv_heads, int head_dim,
                               const float* bias, const float* q_gain, const float* k_gain, const float* cos_table,
                               const float* sin_table, float eps, void* q_out, void* k_pool, void* v_pool,
                               const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride,
                               int* status, void* stream) {
  SLB_REQUIRE(head_dim == 64 || head_dim == 128, "gemm_tc_qkv: head size 64 or 128, got %d", head_dim);
  SLB_REQUIRE(heads > 0 && kv_heads >= 0, "gemm_tc_qkv: heads=%d kv_heads=%d", heads, kv_heads);
  const int N = (heads + 2 * kv_heads) * head_dim;
  SLB_REQUIRE(slb_gemm_tc_supported(M, N, K), "gemm_tc_qkv: M=%d N=%d K=%d is not taken (K must be a multiple of 8)", M, N, K);
  SLB_REQUIRE((q_gain == nullptr) == (k_gain == nullptr) || kv_heads == 0, "gemm_tc_qkv: q and k gains go together");
  SLB_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "gemm_tc_qkv: cos and sin tables go together");
  SLB_REQUIRE(q_out != nullptr && tok_pos != nullptr && status != nullptr, "gemm_tc_qkv: q_out, tok_pos and status are needed");
  SLB_REQUIRE(kv_heads == 0 || (k_pool && v_pool && tok_seq && block_table && table_stride > 0),
              "gemm_tc_qkv: the cache pools and the block table are needed to store keys and values");
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)bias % 16 == 0) &&
              ((uintptr_t)q_gain % 16 == 0) && ((uintptr_t)k_gain % 16 == 0), "gemm_tc_qkv: every tensor must be 16-byte aligned");
  SLB_REQUIRE(((uintptr_t)q_out % 32 == 0) && ((uintptr_t)k_pool % 32 == 0) && ((uintptr_t)v_pool % 32 == 0) &&
              ((uintptr_t)cos_table % 32 == 0) && ((uintptr_t)sin_table % 32 == 0),
              "gemm_tc_qkv: q_out, the pools and the rotation tables must be 32-byte aligned (they are read and written 32 bytes at a time)");
  CUtensorMap mx, mw;
  int rc = make_map(&mx, X, M, K, kTcBM);
  if (rc) return rc;
  rc = make_map(&mw, W, N, K, 128);
  if (rc) return rc;
  TcArgs a;
  a.C = nullptr; a.M = M; a.N = N; a.K = K; a.ldc = N; a.mode = kTcQkv; a.up_row0 = N; a.status = status;
  TcQkv qa;
  qa.bias = bias; qa.q_gain = q_gain; qa.k_gain = k_gain; qa.cos_table = cos_table; qa.sin_table = sin_table;
  qa.q_out = (__nv_bfloat16*)q_out; qa.k_pool = (__nv_bfloat16*)k_pool; qa.v_pool = (__nv_bfloat16*)v_pool;
  qa.tok_seq = tok_seq; qa.tok_pos = tok_pos; qa.block_table = block_table; qa.table_stride = table_stride;
  qa.heads = heads; qa.kv_heads = kv_heads; qa.head_dim = head_dim; qa.eps = eps;
  cudaStream_t s = (cudaStream_t)stream;
  return launch_tc<256, true>(mx, mw, a, s, qa);
}
