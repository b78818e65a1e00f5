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
constexpr int tc_stages(int bn) {
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
    if (rotate) {
      const float* cs = q.cos_table + (size_t)pos * HALF + c0;
      const float* sn = q.sin_table + (size_t)pos * HALF + c0;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 co = *reinterpret_cast<const float4*>(cs + j), si = *reinterpret_cast<const float4*>(sn + j);
        const float cc[4] = {co.x, co.y, co.z, co.w}, sv[4] = {si.x, si.y, si.z, si.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a0 = x[j + e], b0 = y[j + e];
          x[j + e] = a0 * cc[e] + (-b0) * sv[e];
          y[j + e] = b0 * cc[e] + a0 * sv[e];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 o;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(x[j], x[j + 1]), p1 = __floats2bfloat162_rn(x[j + 2], x[j + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(x[j + 4], x[j + 5]), p3 = __floats2bfloat162_rn(x[j + 6], x[j + 7]);
      o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
      o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(dst + c0 + j) = o;
      p0 = __floats2bfloat162_rn(y[j], y[j + 1]); p1 = __floats2bfloat162_rn(y[j + 2], y[j + 3]);
      p2 = __floats2bfloat162_rn(y[j + 4], y[j + 5]); p3 = __floats2bfloat162_rn(y[j + 6], y[j + 7]);
      o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
      o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(dst + HALF + c0 + j) = o;
    }
  }
}

__device__ __forceinline__ float fast_silu(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Stores 32 consecutive float32 accumulator values of one row according to the mode.
__device__ __forceinline__ void store_row32(const TcArgs& a, int row, int col0, const float (&v)[32]) {
  const bool full = col0 + 32 <= a.N;
  if (a.mode == kTcBf16 || a.mode == kTcSwiglu) {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.C) + (size_t)row * a.ldc + col0;
    if (full && (a.ldc % 8 == 0)) {
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
    if (full && (a.ldc % 4 == 0)) {
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
template <int BN, bool QKV>
__global__ void __launch_bounds__(QKV ? kTcThreads + 128 : kTcThreads)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, TcArgs a, TcQkv qa) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // tiles first (each a multiple of 1024 bytes, as the swizzle wants), barriers after
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_BYTES = kTcBM * kTcBK * 2, B_BYTES = BN * kTcBK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int S = tc_stages(BN);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * STAGE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8 * S, tfull0 = empty0 + 8 * S, tempty0 = tfull0 + 16;
  const uint32_t tiles = smem_addr(smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gated = a.mode == kTcSwiglu;
  const int cols_per_tile = gated ? BN / 2 : BN;
  const int m_tiles = (a.M + kTcBM - 1) / kTcBM, n_tiles = (a.N + cols_per_tile - 1) / cols_per_tile;
  const int total = m_tiles * n_tiles;
  const int k_tiles = (a.K + kTcBK - 1) / kTcBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull0 + 8 * i, 1);
      mbar_init(tempty0 + 8 * i, QKV ? 8 : 4);        // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {     // one warp allocates both accumulators: 2 * BN columns of tensor memory
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  pdl_launch_dependents();
  pdl_wait();          // X is the previous kernel's output

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer ----
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * kTcBM, n0 = (tile / m_tiles) * cols_per_tile;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S;
          if (it >= S && !mbar_wait(empty0 + 8 * s, ((it / S) - 1) & 1)) {
            atomicExch(a.status, 1);
            ok = false;
            break;
          }
          const uint32_t sa = tiles + s * STAGE, sb = sa + A_BYTES;
          mbar_expect_tx(full0 + 8 * s, STAGE);
          tma_load_2d(sa, &map_x, kt * kTcBK, m0, full0 + 8 * s);
          tma_load_2d(sb, &map_w, kt * kTcBK, n0, full0 + 8 * s);
          if (gated) tma_load_2d(sb + B_BYTES / 2, &map_w, kt * kTcBK, a.up_row0 + n0, full0 + 8 * s);
          else if (BN == 256) tma_load_2d(sb + B_BYTES / 2, &map_w, kt * kTcBK, n0 + 128, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp walks the loop (its counters and descriptors then live in uniform registers),
    // one lane issues the products and the commits ----
    constexpr uint32_t idesc = instr_desc(kTcBM, BN);
    constexpr uint32_t kAll = 0xffffffffu;
    int it = 0, t = 0;
    bool ok = true;
    bool next_ready = false;
    for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++t) {
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
          for (int k4 = 0; k4 < kTcBK / 16; ++k4)    // 16 elements = 32 bytes further along K inside the swizzle row
            mma_bf16_ss(acc, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
          mma_commit(empty0 + 8 * s);                // fires when these MMAs have read the stage
        }
        next_ready = __all_sync(kAll, probe != 0);
      }
      if (ok && lane == 0) mma_commit(tfull0 + 8 * buf);        // fires when the whole tile has been accumulated
      __syncwarp();
    }
  } else {
    // ---- epilogue: warps 2..5, tensor-memory lanes 32 * (warp % 4) .. + 31 ----
    const int quad = warp & 3;
    int t = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      const int m0 = (tile % m_tiles) * kTcBM, n0 = (tile / m_tiles) * cols_per_tile;
      const int row = m0 + quad * 32 + lane;
      // Adding into the stream: the old values of this thread's row are fetched while the products still run, so
      // that the epilogue (which nothing hides when a block has a single tile) does not wait for them.
      constexpr bool kPreload = !QKV && BN <= 128;
      float old[kPreload ? BN : 1];
      // (the whole warp or none of it: the tensor-memory loads are collective; a warp with rows beyond the matrix
      // takes the general path)
      const bool preloaded = kPreload && __all_sync(0xffffffffu, a.mode == kTcAddF32 && row < a.M && n0 + BN <= a.N &&
                                                                    (a.ldc % 4 == 0));
      if constexpr (kPreload) {
        if (preloaded) {
          const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.C) + (size_t)row * a.ldc + n0);
#pragma unroll
          for (int j = 0; j < BN / 4; ++j) {
            const float4 o = src[j];
            old[4 * j] = o.x; old[4 * j + 1] = o.y; old[4 * j + 2] = o.z; old[4 * j + 3] = o.w;
          }
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
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dst + c + j) =
                  make_float4(old[c + j] + __uint_as_float(r[j]), old[c + j + 1] + __uint_as_float(r[j + 1]),
                              old[c + j + 2] + __uint_as_float(r[j + 2]), old[c + j + 3] + __uint_as_float(r[j + 3]));
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
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
      if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
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

template <int BN, bool QKV = false>
static int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, const TcArgs& a, cudaStream_t s, const TcQkv& qa = TcQkv{}) {
  constexpr int kStages = tc_stages(BN);
  const int smem = kStages * (kTcBM * kTcBK * 2 + BN * kTcBK * 2) + (2 * kStages + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, QKV>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(2, "gemm_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int cols_per_tile = a.mode == kTcSwiglu ? BN / 2 : BN;
  const long long total = (long long)((a.N + cols_per_tile - 1) / cols_per_tile) * ((a.M + kTcBM - 1) / kTcBM);
  const int sms = sm_count();
  dim3 grid((unsigned)(total < sms ? total : sms));
  launch_prefetching(gemm_tc_kernel<BN, QKV>, grid, dim3(QKV ? kTcThreads + 128 : kTcThreads), (size_t)smem, s, mx, mw, a, qa);
  return check_launch("gemm_tc");
}

}  // namespace slb

using namespace slb;

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
  const long long m_tiles = (M + 127) / 128;
  const int sms = sm_count();
  int bn = 256;
  for (int cand = gated ? 64 : 32; cand <= 256; cand <<= 1) {
    const int cols = gated ? cand / 2 : cand;
    if (m_tiles * ((N + cols - 1) / cols) <= sms) { bn = cand; break; }
  }
  CUtensorMap mx, mw;
  int rc = make_map(&mx, X, M, K, kTcBM);
  if (rc) return rc;
  rc = make_map(&mw, W, gated ? 2ll * N : N, K, gated ? bn / 2 : (bn < 128 ? bn : 128));
  if (rc) return rc;
  TcArgs a;
  a.C = C; a.M = M; a.N = N; a.K = K; a.ldc = ldc; a.mode = mode; a.up_row0 = N; a.status = status;
  cudaStream_t s = (cudaStream_t)stream;
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
  SLB_REQUIRE(((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
              ((uintptr_t)k_pool % 16 == 0) && ((uintptr_t)v_pool % 16 == 0) && ((uintptr_t)bias % 16 == 0) &&
              ((uintptr_t)q_gain % 16 == 0) && ((uintptr_t)k_gain % 16 == 0) && ((uintptr_t)cos_table % 16 == 0) &&
              ((uintptr_t)sin_table % 16 == 0), "gemm_tc_qkv: every tensor must be 16-byte aligned");
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
