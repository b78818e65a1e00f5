// A whole run of decoder layers for a step in which every sequence brings one token, as ONE persistent kernel.
//
// Launched one at a time, the six kernels of a layer spend most of a small-batch step on their boundaries: each
// waits for the one in front, then starts its weight stream from nothing. Here one block per SM stays resident for
// all layers (a cooperative launch), and the two things a step consists of are taken apart:
//   * the stream. Every byte the step reads in bulk (weight matrices, key and value pages) depends on nothing the
//     step computes, so one producer warp per block walks the block's share of it for ALL layers ahead of time and
//     asks TMA for it, chunk by chunk, into a ring of shared-memory slots: weight rows by cp.async.bulk, cache
//     pages by cp.async.bulk.tensor (128-byte swizzle, straight from the pool). It is held up by nothing but free
//     slots, so memory keeps streaming across the phases and layers.
//   * the chain. Eight consumer warps per block do the arithmetic of each phase from the slots as they fill
//     (mma.sync m16n8k16: up to 16 token rows by 8 output features, the eight warps splitting a chunk's inner
//     dimension; attention as in attention_flash.cu, each warp taking 8 of a page's 64 keys), and the blocks meet
//     at a grid-wide barrier where a phase needs all of the one before: q/k/v product | attention | o-proj |
//     gate/up | down, five barriers a layer. Only the few token rows cross a barrier (through L2).
// Formulas are those of the separate kernels: RMSNorm sleuth/forge/model/norm.py:50; q/k/v, per-head QK-norm,
// rotation, cache append, causal GQA softmax sleuth/forge/model/attention.py:101-206 and rope.py:41-55; SwiGLU
// sleuth/forge/model/mlp.py:37-41; residual sums sleuth/forge/model/transformer.py:78-99. Softmax, norms, rotation
// and the residual stream are float32; sums over the inner dimension are added in a fixed order.
//
// Work split. A product's output features go in tiles of 8 to the blocks in turn, the turn carried on from phase
// to phase so that the blocks' shares of the stream even out. Attention flattens the pages of all (sequence, kv
// head) units into one list and gives every block an equal run of it; a run that ends inside a unit leaves a
// partial result (max, sum, weighted values) in scratch memory, and the block that finishes a unit last (a ticket)
// merges its parts in order. The new token's key and value are worked out by the block that holds the unit's last
// page, stored to the cache, and patched into that block's copy of the page.
//
// Every wait is a bounded poll (mbarriers, the grid barrier): one that runs out records a code in `status`, raises
// an abort word that the other blocks see at their next barrier, and the block drains its copies in flight and
// returns. No TMA load uses cluster multicast.
//
// Where it stands. The kernel is correct (it is tested against the plain implementation like the separate kernels)
// and it is NOT the default: on a B200 with the Qwen3-0.6B shapes a layer takes 39 us at batch 1 and 61 us at batch 8
// against 25 and 33 us launch by launch. A launch may be given a trace buffer (DlArgs::trace), which says where the
// time goes: the stream is never the limit (a phase waits 0.2-0.5 us for its data, attention at batch 8 3.4 us); a
// grid barrier costs 2.0-2.5 us, five times a layer, as much as the kernel boundaries it replaces; and between the
// barriers eight warps per SM walk through each phase as one chain of dependent instructions (0.2 instructions a
// cycle and scheduler; the separate kernels keep 12 to 24 independent warps on an SM). The engine runs it when
// SLEUTH_B200_DECODE=fused.
#include <math.h>

#include "mma_sync.cuh"
#include "tcgen05.cuh"

namespace slb {

constexpr int kDlConsumerWarps = 8;
constexpr int kDlConsumers = kDlConsumerWarps * 32;
constexpr int kDlThreads = kDlConsumers + 32;        // + the producer warp
constexpr int kDlKC = 1024;                          // inner-dimension elements of a weight chunk (8 rows of them)
constexpr int kDlRowStride = kDlKC * 2 + 64;         // bytes between the 8 rows of a chunk in its slot: no bank conflicts
constexpr int kDlSlot = 17 * 1024;                   // bytes of a ring slot (a chunk, or one key or value page of a kv head)
constexpr int kDlMaxSlots = 12;
constexpr int kDlMaxUnits = 256;                     // (sequence, kv head) pairs
constexpr int kDlMaxPlans = 4;                       // distinct (window, kv heads) among the layers
constexpr int kDlMaxGroup = 8;                       // query heads per kv head
constexpr int kDlMaxAcc = 8;                         // output tiles (gate and up counted apart) a block multiplies before it adds up the warps
constexpr int kDlMaxCombos = 4;                      // distinct (page plan, cache group) among the layers
constexpr int kDlMaxRun = 192;                       // pages of a block's run whose places are looked up ahead of time
constexpr uint32_t kDlBarrierPolls = 4000000u;

// What is fixed per layer (an array of these lives in device memory).
struct DlLayer {
  const __nv_bfloat16* w_qkv;    // [(H + 2K) * hd, d]
  const __nv_bfloat16* w_o;      // [d, H * hd]
  const __nv_bfloat16* w_gu;     // [2 * inter, d]: gate rows, then up rows
  const __nv_bfloat16* w_down;   // [d, inter]
  const float* norm1;            // [d]
  const float* norm2;            // [d]
  const float* bias;             // [(H + 2K) * hd] or null
  const float* q_gain;           // [hd] or null
  const float* k_gain;           // [hd] or null
  const float* cos_table;        // [positions, hd / 2] or null: the whole head rotates, or nothing does
  const float* sin_table;
  __nv_bfloat16* k_pool;         // [pages, K, 64, hd]: where the new token's key goes
  __nv_bfloat16* v_pool;
  long long k_row0;              // first row of k_pool in its group's tensor map ([rows, hd]); v likewise
  long long v_row0;
  float eps1, eps2, qk_eps, scale_log2;
  int heads, kv_heads, inter, window;
  int group;                     // which block table and tensor map
  int plan;                      // which page plan (window, kv heads)
  int combo;                     // which (plan, group) pair: the producer keeps a list of page places for each
  int pad1;
};

// What a launch brings.
struct DlArgs {
  const DlLayer* layers;
  float* x;                      // [B, d] the residual stream, updated in place
  __nv_bfloat16* qkv;            // [B, max (H + 2K) * hd] scratch: the raw projection of the new tokens
  __nv_bfloat16* y;              // [B, max H * hd] scratch: attention output
  __nv_bfloat16* act;            // [B, max inter] scratch: gated activation
  float* parts;                  // [(blocks + units), kDlMaxGroup * hd + 2 * kDlMaxGroup] partial attention results
  int* tickets;                  // [kDlMaxUnits] zero between launches
  unsigned int* barrier;         // [0] arrivals, [1] abort word; zeroed before the launch
  int* status;                   // 0, or the code of a wait that gave up
  const int* past;               // [B] position of each sequence's new token
  unsigned long long* trace;     // null, or [blocks][layers][24]: nanosecond stamps and waiting cycles: where a step's time goes (diagnostic)
  const int* tables[2];          // block table of each cache group [B, table_stride]
  int table_stride[2];
  int plan_window[kDlMaxPlans], plan_kv_heads[kDlMaxPlans];
  int combo_plan[kDlMaxCombos], combo_group[kDlMaxCombos];
  int n_plans, n_combos, n_layers, B, d, n_slots, stage_bytes, pad;
};

struct DlCtx {
  unsigned char* ring;           // n_slots slots
  unsigned char* stage;          // the A operand of a product (token rows, bfloat16), or the merge area of attention
  float* red;                    // [kDlMaxAcc][8 warps][B][9] partial sums of the tiles of a pass
  unsigned char* sq;             // [16][hd] query rows, swizzled
  float* ss;                     // [16][8] partial sums of squares of the rows being normalised
  const int* pre;                // [plans][kDlMaxUnits + 1] first page of each unit in the flattened list
  const int* past;               // [B] the sequences' positions, in shared memory
  int norm_parts;                // pieces each row's sum of squares came in
  int* flag;                     // [0] a ticket, or whether a grid barrier was passed (consumers), [1] block-wide abort
  uint32_t full0, empty0;        // shared-memory addresses of the slots' barriers
  unsigned int fill;             // slots consumed (or produced) so far
  unsigned int epoch;            // grid barriers passed
  long long waited;              // clock cycles spent waiting for slots to fill (diagnostic, read by traced launches)
  int rot;                       // whose turn the next product's first tile is
  int cta, nblocks, n_slots;
};

// A stamp of the global nanosecond timer at a phase boundary, for the launches that ask for a trace.
__device__ __forceinline__ void dl_stamp(const DlArgs& a, int layer, int i) {
  if (a.trace != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    a.trace[((size_t)blockIdx.x * a.n_layers + layer) * 24 + i] = t;
  }
}
// ... and the cycles the phase that just ended spent waiting for its slots
__device__ __forceinline__ void dl_stamp_wait(const DlArgs& a, DlCtx& c, int layer, int i) {
  if (a.trace != nullptr && threadIdx.x == 0) a.trace[((size_t)blockIdx.x * a.n_layers + layer) * 24 + i] = (unsigned long long)c.waited;
  c.waited = 0;
}

__device__ __forceinline__ void dl_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kDlConsumers) : "memory"); }

__device__ __forceinline__ void dl_fail(const DlArgs& a, DlCtx& c, int code) {
  atomicCAS(a.status, 0, code);
  atomicExch(a.barrier + 1, 1u);
  atomicExch(c.flag + 1, 1);
}

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// ------------------------------------------------------------------------------------ consumers: the ring ----
__device__ __forceinline__ bool slot_wait(const DlArgs& a, DlCtx& c, unsigned int fill) {
  const unsigned int s = fill % c.n_slots;
  if (a.trace != nullptr) {
    const long long t0 = clock64();
    const bool ok = mbar_wait(c.full0 + 8 * s, (fill / c.n_slots) & 1);
    c.waited += clock64() - t0;
    if (ok) return true;
  } else if (mbar_wait(c.full0 + 8 * s, (fill / c.n_slots) & 1)) return true;
  dl_fail(a, c, 41);
  return false;
}
__device__ __forceinline__ void slot_release(DlCtx& c, unsigned int fill) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(c.empty0 + 8 * (fill % c.n_slots));
}

// All blocks meet. Returns false when the wait ran out or another block gave up. The consumers' barrier in front
// orders every thread's stores before thread 0's arrival, which releases them at device scope; the poll acquires the
// other blocks' stores, and the barrier behind hands them on to the block's threads.
__device__ bool grid_barrier(const DlArgs& a, DlCtx& c) {
  dl_bar();
  if (threadIdx.x == 0) {
    int ok = 1;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.barrier) : "memory");
    const unsigned int target = (c.epoch + 1) * (unsigned int)c.nblocks;
    uint32_t polls = 0;
    for (;;) {
      unsigned int seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.barrier) : "memory");
      if (seen >= target) break;
      if ((++polls & 63u) == 0) {
        unsigned int gone;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(gone) : "l"(a.barrier + 1) : "memory");
        if (gone || polls > kDlBarrierPolls) {
          if (!gone) dl_fail(a, c, 40);
          ok = 0;
          break;
        }
      }
    }
    c.flag[0] = ok;
  }
  dl_bar();
  ++c.epoch;
  // (thread 0 writes flag[0] again only behind a later barrier of the consumers, which every thread reaches after this read)
  return c.flag[0] != 0 && c.flag[1] == 0;
}

// ------------------------------------------------------------------------------------ staging the token rows ----
__device__ __forceinline__ int stage_stride(int kdim) { return ((kdim * 2 + 127) & ~127) + 64; }

// The rows of the float32 stream on their way into a product that follows an RMSNorm
// (y = (x / sqrt(mean(x^2) + eps)) * gain): stage[r] = bfloat16(x[r] * gain), and the pieces of each row's sum of
// squares go to `ss`; the factor 1 / rms, one number per row, multiplies the product's float32 sums instead of its
// inputs (`row_scale`), so the rows are read once and nothing waits for the sum. All loads of a lane go out together.
__device__ void stage_scaled(const DlArgs& a, DlCtx& c, const float* gain) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int d = a.d, B = a.B, AS = stage_stride(d);
  // a row is cut into `parts` pieces, one per warp, when there are fewer rows than warps
  int parts = 1;
  while (parts * 2 * B <= kDlConsumerWarps && (d / (parts * 2)) % 128 == 0) parts *= 2;
  c.norm_parts = parts;
  const int seg = d / parts, n4 = seg / 4;
  for (int r0 = 0; r0 < B; r0 += kDlConsumerWarps / parts) {
    const int r = r0 + warp / parts, part = warp % parts;
    if (r < B) {
      const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)r * d + part * seg);
      const float4* gn = reinterpret_cast<const float4*>(gain + part * seg);
      uint2* dst = reinterpret_cast<uint2*>(c.stage + (size_t)r * AS + (size_t)part * seg * 2);
      float ssq = 0.0f;
      for (int i0 = 0; i0 < n4; i0 += 8 * 32) {
        float4 v[8], g4[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = i0 + j * 32 + lane;
          v[j] = i < n4 ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          g4[j] = i < n4 ? gn[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int i = i0 + j * 32 + lane;
          ssq += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
          if (i < n4) dst[i] = make_uint2(pack_bf16(v[j].x * g4[j].x, v[j].y * g4[j].y), pack_bf16(v[j].z * g4[j].z, v[j].w * g4[j].w));
        }
      }
      ssq = warp_sum(ssq);
      if (lane == 0) c.ss[(r & 15) * 8 + part] = ssq;
    }
  }
  dl_bar();
}

// 1 / rms of row r, from the pieces stage_scaled left (added in a fixed order)
__device__ __forceinline__ float row_scale(const DlArgs& a, const DlCtx& c, int r, float eps) {
  float tot = 0.0f;
  for (int p = 0; p < c.norm_parts; ++p) tot += c.ss[(r & 15) * 8 + p];
  return 1.0f / sqrtf(tot / (float)a.d + eps);
}

// stage[r] = src[r] (bfloat16 rows of kdim values that other blocks wrote before the last barrier).
__device__ void stage_copy(const DlArgs& a, DlCtx& c, const __nv_bfloat16* src, int kdim) {
  const int AS = stage_stride(kdim), per_row = kdim / 8;
  const uint32_t dst = smem_u32(c.stage);
  for (int i = threadIdx.x; i < a.B * per_row; i += kDlConsumers) {
    const int r = i / per_row, ch = i % per_row;
    cp_async16(dst + r * AS + ch * 16, src + (size_t)r * kdim + ch * 8);
  }
  cp_async_commit();
  cp_async_wait<0>();
  dl_bar();
}

// ------------------------------------------------------------------------------------ a product phase ----
enum DlMode : int { kDlStoreBf16 = 0, kDlAddF32 = 1, kDlSwiglu = 2 };

__device__ __forceinline__ void mma_16816_regs(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// out[r, n] (+)= scale_r * sum_k stage[r, k] * W[n, k] for this block's tiles of 8 features (scale_r = 1 / rms of row r
// when the rows came through stage_scaled: eps > 0). SUBS = 2: W holds N gate rows and, `N` rows further, N up rows;
// the output is silu(gate) * up. A block multiplies up to kDlMaxAcc tiles (a pass) before its warps' partial sums are
// added, in warp order, through shared memory: one exchange per pass instead of one per tile. A warp keeps two
// accumulators per tile, which halves the chain of dependent instructions.
template <int SUBS>
__device__ bool gemm_phase(const DlArgs& a, DlCtx& c, int N, int kdim, int mode, void* out, int ldo, float eps) {
  constexpr int MAXT = kDlMaxAcc / SUBS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int B = a.B, AS = stage_stride(kdim);
  const int tiles = (N + 7) / 8, chunks = (kdim + kDlKC - 1) / kDlKC;
  const int first = (c.cta - c.rot + c.nblocks) % c.nblocks;
  const int mine = first < tiles ? (tiles - first + c.nblocks - 1) / c.nblocks : 0;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const unsigned char* xa = c.stage + (size_t)g * AS + t * 16;
  const unsigned char* xb = c.stage + (size_t)(g + 8) * AS + t * 16;
  const bool has_a = g < B, has_b = g + 8 < B;
  // thread (row er, feature ec of a tile) adds up and stores that output of every tile; 1 / rms of its row once
  const int er = threadIdx.x >> 3, ec = threadIdx.x & 7;
  const bool stores = threadIdx.x < 128 && er < B;
  const float scale = (stores && eps > 0.0f) ? row_scale(a, c, er, eps) : 1.0f;
  for (int t0 = 0; t0 < mine; t0 += MAXT) {
    const int nt = min(MAXT, mine - t0);
    // Tile after tile (a plain loop: the code stays small enough for the instruction cache): the products of a tile,
    // then this warp's partial sums of it into shared memory, rows that exist only. No warp waits for another here.
#pragma unroll 1
    for (int ti = 0; ti < nt; ++ti) {
      float acc[SUBS][2][4];
#pragma unroll
      for (int sb = 0; sb < SUBS; ++sb)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[sb][0][e] = acc[sb][1][e] = 0.0f;
#pragma unroll
      for (int sb = 0; sb < SUBS; ++sb) {
#pragma unroll 1
        for (int ch = 0; ch < chunks; ++ch) {
          const unsigned int fill = c.fill++;
          if (!slot_wait(a, c, fill)) return false;
          const int kc = min(kDlKC, kdim - ch * kDlKC);
          const unsigned char* wrow = c.ring + (size_t)(fill % c.n_slots) * kDlSlot + g * kDlRowStride + t * 16;
#pragma unroll 2
          for (int kb = warp; kb < kc / 32; kb += kDlConsumerWarps) {
            const uint4 w = *reinterpret_cast<const uint4*>(wrow + kb * 64);
            const size_t ko = ((size_t)ch * kDlKC + kb * 32) * 2;
            const uint4 x0 = has_a ? *reinterpret_cast<const uint4*>(xa + ko) : zero;
            const uint4 x1 = has_b ? *reinterpret_cast<const uint4*>(xb + ko) : zero;
            mma_16816_regs(acc[sb][0], x0.x, x1.x, x0.y, x1.y, w.x, w.y);
            mma_16816_regs(acc[sb][1], x0.z, x1.z, x0.w, x1.w, w.z, w.w);
          }
          slot_release(c, fill);
        }
      }
#pragma unroll
      for (int sb = 0; sb < SUBS; ++sb) {
        float* rw = c.red + ((size_t)(ti * SUBS + sb) * kDlConsumerWarps + warp) * (B * 9);
        if (has_a) {
          rw[g * 9 + 2 * t] = acc[sb][0][0] + acc[sb][1][0];
          rw[g * 9 + 2 * t + 1] = acc[sb][0][1] + acc[sb][1][1];
        }
        if (has_b) {
          rw[(g + 8) * 9 + 2 * t] = acc[sb][0][2] + acc[sb][1][2];
          rw[(g + 8) * 9 + 2 * t + 1] = acc[sb][0][3] + acc[sb][1][3];
        }
      }
    }
    dl_bar();
    if (stores) {
#pragma unroll 1
      for (int ti = 0; ti < nt; ++ti) {
        const int feat = (first + (t0 + ti) * c.nblocks) * 8 + ec;
        if (feat >= N) continue;
        const float* rr = c.red + (size_t)(ti * SUBS) * kDlConsumerWarps * (B * 9) + er * 9 + ec;
        float v = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < kDlConsumerWarps; ++w8) v += rr[(size_t)w8 * (B * 9)];
        v *= scale;
        if (SUBS == 2) {
          float u = 0.0f;
#pragma unroll
          for (int w8 = 0; w8 < kDlConsumerWarps; ++w8) u += rr[(size_t)(kDlConsumerWarps + w8) * (B * 9)];
          u *= scale;
          v = (v / (1.0f + expf(-v))) * u;
        }
        // Adding into the stream: every element of it belongs to exactly one thread of the grid in a phase, so the one
        // addition can be left to the memory system (a reduction that returns nothing) and nothing waits for the old value.
        if (mode == kDlAddF32) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(reinterpret_cast<float*>(out) + (size_t)er * ldo + feat), "f"(v) : "memory");
        else reinterpret_cast<__nv_bfloat16*>(out)[(size_t)er * ldo + feat] = __float2bfloat16_rn(v);
      }
    }
    dl_bar();        // the partial sums are rewritten by the next pass or phase
  }
  c.rot = (c.rot + tiles) % c.nblocks;
  return true;
}

// ------------------------------------------------------------------------------------ attention ----
// byte offset of (row, col) in a page as TMA leaves it in a slot: boxes of 64 channels, rows of 128 bytes, the
// 16-byte chunks of a row XOR-ed with the row number (128-byte swizzle); col is a multiple of 8
__device__ __forceinline__ uint32_t tma_swz(int row, int col) {
  return (uint32_t)((col >> 6) * 8192 + row * 128 + ((((col >> 3) & 7) ^ (row & 7)) << 4));
}
// the same for the query tile [16][HD], which this kernel writes itself
template <int HD> __device__ __forceinline__ uint32_t q_swz(int row, int col) {
  return (uint32_t)(row * (HD * 2) + ((((col >> 3) ^ (row & 7))) << 4));
}

// One row of the raw projection: + bias, RMSNorm over the head (when `gain`), rotation of the whole head (when
// `rotate`), float32 throughout; lane l gets channels l * EPL .. (the arithmetic of csrc/qkv_post.cu).
template <int HD>
__device__ __forceinline__ void dl_post_row(const __nv_bfloat16* src, const float* bias, const float* gain, float eps, bool rotate,
                                            const float (&cs)[HD / 32], const float (&sn)[HD / 32], int lane, float (&v)[HD / 32]) {
  constexpr int EPL = HD / 32;
  const int c0 = lane * EPL;
  float ss = 0.0f;
  if constexpr (EPL == 4) {
    const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(src + c0));
    const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 q = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = p.x; v[1] = p.y; v[2] = q.x; v[3] = q.y;
  } else {
    const unsigned int raw = __ldcg(reinterpret_cast<const unsigned int*>(src + c0));
    const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
    v[0] = p.x; v[1] = p.y;
  }
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    if (bias) v[e] += bias[c0 + e];
    ss = fmaf(v[e], v[e], ss);
  }
  if (gain) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = (v[e] * inv) * gain[c0 + e];
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

template <int HD>
__device__ __forceinline__ void dl_put(unsigned char* at, const float (&v)[HD / 32]) {
  if constexpr (HD == 128) {
    uint2 pk;
    pk.x = pack_bf16(v[0], v[1]);
    pk.y = pack_bf16(v[2], v[3]);
    *reinterpret_cast<uint2*>(at) = pk;
  } else {
    *reinterpret_cast<uint32_t*>(at) = pack_bf16(v[0], v[1]);
  }
}

// the block that holds page q of the flattened list when P pages are cut into `blocks` equal runs
__device__ __forceinline__ int block_of_page(int q, int P, int blocks) { return (int)((((long long)q + 1) * blocks - 1) / P); }

template <int HD>
__device__ bool attention_phase(const DlArgs& a, DlCtx& c, const DlLayer& L) {
  constexpr int EPL = HD / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int Kh = L.kv_heads, G = L.heads / Kh, H = L.heads;
  const int n_units = a.B * Kh, n_qkv = (H + 2 * Kh) * HD;
  const int* pre = c.pre + L.plan * (kDlMaxUnits + 1);
  const int P = pre[n_units];
  // the P pages are cut into equal runs for the first min(blocks, P) blocks: every one of them then has a page, so the
  // blocks that share a unit are consecutive and a unit's parts can be counted from its first and last page
  const int nb = min(c.nblocks, P);
  if (c.cta >= nb) return true;
  const int lo = (int)((long long)c.cta * P / nb), hi = (int)((long long)(c.cta + 1) * P / nb);
  int u = 0;
  {   // the unit that holds page lo: the last u with pre[u] <= lo
    int left = 0, right = n_units - 1;
    while (left < right) {
      const int mid = (left + right + 1) >> 1;
      if (pre[mid] <= lo) left = mid; else right = mid - 1;
    }
    u = left;
  }
  const uint32_t sQ = smem_u32(c.sq);
  float* mo = reinterpret_cast<float*>(c.stage);                 // [8 warps][G][HD]
  float* mm = mo + kDlConsumerWarps * kDlMaxGroup * HD;           // [8][8]
  float* ml = mm + kDlConsumerWarps * kDlMaxGroup;                // [8][8]
  const int part_floats = kDlMaxGroup * HD + 2 * kDlMaxGroup;
  const int* table_base = a.tables[L.group];
  const int stride = a.table_stride[L.group];

  for (int q = lo; q < hi; ++u) {
    const int seg_end = min(hi, pre[u + 1]);
    const int seq = u / Kh, kh = u % Kh;
    const int pos = c.past[seq];
    const int key_lo = L.window > 0 ? max(0, pos - L.window + 1) : 0;
    const int page_lo = key_lo / 64, page_hi = pos / 64;
    const int first_page = page_lo + (q - pre[u]), n_pg = seg_end - q;
    const bool owns_last = seg_end == pre[u + 1];
    const int* table = table_base + (size_t)seq * stride;
    const __nv_bfloat16* raw = a.qkv + (size_t)seq * n_qkv;

    // ---- the unit's query rows (and, where the unit's last page is here, the new token's key and value) ----
    float cos_l[EPL], sin_l[EPL];
    const bool rotate = L.cos_table != nullptr;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      cos_l[e] = rotate ? L.cos_table[(size_t)pos * (HD / 2) + (lane & 15) * EPL + e] : 1.0f;
      sin_l[e] = rotate ? L.sin_table[(size_t)pos * (HD / 2) + (lane & 15) * EPL + e] : 0.0f;
    }
    for (int row = warp; row < 16; row += kDlConsumerWarps) {
      float v[EPL];
      if (row < G) {
        const int head = kh * G + row;
        dl_post_row<HD>(raw + (size_t)head * HD, L.bias ? L.bias + (size_t)head * HD : nullptr, L.q_gain, L.qk_eps, rotate, cos_l, sin_l, lane, v);
      } else {
#pragma unroll
        for (int e = 0; e < EPL; ++e) v[e] = 0.0f;
      }
      dl_put<HD>(c.sq + q_swz<HD>(row, (lane * EPL) & ~7) + ((lane * EPL) & 7) * 2, v);
    }
    float new_kv[EPL];
    const int kv_warp_k = kDlConsumerWarps - 2, kv_warp_v = kDlConsumerWarps - 1;     // the warps with no query row of their own
    if (owns_last && (warp == kv_warp_k || warp == kv_warp_v)) {
      const bool is_k = warp == kv_warp_k;
      const int r = H + (is_k ? 0 : Kh) + kh;
      dl_post_row<HD>(raw + (size_t)r * HD, L.bias ? L.bias + (size_t)r * HD : nullptr, is_k ? L.k_gain : nullptr, L.qk_eps,
                      is_k && rotate, cos_l, sin_l, lane, new_kv);
      __nv_bfloat16* pool = is_k ? L.k_pool : L.v_pool;
      __nv_bfloat16* dst = pool + (((size_t)table[page_hi] * Kh + kh) * 64 + (pos % 64)) * HD + lane * EPL;
      dl_put<HD>(reinterpret_cast<unsigned char*>(dst), new_kv);
    }
    dl_bar();
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int kb = 0; kb < HD / 16; ++kb) ldmatrix_x4(qf[kb], sQ + q_swz<HD>(lane & 15, kb * 16 + ((lane >> 4) << 3)));

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.0f, 0.0f};

    for (int pg = 0; pg < n_pg; ++pg) {
      const int page = first_page + pg;
      const unsigned int fk = c.fill++, fv = c.fill++;
      unsigned char* slot_k = c.ring + (size_t)(fk % c.n_slots) * kDlSlot;
      unsigned char* slot_v = c.ring + (size_t)(fv % c.n_slots) * kDlSlot;
      if (!slot_wait(a, c, fk)) return false;
      if (owns_last && page == page_hi) {
        // the cache's copy of this page has a stale row where the new token goes, and leftovers of another sequence
        // behind it: the new key and value go in, the value rows behind are cleared (0 * inf would poison the sum)
        if (!slot_wait(a, c, fv)) return false;
        const int r = pos % 64;
        if (warp == kv_warp_k) dl_put<HD>(slot_k + tma_swz(r, (lane * EPL) & ~7) + ((lane * EPL) & 7) * 2, new_kv);
        if (warp == kv_warp_v) dl_put<HD>(slot_v + tma_swz(r, (lane * EPL) & ~7) + ((lane * EPL) & 7) * 2, new_kv);
        for (int i = threadIdx.x; i < (63 - r) * (HD / 8); i += kDlConsumers) {
          const int row = r + 1 + i / (HD / 8), ch = i % (HD / 8);
          *reinterpret_cast<uint4*>(slot_v + tma_swz(row, ch * 8)) = make_uint4(0, 0, 0, 0);
        }
        fence_smem_to_async();      // these slots are written by TMA again later
        dl_bar();
      }
      const int key0 = page * 64 + warp * 8;          // this warp's 8 keys of the page
      const bool live = key0 <= pos && key0 + 7 >= key_lo;
      uint32_t pf[2] = {0u, 0u};
      float alpha[2] = {1.0f, 1.0f};
      if (live) {
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t kS = smem_u32(slot_k);
#pragma unroll
        for (int kb2 = 0; kb2 < HD / 32; ++kb2) {
          uint32_t kf[4];
          ldmatrix_x4(kf, kS + tma_swz(warp * 8 + (lane & 7), kb2 * 32 + ((lane >> 3) << 3)));
          mma_bf16(s, qf[2 * kb2], kf[0], kf[1]);
          mma_bf16(s2, qf[2 * kb2 + 1], kf[2], kf[3]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] += s2[e];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + 2 * t4 + (e & 1);
          float v = s[e] * L.scale_log2;
          if (key > pos || key < key_lo) v = -INFINITY;
          s[e] = v;
        }
        float mx[2] = {fmaxf(s[0], s[1]), fmaxf(s[2], s[3])}, m_use[2], sum[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
          mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
          const float m_new = fmaxf(m_r[h], mx[h]);
          m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
          alpha[h] = exp2f(m_r[h] - m_use[h]);
          m_r[h] = m_new;
        }
        const float p0 = exp2f(s[0] - m_use[0]), p1 = exp2f(s[1] - m_use[0]);
        const float p2 = exp2f(s[2] - m_use[1]), p3 = exp2f(s[3] - m_use[1]);
        sum[0] = p0 + p1;
        sum[1] = p2 + p3;
        pf[0] = pack_bf16(p0, p1);
        pf[1] = pack_bf16(p2, p3);
#pragma unroll
        for (int h = 0; h < 2; ++h) l_r[h] = l_r[h] * alpha[h] + sum[h];
      }
      slot_release(c, fk);
      if (!(owns_last && page == page_hi) && !slot_wait(a, c, fv)) return false;
      if (live) {
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
          o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        const uint32_t vS = smem_u32(slot_v);
        const uint32_t pa[4] = {pf[0], pf[1], 0u, 0u};        // the tile's second eight keys do not exist
#pragma unroll
        for (int cb = 0; cb < HD / 32; ++cb) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, vS + tma_swz(warp * 8 + (lane & 7), cb * 32 + ((lane >> 3) << 3)));
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16(o[4 * cb + j], pa, vf[j], 0u);
        }
      }
      slot_release(c, fv);
    }

    // ---- merge the eight warps (each saw other keys), rows of the group only ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 1);
      l_r[h] += __shfl_xor_sync(0xffffffffu, l_r[h], 2);
    }
    if (g < G) {
      if (t4 == 0) { mm[warp * kDlMaxGroup + g] = m_r[0]; ml[warp * kDlMaxGroup + g] = l_r[0]; }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(mo + ((size_t)warp * kDlMaxGroup + g) * HD + i * 8 + 2 * t4) = make_float2(o[i][0], o[i][1]);
    }
    dl_bar();
    const int first_blk = block_of_page(pre[u], P, nb), last_blk = block_of_page(pre[u + 1] - 1, P, nb);
    const int n_parts = last_blk - first_blk + 1;
    float* my_part = a.parts + (size_t)(c.cta + u) * part_floats;
    for (int idx = threadIdx.x; idx < G * HD; idx += kDlConsumers) {
      const int row = idx / HD, dch = idx % HD;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDlConsumerWarps; ++w) m = fmaxf(m, mm[w * kDlMaxGroup + row]);
      const float m_use = m == -INFINITY ? 0.0f : m;
      float l = 0.0f, acc = 0.0f;
#pragma unroll
      for (int w = 0; w < kDlConsumerWarps; ++w) {
        const float f = exp2f(mm[w * kDlMaxGroup + row] - m_use);
        l += ml[w * kDlMaxGroup + row] * f;
        acc += mo[((size_t)w * kDlMaxGroup + row) * HD + dch] * f;
      }
      if (n_parts == 1) {
        a.y[((size_t)seq * H + kh * G + row) * HD + dch] = __float2bfloat16_rn(acc / l);
      } else {
        my_part[row * HD + dch] = acc;
        if (dch == 0) { my_part[kDlMaxGroup * HD + 2 * row] = m; my_part[kDlMaxGroup * HD + 2 * row + 1] = l; }
      }
    }
    if (n_parts > 1) {
      // the part is published, then a ticket taken (one release-acquire operation between two barriers of the
      // consumers); whoever holds the unit's last ticket reads all parts back, in block order
      dl_bar();
      if (threadIdx.x == 0) {
        int got;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(got) : "l"(a.tickets + u) : "memory");
        c.flag[0] = got;
      }
      dl_bar();
      if (c.flag[0] == n_parts - 1) {
        for (int idx = threadIdx.x; idx < G * HD; idx += kDlConsumers) {
          const int row = idx / HD, dch = idx % HD;
          float m = -INFINITY, l = 0.0f, acc = 0.0f;
          for (int j = 0; j < n_parts; ++j) {
            const float* part = a.parts + (size_t)(first_blk + j + u) * part_floats;
            const float pm = __ldcg(part + kDlMaxGroup * HD + 2 * row), pl = __ldcg(part + kDlMaxGroup * HD + 2 * row + 1);
            const float po = __ldcg(part + row * HD + dch);
            const float m_new = fmaxf(m, pm);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float keep = exp2f(m - m_use), f = exp2f(pm - m_use);
            l = l * keep + pl * f;
            acc = acc * keep + po * f;
            m = m_new;
          }
          a.y[((size_t)seq * H + kh * G + row) * HD + dch] = __float2bfloat16_rn(acc / l);
        }
        if (threadIdx.x == 0) a.tickets[u] = 0;
      }
    }
    dl_bar();          // the merge area and the query tile are free again
    q = seg_end;
  }
  return true;
}

// ------------------------------------------------------------------------------------ the producer ----
struct DlProducer {
  uint32_t ring, full0, empty0;
  unsigned int fill;
  int n_slots;
};

// Claims the next slot: waits until the consumers have left it, arms its barrier for `bytes`. 0 = the wait ran out.
__device__ __forceinline__ uint32_t produce_slot(const DlArgs& a, DlCtx& c, DlProducer& p, uint32_t bytes, uint32_t& bar) {
  const unsigned int f = p.fill++, s = f % p.n_slots;
  if (f >= (unsigned int)p.n_slots && !mbar_wait(p.empty0 + 8 * s, ((f / p.n_slots) - 1) & 1)) {
    --p.fill;
    dl_fail(a, c, 42);
    return 0;
  }
  bar = p.full0 + 8 * s;
  mbar_expect_tx(bar, bytes);
  return p.ring + s * kDlSlot;
}

__device__ bool produce_gemm(const DlArgs& a, DlCtx& c, DlProducer& p, const __nv_bfloat16* W, int N, int kdim, int subs) {
  const int tiles = (N + 7) / 8, chunks = (kdim + kDlKC - 1) / kDlKC;
  for (int tile = (c.cta - c.rot + c.nblocks) % c.nblocks; tile < tiles; tile += c.nblocks) {
    const int rows = min(8, N - tile * 8);
    for (int s = 0; s < subs; ++s) {
      const __nv_bfloat16* w0 = W + ((size_t)s * N + (size_t)tile * 8) * kdim;
      for (int ch = 0; ch < chunks; ++ch) {
        const int kc = min(kDlKC, kdim - ch * kDlKC);
        uint32_t bar;
        const uint32_t dst = produce_slot(a, c, p, (uint32_t)(rows * kc * 2), bar);
        if (!dst) return false;
        for (int r = 0; r < rows; ++r)
          bulk_copy(dst + r * kDlRowStride, w0 + (size_t)r * kdim + (size_t)ch * kDlKC, (uint32_t)(kc * 2), bar);
      }
    }
  }
  c.rot = (c.rot + tiles) % c.nblocks;
  return true;
}

// The place of page q of the flattened list of plan `plan` in cache group `group`: (physical page * kv heads + kv head),
// i.e. the page's first row in the pool divided by 64.
__device__ __forceinline__ int page_place(const DlArgs& a, const int* pre, const int* past, int plan, int group, int q, int n_units) {
  const int Kh = a.plan_kv_heads[plan], W = a.plan_window[plan];
  int left = 0, right = n_units - 1;
  while (left < right) {          // the unit that holds page q: the last u with pre[u] <= q
    const int mid = (left + right + 1) >> 1;
    if (pre[mid] <= q) left = mid; else right = mid - 1;
  }
  const int seq = left / Kh, kh = left % Kh, pos = past[seq];
  const int page = (W > 0 ? max(0, pos - W + 1) : 0) / 64 + (q - pre[left]);
  return a.tables[group][(size_t)seq * a.table_stride[group] + page] * Kh + kh;
}

template <int HD>
__device__ bool produce_attention(const DlArgs& a, DlCtx& c, DlProducer& p, const DlLayer& L, const CUtensorMap* map, const int* places) {
  const int n_units = a.B * L.kv_heads;
  const int* pre = c.pre + L.plan * (kDlMaxUnits + 1);
  const int P = pre[n_units];
  const int nb = min(c.nblocks, P);
  if (c.cta >= nb) return true;
  const int lo = (int)((long long)c.cta * P / nb), hi = (int)((long long)(c.cta + 1) * P / nb);
  for (int q = lo; q < hi; ++q) {
    // looked up ahead of time by the whole warp (fill_places); beyond that list, here
    const int place = q - lo < kDlMaxRun ? places[q - lo] : page_place(a, pre, c.past, L.plan, L.group, q, n_units);
    const long long row = (long long)place * 64;
    for (int kv = 0; kv < 2; ++kv) {
      uint32_t bar;
      const uint32_t dst = produce_slot(a, c, p, (uint32_t)(64 * HD * 2), bar);
      if (!dst) return false;
      const int y = (int)((kv ? L.v_row0 : L.k_row0) + row);
#pragma unroll
      for (int h = 0; h < HD / 64; ++h) tma_load_2d(dst + h * 8192, map, h * 64, y, bar);
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------ the kernel ----
template <int HD>
__global__ void __launch_bounds__(kDlThreads, 1)
decode_layers_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1, DlArgs a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bars[2 * kDlMaxSlots];
  __shared__ __align__(16) DlLayer layer_now[2];                  // this layer's description and the next one's
  __shared__ int pre[kDlMaxPlans * (kDlMaxUnits + 1)];
  __shared__ int places[kDlMaxCombos * kDlMaxRun];                // where the pages of this block's runs lie
  __shared__ int past[16];
  __shared__ float ss[16 * 8];
  __shared__ int flag[2];

  DlCtx c;
  c.ring = smem;
  c.stage = smem + (size_t)a.n_slots * kDlSlot;
  c.red = reinterpret_cast<float*>(c.stage + a.stage_bytes);
  c.sq = reinterpret_cast<unsigned char*>(c.red + (size_t)kDlMaxAcc * kDlConsumerWarps * a.B * 9);
  c.ss = ss;
  c.pre = pre;
  c.past = past;
  c.flag = flag;
  c.full0 = smem_addr(bars);
  c.empty0 = c.full0 + 8 * kDlMaxSlots;
  c.fill = 0;
  c.epoch = 0;
  c.rot = 0;
  c.waited = 0;
  c.norm_parts = 1;
  c.cta = blockIdx.x;
  c.nblocks = gridDim.x;
  c.n_slots = a.n_slots;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.n_slots; ++s) {
      mbar_init(c.full0 + 8 * s, 1);
      mbar_init(c.empty0 + 8 * s, kDlConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    flag[0] = 0;
    flag[1] = 0;
  }
  if (threadIdx.x < 16) past[threadIdx.x] = threadIdx.x < a.B ? a.past[threadIdx.x] : 0;
  if (warp == 1) {        // the first layer's description
    const unsigned long long* src = reinterpret_cast<const unsigned long long*>(a.layers);
    for (int i = lane; i < (int)(sizeof(DlLayer) / 8); i += 32) reinterpret_cast<unsigned long long*>(&layer_now[0])[i] = src[i];
  }
  // where each (sequence, kv head) unit's pages begin in the flattened list, per plan
  for (int i = threadIdx.x; i < a.n_plans * (kDlMaxUnits + 1); i += kDlThreads) {
    const int plan = i / (kDlMaxUnits + 1), u = i % (kDlMaxUnits + 1);
    const int Kh = a.plan_kv_heads[plan], W = a.plan_window[plan];
    int first = 0;
    if (u <= a.B * Kh) {
      const int seq = u / Kh, kh = u % Kh;
      for (int s = 0; s <= seq && s < a.B; ++s) {
        const int pos = a.past[s];
        const int n = pos / 64 - (W > 0 ? max(0, pos - W + 1) : 0) / 64 + 1;
        first += s < seq ? n * Kh : n * kh;
      }
    }
    pre[i] = first;
  }
  __syncthreads();

  if (warp == kDlConsumerWarps) {
    // ---- the producer ----
    // All lanes first look up where this block's pages lie, for each (plan, cache group) pair among the layers: the
    // block table is read through two dependent loads per page, which the one lane that issues the copies would
    // otherwise wait for page by page.
    for (int cb = 0; cb < a.n_combos; ++cb) {
      const int plan = a.combo_plan[cb], group = a.combo_group[cb];
      const int n_units = a.B * a.plan_kv_heads[plan];
      const int* pr = pre + plan * (kDlMaxUnits + 1);
      const int P = pr[n_units], nb = min(c.nblocks, P);
      if (c.cta >= nb) continue;
      const int lo = (int)((long long)c.cta * P / nb), hi = (int)((long long)(c.cta + 1) * P / nb);
      for (int q = lo + lane; q < hi && q - lo < kDlMaxRun; q += 32)
        places[cb * kDlMaxRun + q - lo] = page_place(a, pr, past, plan, group, q, n_units);
    }
    __syncwarp();
    if (lane == 0) {
      // one lane walks this block's share of the whole step's stream
      DlProducer p;
      p.ring = smem_addr(c.ring);
      p.full0 = c.full0;
      p.empty0 = c.empty0;
      p.fill = 0;
      p.n_slots = a.n_slots;
      bool ok = true;
      for (int li = 0; li < a.n_layers && ok; ++li) {
        const DlLayer L = a.layers[li];
        const int n_qkv = (L.heads + 2 * L.kv_heads) * HD;
        ok = produce_gemm(a, c, p, L.w_qkv, n_qkv, a.d, 1);
        ok = ok && produce_attention<HD>(a, c, p, L, L.group == 0 ? &map0 : &map1, places + L.combo * kDlMaxRun);
        ok = ok && produce_gemm(a, c, p, L.w_o, a.d, L.heads * HD, 1);
        ok = ok && produce_gemm(a, c, p, L.w_gu, L.inter, a.d, 2);
        ok = ok && produce_gemm(a, c, p, L.w_down, a.d, L.inter, 1);
      }
      // Whatever the consumers do from here on (they may give up a wait): the copies asked for last are waited for
      // here, bounded, so that none is in flight when the block's shared memory goes away. A slot's barrier completes
      // when its bytes have landed, whether or not anybody consumes them.
      const unsigned int issued = p.fill;
      for (unsigned int f = issued > (unsigned int)p.n_slots ? issued - p.n_slots : 0; f < issued; ++f)
        mbar_wait(p.full0 + 8 * (f % p.n_slots), (f / p.n_slots) & 1, 1000000u);
    }
  } else {
    // ---- the consumers ----
    bool ok = true;
    for (int li = 0; li < a.n_layers && ok; ++li) {
      const DlLayer& L = layer_now[li & 1];
      // the next layer's description comes in meanwhile; the barriers of this layer stand between this write and its use
      if (warp == 1 && li + 1 < a.n_layers) {
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(a.layers + li + 1);
        for (int i = lane; i < (int)(sizeof(DlLayer) / 8); i += 32)
          reinterpret_cast<unsigned long long*>(&layer_now[(li + 1) & 1])[i] = src[i];
      }
      const int n_qkv = (L.heads + 2 * L.kv_heads) * HD;
      dl_stamp(a, li, 0);
      stage_scaled(a, c, L.norm1);
      dl_stamp(a, li, 1);
      ok = gemm_phase<1>(a, c, n_qkv, a.d, kDlStoreBf16, a.qkv, n_qkv, L.eps1);
      dl_stamp(a, li, 2);
      dl_stamp_wait(a, c, li, 15);
      ok = ok && grid_barrier(a, c);
      dl_stamp(a, li, 3);
      ok = ok && attention_phase<HD>(a, c, L);
      dl_stamp(a, li, 4);
      dl_stamp_wait(a, c, li, 16);
      ok = ok && grid_barrier(a, c);
      dl_stamp(a, li, 5);
      if (!ok) break;
      stage_copy(a, c, a.y, L.heads * HD);
      dl_stamp(a, li, 6);
      ok = gemm_phase<1>(a, c, a.d, L.heads * HD, kDlAddF32, a.x, a.d, 0.0f);
      dl_stamp(a, li, 7);
      dl_stamp_wait(a, c, li, 17);
      ok = ok && grid_barrier(a, c);
      dl_stamp(a, li, 8);
      if (!ok) break;
      stage_scaled(a, c, L.norm2);
      dl_stamp(a, li, 9);
      ok = gemm_phase<2>(a, c, L.inter, a.d, kDlSwiglu, a.act, L.inter, L.eps2);
      dl_stamp(a, li, 10);
      dl_stamp_wait(a, c, li, 18);
      ok = ok && grid_barrier(a, c);
      dl_stamp(a, li, 11);
      if (!ok) break;
      stage_copy(a, c, a.act, L.inter);
      dl_stamp(a, li, 12);
      ok = gemm_phase<1>(a, c, a.d, L.inter, kDlAddF32, a.x, a.d, 0.0f);
      dl_stamp(a, li, 13);
      dl_stamp_wait(a, c, li, 19);
      ok = ok && grid_barrier(a, c);
      dl_stamp(a, li, 14);
    }
    if (!ok) atomicExch(flag + 1, 1);
  }
  __syncthreads();
}

// ------------------------------------------------------------------------------------ host side ----
struct DlHost {        // what the launcher is handed (mirrored by a ctypes structure in kernels/ops.py)
  DlArgs args;
  const void* pool_base[2];      // each cache group's whole pool tensor, seen as [pool_rows, head_dim] bfloat16
  long long pool_rows[2];
  int head_dim, n_groups;
};

static int encode_pool_map(CUtensorMap* map, const void* base, long long rows, int head_dim) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(2, "decode_layers: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64, 64};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(2, "decode_layers: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

constexpr int kDlFixedSmem = 16 * 128 * 2 + 1024;      // query tile, alignment
static int dl_red_bytes(int rows) { return kDlMaxAcc * kDlConsumerWarps * rows * 9 * 4; }   // the warps' partial sums of a pass

template <int HD>
static int launch_decode_layers(const DlHost& h, const CUtensorMap& m0, const CUtensorMap& m1, int smem, cudaStream_t s) {
  static int configured = 0;
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(2, "decode_layers: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel<HD>, kDlThreads, smem);
  if (e != cudaSuccess || per_sm < 1) return fail(2, "decode_layers: a block does not fit an SM (%s)", cudaGetErrorString(e));
  e = cudaMemsetAsync(h.args.barrier, 0, 2 * sizeof(unsigned int), s);
  if (e != cudaSuccess) return fail(2, "decode_layers: clearing the barrier failed: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count());
  cfg.blockDim = dim3(kDlThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;        // all blocks resident at once: they wait for one another
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_layers_kernel<HD>, m0, m1, h.args);
  if (e != cudaSuccess) note_launch_error(e);
  return check_launch("decode_layers");
}

}  // namespace slb

using namespace slb;

// Shared memory the kernel needs beside its ring, for `rows` token rows whose widest product input has `kmax` values,
// groups of up to 8 query heads and this head size; and how many ring slots then fit.
extern "C" int slb_decode_layers_stage_bytes(int rows, int kmax, int head_dim) {
  const int a_bytes = rows * (((kmax * 2 + 127) & ~127) + 64);
  const int merge = (kDlConsumerWarps * kDlMaxGroup * head_dim + 2 * kDlConsumerWarps * kDlMaxGroup) * 4;
  const int need = a_bytes > merge ? a_bytes : merge;
  return (need + 1023) & ~1023;
}

extern "C" int slb_decode_layers_slots(int stage_bytes, int rows) {
  int dev = 0, most = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&most, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
  const int room = most - 14 * 1024 - kDlFixedSmem - dl_red_bytes(rows) - stage_bytes;      // 14 KB: the kernel's static arrays and a margin
  const int n = room / kDlSlot;
  return n > kDlMaxSlots ? kDlMaxSlots : n;
}

extern "C" int slb_decode_layers(const DlHost* host, void* stream) {
  SLB_REQUIRE(host != nullptr, "decode_layers: no arguments");
  const DlHost& h = *host;
  const DlArgs& a = h.args;
  SLB_REQUIRE(h.head_dim == 64 || h.head_dim == 128, "decode_layers: head size 64 or 128, got %d", h.head_dim);
  SLB_REQUIRE(a.B >= 1 && a.B <= 16, "decode_layers: 1 to 16 sequences, got %d", a.B);
  SLB_REQUIRE(a.d >= 128 && a.d % 128 == 0, "decode_layers: the width must be a multiple of 128, got %d", a.d);
  SLB_REQUIRE(a.n_layers >= 1 && a.layers != nullptr, "decode_layers: no layers");
  SLB_REQUIRE(a.n_plans >= 1 && a.n_plans <= kDlMaxPlans && h.n_groups >= 1 && h.n_groups <= 2 && a.n_combos >= 1 &&
              a.n_combos <= kDlMaxCombos,
              "decode_layers: %d page plans (at most %d), %d cache groups (at most 2), %d pairs of them (at most %d)", a.n_plans,
              kDlMaxPlans, h.n_groups, a.n_combos, kDlMaxCombos);
  for (int cb = 0; cb < a.n_combos; ++cb)
    SLB_REQUIRE(a.combo_plan[cb] >= 0 && a.combo_plan[cb] < a.n_plans && a.combo_group[cb] >= 0 && a.combo_group[cb] < h.n_groups,
                "decode_layers: pair %d names plan %d, group %d", cb, a.combo_plan[cb], a.combo_group[cb]);
  for (int p = 0; p < a.n_plans; ++p)
    SLB_REQUIRE(a.plan_kv_heads[p] >= 1 && a.B * a.plan_kv_heads[p] <= kDlMaxUnits && a.plan_window[p] >= 0,
                "decode_layers: %d sequences x %d kv heads are more than %d units", a.B, a.plan_kv_heads[p], kDlMaxUnits);
  SLB_REQUIRE(a.n_slots >= 4 && a.n_slots <= kDlMaxSlots, "decode_layers: %d ring slots (4 to %d)", a.n_slots, kDlMaxSlots);
  SLB_REQUIRE(a.x && a.qkv && a.y && a.act && a.parts && a.tickets && a.barrier && a.status && a.past && a.tables[0],
              "decode_layers: a buffer is missing");
  for (int g = 0; g < h.n_groups; ++g)
    SLB_REQUIRE(h.pool_base[g] != nullptr && (uintptr_t)h.pool_base[g] % 16 == 0 && h.pool_rows[g] > 0 &&
                h.pool_rows[g] < (1ll << 31) && a.tables[g] != nullptr && a.table_stride[g] > 0,
                "decode_layers: cache group %d: pool or block table missing, or more than 2^31 rows", g);
  CUtensorMap m0, m1;
  int rc = encode_pool_map(&m0, h.pool_base[0], h.pool_rows[0], h.head_dim);
  if (rc) return rc;
  rc = encode_pool_map(&m1, h.pool_base[h.n_groups > 1 ? 1 : 0], h.pool_rows[h.n_groups > 1 ? 1 : 0], h.head_dim);
  if (rc) return rc;
  const int smem = a.n_slots * kDlSlot + a.stage_bytes + dl_red_bytes(a.B) + kDlFixedSmem;
  return h.head_dim == 64 ? launch_decode_layers<64>(h, m0, m1, smem, (cudaStream_t)stream)
                          : launch_decode_layers<128>(h, m0, m1, smem, (cudaStream_t)stream);
}
