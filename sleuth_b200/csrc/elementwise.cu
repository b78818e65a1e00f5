// Row-wise kernels between the matrix products: embedding lookup, RMSNorm, residual add, gated activation.
#include "common.cuh"

namespace slb {

// x[t, :] = table[ids[t], :] * scale, into the float32 residual stream.
// (Token rows looked up without scaling unless the model sets one: sleuth/forge/model/transformer.py:345-348.)
// With `map`, row t takes token ids[map[t]]: a decode step can then read the tokens the sampler left on the
// device for the previous batch, whose rows need not be this batch's rows.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ map, const TW* __restrict__ table,
                             float* __restrict__ x, int dim, int vocab, float scale) {
  Tracer trace(kTraceEmbed);
  pdl_enter();
  trace.mark(1);
  const int t = blockIdx.x;
  int tok = ids[map ? map[t] : t];
  tok = min(max(tok, 0), vocab - 1);
  const TW* row = table + (size_t)tok * dim;
  float* out = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

// out[r, :] = (x[row(r), :] * (1 / sqrt(mean(x^2) + eps))) * w, float32 arithmetic, one rounding at the store.
// row(r) = rows[r] when `rows` is given (the final norm runs only on the rows whose logits are wanted).
// (sleuth/forge/model/norm.py:50; the reference's own fused form: sleuth/forge/model/fused_ops.py:41-51.)
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps) {
  pdl_enter();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float v = xr[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>((xr[i] * inv) * w[i]);
}

// The same for widths that are multiples of 4: 16-byte loads, the row kept in registers between the two passes.
template <typename TO, int PER_THREAD>
__global__ void rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int dim, float eps) {
  Tracer trace(kTraceNorm);
  pdl_enter();
  trace.mark(1);
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  const float4* w4 = reinterpret_cast<const float4*>(w);
  float4 v[PER_THREAD], gains[PER_THREAD];      // the gains are asked for with the row, not after the sum
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    gains[i] = c < n4 ? w4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* o = out + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c >= n4) continue;
    const float4 g = gains[i];
    const float a = (v[i].x * inv) * g.x, b = (v[i].y * inv) * g.y, cc = (v[i].z * inv) * g.z, d = (v[i].w * inv) * g.w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(o)[c] = make_float4(a, b, cc, d);
    } else {
      __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(o)[c] = pk;
    }
  }
}

// x += delta (delta in the activation dtype), float32 sum.
template <typename TD>
__global__ void add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) x[i] += to_f32(delta[i]);
}

// act[t, j] = silu(gu[t, j]) * gu[t, inter + j], silu(z) = z / (1 + exp(-z)); float32 arithmetic.
// (sleuth/forge/model/mlp.py:37-40.)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / inter, j = i - t * inter;
    const float g = to_f32(gu[t * 2 * inter + j]);
    const float u = to_f32(gu[t * 2 * inter + inter + j]);
    act[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
  }
}

// bfloat16, inter a multiple of 8: 16 bytes of gate and of up per thread.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, int inter,
                                     size_t total8) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  const int per_row = inter >> 3;
  for (; i < total8; i += step) {
    const size_t t = i / per_row, j = (i - t * per_row) << 3;
    const Bf16x8 g = *reinterpret_cast<const Bf16x8*>(gu + t * 2 * inter + j);
    const Bf16x8 u = *reinterpret_cast<const Bf16x8*>(gu + t * 2 * inter + inter + j);
    float gf[8], uf[8];
    unpack8(g, gf);
    unpack8(u, uf);
    Bf16x8 o;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float a = (gf[2 * e] / (1.0f + expf(-gf[2 * e]))) * uf[2 * e];
      const float b = (gf[2 * e + 1] / (1.0f + expf(-gf[2 * e + 1]))) * uf[2 * e + 1];
      o.v[e] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<Bf16x8*>(act + t * inter + j) = o;
  }
}

static int norm_threads(int dim) {
  int t = 32;
  while (t < 512 && t * 4 < dim) t <<= 1;
  return t;
}

}  // namespace slb

using namespace slb;
SLB_TIMELINE_SETTER(elementwise)

extern "C" int slb_embed(const int* ids, const int* map, const void* table, int table_dtype, float* x, int tokens,
                         int dim, int vocab, float scale, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0, "embed: tokens=%d dim=%d vocab=%d", tokens, dim, vocab);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = dim >= 256 ? 256 : 64;
  if (table_dtype == kF32)
    launch(embed_kernel<float>, dim3(tokens), dim3(threads), 0, s, ids, map, (const float*)table, x, dim, vocab, scale);
  else if (table_dtype == kBF16)
    launch(embed_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, s, ids, map, (const __nv_bfloat16*)table, x, dim, vocab, scale);
  else
    return fail(1, "embed: unknown dtype %d", table_dtype);
  return check_launch("embed");
}

extern "C" int slb_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows,
                           int dim, float eps, void* stream) {
  SLB_REQUIRE(n_rows >= 0 && dim > 0 && eps > 0.0f, "rmsnorm: rows=%d dim=%d eps=%g", n_rows, dim, (double)eps);
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  SLB_REQUIRE(out_dtype == kF32 || out_dtype == kBF16, "rmsnorm: unknown dtype %d", out_dtype);
  if (dim % 4 == 0 && dim <= 8192 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    const int n4 = dim / 4;
    int threads = n4 <= 64 ? 64 : (n4 <= 128 ? 128 : 256);
    // Many rows (prompts), bfloat16 run: half the threads per row, so that twice as many rows are resident and a
    // 2,048-row call runs in one round of blocks instead of two. The float32 run keeps one block shape whatever
    // the row count, so that a row's sum is formed in the same order in every step.
    if (out_dtype == kBF16 && n_rows >= 1024 && threads == 256 && n4 <= 8 * 128) threads = 128;
    const int per = (n4 + threads - 1) / threads;      // at most 8
    #define SLB_NORM(P)                                                                                              \
      if (out_dtype == kF32) launch(rmsnorm_vec_kernel<float, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (float*)out, rows, dim, eps); \
      else launch(rmsnorm_vec_kernel<__nv_bfloat16, P>, dim3(n_rows), dim3(threads), 0, s, x, w, (__nv_bfloat16*)out, rows, dim, eps)
    if (per <= 1) { SLB_NORM(1); } else if (per <= 2) { SLB_NORM(2); } else if (per <= 4) { SLB_NORM(4); } else { SLB_NORM(8); }
    #undef SLB_NORM
    return check_launch("rmsnorm");
  }
  const int threads = norm_threads(dim);
  if (out_dtype == kF32)
    launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, w, (float*)out, rows, dim, eps);
  else
    launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, x, w, (__nv_bfloat16*)out, rows, dim, eps);
  return check_launch("rmsnorm");
}

extern "C" int slb_add(float* x, const void* delta, int delta_dtype, long long n, void* stream) {
  SLB_REQUIRE(n >= 0, "add: n=%lld", n);
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (delta_dtype == kF32)
    launch(add_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, x, (const float*)delta, (size_t)n);
  else if (delta_dtype == kBF16)
    launch(add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, x, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return fail(1, "add: unknown dtype %d", delta_dtype);
  return check_launch("add");
}

extern "C" int slb_swiglu(const void* gu, void* act, int dtype, int tokens, int inter, void* stream) {
  SLB_REQUIRE(tokens >= 0 && inter > 0, "swiglu: tokens=%d inter=%d", tokens, inter);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t total = (size_t)tokens * inter;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > sm_count() * 16) blocks = sm_count() * 16;
  if (dtype == kBF16 && inter % 8 == 0 && ((uintptr_t)gu % 16 == 0) && ((uintptr_t)act % 16 == 0)) {
    const size_t total8 = total / 8;
    size_t b8 = (total8 + threads - 1) / threads;
    if (b8 > sm_count() * 32) b8 = sm_count() * 32;
    launch(swiglu_bf16x8_kernel, dim3((int)b8), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act, inter, total8);
    return check_launch("swiglu");
  }
  if (dtype == kF32)
    launch(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, s, (const float*)gu, (float*)act, inter, total);
  else if (dtype == kBF16)
    launch(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)act,
                                                               inter, total);
  else
    return fail(1, "swiglu: unknown dtype %d", dtype);
  return check_launch("swiglu");
}
