// Row-wise kernels between the matrix products: embedding lookup, RMSNorm, residual add, gated activation.
#include "common.cuh"

namespace slb {

// x[t, :] = table[ids[t], :] * scale, into the float32 residual stream.
// (Token rows looked up without scaling unless the model sets one: sleuth/forge/model/transformer.py:345-348.)
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ x,
                             int dim, float scale) {
  const int t = blockIdx.x;
  const TW* row = table + (size_t)ids[t] * dim;
  float* out = x + (size_t)t * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

// out[r, :] = (x[row(r), :] * (1 / sqrt(mean(x^2) + eps))) * w, float32 arithmetic, one rounding at the store.
// row(r) = rows[r] when `rows` is given (the final norm runs only on the rows whose logits are wanted).
// (sleuth/forge/model/norm.py:50; the reference's own fused form: sleuth/forge/model/fused_ops.py:41-51.)
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps) {
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

// x += delta (delta in the activation dtype), float32 sum.
template <typename TD>
__global__ void add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) x[i] += to_f32(delta[i]);
}

// act[t, j] = silu(gu[t, j]) * gu[t, inter + j], silu(z) = z / (1 + exp(-z)); float32 arithmetic.
// (sleuth/forge/model/mlp.py:37-40.)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ act, int inter, size_t total) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / inter, j = i - t * inter;
    const float g = to_f32(gu[t * 2 * inter + j]);
    const float u = to_f32(gu[t * 2 * inter + inter + j]);
    act[i] = from_f32<T>((g / (1.0f + expf(-g))) * u);
  }
}

static int norm_threads(int dim) {
  int t = 32;
  while (t < 512 && t * 4 < dim) t <<= 1;
  return t;
}

}  // namespace slb

using namespace slb;

extern "C" int slb_embed(const int* ids, const void* table, int table_dtype, float* x, int tokens, int dim,
                         float scale, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0, "embed: tokens=%d dim=%d", tokens, dim);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = dim >= 256 ? 256 : 64;
  if (table_dtype == kF32)
    embed_kernel<float><<<tokens, threads, 0, s>>>(ids, (const float*)table, x, dim, scale);
  else if (table_dtype == kBF16)
    embed_kernel<__nv_bfloat16><<<tokens, threads, 0, s>>>(ids, (const __nv_bfloat16*)table, x, dim, scale);
  else
    return fail(1, "embed: unknown dtype %d", table_dtype);
  return check_launch("embed");
}

extern "C" int slb_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows,
                           int dim, float eps, void* stream) {
  SLB_REQUIRE(n_rows >= 0 && dim > 0 && eps > 0.0f, "rmsnorm: rows=%d dim=%d eps=%g", n_rows, dim, (double)eps);
  if (n_rows == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = norm_threads(dim);
  if (out_dtype == kF32)
    rmsnorm_kernel<float><<<n_rows, threads, 0, s>>>(x, w, (float*)out, rows, dim, eps);
  else if (out_dtype == kBF16)
    rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, s>>>(x, w, (__nv_bfloat16*)out, rows, dim, eps);
  else
    return fail(1, "rmsnorm: unknown dtype %d", out_dtype);
  return check_launch("rmsnorm");
}

extern "C" int slb_add(float* x, const void* delta, int delta_dtype, long long n, void* stream) {
  SLB_REQUIRE(n >= 0, "add: n=%lld", n);
  if (n == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (delta_dtype == kF32)
    add_kernel<float><<<(int)blocks, threads, 0, s>>>(x, (const float*)delta, (size_t)n);
  else if (delta_dtype == kBF16)
    add_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, s>>>(x, (const __nv_bfloat16*)delta, (size_t)n);
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
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == kF32)
    swiglu_kernel<float><<<(int)blocks, threads, 0, s>>>((const float*)gu, (float*)act, inter, total);
  else if (dtype == kBF16)
    swiglu_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)act,
                                                               inter, total);
  else
    return fail(1, "swiglu: unknown dtype %d", dtype);
  return check_launch("swiglu");
}
