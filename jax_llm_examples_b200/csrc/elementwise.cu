// Embedding gather, RMSNorm fused with the residual sum, and SiLU(gate)*up.
//
// The residual stream is 32-bit in every precision mode: the sum x + delta and the norm's mean of
// squares are computed in 32-bit (reference: llama4/llama4_jax/model.py:885-888 computes the mean in
// float32; model.py:1173,1181 are the residual sums).
#include "common.cuh"

// x[n, :] = table[ids[n], :]                                     (model.py:1191)
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ x,
                             int D, int V, int* status) {
  const int n = blockIdx.x;
  int id = ids[n];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_TOKEN);
    id = 0;
  }
  const TW* row = table + (size_t)id * D;
  float* out = x + (size_t)n * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = to_f32<TW>(row[d]);
}

JLX_API int jlx_embed(const int* ids, const void* table, int table_dtype, float* x, int N, int D, int V,
                      int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0 && V > 0, "embed: bad sizes N=%d D=%d V=%d", N, D, V);
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(table_dtype, TW, (embed_kernel<TW><<<N, 256, 0, stream>>>(ids, (const TW*)table, x, D, V, status)));
  JLX_LAUNCH_CHECK("embed");
  return 0;
}

// Row n (source row r = row_index ? row_index[n] : n):
//   s = x[r] + delta[r]            (delta optional; written back to x[r] unless rows are gathered)
//   out[n] = gamma * s / sqrt(mean(s^2) + eps)      (gamma optional: weightless norm)
// `out` in the activation type and/or `out32` in 32-bit (for the router, which wants unrounded input).
template <typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                   const float* __restrict__ gamma, float eps, TO* __restrict__ out,
                                   float* __restrict__ out32, const int* __restrict__ row_index, int D) {
  __shared__ float scratch[33];
  const int n = blockIdx.x;
  const size_t r = row_index ? (size_t)row_index[n] : (size_t)n;
  float* xr = x + r * D;
  const float* dr = delta ? delta + r * D : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = xr[d];
    if (dr) {
      s += dr[d];
      if (!row_index) xr[d] = s;
    }
    ss += s * s;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float s = xr[d];
    if (dr && row_index) s += dr[d];
    float v = (gamma ? gamma[d] * s : s) / rms;
    if (out) out[(size_t)n * D + d] = from_f32<TO>(v);
    if (out32) out32[(size_t)n * D + d] = v;
  }
}

JLX_API int jlx_add_rmsnorm(float* x, const float* delta, const float* gamma, float eps, void* out, int out_dtype,
                            float* out32, const int* row_index, int N, int D, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0, "add_rmsnorm: bad sizes N=%d D=%d", N, D);
  JLX_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
  if (N == 0) return 0;
  const int threads = D >= 1024 ? 256 : 128;
  JLX_DISPATCH_DTYPE(out_dtype, TO,
                     (add_rmsnorm_kernel<TO><<<N, threads, 0, stream>>>(x, delta, gamma, eps, (TO*)out, out32, row_index, D)));
  JLX_LAUNCH_CHECK("add_rmsnorm");
  return 0;
}

// out[i, f] = silu(gu[i, f]) * gu[i, F + f]                       (model.py:1146-1151)
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, const int* __restrict__ n_rows_dev,
                                int rows, int F) {
  const int i = blockIdx.x;
  if (n_rows_dev && i >= *n_rows_dev) return;
  const T* g = gu + (size_t)i * 2 * F;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    float a = to_f32<T>(g[f]), b = to_f32<T>(g[F + f]);
    float s = a / (1.f + expf(-a));
    out[(size_t)i * F + f] = from_f32<T>(s * b);
  }
}

JLX_API int jlx_silu_mul(const void* gu, void* out, int dtype, const int* n_rows_dev, int rows, int F,
                         cudaStream_t stream) {
  JLX_REQUIRE(rows >= 0 && F > 0, "silu_mul: bad sizes rows=%d F=%d", rows, F);
  if (rows == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T, (silu_mul_kernel<T><<<rows, 256, 0, stream>>>((const T*)gu, (T*)out, n_rows_dev, rows, F)));
  JLX_LAUNCH_CHECK("silu_mul");
  return 0;
}

// dst[i] = src[i] converted between element types (activations entering a 32-bit weight's product).
template <typename TS, typename TD>
__global__ void convert_kernel(const TS* __restrict__ src, TD* __restrict__ dst, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}

JLX_API int jlx_convert(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  int blocks = (int)((n + 255) / 256 < 65535 ? (n + 255) / 256 : 65535);
  JLX_DISPATCH_DTYPE(src_dtype, TS, JLX_DISPATCH_DTYPE(dst_dtype, TD,
      (convert_kernel<TS, TD><<<blocks, 256, 0, stream>>>((const TS*)src, (TD*)dst, (size_t)n))));
  JLX_LAUNCH_CHECK("convert");
  return 0;
}
