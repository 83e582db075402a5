// Paged attention for any head size, head count, group size, page size and query length, in 32-bit
// or bfloat16 storage with 32-bit scores, softmax and accumulation.  It is the attention of the
// 32-bit path and the fallback of the bfloat16 path for sizes that the tensor-core kernels refuse.
//
// One block serves one query token and one KV head (all G query heads of the group share each key
// and value tile).  A query at position p of request r attends keys at positions [start, p] with
//   start = max(chunk  ? floor(p / chunk) * chunk : 0,  window ? p - window + 1 : 0)
// (causal and same-chunk mask of llama4/llama4_jax/model.py:731-742; scale dh^-0.5, model.py:774;
// 32-bit softmax, model.py:789).  Queries of layers with temperature tuning are scaled by
// 1 + attn_scale * ln(1 + floor((p + 1) / floor_scale)).
// The order of the key loop depends only on (start, p): a position's result does not change with
// what else is in the batch or how the prompt was cut into steps.
#include "common.cuh"

#define ATT_TILE 32
#define ATT_MAX_WARPS 8
#define ATT_MAX_D32 16  // head size up to 512

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ pages,
                                         const int* __restrict__ block_table, int bt_stride,
                                         const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                         T* __restrict__ out, int Hq, int Hkv, int dh, int page_size, int num_pages,
                                         float scale, int chunk, int window, float attn_scale, float floor_scale,
                                         int* status) {
  JLX_TL(TL_ATTN_GENERIC);
  extern __shared__ float smem[];
  const int n = blockIdx.x, hk = blockIdx.y;
  const int G = Hq / Hkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int ldk = dh + 1;
  float* qs = smem;                        // [nwarp][dh]
  float* ks = qs + nwarp * dh;             // [ATT_TILE][dh + 1]
  float* vs = ks + ATT_TILE * ldk;         // [ATT_TILE][dh + 1]

  const int p = positions[n];
  const int r = req_of_token[n];
  int start = 0;
  if (chunk > 0) start = (p / chunk) * chunk;
  if (window > 0) start = max(start, p - window + 1);
  float qscale = scale;
  if (attn_scale != 0.f) qscale *= 1.f + attn_scale * log1pf(floorf(((float)p + 1.f) / floor_scale));
  const int nd = (dh + 31) >> 5;
  const size_t page_elems = (size_t)2 * Hkv * page_size * dh;

  for (int g0 = 0; g0 < G; g0 += nwarp) {
    const int g = g0 + warp;
    const bool active = g < G;
    const int h = hk * G + g;
    if (active)
      for (int d = lane; d < dh; d += 32) qs[warp * dh + d] = to_f32<T>(q[((size_t)n * Hq + h) * dh + d]);
    float m = -INFINITY, l = 0.f;
    float acc[ATT_MAX_D32];
#pragma unroll
    for (int i = 0; i < ATT_MAX_D32; ++i) acc[i] = 0.f;

    for (int t0 = start; t0 <= p; t0 += ATT_TILE) {
      __syncthreads();  // previous tile fully consumed; qs visible
      const int cnt = min(ATT_TILE, p - t0 + 1);
      for (int idx = threadIdx.x; idx < cnt * dh; idx += blockDim.x) {
        const int j = idx / dh, d = idx - j * dh;
        const int pos = t0 + j;
        const int page = block_table[(size_t)r * bt_stride + pos / page_size];
        float kv = 0.f, vv = 0.f;
        if (page < 0 || page >= num_pages) {
          atomicOr(status, JLX_STATUS_BAD_PAGE);
        } else {
          const T* base = pages + (size_t)page * page_elems + ((size_t)hk * page_size + pos % page_size) * dh + d;
          kv = to_f32<T>(base[0]);
          vv = to_f32<T>(base[(size_t)Hkv * page_size * dh]);
        }
        ks[j * ldk + d] = kv;
        vs[j * ldk + d] = vv;
      }
      __syncthreads();
      if (active) {
        float s = -INFINITY;
        if (lane < cnt) {
          float dot = 0.f;
          const float* kr = ks + lane * ldk;
          const float* qr = qs + warp * dh;
          for (int d = 0; d < dh; ++d) dot += qr[d] * kr[d];
          s = dot * qscale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);  // m = -inf on the first tile: exp(-inf) = 0
        const float pj = lane < cnt ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int i = 0; i < ATT_MAX_D32; ++i) {
          if (i < nd) {
            const int d = lane + 32 * i;
            float a = acc[i] * corr;
            for (int j = 0; j < cnt; ++j) {
              const float pv = __shfl_sync(0xffffffffu, pj, j);
              if (d < dh) a += pv * vs[j * ldk + d];
            }
            acc[i] = a;
          }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int i = 0; i < ATT_MAX_D32; ++i) {
        const int d = lane + 32 * i;
        if (i < nd && d < dh) out[((size_t)n * Hq + h) * dh + d] = from_f32<T>(acc[i] / l);
      }
    }
    __syncthreads();
  }
}

JLX_API int jlx_attention_generic(const void* q, const void* pages, int dtype, const int* block_table, int bt_stride,
                                  const int* req_of_token, const int* positions, void* out, int N, int Hq, int Hkv,
                                  int dh, int page_size, int num_pages, float scale, int chunk, int window,
                                  float attn_scale, float floor_scale, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && Hq > 0 && Hkv > 0 && dh > 0 && page_size > 0 && num_pages > 0, "attention: bad sizes");
  JLX_REQUIRE(Hq % Hkv == 0, "attention: %d query heads are no multiple of %d KV heads", Hq, Hkv);
  JLX_REQUIRE(dh <= 32 * ATT_MAX_D32, "attention: head size %d is above the supported maximum %d", dh, 32 * ATT_MAX_D32);
  JLX_REQUIRE(attn_scale == 0.f || floor_scale > 0.f, "attention: floor_scale must be positive");
  if (N == 0) return 0;
  const int G = Hq / Hkv;
  const int nwarp = G < ATT_MAX_WARPS ? G : ATT_MAX_WARPS;
  const size_t smem = sizeof(float) * ((size_t)nwarp * dh + 2 * (size_t)ATT_TILE * (dh + 1));
  JLX_REQUIRE(Hkv <= 65535, "attention: too many KV heads (%d)", Hkv);
  JLX_DISPATCH_DTYPE(dtype, T, {
    if (smem > 48 * 1024)
      JLX_CUDA(cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attention_generic_kernel<T><<<dim3(N, Hkv), nwarp * 32, smem, stream>>>(
        (const T*)q, (const T*)pages, block_table, bt_stride, req_of_token, positions, (T*)out, Hq, Hkv, dh, page_size,
        num_pages, scale, chunk, window, attn_scale, floor_scale, status);
  });
  JLX_LAUNCH_CHECK("attention_generic");
  return 0;
}
