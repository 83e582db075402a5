// Position encoding of q and k, weightless L2 norm of q and k, and the write of k and v into
// the paged cache, in one pass over a step's projected rows.
//
// Rotation: adjacent pairs (2j, 2j+1) turn by angle position * inv_freq[j]
// (llama4/llama4_jax/model.py:712-728); the angle, sine and cosine are 32-bit.  The norm follows the
// rotation (model.py:915-917) and divides by sqrt(mean(v^2) + eps) (model.py:885-888 with gamma None).
// Layers without position encoding pass inv_freq = null and l2norm = 0: their rows are copied.
//
// Cache layout of one layer: pages[page][0 = K, 1 = V][kv head][slot in page][dh].
#include "common.cuh"

template <typename T>
__global__ void rope_kv_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ pages,
                                     const int* __restrict__ block_table, int bt_stride,
                                     const int* __restrict__ req_of_token, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq, int l2norm, float eps, int Hq, int Hkv,
                                     int dh, int page_size, int num_pages, int store_kv, int* status) {
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int pos = positions[n];
  const int heads = Hq + 2 * Hkv;
  const int half = dh >> 1;
  const T* row = qkv + (size_t)n * heads * dh;

  T* kdst = nullptr;
  T* vdst = nullptr;
  if (store_kv) {
    const int r = req_of_token[n];
    const int page = block_table[(size_t)r * bt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_PAGE);
    } else {
      T* base = pages + (size_t)page * 2 * Hkv * page_size * dh;
      kdst = base + (size_t)(pos % page_size) * dh;
      vdst = base + (size_t)Hkv * page_size * dh + (size_t)(pos % page_size) * dh;
    }
  }

  for (int h = warp; h < heads; h += nwarp) {
    const T* src = row + (size_t)h * dh;
    if (h >= Hq + Hkv) {  // value head: copy
      if (vdst) {
        T* dst = vdst + (size_t)(h - Hq - Hkv) * page_size * dh;
        for (int d = lane; d < dh; d += 32) dst[d] = src[d];
      }
      continue;
    }
    T* dst = h < Hq ? q_out + ((size_t)n * Hq + h) * dh : (kdst ? kdst + (size_t)(h - Hq) * page_size * dh : nullptr);
    // pass 1: rotate, accumulate the sum of squares
    float ss = 0.f;
    for (int j = lane; j < half; j += 32) {
      float a = to_f32<T>(src[2 * j]), b = to_f32<T>(src[2 * j + 1]);
      if (inv_freq) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      ss += a * a + b * b;
    }
    float inv = 1.f;
    if (l2norm) {
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / (float)dh + eps);
    }
    if (!dst) continue;
    // pass 2: recompute the rotation (cheaper than keeping dh values live for any dh) and write
    for (int j = lane; j < half; j += 32) {
      float a = to_f32<T>(src[2 * j]), b = to_f32<T>(src[2 * j + 1]);
      if (inv_freq) {
        float s, c;
        sincosf((float)pos * inv_freq[j], &s, &c);
        float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      dst[2 * j] = from_f32<T>(a * inv);
      dst[2 * j + 1] = from_f32<T>(b * inv);
    }
  }
}

JLX_API int jlx_rope_kv_store(const void* qkv, void* q_out, void* pages, int dtype, const int* block_table,
                              int bt_stride, const int* req_of_token, const int* positions, const float* inv_freq,
                              int l2norm, float eps, int N, int Hq, int Hkv, int dh, int page_size, int num_pages,
                              int store_kv, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && Hq > 0 && Hkv >= 0 && dh > 0, "rope_kv_store: bad sizes N=%d Hq=%d Hkv=%d dh=%d", N, Hq, Hkv, dh);
  JLX_REQUIRE(dh % 2 == 0, "rope_kv_store: head size %d must be even (rotary pairs)", dh);
  JLX_REQUIRE(!store_kv || (page_size > 0 && num_pages > 0 && bt_stride > 0), "rope_kv_store: bad cache sizes");
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T,
                     (rope_kv_store_kernel<T><<<N, 128, 0, stream>>>(
                         (const T*)qkv, (T*)q_out, (T*)pages, block_table, bt_stride, req_of_token, positions, inv_freq,
                         l2norm, eps, Hq, Hkv, dh, page_size, num_pages, store_kv, status)));
  JLX_LAUNCH_CHECK("rope_kv_store");
  return 0;
}

// Plain write of already-encoded k and v rows into pages (for position encodings that are not fused).
// k, v: [N, Hkv, dh]
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ pages,
                                const int* __restrict__ block_table, int bt_stride,
                                const int* __restrict__ req_of_token, const int* __restrict__ positions, int Hkv,
                                int dh, int page_size, int num_pages, int* status) {
  const int n = blockIdx.x;
  const int pos = positions[n];
  const int page = block_table[(size_t)req_of_token[n] * bt_stride + pos / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_PAGE);
    return;
  }
  T* base = pages + (size_t)page * 2 * Hkv * page_size * dh;
  for (int i = threadIdx.x; i < Hkv * dh; i += blockDim.x) {
    const int h = i / dh, d = i % dh;
    const size_t o = ((size_t)h * page_size + pos % page_size) * dh + d;
    base[o] = k[(size_t)n * Hkv * dh + i];
    base[(size_t)Hkv * page_size * dh + o] = v[(size_t)n * Hkv * dh + i];
  }
}

JLX_API int jlx_kv_store(const void* k, const void* v, void* pages, int dtype, const int* block_table, int bt_stride,
                         const int* req_of_token, const int* positions, int N, int Hkv, int dh, int page_size,
                         int num_pages, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && Hkv > 0 && dh > 0 && page_size > 0 && num_pages > 0, "kv_store: bad sizes");
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(dtype, T,
                     (kv_store_kernel<T><<<N, 128, 0, stream>>>((const T*)k, (const T*)v, (T*)pages, block_table,
                                                                bt_stride, req_of_token, positions, Hkv, dh, page_size,
                                                                num_pages, status)));
  JLX_LAUNCH_CHECK("kv_store");
  return 0;
}
