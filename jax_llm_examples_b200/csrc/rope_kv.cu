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

#define ROPE_REG_PAIRS 4  // head sizes up to 256 keep a lane's pairs in registers

// A rotary pair (2j, 2j+1) as one access.
template <typename T> __device__ __forceinline__ float2 load_pair(const T* p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 load_pair<bf16>(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T> __device__ __forceinline__ void store_pair(T* p, float a, float b);
template <> __device__ __forceinline__ void store_pair<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <> __device__ __forceinline__ void store_pair<bf16>(bf16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// TI: element type of the projected rows (the activation type, or float32 split-K partials that are
// added first); T: element type of q_out and of the cache.
// HPW: heads per warp.  A block takes 8 * HPW heads of one token (head h0 + 8 i for warp h0's i-th turn).  With many
// tokens a block's fixed chain of dependent loads (position, request, block table) is paid once for more heads,
// and a warp's loads of all its heads are in flight together; with few tokens one head per warp gives the most blocks.
template <typename TI, typename T, int HPW>
__global__ void __launch_bounds__(256)
rope_kv_store_kernel(const TI* __restrict__ qkv, int splits, long long split_stride, T* __restrict__ q_out,
                     T* __restrict__ pages, const int* __restrict__ block_table, int bt_stride,
                     const int* __restrict__ req_of_token, const int* __restrict__ positions,
                     const float* __restrict__ inv_freq, int l2norm, float eps, int Hq, int Hkv, int dh, int page_size,
                     int num_pages, int store_kv, int* status) {
  JLX_TL(TL_ROPE);
  extern __shared__ float sc[];  // [dh / 2][2]: sine and cosine of this token's angles
  pdl_launch_dependents();
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int heads = Hq + 2 * Hkv;
  const int half = dh >> 1;
  const TI* row = qkv + (size_t)n * heads * dh;
  // What does not depend on the kernels before this one in the stream comes first: the token's position, its request
  // and page (the step's description, copied to the device before the step began), and the sines and cosines of
  // its angles.  The block starts while its predecessor still runs, so this chain of dependent loads and the
  // transcendental functions cost the step nothing; only the projected rows wait for the predecessor.
  const int pos = positions[n];
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
  if (inv_freq) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sc[2 * j], &sc[2 * j + 1]);
    __syncthreads();
  }
  // With the pairs kept in registers a warp's loads of all its heads are issued together.
  const int h0 = blockIdx.y * 8 * HPW + warp;
  const bool in_regs = half <= 32 * ROPE_REG_PAIRS;
  float va[HPW][ROPE_REG_PAIRS], vb[HPW][ROPE_REG_PAIRS];
  // A decode step's few blocks rehearse (see jlx_rehearses): the rest of the kernel runs once without its loads
  // and stores while the predecessor still works, and then for real.
#pragma unroll 1
  for (int pass = in_regs && jlx_rehearses() ? 0 : 1; pass < 2; ++pass) {
  const bool real = pass == 1;
  if (real) pdl_wait();
  if (in_regs) {
#pragma unroll
    for (int t = 0; t < HPW; ++t) {
      const int h = h0 + 8 * t;
      const TI* src = row + (size_t)h * dh;
#pragma unroll
      for (int i = 0; i < ROPE_REG_PAIRS; ++i) {
        const int j = lane + 32 * i;
        float a = 0.f, b = 0.f;
        if (real && h < heads && j < half) {
          // the split-K partials of a pair are fetched eight at a time and then added in ascending order: a loop
          // that added each as it came paid one memory latency per partial
          for (int z0 = 0; z0 < splits; z0 += 8) {
            float2 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (z0 + u < splits) v[u] = load_pair<TI>(src + (size_t)(z0 + u) * split_stride + 2 * j);
#pragma unroll
            for (int u = 0; u < 8; ++u)
              if (z0 + u < splits) {
                if (z0 + u == 0) { a = v[u].x; b = v[u].y; }
                else { a += v[u].x; b += v[u].y; }
              }
          }
        }
        va[t][i] = a;
        vb[t][i] = b;
      }
    }
  }

  JLX_TL_MARK(0);
#pragma unroll
  for (int t = 0; t < HPW; ++t) {
    const int h = h0 + 8 * t;
    if (h >= heads) break;
    const TI* src = row + (size_t)h * dh;
    const bool is_v = h >= Hq + Hkv;  // value heads are copied (the sum of the partials): no rotation, no norm
    T* dst = h < Hq ? q_out + ((size_t)n * Hq + h) * dh
                    : (is_v ? (vdst ? vdst + (size_t)(h - Hq - Hkv) * page_size * dh : nullptr)
                            : (kdst ? kdst + (size_t)(h - Hq) * page_size * dh : nullptr));
    if (in_regs) {
      // one pass: a lane keeps its pairs in registers between the sum of squares and the write
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < ROPE_REG_PAIRS; ++i) {
        const int j = lane + 32 * i;
        if (j < half) {
          float a = va[t][i], b = vb[t][i];
          if (inv_freq && !is_v) {
            const float s = sc[2 * j], c = sc[2 * j + 1];
            const float ra = a * c - b * s, rb = b * c + a * s;
            a = ra;
            b = rb;
          }
          ss += a * a + b * b;
          va[t][i] = a;
          vb[t][i] = b;
        }
      }
      float inv = 1.f;
      if (l2norm && !is_v) {
        ss = warp_sum(ss);
        inv = 1.f / sqrtf(ss / (float)dh + eps);
      }
      if (!dst) continue;
#pragma unroll
      for (int i = 0; i < ROPE_REG_PAIRS; ++i) {
        const int j = lane + 32 * i;
        if (real && j < half) store_pair<T>(dst + 2 * j, va[t][i] * inv, vb[t][i] * inv);
      }
      continue;
    }
    if (is_v) {
      if (dst) {
        for (int j = lane; j < half; j += 32) {
          float a = 0.f, b = 0.f;
          for (int z = 0; z < splits; ++z) {
            const float2 v = load_pair<TI>(src + (size_t)z * split_stride + 2 * j);
            a += v.x;
            b += v.y;
          }
          store_pair<T>(dst + 2 * j, a, b);
        }
      }
      continue;
    }
    // larger heads: pass 1 rotates and accumulates the sum of squares
    float ss = 0.f;
    for (int j = lane; j < half; j += 32) {
      float a = 0.f, b = 0.f;
      for (int z = 0; z < splits; ++z) {
        a += to_f32<TI>(src[(size_t)z * split_stride + 2 * j]);
        b += to_f32<TI>(src[(size_t)z * split_stride + 2 * j + 1]);
      }
      if (inv_freq) {
        const float s = sc[2 * j], c = sc[2 * j + 1];
        const float ra = a * c - b * s, rb = b * c + a * s;
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
    // pass 2: the same values again, scaled and written
    for (int j = lane; j < half; j += 32) {
      float a = 0.f, b = 0.f;
      for (int z = 0; z < splits; ++z) {
        a += to_f32<TI>(src[(size_t)z * split_stride + 2 * j]);
        b += to_f32<TI>(src[(size_t)z * split_stride + 2 * j + 1]);
      }
      if (inv_freq) {
        const float s = sc[2 * j], c = sc[2 * j + 1];
        const float ra = a * c - b * s, rb = b * c + a * s;
        a = ra;
        b = rb;
      }
      dst[2 * j] = from_f32<T>(a * inv);
      dst[2 * j + 1] = from_f32<T>(b * inv);
    }
  }
  }
}

// The same for many tokens in bfloat16 (a prompt portion): one block per token takes ALL its heads, eight elements
// (four rotary pairs, 16 bytes) per thread and access, so that a token's angles are computed once (not once per
// group of heads) and every load and store is 16 bytes wide.  A head's dh / 8 threads are neighbours in a warp and
// add their squares by shuffles.  Needs dh / 8 a power of two up to 32 (head sizes 8, 16, 32, 64, 128, 256).
// The arithmetic of an element is the general kernel's; only the order of the sum of squares differs.
__global__ void __launch_bounds__(256)
rope_kv_store_rows_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ pages,
                          const int* __restrict__ block_table, int bt_stride, const int* __restrict__ req_of_token,
                          const int* __restrict__ positions, const float* __restrict__ inv_freq, int l2norm, float eps, int Hq,
                          int Hkv, int dh, int page_size, int num_pages, int store_kv, int* status) {
  JLX_TL(TL_ROPE);
  extern __shared__ float sc[];  // [dh / 2][2]: sine and cosine of this token's angles
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int heads = Hq + 2 * Hkv, per_head = dh >> 3, vectors = heads * per_head;
  const uint4* row = reinterpret_cast<const uint4*>(qkv + (size_t)n * heads * dh);
  // this thread's vectors first: the loads depend on nothing and fly during the dependent loads below
  constexpr int MAXV = 4;
  uint4 v[MAXV];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < vectors) v[i] = row[idx];
  }
  const int pos = positions[n];
  bf16* kdst = nullptr;
  bf16* vdst = nullptr;
  if (store_kv) {
    const int r = req_of_token[n];
    const int page = block_table[(size_t)r * bt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_PAGE);
    } else {
      bf16* base = pages + (size_t)page * 2 * Hkv * page_size * dh;
      kdst = base + (size_t)(pos % page_size) * dh;
      vdst = base + (size_t)Hkv * page_size * dh + (size_t)(pos % page_size) * dh;
    }
  }
  if (inv_freq) {
    for (int j = threadIdx.x; j < (dh >> 1); j += blockDim.x) sincosf((float)pos * inv_freq[j], &sc[2 * j], &sc[2 * j + 1]);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * 256;
    const bool mine = idx < vectors;  // (no early exit: the shuffles below need the whole warp)
    const int h = mine ? idx / per_head : 0, part = idx % per_head;
    const bool is_v = h >= Hq + Hkv;
    float f[8];
    {
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 t = mine ? __bfloat1622float2(p2[u]) : make_float2(0.f, 0.f);
        f[2 * u] = t.x;
        f[2 * u + 1] = t.y;
      }
    }
    float ss = 0.f;
    if (!is_v) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float a = f[2 * u], b = f[2 * u + 1];
        if (inv_freq) {
          const int j = part * 4 + u;
          const float s = sc[2 * j], c = sc[2 * j + 1];
          const float ra = a * c - b * s, rb = b * c + a * s;
          a = ra;
          b = rb;
        }
        ss += a * a + b * b;
        f[2 * u] = a;
        f[2 * u + 1] = b;
      }
    }
    float inv = 1.f;
    if (l2norm) {  // uniform over the block
      for (int o = per_head >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!is_v) inv = 1.f / sqrtf(ss / (float)dh + eps);
    }
    if (!mine) continue;
    bf16* dst = h < Hq ? q_out + ((size_t)n * Hq + h) * dh
                       : (is_v ? (vdst ? vdst + (size_t)(h - Hq - Hkv) * page_size * dh : nullptr)
                               : (kdst ? kdst + (size_t)(h - Hq) * page_size * dh : nullptr));
    if (!dst) continue;
    uint4 o;
    if (is_v) {
      o = v[i];  // values are copied as they are
    } else {
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int u = 0; u < 4; ++u) o2[u] = __floats2bfloat162_rn(f[2 * u] * inv, f[2 * u + 1] * inv);
    }
    *reinterpret_cast<uint4*>(dst + part * 8) = o;
  }
}

JLX_API int jlx_rope_kv_store(const void* qkv, int in_dtype, int splits, long long split_stride, void* q_out, void* pages,
                              int dtype, const int* block_table, int bt_stride, const int* req_of_token,
                              const int* positions, const float* inv_freq, int l2norm, float eps, int N, int Hq, int Hkv,
                              int dh, int page_size, int num_pages, int store_kv, int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && Hq > 0 && Hkv >= 0 && dh > 0, "rope_kv_store: bad sizes N=%d Hq=%d Hkv=%d dh=%d", N, Hq, Hkv, dh);
  JLX_REQUIRE(dh % 2 == 0, "rope_kv_store: head size %d must be even (rotary pairs)", dh);
  JLX_REQUIRE(dh <= 8192, "rope_kv_store: head size %d is above the supported maximum 8192", dh);
  JLX_REQUIRE(!store_kv || (page_size > 0 && num_pages > 0 && bt_stride > 0), "rope_kv_store: bad cache sizes");
  JLX_REQUIRE(splits >= 1 && (splits == 1 || in_dtype == JLX_F32), "rope_kv_store: split-K partials are float32");
  JLX_REQUIRE((Hq + 2 * Hkv + 7) / 8 <= 65535, "rope_kv_store: too many heads");
  if (N == 0) return 0;
  const size_t smem = (size_t)dh * sizeof(float);
  const int heads = Hq + 2 * Hkv;
  // many tokens (prompt portions): two heads per warp; few (decoding): one, for the most blocks
  const bool wide = N >= 256 && heads > 8;
  // many tokens in bfloat16: the kernel that takes a token's heads 16 bytes at a time
  const int per_head = dh / 8;
  if (N >= 256 && in_dtype == JLX_BF16 && dtype == JLX_BF16 && splits == 1 && dh % 8 == 0 && per_head <= 32 &&
      (per_head & (per_head - 1)) == 0 && heads * per_head <= 4 * 256 &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0) {
    JLX_CUDA(jlx_launch_pdl(rope_kv_store_rows_kernel, dim3(N), dim3(256), smem, stream, (const bf16*)qkv, (bf16*)q_out,
                            (bf16*)pages, block_table, bt_stride, req_of_token, positions, inv_freq, l2norm, eps, Hq, Hkv, dh,
                            page_size, num_pages, store_kv, status));
    return 0;
  }
  JLX_DISPATCH_DTYPE(in_dtype, TI, JLX_DISPATCH_DTYPE(dtype, T, {
    if (wide) {
      JLX_CUDA(jlx_launch_pdl(rope_kv_store_kernel<TI, T, 2>, dim3(N, (heads + 15) / 16), dim3(256), smem, stream,
                              (const TI*)qkv, splits, split_stride, (T*)q_out, (T*)pages, block_table, bt_stride, req_of_token,
                              positions, inv_freq, l2norm, eps, Hq, Hkv, dh, page_size, num_pages, store_kv, status));
    } else {
      JLX_CUDA(jlx_launch_pdl(rope_kv_store_kernel<TI, T, 1>, dim3(N, (heads + 7) / 8), dim3(256), smem, stream,
                              (const TI*)qkv, splits, split_stride, (T*)q_out, (T*)pages, block_table, bt_stride, req_of_token,
                              positions, inv_freq, l2norm, eps, Hq, Hkv, dh, page_size, num_pages, store_kv, status));
    }
  }));
  return 0;
}

// Plain write of already-encoded k and v rows into pages (for position encodings that are not fused).
// k, v: [N, Hkv, dh]
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ pages,
                                const int* __restrict__ block_table, int bt_stride,
                                const int* __restrict__ req_of_token, const int* __restrict__ positions, int Hkv,
                                int dh, int page_size, int num_pages, int* status) {
  JLX_TL(TL_KV_STORE);
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
