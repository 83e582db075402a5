// Next-token choice from 32-bit logits: argmax, or temperature sampling over the k most likely
// tokens (all of them when k = 0) with a counter-based random number per request.
//
// Reference: llama4 decodes by argmax only (llama4/llama4_jax/model.py:1266,1275).  The repository's
// sampler is gpt_oss/gpt_oss_jax/model.py:1125-1147: softmax(logits / temp), top-k, normalised
// cumulative sum, first index whose cumulative probability reaches the uniform draw; temp <= 1e-3
// means argmax.  The draw here is Philox-4x32-10 keyed by (seed, request stream) with the request's
// step as counter, so a request's tokens do not depend on what else is in the batch.
#include "common.cuh"
#include "sampling_noalloc.h"

#define SAMPLE_MAX_K 64

__device__ __forceinline__ void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += W0; k1 += W1;
  }
}

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; equal values: lower index wins; index -1 = empty
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  if (warp == 0) {
    ArgMax t = lane < nwarp ? scratch[lane] : ArgMax{0.f, -1};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b;
      b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
      b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
      t = better(t, b);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// One block per row.  params per row: temperature[m], top_k[m], stream[m] (request's random stream),
// counter[m] (request's step).  Rows with temperature <= 1e-3 take the argmax.
__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int V, long long ld, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const unsigned long long* __restrict__ streams,
              const unsigned long long* __restrict__ counters, unsigned long long seed, int* __restrict__ out) {
  JLX_TL(TL_SAMPLE);
  __shared__ ArgMax scratch[33];
  __shared__ float fscratch[33];
  __shared__ float topv[SAMPLE_MAX_K];
  __shared__ int topi[SAMPLE_MAX_K];
  __shared__ float partial[1024];
  const int m = blockIdx.x;
  const float* row = logits + (size_t)m * ld;
  const float temp = temperature ? temperature[m] : 0.f;

  ArgMax best{0.f, -1};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (!isnan(v)) best = better(best, ArgMax{v, i});
  }
  best = block_argmax(best, scratch);
  if (temp <= 1e-3f || best.i < 0) {
    if (threadIdx.x == 0) out[m] = best.i < 0 ? 0 : best.i;
    return;
  }
  // uniform draw for this (request stream, step)
  uint32_t c[4] = {(uint32_t)counters[m], (uint32_t)(counters[m] >> 32), (uint32_t)streams[m], (uint32_t)(streams[m] >> 32)};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  const float u = (float)(c[0] >> 8) * (1.0f / 16777216.0f);
  const float inv_t = 1.f / temp;
  const float mx = best.v;
  int k = top_k ? top_k[m] : 0;
  if (k > V) k = V;
  if (k > SAMPLE_MAX_K) k = SAMPLE_MAX_K;  // the host refuses larger k before the launch

  if (k > 0) {
    // k rounds of argmax over what is not yet taken: (value, index) strictly below the last pick
    // in the order "larger value first, lower index first".
    float lastv = INFINITY;
    int lasti = -1;
    for (int j = 0; j < k; ++j) {
      ArgMax b{0.f, -1};
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (isnan(v)) continue;
        const bool after = (v < lastv) || (v == lastv && i > lasti);
        if (after) b = better(b, ArgMax{v, i});
      }
      b = block_argmax(b, scratch);
      if (b.i < 0) { k = j; break; }
      if (threadIdx.x == 0) {
        topv[j] = expf((b.v - mx) * inv_t);
        topi[j] = b.i;
      }
      lastv = b.v;
      lasti = b.i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int j = 0; j < k; ++j) total += topv[j];
      float run = 0.f;
      int pick = topi[k - 1];
      for (int j = 0; j < k; ++j) {
        run += topv[j];
        if (u <= run / total) { pick = topi[j]; break; }
      }
      out[m] = pick;
    }
    return;
  }
  // whole vocabulary, cumulative sum in index order: thread t owns one contiguous span
  const int span = (V + blockDim.x - 1) / blockDim.x;
  const int lo = min(V, (int)threadIdx.x * span), hi = min(V, lo + span);
  float s = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float v = row[i];
    if (!isnan(v)) s += expf((v - mx) * inv_t);
  }
  partial[threadIdx.x] = s;
  const float total = block_sum(s, fscratch);
  __syncthreads();
  if (threadIdx.x == 0) {
    // find the span, then the index inside it
    float run = 0.f;
    int t = 0;
    for (; t < (int)blockDim.x - 1; ++t) {
      if (u <= (run + partial[t]) / total) break;
      run += partial[t];
    }
    const int l2 = min(V, t * span), h2 = min(V, l2 + span);
    int pick = -1;
    for (int i = l2; i < h2; ++i) {
      const float v = row[i];
      if (isnan(v)) continue;
      run += expf((v - mx) * inv_t);
      if (u <= run / total) { pick = i; break; }
    }
    if (pick < 0) {  // rounding at the very end of the range: last token with weight
      pick = best.i;
      for (int i = V - 1; i >= 0; --i)
        if (!isnan(row[i]) && expf((row[i] - mx) * inv_t) > 0.f) { pick = i; break; }
    }
    out[m] = pick;
  }
}

// Greedy choice in two stages so that a handful of rows still uses the whole GPU: each block finds the
// best (value, index) of one chunk of a row; one block per row then picks among the chunks.  Ties go to
// the lower index in both stages.
#define ARGMAX_CHUNKS 32
__global__ void __launch_bounds__(256)
argmax_chunk_kernel(const float* __restrict__ logits, int V, long long ld, float* __restrict__ part_v, int* __restrict__ part_i) {
  JLX_TL(TL_ARGMAX);
  __shared__ ArgMax scratch[33];
  const int m = blockIdx.y, c = blockIdx.x;
  const int span = ((V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS + 3) / 4 * 4;  // a multiple of 4: chunks start 16-byte aligned
  const int lo = min(V, c * span), hi = min(V, lo + span);
  const float* row = logits + (size_t)m * ld;
  ArgMax best{0.f, -1};
  if ((ld & 3) == 0 && ((uintptr_t)logits & 15) == 0) {
    // four values per access and a thread's accesses in flight together: a step's one or few rows are read at the speed
    // of a memory latency per round, so there should be few rounds
    constexpr int AHEAD = 4;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int lo4 = lo >> 2, hi4 = hi >> 2;  // whole vectors; the row's last 1..3 values follow below
    for (int i0 = lo4 + threadIdx.x; i0 < hi4; i0 += AHEAD * blockDim.x) {
      float4 v[AHEAD];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u)
        if (i0 + u * blockDim.x < hi4) v[u] = row4[i0 + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < hi4) {
          if (!isnan(v[u].x)) best = better(best, ArgMax{v[u].x, 4 * i});
          if (!isnan(v[u].y)) best = better(best, ArgMax{v[u].y, 4 * i + 1});
          if (!isnan(v[u].z)) best = better(best, ArgMax{v[u].z, 4 * i + 2});
          if (!isnan(v[u].w)) best = better(best, ArgMax{v[u].w, 4 * i + 3});
        }
      }
    }
    for (int i = (hi4 << 2) + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = row[i];
      if (!isnan(v)) best = better(best, ArgMax{v, i});
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = row[i];
      if (!isnan(v)) best = better(best, ArgMax{v, i});
    }
  }
  best = block_argmax(best, scratch);
  if (threadIdx.x == 0) {
    part_v[m * ARGMAX_CHUNKS + c] = best.v;
    part_i[m * ARGMAX_CHUNKS + c] = best.i;
  }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out) {
  JLX_TL(TL_ARGMAX);
  const int m = blockIdx.x, lane = threadIdx.x;
  ArgMax a{part_v[m * ARGMAX_CHUNKS + lane], part_i[m * ARGMAX_CHUNKS + lane]};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  if (lane == 0) out[m] = a.i < 0 ? 0 : a.i;
}

// part_v: float [M * 32], part_i: int [M * 32] scratch.
JLX_API int jlx_argmax(const float* logits, int M, int V, long long ld, float* part_v, int* part_i, int* out,
                       cudaStream_t stream) {
  JLX_REQUIRE(M >= 0 && V > 0 && ld >= V, "argmax: bad sizes M=%d V=%d", M, V);
  JLX_REQUIRE(part_v && part_i, "argmax: scratch missing");
  JLX_REQUIRE(M <= 65535, "argmax: too many rows");
  if (M == 0) return 0;
  argmax_chunk_kernel<<<dim3(ARGMAX_CHUNKS, M), 256, 0, stream>>>(logits, V, ld, part_v, part_i);
  JLX_LAUNCH_CHECK("argmax_chunk");
  argmax_final_kernel<<<M, 32, 0, stream>>>(part_v, part_i, out);
  JLX_LAUNCH_CHECK("argmax_final");
  return 0;
}

// ---- the variant for callers that cannot allocate: see sampling_noalloc.h for who they are and the rules.
// Layout of the array: ARGMAX_CHUNKS * MAX_ROWS best values (float) followed by as many best indices (int).
static __device__ __align__(256) unsigned char jlx_argmax_noalloc_scratch[JLX_ARGMAX_NOALLOC_MAX_ROWS * ARGMAX_CHUNKS * 8];

// In host code the array's name stands for a host-side shadow, not for device memory: the device address
// has to be asked for, once per device, while that device is current.
static int noalloc_scratch_address(unsigned char** ptr) {
  enum { MAX_DEVICES = 64 };
  static unsigned char* cached[MAX_DEVICES] = {nullptr};
  int dev = -1;
  JLX_CUDA(cudaGetDevice(&dev));
  JLX_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "argmax_noalloc: device ordinal %d is outside 0..%d", dev, MAX_DEVICES - 1);
  if (!cached[dev]) {
    void* p = nullptr;
    JLX_CUDA(cudaGetSymbolAddress(&p, jlx_argmax_noalloc_scratch));
    JLX_REQUIRE(p != nullptr, "argmax_noalloc: the scratch array has no device address");
    cached[dev] = static_cast<unsigned char*>(p);
  }
  *ptr = cached[dev];
  return 0;
}

JLX_API int jlx_argmax_noalloc(const float* logits, int M, int V, long long ld, int* out, cudaStream_t stream) {
  JLX_REQUIRE(M >= 0 && V > 0 && ld >= V, "argmax_noalloc: bad sizes M=%d V=%d", M, V);
  JLX_REQUIRE(M <= JLX_ARGMAX_NOALLOC_MAX_ROWS,
              "argmax_noalloc: %d rows, but the built-in scratch holds %d; use jlx_argmax with your own scratch", M,
              JLX_ARGMAX_NOALLOC_MAX_ROWS);
  JLX_REQUIRE(logits && out, "argmax_noalloc: null input or output");
  if (M == 0) return 0;
  unsigned char* base = nullptr;
  if (noalloc_scratch_address(&base)) return 1;
  float* part_v = reinterpret_cast<float*>(base);
  int* part_i = reinterpret_cast<int*>(base + (size_t)JLX_ARGMAX_NOALLOC_MAX_ROWS * ARGMAX_CHUNKS * sizeof(float));
  // every slot that the second kernel reads (M * ARGMAX_CHUNKS of each half) is written by the first
  argmax_chunk_kernel<<<dim3(ARGMAX_CHUNKS, M), 256, 0, stream>>>(logits, V, ld, part_v, part_i);
  JLX_LAUNCH_CHECK("argmax_chunk");
  argmax_final_kernel<<<M, 32, 0, stream>>>(part_v, part_i, out);
  JLX_LAUNCH_CHECK("argmax_final");
  return 0;
}

JLX_API int jlx_sample_max_top_k() { return SAMPLE_MAX_K; }

JLX_API int jlx_sample(const float* logits, int M, int V, long long ld, const float* temperature, const int* top_k,
                       const unsigned long long* streams, const unsigned long long* counters, unsigned long long seed,
                       int* out, cudaStream_t stream) {
  JLX_REQUIRE(M >= 0 && V > 0 && ld >= V, "sample: bad sizes M=%d V=%d", M, V);
  JLX_REQUIRE(!temperature || (streams && counters), "sample: temperature sampling needs streams and counters");
  if (M == 0) return 0;
  sample_kernel<<<M, 1024, 0, stream>>>(logits, V, ld, temperature, top_k, streams, counters, seed, out);
  JLX_LAUNCH_CHECK("sample");
  return 0;
}
