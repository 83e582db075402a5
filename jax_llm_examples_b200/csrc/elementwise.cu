// Embedding gather, RMSNorm fused with the residual sum, and SiLU(gate)*up.
//
// The residual stream is 32-bit in every precision mode: the sum x + delta and the norm's mean of
// squares are computed in 32-bit (reference: llama4/llama4_jax/model.py:885-888 computes the mean in
// float32; model.py:1173,1181 are the residual sums).
#include <cooperative_groups.h>

#include "common.cuh"
#include "expert_sort.cuh"

// x[n, :] = table[ids[n], :]                                     (model.py:1191)
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ x,
                             int D, int V, int* status) {
  JLX_TL(TL_EMBED);
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  int id = ids[n];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicOr(status, JLX_STATUS_BAD_TOKEN);
    id = 0;
  }
  const TW* row = table + (size_t)id * D;
  float* out = x + (size_t)n * D;
  if (sizeof(TW) == 2 && (D & 7) == 0 && (((uintptr_t)table | (uintptr_t)x) & 15) == 0) {
    // eight bfloat16 values per access, and a thread's accesses all in flight before the first is used: with one
    // row a step this kernel is a chain of memory latencies (the row comes from HBM), not a stream
    constexpr int AHEAD = 4;
    const uint4* row8 = reinterpret_cast<const uint4*>(row);
    const int D8 = D >> 3;
    for (int i0 = threadIdx.x; i0 < D8; i0 += AHEAD * blockDim.x) {
      uint4 v[AHEAD];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u)
        if (i0 + u * blockDim.x < D8) v[u] = row8[i0 + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const int i = i0 + u * blockDim.x;
        if (i < D8) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
          const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]), c = __bfloat1622float2(h[2]), e = __bfloat1622float2(h[3]);
          reinterpret_cast<float4*>(out)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
          reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(c.x, c.y, e.x, e.y);
        }
      }
    }
    return;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) out[d] = to_f32<TW>(row[d]);
}

JLX_API int jlx_embed(const int* ids, const void* table, int table_dtype, float* x, int N, int D, int V,
                      int* status, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0 && V > 0, "embed: bad sizes N=%d D=%d V=%d", N, D, V);
  if (N == 0) return 0;
  JLX_DISPATCH_DTYPE(table_dtype, TW, { JLX_CUDA(jlx_launch_pdl(embed_kernel<TW>, dim3(N), dim3(256), 0, stream, ids, (const TW*)table, x, D, V, status)); });
  return 0;
}

// Row n (source row r = row_index ? row_index[n] : n):
//   s = x[r] + sum over splits of delta[z][r]   (delta optional; split-K partials are added in ascending
//                                                 order; s is written back to x[r] unless rows are gathered)
//   out[n] = gamma * s / sqrt(mean(s^2) + eps)   (gamma optional: weightless norm)
// `out` in the activation type and/or `out32` in 32-bit (for the router, which wants unrounded input).
// With w_router the same block also routes the token (llama4/llama4_jax/model.py:958-972): scores =
// normed row . w_router[e] in 32-bit, top-k of the raw scores (lower index wins ties), weight = sigmoid.
#define ROUTER_MAX_E 256
// Four consecutive outputs as one access (the address is a multiple of 4 elements).
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float4 v) {
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = o;
}
#define ROUTER_MAX_PARTS 4
// Router scores of one row over the columns [lo, hi) (lo a multiple of 4 when the row is 16-byte aligned):
// partial[e * ROUTER_MAX_PARTS + part] for every expert.  `row` points at column lo of the normed row in
// shared memory.  The walk over a router row waits on memory, so it is spread wide: `parts` warps share one
// expert (each a contiguous piece of the range, added in a fixed order afterwards), every lane keeps eight
// independent 16-byte loads in flight.  Returns `parts`.
__device__ __forceinline__ int router_partials(const float* __restrict__ row, const float* __restrict__ w_router, int D, int lo,
                                               int hi, int E, float* partial) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  int parts = nwarp / E;
  parts = parts < 1 ? 1 : (parts > ROUTER_MAX_PARTS ? ROUTER_MAX_PARTS : parts);
  const int piece = (((hi - lo + parts - 1) / parts) + 127) / 128 * 128;  // a multiple of a warp's 128 floats
  for (int item = warp; item < E * parts; item += nwarp) {
    const int e = item / parts, part = item - e * parts;
    const float* wr = w_router + (size_t)e * D;
    const int p_lo = lo + part * piece, p_hi = min(hi, p_lo + piece);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int d = p_lo + lane * 4;
    if ((D & 3) == 0 && (lo & 3) == 0 && (((uintptr_t)w_router) & 15) == 0) {
      for (; d < p_hi; d += 8 * 128) {  // the last round's loads are guarded, not looped: all are in flight at once
        float4 wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          wv[u] = d + 128 * u < p_hi ? *reinterpret_cast<const float4*>(wr + d + 128 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (d + 128 * u < p_hi) {
            const float4 xv = *reinterpret_cast<const float4*>(row + (d - lo) + 128 * u);
            acc[u] = fmaf(xv.x, wv[u].x, fmaf(xv.y, wv[u].y, fmaf(xv.z, wv[u].z, fmaf(xv.w, wv[u].w, acc[u]))));
          }
        }
      }
    } else {
      for (int i = p_lo + lane; i < p_hi; i += 32) acc[0] = fmaf(row[i - lo], wr[i], acc[0]);
    }
    const float s = warp_sum(((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7])));
    if (lane == 0) partial[e * ROUTER_MAX_PARTS + part] = s;
  }
  return parts;
}

// Top-k of the raw scores by one thread (lower index wins ties; NaN never wins), weight = sigmoid of the score.
// Destroys `scores`.
// With keep_idx / keep_w the choices are also left there (shared memory of the caller).
__device__ __forceinline__ void router_topk(float* scores, int E, int k, size_t n, int* topk_idx, float* topk_w,
                                            int* keep_idx = nullptr, float* keep_w = nullptr) {
  for (int j = 0; j < k; ++j) {
    int best = -1;
    float bv = 0.f;
    for (int e = 0; e < E; ++e) {
      const float v = scores[e];
      if (isnan(v)) continue;
      if (best < 0 || v > bv) {
        best = e;
        bv = v;
      }
    }
    if (best < 0) best = j;
    const float weight = 1.f / (1.f + expf(-bv));
    topk_idx[n * k + j] = best;
    topk_w[n * k + j] = weight;
    if (keep_idx) {
      keep_idx[j] = best;
      keep_w[j] = weight;
    }
    scores[best] = NAN;
  }
}

// What a norm adds to the residual stream before it normalises: up to DELTA_MAX_TERMS terms, added in the order given.
// A term is `splits` float32 partials [z][rows][D] (z ascending, `stride` elements apart), of which token r takes row
// base + r, or, with `index`, the k rows index[r * k + j], j ascending (an expert layer's rows in expert order: the
// norm then does the un-permute and the sum over a token's experts that a kernel of its own would do).
#define DELTA_MAX_TERMS 3
struct DeltaTerm {
  const float* p;
  long long stride;
  const int* index;
  int splits, k, base;
};
struct DeltaSpec {
  int n;
  DeltaTerm t[DELTA_MAX_TERMS];
};

// The rows that token r adds, resolved once per block into shared memory as a flat list of streams: one per (term,
// row of the term, split) in that order, which is the order in which they are added.  The kernels then fetch a thread's
// element from up to DELTA_CHUNK streams at once: with one or a few rows a step the norm is a chain of memory
// latencies, and a loop that added stream after stream paid one latency per stream.
#define DELTA_MAX_STREAMS 64
#define DELTA_CHUNK 8
struct DeltaSources {
  const float* ptr[DELTA_MAX_STREAMS];
  int n;
};
// Called by every thread; thread 0 fills `src`, a barrier follows.
// (`real` false: a rehearsal, which loads nothing that a predecessor writes; the pointers it makes are never used)
__device__ __forceinline__ void resolve_delta(DeltaSources& src, const DeltaSpec& ds, size_t r, int D, bool real = true) {
  if (threadIdx.x == 0) {
    int n = 0;
#pragma unroll
    for (int q = 0; q < DELTA_MAX_TERMS; ++q) {  // unrolled: the terms stay in the kernel's parameter space
      if (q >= ds.n) break;
      const DeltaTerm& t = ds.t[q];
      const int rows = t.index ? t.k : 1;
      for (int j = 0; j < rows; ++j) {
        const size_t row = t.index && real ? (size_t)t.index[r * t.k + j] : (size_t)t.base + r;
        for (int z = 0; z < t.splits && n < DELTA_MAX_STREAMS; ++z) src.ptr[n++] = t.p + (size_t)z * t.stride + row * D;
      }
    }
    src.n = n;
  }
  __syncthreads();
}

// s += the streams' 16-byte element i, in stream order; a chunk of streams is in flight at once.
__device__ __forceinline__ void add_streams4(float4& s, const DeltaSources& src, int i, bool real = true) {
  for (int q0 = 0; q0 < src.n; q0 += DELTA_CHUNK) {
    float4 v[DELTA_CHUNK];
#pragma unroll
    for (int u = 0; u < DELTA_CHUNK; ++u) {
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (real && q0 + u < src.n) v[u] = reinterpret_cast<const float4*>(src.ptr[q0 + u])[i];
    }
#pragma unroll
    for (int u = 0; u < DELTA_CHUNK; ++u)
      if (q0 + u < src.n) { s.x += v[u].x; s.y += v[u].y; s.z += v[u].z; s.w += v[u].w; }
  }
}

template <typename TO>
__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(float* __restrict__ x, const DeltaSpec ds,
                   const float* __restrict__ gamma, float eps, TO* __restrict__ out, float* __restrict__ out32,
                   const int* __restrict__ row_index, int D, int row_in_smem, const float* __restrict__ w_router, int E,
                   int k, int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  JLX_TL(TL_NORM);
  extern __shared__ __align__(16) float rowbuf[];  // [D] when row_in_smem
  __shared__ float scratch[33];
  __shared__ float scores[ROUTER_MAX_E];
  __shared__ float partial[ROUTER_MAX_E * ROUTER_MAX_PARTS];
  pdl_launch_dependents();
  // 16-byte accesses when the row allows it (width a multiple of 4, row kept in shared memory)
  bool vec = row_in_smem && (D & 3) == 0;
#pragma unroll
  for (int q = 0; q < DELTA_MAX_TERMS; ++q) vec = vec && (q >= ds.n || (ds.t[q].stride & 3) == 0);
  // The norm's weights depend on no kernel: a thread's first elements of them are fetched before the wait for the
  // predecessor.
  const float4 g_ahead = vec && gamma && (int)threadIdx.x < (D >> 2) ? reinterpret_cast<const float4*>(gamma)[threadIdx.x]
                                                                      : make_float4(1.f, 1.f, 1.f, 1.f);
  if (gridDim.x <= 64) {  // a decode step's few rows: the weights have left L2 since the layer before
    if (gamma) l2_prefetch_block(gamma, (size_t)D * 4);
    if (w_router) l2_prefetch_block(w_router, (size_t)E * D * 4);
  }
  const int n = blockIdx.x;
  const bool has_delta = ds.n > 0;
  __shared__ DeltaSources src;
  // (No rehearsal here, see jlx_rehearses: measured, it made this kernel slower, whether its block started just before
  // the end of the matrix product in front of it or, with fewer threads, long before.)
  pdl_wait();
  const size_t r = row_index ? (size_t)row_index[n] : (size_t)n;
  float* xr = x + r * D;
  if (has_delta) resolve_delta(src, ds, r, D);
  JLX_TL_MARK(0);
  float ss = 0.f;
  if (vec) {
    const int D4 = D >> 2;
    float4* x4 = reinterpret_cast<float4*>(xr);
    float4* row4 = reinterpret_cast<float4*>(rowbuf);
    for (int i = threadIdx.x; i < D4; i += blockDim.x) {
      float4 t = x4[i];  // in flight together with the first chunk of streams
      if (has_delta) {
        add_streams4(t, src, i);
        if (!row_index) x4[i] = t;
      }
      row4[i] = t;
      ss += (t.x * t.x + t.y * t.y) + (t.z * t.z + t.w * t.w);
    }
    JLX_TL_MARK(1);
    ss = block_sum(ss, scratch);
    JLX_TL_MARK(2);
    const float rms = sqrtf(ss / (float)D + eps);
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    int turn = 0;
    for (int i = threadIdx.x; i < D4; i += blockDim.x, ++turn) {
      const float4 t = row4[i];
      const float4 g = turn == 0 ? g_ahead : (gamma ? g4[i] : make_float4(1.f, 1.f, 1.f, 1.f));
      const float4 v = make_float4(g.x * t.x / rms, g.y * t.y / rms, g.z * t.z / rms, g.w * t.w / rms);
      if (out) store4<TO>(out + (size_t)n * D + 4 * i, v);
      if (out32) reinterpret_cast<float4*>(out32 + (size_t)n * D)[i] = v;
      row4[i] = v;
    }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float s = xr[d];
      if (has_delta) {
        for (int q = 0; q < src.n; ++q) s += src.ptr[q][d];
        if (!row_index) xr[d] = s;
      }
      if (row_in_smem) rowbuf[d] = s;
      ss += s * s;
    }
    ss = block_sum(ss, scratch);
    const float rms = sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float s;
      if (row_in_smem) {
        s = rowbuf[d];
      } else {
        s = xr[d];
        if (has_delta && row_index)
          for (int q = 0; q < src.n; ++q) s += src.ptr[q][d];
      }
      const float v = (gamma ? gamma[d] * s : s) / rms;
      if (out) out[(size_t)n * D + d] = from_f32<TO>(v);
      if (out32) out32[(size_t)n * D + d] = v;
      if (row_in_smem) rowbuf[d] = v;
    }
  }
  JLX_TL_MARK(3);
  if (w_router) {
    __syncthreads();
    const int parts = router_partials(rowbuf, w_router, D, 0, D, E, partial);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      float s = 0.f;
      for (int part = 0; part < parts; ++part) s += partial[e * ROUTER_MAX_PARTS + part];
      scores[e] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) router_topk(scores, E, k, (size_t)n, topk_idx, topk_w);
  }
}

// The same for a handful of rows (a decode step), with or without a router, where one block per row would leave the
// row to a single SM: its instructions (32 warps through four schedulers) and the router's weights (E * D * 4
// bytes) then take longer than the memory latencies.  A cluster of blocks shares the row.  Each block takes a slice of
// the columns: its part of the sum of squares and of every expert's score goes through distributed shared
// memory, block 0 of the cluster adds the parts in rank order and chooses the experts.  bfloat16 output only:
// the order of the sums differs from the one-block kernel's, which the 32-bit path must not depend on.
// What a decode step's routed feed-forward needs after the router, done by the same kernel when it is asked to (`counter`
// not null): the sort of the step's (token, choice) pairs by expert and the gather of the scaled rows in expert order,
// which as kernels of their own are two more links in the step's chain of dependent launches.  See expert_sort_kernel
// and permute_scale_kernel (moe.cu) for the outputs' meaning.  The rows' clusters take a ticket each from `counter`
// (zero before the launch and after it); the cluster that takes the last one does the work for all rows.
#define DISPATCH_MAX_ROWS 16    // tokens
#define DISPATCH_MAX_PAIRS 64   // tokens x choices
struct DispatchArgs {
  int* counter;
  int* offsets;
  int* sorted_pair;
  int* sorted_pos;
  int* tile_list;   // with tile_rows > 0
  int* n_tiles;
  void* a_sorted;   // [pairs + extra_rows, D], the kernel's output type
  int extra_rows, tile_rows;
  int* status;
};

#define NORM_CLUSTER 8
// ROUTER: with the router (else w_router is not used, and the kernel is two of everything leaner).
template <typename TO, bool ROUTER>
__global__ void __launch_bounds__(ROUTER ? 512 : 256, 1)
add_rmsnorm_router_cluster_kernel(float* __restrict__ x, const DeltaSpec ds,
                                  const float* __restrict__ gamma, float eps, TO* __restrict__ out, float* __restrict__ out32, int D,
                                  int slice,
                                  const float* __restrict__ w_router, int E, int k, int* __restrict__ topk_idx,
                                  float* __restrict__ topk_w, const DispatchArgs dp) {
  JLX_TL(TL_NORM_ROUTER);
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  constexpr int C = NORM_CLUSTER;  // known at compile time: the loops over the ranks' shared memory unroll, their loads overlap
  extern __shared__ __align__(16) float rowbuf[];  // [slice]
  __shared__ float scratch[33];
  __shared__ float cl_ss[NORM_CLUSTER];                       // every block's part of the sum of squares (each block has all)
  __shared__ float cl_scores[NORM_CLUSTER][ROUTER_MAX_E];    // every block's part of every expert's score (used in block 0)
  __shared__ float scores[ROUTER_MAX_E];
  __shared__ float partial[ROUTER_MAX_E * ROUTER_MAX_PARTS];
  __shared__ int choice[DISPATCH_MAX_PAIRS], order[DISPATCH_MAX_PAIRS];  // for the sort and gather (see DispatchArgs)
  __shared__ float choice_w[DISPATCH_MAX_PAIRS], order_w[DISPATCH_MAX_PAIRS];
  __shared__ int counts[ROUTER_MAX_E + 1];
  pdl_launch_dependents();
  const int n = blockIdx.x / C;
  const int lo = min(D, rank * slice), hi = min(D, lo + slice);  // multiples of 4
  float4* x4 = reinterpret_cast<float4*>(x + (size_t)n * D);
  float4* row4 = reinterpret_cast<float4*>(rowbuf);
  __shared__ DeltaSources src;
  // this block's slices of the norm's and the router's weights have left L2 since the layer before: they are asked
  // back while the predecessor still runs.  (No rehearsal, see jlx_rehearses: the kernel follows a matrix product
  // whose blocks fill the GPU, its cluster starts only microseconds before that ends, and a rehearsal then still runs
  // when the real work could begin.)
  if (gamma) l2_prefetch_block(gamma + lo, (size_t)(hi - lo) * 4);
  if (ROUTER)
    for (int e = 0; e < E; ++e) l2_prefetch_block(w_router + (size_t)e * D + lo, (size_t)(hi - lo) * 4);
  // A thread's norm weights wait in a register.  The blocks of the cluster meet once here, where it costs nothing:
  // from then on all of them run, so that a block may WRITE its partial results into the others' shared memory
  // before the barriers below instead of reading theirs after (a remote read is a round trip on the critical path,
  // a remote write is not), and block 0 needs nobody after the last barrier.
  const int mine = (lo >> 2) + threadIdx.x;
  const float4 g_ahead = gamma && mine < (hi >> 2) ? reinterpret_cast<const float4*>(gamma)[mine] : make_float4(1.f, 1.f, 1.f, 1.f);
  cluster.sync();
  // Without a router the blocks are lean enough to sit beside the blocks of the matrix product before; with one row
  // in the step that product leaves room on the SMs (240 blocks at Scout's sizes), the cluster starts long before it
  // ends, and rehearses (see jlx_rehearses).  With more rows the product fills the GPU to its end, with a router
  // the blocks are not lean: the cluster then starts only microseconds before its work, and does not rehearse.
#pragma unroll 1
  for (int pass = ROUTER || gridDim.x > C ? 1 : 0; pass < 2; ++pass) {
  const bool real = pass == 1;
  if (real) pdl_wait();
  if (ds.n > 0) resolve_delta(src, ds, (size_t)n, D, real);
  float ss = 0.f;
  for (int i = (lo >> 2) + threadIdx.x; i < (hi >> 2); i += blockDim.x) {
    float4 s = make_float4(1.f, 1.f, 1.f, 1.f);
    if (real) s = x4[i];
    if (ds.n > 0) {
      add_streams4(s, src, i, real);
      if (real) x4[i] = s;
    }
    row4[i - (lo >> 2)] = s;
    ss += (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w);
  }
  JLX_TL_MARK(0);
  ss = block_sum(ss, scratch);  // (every thread has the sum)
  if (threadIdx.x < C) *cluster.map_shared_rank(&cl_ss[rank], threadIdx.x) = ss;
  cluster.sync();
  JLX_TL_MARK(1);
  float total = 0.f;
#pragma unroll
  for (int r = 0; r < C; ++r) total += cl_ss[r];
  // One division, then products: four exact divisions per thread are some fifty instructions with branches, and in a
  // block that runs this code once, cold, instructions cost more than arithmetic.  (The result differs from the
  // quotient's by a rounding of 32-bit; this kernel's output is bfloat16.)
  const float inv_rms = 1.f / sqrtf(total / (float)D + eps);
  const float4* g4 = reinterpret_cast<const float4*>(gamma);
  if (!ROUTER) JLX_TL_MARK(2);
  for (int i = (lo >> 2) + threadIdx.x; i < (hi >> 2); i += blockDim.x) {
    const float4 s = row4[i - (lo >> 2)];
    const float4 g = i == mine ? g_ahead : (gamma ? g4[i] : make_float4(1.f, 1.f, 1.f, 1.f));
    const float4 v = make_float4(g.x * s.x * inv_rms, g.y * s.y * inv_rms, g.z * s.z * inv_rms, g.w * s.w * inv_rms);
    if (real) store4<TO>(out + (size_t)n * D + 4 * i, v);
    if (real && out32) reinterpret_cast<float4*>(out32 + (size_t)n * D)[i] = v;
    row4[i - (lo >> 2)] = v;
  }
  if (!ROUTER) JLX_TL_MARK(3);
  if (!ROUTER) {  // a norm without a router: no remote access after the barrier above
    if (real) return;
    cluster.sync();  // ... of the rehearsal, whose values nobody may still be reading when the real ones are written
    continue;
  }
  __syncthreads();
  const int parts = router_partials(rowbuf, w_router, D, lo, hi, E, partial);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float s = 0.f;
    for (int part = 0; part < parts; ++part) s += partial[e * ROUTER_MAX_PARTS + part];
    cluster.map_shared_rank(&cl_scores[rank][0], 0)[e] = s;  // into block 0's shared memory
  }
  JLX_TL_MARK(2);
  cluster.sync();  // the last remote access of the kernel is before this barrier: the other blocks may leave
  JLX_TL_MARK(3);
  if (rank == 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int r = 0; r < C; ++r) s += cl_scores[r][e];
      scores[e] = s;
    }
    __syncthreads();
    if (threadIdx.x == 0) router_topk(scores, E, k, (size_t)n, topk_idx, topk_w, k <= DISPATCH_MAX_PAIRS ? choice : nullptr, choice_w);
  }
  if (ROUTER && dp.counter) {
    // ---- the sort and the gather.  One row in the step: this cluster, from the choices that block 0 still holds.
    // More rows: the cluster whose row is the last to have its experts, from all rows' choices in global memory.
    __shared__ int cl_last;
    const int rows = gridDim.x / C, P = rows * k;
    if (rows > 1) {
      if (rank == 0 && threadIdx.x == 0) {
        __threadfence();  // this row's normed values (all blocks', by way of the barrier above) and choices, before the ticket
        const int last = atomicAdd(dp.counter, 1) == rows - 1;
        if (last) *dp.counter = 0;  // as the next launch expects it
        __threadfence();  // ... and the other rows' after it
#pragma unroll
        for (int r = 0; r < C; ++r) *cluster.map_shared_rank(&cl_last, r) = last;
      }
      cluster.sync();
      if (!cl_last) return;
    }
    if (rank == 0) {
      __syncthreads();  // (one row: the choices that thread 0 kept)
      if (rows > 1)
        for (int i = threadIdx.x; i < P; i += blockDim.x) {  // other clusters' writes: past L1
          choice[i] = __ldcg(topk_idx + i);
          choice_w[i] = __ldcg(topk_w + i);
        }
      __syncthreads();
      for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < P; ++i) c += choice[i] == e;
        counts[e] = c;
      }
      __syncthreads();
      if (threadIdx.x < 32) expert_offsets_and_tiles(counts, E, P, dp.extra_rows, dp.tile_rows, dp.offsets, dp.tile_list, dp.n_tiles, dp.status, true);
      __syncthreads();
      for (int i = threadIdx.x; i < P; i += blockDim.x) {  // stable: a pair follows the earlier pairs of its expert
        const int e = choice[i];
        if (e < 0 || e >= E) continue;  // (never chosen by the router above; the count check has raised the status)
        int dst = counts[e];
        for (int j = 0; j < i; ++j) dst += choice[j] == e;
        dp.sorted_pair[dst] = i;
        dp.sorted_pos[i] = dst;
        // the sorted order and the weights go into every block's shared memory: the gather below waits for no load
#pragma unroll
        for (int r = 0; r < C; ++r) {
          cluster.map_shared_rank(order, r)[dst] = i;
          cluster.map_shared_rank(order_w, r)[dst] = choice_w[i];
        }
      }
    }
    cluster.sync();
    // every block: its columns of every sorted row (see permute_scale_kernel); this row's own values are still in rowbuf
    const int n4 = (hi - lo) >> 2;
    for (int item = threadIdx.x; item < (P + dp.extra_rows) * n4; item += blockDim.x) {
      const int i = item / n4, c = item - i * n4;
      const int pair = i < P ? order[i] : 0;
      const float w = i < P ? order_w[i] : 1.f;
      const int tok = i < P ? pair / k : i - P;
      const float4 v = tok == n ? row4[c] : __ldcg(reinterpret_cast<const float4*>(out32 + (size_t)tok * D + lo) + c);
      store4<TO>(reinterpret_cast<TO*>(dp.a_sorted) + (size_t)i * D + lo + 4 * c, make_float4(w * v.x, w * v.y, w * v.z, w * v.w));
    }
  }
  }
}

// delta: what to add to x first (null: nothing), see DeltaSpec; the struct is read on the host.
// dispatch (optional, with a router): the sort and gather that a routed feed-forward would launch next, see DispatchArgs;
// *dispatched tells whether this call did them (it does when it runs the cluster kernel and the step is small enough).
JLX_API int jlx_add_rmsnorm(float* x, const DeltaSpec* delta, const float* gamma,
                            float eps, void* out, int out_dtype, float* out32, const int* row_index, int N, int D,
                            const float* w_router, int E, int k, int* topk_idx, float* topk_w, const DispatchArgs* dispatch,
                            int* dispatched, cudaStream_t stream) {
  if (dispatched) *dispatched = 0;
  JLX_REQUIRE(N >= 0 && D > 0, "add_rmsnorm: bad sizes N=%d D=%d", N, D);
  JLX_REQUIRE(eps > 0.f, "add_rmsnorm: eps must be positive");
  DeltaSpec ds = {};
  if (delta) ds = *delta;
  JLX_REQUIRE(ds.n >= 0 && ds.n <= DELTA_MAX_TERMS, "add_rmsnorm: %d terms to add; up to %d are supported", ds.n, DELTA_MAX_TERMS);
  bool aligned = true;
  int streams = 0;
  for (int q = 0; q < ds.n; ++q) {
    JLX_REQUIRE(ds.t[q].p && ds.t[q].splits >= 1 && (!ds.t[q].index || (ds.t[q].k >= 1 && ds.t[q].k <= 16)), "add_rmsnorm: bad term %d", q);
    aligned = aligned && (ds.t[q].stride & 3) == 0 && ((uintptr_t)ds.t[q].p & 15) == 0;
    streams += (ds.t[q].index ? ds.t[q].k : 1) * ds.t[q].splits;
  }
  JLX_REQUIRE(streams <= DELTA_MAX_STREAMS, "add_rmsnorm: a token would add %d rows (terms x rows x split-K partials); up to %d are supported",
              streams, DELTA_MAX_STREAMS);
  if (N == 0) return 0;
  const int row_in_smem = (size_t)D * 4 <= 64 * 1024;
  if (w_router) {
    JLX_REQUIRE(E >= 1 && E <= ROUTER_MAX_E, "router: %d experts; supported 1..%d", E, ROUTER_MAX_E);
    JLX_REQUIRE(k >= 1 && k <= E && k <= 16, "router: top-%d of %d experts; supported k in 1..min(E, 16)", k, E);
    JLX_REQUIRE(row_in_smem, "router fused with the norm needs width <= 16384 (got %d)", D);
    JLX_REQUIRE(topk_idx && topk_w, "router: outputs missing");
  }
  const size_t smem = row_in_smem ? (size_t)D * 4 : 0;
  // A few rows: a cluster of 8 blocks per row (all rows resident at once), bfloat16 output only.
  if (out_dtype == JLX_BF16 && !row_index && out && N <= 32 && (D & 3) == 0 && D >= 1024 && aligned &&
      (((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)out | (uintptr_t)out32) & 15) == 0) {
    const int C = NORM_CLUSTER;
    const int slice = ((D / 4 + C - 1) / C) * 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(N * C);
    // with a router the experts' rows are spread over 16 warps; without, a thread per 16 bytes of the slice is enough
    const int lean = ((slice / 4 + 31) / 32) * 32;
    cfg.blockDim = dim3(w_router ? 512 : (lean < 64 ? 64 : (lean > 256 ? 256 : lean)));
    cfg.dynamicSmemBytes = (size_t)slice * 4;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = C;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    DispatchArgs dp = {};
    if (w_router && dispatch && dispatch->counter && out32 && N <= DISPATCH_MAX_ROWS && N * k <= DISPATCH_MAX_PAIRS) {
      JLX_REQUIRE(dispatch->offsets && dispatch->sorted_pair && dispatch->sorted_pos && dispatch->a_sorted && dispatch->status &&
                  dispatch->extra_rows >= 0 && (dispatch->tile_rows == 0 || (dispatch->tile_list && dispatch->n_tiles)),
                  "add_rmsnorm: incomplete dispatch request");
      JLX_REQUIRE(((uintptr_t)dispatch->a_sorted & 15) == 0, "add_rmsnorm: the gathered rows must be 16-byte aligned");
      dp = *dispatch;
      if (dispatched) *dispatched = 1;
    }
    if (w_router)
      JLX_CUDA(cudaLaunchKernelEx(&cfg, add_rmsnorm_router_cluster_kernel<bf16, true>, x, ds, gamma, eps,
                                  (bf16*)out, out32, D, slice, w_router, E, k, topk_idx, topk_w, dp));
    else
      JLX_CUDA(cudaLaunchKernelEx(&cfg, add_rmsnorm_router_cluster_kernel<bf16, false>, x, ds, gamma, eps,
                                  (bf16*)out, out32, D, slice, w_router, E, k, topk_idx, topk_w, dp));
    JLX_LAUNCH_CHECK("add_rmsnorm (cluster)");
    return 0;
  }
  JLX_DISPATCH_DTYPE(out_dtype, TO, {
    if (smem > 48 * 1024) {
      static bool cfg = false;
      if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(add_rmsnorm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024)); cfg = true; }
    }
    // Wide rows with few tokens are latency-bound: more threads per row keep more loads in flight; with many
    // rows smaller blocks give more blocks per SM and cheaper barriers.  The block size fixes the order of the
    // sum of squares, so in 32-bit output (the exact path) it depends on the width alone: a row's result must
    // not change with the number of rows that happen to share its step.
    const bool exact = out_dtype == JLX_F32;
    const int threads = (D >= 2048 && (exact || N <= 256)) ? 1024 : 256;
    JLX_CUDA(jlx_launch_pdl(add_rmsnorm_kernel<TO>, dim3(N), dim3(threads), smem, stream, x, ds,
                            gamma, eps, (TO*)out, out32, row_index, D, row_in_smem, w_router, E, k, topk_idx, topk_w));
  });
  JLX_LAUNCH_CHECK("add_rmsnorm");
  return 0;
}

// out[i, f] = silu(gate) * up of row i (llama4/llama4_jax/model.py:1146-1151).  The input row holds 2F values,
// either [gate(0..F), up(0..F)] or, interleaved, blocks of [16 gate, 16 up]; it may come as `splits` float32
// split-K partials that are added first.
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, int splits, long long split_stride, TO* __restrict__ out,
                                int F, int interleaved) {
  JLX_TL(TL_SILU_MUL);
  const int i = blockIdx.x;
  const TI* g = gu + (size_t)i * 2 * F;
  for (int f = threadIdx.x; f < F; f += blockDim.x) {
    const int gi = interleaved ? ((f >> 4) << 5) + (f & 15) : f;
    const int ui = interleaved ? gi + 16 : F + f;
    float a = 0.f, b = 0.f;
    for (int z = 0; z < splits; ++z) {
      a += to_f32<TI>(g[(size_t)z * split_stride + gi]);
      b += to_f32<TI>(g[(size_t)z * split_stride + ui]);
    }
    const float s = a / (1.f + expf(-a));
    out[(size_t)i * F + f] = from_f32<TO>(s * b);
  }
}

// The common case in prompts: bfloat16 in and out, no partials; eight outputs per thread with 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int F, int interleaved) {
  JLX_TL(TL_SILU_MUL);
  const size_t i = blockIdx.x;
  const bf16* g = gu + i * 2 * F;
  for (int f0 = threadIdx.x * 8; f0 < F; f0 += blockDim.x * 8) {
    const int gi = interleaved ? ((f0 >> 4) << 5) + (f0 & 15) : f0;
    const int ui = interleaved ? gi + 16 : F + f0;
    const uint4 a = *reinterpret_cast<const uint4*>(g + gi), b = *reinterpret_cast<const uint4*>(g + ui);
    const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __bfloat1622float2(ap[j]), y = __bfloat1622float2(bp[j]);
      op[j] = __floats2bfloat162_rn(x.x / (1.f + expf(-x.x)) * y.x, x.y / (1.f + expf(-x.y)) * y.y);
    }
    *reinterpret_cast<uint4*>(out + i * F + f0) = o;
  }
}

JLX_API int jlx_silu_mul(const void* gu, int in_dtype, int splits, long long split_stride, void* out, int out_dtype,
                         int rows, int F, int interleaved, cudaStream_t stream) {
  JLX_REQUIRE(rows >= 0 && F > 0 && splits >= 1, "silu_mul: bad sizes rows=%d F=%d splits=%d", rows, F, splits);
  JLX_REQUIRE(!interleaved || F % 16 == 0, "silu_mul: the interleaved layout needs a width that is a multiple of 16");
  JLX_REQUIRE(splits == 1 || in_dtype == JLX_F32, "silu_mul: split-K partials are float32");
  if (rows == 0) return 0;
  if (in_dtype == JLX_BF16 && out_dtype == JLX_BF16 && splits == 1 && F % 16 == 0 && ((uintptr_t)gu & 15) == 0 &&
      ((uintptr_t)out & 15) == 0) {
    silu_mul_bf16x8_kernel<<<rows, 256, 0, stream>>>((const bf16*)gu, (bf16*)out, F, interleaved);
    JLX_LAUNCH_CHECK("silu_mul");
    return 0;
  }
  JLX_DISPATCH_DTYPE(in_dtype, TI, JLX_DISPATCH_DTYPE(out_dtype, TO,
      (silu_mul_kernel<TI, TO><<<rows, 256, 0, stream>>>((const TI*)gu, splits, split_stride, (TO*)out, F, interleaved))));
  JLX_LAUNCH_CHECK("silu_mul");
  return 0;
}
