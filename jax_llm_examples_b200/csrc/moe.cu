// Routing of tokens to experts: router scores, top-k, sigmoid weights, the expert-sorted row order,
// the scaled gather of rows into that order, and the sum of expert outputs back per token.
//
// Reference: llama4/llama4_jax/model.py:958-972 (scores = h W_router in 32-bit, top-k on the raw
// scores, sigmoid of the chosen), model.py:1049-1073 (sort pairs by expert, gather rows, scale the
// INPUT row by its router weight, group sizes), model.py:1109-1111 (unsort, sum over k),
// model.py:1139 (add the shared expert).  Ties go to the lower expert index (jax.lax.top_k order).
#include "common.cuh"
#include "expert_sort.cuh"

#define ROUTER_MAX_E 256
#define ROUTER_MAX_K 16

// One block per token.  Warp w computes the scores of experts w, w + nwarp, ...: a fixed order of
// the D products per (token, expert), so a token's routing does not depend on the batch.
__global__ void router_kernel(const float* __restrict__ h, const float* __restrict__ w_router, int* __restrict__ topk_idx,
                              float* __restrict__ topk_w, float* __restrict__ scores_out, int D, int E, int k) {
  JLX_TL(TL_ROUTER);
  __shared__ float scores[ROUTER_MAX_E];
  const int n = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const float* hr = h + (size_t)n * D;
  for (int e = warp; e < E; e += nwarp) {
    const float* wr = w_router + (size_t)e * D;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) s = fmaf(hr[d], wr[d], s);
    s = warp_sum(s);
    if (lane == 0) scores[e] = s;
  }
  __syncthreads();
  if (scores_out)
    for (int e = threadIdx.x; e < E; e += blockDim.x) scores_out[(size_t)n * E + e] = scores[e];
  if (threadIdx.x == 0) {
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = 0.f;
      for (int e = 0; e < E; ++e) {
        const float v = scores[e];
        if (isnan(v)) continue;
        if (best < 0 || v > bv) {  // strict: the lower index wins a tie
          best = e;
          bv = v;
        }
      }
      if (best < 0) best = j;  // all NaN: still a valid expert index
      topk_idx[(size_t)n * k + j] = best;
      topk_w[(size_t)n * k + j] = 1.f / (1.f + expf(-bv));
      scores[best] = NAN;  // taken
    }
  }
}

// Many tokens (prompt portions): a block takes ROWS tokens, so that a router row that a warp fetches serves all
// of them (one block per token would fetch all E * D weights once per token).  Warp w computes the scores of
// EPW experts at a time for all the block's rows: per step of 128 columns it loads each row's four values once
// and each expert's four weights once.  The order of the D products of a (token, expert) pair is fixed by the
// column alone, so a token's routing does not depend on which tokens share its block.  D % 4 == 0.
#define ROUTER_ROWS 8
template <int EPW>
__global__ void __launch_bounds__(256, 2)
router_rows_kernel(const float* __restrict__ h, const float* __restrict__ w_router, int* __restrict__ topk_idx,
                   float* __restrict__ topk_w, int N, int D, int E, int k) {
  JLX_TL(TL_ROUTER);
  __shared__ float scores[ROUTER_ROWS][ROUTER_MAX_E];
  pdl_launch_dependents();
  pdl_wait();
  const int n0 = blockIdx.x * ROUTER_ROWS;
  const int rows = min(ROUTER_ROWS, N - n0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int e0 = warp * EPW; e0 < E; e0 += nwarp * EPW) {
    float acc[EPW][ROUTER_ROWS];
#pragma unroll
    for (int i = 0; i < EPW; ++i)
#pragma unroll
      for (int r = 0; r < ROUTER_ROWS; ++r) acc[i][r] = 0.f;
    // two steps' loads are in flight together: the walk waits on memory, not on arithmetic
#pragma unroll 2
    for (int d = lane * 4; d < D; d += 128) {
      float4 xv[ROUTER_ROWS], wv[EPW];
#pragma unroll
      for (int r = 0; r < ROUTER_ROWS; ++r)
        xv[r] = r < rows ? *reinterpret_cast<const float4*>(h + (size_t)(n0 + r) * D + d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < EPW; ++i)
        wv[i] = e0 + i < E ? *reinterpret_cast<const float4*>(w_router + (size_t)(e0 + i) * D + d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < EPW; ++i)
#pragma unroll
        for (int r = 0; r < ROUTER_ROWS; ++r)
          acc[i][r] = fmaf(xv[r].x, wv[i].x, fmaf(xv[r].y, wv[i].y, fmaf(xv[r].z, wv[i].z, fmaf(xv[r].w, wv[i].w, acc[i][r]))));
    }
#pragma unroll
    for (int i = 0; i < EPW; ++i)
#pragma unroll
      for (int r = 0; r < ROUTER_ROWS; ++r) {
        const float s = warp_sum(acc[i][r]);
        if (lane == 0 && e0 + i < E) scores[r][e0 + i] = s;
      }
  }
  __syncthreads();
  if (threadIdx.x < rows) {
    float* sc = scores[threadIdx.x];
    const size_t n = (size_t)n0 + threadIdx.x;
    for (int j = 0; j < k; ++j) {
      int best = -1;
      float bv = 0.f;
      for (int e = 0; e < E; ++e) {
        const float v = sc[e];
        if (isnan(v)) continue;
        if (best < 0 || v > bv) {  // strict: the lower index wins a tie
          best = e;
          bv = v;
        }
      }
      if (best < 0) best = j;  // all NaN: still a valid expert index
      topk_idx[n * k + j] = best;
      topk_w[n * k + j] = 1.f / (1.f + expf(-bv));
      sc[best] = NAN;  // taken
    }
  }
}

// many_rows: the kernel that shares router rows among eight tokens (another order of the sums than the
// one-token kernel's: a caller whose results must not depend on the batch uses one of the two throughout).
JLX_API int jlx_router(const float* h, const float* w_router, int* topk_idx, float* topk_w, float* scores_out, int N,
                       int D, int E, int k, int many_rows, cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0, "router: bad sizes N=%d D=%d", N, D);
  JLX_REQUIRE(E >= 1 && E <= ROUTER_MAX_E, "router: %d experts; supported 1..%d", E, ROUTER_MAX_E);
  JLX_REQUIRE(k >= 1 && k <= E && k <= ROUTER_MAX_K, "router: top-%d of %d experts; supported k in 1..min(E, %d)", k, E, ROUTER_MAX_K);
  if (N == 0) return 0;
  if (many_rows && !scores_out && D % 4 == 0 && (((uintptr_t)h | (uintptr_t)w_router) & 15) == 0) {
    const dim3 grid((N + ROUTER_ROWS - 1) / ROUTER_ROWS);
    if (E <= 16) JLX_CUDA(jlx_launch_pdl(router_rows_kernel<2>, grid, dim3(256), 0, stream, h, w_router, topk_idx, topk_w, N, D, E, k));
    else JLX_CUDA(jlx_launch_pdl(router_rows_kernel<4>, grid, dim3(256), 0, stream, h, w_router, topk_idx, topk_w, N, D, E, k));
    JLX_LAUNCH_CHECK("router_rows");
    return 0;
  }
  router_kernel<<<N, 256, 0, stream>>>(h, w_router, topk_idx, topk_w, scores_out, D, E, k);
  JLX_LAUNCH_CHECK("router");
  return 0;
}

// Counting sort of the P = N * k (token, choice) pairs by expert, stable in pair order.  One block;
// warp w owns experts w, w + nwarp, ...  Writes offsets[E + 1], sorted_pair[P] (pair id at each sorted
// row) and sorted_pos[P] (sorted row of each pair).
// With extra_rows > 0 one more group is appended after the experts (offsets has E + 2 entries): rows
// [P, P + extra_rows), used for a shared expert that takes every token.
// With tile_rows > 0 it also lists the row tiles of the grouped products that follow: tile_list[t] =
// (group, first row) for every tile of tile_rows rows that holds at least one row, and n_tiles[0] = how many,
// so that a product's blocks find their work with one load instead of a walk over the offsets.
__global__ void expert_sort_kernel(const int* __restrict__ topk_idx, int* __restrict__ offsets,
                                   int* __restrict__ sorted_pair, int* __restrict__ sorted_pos, int P, int E, int extra_rows,
                                   int tile_rows, int* __restrict__ tile_list, int* __restrict__ n_tiles, int* status,
                                   int in_smem) {
  JLX_TL(TL_SORT);
  __shared__ int counts[ROUTER_MAX_E + 1];
  extern __shared__ int staged[];  // the choices, when `in_smem`: both passes below walk them once per expert
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  // One block, once per layer: it rehearses (see jlx_rehearses): every load replaced by "no choice", every store left out.
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const bool real = pass == 1;
    if (real) pdl_wait();
    if (in_smem) {
      for (int i = threadIdx.x; i < P; i += blockDim.x) staged[i] = real ? topk_idx[i] : -1;
      __syncthreads();
    }
    if (real) JLX_TL_MARK(0);
    const int* choice = in_smem ? staged : topk_idx;
    for (int e = warp; e < E; e += nwarp) {
      int c = 0;
      for (int base = 0; base < P; base += 32) {
        const int i = base + lane;
        const int v = i < P && (real || in_smem) ? choice[i] : -1;
        c += __popc(__ballot_sync(0xffffffffu, v == e));
      }
      if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    if (warp == 0) {
      expert_offsets_and_tiles(counts, E, P, extra_rows, tile_rows, offsets, tile_list, n_tiles, status, real);
      if (real) JLX_TL_MARK(1);
    }
    __syncthreads();
    for (int e = warp; e < E; e += nwarp) {
      int at = counts[e];
      for (int base = 0; base < P; base += 32) {
        const int i = base + lane;
        const int v = i < P && (real || in_smem) ? choice[i] : -1;
        const unsigned mask = __ballot_sync(0xffffffffu, v == e);
        if (v == e) {
          const int dst = at + __popc(mask & ((1u << lane) - 1u));
          sorted_pair[dst] = i;
          sorted_pos[i] = dst;
        }
        at += __popc(mask);
      }
    }
    __syncthreads();
  }
}

// tile_list: int [(ceil((P + extra_rows) / tile_rows) + groups) * 2]; n_tiles: int [1]; both unused if tile_rows == 0.
JLX_API int jlx_expert_sort(const int* topk_idx, int* offsets, int* sorted_pair, int* sorted_pos, int P, int E,
                            int extra_rows, int tile_rows, int* tile_list, int* n_tiles, int* status, cudaStream_t stream) {
  JLX_REQUIRE(tile_rows == 0 || (tile_list && n_tiles), "expert_sort: tile list outputs missing");
  JLX_REQUIRE(P >= 0 && E >= 1 && E <= ROUTER_MAX_E && extra_rows >= 0, "expert_sort: bad sizes P=%d E=%d", P, E);
  const int warps = E < 32 ? E : 32;
  const int in_smem = (size_t)P * sizeof(int) <= 40 * 1024;
  JLX_CUDA(jlx_launch_pdl(expert_sort_kernel, dim3(1), dim3(warps * 32), in_smem ? (size_t)P * sizeof(int) : 0, stream, topk_idx,
                          offsets, sorted_pair, sorted_pos, P, E, extra_rows, tile_rows, tile_list, n_tiles, status, in_smem));
  return 0;
}

// a_sorted[i, :] = weight(pair) * h[token(pair), :]  with pair = sorted_pair[i], token = pair / k;
// rows i >= P (the appended group of a shared expert) are the unscaled rows h[i - P].
template <typename T>
__global__ void permute_scale_kernel(const float* __restrict__ h, const int* __restrict__ sorted_pair,
                                     const float* __restrict__ topk_w, T* __restrict__ a_sorted, int D, int k, int P) {
  JLX_TL(TL_PERMUTE);
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int pair = i < P ? sorted_pair[i] : 0;
  const float w = i < P ? topk_w[pair] : 1.f;
  const float* src = h + (size_t)(i < P ? pair / k : i - P) * D;
  T* dst = a_sorted + (size_t)i * D;
  if ((D & 3) == 0) {  // rows are 16-byte aligned: four elements per thread and access
    for (int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4; d < D; d += gridDim.y * blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(src + d);
      dst[d] = from_f32<T>(w * v.x);
      dst[d + 1] = from_f32<T>(w * v.y);
      dst[d + 2] = from_f32<T>(w * v.z);
      dst[d + 3] = from_f32<T>(w * v.w);
    }
    return;
  }
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) dst[d] = from_f32<T>(w * src[d]);
}

JLX_API int jlx_permute_scale(const float* h, const int* sorted_pair, const float* topk_w, void* a_sorted, int dtype,
                              int P, int extra_rows, int D, int k, cudaStream_t stream) {
  JLX_REQUIRE(P >= 0 && D > 0 && k >= 1 && extra_rows >= 0, "permute_scale: bad sizes");
  const int rows = P + extra_rows;
  if (rows == 0) return 0;
  // few rows: spread each row over several blocks
  const int ysplit = rows >= 512 ? 1 : (D + 1023) / 1024;  // four columns per thread: 1024 columns per block
  JLX_DISPATCH_DTYPE(dtype, T, { JLX_CUDA(jlx_launch_pdl(permute_scale_kernel<T>, dim3(rows, ysplit), dim3(256), 0, stream, h, sorted_pair, topk_w, (T*)a_sorted, D, k, P)); });
  return 0;
}

// delta[n, :] = sum_j y[sorted_pos[n * k + j], :]  (+ y[extra_base + n, :] if extra_base >= 0: the appended
// shared-expert group)  (+ shared[n, :]), where y and shared may be split-K partials [z][rows][D] that are
// added first, z ascending; j ascending: a fixed order.
__global__ void moe_combine_kernel(const float* __restrict__ y, int y_splits, long long y_stride, int extra_base,
                                   const float* __restrict__ shared, int splits, long long split_stride,
                                   const int* __restrict__ sorted_pos, float* __restrict__ delta, int D, int k) {
  JLX_TL(TL_MOE_COMBINE);
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  if ((D & 3) == 0 && (y_stride & 3) == 0 && (split_stride & 3) == 0) {  // the same sums, four columns at a time
    for (int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4; d < D; d += gridDim.y * blockDim.x * 4) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      auto add = [&s](const float* p) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      };
      if (shared)
        for (int z = 0; z < splits; ++z) add(shared + (size_t)z * split_stride + (size_t)n * D + d);
      if (extra_base >= 0)
        for (int z = 0; z < y_splits; ++z) add(y + (size_t)z * y_stride + (size_t)(extra_base + n) * D + d);
      for (int j = 0; j < k; ++j) {
        const size_t row = (size_t)sorted_pos[(size_t)n * k + j] * D + d;
        for (int z = 0; z < y_splits; ++z) add(y + (size_t)z * y_stride + row);
      }
      *reinterpret_cast<float4*>(delta + (size_t)n * D + d) = s;
    }
    return;
  }
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    float s = 0.f;
    if (shared)
      for (int z = 0; z < splits; ++z) s += shared[(size_t)z * split_stride + (size_t)n * D + d];
    if (extra_base >= 0)
      for (int z = 0; z < y_splits; ++z) s += y[(size_t)z * y_stride + (size_t)(extra_base + n) * D + d];
    for (int j = 0; j < k; ++j) {
      const size_t row = (size_t)sorted_pos[(size_t)n * k + j] * D + d;
      for (int z = 0; z < y_splits; ++z) s += y[(size_t)z * y_stride + row];
    }
    delta[(size_t)n * D + d] = s;
  }
}

JLX_API int jlx_moe_combine(const float* y, int y_splits, long long y_stride, int extra_base, const float* shared,
                            int splits, long long split_stride, const int* sorted_pos, float* delta, int N, int D, int k,
                            cudaStream_t stream) {
  JLX_REQUIRE(N >= 0 && D > 0 && k >= 1 && splits >= 1 && y_splits >= 1, "moe_combine: bad sizes");
  if (N == 0) return 0;
  const int ysplit = N >= 512 ? 1 : (D + 1023) / 1024;  // four columns per thread: 1024 columns per block
  JLX_CUDA(jlx_launch_pdl(moe_combine_kernel, dim3(N, ysplit), dim3(256), 0, stream, y, y_splits, y_stride, extra_base, shared,
                          splits, split_stride, sorted_pos, delta, D, k));
  return 0;
}
