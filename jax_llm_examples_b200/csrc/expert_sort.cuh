// The part of the experts' counting sort that one warp does, shared by the sort kernel (moe.cu) and by the norm +
// router kernel that sorts a decode step's few pairs itself (elementwise.cu).
#pragma once
#include "common.cuh"

// Called by all 32 lanes of one warp.  counts[0..E) in shared memory holds the pairs per expert and becomes the
// exclusive prefix sums (counts[E] = P).  With `real` the sums go to offsets[0..E] (and offsets[E + 1] = P +
// extra_rows when a group of extra_rows rows is appended after the experts), and with tile_rows > 0 the row tiles
// of the grouped products that follow are listed: tile_list[t] = (group, first row) for every tile of tile_rows rows
// that holds at least one row, n_tiles[0] = how many.  Prefix sums 32 experts at a time by shuffles (a single thread
// walking the experts and then the tiles was a third of the sort kernel's time in a decode step).
__device__ __forceinline__ void expert_offsets_and_tiles(int* counts, int E, int P, int extra_rows, int tile_rows,
                                                         int* __restrict__ offsets, int* __restrict__ tile_list,
                                                         int* __restrict__ n_tiles, int* status, bool real) {
  const int lane = threadIdx.x & 31;
  int run = 0;
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    const int c = e < E ? counts[e] : 0;
    int incl = c;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    __syncwarp();
    if (e < E) {
      counts[e] = run + incl - c;
      if (real) offsets[e] = run + incl - c;
    }
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) {
    counts[E] = run;
    if (real) {
      offsets[E] = run;
      if (extra_rows > 0) offsets[E + 1] = run + extra_rows;
      if (run != P) atomicOr(status, JLX_STATUS_BAD_EXPERT);
    }
  }
  __syncwarp();
  if (tile_rows > 0) {
    // the tiles of group g follow those of the groups before it: the same scan over the groups' tile counts
    const int groups = extra_rows > 0 ? E + 1 : E;
    int t_run = 0;
    for (int g0 = 0; g0 < groups; g0 += 32) {
      const int g = g0 + lane;
      // (a lane beyond the last group has no rows: lo = hi = 0, so that it lists nothing below)
      const int lo = g < groups ? counts[g] : 0, hi = g >= groups ? 0 : (g < E ? counts[g + 1] : run + extra_rows);
      const int tiles = (hi - lo + tile_rows - 1) / tile_rows;
      int incl = tiles;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      if (real) {
        int t = t_run + incl - tiles;
        for (int r = lo; r < hi; r += tile_rows, ++t) {
          tile_list[2 * t] = g;
          tile_list[2 * t + 1] = r;
        }
      }
      t_run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (real && lane == 0) n_tiles[0] = t_run;
  }
}
