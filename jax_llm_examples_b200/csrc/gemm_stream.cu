// Weight-streaming GEMM for sm_100a: C = A * W^T in bfloat16 with 32-bit accumulation, on the
// 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory), operands staged by TMA.
//
// It is built for the products whose cost is reading the weights once: every product of a decode
// step (few token rows), and the routed experts at any batch (llama4/llama4_jax/model.py:975-996 is
// the reference's ragged product; its decode kernel, decode_ragged_dot.py:26-116, is the TPU
// counterpart).  The operands are swapped with respect to the usual tiling: a tile of 128 weight rows
// is the MMA's M side (one row per tensor-memory lane) and the token rows are its N side (BT columns,
// 16..256), so that a handful of tokens still fills the instruction.  K advances in stages of 64
// elements (one 128-byte swizzled row per operand row).
//
//   A: [rows, K] row-major (tokens).  W: [E * N, K] row-major ([out, in] weights of E groups).
//   C: [rows, N].  Grouped: token rows [offsets[e], offsets[e+1]) use weight rows [e*N, (e+1)*N).
//   split-K: blockIdx.z takes a K range and writes a 32-bit partial [z][rows][N]; a second kernel
//   adds the partials in a fixed order.
//
// One block = one (weight tile, token tile, K range).  Warp 0 issues TMA loads, warp 1 allocates tensor
// memory and issues the MMAs, warps 2..9 read the accumulator back (two per 32-lane quarter) and
// store it transposed (for a fixed token, 32 consecutive outputs per warp: coalesced).
// Every wait on a barrier is bounded; on a timeout the block raises JLX_STATUS_WAIT_TIMEOUT, drains its
// own copies, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "mbarrier.cuh"

#define WN 128          // weight rows per tile (MMA M)
#define BK 64           // K elements per stage (128 bytes of bfloat16)
#define UMMA_K 16
#define NTHREADS 320     // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue (two per quarter of the tensor-memory lanes)
#define WAIT_LIMIT JLX_WAIT_LIMIT

// ------------------------------------------------------------------------------------ PTX wrappers
// Fetches a tensor map's descriptor ahead of its first use by a copy.
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


// ---- wrappers for a pair of blocks (a cluster of two) that share one MMA: cta_group::2
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {  // the same location in another block of the cluster
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The copy lands in this block's shared memory; its bytes are counted on a barrier that may lie in the pair's other block.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives, once the MMAs issued so far are complete, on the barrier at this offset in both blocks of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the
// 128-byte swizzle (as TMA writes it): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)0 << 16;                   // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                   // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                   // layout: 128-byte swizzle
  return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = bt.
__host__ __device__ constexpr uint32_t make_idesc(int bt, int m = WN) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bt >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------ kernel
struct StreamArgs {
  int N;                 // outputs per group
  int K;
  int rows;              // token rows in A (upper bound of offsets[E])
  const int* offsets;    // null: one group over all rows
  int E;
  const int* tile_list;  // optional, with offsets: (group, first row) of every row tile that has rows
  const int* n_tiles;    // ... and how many there are
  void* out;             // [rows, N] (bf16 or f32), or partials [splits][rows][N] f32 when splits > 1
  int out_is_f32;
  int silu;              // 1: rows come in blocks of [16 gate, 16 up]; out[m, j] = silu(gate_j) * up_j, [rows, N / 2]
  int splits;
  int k_per_split;       // multiple of BK
  int offsets_settled;   // grouped: offsets and tile list were complete before the kernel in front of this one began its work
  int* status;
};

// Epilogue of warps 2..9: the accumulator (tensor-memory lanes = weight rows n0.., columns = token rows row_lo..)
// goes to global memory transposed, optionally through SiLU(gate) * up.
template <int BT, int WT>
__device__ __forceinline__ void stream_epilogue(const StreamArgs& args, int warp, int lane, uint32_t bar_acc, volatile int* failed,
                                                uint32_t tmem_acc, int n0, int row_lo, int row_hi) {
  const int quarter = warp & 3;         // tensor-memory lanes [32 * quarter, 32 * quarter + 32): fixed by the warp's number
  const int half = (warp - 2) >> 2;     // the two warps of a quarter take alternate blocks of 16 token columns
  pdl_wait();  // the output buffer may still be read by a predecessor
  bool ok = mbar_wait_long(bar_acc, 0);
  if (*(volatile int*)failed) ok = false;
  ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below need the whole warp
  if (ok) {
    tc_fence_after();
    const size_t split_off = args.splits > 1 ? (size_t)blockIdx.z * args.rows * args.N : 0;
#pragma unroll 1
    for (int w = 0; w < WT; ++w) {
      const int nb = n0 + w * WN + quarter * 32;  // first weight row of this warp in tile w
      const int n = nb + lane;
      const bool n_ok = n < args.N;
      if (nb >= args.N) break;  // uniform across the warp
#pragma unroll 1
      for (int c0 = half * 16; c0 < BT; c0 += 32) {
        if (row_lo + c0 >= row_hi) break;  // uniform across the warp
        uint32_t r[16];
        tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + w * BT + c0, r);
        tmem_ld_wait();
        if (args.silu) {
          // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows of the same 32-row block.  Of two
          // token columns the lower lanes finish the even one and the upper lanes the odd one: one exchange
          // gives the lower lanes the even column's up values and the upper lanes the odd column's gates.
          const size_t half_n = (size_t)(args.N >> 1);
          const bool upper = lane >= 16;
          const size_t col = (size_t)(nb >> 1) + (lane & 15);
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float mine = __uint_as_float(upper ? r[j + 1] : r[j]);   // gate (lower) or up (upper) of my column
            const float send = __uint_as_float(upper ? r[j] : r[j + 1]);
            const float got = __shfl_xor_sync(0xffffffffu, send, 16);
            const float gate = upper ? got : mine, up = upper ? mine : got;
            const int m = row_lo + c0 + j + (upper ? 1 : 0);
            if (m < row_hi) {  // N % 32 == 0: a block of 32 weight rows that starts below N lies wholly below it
              const float act = __fdividef(gate, 1.f + __expf(-gate)) * up;
              if (args.out_is_f32) ((float*)args.out)[(size_t)m * half_n + col] = act;
              else ((bf16*)args.out)[(size_t)m * half_n + col] = __float2bfloat16_rn(act);
            }
          }
        } else if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = row_lo + c0 + j;
            if (m < row_hi) {
              if (args.out_is_f32 || args.splits > 1)
                ((float*)args.out)[split_off + (size_t)m * args.N + n] = __uint_as_float(r[j]);
              else
                ((bf16*)args.out)[(size_t)m * args.N + n] = __float2bfloat16_rn(__uint_as_float(r[j]));
            }
          }
        }
      }
    }
  } else if (lane == 0) {
    atomicOr(args.status, JLX_STATUS_WAIT_TIMEOUT);
  }
}

// WT: weight tiles of 128 rows per block.  With many token rows per group the token tile is the larger part of
// a stage; two weight tiles (two accumulators in tensor memory) per token tile halve its traffic.
// SW, SA: stages of the weight ring and of the token ring.  Weights come from HBM and need many bytes in
// flight; token tiles are read again by every weight tile of the group, come from L2 and need fewer.
template <int BT, int SW, int SA, int WT>
__global__ void __launch_bounds__(NTHREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const StreamArgs args) {
  JLX_TL(TL_GEMM);
  constexpr uint32_t W_TILE = WN * BK * 2, W_BYTES = WT * W_TILE, A_BYTES = BT * BK * 2;
  constexpr uint32_t TMEM_NEED = WT * BT;  // allocations are powers of two from 32 columns
  constexpr uint32_t TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_w = (smem_u32(smem_raw) + 1023u) & ~1023u, smem_a = smem_w + SW * W_BYTES;
  __shared__ __align__(8) uint64_t bars[2 * SW + 2 * SA + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A grouped product lets its successor start only after its own wait for its predecessor (below): the successor
  // then knows, before its own wait, that everything older than this product is complete.  That is what
  // `offsets_settled` of the NEXT grouped product over the same offsets (an expert layer's down product after its
  // gate/up product) rests on: it reads the offsets and the tile list at once and asks for its first weight tiles
  // while this product still runs, as a dense product does.
  if (!args.offsets) pdl_launch_dependents();
  if (threadIdx.x == 0) {
    prefetch_map(&map_w);
    prefetch_map(&map_a);
  }

  // ---- which tile.  The group offsets are written by an earlier kernel of the stream: wait for it first, unless
  // they are known to be settled (then they are read past L1, which may hold lines of an earlier step).
  int row_lo, row_hi, group = 0;
  const bool settled = args.offsets && args.offsets_settled;
  if (args.offsets) {
    if (!settled) {
      pdl_wait();
      pdl_launch_dependents();
    }
    int t = blockIdx.y, found = 0;
    if (args.tile_list) {
      if (t >= __ldcg(args.n_tiles)) return;
      group = __ldcg(args.tile_list + 2 * t);
      row_lo = __ldcg(args.tile_list + 2 * t + 1);
      row_hi = __ldcg(args.offsets + group + 1);
      found = 1;
    }
    for (int e = 0; !found && e < args.E; ++e) {
      const int lo = __ldcg(args.offsets + e), hi = __ldcg(args.offsets + e + 1);
      const int tiles = (hi - lo + BT - 1) / BT;
      if (t < tiles) { row_lo = lo + t * BT; row_hi = hi; group = e; found = 1; break; }
      t -= tiles;
    }
    if (!found) return;
  } else {
    row_lo = blockIdx.y * BT;
    row_hi = args.rows;
    if (row_lo >= row_hi) return;
  }
  const int n0 = blockIdx.x * (WN * WT);
  const int k_begin = blockIdx.z * args.k_per_split;
  const int k_end = min(args.K, k_begin + args.k_per_split);
  const int k_iters = (k_end - k_begin + BK - 1) / BK;

  const uint32_t w_full = smem_u32(&bars[0]), w_empty = w_full + 8 * SW, a_full = w_empty + 8 * SW, a_empty = a_full + 8 * SA,
                 bar_acc = a_empty + 8 * SA;
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * SW + 2 * SA + 1; ++s) mbar_init(w_full + 8 * s, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The weights depend on no earlier kernel: the first stages' weight tiles are requested before the
      // wait for the predecessor, whose tail they overlap; the token tiles follow after it.
      auto load_w = [&](int it) {
        const int s = it % SW;
        mbar_expect_tx(w_full + 8 * s, W_BYTES);
#pragma unroll
        for (int w = 0; w < WT; ++w)  // rows beyond this group's N belong to the next group or to nobody: never stored
          tma_load_2d(smem_w + s * W_BYTES + w * W_TILE, &map_w, k_begin + it * BK, group * args.N + n0 + w * WN, w_full + 8 * s);
      };
      auto load_a = [&](int it) {
        const int s = it % SA;
        mbar_expect_tx(a_full + 8 * s, A_BYTES);
        tma_load_2d(smem_a + s * A_BYTES, &map_a, k_begin + it * BK, row_lo, a_full + 8 * s);
      };
      int iw = 0, ia = 0;
      for (; iw < k_iters && iw < SW; ++iw) load_w(iw);
      pdl_wait();
      if (settled) pdl_launch_dependents();  // (see the top of the kernel)
      for (; ia < k_iters && ia < SA; ++ia) load_a(ia);
      // both rings advance as their stages come free; neither waits for the other
      uint32_t idle = 0;
      bool ok = true;
      while ((iw < k_iters || ia < k_iters) && ok) {
        bool moved = false;
        if (iw < k_iters && mbar_try_wait(w_empty + 8 * (iw % SW), ((iw / SW) & 1) ^ 1)) { load_w(iw); ++iw; moved = true; }
        if (ia < k_iters && mbar_try_wait(a_empty + 8 * (ia % SA), ((ia / SA) & 1) ^ 1)) { load_a(ia); ++ia; moved = true; }
        if (moved) idle = 0;
        else if (++idle >= WAIT_LIMIT || *(volatile int*)&failed) ok = false;
      }
      if (!ok) {
        atomicOr(args.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
        // let this block's copies in flight land before its shared memory is given up
        for (int it = max(0, iw - SW); it < iw; ++it) mbar_wait(w_full + 8 * (it % SW), (it / SW) & 1);
        for (int it = max(0, ia - SA); it < ia; ++it) mbar_wait(a_full + 8 * (it % SA), (it / SA) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BT);
      bool ok = true;
      for (int it = 0; it < k_iters; ++it) {
        const int sw = it % SW, sa = it % SA;
        ok = mbar_wait(w_full + 8 * sw, (it / SW) & 1) && mbar_wait(a_full + 8 * sa, (it / SA) & 1);
        if (!ok || *(volatile int*)&failed) { ok = false; break; }
        tc_fence_after();
        const uint32_t w_addr = smem_w + sw * W_BYTES;
        const uint64_t adesc = smem_desc_sw128(smem_a + sa * A_BYTES);
#pragma unroll
        for (int w = 0; w < WT; ++w) {
          const uint64_t wdesc = smem_desc_sw128(w_addr + w * W_TILE);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 16 elements = 32 bytes further along K inside the swizzled row: +2 in the address field
            umma_bf16(tmem_acc + w * BT, wdesc + 2 * k, adesc + 2 * k, idesc, (it | k) != 0);
          }
        }
        umma_commit(w_empty + 8 * sw);  // frees the stages when these MMAs have read them
        umma_commit(a_empty + 8 * sa);
      }
      if (ok) {
        umma_commit(bar_acc);  // accumulator complete
      } else {
        atomicOr(args.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
      }
    }
  } else {
    stream_epilogue<BT, WT>(args, warp, lane, bar_acc, &failed, tmem_acc, n0, row_lo, row_hi);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_acc, TMEM_COLS);
  }
}

// The same product by a pair of blocks on neighbouring SMs (a cluster of two) that share each MMA
// (cta_group::2, M = 256): block r of the pair stages its own 128 weight rows and half of the token tile, the
// MMA reads both halves, and each block's tensor memory receives the accumulator of its own weight rows.  A
// token tile is so fetched once per 256 weight rows and a stage is a quarter smaller, which buys a fourth stage
// where the one-block kernel has three.  Block 0 issues the MMAs; the copies of both blocks count on block 0's
// `full` barriers, and its commits arrive on the `empty` barriers of both.
template <int BT, int ST>
__global__ void __launch_bounds__(NTHREADS)
gemm_stream_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const StreamArgs args) {
  JLX_TL(TL_GEMM_PAIR);
  constexpr uint32_t W_BYTES = WN * BK * 2, A_HALF = (BT / 2) * BK * 2;
  constexpr uint32_t TMEM_COLS = BT <= 32 ? 32 : BT <= 64 ? 64 : BT <= 128 ? 128 : 256;
  static_assert(BT % 16 == 0 && A_HALF % 1024 == 0, "half a token tile must be whole 8-row swizzle groups");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_w = (smem_u32(smem_raw) + 1023u) & ~1023u, smem_a = smem_w + ST * W_BYTES;
  __shared__ __align__(8) uint64_t bars[2 * ST + 1];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();  // 0 or 1: blockIdx.x is even or odd
  if (!args.offsets) pdl_launch_dependents();  // grouped: after the wait, as in gemm_stream_kernel
  if (threadIdx.x == 0) {
    prefetch_map(&map_w);
    prefetch_map(&map_a);
  }

  // ---- which tile (both blocks of a pair have the same blockIdx.y and decide alike)
  int row_lo, row_hi, group = 0;
  if (args.offsets) {
    pdl_wait();
    pdl_launch_dependents();
    int t = blockIdx.y, found = 0;
    if (args.tile_list) {
      if (t >= args.n_tiles[0]) return;
      group = args.tile_list[2 * t];
      row_lo = args.tile_list[2 * t + 1];
      row_hi = args.offsets[group + 1];
      found = 1;
    }
    for (int e = 0; !found && e < args.E; ++e) {
      const int lo = args.offsets[e], hi = args.offsets[e + 1];
      const int tiles = (hi - lo + BT - 1) / BT;
      if (t < tiles) { row_lo = lo + t * BT; row_hi = hi; group = e; found = 1; break; }
      t -= tiles;
    }
    if (!found) return;
  } else {
    row_lo = blockIdx.y * BT;
    row_hi = args.rows;
    if (row_lo >= row_hi) return;
  }
  const int n0 = blockIdx.x * WN;  // this block's weight rows
  const int k_begin = blockIdx.z * args.k_per_split;
  const int k_end = min(args.K, k_begin + args.k_per_split);
  const int k_iters = (k_end - k_begin + BK - 1) / BK;

  const uint32_t bar_full = smem_u32(&bars[0]), bar_empty = bar_full + 8 * ST, bar_acc = bar_empty + 8 * ST;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * ST + 1; ++i) mbar_init(bar_full + 8 * i, 1);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_slot), TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();  // both blocks' barriers exist before either block's copies or commits reach them
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (one per block)
    if (lane == 0) {
      const uint32_t full0 = map_to_rank(bar_full, 0);  // block 0's `full` barriers
      const int a_row = row_lo + (int)rank * (BT / 2);
      auto load_w = [&](int it) {
        const int s = it % ST;
        if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * (W_BYTES + A_HALF));  // the bytes of both blocks
        tma_load_2d_pair(smem_w + s * W_BYTES, &map_w, k_begin + it * BK, group * args.N + n0, full0 + 8 * s);
      };
      auto load_a = [&](int it) {
        const int s = it % ST;
        tma_load_2d_pair(smem_a + s * A_HALF, &map_a, k_begin + it * BK, a_row, full0 + 8 * s);
      };
      // the weights depend on no earlier kernel: their first stages are requested before the wait for it
      const int early = k_iters < ST ? k_iters : ST;
      for (int it = 0; it < early; ++it) load_w(it);
      pdl_wait();
      for (int it = 0; it < early; ++it) load_a(it);
      int issued = early;
      bool ok = true;
      for (int it = early; it < k_iters && ok; ++it) {
        const int s = it % ST;
        ok = mbar_wait(bar_empty + 8 * s, ((it / ST) & 1) ^ 1);
        if (!ok || *(volatile int*)&failed) { ok = false; break; }
        load_w(it);
        load_a(it);
        issued = it + 1;
      }
      if (!ok) {
        atomicOr(args.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
        // block 0 can see its copies land; block 1's are counted there too, so it waits for the accumulator
        // barrier or for its own time limit in the epilogue warps before it leaves
        if (rank == 0)
          for (int it = max(0, issued - ST); it < issued; ++it) mbar_wait(bar_full + 8 * (it % ST), (it / ST) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (block 0 only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(BT, 2 * WN);
      bool ok = true;
      for (int it = 0; it < k_iters; ++it) {
        const int s = it % ST;
        ok = mbar_wait(bar_full + 8 * s, (it / ST) & 1);
        if (!ok || *(volatile int*)&failed) { ok = false; break; }
        tc_fence_after();
        const uint64_t wdesc = smem_desc_sw128(smem_w + s * W_BYTES), adesc = smem_desc_sw128(smem_a + s * A_HALF);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(tmem_acc, wdesc + 2 * k, adesc + 2 * k, idesc, (it | k) != 0);
        umma_commit_pair(bar_empty + 8 * s);  // frees the stage in both blocks
      }
      if (ok) {
        umma_commit_pair(bar_acc);  // accumulators complete in both blocks
      } else {
        atomicOr(args.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
      }
    }
  } else {
    stream_epilogue<BT, 1>(args, warp, lane, bar_acc, &failed, tmem_acc, n0, row_lo, row_hi);
  }
  tc_fence_before();
  cluster_sync_all();  // neither block gives up shared or tensor memory that the pair's MMAs may still use
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_acc, TMEM_COLS);
  }
}

// out[m, n] = sum over splits (ascending) of partial[z][m][n]
template <typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TO* __restrict__ out, long long total, int splits) {
  JLX_TL(TL_SPLITK_REDUCE);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += partial[(size_t)z * total + i];
    out[i] = from_f32<TO>(s);
  }
}

// -------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D bfloat16 tensor [rows, K] row-major, boxes of [box_rows, 64] with the 128-byte swizzle; reads
// outside the tensor give zeros.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  JLX_REQUIRE(fn != nullptr, "gemm_stream: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  JLX_REQUIRE(r == CUDA_SUCCESS, "gemm_stream: cuTensorMapEncodeTiled failed (%d) for a [%lld, %lld] tensor", (int)r, rows, K);
  return 0;
}

template <int BT, int SW, int SA, int WT>
static int launch(const CUtensorMap& mw, const CUtensorMap& ma, const StreamArgs& a, int row_tiles, cudaStream_t stream) {
  constexpr size_t smem = (size_t)SW * (WT * WN * BK * 2) + (size_t)SA * (BT * BK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    JLX_CUDA(cudaFuncSetAttribute(gemm_stream_kernel<BT, SW, SA, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid((a.N + WN * WT - 1) / (WN * WT), row_tiles, a.splits);
  JLX_CUDA(jlx_launch_pdl(gemm_stream_kernel<BT, SW, SA, WT>, grid, dim3(NTHREADS), smem, stream, mw, ma, a));
  return 0;
}

template <int BT, int ST>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& ma, const StreamArgs& a, int row_tiles, cudaStream_t stream) {
  constexpr size_t smem = (size_t)ST * (WN * BK * 2 + (BT / 2) * BK * 2) + 1024;
  static bool configured = false;
  if (!configured) {
    JLX_CUDA(cudaFuncSetAttribute(gemm_stream_pair_kernel<BT, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.N / WN, row_tiles, a.splits);
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  JLX_CUDA(cudaLaunchKernelEx(&cfg, gemm_stream_pair_kernel<BT, ST>, mw, ma, a));
  return 0;
}

// Token-tile width (the MMA's N, a multiple of 16) for a product whose groups have up to about `rows_hint` rows.
static int pick_bt(int rows_hint) {
  static const int widths[] = {16, 32, 64, 96, 128, 160, 192, 224, 256};
  for (int w : widths)
    if (rows_hint <= w) return w;
  return 256;
}

JLX_API int jlx_gemm_stream_supported(int K) { return K % 8 == 0 && K >= 8; }

// The token-tile width that jlx_gemm_stream uses for this hint (a tile list must be made for the same width).
JLX_API int jlx_gemm_stream_token_tile(int rows_hint) { return pick_bt(rows_hint); }

// rows: token rows of A (grouped: an upper bound of offsets[E]); rows_hint: typical rows per group
// (chooses the token-tile width).
// mode 0: out[rows, N] (bfloat16 or float32); with splits > 1 the partials go to `scratch` (float32
//         [splits * rows * N]) and a second kernel adds them in ascending order.
// mode 1: out receives the float32 partials themselves, [splits][rows][N], for a consumer that adds them.
// mode 2: fused SwiGLU epilogue: weight rows are interleaved in blocks of [16 gate, 16 up], out is
//         [rows, N / 2] = silu(gate) * up; no split-K.
// tile_list / n_tiles (optional, grouped only): the row tiles that have rows, made by jlx_expert_sort for the
// tile width jlx_gemm_stream_token_tile(rows_hint); without them every block walks the offsets.
// offsets_settled (grouped only): the caller's word that the kernel launched just before this one on the stream is a
// grouped product of this library over the same offsets and tile list (so that these were complete before it began).
// Returns the split count used through *splits_used (it may be lower than asked).
JLX_API int jlx_gemm_stream(const void* A, const void* W, void* out, int out_is_f32, int rows, int N, int K,
                            const int* offsets, int E, int rows_hint, int splits, float* scratch, int mode,
                            const int* tile_list, const int* n_tiles, int offsets_settled, int* splits_used, int* status,
                            cudaStream_t stream) {
  JLX_REQUIRE(rows >= 0 && N > 0 && K > 0, "gemm_stream: bad sizes rows=%d N=%d K=%d", rows, N, K);
  JLX_REQUIRE(K % 8 == 0, "gemm_stream: K = %d is no multiple of 8 (TMA needs 16-byte row strides); use the SIMT product", K);
  JLX_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_stream: operands must be 16-byte aligned");
  JLX_REQUIRE(!offsets || E > 0, "gemm_stream: a grouped product needs a group count");
  JLX_REQUIRE(!tile_list || n_tiles, "gemm_stream: a tile list needs its count");
  JLX_REQUIRE(mode >= 0 && mode <= 2, "gemm_stream: unknown mode %d", mode);
  JLX_REQUIRE(splits >= 1 && (splits == 1 || mode == 1 || scratch), "gemm_stream: split-K needs scratch memory");
  JLX_REQUIRE(mode != 2 || (splits == 1 && N % 32 == 0), "gemm_stream: the SwiGLU epilogue needs N %% 32 == 0 and no split-K");
  JLX_REQUIRE(mode != 1 || out_is_f32, "gemm_stream: partials are float32");
  if (splits_used) *splits_used = 1;
  if (rows == 0) return 0;
  const int groups = offsets ? E : 1;
  const int bt = pick_bt(rows_hint > 0 ? rows_hint : rows);
  CUtensorMap mw, ma;
  if (make_map(&mw, W, (long long)groups * N, K, WN)) return 1;
  if (make_map(&ma, A, rows, K, bt)) return 1;
  int kps = K;
  if (splits > 1) {
    kps = ((K + splits - 1) / splits + BK - 1) / BK * BK;
    splits = (K + kps - 1) / kps;
  }
  if (splits_used) *splits_used = splits;
  StreamArgs a;
  a.N = N; a.K = K; a.rows = rows; a.offsets = offsets; a.E = E;
  a.tile_list = offsets ? tile_list : nullptr; a.n_tiles = n_tiles;
  a.out = (splits > 1 && mode == 0) ? (void*)scratch : out;
  a.out_is_f32 = out_is_f32; a.silu = mode == 2; a.splits = splits; a.k_per_split = kps; a.status = status;
  a.offsets_settled = offsets && offsets_settled;
  // Row tiles to launch blocks for.  Grouped: a group of r rows has ceil(r / bt) <= r / bt + 1 tiles and only a group
  // with rows has any, so there are at most rows / bt + min(E, rows) of them.  (A looser bound costs time: a block
  // without a tile returns at once, but with the kernel's shared memory only two blocks fit an SM at a time, and with
  // 128 experts and a handful of rows the blocks without work were a hundred times the blocks with.)
  const int row_tiles = offsets ? rows / bt + (E < rows ? E : rows) : (rows + bt - 1) / bt;
  JLX_REQUIRE(row_tiles <= 65535, "gemm_stream: too many row tiles");
  int rc;
  // Wide token tiles (prompt portions): a pair of blocks per 256 weight rows, when the rows divide so.
  const bool pair = bt >= 96 && N % (2 * WN) == 0;
  if (pair) {
    CUtensorMap ma_half;
    if (make_map(&ma_half, A, rows, K, bt / 2)) return 1;
    switch (bt) {
      case 96: rc = launch_pair<96, 4>(mw, ma_half, a, row_tiles, stream); break;
      case 128: rc = launch_pair<128, 4>(mw, ma_half, a, row_tiles, stream); break;
      case 160: rc = launch_pair<160, 4>(mw, ma_half, a, row_tiles, stream); break;
      case 192: rc = launch_pair<192, 4>(mw, ma_half, a, row_tiles, stream); break;
      case 224: rc = launch_pair<224, 3>(mw, ma_half, a, row_tiles, stream); break;
      default: rc = launch_pair<256, 3>(mw, ma_half, a, row_tiles, stream); break;
    }
  } else
  switch (bt) {
    // up to 192 token rows: one weight tile and stages sized so that two blocks share an SM (about 100 KB
    // each): one block's epilogue (tensor memory -> registers -> global) overlaps the other's main loop.
    // wider: two weight tiles per block (the token tile is fetched once for both), one block per SM.
    case 16: rc = launch<16, 5, 5, 1>(mw, ma, a, row_tiles, stream); break;
    case 32: rc = launch<32, 5, 5, 1>(mw, ma, a, row_tiles, stream); break;
    case 64: rc = launch<64, 4, 4, 1>(mw, ma, a, row_tiles, stream); break;
    case 96: rc = launch<96, 3, 3, 1>(mw, ma, a, row_tiles, stream); break;
    case 128: rc = launch<128, 3, 3, 1>(mw, ma, a, row_tiles, stream); break;
    case 160: rc = launch<160, 3, 3, 1>(mw, ma, a, row_tiles, stream); break;
    case 192: rc = launch<192, 2, 2, 1>(mw, ma, a, row_tiles, stream); break;
    case 224: rc = launch<224, 3, 3, 2>(mw, ma, a, row_tiles, stream); break;  // 60 KB
    default: rc = launch<256, 3, 3, 2>(mw, ma, a, row_tiles, stream); break;   // 64 KB
  }
  if (rc) return rc;
  if (splits > 1 && mode == 0) {
    const long long total = (long long)rows * N;
    const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (out_is_f32)
      splitk_reduce_kernel<float><<<blocks, 256, 0, stream>>>(scratch, (float*)out, total, splits);
    else
      splitk_reduce_kernel<bf16><<<blocks, 256, 0, stream>>>(scratch, (bf16*)out, total, splits);
    JLX_LAUNCH_CHECK("splitk_reduce");
  }
  return 0;
}
