// Flash attention for prompt portions on the 5th-generation tensor cores (tcgen05), bfloat16, head size 128.
//
// A work item = 128 consecutive query tokens of one request and one query head; a persistent block (one per SM)
// walks its share of the items (see the kernel).  Keys and values come from the paged cache in tiles of 128 keys.
// Per tile:
//   S = Q K^T        tcgen05.mma, Q and K from shared memory (TMA, 128-byte swizzle), S in tensor memory
//   P = softmax part PARTS threads per query row read their parts of its row of S from tensor memory, keep the
//                    running reference (the maximum, updated lazily) and sum in 32-bit, and write P (bfloat16, two
//                    keys per 32-bit column) back over the first half of the same S buffer; when a row's maximum
//                    outgrew its reference by 2^LAZY_GROWTH they rescale O
//   O += P V         tcgen05.mma with P as the operand in tensor memory and V from shared memory as an MN-major
//                    operand (the cache keeps values as [key][dh], so dh is the contiguous direction), O in
//                    tensor memory
// S is double-buffered in tensor memory, so the product of the next tile runs while this tile's softmax does.
// MMAs run in the order of their issue: the score product of tile g+2, which overwrites the buffer of S_g and
// P_g, is issued after O += P_g V_g and so needs no barrier of its own;
// K and V tiles are double-buffered in shared memory.  Warp 0 issues TMA copies, warp 1 issues the MMAs, the other
// warps (PARTS threads per query row = per tensor-memory lane, each a part of the tile's keys) do softmax,
// rescaling and the final store.
//
// Mask, scale and softmax are those of llama4/llama4_jax/model.py:731-794 (causal, same chunk, optional
// window; scale dh^-0.5; 32-bit softmax), with the attention temperature on layers that have it.  The
// reference sends prefill attention to a TPU library (model.py:842-864).
//
// Every wait on a barrier is bounded; after a timeout the block raises JLX_STATUS_WAIT_TIMEOUT, waits
// (bounded) for its own copies, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "mbarrier.cuh"

#define DH 128
#define BQ 128           // query rows per block
#define BKV 128          // keys per tile
#define PARTS 4          // softmax threads per query row: each takes BKV / PARTS of a tile's keys and DH / PARTS of O's columns
#define NTHREADS (64 + 128 * PARTS)  // warp 0: TMA, warp 1: MMA, then PARTS softmax warps for each quarter of the query rows
#define CP (BKV / PARTS)  // key columns of a tile per softmax thread
#define WAIT_LIMIT JLX_WAIT_LIMIT
#define NEG_BIG (-1.0e30f)
#define LAZY_GROWTH 6.0f  // see the softmax warps: how far a row's maximum may outgrow its reference before O is rescaled

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
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
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors for tiles whose rows are 128 bytes (64 bfloat16) with the 128-byte
// swizzle, 8-row groups 1024 bytes apart.  K-major: the 64 elements of a row run along K.  MN-major: they run
// along the operand's M/N direction and rows are K steps; blocks of 64 along M/N are `lbo_bytes` apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo_bytes) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: bfloat16 operands, float32 accumulator, M = 128, N = n; A K-major; B K- or MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct TcParams {
  const int* block_table;
  int bt_stride;
  const int* req_of_token;
  const int* positions;
  bf16* out;            // [N, Hq, DH]
  const int* tiles;     // [n_tiles][2] = (first token row, count <= 128), one request each
  int Hq, Hkv, page_size, num_pages;
  float scale_log2;
  int chunk, window;
  float attn_scale, floor_scale;
  int* status;
};

__device__ __forceinline__ int first_key(int p, int chunk, int window) {
  int s = 0;
  if (chunk > 0) s = p - p % chunk;
  if (window > 0) s = max(s, p - window + 1);
  return s;
}

// Shared-memory plan (bytes from a 1024-aligned base): Q [2 halves][128][128B] = 32 KB, then K and V
// stages [2][2 halves][128][128B] = 64 KB each.
#define TILE_BYTES (2 * 128 * 128)  // one [128 rows][128 elements] operand: two halves of 16 KB
#define HALF_BYTES (128 * 128)

// A work item: one tile of up to 128 query tokens of one request, and one query head.
struct Item {
  int head, hk, n0, cnt, p_first, p_last, key_begin, n_kv;
  const int* table;
};

// The kernel is persistent: one block per SM walks a list of work items.  Items are numbered heaviest first (the tile
// list's order, heads fastest), and block c takes, of every round of gridDim.x items, the c-th in even rounds and the
// c-th from the end in odd ones, so that all blocks get about the same number of key tiles.  The key tiles of a block's
// items form one stream: barriers, rings and buffers are indexed by a tile's number g in that stream, and the score
// product of the next item's first tile is issued while the softmax of this item's last tile runs.  What an item costs
// beyond its tiles (the block's start, set-up, the first loads, the pipeline's fill) is so paid once per block, not
// once per item; only the wait for the last product and the store of the output remain between two items.
__global__ void __launch_bounds__(NTHREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const TcParams P,
                            int n_items) {
  JLX_TL(TL_ATTN_PREFILL);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = base + TILE_BYTES, v_s = k_s + 2 * TILE_BYTES;
  // barriers (each use flips a phase bit; g = a tile's number in the block's stream, i = an item's number in the block)
  enum { B_QFULL = 0,    // Q of item i has landed                      phase i
         B_QEMPTY = 1,   // the last score product of item i is done    phase i
         B_KFULL = 2,    // [2] K of tile g has landed                  stage g % 2, phase g / 2
         B_KEMPTY = 4,   // [2] the score product of tile g is done
         B_VFULL = 6,    // [2] V of tile g has landed
         B_VEMPTY = 8,   // [2] the product with P of tile g is done
         B_SFULL = 10,   // [2] S of tile g is complete
         B_PREADY = 12,  // P of tile g is in tensor memory, O rescaled  phase g
         B_ODONE = 13,   // O holds the item's tiles up to g            phase g
         B_MEET = 14,    // [4] the threads of a quarter of the rows have met
         N_BARS = 18 };
  __shared__ __align__(8) uint64_t bars[N_BARS];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  __shared__ float xmax[2][PARTS][BQ];  // [meeting parity][part of the keys][row]: what the threads of a row exchange
  __shared__ float xsum[2][PARTS][BQ];
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [bar0](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = P.Hq / P.Hkv;
  // the block's i-th item, or n_kv = 0 when it has no more
  auto item = [&](int i) {
    Item it;
    it.n_kv = 0;
    const int rank = (i & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const long long w = (long long)i * gridDim.x + rank;
    if (w >= n_items) return it;
    const int tile = (int)(w / P.Hq);
    it.head = (int)(w % P.Hq);
    it.hk = it.head / G;
    it.n0 = P.tiles[2 * tile];
    it.cnt = P.tiles[2 * tile + 1];
    it.p_first = P.positions[it.n0];
    it.p_last = it.p_first + it.cnt - 1;
    it.key_begin = first_key(it.p_first, P.chunk, P.window) / BKV * BKV;
    it.n_kv = (it.p_last - it.key_begin) / BKV + 1;
    it.table = P.block_table + (size_t)P.req_of_token[it.n0] * P.bt_stride;
    return it;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(BAR(i), 1);  // a TMA transaction count or a tcgen05.commit each, but:
    mbar_init(BAR(B_PREADY), 128 * PARTS);
    for (int i = 0; i < 4; ++i) mbar_init(BAR(B_MEET + i), 32 * PARTS);
    failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 512);  // S0, S1 (128 columns each), O (128): 384 -> 512
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tm_s0 = tmem, tm_o = tmem + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int g0 = 0;  // stream number of the item's first tile
      bool ok = true;
      for (int i = 0; ok; ++i) {
        const Item it = item(i);
        if (it.n_kv == 0) break;
        // Q's buffer is free when the previous item's last score product is done
        if (i > 0) ok = mbar_wait(BAR(B_QEMPTY), (i - 1) & 1);
        if (!ok || *(volatile int*)&failed) { ok = false; break; }
        mbar_expect_tx(BAR(B_QFULL), TILE_BYTES);
        tma_load_3d(q_s, &map_q, 0, it.head, it.n0, BAR(B_QFULL));
        tma_load_3d(q_s + HALF_BYTES, &map_q, 64, it.head, it.n0, BAR(B_QFULL));
        // One tile of keys (which = 0) or values (which = 1) into stage g & 1: four boxes of 64 rows x 64 elements.
        auto load_tile = [&](int j, int which) {
          const int st = (g0 + j) & 1;
          const uint32_t bar = BAR((which ? B_VFULL : B_KFULL) + st);
          const uint32_t dst = (which ? v_s : k_s) + st * TILE_BYTES;
          mbar_expect_tx(bar, TILE_BYTES);
          for (int b = 0; b < BKV / 64; ++b) {  // pages hold whole 64-key blocks
            const int pos = it.key_begin + j * BKV + b * 64;
            const int pi = pos / P.page_size;
            int page = pi < P.bt_stride ? it.table[pi] : -1;
            if (page >= P.num_pages) { atomicOr(P.status, JLX_STATUS_BAD_PAGE); page = 0; }
            if (page < 0) page = 0;  // no page there: every key of the block is masked
            const int row = ((page * 2 + which) * P.Hkv + it.hk) * P.page_size + (pos - pi * P.page_size);
            for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * HALF_BYTES + b * 64 * 128, &map_kv, h * 64, row, bar);
          }
        };
        // Keys are free again after their score product, values after the product with P, which comes a tile
        // later: each ring advances as soon as its own stage is free.
        int ik = 0, iv = 0;
        uint32_t idle = 0;
        while ((ik < it.n_kv || iv < it.n_kv) && ok) {
          bool moved = false;
          const int gk = g0 + ik, gv = g0 + iv;
          if (ik < it.n_kv && (gk < 2 || mbar_try_wait(BAR(B_KEMPTY + (gk & 1)), ((gk >> 1) - 1) & 1))) { load_tile(ik, 0); ++ik; moved = true; }
          if (iv < it.n_kv && (gv < 2 || mbar_try_wait(BAR(B_VEMPTY + (gv & 1)), ((gv >> 1) - 1) & 1))) { load_tile(iv, 1); ++iv; moved = true; }
          if (moved) idle = 0;
          else if (++idle >= WAIT_LIMIT || *(volatile int*)&failed) ok = false;
        }
        g0 += it.n_kv;
        if (!ok) {  // let the copies in flight land before the block's shared memory is given up
          for (int j = max(0, ik - 2); j < ik; ++j) mbar_wait(BAR(B_KFULL + ((g0 - it.n_kv + j) & 1)), ((g0 - it.n_kv + j) >> 1) & 1);
          for (int j = max(0, iv - 2); j < iv; ++j) mbar_wait(BAR(B_VFULL + ((g0 - it.n_kv + j) & 1)), ((g0 - it.n_kv + j) >> 1) & 1);
        }
      }
      if (!ok) {
        atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------ MMA issuer
    // One thread issues all products, in the order of the stream: the score product of the tile after next... of
    // the NEXT tile (which may be the next item's first) goes out before this tile's product with P is waited for.
    // Products run in the order of their issue: the score product of tile g + 1 overwrites the buffer of S and P of
    // tile g - 1, whose product with P was issued before it.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BKV, 0), idesc_pv = make_idesc(DH, 1);
      bool ok = true;
      // S[g & 1] = Q K^T for tile g; `first` / `last`: the item's first / last tile; i: the item's number
      auto issue_qk = [&](int g, int i, bool first, bool last) {
        const int st = g & 1;
        if (first) ok = mbar_wait(BAR(B_QFULL), i & 1);
        if (ok) ok = mbar_wait(BAR(B_KFULL + st), (g >> 1) & 1);
        if (!ok || *(volatile int*)&failed) { ok = false; return; }
        tc_fence_after();
        const uint32_t kb = k_s + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;  // 16 elements = 32 bytes along the row
          umma_bf16(tm_s0 + st * 128, desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, kk != 0);
        }
        umma_commit(BAR(B_SFULL + st));   // S is complete
        umma_commit(BAR(B_KEMPTY + st));  // K may be overwritten
        if (last) umma_commit(BAR(B_QEMPTY));  // and so may Q
      };
      Item cur = item(0);
      int g = 0;
      if (cur.n_kv > 0) issue_qk(0, 0, true, cur.n_kv == 1);
      for (int i = 0; cur.n_kv > 0 && ok; ++i) {
        const Item nxt = item(i + 1);
        for (int j = 0; j < cur.n_kv && ok; ++j, ++g) {
          const int st = g & 1;
          if (j + 1 < cur.n_kv) issue_qk(g + 1, i, false, j + 2 == cur.n_kv);
          else if (nxt.n_kv > 0) issue_qk(g + 1, i + 1, true, nxt.n_kv == 1);
          if (!ok) break;
          ok = mbar_wait(BAR(B_PREADY), g & 1);                    // P is in tensor memory, O is rescaled
          if (ok) ok = mbar_wait(BAR(B_VFULL + st), (g >> 1) & 1);  // V has landed
          if (!ok || *(volatile int*)&failed) { ok = false; break; }
          tc_fence_after();
          const uint32_t vb = v_s + st * TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BKV / 16; ++kk) {
            // P: 16 keys = 8 columns of tensor memory; V: MN-major, 16 keys = 16 rows of 128 bytes
            umma_bf16_a_tmem(tm_o, tm_s0 + st * 128 + kk * 8, desc_mn_major(vb + kk * 16 * 128, HALF_BYTES), idesc_pv, (j | kk) != 0);
          }
          umma_commit(BAR(B_VEMPTY + st));  // V may be overwritten
          umma_commit(BAR(B_ODONE));        // O holds the item's tiles up to this one
        }
        cur = nxt;
      }
      if (!ok) {
        atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------------------ softmax, rescale, store
    // A warp reaches the tensor-memory lanes [32 * (warp & 3), +32), so PARTS warps share each quarter of the query
    // rows and split the tile's 128 key columns (and the output's 128 columns) among them.  The threads of a row
    // meet once per tile to agree on the row's maximum; each keeps the sum of its own part.  More, narrower threads
    // per row keep four warps on every scheduler: the chain load -> max -> exponentials -> store of one warp is
    // full of waits that the others fill.
    const int quarter = warp & 3, part = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;             // query row = tensor-memory lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int col0 = part * CP;
    bool ok = true;
    int g = 0;      // the tile's number in the block's stream
    int meets = 0;  // meetings of this quarter's threads so far (the phase of their barrier)
    Item upcoming = item(0);
    for (int i = 0; ok; ++i) {
      const Item it = upcoming;
      if (it.n_kv == 0) break;
      const bool live = row < it.cnt;
      const int p_row = it.p_first + min(row, it.cnt - 1);
      const int lo_row = first_key(p_row, P.chunk, P.window);
      const int lo_last = first_key(it.p_last, P.chunk, P.window);
      float sc = P.scale_log2;  // positive: raw scores and scaled scores have their maximum at the same key
      if (P.attn_scale != 0.f) sc *= 1.f + P.attn_scale * log1pf(floorf(((float)p_row + 1.f) / P.floor_scale));
      float m = NEG_BIG, l = 0.f;  // the running maximum (of scaled scores, in powers of two) and this thread's sum
      for (int j = 0; j < it.n_kv; ++j, ++g) {
        const int st = g & 1;
        ok = mbar_wait(BAR(B_SFULL + st), (g >> 1) & 1);
        if (*(volatile int*)&failed) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const int tile_key = it.key_begin + j * BKV + col0;
        const bool need_mask = it.key_begin + j * BKV + BKV - 1 > it.p_first || it.key_begin + j * BKV < lo_last;
        const uint32_t s_addr = tm_s0 + st * 128 + lane_addr + col0;
        // this thread's raw scores of the row come into registers once
        uint32_t v[CP];
#pragma unroll
        for (int c = 0; c < CP; c += 32) tmem_ld32(s_addr + c, v + c);
        tmem_ld_wait();
        float mx4[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG};  // four chains instead of one long chain of dependent steps
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < CP; ++c) {
            const int key = tile_key + c;
            const float sv = (key >= lo_row && key <= p_row) ? __uint_as_float(v[c]) : NEG_BIG;
            v[c] = __float_as_uint(sv);
            mx4[c & 3] = fmaxf(mx4[c & 3], sv);
          }
        } else {
#pragma unroll
          for (int c = 0; c < CP; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(v[c]));
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // the row's maximum over all parts (double-buffered by the meeting's parity: a partner may be a tile ahead)
        const int mp = meets & 1;
        xmax[mp][part][row] = mx;
        mbar_arrive(BAR(B_MEET + quarter));
        ok = mbar_wait(BAR(B_MEET + quarter), mp);
        ++meets;
        if (*(volatile int*)&failed) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
#pragma unroll
        for (int q = 0; q < PARTS; ++q) mx = fmaxf(mx, xmax[mp][q][row]);
        // raw -> scaled; a row whose keys are all masked so far keeps NEG_BIG (NEG_BIG * sc does not overflow)
        mx = fmaxf(m, mx > 0.5f * NEG_BIG ? mx * sc : NEG_BIG);
        // The reference point of the exponents need not be the maximum itself: while no row of this quarter has grown
        // by more than LAZY_GROWTH (in powers of two) beyond its reference, the references stay, the probabilities
        // may exceed 1 (up to 2^LAZY_GROWTH: no trouble for a 32-bit sum or a bfloat16 P), and O is not rescaled.
        // All threads of these rows decide alike: they hold the same references and have just exchanged the maxima.
        if (__all_sync(0xffffffffu, mx - m <= LAZY_GROWTH)) mx = m;
        const float corr = fast_exp2(m - mx);
        // probabilities 2^(s * sc - mx) and their sum; a masked score gives exactly 0, also in a row whose scores are
        // all masked so far (mx = NEG_BIG)
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t packed[CP / 2];
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < CP; c += 2) {
            const float s0 = __uint_as_float(v[c]), s1 = __uint_as_float(v[c + 1]);
            const float p0 = s0 > 0.5f * NEG_BIG ? fast_exp2(fmaf(s0, sc, -mx)) : 0.f;
            const float p1 = s1 > 0.5f * NEG_BIG ? fast_exp2(fmaf(s1, sc, -mx)) : 0.f;
            rs4[(c >> 1) & 3] += p0 + p1;
            __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
            packed[c >> 1] = *reinterpret_cast<uint32_t*>(&b2);
          }
        } else {
#pragma unroll
          for (int c = 0; c < CP; c += 2) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[c]), sc, -mx)), p1 = fast_exp2(fmaf(__uint_as_float(v[c + 1]), sc, -mx));
            rs4[(c >> 1) & 3] += p0 + p1;
            __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
            packed[c >> 1] = *reinterpret_cast<uint32_t*>(&b2);
          }
        }
        const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
        // P over the first half of this S buffer: keys 2c and 2c+1 in column c (the partners have read their scores:
        // they met after their loads)
        if (CP == 64) tmem_st32(tm_s0 + st * 128 + lane_addr + part * (CP / 2), packed);
        else tmem_st16(tm_s0 + st * 128 + lane_addr + part * (CP / 2), packed);
        l = l * corr + rs;
        m = mx;
        // The product of the previous tile must be complete before O is rescaled, and every thread waits for it
        // whether it rescales or not: a barrier's phase bit tells a waiter the truth only if the waiter has seen
        // the phase before, so no phase of this barrier is skipped.  (Nothing to wait for before an item's first
        // product: the phase before it was seen at the previous item's end.)
        if (j > 0) {
          ok = mbar_wait(BAR(B_ODONE), (g - 1) & 1);
          if (*(volatile int*)&failed) ok = false;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        // Rescale this thread's part of O's columns when a row of the warp moved its maximum.
        if (j > 0 && !__all_sync(0xffffffffu, corr == 1.f)) {
          tc_fence_after();
          uint32_t o[32];
#pragma unroll 1
          for (int c0 = part * (DH / PARTS); c0 < (part + 1) * (DH / PARTS); c0 += 32) {
            tmem_ld32(tm_o + lane_addr + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
            tmem_st32(tm_o + lane_addr + c0, o);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(BAR(B_PREADY));
      }
      if (!ok) break;
      // the next item's description is fetched now (a chain of dependent loads), behind the wait for the last product
      upcoming = item(i + 1);
      // the item's end: its last product, the row's sum (the sum of the parts' sums), the store
      ok = mbar_wait(BAR(B_ODONE), (g - 1) & 1);
      if (*(volatile int*)&failed) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int mp = meets & 1;
      xsum[mp][part][row] = l;
      mbar_arrive(BAR(B_MEET + quarter));
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(B_MEET + quarter), mp));
      ++meets;
      if (!ok) break;
      float total = 0.f;
#pragma unroll
      for (int q = 0; q < PARTS; ++q) total += xsum[mp][q][row];
      const float inv = 1.f / total;
      bf16* dst = P.out + ((size_t)(it.n0 + row) * P.Hq + it.head) * DH;
      uint32_t v[32];
#pragma unroll 1
      for (int c0 = part * (DH / PARTS); c0 < (part + 1) * (DH / PARTS); c0 += 32) {
        tmem_ld32(tm_o + lane_addr + c0, v);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 o;
            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int u = 0; u < 4; ++u)
              op[u] = __floats2bfloat162_rn(__uint_as_float(v[c + 2 * u]) * inv, __uint_as_float(v[c + 2 * u + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c0 + c) = o;
          }
        }
      }
      // (the next item's first product with P overwrites O; it waits for this warp's arrival at that tile's barrier,
      // which comes after these loads)
      tc_fence_before();
    }
    if (!ok && lane == 0) {
      atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
      failed = 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
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

JLX_API int jlx_attention_prefill_tc_supported(int Hq, int Hkv, int dh, int page_size) {
  return Hkv > 0 && Hq % Hkv == 0 && dh == DH && page_size >= 64 && page_size % 64 == 0;
}

// q: [N, Hq, 128] bfloat16; pages: [P, 2, Hkv, page_size, 128] bfloat16 with page_size a multiple of 64;
// tiles: int32 [n_tiles][2] on the device = (first token row, count <= 128), tokens of one request each.
JLX_API int jlx_attention_prefill_tc(const void* q, const void* pages, const int* block_table, int bt_stride,
                                     const int* req_of_token, const int* positions, void* out, const int* tiles,
                                     int n_tiles, int N, int Hq, int Hkv, int dh, int page_size, int num_pages, float scale,
                                     int chunk, int window, float attn_scale, float floor_scale, int* status,
                                     cudaStream_t stream) {
  JLX_REQUIRE(jlx_attention_prefill_tc_supported(Hq, Hkv, dh, page_size),
              "attention_prefill_tc: needs head size 128 and pages of a multiple of 64 tokens (got %d, %d)", dh, page_size);
  JLX_REQUIRE(N > 0 && num_pages > 0 && bt_stride > 0, "attention_prefill_tc: bad sizes");
  JLX_REQUIRE((long long)num_pages * 2 * Hkv * page_size < (1ll << 31), "attention_prefill_tc: cache too large for 32-bit rows");
  JLX_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)pages & 15) == 0 && ((uintptr_t)out & 15) == 0,
              "attention_prefill_tc: q, pages and out must be 16-byte aligned");
  JLX_REQUIRE(attn_scale == 0.f || floor_scale > 0.f, "attention: floor_scale must be positive");
  JLX_REQUIRE(Hq <= 65535, "attention_prefill_tc: too many heads");
  if (n_tiles == 0) return 0;
  EncodeTiledFn fn = encode_fn();
  JLX_REQUIRE(fn != nullptr, "attention_prefill_tc: the driver does not offer cuTensorMapEncodeTiled");
  CUtensorMap map_q, map_kv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)dh, (cuuint64_t)Hq, (cuuint64_t)N};
    cuuint64_t strides[2] = {(cuuint64_t)dh * 2, (cuuint64_t)Hq * dh * 2};
    cuuint32_t box[3] = {64, 1, BQ};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    JLX_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tc: tensor map of q failed (%d)", (int)r);
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)dh, (cuuint64_t)num_pages * 2 * Hkv * page_size};
    cuuint64_t strides[1] = {(cuuint64_t)dh * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    JLX_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tc: tensor map of the cache failed (%d)", (int)r);
  }
  TcParams P;
  P.block_table = block_table; P.bt_stride = bt_stride; P.req_of_token = req_of_token; P.positions = positions;
  P.out = (bf16*)out; P.tiles = tiles; P.Hq = Hq; P.Hkv = Hkv; P.page_size = page_size; P.num_pages = num_pages;
  P.scale_log2 = scale * 1.4426950408889634f; P.chunk = chunk; P.window = window; P.attn_scale = attn_scale;
  P.floor_scale = floor_scale; P.status = status;
  const size_t smem = 5 * (size_t)TILE_BYTES + 1024;
  static bool cfg = false;
  if (!cfg) {
    JLX_CUDA(cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cfg = true;
  }
  JLX_REQUIRE((long long)n_tiles * Hq < (1ll << 31), "attention_prefill_tc: too many tiles");
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    JLX_CUDA(cudaGetDevice(&dev));
    JLX_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int n_items = n_tiles * Hq;
  attention_prefill_tc_kernel<<<dim3(n_items < sms ? n_items : sms), NTHREADS, smem, stream>>>(map_q, map_kv, P, n_items);
  JLX_LAUNCH_CHECK("attention_prefill_tc");
  return 0;
}
