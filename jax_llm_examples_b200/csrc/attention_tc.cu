// Flash attention for prompt portions on the 5th-generation tensor cores (tcgen05), bfloat16, head size 128.
//
// One block = 128 consecutive query tokens of one request and one query head.  Keys and values come from
// the paged cache in tiles of 128 keys.  Per tile:
//   S = Q K^T        tcgen05.mma, Q and K from shared memory (TMA, 128-byte swizzle), S in tensor memory
//   P = softmax part PARTS threads per query row read their parts of its row of S from tensor memory, keep the running
//                    max and sum in 32-bit, and write P (bfloat16, two keys per 32-bit column) back over the
//                    first half of the same S buffer; when a row's maximum moved they rescale O
//   O += P V         tcgen05.mma with P as the operand in tensor memory and V from shared memory as an MN-major
//                    operand (the cache keeps values as [key][dh], so dh is the contiguous direction), O in
//                    tensor memory
// S is double-buffered in tensor memory, so the product of the next tile runs while this tile's softmax does.
// MMAs run in the order of their issue: the score product of tile j+2, which overwrites the buffer of S_j and
// P_j, is issued after O += P_j V_j and so needs no barrier of its own;
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

__global__ void __launch_bounds__(NTHREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const TcParams P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = base + TILE_BYTES, v_s = k_s + 2 * TILE_BYTES;
  // barriers: 0 q_full | 1,2 k_full | 3,4 v_full | 5,6 v_empty | 7,8 s_full | 9,10 free | 11 p_ready | 12 o_done | 13,14 k_empty |
  // 15..18 the meeting of the two softmax warps of each quarter of the rows
  __shared__ __align__(8) uint64_t bars[19];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;
  __shared__ float xmax[2][PARTS][BQ];  // [tile parity][part of the keys][row]: what the threads of a row exchange
  __shared__ float xsum[PARTS][BQ];
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [bar0](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // blocks are handed out in the order of blockIdx.x, then y: all heads of the first tile of the list (the
  // one with the most keys, see the engine's tile order) start before any head of a lighter tile
  const int head = blockIdx.x, tile = blockIdx.y;
  const int G = P.Hq / P.Hkv, hk = head / G;
  const int n0 = P.tiles[2 * tile], cnt = P.tiles[2 * tile + 1];
  const int r = P.req_of_token[n0];
  const int p_first = P.positions[n0], p_last = p_first + cnt - 1;
  const int lo_tile = first_key(p_first, P.chunk, P.window);
  const int key_begin = lo_tile / BKV * BKV;
  const int n_kv = (p_last - key_begin) / BKV + 1;
  const int* table = P.block_table + (size_t)r * P.bt_stride;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 9; ++i) mbar_init(BAR(i), 1);
    mbar_init(BAR(9), 1);
    mbar_init(BAR(10), 1);
    mbar_init(BAR(11), 128 * PARTS);
    mbar_init(BAR(12), 1);
    mbar_init(BAR(13), 1);
    mbar_init(BAR(14), 1);
    for (int i = 15; i < 19; ++i) mbar_init(BAR(i), 32 * PARTS);
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
      mbar_expect_tx(BAR(0), TILE_BYTES);
      tma_load_3d(q_s, &map_q, 0, head, n0, BAR(0));
      tma_load_3d(q_s + HALF_BYTES, &map_q, 64, head, n0, BAR(0));
      // One tile of keys (which = 0) or values (which = 1) into stage j & 1: four boxes of 64 rows x 64 elements.
      auto load_tile = [&](int j, int which) {
        const int st = j & 1;
        const uint32_t bar = BAR((which ? 3 : 1) + st);
        const uint32_t dst = (which ? v_s : k_s) + st * TILE_BYTES;
        mbar_expect_tx(bar, TILE_BYTES);
        for (int b = 0; b < BKV / 64; ++b) {  // pages hold whole 64-key blocks
          const int pos = key_begin + j * BKV + b * 64;
          const int pi = pos / P.page_size;
          int page = pi < P.bt_stride ? table[pi] : -1;
          if (page >= P.num_pages) { atomicOr(P.status, JLX_STATUS_BAD_PAGE); page = 0; }
          if (page < 0) page = 0;  // no page there: every key of the block is masked
          const int row = ((page * 2 + which) * P.Hkv + hk) * P.page_size + (pos - pi * P.page_size);
          for (int h = 0; h < 2; ++h) tma_load_2d(dst + h * HALF_BYTES + b * 64 * 128, &map_kv, h * 64, row, bar);
        }
      };
      // Keys are free again after their score product, values after the product with P, which comes a tile
      // later: each ring advances as soon as its own stage is free.
      int ik = 0, iv = 0;
      uint32_t idle = 0;
      bool ok = true;
      while ((ik < n_kv || iv < n_kv) && ok) {
        bool moved = false;
        if (ik < n_kv && (ik < 2 || mbar_try_wait(BAR(13 + (ik & 1)), ((ik >> 1) - 1) & 1))) { load_tile(ik, 0); ++ik; moved = true; }
        if (iv < n_kv && (iv < 2 || mbar_try_wait(BAR(5 + (iv & 1)), ((iv >> 1) - 1) & 1))) { load_tile(iv, 1); ++iv; moved = true; }
        if (moved) idle = 0;
        else if (++idle >= WAIT_LIMIT || *(volatile int*)&failed) ok = false;
      }
      if (!ok) {
        atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
        failed = 1;
        for (int j = max(0, ik - 2); j < ik; ++j) mbar_wait(BAR(1 + (j & 1)), (j >> 1) & 1);
        for (int j = max(0, iv - 2); j < iv; ++j) mbar_wait(BAR(3 + (j & 1)), (j >> 1) & 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BKV, 0), idesc_pv = make_idesc(DH, 1);
      bool ok = mbar_wait(BAR(0), 0);
      auto issue_qk = [&](int j) {  // S[j & 1] = Q K_j^T
        const int st = j & 1;
        const uint32_t kb = k_s + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (kk >> 2) * HALF_BYTES + (kk & 3) * 32;  // 16 elements = 32 bytes along the row
          umma_bf16(tm_s0 + st * 128, desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, kk != 0);
        }
        umma_commit(BAR(7 + st));   // S is complete
        umma_commit(BAR(13 + st));  // K_j may be overwritten
      };
      if (ok) ok = mbar_wait(BAR(1), 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < n_kv) {
          const int s1 = (j + 1) & 1;
          ok = mbar_wait(BAR(1 + s1), ((j + 1) >> 1) & 1);  // K_{j+1} has landed
          if (!ok || *(volatile int*)&failed) { ok = false; break; }
          tc_fence_after();
          issue_qk(j + 1);
        }
        ok = mbar_wait(BAR(11), j & 1);                   // P_j is in tensor memory, O is rescaled
        if (ok) ok = mbar_wait(BAR(3 + st), (j >> 1) & 1);  // V_j has landed
        if (!ok || *(volatile int*)&failed) { ok = false; break; }
        tc_fence_after();
        const uint32_t vb = v_s + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // P: 16 keys = 8 columns of tensor memory; V: MN-major, 16 keys = 16 rows of 128 bytes
          umma_bf16_a_tmem(tm_o, tm_s0 + st * 128 + kk * 8, desc_mn_major(vb + kk * 16 * 128, HALF_BYTES), idesc_pv, (j | kk) != 0);
        }
        umma_commit(BAR(5 + st));  // V_j may be overwritten
        umma_commit(BAR(12));      // O holds tiles 0..j
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
    const bool live = row < cnt;
    const int p_row = p_first + min(row, cnt - 1);
    const int lo_row = first_key(p_row, P.chunk, P.window);
    float sc = P.scale_log2;  // positive: raw scores and scaled scores have their maximum at the same key
    if (P.attn_scale != 0.f) sc *= 1.f + P.attn_scale * log1pf(floorf(((float)p_row + 1.f) / P.floor_scale));
    float m = NEG_BIG, l = 0.f;  // the running maximum (of scaled scores, in powers of two) and this thread's sum
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      ok = mbar_wait(BAR(7 + st), (j >> 1) & 1);
      if (*(volatile int*)&failed) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int tile_key = key_begin + j * BKV + col0;
      const bool need_mask = key_begin + j * BKV + BKV - 1 > p_first || key_begin + j * BKV < first_key(p_last, P.chunk, P.window);
      const uint32_t s_addr = tm_s0 + st * 128 + lane_addr + col0;
      // this thread's raw scores of the row come into registers once
      uint32_t v[CP];
#pragma unroll
      for (int c = 0; c < CP; c += 32) tmem_ld32(s_addr + c, v + c);
      tmem_ld_wait();
      float mx4[4] = {NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG};  // four chains instead of one long chain of dependent steps
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < CP; ++i) {
          const int key = tile_key + i;
          const float sv = (key >= lo_row && key <= p_row) ? __uint_as_float(v[i]) : NEG_BIG;
          v[i] = __float_as_uint(sv);
          mx4[i & 3] = fmaxf(mx4[i & 3], sv);
        }
      } else {
#pragma unroll
        for (int i = 0; i < CP; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the row's maximum over all parts (double-buffered by tile parity: a partner may be a tile ahead)
      xmax[st][part][row] = mx;
      mbar_arrive(BAR(15 + quarter));
      ok = mbar_wait(BAR(15 + quarter), j & 1);
      if (*(volatile int*)&failed) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
#pragma unroll
      for (int q = 0; q < PARTS; ++q) mx = fmaxf(mx, xmax[st][q][row]);
      // raw -> scaled; a row whose keys are all masked so far keeps NEG_BIG (NEG_BIG * sc does not overflow)
      mx = fmaxf(m, mx > 0.5f * NEG_BIG ? mx * sc : NEG_BIG);
      const float corr = fast_exp2(m - mx);
      // probabilities 2^(s * sc - mx) and their sum; a masked score gives exactly 0, also in a row whose scores are
      // all masked so far (mx = NEG_BIG)
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[CP / 2];
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < CP; i += 2) {
          const float s0 = __uint_as_float(v[i]), s1 = __uint_as_float(v[i + 1]);
          const float p0 = s0 > 0.5f * NEG_BIG ? fast_exp2(fmaf(s0, sc, -mx)) : 0.f;
          const float p1 = s1 > 0.5f * NEG_BIG ? fast_exp2(fmaf(s1, sc, -mx)) : 0.f;
          rs4[(i >> 1) & 3] += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
      } else {
#pragma unroll
        for (int i = 0; i < CP; i += 2) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), sc, -mx)), p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), sc, -mx));
          rs4[(i >> 1) & 3] += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
      }
      const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      // P over the first half of this S buffer: keys 2c and 2c+1 in column c (the partners have read their scores:
      // they met after their loads)
      if (CP == 64) tmem_st32(tm_s0 + st * 128 + lane_addr + part * (CP / 2), packed);
      else tmem_st16(tm_s0 + st * 128 + lane_addr + part * (CP / 2), packed);
      l = l * corr + rs;
      m = mx;
      // Rescale this thread's part of O's columns when a row of the warp moved its maximum; the product of the
      // previous tile must be complete first (nothing to rescale before the first product).
      if (j > 0 && !__all_sync(0xffffffffu, corr == 1.f)) {
        ok = mbar_wait(BAR(12), (j - 1) & 1);
        if (*(volatile int*)&failed) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint32_t o[32];
#pragma unroll 1
        for (int c0 = part * (DH / PARTS); c0 < (part + 1) * (DH / PARTS); c0 += 32) {
          tmem_ld32(tm_o + lane_addr + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st32(tm_o + lane_addr + c0, o);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(BAR(11));
    }
    if (ok) {
      ok = mbar_wait(BAR(12), (n_kv - 1) & 1);
      if (*(volatile int*)&failed) ok = false;
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      // the row's sum is the sum of the parts' sums
      xsum[part][row] = l;
      mbar_arrive(BAR(15 + quarter));
      ok = __all_sync(0xffffffffu, mbar_wait(BAR(15 + quarter), n_kv & 1));
    }
    if (ok) {
      float total = 0.f;
#pragma unroll
      for (int q = 0; q < PARTS; ++q) total += xsum[q][row];
      const float inv = 1.f / total;
      bf16* dst = P.out + ((size_t)(n0 + row) * P.Hq + head) * DH;
      uint32_t v[32];
#pragma unroll 1
      for (int c0 = part * (DH / PARTS); c0 < (part + 1) * (DH / PARTS); c0 += 32) {
        tmem_ld32(tm_o + lane_addr + c0, v);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int u = 0; u < 4; ++u)
              op[u] = __floats2bfloat162_rn(__uint_as_float(v[i + 2 * u]) * inv, __uint_as_float(v[i + 2 * u + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c0 + i) = o;
          }
        }
      }
    } else if (lane == 0) {
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
  JLX_REQUIRE(n_tiles <= 65535, "attention_prefill_tc: %d tiles; up to 65535 are supported", n_tiles);
  attention_prefill_tc_kernel<<<dim3(Hq, n_tiles), NTHREADS, smem, stream>>>(map_q, map_kv, P);
  JLX_LAUNCH_CHECK("attention_prefill_tc");
  return 0;
}
