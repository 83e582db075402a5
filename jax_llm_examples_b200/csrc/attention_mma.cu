// Paged attention on the tensor cores for bfloat16, head sizes 64 and 128: a split-KV decode
// kernel (one query token per request) and a flash prefill kernel (portions of prompts, also mixed
// with single tokens), both aware of chunks, windows and the attention temperature.
//
// Reference: the reference's decode kernel (llama4/llama4_jax/ragged_attention.py:17-118) keeps
// running max / sum / output in 32-bit over blocks of keys with a per-row [start, length) range; its
// prefill goes to a TPU library (llama4/llama4_jax/model.py:842-864).  Mask, scale and softmax are
// those of model.py:731-794.  Here:
//
//  * rows of the score tile are (query token, query head of the group); all G query heads of a KV head
//    share each key/value tile in shared memory (a tile is read from HBM once per group, not per head);
//  * keys and values come by cp.async in 64-key tiles, found row by row through the block table, so any
//    page size works; shared-memory rows are XOR-swizzled for conflict-free ldmatrix;
//  * scores, softmax statistics and the output accumulator are 32-bit; probabilities are rounded to
//    bfloat16 only as the operand of the P*V product;
//  * key tiles are aligned to absolute positions (multiples of 64), so the order of a position's sums in a
//    prefill does not depend on the batch or on how the prompt was cut; decode splits are aligned multiples
//    of 256 keys whose size follows the batch size (a difference of rounding only).
//
// A query at position p reads keys [start(p), p], start(p) = max(chunk ? p - p % chunk : 0,
// window ? p - window + 1 : 0).  Temperature: scores of a layer with attn_scale != 0 are multiplied by
// 1 + attn_scale * ln(1 + floor((p + 1) / floor_scale)).
#include <cuda.h>

#include "common.cuh"
#include "mbarrier.cuh"

#define KT 64            // keys per tile
#define SPLIT_UNIT 64    // decode splits are multiples of this many keys (one tile), aligned to absolute positions
#define SPLIT_MIN 512    // ... and at least this long: shorter blocks spend their time on set-up
#define DEC_MAX_BOXES 1024  // block-table entries of a decode split kept in shared memory
#define DEC_STAGES 3     // key/value tiles in flight per decode block (96 KB at head size 128: two blocks per SM)
#define NEG_BIG (-1.0e30f)


__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- TMA and mbarrier (decode kernel: whole [rows, 64-element] boxes of a page per instruction)
#define WAIT_LIMIT JLX_WAIT_LIMIT
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

struct AttnParams {
  const bf16* q;        // [N, Hq, DH]
  const bf16* pages;    // [P, 2, Hkv, page, DH]
  const int* block_table;
  int bt_stride;
  const int* req_of_token;
  const int* positions;
  bf16* out;            // [N, Hq, DH]
  int Hq, Hkv, page_size, num_pages;
  float scale_log2;     // dh^-0.5 * log2(e)
  int chunk, window;
  float attn_scale, floor_scale;
  int* status;
  // prefill: tiles of up to 16 consecutive tokens of one request
  const int* tiles;     // [n_tiles][2] = (first token row, token count)
  // decode: partial results
  float* part_o;        // [N, Hq, max_splits, DH]
  float* part_ml;       // [N, Hq, max_splits, 2]
  int max_splits;
  const int* rows;      // optional, decode: the token rows to work on (null: rows 0..N-1); partials are indexed by the list's order
  int split_keys;       // keys per decode split (a multiple of SPLIT_UNIT)
};

__device__ __forceinline__ int first_key(int p, int chunk, int window) {
  int s = 0;
  if (chunk > 0) s = p - p % chunk;
  if (window > 0) s = max(s, p - window + 1);
  return s;
}

__device__ __forceinline__ float temperature(int p, float attn_scale, float floor_scale) {
  return attn_scale != 0.f ? 1.f + attn_scale * log1pf(floorf(((float)p + 1.f) / floor_scale)) : 1.f;
}

// Loads keys [key0, key0 + KT) of request r, KV head hk, into ks / vs (each [KT][DH], swizzled).
// Keys outside [lo, hi] or without a page become zeros.  Consecutive threads take consecutive 16-byte
// chunks of a row, so a warp's copy covers whole rows: full 128-byte lines from L2.
template <int DH>
__device__ __forceinline__ void load_kv_tile(const AttnParams& P, int r, int hk, int key0, int lo, int hi, bf16* ks, bf16* vs,
                                             int NT) {
  constexpr int CH = DH / 8;              // 16-byte chunks per row
  const size_t v_off = (size_t)P.Hkv * P.page_size * DH;
  const int c = threadIdx.x % CH;
  const int* table = P.block_table + (size_t)r * P.bt_stride;
  for (int j = threadIdx.x / CH; j < KT; j += NT / CH) {
    const int pos = key0 + j;
    bool valid = pos >= lo && pos <= hi;
    const bf16* src = P.pages;
    if (valid) {
      const int pi = pos / P.page_size;
      const int page = table[pi];
      if (page < 0 || page >= P.num_pages) {
        atomicOr(P.status, JLX_STATUS_BAD_PAGE);
        valid = false;
      } else {
        src = P.pages + (size_t)page * 2 * v_off + ((size_t)hk * P.page_size + (pos - pi * P.page_size)) * DH + c * 8;
      }
    }
    const int sw = (j * CH + (c ^ (j & 7))) * 8;
    cp_async16(smem_u32(ks + sw), src, valid);
    cp_async16(smem_u32(vs + sw), valid ? src + v_off : src, valid);
  }
}

// ------------------------------------------------------------------------------------ decode
// grid (max_splits, Hkv, R); 128 threads.  Rows of the score tile = the G query heads (G <= 16).  A block
// walks the 64-key tiles of its split through a ring of DEC_STAGES shared-memory stages; warp w takes keys
// [16 w, 16 w + 16) of every tile.  The four warps' results are merged in shared memory and written as one
// partial (unnormalised output, max, sum) per (token, head, split).  The host sizes the splits so that a
// few hundred blocks share the GPU: short-lived blocks would spend their time on set-up.
template <int DH>
__global__ void __launch_bounds__(128) attention_decode_kernel(const AttnParams P) {
  JLX_TL(TL_ATTN_DECODE_PLAIN);
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int CH = DH / 8;
  bf16* ks = reinterpret_cast<bf16*>(smem);                  // [DEC_STAGES][KT][DH]
  bf16* vs = ks + DEC_STAGES * KT * DH;                      // [DEC_STAGES][KT][DH]
  const int slot = blockIdx.z, n = P.rows ? P.rows[slot] : slot, hk = blockIdx.y, split = blockIdx.x;
  const int G = P.Hq / P.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = P.positions[n], r = P.req_of_token[n];
  const int lo = first_key(p, P.chunk, P.window);
  const int key_begin = (lo / P.split_keys + split) * P.split_keys;
  if (key_begin > p) return;
  const int key_end = min(p + 1, key_begin + P.split_keys);
  const int n_tiles = (key_end - key_begin + KT - 1) / KT;

#pragma unroll
  for (int t = 0; t < DEC_STAGES - 1; ++t) {
    if (t < n_tiles) load_kv_tile<DH>(P, r, hk, key_begin + t * KT, lo, p, ks + t * KT * DH, vs + t * KT * DH, 128);
    cp_async_commit();
  }

  // Q fragments: row = head g (rows >= G are zero)
  uint32_t qf[DH / 16][4];
  {
    const int g0 = lane >> 2, g1 = g0 + 8, kk = (lane & 3) * 2;
    const bf16* q0 = P.q + ((size_t)n * P.Hq + hk * G + g0) * DH;
    const bf16* q1 = P.q + ((size_t)n * P.Hq + hk * G + g1) * DH;
#pragma unroll
    for (int s = 0; s < DH / 16; ++s) {
      qf[s][0] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk) : 0u;
      qf[s][1] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk) : 0u;
      qf[s][2] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk + 8) : 0u;
      qf[s][3] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk + 8) : 0u;
    }
  }
  const float sc = P.scale_log2 * temperature(p, P.attn_scale, P.floor_scale);
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  float o[DH / 8][4];
#pragma unroll
  for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<DEC_STAGES - 2>();  // tile t has landed
    __syncthreads();                  // ... for every thread, and the stage of tile t - 1 is free
    {
      const int nt = t + DEC_STAGES - 1, st = nt % DEC_STAGES;
      if (nt < n_tiles) load_kv_tile<DH>(P, r, hk, key_begin + nt * KT, lo, p, ks + st * KT * DH, vs + st * KT * DH, 128);
      cp_async_commit();
    }
    const int tile_key = key_begin + t * KT;
    const bf16* kt = ks + (t % DEC_STAGES) * KT * DH;
    const bf16* vt = vs + (t % DEC_STAGES) * KT * DH;
    // S = Q K^T for this warp's 16 keys: two n-tiles of 8 keys
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kstep = 0; kstep < DH / 16; ++kstep) {
      const int key = warp * 16 + (lane >> 4) * 8 + (lane & 7);
      const int c = kstep * 2 + ((lane >> 3) & 1);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(smem_u32(kt + (key * CH + (c ^ (key & 7))) * 8), b0, b1, b2, b3);
      mma_bf16(s[0], qf[kstep], b0, b1);
      mma_bf16(s[1], qf[kstep], b2, b3);
    }
    // mask, online softmax (rows lane/4 and lane/4 + 8)
    float mx[2] = {m[0], m[1]};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = tile_key + warp * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const bool ok = key >= lo && key <= p;
        s[nt][e] = ok ? s[nt][e] * sc : NEG_BIG;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) corr[h] = exp2f(m[h] - mx[h]);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = s[nt][e] > 0.5f * NEG_BIG ? exp2f(s[nt][e] - mx[e >> 1]) : 0.f;
        s[nt][e] = pv;
        rs[e >> 1] += pv;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l[h] = l[h] * corr[h] + rs[h];
      m[h] = mx[h];
    }
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    // O += P V over this warp's 16 keys
    uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
    for (int np = 0; np < DH / 16; ++np) {
      const int key = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int c = np * 2 + (lane >> 4);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(smem_u32(vt + (key * CH + (c ^ (key & 7))) * 8), b0, b1, b2, b3);
      mma_bf16(o[np * 2], pa, b0, b1);
      mma_bf16(o[np * 2 + 1], pa, b2, b3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge the four warps: shared memory is reused as float [4][16][DH + 2]
  float* red = reinterpret_cast<float*>(smem);
  constexpr int LD = DH + 2;
  {
    const int r0 = lane >> 2, r1 = r0 + 8, col = (lane & 3) * 2;
    float* w0 = red + (warp * 16 + r0) * LD;
    float* w1 = red + (warp * 16 + r1) * LD;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      w0[i * 8 + col] = o[i][0]; w0[i * 8 + col + 1] = o[i][1];
      w1[i * 8 + col] = o[i][2]; w1[i * 8 + col + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      w0[DH] = m[0]; w0[DH + 1] = l[0];
      w1[DH] = m[1]; w1[DH + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * DH; idx += 128) {
    const int g = idx / DH, d = idx % DH;
    float mm = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + g) * LD + DH]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(red[(w * 16 + g) * LD + DH] - mm);
      acc += red[(w * 16 + g) * LD + d] * f;
      ll += red[(w * 16 + g) * LD + DH + 1] * f;
    }
    const size_t row = ((size_t)slot * P.Hq + hk * G + g) * P.max_splits + split;
    P.part_o[row * DH + d] = acc;
    if (d == 0) {
      P.part_ml[row * 2] = mm;
      P.part_ml[row * 2 + 1] = ll;
    }
  }
}

// The same decode kernel with the tiles brought in by TMA: the cache of one layer is a 2-D tensor
// [pages * 2 * Hkv * page_size rows, DH] and a 64-key tile of one KV head is 64 / BOX_ROWS boxes of
// [BOX_ROWS rows, 64 elements] per 128 bytes of head (BOX_ROWS = min(page_size, 64)), written to shared
// memory with the 128-byte swizzle.  One thread issues the copies and the others wait on an mbarrier per
// stage: no per-lane copy instructions, so the load/store units stay free and the queue stays deep.
// Rows of keys outside [lo, p] are copied too (from page 0 where the block table has no page); their
// scores are masked, and their values are finite numbers written by this engine, so 0 * value = 0.
template <int DH>
__global__ void __launch_bounds__(128)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map, const AttnParams P, int box_rows) {
  JLX_TL(TL_ATTN_DECODE);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int HALVES = DH / 64;                 // 128-byte column blocks per row
  constexpr uint32_t HALF_BYTES = KT * 128;       // one [64 keys][64 elements] block
  constexpr uint32_t STAGE_BYTES = 2 * HALVES * HALF_BYTES;  // K and V
  __shared__ __align__(8) uint64_t full_bar[DEC_STAGES];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  pdl_launch_dependents();
  // Until pdl_wait() below, only what no kernel of this step writes is read: the step's description (rows,
  // positions, requests, block table: on the device before the step began) and keys and values of earlier steps.
  const int slot = blockIdx.z, n = P.rows ? P.rows[slot] : slot, hk = blockIdx.y, split = blockIdx.x;
  const int G = P.Hq / P.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = P.positions[n], r = P.req_of_token[n];
  const int lo = first_key(p, P.chunk, P.window);
  const int key_begin = (lo / P.split_keys + split) * P.split_keys;
  if (key_begin > p) return;
  const int key_end = min(p + 1, key_begin + P.split_keys);
  const int n_tiles = (key_end - key_begin + KT - 1) / KT;
  const int* table = P.block_table + (size_t)r * P.bt_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_STAGES; ++s) mbar_init(smem_u32(&full_bar[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // The block-table entries of the whole split come into shared memory first (all threads, one round of
  // loads), so that the producer's copies never wait on a global load.
  __shared__ int page_of_box[DEC_MAX_BOXES];
  const int boxes_per_tile = KT / box_rows;
  const int n_boxes = n_tiles * boxes_per_tile;
  const bool cached = n_boxes <= DEC_MAX_BOXES;
  if (cached) {
    for (int b = threadIdx.x; b < n_boxes; b += blockDim.x) {
      const int pi = (key_begin + b * box_rows) / P.page_size;
      page_of_box[b] = pi < P.bt_stride ? table[pi] : -1;
    }
    __syncthreads();
  }
  // producer: thread 0 issues all boxes of a tile
  auto issue = [&](int t) {
    const int st = t % DEC_STAGES;
    const uint32_t bar = smem_u32(&full_bar[st]);
    const uint32_t dst = base + st * STAGE_BYTES;
    mbar_expect_tx(bar, STAGE_BYTES);
    const int key0 = key_begin + t * KT;
    for (int b = 0; b < boxes_per_tile; ++b) {
      const int pos = key0 + b * box_rows;
      const int pi = pos / P.page_size;
      int page = cached ? page_of_box[t * boxes_per_tile + b] : (pi < P.bt_stride ? table[pi] : -1);
      if (page >= P.num_pages) { atomicOr(P.status, JLX_STATUS_BAD_PAGE); page = 0; }
      if (page < 0) page = 0;  // no page there: every key of the box is masked
      const int row_k = ((page * 2 + 0) * P.Hkv + hk) * P.page_size + (pos - pi * P.page_size);
      const int row_v = ((page * 2 + 1) * P.Hkv + hk) * P.page_size + (pos - pi * P.page_size);
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tma_load_2d(dst + h * HALF_BYTES + b * box_rows * 128, &map, h * 64, row_k, bar);
        tma_load_2d(dst + (HALVES + h) * HALF_BYTES + b * box_rows * 128, &map, h * 64, row_v, bar);
      }
    }
  };
  // The token's own key and value (position p) are written by the kernel before this one; every other key is older
  // than the step.  Tiles that end below p are asked for at once, while the predecessor still runs; the query, and
  // the tile that holds p, wait for it.
  int issued = 0;
  if (threadIdx.x == 0)
    for (; issued < DEC_STAGES && issued < n_tiles && key_begin + (issued + 1) * KT <= p; ++issued) issue(issued);
  pdl_wait();
  if (threadIdx.x == 0)
    for (; issued < DEC_STAGES && issued < n_tiles; ++issued) issue(issued);

  uint32_t qf[DH / 16][4];
  {
    const int g0 = lane >> 2, g1 = g0 + 8, kk = (lane & 3) * 2;
    const bf16* q0 = P.q + ((size_t)n * P.Hq + hk * G + g0) * DH;
    const bf16* q1 = P.q + ((size_t)n * P.Hq + hk * G + g1) * DH;
#pragma unroll
    for (int s = 0; s < DH / 16; ++s) {
      qf[s][0] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk) : 0u;
      qf[s][1] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk) : 0u;
      qf[s][2] = g0 < G ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk + 8) : 0u;
      qf[s][3] = g1 < G ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk + 8) : 0u;
    }
  }
  JLX_TL_MARK(0);
  const float sc = P.scale_log2 * temperature(p, P.attn_scale, P.floor_scale);
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  float o[DH / 8][4];
#pragma unroll
  for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  bool ok = true;
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t % DEC_STAGES;
    ok = __syncthreads_and(mbar_wait(smem_u32(&full_bar[st]), (t / DEC_STAGES) & 1));  // the same verdict for all
    if (!ok) {
      // a wait gave up: let the copies that are still under way land before the block leaves
      if (threadIdx.x == 0) {
        atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
        for (int u = t + 1; u < n_tiles && u < t + DEC_STAGES; ++u) mbar_wait(smem_u32(&full_bar[u % DEC_STAGES]), (u / DEC_STAGES) & 1);
      }
      break;
    }
    const int tile_key = key_begin + t * KT;
    const uint32_t kt = base + st * STAGE_BYTES, vt = kt + HALVES * HALF_BYTES;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kstep = 0; kstep < DH / 16; ++kstep) {
      const int key = warp * 16 + (lane >> 4) * 8 + (lane & 7);
      const int c = kstep * 2 + ((lane >> 3) & 1);  // 16-byte chunk of the row
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(kt + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
      mma_bf16(s[0], qf[kstep], b0, b1);
      mma_bf16(s[1], qf[kstep], b2, b3);
    }
    float mx[2] = {m[0], m[1]};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = tile_key + warp * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const bool in = key >= lo && key <= p;
        s[nt][e] = in ? s[nt][e] * sc : NEG_BIG;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) corr[h] = exp2f(m[h] - mx[h]);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = s[nt][e] > 0.5f * NEG_BIG ? exp2f(s[nt][e] - mx[e >> 1]) : 0.f;
        s[nt][e] = pv;
        rs[e >> 1] += pv;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
      rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
      l[h] = l[h] * corr[h] + rs[h];
      m[h] = mx[h];
    }
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
    for (int np = 0; np < DH / 16; ++np) {
      const int key = warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
      const int c = np * 2 + (lane >> 4);
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vt + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
      mma_bf16(o[np * 2], pa, b0, b1);
      mma_bf16(o[np * 2 + 1], pa, b2, b3);
    }
    __syncthreads();  // every warp is done reading this stage
    if (threadIdx.x == 0 && t + DEC_STAGES < n_tiles) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // order those reads before the copy's writes
      issue(t + DEC_STAGES);
    }
  }
  JLX_TL_MARK(1);
  if (!ok) return;
  float* red = reinterpret_cast<float*>(smem_raw + (base - smem_u32(smem_raw)));
  constexpr int LD = DH + 2;
  {
    const int r0 = lane >> 2, r1 = r0 + 8, col = (lane & 3) * 2;
    float* w0 = red + (warp * 16 + r0) * LD;
    float* w1 = red + (warp * 16 + r1) * LD;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      w0[i * 8 + col] = o[i][0]; w0[i * 8 + col + 1] = o[i][1];
      w1[i * 8 + col] = o[i][2]; w1[i * 8 + col + 1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      w0[DH] = m[0]; w0[DH + 1] = l[0];
      w1[DH] = m[1]; w1[DH + 1] = l[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * DH; idx += 128) {
    const int g = idx / DH, d = idx % DH;
    float mm = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, red[(w * 16 + g) * LD + DH]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(red[(w * 16 + g) * LD + DH] - mm);
      acc += red[(w * 16 + g) * LD + d] * f;
      ll += red[(w * 16 + g) * LD + DH + 1] * f;
    }
    const size_t row = ((size_t)slot * P.Hq + hk * G + g) * P.max_splits + split;
    P.part_o[row * DH + d] = acc;
    if (d == 0) {
      P.part_ml[row * 2] = mm;
      P.part_ml[row * 2 + 1] = ll;
    }
  }
}

// out[n, h, :] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m), splits in ascending order.
// The splits' (m, l) pairs are fetched by as many threads at once and kept in shared memory; with more than
// COMBINE_CACHE splits they are read from global memory again.
#define COMBINE_CACHE 512
template <int DH>
__global__ void attention_combine_kernel(const AttnParams P) {
  JLX_TL(TL_ATTN_COMBINE);
  __shared__ float ms[COMBINE_CACHE], wgt[COMBINE_CACHE];
  pdl_launch_dependents();
  // the token's row and position belong to the step's description, which no kernel of the step writes: they are read
  // while the split kernel still runs
  const int slot = blockIdx.x, n = P.rows ? P.rows[slot] : slot, h = blockIdx.y;
  const int p = P.positions[n];
  const int lo = first_key(p, P.chunk, P.window);
  const int splits = p / P.split_keys - lo / P.split_keys + 1;
  const size_t row = ((size_t)slot * P.Hq + h) * P.max_splits;
  const float2* ml = reinterpret_cast<const float2*>(P.part_ml) + row;
  const bool cached = splits <= COMBINE_CACHE;
  float mm = NEG_BIG, ll = 0.f;
  pdl_wait();
  if (cached) {
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
      const float2 v = ml[s];
      ms[s] = v.x;
      wgt[s] = v.y;
    }
    __syncthreads();
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, ms[s]);
    for (int s = 0; s < splits; ++s) ll += wgt[s] * exp2f(ms[s] - mm);
    __syncthreads();
    for (int s = threadIdx.x; s < splits; s += blockDim.x) wgt[s] = exp2f(ms[s] - mm) / ll;
    __syncthreads();
  } else {
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, ml[s].x);
    for (int s = 0; s < splits; ++s) ll += ml[s].y * exp2f(ml[s].x - mm);
  }
  const float* po = P.part_o + row * DH;
  for (int d = threadIdx.x; d < DH; d += blockDim.x) {
    float acc = 0.f;
    if (cached) {
#pragma unroll 8
      for (int s = 0; s < splits; ++s) acc += po[(size_t)s * DH + d] * wgt[s];
    } else {
      for (int s = 0; s < splits; ++s) acc += po[(size_t)s * DH + d] * (exp2f(ml[s].x - mm) / ll);
    }
    P.out[((size_t)n * P.Hq + h) * DH + d] = __float2bfloat16_rn(acc);
  }
}

// ----------------------------------------------------------------------------------- prefill
// grid (Hkv, n_tiles); G warps.  A tile is up to 16 consecutive tokens of one request; warp g owns the
// 16 x DH rows of query head g.  Key tiles of 64 are double-buffered.
template <int DH>
__global__ void __launch_bounds__(256) attention_prefill_kernel(const AttnParams P) {
  JLX_TL(TL_ATTN_PREFILL_MMA);
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int CH = DH / 8;
  constexpr int STAGES = 2;
  bf16* ks = reinterpret_cast<bf16*>(smem);          // [STAGES][KT][DH]
  bf16* vs = ks + STAGES * KT * DH;
  const int hk = blockIdx.x, tile = blockIdx.y;
  const int G = P.Hq / P.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = P.tiles[2 * tile], cnt = P.tiles[2 * tile + 1];
  const int r = P.req_of_token[n0];
  const int p_first = P.positions[n0], p_last = p_first + cnt - 1;
  const int lo_tile = first_key(p_first, P.chunk, P.window);  // start(p) grows with p: the tile's lowest
  const int key_begin = lo_tile / KT * KT;
  const int n_tiles = (p_last - key_begin) / KT + 1;
  const int NT = blockDim.x;

  // this thread's two rows: tokens lane/4 and lane/4 + 8 of head `warp`
  const int t0 = lane >> 2, t1 = t0 + 8;
  const int p0 = p_first + min(t0, cnt - 1), p1 = p_first + min(t1, cnt - 1);
  const int lo0 = first_key(p0, P.chunk, P.window), lo1 = first_key(p1, P.chunk, P.window);
  const bool row0 = t0 < cnt, row1 = t1 < cnt;
  uint32_t qf[DH / 16][4];
  {
    const int kk = (lane & 3) * 2;
    const bf16* q0 = P.q + ((size_t)(n0 + min(t0, cnt - 1)) * P.Hq + hk * G + warp) * DH;
    const bf16* q1 = P.q + ((size_t)(n0 + min(t1, cnt - 1)) * P.Hq + hk * G + warp) * DH;
#pragma unroll
    for (int s = 0; s < DH / 16; ++s) {
      qf[s][0] = row0 ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk) : 0u;
      qf[s][1] = row1 ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk) : 0u;
      qf[s][2] = row0 ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk + 8) : 0u;
      qf[s][3] = row1 ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk + 8) : 0u;
    }
  }
  const float sc0 = P.scale_log2 * temperature(p0, P.attn_scale, P.floor_scale);
  const float sc1 = P.scale_log2 * temperature(p1, P.attn_scale, P.floor_scale);
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  float o[DH / 8][4];
#pragma unroll
  for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // prologue: first tile
  load_kv_tile<DH>(P, r, hk, key_begin, lo_tile, p_last, ks, vs, NT);
  cp_async_commit();

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    // request the next tile into the other buffer (free since the barrier at the end of the last round)
    if (t + 1 < n_tiles)
      load_kv_tile<DH>(P, r, hk, key_begin + (t + 1) * KT, lo_tile, p_last, ks + (buf ^ 1) * KT * DH, vs + (buf ^ 1) * KT * DH, NT);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int tile_key = key_begin + t * KT;
    const bf16* kt = ks + buf * KT * DH;
    const bf16* vt = vs + buf * KT * DH;
    if (warp < G) {
      float s[KT / 8][4];
#pragma unroll
      for (int i = 0; i < KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kstep = 0; kstep < DH / 16; ++kstep) {
#pragma unroll
        for (int np = 0; np < KT / 16; ++np) {
          const int key = np * 16 + (lane >> 4) * 8 + (lane & 7);
          const int c = kstep * 2 + ((lane >> 3) & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(smem_u32(kt + (key * CH + (c ^ (key & 7))) * 8), b0, b1, b2, b3);
          mma_bf16(s[np * 2], qf[kstep], b0, b1);
          mma_bf16(s[np * 2 + 1], qf[kstep], b2, b3);
        }
      }
      float mx[2] = {m[0], m[1]};
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = tile_key + nt * 8 + (lane & 3) * 2 + (e & 1);
          const bool ok = (e < 2) ? (row0 && key >= lo0 && key <= p0) : (row1 && key >= lo1 && key <= p1);
          s[nt][e] = ok ? s[nt][e] * ((e < 2) ? sc0 : sc1) : NEG_BIG;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      }
      float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) corr[h] = exp2f(m[h] - mx[h]);
#pragma unroll
      for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = s[nt][e] > 0.5f * NEG_BIG ? exp2f(s[nt][e] - mx[e >> 1]) : 0.f;
          s[nt][e] = pv;
          rs[e >> 1] += pv;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
        l[h] = l[h] * corr[h] + rs[h];
        m[h] = mx[h];
      }
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
#pragma unroll
      for (int kp = 0; kp < KT / 16; ++kp) {
        uint32_t pa[4] = {pack_bf16(s[kp * 2][0], s[kp * 2][1]), pack_bf16(s[kp * 2][2], s[kp * 2][3]),
                          pack_bf16(s[kp * 2 + 1][0], s[kp * 2 + 1][1]), pack_bf16(s[kp * 2 + 1][2], s[kp * 2 + 1][3])};
#pragma unroll
        for (int np = 0; np < DH / 16; ++np) {
          const int key = kp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int c = np * 2 + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(smem_u32(vt + (key * CH + (c ^ (key & 7))) * 8), b0, b1, b2, b3);
          mma_bf16(o[np * 2], pa, b0, b1);
          mma_bf16(o[np * 2 + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();  // everyone is done with this buffer before the next round overwrites it
  }
  cp_async_wait<0>();
  if (warp < G) {
    const int col = (lane & 3) * 2;
    const float i0 = 1.f / l[0], i1 = 1.f / l[1];
    bf16* o0 = P.out + ((size_t)(n0 + t0) * P.Hq + hk * G + warp) * DH;
    bf16* o1 = P.out + ((size_t)(n0 + t1) * P.Hq + hk * G + warp) * DH;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      if (row0) *reinterpret_cast<__nv_bfloat162*>(o0 + i * 8 + col) = __floats2bfloat162_rn(o[i][0] * i0, o[i][1] * i0);
      if (row1) *reinterpret_cast<__nv_bfloat162*>(o1 + i * 8 + col) = __floats2bfloat162_rn(o[i][2] * i1, o[i][3] * i1);
    }
  }
}

// ---------------------------------------------------------------------------- prefill with TMA
// The flash kernel with its key/value tiles brought in by TMA (one thread issues a tile's boxes, as in the
// decode kernel) through a ring of PRE_STAGES stages, and with the 64-key tile scored in two halves of 32 keys
// so that the score fragment takes 16 registers instead of 32: two blocks share an SM.
#define PRE_STAGES 3

template <int DH>
__device__ __forceinline__ void tma_issue_tile(const CUtensorMap* map, const AttnParams& P, const int* table, int hk, int key0,
                                               uint32_t dst, uint32_t bar, int box_rows) {
  constexpr int HALVES = DH / 64;
  constexpr uint32_t HALF_BYTES = KT * 128;
  mbar_expect_tx(bar, 2 * HALVES * HALF_BYTES);
  for (int b = 0; b < KT / box_rows; ++b) {
    const int pos = key0 + b * box_rows;
    const int pi = pos / P.page_size;
    int page = pi < P.bt_stride ? table[pi] : -1;
    if (page >= P.num_pages) { atomicOr(P.status, JLX_STATUS_BAD_PAGE); page = 0; }
    if (page < 0) page = 0;  // no page there: every key of the box is masked
    const int row_k = ((page * 2 + 0) * P.Hkv + hk) * P.page_size + (pos - pi * P.page_size);
    const int row_v = ((page * 2 + 1) * P.Hkv + hk) * P.page_size + (pos - pi * P.page_size);
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
      tma_load_2d(dst + h * HALF_BYTES + b * box_rows * 128, map, h * 64, row_k, bar);
      tma_load_2d(dst + (HALVES + h) * HALF_BYTES + b * box_rows * 128, map, h * 64, row_v, bar);
    }
  }
}

template <int DH, int MAXW, int MINB>
__global__ void __launch_bounds__(MAXW * 32, MINB)
attention_prefill_tma_kernel(const __grid_constant__ CUtensorMap map, const AttnParams P, int box_rows) {
  JLX_TL(TL_ATTN_PREFILL_MMA);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  constexpr int HALVES = DH / 64;
  constexpr uint32_t HALF_BYTES = KT * 128;
  constexpr uint32_t STAGE_BYTES = 2 * HALVES * HALF_BYTES;
  __shared__ __align__(8) uint64_t full_bar[PRE_STAGES];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int hk = blockIdx.x, tile = blockIdx.y;
  const int G = P.Hq / P.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = P.tiles[2 * tile], cnt = P.tiles[2 * tile + 1];
  const int r = P.req_of_token[n0];
  const int p_first = P.positions[n0], p_last = p_first + cnt - 1;
  const int lo_tile = first_key(p_first, P.chunk, P.window);
  const int key_begin = lo_tile / KT * KT;
  const int n_tiles = (p_last - key_begin) / KT + 1;
  const int* table = P.block_table + (size_t)r * P.bt_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PRE_STAGES; ++s) mbar_init(smem_u32(&full_bar[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int t = 0; t < PRE_STAGES && t < n_tiles; ++t)
      tma_issue_tile<DH>(&map, P, table, hk, key_begin + t * KT, base + t * STAGE_BYTES, smem_u32(&full_bar[t]), box_rows);

  const int t0 = lane >> 2, t1 = t0 + 8;
  const int p0 = p_first + min(t0, cnt - 1), p1 = p_first + min(t1, cnt - 1);
  const int lo0 = first_key(p0, P.chunk, P.window), lo1 = first_key(p1, P.chunk, P.window);
  const bool row0 = t0 < cnt, row1 = t1 < cnt;
  uint32_t qf[DH / 16][4];
  {
    const int kk = (lane & 3) * 2;
    const bf16* q0 = P.q + ((size_t)(n0 + min(t0, cnt - 1)) * P.Hq + hk * G + warp) * DH;
    const bf16* q1 = P.q + ((size_t)(n0 + min(t1, cnt - 1)) * P.Hq + hk * G + warp) * DH;
#pragma unroll
    for (int s = 0; s < DH / 16; ++s) {
      qf[s][0] = row0 ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk) : 0u;
      qf[s][1] = row1 ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk) : 0u;
      qf[s][2] = row0 ? *reinterpret_cast<const uint32_t*>(q0 + s * 16 + kk + 8) : 0u;
      qf[s][3] = row1 ? *reinterpret_cast<const uint32_t*>(q1 + s * 16 + kk + 8) : 0u;
    }
  }
  const float sc0 = P.scale_log2 * temperature(p0, P.attn_scale, P.floor_scale);
  const float sc1 = P.scale_log2 * temperature(p1, P.attn_scale, P.floor_scale);
  float m[2] = {NEG_BIG, NEG_BIG}, l[2] = {0.f, 0.f};
  float o[DH / 8][4];
#pragma unroll
  for (int i = 0; i < DH / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  bool ok = true;
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t % PRE_STAGES;
    ok = __syncthreads_and(mbar_wait(smem_u32(&full_bar[st]), (t / PRE_STAGES) & 1));
    if (!ok) {
      if (threadIdx.x == 0) {
        atomicOr(P.status, JLX_STATUS_WAIT_TIMEOUT);
        for (int u = t + 1; u < n_tiles && u < t + PRE_STAGES; ++u) mbar_wait(smem_u32(&full_bar[u % PRE_STAGES]), (u / PRE_STAGES) & 1);
      }
      break;
    }
    const int tile_key = key_begin + t * KT;
    const uint32_t kt = base + st * STAGE_BYTES, vt = kt + HALVES * HALF_BYTES;
    // rows of this thread that see no key of the tile at all skip nothing: the masks below handle it
    const bool need_mask = tile_key + KT - 1 > p_first || tile_key < first_key(p_last, P.chunk, P.window) || cnt < 16;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kstep = 0; kstep < DH / 16; ++kstep) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          const int key = half * 32 + np * 16 + (lane >> 4) * 8 + (lane & 7);
          const int c = kstep * 2 + ((lane >> 3) & 1);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(kt + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma_bf16(s[np * 2], qf[kstep], b0, b1);
          mma_bf16(s[np * 2 + 1], qf[kstep], b2, b3);
        }
      }
      float mx[2] = {m[0], m[1]};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          bool in = true;
          if (need_mask) {
            const int key = tile_key + half * 32 + nt * 8 + (lane & 3) * 2 + (e & 1);
            in = (e < 2) ? (row0 && key >= lo0 && key <= p0) : (row1 && key >= lo1 && key <= p1);
          }
          s[nt][e] = in ? s[nt][e] * ((e < 2) ? sc0 : sc1) : NEG_BIG;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      }
      float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) corr[h] = exp2f(m[h] - mx[h]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = s[nt][e] > 0.5f * NEG_BIG ? exp2f(s[nt][e] - mx[e >> 1]) : 0.f;
          s[nt][e] = pv;
          rs[e >> 1] += pv;
        }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
        rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
        l[h] = l[h] * corr[h] + rs[h];
        m[h] = mx[h];
      }
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
#pragma unroll
      for (int kp = 0; kp < 2; ++kp) {
        uint32_t pa[4] = {pack_bf16(s[kp * 2][0], s[kp * 2][1]), pack_bf16(s[kp * 2][2], s[kp * 2][3]),
                          pack_bf16(s[kp * 2 + 1][0], s[kp * 2 + 1][1]), pack_bf16(s[kp * 2 + 1][2], s[kp * 2 + 1][3])};
#pragma unroll
        for (int np = 0; np < DH / 16; ++np) {
          const int key = half * 32 + kp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
          const int c = np * 2 + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(vt + (c >> 3) * HALF_BYTES + key * 128 + (((c & 7) ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma_bf16(o[np * 2], pa, b0, b1);
          mma_bf16(o[np * 2 + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();  // every warp is done reading this stage
    if (threadIdx.x == 0 && t + PRE_STAGES < n_tiles) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tma_issue_tile<DH>(&map, P, table, hk, key_begin + (t + PRE_STAGES) * KT, base + st * STAGE_BYTES,
                         smem_u32(&full_bar[st]), box_rows);
    }
  }
  if (!ok) return;
  {
    const int col = (lane & 3) * 2;
    const float i0 = 1.f / l[0], i1 = 1.f / l[1];
    bf16* o0 = P.out + ((size_t)(n0 + t0) * P.Hq + hk * G + warp) * DH;
    bf16* o1 = P.out + ((size_t)(n0 + t1) * P.Hq + hk * G + warp) * DH;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
      if (row0) *reinterpret_cast<__nv_bfloat162*>(o0 + i * 8 + col) = __floats2bfloat162_rn(o[i][0] * i0, o[i][1] * i0);
      if (row1) *reinterpret_cast<__nv_bfloat162*>(o1 + i * 8 + col) = __floats2bfloat162_rn(o[i][2] * i1, o[i][3] * i1);
    }
  }
}

// --------------------------------------------------------------------------------------- host
static int fill_params(AttnParams& P, const void* q, const void* pages, const int* block_table, int bt_stride,
                       const int* req_of_token, const int* positions, void* out, int Hq, int Hkv, int dh, int page_size,
                       int num_pages, float scale, int chunk, int window, float attn_scale, float floor_scale, int* status) {
  JLX_REQUIRE(Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "attention: %d query heads are no multiple of %d KV heads", Hq, Hkv);
  JLX_REQUIRE(dh == 64 || dh == 128, "attention_mma: head size %d is not built (64 and 128 are); use the generic kernel", dh);
  JLX_REQUIRE(page_size > 0 && num_pages > 0 && bt_stride > 0, "attention: bad cache sizes");
  JLX_REQUIRE(attn_scale == 0.f || floor_scale > 0.f, "attention: floor_scale must be positive");
  JLX_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)pages & 15) == 0, "attention: q and pages must be 16-byte aligned");
  P.q = (const bf16*)q; P.pages = (const bf16*)pages; P.block_table = block_table; P.bt_stride = bt_stride;
  P.req_of_token = req_of_token; P.positions = positions; P.out = (bf16*)out; P.Hq = Hq; P.Hkv = Hkv;
  P.page_size = page_size; P.num_pages = num_pages; P.scale_log2 = scale * 1.4426950408889634f;
  P.chunk = chunk; P.window = window; P.attn_scale = attn_scale; P.floor_scale = floor_scale; P.status = status;
  P.tiles = nullptr; P.part_o = nullptr; P.part_ml = nullptr; P.max_splits = 0; P.split_keys = SPLIT_UNIT; P.rows = nullptr;
  return 0;
}

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

// The cache of one layer as rows of one head each: [num_pages * 2 * Hkv * page_size, dh], boxes of
// [box_rows, 64 elements], 128-byte swizzle.
static int make_cache_map(CUtensorMap* map, const void* pages, long long rows, int dh, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  JLX_REQUIRE(fn != nullptr, "attention_decode: the driver does not offer cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)dh, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)dh * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  JLX_REQUIRE(r == CUDA_SUCCESS, "attention_decode: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}

JLX_API int jlx_attention_mma_supported(int Hq, int Hkv, int dh, int decode) {
  if (Hkv <= 0 || Hq % Hkv) return 0;
  const int G = Hq / Hkv;
  return (dh == 64 || dh == 128) && G <= (decode ? 16 : 8);
}

// Multiprocessors of the current device (asked once per device).
static int sm_count() {
  static int cached[64] = {0};
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Keys per decode split for `pairs` (request, KV head) pairs that read up to max_kv_len keys: a multiple
// of SPLIT_UNIT chosen so that all blocks are resident at once (two per SM): a second, partly filled round of
// blocks costs more than longer splits do.
JLX_API int jlx_attention_decode_split_keys(int max_kv_len, int chunk, int window, int pairs) {
  int span = max_kv_len;
  if (chunk > 0 && chunk < span) span = chunk;
  if (window > 0 && window < span) span = window;
  int want_splits = 2 * sm_count() / (pairs > 0 ? pairs : 1);
  if (want_splits < 1) want_splits = 1;
  int keys = (span + want_splits - 1) / (want_splits > 0 ? want_splits : 1);
  keys = (keys + SPLIT_UNIT - 1) / SPLIT_UNIT * SPLIT_UNIT;
  return keys < SPLIT_MIN ? SPLIT_MIN : keys;
}

// Splits a decode launch needs for requests of up to max_kv_len keys with that split size.
JLX_API int jlx_attention_decode_splits(int max_kv_len, int chunk, int window, int split_keys) {
  int span = max_kv_len;
  if (chunk > 0 && chunk < span) span = chunk;
  if (window > 0 && window < span) span = window;
  return (span + split_keys - 1) / split_keys + 1;
}

// One query token per request.  part_o: float [N * Hq * max_splits * dh]; part_ml: float [N * Hq * max_splits * 2].
// rows (optional): int [N], the token rows of q / positions / req_of_token / out to work on (a step that mixes
// prompt portions with decoded tokens sends only the latter here); null: rows 0..N-1.
JLX_API int jlx_attention_decode(const void* q, const void* pages, const int* block_table, int bt_stride,
                                 const int* req_of_token, const int* positions, void* out, int N, int Hq, int Hkv, int dh,
                                 int page_size, int num_pages, float scale, int chunk, int window, float attn_scale,
                                 float floor_scale, float* part_o, float* part_ml, int max_splits, int split_keys,
                                 const int* rows, int* status, cudaStream_t stream) {
  AttnParams P;
  if (fill_params(P, q, pages, block_table, bt_stride, req_of_token, positions, out, Hq, Hkv, dh, page_size, num_pages,
                  scale, chunk, window, attn_scale, floor_scale, status)) return 1;
  JLX_REQUIRE(Hq / Hkv <= 16, "attention_decode: %d query heads per KV head; up to 16 are supported", Hq / Hkv);
  JLX_REQUIRE(part_o && part_ml && max_splits > 0, "attention_decode: scratch for the partial results is missing");
  JLX_REQUIRE(split_keys > 0 && split_keys % SPLIT_UNIT == 0, "attention_decode: split size %d is no multiple of %d", split_keys, SPLIT_UNIT);
  JLX_REQUIRE(N <= 65535 && Hkv <= 65535, "attention_decode: too many rows");
  if (N == 0) return 0;
  P.part_o = part_o; P.part_ml = part_ml; P.max_splits = max_splits; P.split_keys = split_keys; P.rows = rows;
  const size_t smem = (size_t)2 * DEC_STAGES * KT * dh * 2;
  dim3 grid(max_splits, Hkv, N);
  // pages that hold whole 64-key tiles, or divide them, go through TMA; other page sizes through cp.async
  const bool tma = (page_size % KT == 0 || KT % page_size == 0) && page_size >= 8 &&
                   (long long)num_pages * 2 * Hkv * page_size < (1ll << 31);
  if (tma) {
    CUtensorMap map;
    const int box_rows = page_size < KT ? page_size : KT;
    if (make_cache_map(&map, pages, (long long)num_pages * 2 * Hkv * page_size, dh, box_rows)) return 1;
    if (dh == 128) {
      static bool cfg = false;
      if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem + 1024)); cfg = true; }
      JLX_CUDA(jlx_launch_pdl(attention_decode_tma_kernel<128>, grid, dim3(128), smem + 1024, stream, map, P, box_rows));
    } else {
      static bool cfg = false;
      if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(attention_decode_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem + 1024)); cfg = true; }
      JLX_CUDA(jlx_launch_pdl(attention_decode_tma_kernel<64>, grid, dim3(128), smem + 1024, stream, map, P, box_rows));
    }
    JLX_LAUNCH_CHECK("attention_decode_tma");
  } else if (dh == 128) {
    static bool cfg = false;
    if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(attention_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); cfg = true; }
    attention_decode_kernel<128><<<grid, 128, smem, stream>>>(P);
    JLX_LAUNCH_CHECK("attention_decode");
  } else {
    static bool cfg = false;
    if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(attention_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); cfg = true; }
    attention_decode_kernel<64><<<grid, 128, smem, stream>>>(P);
    JLX_LAUNCH_CHECK("attention_decode");
  }
  if (dh == 128) JLX_CUDA(jlx_launch_pdl(attention_combine_kernel<128>, dim3(N, Hq), dim3(128), 0, stream, P));
  else JLX_CUDA(jlx_launch_pdl(attention_combine_kernel<64>, dim3(N, Hq), dim3(64), 0, stream, P));
  JLX_LAUNCH_CHECK("attention_combine");
  return 0;
}

// tiles: int32 [n_tiles][2] on the device: (first token row, count <= 16), tokens of one request each.
JLX_API int jlx_attention_prefill(const void* q, const void* pages, const int* block_table, int bt_stride,
                                  const int* req_of_token, const int* positions, void* out, const int* tiles, int n_tiles,
                                  int Hq, int Hkv, int dh, int page_size, int num_pages, float scale, int chunk, int window,
                                  float attn_scale, float floor_scale, int* status, cudaStream_t stream) {
  AttnParams P;
  if (fill_params(P, q, pages, block_table, bt_stride, req_of_token, positions, out, Hq, Hkv, dh, page_size, num_pages,
                  scale, chunk, window, attn_scale, floor_scale, status)) return 1;
  const int G = Hq / Hkv;
  JLX_REQUIRE(G <= 8, "attention_prefill: %d query heads per KV head; up to 8 are supported", G);
  JLX_REQUIRE(Hkv <= 65535, "attention_prefill: too many KV heads");
  if (n_tiles == 0) return 0;
  P.tiles = tiles;
  // blocks are handed out by blockIdx.x first: every head of the list's first (heaviest) tile before lighter tiles
  JLX_REQUIRE(n_tiles <= 65535, "attention_prefill: %d tiles; up to 65535 are supported", n_tiles);
  dim3 grid(Hkv, n_tiles);
  const bool tma = (page_size % KT == 0 || KT % page_size == 0) && page_size >= 8 &&
                   (long long)num_pages * 2 * Hkv * page_size < (1ll << 31);
  if (tma) {
    CUtensorMap map;
    const int box_rows = page_size < KT ? page_size : KT;
    if (make_cache_map(&map, pages, (long long)num_pages * 2 * Hkv * page_size, dh, box_rows)) return 1;
    const size_t smem = (size_t)PRE_STAGES * 2 * KT * dh * 2 + 1024;
#define PREFILL_TMA(DHV, MAXW, MINB)                                                                                       \
    do {                                                                                                                   \
      static bool cfg = false;                                                                                             \
      if (!cfg) {                                                                                                          \
        JLX_CUDA(cudaFuncSetAttribute(attention_prefill_tma_kernel<DHV, MAXW, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        JLX_CUDA(cudaFuncSetAttribute(attention_prefill_tma_kernel<DHV, MAXW, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));    \
        cfg = true;                                                                                                        \
      }                                                                                                                    \
      attention_prefill_tma_kernel<DHV, MAXW, MINB><<<grid, G * 32, smem, stream>>>(map, P, box_rows);                      \
    } while (0)
    if (dh == 128 && G <= 5) PREFILL_TMA(128, 5, 2);
    else if (dh == 128) PREFILL_TMA(128, 8, 1);
    else if (G <= 5) PREFILL_TMA(64, 5, 2);
    else PREFILL_TMA(64, 8, 1);
#undef PREFILL_TMA
    JLX_LAUNCH_CHECK("attention_prefill_tma");
    return 0;
  }
  const size_t smem = (size_t)2 * 2 * KT * dh * 2;
  if (dh == 128) {
    static bool cfg = false;
    if (!cfg) { JLX_CUDA(cudaFuncSetAttribute(attention_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); cfg = true; }
    attention_prefill_kernel<128><<<grid, G * 32, smem, stream>>>(P);
  } else {
    attention_prefill_kernel<64><<<grid, G * 32, smem, stream>>>(P);
  }
  JLX_LAUNCH_CHECK("attention_prefill");
  return 0;
}
