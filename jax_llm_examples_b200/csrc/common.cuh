// Shared helpers of the kernel libraries.  Every .cu file of this folder is built into a
// shared library of its own (sm_100a) and exports plain C launchers: raw device pointers, sizes
// and a stream in, an error code out (0 = launched; otherwise jlx_last_error() has the reason).
// A launcher refuses sizes that its kernel cannot take; it never runs with a wrong result.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define JLX_API extern "C" __attribute__((visibility("default")))

// element types at the C boundary
enum { JLX_F32 = 0, JLX_BF16 = 1 };

// bits of the device status word that kernels raise instead of faulting
enum {
  JLX_STATUS_BAD_PAGE = 1,      // a block-table entry outside the page pool
  JLX_STATUS_BAD_TOKEN = 2,     // a token id outside the vocabulary
  JLX_STATUS_BAD_EXPERT = 4,    // a routed expert index outside the expert count
  JLX_STATUS_WAIT_TIMEOUT = 8,  // a bounded wait on a barrier gave up
};

static thread_local char jlx_error_text[512] = "";

JLX_API const char* jlx_last_error() { return jlx_error_text; }

#define JLX_REQUIRE(cond, ...)                                   \
  do {                                                           \
    if (!(cond)) {                                               \
      snprintf(jlx_error_text, sizeof(jlx_error_text), __VA_ARGS__); \
      return 1;                                                  \
    }                                                            \
  } while (0)

#define JLX_LAUNCH_CHECK(name)                                                             \
  do {                                                                                     \
    cudaError_t e__ = cudaGetLastError();                                                  \
    if (e__ != cudaSuccess) {                                                              \
      snprintf(jlx_error_text, sizeof(jlx_error_text), "%s: %s", name, cudaGetErrorString(e__)); \
      return 2;                                                                            \
    }                                                                                      \
  } while (0)

#define JLX_CUDA(call)                                                                     \
  do {                                                                                     \
    cudaError_t e__ = (call);                                                              \
    if (e__ != cudaSuccess) {                                                              \
      snprintf(jlx_error_text, sizeof(jlx_error_text), "%s: %s", #call, cudaGetErrorString(e__)); \
      return 2;                                                                            \
    }                                                                                      \
  } while (0)

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Dispatch a runtime element type to a template argument.
#define JLX_DISPATCH_DTYPE(dtype, T, ...)                          \
  do {                                                             \
    if ((dtype) == JLX_F32) { typedef float T; __VA_ARGS__; }      \
    else if ((dtype) == JLX_BF16) { typedef bf16 T; __VA_ARGS__; } \
    else JLX_REQUIRE(false, "unknown element type code %d", (int)(dtype)); \
  } while (0)

// ---- programmatic dependent launch: a kernel launched with JLX_LAUNCH_PDL may start while its predecessor in
// the stream still runs.  It must call pdl_wait() before it reads or writes anything that a predecessor
// touches; what comes before (barrier set-up, tensor-memory allocation, loads of weights) overlaps the
// predecessor's tail.  pdl_launch_dependents() lets the successor start the same way.
// ---- device timeline (only when compiled with -DJLX_TIMELINE): thread 0 of every block notes the global timer when
// the block starts, when its wait for the predecessor ends and when it leaves, so that the kernels of a replayed
// graph, which no host-side timer can tell apart, can be laid out on one time axis.  A record is eight 64-bit
// words: {kernel id | gridDim.x << 8 | gridDim.y << 24 | gridDim.z << 40 | (block 0 of the grid) << 63, start, waited
// (0: the thread never waited), end, mark 0..3 (0: not passed)}; word 0 of the buffer counts the records asked for.  JLX_TL_MARK(i) notes
// the time at a place inside a kernel (thread 0 only), to see which stretch of a short kernel takes its time.
enum JlxTimelineId {
  TL_EMBED = 1, TL_NORM, TL_NORM_ROUTER, TL_GEMM, TL_GEMM_PAIR, TL_ROPE, TL_ATTN_DECODE, TL_ATTN_COMBINE, TL_SORT, TL_PERMUTE,
  TL_ARGMAX, TL_ATTN_PREFILL, TL_ROUTER, TL_OTHER, TL_ATTN_GENERIC, TL_GEMM_SIMT, TL_SAMPLE, TL_KV_STORE, TL_MOE_COMBINE,
  TL_SPLITK_REDUCE, TL_SILU_MUL, TL_ATTN_PREFILL_MMA, TL_ATTN_DECODE_PLAIN
};
#ifdef JLX_TIMELINE
__device__ unsigned long long* jlx_tl_buf = nullptr;
__device__ unsigned int jlx_tl_cap = 0;
JLX_API int jlx_timeline_set(unsigned long long* buf, unsigned int cap) {
  if (cudaMemcpyToSymbol(jlx_tl_buf, &buf, sizeof(buf)) != cudaSuccess) return 1;
  return cudaMemcpyToSymbol(jlx_tl_cap, &cap, sizeof(cap)) != cudaSuccess;
}
__device__ __forceinline__ unsigned long long jlx_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long* jlx_tl_waited() {
  __shared__ unsigned long long t[5];  // the end of the wait, then the marks
  return t;
}
struct JlxTimelineScope {
  unsigned long long t0;
  int id;
  __device__ __forceinline__ explicit JlxTimelineScope(int id_) : t0(jlx_now()), id(id_) {
    if (threadIdx.x == 0 && threadIdx.y == 0)
      for (int i = 0; i < 5; ++i) jlx_tl_waited()[i] = 0;
  }
  __device__ __forceinline__ ~JlxTimelineScope() {
    if (threadIdx.x != 0 || threadIdx.y != 0 || jlx_tl_buf == nullptr) return;
    const unsigned long long t_end = jlx_now();  // before the atomic below, whose round trip is no part of the kernel
    const unsigned long long slot = atomicAdd(jlx_tl_buf, 1ull);
    if (slot >= jlx_tl_cap) return;
    unsigned long long* r = jlx_tl_buf + 1 + 8 * slot;
    const bool first = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    r[0] = (unsigned long long)id | ((unsigned long long)(gridDim.x & 0xffff) << 8) | ((unsigned long long)(gridDim.y & 0xffff) << 24) |
           ((unsigned long long)(gridDim.z & 0xff) << 40) | ((unsigned long long)first << 63);
    r[1] = t0;
    r[2] = *jlx_tl_waited();
    r[3] = t_end;
    for (int i = 0; i < 4; ++i) r[4 + i] = jlx_tl_waited()[1 + i];
  }
};
#define JLX_TL(id) JlxTimelineScope jlx_tl_scope(id)
#define JLX_TL_MARK(i) do { if (threadIdx.x == 0 && threadIdx.y == 0) jlx_tl_waited()[1 + (i)] = jlx_now(); } while (0)
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0 && threadIdx.y == 0) *jlx_tl_waited() = jlx_now();
}
#else
#define JLX_TL(id) do { } while (0)
#define JLX_TL_MARK(i) do { } while (0)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Rehearsal.  A short kernel of a decode step runs on a block or a handful, once per layer, on whichever SM is free:
// it finds none of its code in that SM's instruction cache, and fetching it line by line after the wait for the
// predecessor took as long as the kernel's work.  Such a kernel starts while its predecessor still runs (programmatic
// dependent launch) and has nothing to do until that ends, so it spends the wait running its own code once with
// every load of a predecessor's data and every store switched off (a pass of a loop that the compiler may not
// unroll, so that both passes are the same instructions), which brings the code in.  Only small grids do this: with
// many blocks the code is warm after the first and the second pass would only cost time.  And only kernels that start
// well before their predecessor ends: one that follows a matrix product whose blocks fill every SM gets its SMs
// microseconds before its work, and a rehearsal would then delay it (measured; see the norm kernels).
#define JLX_REHEARSAL_MAX_BLOCKS 512
__device__ __forceinline__ bool jlx_rehearses() { return gridDim.x * gridDim.y * gridDim.z <= JLX_REHEARSAL_MAX_BLOCKS; }

// Asks [p, p + bytes) into L2, the block's threads taking a line each; nothing waits for it.  For weights that a
// short kernel reads right after its wait for the predecessor: asked for before the wait, they arrive during it.
__device__ __forceinline__ void l2_prefetch_block(const void* p, size_t bytes) {
  const char* c = reinterpret_cast<const char*>(p);
  for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)blockDim.x * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}

template <typename... KArgs, typename... Args>
static cudaError_t jlx_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
