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
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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
