// C = A * W^T on the CUDA cores with 32-bit FMA: the matrix product of the true 32-bit path (no
// tensor cores, so no reduced-precision matrix mode can slip in), and of weights that are stored
// in 32-bit while activations are bfloat16.  A: [M, K] row-major, W: [N, K] row-major (the [out, in]
// orientation of the stored Linear weights), C: [M, N].
//
// Grouped form: rows [offsets[e], offsets[e+1]) of A multiply W_e = W + e * w_group_stride
// (the ragged product of llama4/llama4_jax/model.py:975-996).  offsets live on the device, so the
// grid is sized for the worst case and surplus blocks leave at once.
//
// Every output element sums its K products in the same order whatever M is, so a row's result does
// not depend on the other rows of the batch.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16
#define LDS 68  // padded row of the shared tiles (floats); 16-byte aligned for float4 reads

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C, int M, int N, int K,
                 long long lda, long long ldw, long long ldc, const int* __restrict__ offsets, int E,
                 long long w_group_stride) {
  JLX_TL(TL_GEMM_SIMT);
  __shared__ __align__(16) float As[BK][LDS];
  __shared__ __align__(16) float Ws[BK][LDS];

  int m0, m_end;
  const TW* Wg = W;
  if (offsets) {
    // find this block's (group, row tile)
    int t = blockIdx.y, e = 0, found = 0;
    for (; e < E; ++e) {
      const int lo = offsets[e], hi = offsets[e + 1];
      const int tiles = (hi - lo + BM - 1) / BM;
      if (t < tiles) {
        m0 = lo + t * BM;
        m_end = hi;
        found = 1;
        break;
      }
      t -= tiles;
    }
    if (!found) return;
    Wg = W + (size_t)e * w_group_stride;
  } else {
    m0 = blockIdx.y * BM;
    m_end = M;
    if (m0 >= M) return;
  }
  const int n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int lr = tid >> 2, lk = (tid & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + j][lr] = (am < m_end && k < K) ? to_f32<TA>(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + j][lr] = (wn < N && k < K) ? to_f32<TW>(Wg[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                  long long ldc, const int* offsets, int E, long long wgs, cudaStream_t stream) {
  const int row_tiles = (M + BM - 1) / BM + (offsets ? E : 0);
  JLX_REQUIRE(row_tiles <= 65535, "gemm_simt: too many row tiles (%d)", row_tiles);
  dim3 grid((N + BN - 1) / BN, row_tiles);
  gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc,
                                                        offsets, E, wgs);
  JLX_LAUNCH_CHECK("gemm_simt");
  return 0;
}

// M is the row count (dense) or an upper bound of offsets[E] (grouped).
JLX_API int jlx_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M, int N,
                          int K, long long lda, long long ldw, long long ldc, const int* offsets, int E,
                          long long w_group_stride, cudaStream_t stream) {
  JLX_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  JLX_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_simt: a leading dimension is smaller than its row");
  JLX_REQUIRE(!offsets || E > 0, "gemm_simt: grouped product needs a group count");
  if (M == 0) return 0;
#define GO(TA, TW, TC) return launch<TA, TW, TC>(A, W, C, M, N, K, lda, ldw, ldc, offsets, E, w_group_stride, stream)
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
  switch (code) {
    case 0: GO(float, float, float);
    case 1: GO(float, float, bf16);
    case 2: GO(float, bf16, float);
    case 3: GO(float, bf16, bf16);
    case 4: GO(bf16, float, float);
    case 5: GO(bf16, float, bf16);
    case 6: GO(bf16, bf16, float);
    case 7: GO(bf16, bf16, bf16);
  }
#undef GO
  JLX_REQUIRE(false, "gemm_simt: unknown element type codes %d %d %d", a_dtype, w_dtype, c_dtype);
}
