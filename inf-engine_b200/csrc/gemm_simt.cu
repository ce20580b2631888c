// C[M,N] = A[M,K] * W[N,K]^T on CUDA cores in float32 (FFMA, no tensor cores,
// no reduced-precision mode), for the true 32-bit path and for weights that a
// checkpoint stores in 32-bit.  Weights keep the (out, in) layout of the
// checkpoint, y = x W^T (engine/layers.py:48-50).
//
// Every output element is one accumulator that walks k = 0..K-1 in ascending
// order, so a row's result does not depend on how many rows share the launch.
// A, W and C may each be float32 or bfloat16; products and sums are float32.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16
#define GS_THREADS 256

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(GS_THREADS) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                                TC* __restrict__ C, int M, int N, int K, int lda,
                                                                int ldw, int ldc, long long a_batch, long long w_batch,
                                                                long long c_batch) {
  pdl_trigger();
  pdl_wait();
  A += (size_t)blockIdx.z * a_batch;      // a batch of independent products (blockIdx.z), each with its own offsets
  W += (size_t)blockIdx.z * w_batch;
  C += (size_t)blockIdx.z * c_batch;
  __shared__ float As[GS_BK][GS_BM + 4];
  __shared__ float Ws[GS_BK][GS_BN + 4];
  const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads, 4 x 4 outputs each
  const int lr = tid >> 2, lc = (tid & 3) * 4;  // loader: row 0..63, k offset 0,4,8,12
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lc + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lc + u][lr] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.f;
      Ws[lc + u][lr] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GS_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch_gemm(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                       cudaStream_t stream, int batch = 1, long long a_batch = 0, long long w_batch = 0,
                       long long c_batch = 0) {
  dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM, batch);
  return launch_k(gemm_simt_kernel<TA, TW, TC>, grid, GS_THREADS, 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N,
                  K, lda, ldw, ldc, a_batch, w_batch, c_batch);
}

extern "C" int ie_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M,
                            int N, int K, int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IE_OK;
  if (K <= 0) return IE_BAD_SIZE;
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
  switch (code) {
    case 0: return launch_gemm<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 2: return launch_gemm<float, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 4: return launch_gemm<bf16, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 5: return launch_gemm<bf16, float, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 6: return launch_gemm<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    case 7: return launch_gemm<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
    default: return IE_BAD_DTYPE;
  }
}

// `batch` independent products in one launch: product b reads A + b * a_batch, W + b * w_batch and writes
// C + b * c_batch (offsets in elements).  A block-diagonal matrix applied to the rows of A is such a batch: block b
// reads columns b * K .. of A and writes columns b * N .. of C.
extern "C" int ie_gemm_simt_batched(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype, int M,
                                    int N, int K, int lda, int ldw, int ldc, int batch, long long a_batch,
                                    long long w_batch, long long c_batch, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return IE_OK;
  if (K <= 0 || batch > 65535) return IE_BAD_SIZE;
  const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
  switch (code) {
    case 0: return launch_gemm<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream, batch, a_batch, w_batch, c_batch);
    case 2: return launch_gemm<float, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream, batch, a_batch, w_batch, c_batch);
    case 4: return launch_gemm<bf16, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream, batch, a_batch, w_batch, c_batch);
    case 6: return launch_gemm<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream, batch, a_batch, w_batch, c_batch);
    default: return IE_BAD_DTYPE;
  }
}

// ------------------------------------------------------------------ few output columns (a router)
// C[m, n] = sum_k A[m, k] W[n, k] for N of a few dozen: the tile kernel above would give all of it to one block
// that walks K alone.  Here a block takes a row of A into shared memory and each of its eight warps takes outputs
// n = warp, warp + 8, ...: the lanes stride k with four partial sums each, then a tree over the lanes.  The order is
// fixed by (n, k) alone, so a row's result does not depend on how many rows share the launch.  float32 arithmetic.
template <typename TA, typename TW>
__global__ void __launch_bounds__(256) gemm_rowdot_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                          float* __restrict__ C, int N, int K, int lda, int ldw, int ldc) {
  extern __shared__ float a_s[];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  for (int k = threadIdx.x; k < K; k += blockDim.x) a_s[k] = to_f32(A[(size_t)m * lda + k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // blocks along y share a row's outputs in groups of eight (a few rows then still fill the device)
  for (int n = blockIdx.y * 8 + warp; n < N; n += 8 * gridDim.y) {
    const TW* w = W + (size_t)n * ldw;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int k = lane;
    for (; k + 96 < K; k += 128) {
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = fmaf(a_s[k + 32 * u], to_f32(w[k + 32 * u]), acc[u]);
    }
    for (int u = 0; k < K; k += 32, ++u) acc[u & 3] = fmaf(a_s[k], to_f32(w[k]), acc[u & 3]);
    const float total = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
    if (lane == 0) C[(size_t)m * ldc + n] = total;
  }
}

extern "C" int ie_gemm_rowdot(const void* A, int a_dtype, const void* W, int w_dtype, float* C, int M, int N, int K,
                              int lda, int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IE_OK;
  if (K <= 0 || (size_t)K * sizeof(float) > 200 * 1024) return IE_BAD_SIZE;
  const size_t smem = (size_t)K * sizeof(float);
  // few rows (decode tokens): a block a row and eight outputs, so that the weight rows stream through many blocks
  const dim3 grid(M, M <= 128 ? (N + 7) / 8 : 1);
#define RD_GO(TA, TW)                                                                                              \
  {                                                                                                                \
    if (smem > 47 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(gemm_rowdot_kernel<TA, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                             \
      if (e != cudaSuccess) return (int)e;                                                                         \
    }                                                                                                              \
    return launch_k(gemm_rowdot_kernel<TA, TW>, grid, 256, smem, stream, (const TA*)A, (const TW*)W, C, N, K, lda, ldw, \
                    ldc);                                                                                          \
  }
  if (a_dtype == IE_F32 && w_dtype == IE_F32) RD_GO(float, float);
  if (a_dtype == IE_F32 && w_dtype == IE_BF16) RD_GO(float, bf16);
  if (a_dtype == IE_BF16 && w_dtype == IE_F32) RD_GO(bf16, float);
  if (a_dtype == IE_BF16 && w_dtype == IE_BF16) RD_GO(bf16, bf16);
#undef RD_GO
  return IE_BAD_DTYPE;
}
