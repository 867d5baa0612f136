// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores: plain float32 multiply-adds, no tensor
// cores, no reduced-precision mode.  This is the matrix product of the true 32-bit path and
// the fallback for shapes the tensor-core kernels refuse.  The reference's GEMV
// (cuda/src/cuda_backend.cu:291-312, out[r] = dot(W[r,:], x)) computes the same numbers one
// row at a time.
//
// Each output element is accumulated by one thread walking k = 0..K-1 in ascending order,
// so a value does not depend on M, on the tile it falls in, or on anything else in the batch.
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A,
                                                        const TW* __restrict__ W, int M, int N, int K,
                                                        int lda, int ldw, int ldc, int accumulate) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 elements per operand, 256 threads -> 4 each; consecutive threads read along k
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int e = tid + it * 256;
      const int r = e >> 4, kk = e & 15;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? to_f(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[kk][r] = (gn < N && gk < K) ? to_f(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      TC* c = C + (size_t)gm * ldc + gn;
      float v = acc[i][j];
      if (accumulate) v += to_f(*c);
      *c = from_f<TC>(v);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch(void* C, const void* A, const void* W, int M, int N, int K, int lda, int ldw,
                  int ldc, int accumulate, cudaStream_t st) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return QV_ERR_TOO_LARGE;
  gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, st>>>((TC*)C, (const TA*)A, (const TW*)W, M, N, K, lda,
                                                     ldw, ldc, accumulate);
  return qv_launch_status();
}

// dtypes: a_dt/w_dt/c_dt in {f32, bf16}; accumulate != 0 adds to what C holds.
extern "C" int qv_gemm_simt(void* C, const void* A, const void* W, int M, int N, int K, int lda,
                            int ldw, int ldc, int a_dt, int w_dt, int c_dt, int accumulate,
                            void* stream) {
  if (M <= 0 || N <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int key = a_dt * 4 + w_dt * 2 + c_dt;
  switch (key) {
    case 0: return launch<float, float, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 1: return launch<float, float, bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 2: return launch<float, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 3: return launch<float, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 4: return launch<bf16, float, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 5: return launch<bf16, float, bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 6: return launch<bf16, bf16, float>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
    case 7: return launch<bf16, bf16, bf16>(C, A, W, M, N, K, lda, ldw, ldc, accumulate, st);
  }
  return QV_ERR_UNSUPPORTED;
}
