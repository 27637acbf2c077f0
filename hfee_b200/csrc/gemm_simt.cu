// out[M,N] (+)= A[M,K] . W[N,K]^T with float32 FFMA accumulation on the CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no
// reduced-precision mode) and the fallback of the bfloat16 path for shapes the
// tensor-core kernels refuse.  Every output element is the sum over k = 0..K-1 in
// that order, whatever M is, so a row's result does not depend on the batch.
// Reference: out[t*Rows+r] = Dot(W[r,:], x[t,:]), hostfog/hfee internal/ggml/ops.go:54-70.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename T>
__device__ __forceinline__ float load_guarded(const T* p, long long ld, int r, int c, int rows, int cols) {
  return (r < rows && c < cols) ? to_f32<T>(p[(long long)r * ld + c]) : 0.f;
}

// TOut: float or bf16.  ACCUM (float out only): out += product (the residual add).
template <typename TIn, typename TOut, bool ACCUM>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const TIn* __restrict__ A, long long lda, const TIn* __restrict__ W, long long ldw,
                 TOut* __restrict__ C, long long ldc, int M, int N, int K) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  int tid = threadIdx.x;
  int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int tr = tid / (BN / TN), tc = tid % (BN / TN);   // 16 x 16 thread grid
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread stages 4 consecutive k of one row of A and one row of W
  int lr = tid / (BK / 4), lk = (tid % (BK / 4)) * 4;   // 64 rows x 4 groups
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      As[lk + j][lr] = load_guarded(A, lda, m0 + lr, k0 + lk + j, M, K);
      Ws[lk + j][lr] = load_guarded(W, ldw, n0 + lr, k0 + lk + j, N, K);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][tr * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tc * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int r = m0 + tr * TM + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int c = n0 + tc * TN + j;
      if (c >= N) continue;
      long long o = (long long)r * ldc + c;
      if constexpr (ACCUM) C[o] = to_f32<TOut>(C[o]) + acc[i][j];
      else C[o] = from_f32<TOut>(acc[i][j]);
    }
  }
}

template <typename TIn>
int launch(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
           int accumulate, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (out_dtype == HFEE_F32) {
    if (accumulate)
      hfee_launch(gemm_simt_kernel<TIn, float, true>, dim3(grid), dim3(THREADS), 0, stream, (const TIn*)A, lda, (const TIn*)W, ldw, (float*)C, ldc, M, N, K);
    else
      hfee_launch(gemm_simt_kernel<TIn, float, false>, dim3(grid), dim3(THREADS), 0, stream, (const TIn*)A, lda, (const TIn*)W, ldw, (float*)C, ldc, M, N, K);
  } else if (out_dtype == HFEE_BF16) {
    if (accumulate) return hfee_fail(HFEE_ERR_ARG, "gemm_simt: accumulate needs a float32 output");
    hfee_launch(gemm_simt_kernel<TIn, __nv_bfloat16, false>, dim3(grid), dim3(THREADS), 0, stream, (const TIn*)A, lda, (const TIn*)W, ldw, (__nv_bfloat16*)C, ldc, M, N, K);
  } else {
    return hfee_fail(HFEE_ERR_ARG, "gemm_simt: unknown output dtype %d", out_dtype);
  }
  return hfee_check_launch("gemm_simt");
}

}  // namespace

HFEE_API int hfee_gemm_simt(const void* A, long long lda, const void* W, long long ldw, int in_dtype, void* C,
                            long long ldc, int out_dtype, int accumulate, int M, int N, int K,
                            cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N,
               "gemm_simt: bad sizes M=%d N=%d K=%d lda=%lld ldw=%lld ldc=%lld", M, N, K, lda, ldw, ldc);
  HFEE_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_simt: M=%d is too large", M);
  if (in_dtype == HFEE_F32) return launch<float>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
  if (in_dtype == HFEE_BF16) return launch<__nv_bfloat16>(A, lda, W, ldw, C, ldc, out_dtype, accumulate, M, N, K, stream);
  return hfee_fail(HFEE_ERR_ARG, "gemm_simt: unknown input dtype %d", in_dtype);
}
