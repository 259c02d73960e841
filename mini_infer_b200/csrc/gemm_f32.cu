// True 32-bit matrix product on CUDA cores:  C[M,N] = A[M,K] * W[N,K]^T
// (both operands K-contiguous, as linear layers store them).  No tensor cores, no
// reduced-precision mode.  Every output element is accumulated over k = 0..K-1 in that
// order with fused multiply-adds, whatever tile it falls in and whatever tile shape is
// chosen, so a row's result does not depend on which other rows share the call.
#include "common.cuh"

MI_DEFINE_ERROR_API()

template <int BM, int BN, int BK, int TM, int TN, bool VEC>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C,
                int M, int N, int K, int lda, int ldw, int ldc) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  constexpr int THREADS = (BM / TM) * (BN / TN);
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    if (VEC) {
      // BK % 4 == 0, K % 4 == 0, rows 16-byte aligned
      for (int idx = tid; idx < BM * (BK / 4); idx += THREADS) {
        const int r = idx / (BK / 4), c = (idx % (BK / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m0 + r < M && k0 + c < K) v = *reinterpret_cast<const float4*>(A + (size_t)(m0 + r) * lda + k0 + c);
        As[c + 0][r] = v.x; As[c + 1][r] = v.y; As[c + 2][r] = v.z; As[c + 3][r] = v.w;
      }
      for (int idx = tid; idx < BN * (BK / 4); idx += THREADS) {
        const int r = idx / (BK / 4), c = (idx % (BK / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n0 + r < N && k0 + c < K) v = *reinterpret_cast<const float4*>(W + (size_t)(n0 + r) * ldw + k0 + c);
        Ws[c + 0][r] = v.x; Ws[c + 1][r] = v.y; Ws[c + 2][r] = v.z; Ws[c + 3][r] = v.w;
      }
    } else {
      for (int idx = tid; idx < BM * BK; idx += THREADS) {
        const int r = idx / BK, c = idx % BK;
        As[c][r] = (m0 + r < M && k0 + c < K) ? A[(size_t)(m0 + r) * lda + k0 + c] : 0.f;
      }
      for (int idx = tid; idx < BN * BK; idx += THREADS) {
        const int r = idx / BK, c = idx % BK;
        Ws[c][r] = (n0 + r < N && k0 + c < K) ? W[(size_t)(n0 + r) * ldw + k0 + c] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
    }
  }
}

template <int BM, int BN, int BK, int TM, int TN>
static void launch(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw,
                   int ldc, bool vec, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  constexpr int THREADS = (BM / TM) * (BN / TN);
  if (vec)
    MI_LAUNCH((gemm_f32_kernel<BM, BN, BK, TM, TN, true>), grid, THREADS, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
  else
    MI_LAUNCH((gemm_f32_kernel<BM, BN, BK, TM, TN, false>), grid, THREADS, 0, stream, A, W, C, M, N, K, lda, ldw, ldc);
}

// Zero-padded K tails add exact zeros at the end of the sum, so they do not change it.
extern "C" int mi_gemm_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                           int ldw, int ldc, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) MI_REFUSE("gemm_f32: K must be positive, got %d", K);
  if (lda < K || ldw < K || ldc < N) MI_REFUSE("gemm_f32: leading dimensions too small");
  if ((M + 15) / 16 > 65535) MI_REFUSE("gemm_f32: too many rows (%d)", M);
  const bool vec = (K % 4 == 0) && (lda % 4 == 0) && (ldw % 4 == 0) && mi_aligned(A, 16) && mi_aligned(W, 16);
  if (M <= 16)
    launch<16, 128, 16, 1, 8>(A, W, C, M, N, K, lda, ldw, ldc, vec, stream);
  else if (M <= 64)
    launch<64, 64, 16, 4, 4>(A, W, C, M, N, K, lda, ldw, ldc, vec, stream);
  else
    launch<128, 128, 8, 8, 8>(A, W, C, M, N, K, lda, ldw, ldc, vec, stream);
  MI_RETURN_LAUNCH_STATUS();
}
