// Weight-streaming matrix product for few rows:  out[M, N] = x[M, K] * W[N, K]^T,  M <= 16,
// bfloat16 operands, fp32 accumulation on tensor cores (mma.sync m16n8k16).
//
// At decode time every weight is read once and used for a handful of tokens, so the
// product is bound by HBM; the kernel is organised around the weight stream:
//
//   * W is the A operand (16 rows of W per MMA), x^T is the B operand (8 tokens per MMA).
//   * A lane fetches weights 16 bytes at a time in exactly the shape of its A fragments: the
//     MMA's k index may be any permutation of the true k as long as A and B agree, so a lane
//     that holds 8 consecutive k of one row feeds two MMAs (true k = 32 j + 8 t + 4 u + {0,1}
//     and + {2,3} for k-step u of block j, lane t = lane % 4).  No ldmatrix, no transposes.
//     x is read with the same pattern (it is small and stays in L1/L2).
//   * One block owns 16 rows of W; its 8 warps take the 32-wide k blocks round-robin (so the
//     block as a whole reads contiguous 512-byte runs of each row) and are summed through
//     shared memory in a fixed order.
//
// K must be a multiple of 8 and rows 16-byte aligned; other shapes are refused.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// NT: number of 8-token tiles (1 or 2).  OutT: bf16 or float.
//
// Each warp streams its share of the 16 weight rows through a private ring of SK_STAGES
// shared-memory stages filled by cp.async (SK_GROUP k blocks, both row halves, 16 bytes per
// lane each): a lane only ever reads back the bytes it copied itself, so no block-wide
// barrier is needed, and SK_STAGES - 1 stages (6 KB per warp) are always in flight.
#define SK_STAGES 4
#define SK_GROUP 2

template <int NT, typename OutT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out, int M, int N,
                   int K, int ldx, int ldw, int ldo) {
  extern __shared__ __align__(16) unsigned char sk_smem[];
  __shared__ float red[SK_WARPS][16][NT * 8 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qd = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * 16;
  // rows past N are clamped for loading and masked when storing
  const int r0 = min(n0 + qd, N - 1), r1 = min(n0 + qd + 8, N - 1);
  const bf16* w0 = W + (size_t)r0 * ldw + t4 * 8;
  const bf16* w1 = W + (size_t)r1 * ldw + t4 * 8;
  const bf16* xr[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + qd;
    xok[nt] = m < M;
    xr[nt] = x + (size_t)min(m, M - 1) * ldx + t4 * 8;
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  // this warp's ring: [stage][block in group][row half][lane] x 16 bytes
  uint4* ring = reinterpret_cast<uint4*>(sk_smem) + (size_t)warp * (SK_STAGES * SK_GROUP * 2 * 32) + lane;
  const int kblocks = (K + 31) >> 5;
  const int ngroups = (kblocks + SK_GROUP - 1) / SK_GROUP;
  const int n_mine = warp < ngroups ? (ngroups - warp + SK_WARPS - 1) / SK_WARPS : 0;   // groups warp, warp + 8, ...

  auto issue = [&](int i) {
    if (i < n_mine) {
      const int g = warp + SK_WARPS * i;
      uint4* st = ring + (size_t)(i % SK_STAGES) * (SK_GROUP * 2 * 32);
#pragma unroll
      for (int u = 0; u < SK_GROUP; ++u) {
        const int jb = g * SK_GROUP + u;
        const bool ok = jb < kblocks && (jb * 32 + t4 * 8) < K;   // K % 8 == 0: a lane's 8 k are all in or all out
        if (ok) {
          cp_async16(st + (u * 2 + 0) * 32, w0 + (size_t)jb * 32);
          cp_async16(st + (u * 2 + 1) * 32, w1 + (size_t)jb * 32);
        } else {
          st[(u * 2 + 0) * 32] = make_uint4(0u, 0u, 0u, 0u);
          st[(u * 2 + 1) * 32] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int i = 0; i < SK_STAGES - 1; ++i) issue(i);
  for (int i = 0; i < n_mine; ++i) {
    issue(i + SK_STAGES - 1);
    cp_async_wait<SK_STAGES - 1>();
    const int g = warp + SK_WARPS * i;
    const uint4* st = ring + (size_t)(i % SK_STAGES) * (SK_GROUP * 2 * 32);
#pragma unroll
    for (int u = 0; u < SK_GROUP; ++u) {
      const int jb = g * SK_GROUP + u;
      const bool ok = jb < kblocks && (jb * 32 + t4 * 8) < K;
      const uint4 a0 = st[(u * 2 + 0) * 32], a1 = st[(u * 2 + 1) * 32];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 bx = (ok && xok[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + (size_t)jb * 32))
                                         : make_uint4(0u, 0u, 0u, 0u);
        // k-step 0 uses the first 8 bytes of each 16-byte load, k-step 1 the second 8
        mma_bf16(acc[nt], a0.x, a1.x, a0.y, a1.y, bx.x, bx.y);
        mma_bf16(acc[nt], a0.z, a1.z, a0.w, a1.w, bx.z, bx.w);
      }
    }
  }
  // acc[nt][e]: W row (qd + 8 * (e >> 1)), token nt * 8 + 2 * t4 + (e & 1)
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[warp][qd + 8 * (e >> 1)][nt * 8 + 2 * t4 + (e & 1)] = acc[nt][e];
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += SK_THREADS) {
    const int m = idx >> 4, r = idx & 15;   // consecutive threads write consecutive columns of out
    if (m < M && n0 + r < N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) s += red[w][r][m];
      out[(size_t)m * ldo + n0 + r] = mi_from_float<OutT>(s);
    }
  }
}

extern "C" int mi_gemm_skinny_max_rows() { return 16; }

// out_dtype: MI_DTYPE_BF16 or MI_DTYPE_F32.
extern "C" int mi_gemm_skinny(const void* x, const void* W, void* out, int M, int N, int K, int ldx, int ldw,
                              int ldo, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16) MI_REFUSE("gemm_skinny: at most 16 rows, got %d", M);
  if (K <= 0 || K % 8 != 0) MI_REFUSE("gemm_skinny: K must be a positive multiple of 8, got %d", K);
  if (ldx % 8 != 0 || ldw % 8 != 0 || !mi_aligned(x, 16) || !mi_aligned(W, 16))
    MI_REFUSE("gemm_skinny: operand rows must be 16-byte aligned");
  if (ldx < K || ldw < K || ldo < N) MI_REFUSE("gemm_skinny: leading dimensions too small");
  const int grid = (N + 15) / 16;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  const size_t smem = (size_t)SK_WARPS * SK_STAGES * SK_GROUP * 2 * 32 * 16;
#define MI_SKINNY(NT, T)                                                                                  \
  do {                                                                                                    \
    auto kern = gemm_skinny_kernel<NT, T>;                                                                \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    if (e != cudaSuccess) return (int)e;                                                                  \
    kern<<<grid, SK_THREADS, smem, stream>>>(xp, wp, (T*)out, M, N, K, ldx, ldw, ldo);                    \
  } while (0)
  if (out_dtype == MI_DTYPE_BF16) {
    if (M <= 8) MI_SKINNY(1, bf16);
    else MI_SKINNY(2, bf16);
  } else if (out_dtype == MI_DTYPE_F32) {
    if (M <= 8) MI_SKINNY(1, float);
    else MI_SKINNY(2, float);
  } else {
    MI_REFUSE("gemm_skinny: unknown output dtype %d", out_dtype);
  }
#undef MI_SKINNY
  MI_RETURN_LAUNCH_STATUS();
}
