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
//     x is read with the same pattern; one x fragment serves RT row tiles.
//   * A block owns RT * 16 rows of W and one slice of K.  Its 4 warps take the 32-wide k
//     blocks of the slice round-robin, each streaming through a private ring of cp.async
//     stages in shared memory (a lane reads back only what it copied, so there is no
//     block-wide barrier in the loop and 12 KB per warp are always in flight).
//   * Few rows of W (N small) would give too few blocks to fill the GPU; then K is cut into
//     slices across blocks.  Every block writes its partial sums to scratch memory and bumps
//     a counter of its row tile; the block that arrives last adds the slices in slice order
//     (so the result does not depend on arrival order), writes the output and resets the
//     counter.  Nobody waits for anybody.
//
// K must be a multiple of 8 and rows 16-byte aligned; other shapes are refused.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define SK_WARPS 4
#define SK_THREADS (SK_WARPS * 32)
#define SK_STAGES 4
#define SK_UNITS 8   // 512-byte units (one 16-byte load per lane) per stage

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

// RT: row tiles (of 16 rows of W) per block, 1, 2 or 4.  NT: 8-token tiles, 1 or 2.
template <int RT, int NT, typename OutT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, OutT* __restrict__ out,
                   float* __restrict__ partial, int* __restrict__ counters, int M, int N, int K, int ldx,
                   int ldw, int ldo, int ksplit, int blocks_per_split) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  constexpr int G = SK_UNITS / (2 * RT);   // k blocks per stage
  constexpr int ROWS = RT * 16;
  constexpr int MT = NT * 8;
  extern __shared__ __align__(16) unsigned char sk_smem[];
  __shared__ int is_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qd = lane >> 2, t4 = lane & 3;
  const int n0 = blockIdx.x * ROWS;
  const int split = blockIdx.y;
  const int kblocks = (K + 31) >> 5;
  const int kb0 = split * blocks_per_split, kb1 = min(kblocks, kb0 + blocks_per_split);

  // rows past N are clamped for loading and masked when storing
  const bf16* wrow[RT][2];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) {
    wrow[rt][0] = W + (size_t)min(n0 + rt * 16 + qd, N - 1) * ldw + t4 * 8;
    wrow[rt][1] = W + (size_t)min(n0 + rt * 16 + qd + 8, N - 1) * ldw + t4 * 8;
  }
  const bf16* xr[NT];
  bool xok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + qd;
    xok[nt] = m < M;
    xr[nt] = x + (size_t)min(m, M - 1) * ldx + t4 * 8;
  }
  float acc[RT][NT][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[rt][nt][0] = acc[rt][nt][1] = acc[rt][nt][2] = acc[rt][nt][3] = 0.f;

  // this warp's ring: [stage][unit][lane] x 16 bytes; unit = (block in group, row tile, row half)
  uint4* ring = reinterpret_cast<uint4*>(sk_smem) + (size_t)warp * (SK_STAGES * SK_UNITS * 32) + lane;
  const int ngroups = (max(kb1 - kb0, 0) + G - 1) / G;
  const int n_mine = warp < ngroups ? (ngroups - warp + SK_WARPS - 1) / SK_WARPS : 0;   // groups warp, warp + 4, ...

  auto issue = [&](int i) {
    if (i < n_mine) {
      const int g = warp + SK_WARPS * i;
      uint4* st = ring + (size_t)(i % SK_STAGES) * (SK_UNITS * 32);
#pragma unroll
      for (int u = 0; u < G; ++u) {
        const int jb = kb0 + g * G + u;
        const bool ok = jb < kb1 && (jb * 32 + t4 * 8) < K;   // K % 8 == 0: a lane's 8 k are all in or all out
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint4* slot = st + ((u * RT + rt) * 2 + h) * 32;
            if (ok) cp_async16(slot, wrow[rt][h] + (size_t)jb * 32);
            else *slot = make_uint4(0u, 0u, 0u, 0u);
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
    const uint4* st = ring + (size_t)(i % SK_STAGES) * (SK_UNITS * 32);
#pragma unroll
    for (int u = 0; u < G; ++u) {
      const int jb = kb0 + g * G + u;
      const bool ok = jb < kb1 && (jb * 32 + t4 * 8) < K;
      uint4 bx[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        bx[nt] = (ok && xok[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + (size_t)jb * 32))
                                 : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        const uint4 a0 = st[((u * RT + rt) * 2 + 0) * 32], a1 = st[((u * RT + rt) * 2 + 1) * 32];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // k-step 0 uses the first 8 bytes of each 16-byte load, k-step 1 the second 8
          mma_bf16(acc[rt][nt], a0.x, a1.x, a0.y, a1.y, bx[nt].x, bx[nt].y);
          mma_bf16(acc[rt][nt], a0.z, a1.z, a0.w, a1.w, bx[nt].z, bx[nt].w);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();   // every warp is done with its ring: reuse the memory for the reduction

  // red[warp][row][token]; acc[rt][nt][e] is W row rt*16 + qd + 8*(e>>1), token nt*8 + 2*t4 + (e&1)
  float* red = reinterpret_cast<float*>(sk_smem);
  constexpr int RS = MT + 1;
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e)
        red[((size_t)warp * ROWS + rt * 16 + qd + 8 * (e >> 1)) * RS + nt * 8 + 2 * t4 + (e & 1)] = acc[rt][nt][e];
  __syncthreads();

  if (ksplit == 1) {
    for (int idx = threadIdx.x; idx < ROWS * MT; idx += SK_THREADS) {
      const int m = idx / ROWS, r = idx - m * ROWS;   // consecutive threads write consecutive columns of out
      if (m < M && n0 + r < N) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) s += red[((size_t)w * ROWS + r) * RS + m];
        out[(size_t)m * ldo + n0 + r] = mi_from_float<OutT>(s);
      }
    }
    return;
  }

  // K is cut across blocks: park this slice's sums, the last block to arrive adds them up
  for (int idx = threadIdx.x; idx < ROWS * MT; idx += SK_THREADS) {
    const int m = idx / ROWS, r = idx - m * ROWS;
    if (m < M && n0 + r < N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) s += red[((size_t)w * ROWS + r) * RS + m];
      partial[((size_t)split * M + m) * N + n0 + r] = s;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[blockIdx.x], 1) == ksplit - 1) ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < ROWS * MT; idx += SK_THREADS) {
    const int m = idx / ROWS, r = idx - m * ROWS;
    if (m < M && n0 + r < N) {
      float s = 0.f;
      for (int sp = 0; sp < ksplit; ++sp) s += __ldcg(partial + ((size_t)sp * M + m) * N + n0 + r);
      out[(size_t)m * ldo + n0 + r] = mi_from_float<OutT>(s);
    }
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0;   // ready for the next product
}

extern "C" int mi_gemm_skinny_max_rows() { return 16; }

// How the product would be cut: writes rows per block and the number of K slices.
// Scratch needed when slices > 1: slices * M * N floats, and ceil(N / rows) zeroed ints.
extern "C" int mi_gemm_skinny_plan(int M, int N, int K, int sm_count, int* rows_per_block, int* k_slices) {
  const int rows = 64;
  const int row_blocks = (N + rows - 1) / rows;
  const int kblocks = (K + 31) / 32;
  int slices = 1;
  const int target = 2 * sm_count;
  if (row_blocks < target) {
    int want = (target + row_blocks - 1) / row_blocks;
    int most = kblocks / 32;   // a slice keeps at least 32 k blocks (8 per warp)
    if (most < 1) most = 1;
    slices = want < most ? want : most;
  }
  if (slices > 32) slices = 32;
  *rows_per_block = rows;
  *k_slices = slices;
  return 0;
}

// out_dtype: MI_DTYPE_BF16 or MI_DTYPE_F32.  k_slices as planned by mi_gemm_skinny_plan; with
// k_slices > 1, `partial` holds k_slices * M * N floats and `counters` ceil(N / 64) ints that
// are zero on entry (the kernel leaves them zero).
extern "C" int mi_gemm_skinny(const void* x, const void* W, void* out, int M, int N, int K, int ldx, int ldw,
                              int ldo, int out_dtype, int k_slices, float* partial, int* counters,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16) MI_REFUSE("gemm_skinny: at most 16 rows, got %d", M);
  if (K <= 0 || K % 8 != 0) MI_REFUSE("gemm_skinny: K must be a positive multiple of 8, got %d", K);
  if (ldx % 8 != 0 || ldw % 8 != 0 || !mi_aligned(x, 16) || !mi_aligned(W, 16))
    MI_REFUSE("gemm_skinny: operand rows must be 16-byte aligned");
  if (ldx < K || ldw < K || ldo < N) MI_REFUSE("gemm_skinny: leading dimensions too small");
  if (k_slices < 1 || k_slices > 65535) MI_REFUSE("gemm_skinny: bad number of K slices %d", k_slices);
  if (k_slices > 1 && (!partial || !counters)) MI_REFUSE("gemm_skinny: K slices need scratch memory");
  const int kblocks = (K + 31) / 32;
  const int per_split = (kblocks + k_slices - 1) / k_slices;
  dim3 grid((N + 63) / 64, k_slices);
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  const size_t smem = (size_t)SK_WARPS * SK_STAGES * SK_UNITS * 32 * 16;   // 64 KB; also holds the reduction
#define MI_SKINNY(NT, T)                                                                                  \
  do {                                                                                                    \
    auto kern = gemm_skinny_kernel<4, NT, T>;                                                             \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    if (e != cudaSuccess) return (int)e;                                                                  \
    MI_LAUNCH((kern), grid, SK_THREADS, smem, stream, xp, wp, (T*)out, partial, counters, M, N, K, ldx, ldw, ldo,  \
                                             k_slices, per_split);                                        \
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
