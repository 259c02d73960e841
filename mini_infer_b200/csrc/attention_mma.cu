// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16, fp32
// accumulation, fp32 online softmax), keys and values staged in shared memory with
// cp.async (two buffers) and read with ldmatrix.
//
// Two kernels share the machinery:
//
//   decode   every request brings one query token.  A block takes one request, one group
//            of up to 8 query heads that share a key/value head, and one slice of the
//            keys ("split"); its 4 warps take 16 keys each of every 64-key chunk, keep an
//            online softmax of their own and are merged at the end.  With more than one
//            split the block writes an unnormalised partial result (fp32) and its
//            (max, sum) to scratch memory and counts its arrival; the block that arrives
//            last merges the splits.
//   prefill  query portions of any length.  A block takes a tile of tokens of one request
//            and up to 128 rows (token, head-in-group) that share a key/value head; each
//            warp owns 16 rows and walks all keys up to the causal limit.
//
// A query at absolute position p sees keys j with max(0, p - window + 1) <= j <= p.
// Layouts are those of attention_generic.cu (cache pages are [nkv, page_size, d], so the keys of a
// page lie together per key/value head and a 64-key chunk is read as a few long runs).
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define KCHUNK 64
#define NTHREADS 128
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
// the same with a shared-memory address already in hand (32-bit arithmetic in the caller)
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t s) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- bulk asynchronous copies (the copy engine writes shared memory and signals an mbarrier)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// The same copy for data that is read once per step (a decode step reads every key and value of a
// request exactly once, and all layers' caches together are far larger than the L2): marked to be
// evicted first, so that what the step's kernels hand to one another stays in the L2 meanwhile.
// MINI_INFER_L2_HINTS=0 in the environment switches the mark off (for comparisons).
static __device__ int g_stream_once_hint = 1;
__device__ __forceinline__ void bulk_copy_g2s_once(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  if (!g_stream_once_hint) return bulk_copy_g2s(dst, src, bytes, bar);
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;\n" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Wait for a phase of the barrier, but never for ever: after MBAR_SPIN_LIMIT tries the wait
// gives up and records it in *status; the block then leaves its loop, and blocks that start
// later return at once (the output is then wrong and the host finds the status word set;
// nothing hangs).
#define MBAR_SPIN_LIMIT (1 << 16)
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
  for (int it = 0; it < MBAR_SPIN_LIMIT; ++it)
    if (mbar_try_wait(bar, parity)) return true;
  if (status) atomicExch(status, 1);
  return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// two bf16 pairs (x1 in `lo`, their partners x2 in `hi`) rotated by the angles whose sines and cosines follow sn, cn
__device__ __forceinline__ void rotate_words(uint32_t& lo, uint32_t& hi, const float* __restrict__ sn,
                                             const float* __restrict__ cn) {
  const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo));
  const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi));
  float a0, a1, b0, b1;
  mi_rotate(x1.x, x2.x, sn[0], cn[0], a0, b0);
  mi_rotate(x1.y, x2.y, sn[1], cn[1], a1, b1);
  lo = pack_bf16(a0, a1);
  hi = pack_bf16(b0, b1);
}
// the same for every state space: plain stores to global memory that a bulk copy reads next
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;\n" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }

__device__ __forceinline__ int inpage_of(int j, int page_size, int page_shift) {
  return page_shift >= 0 ? (j & (page_size - 1)) : (j % page_size);
}

// Brings 64-key chunks of one request's keys and values into shared memory, [64][d] bf16 each,
// rows unpadded.  The cache stores every row with its 16-byte chunks permuted by the in-page
// offset (common.cuh), so a linear copy lands in a layout that ldmatrix reads without bank
// conflicts; the readers below apply the same permutation.
//
// With a power-of-two page size the keys of a page are one contiguous run per head, and a chunk
// is 64 / min(page, 64) pieces: one thread per piece and tensor issues ONE bulk copy (4 KB for
// 16-key pages of 128-wide heads) that reports to the chunk's mbarrier.  Other page sizes copy
// row by row.  The page id a thread needs is fetched one chunk ahead.  Pieces (rows) that lie
// wholly outside [lo, hi) are not copied; what they leave in shared memory is masked by the
// caller (scores) or zeroed (values, zero_masked_values).
struct PageLoader {
  int pg;
  int t = threadIdx.x;   // which copy this thread issues; a producer warp sets its lane

  static __device__ __forceinline__ int piece_rows(int page_size, int page_shift) {
    return page_shift >= 0 ? min(page_size, KCHUNK) : 1;
  }

  __device__ __forceinline__ void fetch(const int* __restrict__ table, int page_size, int page_shift, int chunk,
                                        int lo, int hi) {
    pg = -1;
    const int rows = piece_rows(page_size, page_shift), n = KCHUNK / rows;
    if (t < 2 * n) {
      const int j0 = chunk * KCHUNK + (t % n) * rows;
      if (j0 < hi && j0 + rows > lo) pg = table[page_shift >= 0 ? (j0 >> page_shift) : (j0 / page_size)];
    }
  }

  // bytes the chunk's copies will deliver (the same for every thread)
  static __device__ __forceinline__ uint32_t chunk_bytes(int chunk, int lo, int hi, int d, int page_size,
                                                         int page_shift) {
    const int rows = piece_rows(page_size, page_shift), n = KCHUNK / rows, cb = chunk * KCHUNK;
    const int first = lo > cb ? (lo - cb) / rows : 0;
    const int last = min(n - 1, (hi - 1 - cb) / rows);
    const int cnt = (hi > cb && last >= first) ? last - first + 1 : 0;
    return (uint32_t)cnt * (uint32_t)rows * (uint32_t)d * 4u;   // keys and values, 2 bytes each
  }

  // kOnce: nobody else reads these keys and values in this step (decode), see bulk_copy_g2s_once
  template <bool kOnce = false>
  __device__ __forceinline__ void issue(bf16* kdst, bf16* vdst, const bf16* __restrict__ kcache,
                                        const bf16* __restrict__ vcache, int page_size, int page_shift, int chunk,
                                        int nkv, int kvh, int d, uint64_t* bar) const {
    const int rows = piece_rows(page_size, page_shift), n = KCHUNK / rows;
    if (t >= 2 * n || pg < 0) return;
    const int piece = t % n;
    const bool is_v = t >= n;
    const int j0 = chunk * KCHUNK + piece * rows;
    const size_t off = (((size_t)pg * nkv + kvh) * page_size + inpage_of(j0, page_size, page_shift)) * d;
    if (kOnce)
      bulk_copy_g2s_once((is_v ? vdst : kdst) + (size_t)piece * rows * d, (is_v ? vcache : kcache) + off,
                         (uint32_t)rows * (uint32_t)d * 2u, bar);
    else
      bulk_copy_g2s((is_v ? vdst : kdst) + (size_t)piece * rows * d, (is_v ? vcache : kcache) + off,
                    (uint32_t)rows * (uint32_t)d * 2u, bar);
  }
};

// Rows of the value tile whose keys are outside [lo, hi) may hold anything (never-written cache
// slots, or shared memory nobody wrote); their probabilities are exactly 0, but 0 * NaN is NaN,
// so they are cleared.  Only a request's first and last chunks have such rows.  Every thread of
// the block must call this (it ends with a barrier when the chunk has masked rows).
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// barrier among the first `count` threads of the block (count a multiple of 32), id 1
__device__ __forceinline__ void consumer_barrier(int count) {
  asm volatile("bar.sync 1, %0;\n" ::"r"(count) : "memory");
}

template <int THREADS, bool NAMED = false>
__device__ __forceinline__ void zero_masked_values(bf16* vtile, int chunk, int lo, int hi, int d) {
  const int cb = chunk * KCHUNK;
  if (cb >= lo && cb + KCHUNK <= hi) return;   // uniform over the calling threads
  const int units = d >> 3;
  for (int idx = threadIdx.x; idx < KCHUNK * units; idx += THREADS) {
    const int r = idx / units, u = idx - r * units;
    const int j = cb + r;
    if (j < lo || j >= hi) *reinterpret_cast<uint4*>(vtile + r * d + u * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
  fence_proxy_async();   // these writes come before the copy engine's next writes to the tile
  if (NAMED) consumer_barrier(THREADS);
  else __syncthreads();
}

// ------------------------------------------------------------------------------- decode
//
// Keys sit on the M side of the first product: S[16 keys x 8 heads] = K[16 x d] * Q^T[d x 8],
// so every MMA row is a real key whatever the group size (query heads would fill only a few
// of 16 rows).  Q fragments stay in registers for the whole kernel.  The second product is
// O^T[d x 8 heads] += V^T[d x 16 keys] * P[16 keys x 8 heads]; V^T comes from ldmatrix.trans,
// and P is moved from the accumulator layout (lane holds keys q, q+8 of heads 2t, 2t+1) to the
// B-operand layout (lane holds keys 2t, 2t+1, 2t+8, 2t+9 of head q) with four shuffles.

#define DEC_HEADS 8   // query heads of one key/value head handled by a block
#define DEC_STAGES 3  // 64-key chunks in the shared-memory ring (two are in flight while one is used)
#define DEC_THREADS (NTHREADS + 32)   // four consumer warps and one producer warp

// After a block has parked its slice's partial result: count arrivals for this (request,
// head group); the block that arrives last merges all slices in slice order,
//   out = sum_s f_s O_s / sum_s f_s l_s,  f_s = 2^(m_s - m),
// writes the output and resets the counter.  Nobody waits for anybody.
template <int DMAX>
__device__ __forceinline__ void decode_merge_when_last(const float* __restrict__ part_o,
                                                       const float* __restrict__ part_ml, int* counters,
                                                       int counter_index, bf16* __restrict__ out,
                                                       int out_stride, int tok, int b, int nq, int d,
                                                       int n_splits, int head0, int heads_here) {
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[counter_index], 1) == n_splits - 1) ? 1 : 0;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int r = threadIdx.x >> 4, cgrp = threadIdx.x & 15;   // 8 heads x 16 threads
  if (n_splits <= 8) {
    // Few slices: every load this thread needs ((max, sum) of its head's slices and its eight
    // output columns of every slice) is issued before the first one is used, so the merge
    // costs one round trip to L2 instead of one per step.
    if (r < heads_here) {
      const int head = head0 + r;
      const float2* ml = reinterpret_cast<const float2*>(part_ml) + (size_t)(b * nq + head) * n_splits;
      const float* po = part_o + (size_t)(b * nq + head) * n_splits * d;
      float2 mls[8];
      float v[8][DMAX / 16];
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        mls[sp] = sp < n_splits ? __ldcg(ml + sp) : make_float2(-INFINITY, 0.f);
#pragma unroll
        for (int i = 0; i < DMAX / 16; ++i)
          v[sp][i] = (sp < n_splits && cgrp + 16 * i < d) ? __ldcg(po + (size_t)sp * d + cgrp + 16 * i) : 0.f;
      }
      float m = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) m = fmaxf(m, mls[sp].x);
      float L = 0.f, acc[DMAX / 16];
#pragma unroll
      for (int i = 0; i < DMAX / 16; ++i) acc[i] = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; ++sp) {
        const float f = (mls[sp].x == -INFINITY) ? 0.f : exp2f(mls[sp].x - m);
        L += mls[sp].y * f;
#pragma unroll
        for (int i = 0; i < DMAX / 16; ++i) acc[i] += f != 0.f ? f * v[sp][i] : 0.f;   // unused slices hold garbage
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* orow = out + (size_t)tok * out_stride + (size_t)head * d;
#pragma unroll
      for (int i = 0; i < DMAX / 16; ++i)
        if (cgrp + 16 * i < d) orow[cgrp + 16 * i] = __float2bfloat16_rn(acc[i] * inv);
    }
  } else {
    // (max, sum) of every (head, slice) first, all loads in flight at once
    __shared__ float sm_m[DEC_HEADS][64], sm_f[DEC_HEADS][64], sm_inv[DEC_HEADS];
    for (int idx = threadIdx.x; idx < heads_here * n_splits; idx += blockDim.x) {
      const int rr = idx / n_splits, sp = idx - rr * n_splits;
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + (size_t)(b * nq + head0 + rr) * n_splits + sp);
      sm_m[rr][sp] = ml.x;
      sm_f[rr][sp] = ml.y;
    }
    __syncthreads();
    if (threadIdx.x < heads_here) {
      const int rr = threadIdx.x;
      float m = -INFINITY;
      for (int sp = 0; sp < n_splits; ++sp) m = fmaxf(m, sm_m[rr][sp]);
      float L = 0.f;
      for (int sp = 0; sp < n_splits; ++sp) {
        const float f = (sm_m[rr][sp] == -INFINITY) ? 0.f : exp2f(sm_m[rr][sp] - m);
        L += sm_f[rr][sp] * f;
        sm_f[rr][sp] = f;
      }
      sm_inv[rr] = L > 0.f ? 1.f / L : 0.f;
    }
    __syncthreads();
    if (r < heads_here) {
      const int head = head0 + r;
      const float* po = part_o + (size_t)(b * nq + head) * n_splits * d;
      bf16* orow = out + (size_t)tok * out_stride + (size_t)head * d;
      float acc[DMAX / 16];
#pragma unroll
      for (int i = 0; i < DMAX / 16; ++i) acc[i] = 0.f;
      for (int sp = 0; sp < n_splits; ++sp) {   // the columns of a slice are loaded together
        const float f = sm_f[r][sp];
        float v[DMAX / 16];
#pragma unroll
        for (int i = 0; i < DMAX / 16; ++i)
          v[i] = (cgrp + 16 * i < d) ? __ldcg(po + (size_t)sp * d + cgrp + 16 * i) : 0.f;
#pragma unroll
        for (int i = 0; i < DMAX / 16; ++i) acc[i] += f != 0.f ? f * v[i] : 0.f;   // unused slices hold garbage
      }
#pragma unroll
      for (int i = 0; i < DMAX / 16; ++i)
        if (cgrp + 16 * i < d) orow[cgrp + 16 * i] = __float2bfloat16_rn(acc[i] * sm_inv[r]);
    }
  }
  if (threadIdx.x == 0) counters[counter_index] = 0;   // ready for the next call
}

template <int DMAX>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ block_table, int bt_stride, const int* __restrict__ table_rows,
                        int page_size, int page_shift,
                        const int* __restrict__ q_start, const int* __restrict__ kv_len, int nq, int nkv,
                        int d, float scale, int window, int n_splits, const int* __restrict__ slice_chunks,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                        int* __restrict__ status) {
  // The next kernel's blocks may be scheduled.  This kernel reads the batch description and
  // the keys and values of earlier positions before it waits for the kernels ahead of it: the
  // description was uploaded before the step's first kernel, and the step's own kernels write
  // only the newest position of each request (kv_len - 1) and the queries.
  mi_pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);          // [DEC_STAGES][64][d]
  bf16* Vs = Ks + DEC_STAGES * KCHUNK * d;               // [DEC_STAGES][64][d]
  const int swz_mask = mi_swizzle_mask(d, 2);
  float* merge_o = reinterpret_cast<float*>(smem_raw);   // [4][8][d] after the main loop
  __shared__ float merge_m[4][DEC_HEADS], merge_l[4][DEC_HEADS];
  __shared__ __align__(8) uint64_t bars[DEC_STAGES];    // "full": a chunk has landed in its stage
  __shared__ __align__(8) uint64_t empty[DEC_STAGES];   // "empty": all four consumer warps are done with it

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = lane >> 2, t4 = lane & 3;
  const int g = nq / nkv;
  const int hblocks = (g + DEC_HEADS - 1) / DEC_HEADS;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y / hblocks, hb = blockIdx.y - kvh * hblocks;
  const int b = blockIdx.z;
  const int kl = kv_len[b];
  const int tok = q_start[b];
  const int lo = window > 0 ? max(0, kl - window) : 0;  // the query sits at position kl - 1
  const int c_first = lo / KCHUNK, c_end = (kl + KCHUNK - 1) / KCHUNK;
  // A slice is the same number of chunks for every request when the caller planned one (a
  // short request then fills fewer slices and a long one is cut into all of them); never
  // fewer than this request needs to be covered by n_splits slices.
  int per_split = (c_end - c_first + n_splits - 1) / n_splits;
  if (slice_chunks) per_split = max(per_split, __ldg(slice_chunks));
  const int c0 = c_first + split * per_split;
  const int c1 = min(c_end, c0 + per_split);
  const int heads_here = min(DEC_HEADS, g - hb * DEC_HEADS);
  const int head0 = kvh * g + hb * DEC_HEADS;
  const int* table = block_table + (size_t)(table_rows ? table_rows[b] : b) * bt_stride;

  if (status && *reinterpret_cast<volatile int*>(status)) return;   // an earlier block gave up waiting
  if (c0 >= c1) {  // nothing for this slice: the request is shorter than the slices before it, or empty
    mi_pdl_wait();
    if (n_splits == 1) {   // a request that holds no key at all: its output rows are zero, no scratch exists
      bf16* orow = out + (size_t)tok * out_stride + (size_t)head0 * d;
      for (int k = tid; k < heads_here * d; k += DEC_THREADS) orow[k] = __float2bfloat16_rn(0.f);
      return;
    }
    for (int r = tid; r < heads_here; r += DEC_THREADS) {
      float* ml = part_ml + ((size_t)(b * nq + head0 + r) * n_splits + split) * 2;
      ml[0] = -INFINITY;
      ml[1] = 0.f;
    }
    decode_merge_when_last<DMAX>(part_o, part_ml, counters, b * gridDim.y + blockIdx.y, out, out_stride, tok, b, nq, d,
                           n_splits, head0, heads_here);
    return;
  }

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < DEC_STAGES; ++i) {
      mbar_init(&bars[i], 1);
      mbar_init(&empty[i], 4);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == 4) {
    // The producer warp: keeps the ring full.  Issuing a copy costs a warp hundreds of cycles;
    // here that is nobody's critical path.
    PageLoader loader;
    loader.t = lane;
    const int pieces = 2 * (KCHUNK / PageLoader::piece_rows(page_size, page_shift));   // copies per chunk
    bool ok = true;
    for (int c = c0; c < c1 && ok; ++c) {
      const int it = c - c0, st = it % DEC_STAGES;
      if (it >= DEC_STAGES)
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[st], ((it / DEC_STAGES) - 1) & 1, status));
      if (!ok) break;
      if ((c + 1) * KCHUNK >= kl) mi_pdl_wait();   // the chunk with the newest position: written by this step
      if (lane == 0) mbar_expect_tx(&bars[st], PageLoader::chunk_bytes(c, lo, kl, d, page_size, page_shift));
      __syncwarp();
      for (int t0 = 0; t0 < pieces; t0 += 32) {   // more than 32 copies only with odd page sizes
        loader.t = t0 + lane;
        loader.fetch(table, page_size, page_shift, c, lo, kl);
        loader.issue<true>(Ks + st * KCHUNK * d, Vs + st * KCHUNK * d, kcache, vcache, page_size, page_shift, c, nkv, kvh,
                     d, &bars[st]);
      }
    }
  }
  if (warp < 4) mi_pdl_wait();   // the queries come from the kernel before this one
  // Q as the B operand: lane (qd, t4) holds head qd, dims ks*16 + 2*t4 + {0,1} and + 8
  const int ksteps = d >> 4;
  uint32_t qb[DMAX / 16][2];
  {
    const bf16* qrow = q + (size_t)tok * q_stride + (size_t)(head0 + qd) * d;
#pragma unroll
    for (int ks = 0; ks < DMAX / 16; ++ks) {
      qb[ks][0] = qb[ks][1] = 0u;
      if (ks < ksteps && qd < heads_here) {
        qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
        qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
      }
    }
  }

  // this lane's heads are 2*t4 and 2*t4 + 1
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[DMAX / 16][4];   // O^T: dims dt*16 + qd (+8), heads 2*t4 (+1)
#pragma unroll
  for (int i = 0; i < DMAX / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float sc = scale * LOG2E;
  // lanes that hold what this lane needs of P: keys 2*t4 and 2*t4 + 1, heads qd (pair qd / 2)
  const int src0 = (2 * t4) * 4 + (qd >> 1), src1 = (2 * t4 + 1) * 4 + (qd >> 1);
  const bool odd_head = qd & 1;

  for (int c = c0; c < c1 && warp < 4; ++c) {
    const int it = c - c0, buf = it % DEC_STAGES;
    const bool arrived =
        __all_sync(0xffffffffu, mbar_wait_bounded(&bars[buf], (it / DEC_STAGES) & 1, status));
    zero_masked_values<NTHREADS, true>(Vs + buf * KCHUNK * d, c, lo, kl, d);
    const int key0 = c * KCHUNK + warp * 16;
    // this lane's ldmatrix rows (keys) in the warp's 16-key slice, with their chunk permutation
    const int kr = lane & 15, vr = (lane & 7) + (lane >> 4) * 8;
    const int ksw = inpage_of(key0 + kr, page_size, page_shift) & swz_mask;
    const int vsw = inpage_of(key0 + vr, page_size, page_shift) & swz_mask;
    const bf16* Kb = Ks + buf * KCHUNK * d + (warp * 16 + kr) * d;
    const bf16* Vb = Vs + buf * KCHUNK * d + (warp * 16 + vr) * d;
    if (arrived && key0 < kl && key0 + 16 > lo) {  // warp-uniform: this warp's 16 keys hold something visible
      // All fragment loads of a group of k-steps are issued before the first MMA that needs
      // them, and two accumulators halve the MMA dependency chain: the warp's critical path is
      // one load latency plus a few MMAs instead of their sum over all k-steps.
      constexpr int GROUP = (DMAX / 16) < 8 ? (DMAX / 16) : 8;
      float s[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int g0 = 0; g0 < DMAX / 16; g0 += GROUP) {
        uint32_t kf[GROUP][4];
#pragma unroll
        for (int i = 0; i < GROUP; ++i)
          if (g0 + i < ksteps) ldmatrix_x4(kf[i], Kb + ((((g0 + i) * 2 + (lane >> 4)) ^ ksw) << 3));
#pragma unroll
        for (int i = 0; i < GROUP; ++i)
          if (g0 + i < ksteps) {
            if (i & 1) mma_bf16(s_odd, kf[i], qb[g0 + i][0], qb[g0 + i][1]);
            else mma_bf16(s, kf[i], qb[g0 + i][0], qb[g0 + i][1]);
          }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) s[e] += s_odd[e];
      // the value fragments of the first group do not depend on the softmax: fetch them now
      uint32_t vf[GROUP][4];
#pragma unroll
      for (int i = 0; i < GROUP; ++i)
        if (i < ksteps)
          ldmatrix_x4_trans(vf[i], Vb + (((i * 2 + ((lane >> 3) & 1)) ^ vsw) << 3));
      // s[0], s[1]: key qd, heads 2t, 2t+1;  s[2], s[3]: key qd + 8
      const int j0 = key0 + qd, j1 = j0 + 8;
      const bool ok0 = j0 < kl && j0 >= lo, ok1 = j1 < kl && j1 >= lo;
      s[0] = ok0 ? s[0] * sc : -INFINITY;
      s[1] = ok0 ? s[1] * sc : -INFINITY;
      s[2] = ok1 ? s[2] * sc : -INFINITY;
      s[3] = ok1 ? s[3] * sc : -INFINITY;
      float alpha[2], p[4];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float mx = fmaxf(s[hh], s[2 + hh]);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run[hh], mx);   // finite: the warp holds at least one visible key
        alpha[hh] = exp2f(m_run[hh] - m_new);
        p[hh] = exp2f(s[hh] - m_new);
        p[2 + hh] = exp2f(s[2 + hh] - m_new);
        m_run[hh] = m_new;
        l_run[hh] = l_run[hh] * alpha[hh] + (p[hh] + p[2 + hh]);
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < DMAX / 16; ++i) {
          o[i][0] *= alpha[0]; o[i][1] *= alpha[1];
          o[i][2] *= alpha[0]; o[i][3] *= alpha[1];
        }
      }
      // P to the B-operand layout
      const uint32_t p_lo = pack_bf16(p[0], p[1]);   // key qd: heads 2t (low half), 2t+1 (high half)
      const uint32_t p_hi = pack_bf16(p[2], p[3]);   // key qd + 8
      const uint32_t x0 = __shfl_sync(0xffffffffu, p_lo, src0), x1 = __shfl_sync(0xffffffffu, p_lo, src1);
      const uint32_t y0 = __shfl_sync(0xffffffffu, p_hi, src0), y1 = __shfl_sync(0xffffffffu, p_hi, src1);
      // b0 = (key 2t, key 2t+1) of head qd; b1 = (key 2t+8, key 2t+9)
      const uint32_t sel = odd_head ? 0x7632u : 0x5410u;
      const uint32_t pb0 = __byte_perm(x0, x1, sel), pb1 = __byte_perm(y0, y1, sel);
      // V^T fragments: a0 (dim q, keys 2t..), a1 (dim q+8, keys 2t..), a2 / a3 keys +8
#pragma unroll
      for (int i = 0; i < GROUP; ++i)
        if (i < ksteps) mma_bf16(o[i], vf[i], pb0, pb1);
#pragma unroll
      for (int g0 = GROUP; g0 < DMAX / 16; g0 += GROUP) {
#pragma unroll
        for (int i = 0; i < GROUP; ++i)
          if (g0 + i < ksteps)
            ldmatrix_x4_trans(vf[i], Vb + ((((g0 + i) * 2 + ((lane >> 3) & 1)) ^ vsw) << 3));
#pragma unroll
        for (int i = 0; i < GROUP; ++i)
          if (g0 + i < ksteps) mma_bf16(o[g0 + i], vf[i], pb0, pb1);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[buf]);   // this warp is done with the stage
    if (!arrived) break;                       // a wait gave up: stop (status is set)
  }
  __syncthreads();   // every warp has left its loop: the ring can be reused

  // merge the four consumer warps
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    float l = l_run[hh];
    l += __shfl_xor_sync(0xffffffffu, l, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 8);
    l += __shfl_xor_sync(0xffffffffu, l, 16);
    if (qd == 0 && warp < 4) {
      merge_m[warp][2 * t4 + hh] = m_run[hh];
      merge_l[warp][2 * t4 + hh] = l;
    }
  }
#pragma unroll
  for (int i = 0; i < DMAX / 16; ++i) {
    if (i < ksteps && warp < 4) {
#pragma unroll
      for (int e = 0; e < 4; ++e)   // o[i][e]: dim i*16 + qd + 8*(e>>1), head 2*t4 + (e&1)
        merge_o[((size_t)warp * DEC_HEADS + 2 * t4 + (e & 1)) * d + i * 16 + qd + 8 * (e >> 1)] = o[i][e];
    }
  }
  __syncthreads();
  const int r = tid >> 4, cgrp = tid & 15;   // 8 heads x 16 threads (the producer warp's r is out of range)
  if (r < heads_here) {
    float m = merge_m[0][r];
#pragma unroll
    for (int w = 1; w < 4; ++w) m = fmaxf(m, merge_m[w][r]);
    float f[4], L = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      f[w] = (merge_m[w][r] == -INFINITY) ? 0.f : exp2f(merge_m[w][r] - m);
      L += merge_l[w][r] * f[w];
    }
    const int head = head0 + r;
    if (n_splits == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* orow = out + (size_t)tok * out_stride + (size_t)head * d;
      for (int k = cgrp; k < d; k += 16) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += f[w] * merge_o[((size_t)w * DEC_HEADS + r) * d + k];
        orow[k] = __float2bfloat16_rn(acc * inv);
      }
    } else {
      const size_t slot = (size_t)(b * nq + head) * n_splits + split;
      float* po = part_o + slot * d;
      for (int k = cgrp; k < d; k += 16) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += f[w] * merge_o[((size_t)w * DEC_HEADS + r) * d + k];
        po[k] = acc;
      }
      if (cgrp == 0) {
        part_ml[slot * 2] = m;
        part_ml[slot * 2 + 1] = L;
      }
    }
  }
  if (n_splits > 1)
    decode_merge_when_last<DMAX>(part_o, part_ml, counters, b * gridDim.y + blockIdx.y, out, out_stride, tok, b, nq, d,
                           n_splits, head0, heads_here);
}

// ------------------------------------------------------------------------------- decode, balanced
//
// The same arithmetic with the work cut evenly.  attention_decode_kernel gives every (request,
// head group) the same number of key slices; when requests differ in length, or when the
// number of blocks that comes out does not fill the GPU's block slots evenly, some SMs stream
// a multiple of what others do.  Here the 64-key chunks of all (request, head group) units are
// numbered in one row, unit after unit, and each of G persistent blocks takes an equal
// contiguous stretch of that row, whatever the lengths are: one long request among short ones
// is spread over many blocks, many short ones share a block.  A block walks its stretch unit
// by unit; for a unit it holds completely it writes the output; otherwise it parks its partial
// result and adds the chunks it did to the unit's counter, and the block that brings the
// counter to the unit's chunk count merges the stretches in block order.  The copy warp runs
// ahead across unit boundaries, so the ring of stages never drains inside a block.
//
// Taking up a unit costs a block about as much as `unit_cost` chunks (its queries, the merge of
// the four warps' shares, the output), so in the row every unit is that many positions longer
// than its chunks: the first `unit_cost` positions of a unit stand for no chunk.  A block whose
// stretch holds a hundred requests of one chunk then gets fewer chunks than one in the middle
// of a long request, and both end at about the same time.
//
// Scratch: slot (unit + block) is unique and increases along the row, so part_o holds
// (units + G) * 8 * d floats, part_ml (units + G) * 8 * 2, counters one int per unit (zero
// between calls).  No host-side plan: the blocks work the stretches out from kv_len themselves.

// The row: request after request, each with U units of (ov + its chunks) positions; request b
// starts at position (cum[b] + ov * b) * U.  The part of the row's stretch [i, i1) that lies in
// the unit holding position i: request b, unit u within it, `seg` chunks from chunk c_rel of the
// unit on (seg is 0 when the part covers only positions that stand for no chunk).  Returns the
// number of positions of the part.
__device__ __forceinline__ int balanced_part(long long i, long long i1, const int* cum, int B, int U, int ov,
                                             int& b, int& u, int& c_rel, int& seg, int& n_b) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {   // the largest b whose first position is <= i
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)(cum[mid] + ov * mid) * U <= i) lo = mid;
    else hi = mid - 1;
  }
  b = lo;
  n_b = cum[b + 1] - cum[b];
  const int nv = n_b + ov;
  const long long r = i - (long long)(cum[b] + ov * b) * U;
  u = (int)(r / nv);
  const int p = (int)(r - (long long)u * nv);
  const int len = (int)min((long long)(nv - p), i1 - i);
  const int first = max(p, ov);
  c_rel = first - ov;
  seg = max(0, p + len - first);
  return len;
}

// The stretches g_first .. g_last of one unit into its output row (head r of the unit's group,
// this thread's columns cgrp, cgrp + 16, ...), in block order.  Out of line: its many loads in
// flight need registers that the main loop's accumulators would otherwise have to share.
template <int DMAX>
__device__ __noinline__ void balanced_merge_unit(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                 int unit, int g_first, int g_last, int r, int cgrp, int d,
                                                 bf16* __restrict__ orow) {
  const float2* ml = reinterpret_cast<const float2*>(part_ml);
  float mm = -INFINITY, LL = 0.f, acc[DMAX / 16];
#pragma unroll
  for (int k = 0; k < DMAX / 16; ++k) acc[k] = 0.f;
  if (g_last - g_first < 8 && DMAX <= 128) {
    // Few stretches (the usual case): everything this thread needs is asked for before any of it
    // is used, so the merge costs one round trip to the L2.
    float2 v[8];
    float po[8][DMAX <= 128 ? DMAX / 16 : 1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool live = g_first + k <= g_last;
      const size_t slot = ((size_t)unit + g_first + k) * DEC_HEADS + r;
      v[k] = live ? __ldcg(ml + slot) : make_float2(-INFINITY, 0.f);
#pragma unroll
      for (int c = 0; c < (DMAX <= 128 ? DMAX / 16 : 1); ++c)
        po[k][c] = (live && cgrp + 16 * c < d) ? __ldcg(part_o + slot * d + cgrp + 16 * c) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) mm = fmaxf(mm, v[k].x);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float fk = (v[k].x == -INFINITY) ? 0.f : exp2f(v[k].x - mm);
      LL += v[k].y * fk;
#pragma unroll
      for (int c = 0; c < (DMAX <= 128 ? DMAX / 16 : 1); ++c) acc[c] += fk != 0.f ? fk * po[k][c] : 0.f;
    }
  } else {
    for (int gb = g_first; gb <= g_last; gb += 8) {   // eight stretches' (max, sum) in flight at a time
      float2 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
        v[k] = gb + k <= g_last ? __ldcg(ml + ((size_t)unit + gb + k) * DEC_HEADS + r) : make_float2(-INFINITY, 0.f);
#pragma unroll
      for (int k = 0; k < 8; ++k) mm = fmaxf(mm, v[k].x);
    }
    for (int gb = g_first; gb <= g_last; gb += 4) {   // four stretches' columns in flight at a time
      float2 v[4];
      float po[4][DMAX / 16];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool live = gb + k <= g_last;
        const size_t slot = ((size_t)unit + gb + k) * DEC_HEADS + r;
        v[k] = live ? __ldcg(ml + slot) : make_float2(-INFINITY, 0.f);
#pragma unroll
        for (int c = 0; c < DMAX / 16; ++c)
          po[k][c] = (live && cgrp + 16 * c < d) ? __ldcg(part_o + slot * d + cgrp + 16 * c) : 0.f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float fk = (v[k].x == -INFINITY) ? 0.f : exp2f(v[k].x - mm);
        LL += v[k].y * fk;
#pragma unroll
        for (int c = 0; c < DMAX / 16; ++c) acc[c] += fk != 0.f ? fk * po[k][c] : 0.f;
      }
    }
  }
  const float inv = LL > 0.f ? 1.f / LL : 0.f;
#pragma unroll
  for (int c = 0; c < DMAX / 16; ++c)
    if (cgrp + 16 * c < d) orow[cgrp + 16 * c] = __float2bfloat16_rn(acc[c] * inv);
}

#define BAL_THREADS (NTHREADS + 64)   // four consumer warps, the copy warp, the store warp (ROPE only)
template <int DMAX, bool ROPE>
__global__ void __launch_bounds__(ROPE ? BAL_THREADS : DEC_THREADS, DMAX <= 128 ? 2 : 1)
attention_decode_balanced_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                                 const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                                 const int* __restrict__ block_table, int bt_stride,
                                 const int* __restrict__ table_rows, int page_size, int page_shift,
                                 const int* __restrict__ q_start, const int* __restrict__ kv_len, int B, int nq,
                                 int nkv, int d, float scale, int window, int min_chunks, int unit_cost,
                                 float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                                 int* __restrict__ status, const float* __restrict__ rope_cs, int store_kv) {
  // ROPE (the head size is then DMAX exactly): rope_cs holds per query token [d / 2] sines then
  // [d / 2] cosines of its rotary angles; q arrives un-rotated and is rotated here, in registers; and with store_kv
  // the block that comes to a request's newest chunk first rotates the new key, writes it and
  // the new value into their page (they follow q in the token's row: q heads, k heads, v heads)
  // and only then copies the chunk.  One kernel and one kernel boundary less per layer.
  mi_pdl_launch_dependents();   // (what this kernel may touch before it waits: see attention_decode_kernel)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);                      // [DEC_STAGES][64][d]
  bf16* Vs = Ks + DEC_STAGES * KCHUNK * d;                           // [DEC_STAGES][64][d]
  float* merge_o = reinterpret_cast<float*>(Vs + DEC_STAGES * KCHUNK * d);   // [4][DEC_HEADS][d]
  int* cum = reinterpret_cast<int*>(merge_o + 4 * DEC_HEADS * d);    // [B + 1] chunks of the requests before b
  const int swz_mask = mi_swizzle_mask(d, 2);
  __shared__ float merge_m[4][DEC_HEADS], merge_l[4][DEC_HEADS];
  __shared__ __align__(8) uint64_t bars[DEC_STAGES], empty[DEC_STAGES], stored;
  __shared__ int is_last;
  __shared__ volatile int dead;   // a warp gave up waiting for a copy: everybody leaves at the next common point

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = lane >> 2, t4 = lane & 3;
  const int g = nq / nkv;
  const int hblocks = (g + DEC_HEADS - 1) / DEC_HEADS;
  const int U = nkv * hblocks;
  if (tid == 0) dead = 0;

  // chunks per request, and their running sum (one warp; B is at most a few hundred)
  for (int b = tid; b < B; b += (ROPE ? BAL_THREADS : DEC_THREADS)) {
    const int kl = kv_len[b];
    const int lo = window > 0 ? max(0, kl - window) : 0;   // (a window skips the chunks below it)
    cum[b + 1] = (kl + KCHUNK - 1) / KCHUNK - lo / KCHUNK;
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int b0 = 0; b0 < B; b0 += 32) {
      int v = b0 + lane < B ? cum[b0 + lane + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += up;
      }
      if (b0 + lane < B) cum[b0 + lane + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) cum[0] = 0;
  }
  __syncthreads();
  int ov = max(0, unit_cost);
  int G;
  {
    // Requests of one length, and fewer units than blocks: a block count that is a multiple of
    // the unit count makes every stretch a whole fraction of one unit (no block straddles two
    // units, every unit has the same number of stretches), which costs fewer partial results
    // than the last few blocks would bring.  Every block then takes up one unit: nothing to weigh.
    const long long units = (long long)B * U, chunks = (long long)cum[B] * U;
    const int n0 = cum[1];
    // a stretch shorter than min_chunks costs more in set-up and merging than it spreads
    const int g_plain = (int)min((long long)gridDim.x, max((long long)1, chunks / max(1, min_chunks)));
    if (units < g_plain && chunks == units * n0) {
      ov = 0;
      G = (int)(units * (g_plain / units));
    } else {
      G = (int)min((long long)gridDim.x, max((long long)1, (chunks + units * ov) / max(1, min_chunks)));
    }
  }
  const long long W = (long long)(cum[B] + ov * B) * U;
  if (W == 0) G = 1;
  if ((int)blockIdx.x >= G) return;
  if (status && *reinterpret_cast<volatile int*>(status)) return;   // an earlier block gave up waiting
  const long long i0 = W * blockIdx.x / G, i1 = W * (blockIdx.x + 1) / G;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < DEC_STAGES; ++i) {
      mbar_init(&bars[i], 1);
      mbar_init(&empty[i], 4);
    }
    mbar_init(&stored, 1);
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == 4) {
    // the copy warp: walks the stretch chunk by chunk and keeps the ring full
    PageLoader loader;
    const int pieces = 2 * (KCHUNK / PageLoader::piece_rows(page_size, page_shift));
    bool ok = true, waited = false, stored_seen = false;
    int it = 0;
    for (long long i = i0; i < i1 && ok;) {
      int b, u, c_rel, seg, n_b;
      const int len = balanced_part(i, i1, cum, B, U, ov, b, u, c_rel, seg, n_b);
      const int kvh = u / hblocks;
      const int kl = kv_len[b];
      const int lo = window > 0 ? max(0, kl - window) : 0;
      const int* table = block_table + (size_t)(table_rows ? table_rows[b] : b) * bt_stride;
      for (int s = 0; s < seg && ok; ++s, ++it) {
        const int c = lo / KCHUNK + c_rel + s, st = it % DEC_STAGES;
        if (it >= DEC_STAGES)
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[st], ((it / DEC_STAGES) - 1) & 1, status));
        if (!ok) break;
        if ((c + 1) * KCHUNK >= kl) {   // the chunk with the newest position: written by this step
          if (!waited) {
            mi_pdl_wait();
            waited = true;
          }
          if (ROPE && store_kv && !stored_seen) {
            // the other warps have rotated and stored the newest keys and values of this block's requests
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&stored, 0, status));
            if (!ok) break;
            fence_proxy_async_all();
            stored_seen = true;
          }
        }
        if (lane == 0) mbar_expect_tx(&bars[st], PageLoader::chunk_bytes(c, lo, kl, d, page_size, page_shift));
        __syncwarp();
        for (int t0 = 0; t0 < pieces; t0 += 32) {
          loader.t = t0 + lane;
          loader.fetch(table, page_size, page_shift, c, lo, kl);
          loader.issue<true>(Ks + st * KCHUNK * d, Vs + st * KCHUNK * d, kcache, vcache, page_size, page_shift, c, nkv, kvh,
                       d, &bars[st]);
        }
      }
      i += len;
    }
    return;
  }

  if (ROPE && warp == 5) {
    // The store warp (only when this kernel rotates and stores by itself): the newest key
    // (rotated) and value of every request whose last chunk this block reads go into their
    // pages, beside the other warps' work and long before the copy warp gets there.  Blocks
    // that read the same chunk (other head groups of the key/value head) write the same bytes.
    if (!store_kv) return;
    mi_pdl_wait();
    const int half = d >> 1, n_rot = half >> 3, cpr = d >> 3, per_unit = n_rot + cpr;
    for (long long i = i0; i < i1;) {
      int b, u, c_rel, seg, n_b;
      const int len = balanced_part(i, i1, cum, B, U, ov, b, u, c_rel, seg, n_b);
      if (seg > 0 && c_rel + seg == n_b) {
        const int kvh = u / hblocks, kl = kv_len[b], tok = q_start[b], pos = kl - 1;
        const int* table = block_table + (size_t)(table_rows ? table_rows[b] : b) * bt_stride;
        const int page = table[page_shift >= 0 ? (pos >> page_shift) : (pos / page_size)];
        const int off = inpage_of(pos, page_size, page_shift), swz = off & swz_mask;
        const bf16* krow = q + (size_t)tok * q_stride + (size_t)(nq + kvh) * d;
        const bf16* vrow = krow + (size_t)nkv * d;
        const size_t row = (((size_t)page * nkv + kvh) * page_size + off) * d;
        bf16* kdst = const_cast<bf16*>(kcache) + row;
        bf16* vdst = const_cast<bf16*>(vcache) + row;
        const float* cs = rope_cs + (size_t)tok * d;
        for (int item = lane; item < per_unit; item += 32) {
          if (item < n_rot) {
            uint4 a = *reinterpret_cast<const uint4*>(krow + item * 8);
            uint4 bb = *reinterpret_cast<const uint4*>(krow + half + item * 8);
            const float* sn = cs + item * 8;
            const float* cn = cs + half + item * 8;
            rotate_words(a.x, bb.x, sn + 0, cn + 0);
            rotate_words(a.y, bb.y, sn + 2, cn + 2);
            rotate_words(a.z, bb.z, sn + 4, cn + 4);
            rotate_words(a.w, bb.w, sn + 6, cn + 6);
            *reinterpret_cast<uint4*>(kdst + ((item ^ swz) << 3)) = a;
            *reinterpret_cast<uint4*>(kdst + (((n_rot + item) ^ swz) << 3)) = bb;
          } else {
            const int j = item - n_rot;
            *reinterpret_cast<uint4*>(vdst + ((j ^ swz) << 3)) = *reinterpret_cast<const uint4*>(vrow + j * 8);
          }
        }
      }
      i += len;
    }
    fence_proxy_async_all();   // a bulk copy reads these plain stores next
    __syncwarp();
    if (lane == 0) mbar_arrive(&stored);
    return;
  }

  mi_pdl_wait();   // the queries come from the kernel before this one
  const int ksteps = d >> 4;
  const float sc = scale * LOG2E;
  const int src0 = (2 * t4) * 4 + (qd >> 1), src1 = (2 * t4 + 1) * 4 + (qd >> 1);
  const bool odd_head = qd & 1;
  const int r = tid >> 4, cgrp = tid & 15;   // the merges' layout: 8 heads x 16 threads
  int it = 0;
  bool warp_dead = false;   // this warp's wait ran out: it keeps in step with the others but computes nothing more
  for (long long i = i0; i < i1;) {
    int b, u, c_rel, seg, n_b;
    const int len = balanced_part(i, i1, cum, B, U, ov, b, u, c_rel, seg, n_b);
    if (seg == 0) {   // only positions that stand for no chunk
      i += len;
      continue;
    }
    const int unit = b * U + u;
    const int kvh = u / hblocks, hb = u - kvh * hblocks;
    const int heads_here = min(DEC_HEADS, g - hb * DEC_HEADS);
    const int head0 = kvh * g + hb * DEC_HEADS;
    const int kl = kv_len[b], tok = q_start[b];
    const int lo = window > 0 ? max(0, kl - window) : 0;

    // Q as the B operand: lane (qd, t4) holds head qd, dims ks*16 + 2*t4 + {0,1} and + 8
    uint32_t qb[DMAX / 16][2];
    {
      const bf16* qrow = q + (size_t)tok * q_stride + (size_t)(head0 + qd) * d;
#pragma unroll
      for (int ks = 0; ks < DMAX / 16; ++ks) {
        qb[ks][0] = qb[ks][1] = 0u;
        if (ks < ksteps && qd < heads_here) {
          qb[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
          qb[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t4);
        }
      }
      if (ROPE && qd < heads_here) {
        // dims below d / 2 pair with the same lane's dims d / 2 further on: DMAX / 32 k steps further on
        const float* cs = rope_cs + (size_t)tok * d;
        constexpr int HK = DMAX / 32;
#pragma unroll
        for (int ks = 0; ks < HK; ++ks)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i0 = ks * 16 + e * 8 + 2 * t4;
            rotate_words(qb[ks][e], qb[ks + HK][e], cs + i0, cs + DMAX / 2 + i0);
          }
      }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[DMAX / 16][4];
#pragma unroll
    for (int k = 0; k < DMAX / 16; ++k) o[k][0] = o[k][1] = o[k][2] = o[k][3] = 0.f;

    for (int s = 0; s < seg; ++s, ++it) {
      const int c = lo / KCHUNK + c_rel + s, buf = it % DEC_STAGES;
      const bool arrived =
          !warp_dead && __all_sync(0xffffffffu, mbar_wait_bounded(&bars[buf], (it / DEC_STAGES) & 1, status));
      if (!arrived && !warp_dead) {
        warp_dead = true;
        if (lane == 0) dead = 1;
      }
      zero_masked_values<NTHREADS, true>(Vs + buf * KCHUNK * d, c, lo, kl, d);
      const int key0 = c * KCHUNK + warp * 16;
      const int kr = lane & 15, vr = (lane & 7) + (lane >> 4) * 8;
      const int ksw = inpage_of(key0 + kr, page_size, page_shift) & swz_mask;
      const int vsw = inpage_of(key0 + vr, page_size, page_shift) & swz_mask;
      const bf16* Kb = Ks + buf * KCHUNK * d + (warp * 16 + kr) * d;
      const bf16* Vb = Vs + buf * KCHUNK * d + (warp * 16 + vr) * d;
      if (arrived && key0 < kl && key0 + 16 > lo) {   // (the arithmetic of attention_decode_kernel)
        constexpr int GROUP = (DMAX / 16) < 8 ? (DMAX / 16) : 8;
        float sa[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g0 = 0; g0 < DMAX / 16; g0 += GROUP) {
          uint32_t kf[GROUP][4];
#pragma unroll
          for (int k = 0; k < GROUP; ++k)
            if (g0 + k < ksteps) ldmatrix_x4(kf[k], Kb + ((((g0 + k) * 2 + (lane >> 4)) ^ ksw) << 3));
#pragma unroll
          for (int k = 0; k < GROUP; ++k)
            if (g0 + k < ksteps) {
              if (k & 1) mma_bf16(s_odd, kf[k], qb[g0 + k][0], qb[g0 + k][1]);
              else mma_bf16(sa, kf[k], qb[g0 + k][0], qb[g0 + k][1]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) sa[e] += s_odd[e];
        uint32_t vf[GROUP][4];
#pragma unroll
        for (int k = 0; k < GROUP; ++k)
          if (k < ksteps) ldmatrix_x4_trans(vf[k], Vb + (((k * 2 + ((lane >> 3) & 1)) ^ vsw) << 3));
        const int j0 = key0 + qd, j1 = j0 + 8;
        const bool ok0 = j0 < kl && j0 >= lo, ok1 = j1 < kl && j1 >= lo;
        sa[0] = ok0 ? sa[0] * sc : -INFINITY;
        sa[1] = ok0 ? sa[1] * sc : -INFINITY;
        sa[2] = ok1 ? sa[2] * sc : -INFINITY;
        sa[3] = ok1 ? sa[3] * sc : -INFINITY;
        float alpha[2], p[4];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          float mx = fmaxf(sa[hh], sa[2 + hh]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m_run[hh], mx);
          alpha[hh] = exp2f(m_run[hh] - m_new);
          p[hh] = exp2f(sa[hh] - m_new);
          p[2 + hh] = exp2f(sa[2 + hh] - m_new);
          m_run[hh] = m_new;
          l_run[hh] = l_run[hh] * alpha[hh] + (p[hh] + p[2 + hh]);
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
          for (int k = 0; k < DMAX / 16; ++k) {
            o[k][0] *= alpha[0]; o[k][1] *= alpha[1];
            o[k][2] *= alpha[0]; o[k][3] *= alpha[1];
          }
        }
        const uint32_t p_lo = pack_bf16(p[0], p[1]), p_hi = pack_bf16(p[2], p[3]);
        const uint32_t x0 = __shfl_sync(0xffffffffu, p_lo, src0), x1 = __shfl_sync(0xffffffffu, p_lo, src1);
        const uint32_t y0 = __shfl_sync(0xffffffffu, p_hi, src0), y1 = __shfl_sync(0xffffffffu, p_hi, src1);
        const uint32_t sel = odd_head ? 0x7632u : 0x5410u;
        const uint32_t pb0 = __byte_perm(x0, x1, sel), pb1 = __byte_perm(y0, y1, sel);
#pragma unroll
        for (int k = 0; k < GROUP; ++k)
          if (k < ksteps) mma_bf16(o[k], vf[k], pb0, pb1);
#pragma unroll
        for (int g0 = GROUP; g0 < DMAX / 16; g0 += GROUP) {
#pragma unroll
          for (int k = 0; k < GROUP; ++k)
            if (g0 + k < ksteps) ldmatrix_x4_trans(vf[k], Vb + ((((g0 + k) * 2 + ((lane >> 3) & 1)) ^ vsw) << 3));
#pragma unroll
          for (int k = 0; k < GROUP; ++k)
            if (g0 + k < ksteps) mma_bf16(o[g0 + k], vf[k], pb0, pb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[buf]);   // this warp is done with the stage
    }

    // the four warps' shares of this stretch into one (m, l, O)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      float l = l_run[hh];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      if (qd == 0) {
        merge_m[warp][2 * t4 + hh] = m_run[hh];
        merge_l[warp][2 * t4 + hh] = l;
      }
    }
#pragma unroll
    for (int k = 0; k < DMAX / 16; ++k)
      if (k < ksteps) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          merge_o[((size_t)warp * DEC_HEADS + 2 * t4 + (e & 1)) * d + k * 16 + qd + 8 * (e >> 1)] = o[k][e];
      }
    consumer_barrier(NTHREADS);
    if (dead) break;   // (status is set; the output is invalid) all four warps see the same value here
    float m = -INFINITY, L = 0.f, f[4];
    if (r < heads_here) {
      m = merge_m[0][r];
#pragma unroll
      for (int w = 1; w < 4; ++w) m = fmaxf(m, merge_m[w][r]);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        f[w] = (merge_m[w][r] == -INFINITY) ? 0.f : exp2f(merge_m[w][r] - m);
        L += merge_l[w][r] * f[w];
      }
    }
    const bool whole = seg == n_b;   // this block held the whole unit: no scratch, no counter
    const int head = head0 + r;
    if (r < heads_here) {
      if (whole) {
        const float inv = L > 0.f ? 1.f / L : 0.f;
        bf16* orow = out + (size_t)tok * out_stride + (size_t)head * d;
        for (int k = cgrp; k < d; k += 16) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) acc += f[w] * merge_o[((size_t)w * DEC_HEADS + r) * d + k];
          orow[k] = __float2bfloat16_rn(acc * inv);
        }
      } else {
        const size_t slot = ((size_t)unit + blockIdx.x) * DEC_HEADS + r;
        float* po = part_o + slot * d;
        for (int k = cgrp; k < d; k += 16) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) acc += f[w] * merge_o[((size_t)w * DEC_HEADS + r) * d + k];
          po[k] = acc;
        }
        if (cgrp == 0) {
          part_ml[slot * 2] = m;
          part_ml[slot * 2 + 1] = L;
        }
      }
    }
    if (!whole) {
      // count this stretch's chunks in; whoever completes the unit merges its stretches in block order
      __threadfence();
      consumer_barrier(NTHREADS);
      if (tid == 0) is_last = (atomicAdd(&counters[unit], seg) + seg == n_b) ? 1 : 0;
      consumer_barrier(NTHREADS);
      if (is_last) {
        __threadfence();
        // the blocks whose stretches hold the unit's chunks: its positions from `ov` on
        const long long start = (long long)(cum[b] + ov * b) * U + (long long)u * (n_b + ov) + ov;
        const int g_first = (int)(((start + 1) * G - 1) / W), g_last = (int)(((start + n_b) * G - 1) / W);
        if (r < heads_here)
          balanced_merge_unit<DMAX>(part_o, part_ml, unit, g_first, g_last, r, cgrp, d,
                                    out + (size_t)tok * out_stride + (size_t)head * d);
        if (tid == 0) counters[unit] = 0;   // ready for the next call
      }
    }
    consumer_barrier(NTHREADS);   // merge_o, merge_m and is_last may be written again
    i += len;
  }
  // a request that holds no key at all has no chunk in the row: its output rows are zero
  if (blockIdx.x == 0)
    for (int b = 0; b < B; ++b)
      if (cum[b + 1] == cum[b]) {
        bf16* orow = out + (size_t)q_start[b] * out_stride;
        for (int k = tid; k < nq * d; k += NTHREADS) orow[k] = __float2bfloat16_rn(0.f);
      }
}

// ------------------------------------------------------------------------------- prefill

// 2^x as one instruction of the special-function unit (2 ulp, results below 2^-126 are 0):
// the prefill kernel computes one per score, and exp2f's range fix-ups double its cost.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define PROWS 128   // rows (token, head in group) per block

// Each warp owns MT groups of 16 rows.  With MT = 2 a key or value fragment fetched from
// shared memory feeds two MMAs instead of one (four warps, 128 threads, up to 255 registers,
// two blocks per SM); head sizes above 128 keep MT = 1 (eight warps), where the output
// accumulators of two row groups would not fit the register file.
template <int DMAX>
struct PrefillShape {
  static constexpr int MT = DMAX <= 128 ? 2 : 1;
  static constexpr int WARPS = PROWS / (16 * MT);
  static constexpr int THREADS = WARPS * 32;
  static constexpr int BLOCKS_PER_SM = DMAX <= 128 ? 2 : 1;
};

template <int DMAX>
__global__ void __launch_bounds__(PrefillShape<DMAX>::THREADS, PrefillShape<DMAX>::BLOCKS_PER_SM)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                         const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                         const int* __restrict__ block_table, int bt_stride, const int* __restrict__ table_rows,
                        int page_size, int page_shift,
                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                         const int* __restrict__ kv_len, const int* __restrict__ tile_req,
                         const int* __restrict__ tile_tok0, int nq, int nkv, int d, float scale, int window,
                         int gb, int tt, int* __restrict__ status) {
  constexpr int MT = PrefillShape<DMAX>::MT;
  constexpr int THREADS = PrefillShape<DMAX>::THREADS;
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int sd = d + 8;
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);   // [2][64][d], rows unpadded (chunks permuted)
  bf16* Vs = Ks + 2 * KCHUNK * d;                 // [2][64][d]
  bf16* Qs = Vs + 2 * KCHUNK * d;                 // [PROWS][sd], rows padded
  const int swz_mask = mi_swizzle_mask(d, 2);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qd = lane >> 2, t4 = lane & 3;
  const int g = nq / nkv;
  const int hblocks = (g + gb - 1) / gb;
  // Blocks start in the order of their index.  The caller lists the tiles with the most keys
  // first, and all head groups of a tile come before the next tile, so the longest blocks of
  // the whole launch start first and the short ones fill the gaps at the end.
  const int n_hg = nkv * hblocks;
  const int tile = blockIdx.x / n_hg, hg = blockIdx.x - tile * n_hg;
  const int kvh = hg / hblocks, hb = hg - kvh * hblocks;
  const int b = tile_req[tile], tok0 = tile_tok0[tile];
  const int ql = q_len[b], kl = kv_len[b], qs = q_start[b];
  const int ntok = min(tt, ql - tok0);
  const int p_first = kl - ql + tok0;
  const int hi = p_first + ntok;  // one past the last key any row of the tile sees
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int heads_here = min(gb, g - hb * gb);
  const int* table = block_table + (size_t)(table_rows ? table_rows[b] : b) * bt_stride;

  if (status && *reinterpret_cast<volatile int*>(status)) return;   // an earlier block gave up waiting
  // row R of the tile: token tok0 + R / gb, head kvh * g + hb * gb + R % gb
  const int units = d >> 3;
  for (int idx = tid; idx < PROWS * units; idx += THREADS) {
    const int R = idx / units, u = idx - R * units;
    const int tk = R / gb, mem = R - tk * gb;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (tk < ntok && mem < heads_here)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(qs + tok0 + tk) * q_stride +
                                          (size_t)(kvh * g + hb * gb + mem) * d + u * 8);
    *reinterpret_cast<uint4*>(Qs + R * sd + u * 8) = v;
  }

  // this lane's rows: two per group of 16
  const int row0 = warp * 16 * MT;   // the warp's first row
  int prow[MT][2], lorow[MT][2];
  bool rvalid[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int R = row0 + mt * 16 + qd + 8 * hr;
      const int tk = R / gb, mem = R - tk * gb;
      rvalid[mt][hr] = tk < ntok && mem < heads_here;
      prow[mt][hr] = p_first + tk;
      lorow[mt][hr] = window > 0 ? max(0, prow[mt][hr] - window + 1) : 0;
    }
  // the warp's rows span tokens [wt0, wt1]
  const int wt0 = row0 / gb, wt1 = min(ntok - 1, (row0 + 16 * MT - 1) / gb);
  const bool warp_active = wt0 < ntok;
  const int warp_hi = p_first + wt1 + 1;                                   // one past its last visible key
  const int warp_lo = window > 0 ? max(0, p_first + wt0 - window + 1) : 0;  // its first visible key

  float m_run[MT][2], l_run[MT][2];
  float o[MT][DMAX / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m_run[mt][0] = m_run[mt][1] = -INFINITY;
    l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
    for (int i = 0; i < DMAX / 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
  }
  const float sc = scale * LOG2E;
  const int ksteps = d >> 4;
  const int c0 = lo / KCHUNK, c1 = (hi + KCHUNK - 1) / KCHUNK;
  const uint32_t q_addr = smem_u32(Qs) + (uint32_t)((row0 + (lane & 15)) * sd + (lane >> 4) * 8) * 2u;

  __shared__ __align__(8) uint64_t bars[2];
  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  PageLoader loader;
  loader.fetch(table, page_size, page_shift, c0, lo, hi);
  if (tid == 0) mbar_expect_tx(&bars[0], PageLoader::chunk_bytes(c0, lo, hi, d, page_size, page_shift));
  loader.issue(Ks, Vs, kcache, vcache, page_size, page_shift, c0, nkv, kvh, d, &bars[0]);
  if (c0 + 1 < c1) loader.fetch(table, page_size, page_shift, c0 + 1, lo, hi);
  __syncthreads();   // the query tile is visible to every warp

  for (int c = c0; c < c1; ++c) {
    const int buf = (c - c0) & 1;
    if (c + 1 < c1) {
      if (tid == 0)
        mbar_expect_tx(&bars[buf ^ 1], PageLoader::chunk_bytes(c + 1, lo, hi, d, page_size, page_shift));
      loader.issue(Ks + (buf ^ 1) * KCHUNK * d, Vs + (buf ^ 1) * KCHUNK * d, kcache, vcache, page_size, page_shift,
                   c + 1, nkv, kvh, d, &bars[buf ^ 1]);
      if (c + 2 < c1) loader.fetch(table, page_size, page_shift, c + 2, lo, hi);
    }
    const bool arrived = __all_sync(0xffffffffu, mbar_wait_bounded(&bars[buf], ((c - c0) >> 1) & 1, status));
    zero_masked_values<THREADS>(Vs + buf * KCHUNK * d, c, lo, hi, d);
    const bf16* Kb = Ks + buf * KCHUNK * d;
    const bf16* Vb = Vs + buf * KCHUNK * d;
    const int key0 = c * KCHUNK;
    // this lane's ldmatrix rows within each group of 16 keys, with their chunk permutations
    const int kr = (lane & 7) + (lane >> 4) * 8, vr = (lane & 7) + ((lane >> 3) & 1) * 8;
    // Shared-memory addresses of the fragments: chunk (2 * step + b) ^ sw of row r lies at
    //   base(r) + (((b ^ sw) & 1) << 4)  +  ((step * 32) ^ ((sw & ~1) << 4))
    // so the inner loops add one constant xor-ed with a per-row pattern.
    uint32_t kaddr[4], kxor[4], vaddr[4], vxor[4];
    {
      const uint32_t kbuf = smem_u32(Kb), vbuf = smem_u32(Vb);
      const int kbit = (lane >> 3) & 1, vbit = lane >> 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ksw = inpage_of(key0 + i * 16 + kr, page_size, page_shift) & swz_mask;
        const int vsw = inpage_of(key0 + i * 16 + vr, page_size, page_shift) & swz_mask;
        kaddr[i] = kbuf + (uint32_t)((i * 16 + kr) * d) * 2u + (uint32_t)(((kbit ^ ksw) & 1) << 4);
        kxor[i] = (uint32_t)((ksw & ~1) << 4);
        vaddr[i] = vbuf + (uint32_t)((i * 16 + vr) * d) * 2u + (uint32_t)(((vbit ^ vsw) & 1) << 4);
        vxor[i] = (uint32_t)((vsw & ~1) << 4);
      }
    }
    if (arrived && warp_active && key0 < warp_hi && key0 + KCHUNK > warp_lo) {
      float s[MT][8][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 8; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < DMAX / 16; ++ks) {
        if (ks < ksteps) {
          uint32_t a[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            ldsm_x4(a[mt], q_addr + (uint32_t)(mt * 16 * sd * 2 + ks * 32));
#pragma unroll
          for (int kp = 0; kp < 4; ++kp) {
            uint32_t kb[4];
            ldsm_x4(kb, kaddr[kp] + ((uint32_t)(ks * 32) ^ kxor[kp]));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16(s[mt][2 * kp], a[mt], kb[0], kb[1]);
              mma_bf16(s[mt][2 * kp + 1], a[mt], kb[2], kb[3]);
            }
          }
        }
      }
      uint32_t pa[MT][4][4];
      // A chunk that every row of the warp sees whole (all of them, in a long prompt, but the
      // few on the diagonal and at a window's edge) needs no mask.  Scores stay unscaled; the
      // scale is folded into the exponent's multiply-add: p = 2^(s * sc - m), m = sc * max(s).
      const bool interior = key0 + KCHUNK - 1 <= p_first + wt0 &&
                            key0 >= (window > 0 ? max(0, p_first + wt1 - window + 1) : 0);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        if (!interior) {
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int hr = e >> 1;
              const int j = key0 + nt * 8 + 2 * t4 + (e & 1);
              if (!(rvalid[mt][hr] && j <= prow[mt][hr] && j >= lorow[mt][hr])) s[mt][nt][e] = -INFINITY;
            }
        }
        // both rows of the lane side by side and sums in four strands: short dependency chains
        float mx[2], alpha[2] = {1.f, 1.f};
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          float m4[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            m4[i] = fmaxf(fmaxf(s[mt][2 * i][2 * hr], s[mt][2 * i][2 * hr + 1]),
                          fmaxf(s[mt][2 * i + 1][2 * hr], s[mt][2 * i + 1][2 * hr + 1]));
          mx[hr] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 1));
          mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 2));
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          const float m_new = fmaxf(m_run[mt][hr], mx[hr] * sc);   // sc > 0
          float sum4[4] = {0.f, 0.f, 0.f, 0.f};
          if (m_new != -INFINITY) {
            alpha[hr] = fast_exp2(m_run[mt][hr] - m_new);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
              s[mt][nt][2 * hr] = fast_exp2(fmaf(s[mt][nt][2 * hr], sc, -m_new));
              s[mt][nt][2 * hr + 1] = fast_exp2(fmaf(s[mt][nt][2 * hr + 1], sc, -m_new));
              sum4[nt & 3] += s[mt][nt][2 * hr] + s[mt][nt][2 * hr + 1];
            }
          } else {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) s[mt][nt][2 * hr] = s[mt][nt][2 * hr + 1] = 0.f;
          }
          m_run[mt][hr] = m_new;
          l_run[mt][hr] = l_run[mt][hr] * alpha[hr] + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        }
        // the accumulators are rescaled only when some row's maximum moved (exact: alpha is 1 otherwise)
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
          for (int i = 0; i < DMAX / 8; ++i) {
            o[mt][i][0] *= alpha[0];
            o[mt][i][1] *= alpha[0];
            o[mt][i][2] *= alpha[1];
            o[mt][i][3] *= alpha[1];
          }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          pa[mt][kk][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
          pa[mt][kk][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
          pa[mt][kk][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
          pa[mt][kk][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
        }
      }
#pragma unroll
      for (int dt = 0; dt < DMAX / 16; ++dt) {
        if (dt < ksteps) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            uint32_t vb[4];
            ldsm_x4_trans(vb, vaddr[kk] + ((uint32_t)(dt * 32) ^ vxor[kk]));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16(o[mt][2 * dt], pa[mt][kk], vb[0], vb[1]);
              mma_bf16(o[mt][2 * dt + 1], pa[mt][kk], vb[2], vb[3]);
            }
          }
        }
      }
    }
    if (__syncthreads_or(!arrived)) break;   // a wait gave up: stop (status is set)
  }

#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float l = l_run[mt][hr];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (!rvalid[mt][hr] || !(l > 0.f)) continue;
      const float inv = 1.f / l;
      const int R = row0 + mt * 16 + qd + 8 * hr;
      const int tk = R / gb, mem = R - tk * gb;
      bf16* orow = out + (size_t)(qs + tok0 + tk) * out_stride + (size_t)(kvh * g + hb * gb + mem) * d;
#pragma unroll
      for (int i = 0; i < DMAX / 8; ++i) {
        if (i * 8 < d) {
          const uint32_t v = pack_bf16(o[mt][i][2 * hr] * inv, o[mt][i][2 * hr + 1] * inv);
          *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * t4) = v;
        }
      }
    }
}

// ------------------------------------------------------------------------------- host side

static int check_common(const void* q, int q_stride, const void* out, int out_stride, const void* kcache,
                        const void* vcache, int nq, int nkv, int d, int page_size, int window) {
  if (!mi_l2_hints_enabled()) {   // once per device: tell the kernels
    static bool told[64];
    int dev = -1;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !told[dev]) {
      const int off = 0;
      if (cudaMemcpyToSymbol(g_stream_once_hint, &off, sizeof(int)) == cudaSuccess) told[dev] = true;
    }
  }
  if (d <= 0 || d % 16 != 0 || d > 256) MI_REFUSE("attention: head size %d is not a multiple of 16 in [16, 256]", d);
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0) MI_REFUSE("attention: %d query heads cannot share %d key/value heads", nq, nkv);
  if (page_size <= 0 || window < 0) MI_REFUSE("attention: bad page size %d or window %d", page_size, window);
  if (!mi_aligned(q, 16) || q_stride % 8 != 0) MI_REFUSE("attention: queries must be 16-byte aligned with a row stride that is a multiple of 8");
  if (!mi_aligned(out, 4) || out_stride % 2 != 0) MI_REFUSE("attention: output rows must be 4-byte aligned");
  if (!mi_aligned(kcache, 16) || !mi_aligned(vcache, 16)) MI_REFUSE("attention: cache must be 16-byte aligned");
  return 0;
}

// Set to 1 by a kernel whose bounded wait for a copy gave up (its output is then invalid).
static __device__ int g_wait_status;
#define MI_MAX_DEVICES 64
static int* g_wait_status_ptr[MI_MAX_DEVICES];

// A word the host shares among its kernel libraries (mi_set_status_word), per device; null:
// this library's own word above.
static int* g_status_word_host[MI_MAX_DEVICES];

static int* wait_status_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MI_MAX_DEVICES) return nullptr;
  if (g_status_word_host[dev]) return g_status_word_host[dev];
  if (!g_wait_status_ptr[dev]) {
    int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_wait_status) != cudaSuccess) return nullptr;
    g_wait_status_ptr[dev] = p;
  }
  return g_wait_status_ptr[dev];
}

// Report give-ups of this library's kernels on the current device into `device_word` (an int in
// device memory that the caller owns and keeps alive; null: back to the library's own word).
extern "C" int mi_set_status_word(int* device_word) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MI_MAX_DEVICES) MI_REFUSE("status word: bad device");
  g_status_word_host[dev] = device_word;
  return 0;
}

// 1 if a kernel of this library gave up waiting for a copy since the last reset (synchronises).
extern "C" int mi_attention_wait_status(int reset) {
  int v = 0;
  int* word = wait_status_ptr();
  if (!word || cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v) cudaMemset(word, 0, sizeof(int));
  return v;
}

static size_t smem_bytes(int q_rows, int d) {   // padded query rows, two unpadded key and value tiles
  return ((size_t)q_rows * (d + 8) + (size_t)4 * KCHUNK * d) * sizeof(bf16);
}

static int shift_of(int page_size) {  // log2 for powers of two, else -1
  if (page_size & (page_size - 1)) return -1;
  int s = 0;
  while ((1 << s) < page_size) ++s;
  return s;
}

// How many arrival counters a call needs (one per request and head group).
extern "C" int mi_attention_decode_counters(int B, int nq, int nkv) {
  const int g = nq / nkv;
  return B * nkv * ((g + DEC_HEADS - 1) / DEC_HEADS);
}

// Scratch: part_o holds B * nq * n_splits * d floats, part_ml holds B * nq * n_splits * 2 floats,
// counters holds mi_attention_decode_counters(B, nq, nkv) ints that are zero on entry (the kernel
// leaves them zero).  All three may be null when n_splits == 1.
// slice_chunks (may be null) points at one int on the device, read when the kernel runs: the
// number of 64-key chunks per slice, the same for every request.  Null cuts every request's
// own span into n_splits equal slices.
extern "C" int mi_attention_decode_sliced(const void* q, int q_stride, void* out, int out_stride,
                                          const void* kcache, const void* vcache, const int* block_table,
                                          int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                          const int* kv_len,
                                          int B, int nq, int nkv, int d, float scale, int window, int n_splits,
                                          const int* slice_chunks, float* part_o, float* part_ml, int* counters,
                                          cudaStream_t stream) {
  if (B <= 0) return 0;
  if (int rc = check_common(q, q_stride, out, out_stride, kcache, vcache, nq, nkv, d, page_size, window)) return rc;
  if (n_splits < 1 || n_splits > 64) MI_REFUSE("attention: n_splits must be in [1, 64], got %d", n_splits);
  const int page_shift = shift_of(page_size);
  if (n_splits > 1 && (!part_o || !part_ml || !counters)) MI_REFUSE("attention: split results need scratch memory");
  // the merge reads (max, sum) pairs as one 8-byte load
  if (n_splits > 1 && (!mi_aligned(part_o, 4) || !mi_aligned(part_ml, 8) || !mi_aligned(counters, 4)))
    MI_REFUSE("attention: scratch must be aligned (part_o and counters to 4 bytes, part_ml to 8)");
  const int g = nq / nkv, hblocks = (g + DEC_HEADS - 1) / DEC_HEADS;
  if (B > 65535 || nkv * hblocks > 65535) MI_REFUSE("attention: batch or head count too large for one launch");
  const size_t smem = (size_t)(2 * DEC_STAGES * KCHUNK) * d * sizeof(bf16);
  dim3 grid(n_splits, nkv * hblocks, B);
#define MI_DECODE(DMAX)                                                                                 \
  do {                                                                                                  \
    auto kern = attention_decode_kernel<DMAX>;                                                          \
    if (smem > 40 * 1024) { /* the kernel also has a few KB of static shared memory */                  \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                              \
    }                                                                                                   \
    MI_LAUNCH((kern), grid, DEC_THREADS, smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,         \
                                           (const bf16*)kcache, (const bf16*)vcache, block_table,       \
                                           bt_stride, table_rows, page_size, page_shift, q_start, kv_len, nq, nkv,  \
                                           d, scale, window, n_splits, slice_chunks, part_o, part_ml,   \
                                           counters, wait_status_ptr());                                \
  } while (0)
  if (d <= 64) MI_DECODE(64);
  else if (d <= 128) MI_DECODE(128);
  else MI_DECODE(256);
#undef MI_DECODE
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                   const void* vcache, const int* block_table, int bt_stride, int page_size,
                                   const int* q_start, const int* kv_len, int B, int nq, int nkv, int d,
                                   float scale, int window, int n_splits, float* part_o, float* part_ml,
                                   int* counters, cudaStream_t stream) {
  return mi_attention_decode_sliced(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride, nullptr, page_size,
                                    q_start, kv_len, B, nq, nkv, d, scale, window, n_splits, nullptr, part_o,
                                    part_ml, counters, stream);
}

// What taking up a unit costs a block, in chunks (attention_decode_balanced_kernel's unit_cost): measured, a unit
// costs about as much as two chunks; times stop falling between three and four.  A negative argument only reads.
static int g_unit_cost = 3;
extern "C" int mi_attention_decode_balanced_unit_cost(int chunks) {
  const int before = g_unit_cost;
  if (chunks >= 0) g_unit_cost = chunks;
  return before;
}

static size_t balanced_smem_bytes(int B, int d) {   // the ring, the warps' merge buffer, the running sum of chunks
  return (size_t)(2 * DEC_STAGES * KCHUNK) * d * sizeof(bf16) + (size_t)4 * DEC_HEADS * d * sizeof(float) +
         (size_t)(B + 1) * sizeof(int);
}

// Blocks the balanced decode kernel should be started with on a GPU of `sms` SMs, and the
// scratch it needs for B requests: floats of part_o and part_ml, ints of counters (zero before
// the first call; the kernel leaves them zero).
extern "C" int mi_attention_decode_balanced_scratch(int B, int nq, int nkv, int d, int sms, int* grid,
                                                    long long* o_floats, long long* ml_floats, int* counter_ints) {
  if (B <= 0 || nq <= 0 || nkv <= 0 || nq % nkv || d <= 0 || sms <= 0) MI_REFUSE("attention: bad sizes");
  const int g = nq / nkv, hblocks = (g + DEC_HEADS - 1) / DEC_HEADS, units = B * nkv * hblocks;
  const size_t smem = balanced_smem_bytes(B, d);
  // two blocks share an SM when both fit its 228 KB (each also takes 1 KB of reserve and its static part)
  *grid = sms * (2 * (smem + 1024 + 512) <= 228 * 1024 ? 2 : 1);
  *o_floats = (long long)(units + *grid) * DEC_HEADS * d;
  *ml_floats = (long long)(units + *grid) * DEC_HEADS * 2;
  *counter_ints = units;
  return 0;
}

// Decode attention with the keys of all requests spread evenly over `grid` persistent blocks
// (attention_decode_balanced_kernel); scratch as mi_attention_decode_balanced_scratch says.
extern "C" int mi_attention_decode_balanced(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                            const void* vcache, const int* block_table, int bt_stride,
                                            const int* table_rows, int page_size, const int* q_start,
                                            const int* kv_len, int B, int nq, int nkv, int d, float scale, int window,
                                            int grid, float* part_o, float* part_ml, int* counters,
                                            const float* rope_cs, int store_kv, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (rope_cs && ((d != 64 && d != 128 && d != 256) || !mi_aligned(rope_cs, 4)))
    MI_REFUSE("attention: rotating inside the decode kernel needs a head size of 64, 128 or 256, got %d", d);
  if (int rc = check_common(q, q_stride, out, out_stride, kcache, vcache, nq, nkv, d, page_size, window)) return rc;
  if (grid <= 0 || !part_o || !part_ml || !counters) MI_REFUSE("attention: the balanced kernel needs its grid and scratch");
  if (!mi_aligned(part_o, 4) || !mi_aligned(part_ml, 8) || !mi_aligned(counters, 4))
    MI_REFUSE("attention: scratch must be aligned (part_o and counters to 4 bytes, part_ml to 8)");
  if (B > 16384) MI_REFUSE("attention: %d requests in one decode step", B);
  const int page_shift = shift_of(page_size);
  const size_t smem = balanced_smem_bytes(B, d);
#define MI_DECODE_BAL(DMAX, ROPE)                                                                         \
  do {                                                                                                    \
    auto kern = attention_decode_balanced_kernel<DMAX, ROPE>;                                             \
    if (smem > 40 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                                \
    }                                                                                                     \
    MI_LAUNCH((kern), grid, ROPE ? BAL_THREADS : DEC_THREADS, smem, stream, (const bf16*)q, q_stride,     \
              (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, block_table, bt_stride,   \
              table_rows, page_size, page_shift, q_start, kv_len, B, nq, nkv, d, scale, window, 4,        \
              g_unit_cost, part_o, part_ml, counters, wait_status_ptr(), rope_cs, store_kv);              \
  } while (0)
  if (rope_cs) {
    if (d == 64) MI_DECODE_BAL(64, true);
    else if (d == 128) MI_DECODE_BAL(128, true);
    else MI_DECODE_BAL(256, true);
  } else if (d <= 64) MI_DECODE_BAL(64, false);
  else if (d <= 128) MI_DECODE_BAL(128, false);
  else MI_DECODE_BAL(256, false);
#undef MI_DECODE_BAL
  MI_RETURN_LAUNCH_STATUS();
}

// Tokens per tile the prefill kernel wants for a group of g query heads per key/value head.
extern "C" int mi_attention_prefill_tile_tokens(int g) {
  const int gb = g < PROWS ? g : PROWS;
  return PROWS / gb;
}

extern "C" int mi_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                    const void* vcache, const int* block_table, int bt_stride, const int* table_rows,
                                    int page_size, const int* q_start, const int* q_len, const int* kv_len,
                                    const int* tile_req, const int* tile_tok0, int n_tiles, int tile_tokens,
                                    int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (int rc = check_common(q, q_stride, out, out_stride, kcache, vcache, nq, nkv, d, page_size, window)) return rc;
  if (!(scale > 0.f)) MI_REFUSE("attention: the score scale must be positive (the row maximum is taken before scaling)");
  const int g = nq / nkv;
  const int gb = g < PROWS ? g : PROWS;
  if (tile_tokens != PROWS / gb) MI_REFUSE("attention: tiles of %d tokens, the kernel wants %d", tile_tokens, PROWS / gb);
  const int hblocks = (g + gb - 1) / gb;
  if ((long long)n_tiles * nkv * hblocks > 0x7fffffffLL) MI_REFUSE("attention: too many blocks for one launch");
  const size_t smem = smem_bytes(PROWS, d);
  const int page_shift = shift_of(page_size);
  dim3 grid((unsigned)(n_tiles * nkv * hblocks));
#define MI_PREFILL(DMAX)                                                                                \
  do {                                                                                                  \
    auto kern = attention_prefill_kernel<DMAX>;                                                         \
    if (smem > 40 * 1024) {                                                                             \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return (int)e;                                                              \
    }                                                                                                   \
    MI_LAUNCH((kern), grid, PrefillShape<DMAX>::THREADS, smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, \
                                           (const bf16*)kcache, (const bf16*)vcache, block_table,       \
                                           bt_stride, table_rows, page_size, page_shift, q_start, q_len, kv_len,    \
                                           tile_req, tile_tok0, nq, nkv, d, scale, window, gb,          \
                                           PROWS / gb, wait_status_ptr());                              \
  } while (0)
  if (d <= 64) MI_PREFILL(64);
  else if (d <= 128) MI_PREFILL(128);
  else MI_PREFILL(256);
#undef MI_PREFILL
  MI_RETURN_LAUNCH_STATUS();
}

// ------------------------------------------------------------------------------- no allocation
//
// The same decode attention with the split-merge scratch in a static device array, for
// callers that cannot allocate (see attention_noalloc.h).

#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[MI_ATTENTION_NOALLOC_MAX_FLOATS];

// In host code `g_noalloc_scratch` is only a handle; the address a kernel can use has to be
// asked for, once per device, with that device current.
#define MI_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_device_ptr[MI_NOALLOC_MAX_DEVICES];

extern "C" int mi_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                           const void* kcache, const void* vcache, const int* block_table,
                                           int bt_stride, int page_size, const int* q_start, const int* kv_len,
                                           int B, int nq, int nkv, int d, float scale, int window, int n_splits,
                                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nq <= 0 || d <= 0 || n_splits < 1) MI_REFUSE("attention (no allocation): bad sizes");
  const size_t slots = (size_t)B * nq * n_splits;
  // The arrival counters come first, rounded up to a multiple of four (16 bytes), so that the
  // partial results behind them start on a 16-byte boundary and the (max, sum) pairs behind
  // those (slots * d floats further, d a multiple of 16) on an 8-byte one.
  const size_t n_counters = ((size_t)mi_attention_decode_counters(B, nq, nkv > 0 ? nkv : 1) + 3) & ~(size_t)3;
  const size_t need = slots * ((size_t)d + 2) + n_counters;
  if (need > (size_t)MI_ATTENTION_NOALLOC_MAX_FLOATS)
    MI_REFUSE("attention (no allocation): %zu floats of scratch needed (B=%d, heads=%d, slices=%d, head size=%d), "
              "the built-in array holds %d",
              need, B, nq, n_splits, d, MI_ATTENTION_NOALLOC_MAX_FLOATS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(g_mi_error, sizeof(g_mi_error), "CUDA: %s", cudaGetErrorString(e));
    return (int)e;
  }
  if (dev < 0 || dev >= MI_NOALLOC_MAX_DEVICES) MI_REFUSE("attention (no allocation): device %d is out of range", dev);
  if (g_noalloc_device_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      snprintf(g_mi_error, sizeof(g_mi_error), "CUDA: cannot resolve the scratch array: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : MI_REFUSED;
    }
    g_noalloc_device_ptr[dev] = p;
  }
  // the arrival counters must be zero when the kernel starts; the array keeps whatever the
  // last call left (a call that was cut short could leave a count behind)
  int* counters = reinterpret_cast<int*>(g_noalloc_device_ptr[dev]);
  float* part_o = g_noalloc_device_ptr[dev] + n_counters;
  float* part_ml = part_o + slots * (size_t)d;
  if (n_splits > 1) {
    e = cudaMemsetAsync(counters, 0, n_counters * sizeof(int), stream);
    if (e != cudaSuccess) {
      snprintf(g_mi_error, sizeof(g_mi_error), "CUDA: %s", cudaGetErrorString(e));
      return (int)e;
    }
  }
  return mi_attention_decode(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride, page_size,
                             q_start, kv_len, B, nq, nkv, d, scale, window, n_splits, part_o, part_ml, counters,
                             stream);
}
