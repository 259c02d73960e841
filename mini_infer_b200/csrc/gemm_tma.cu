// y[M, N] = x[M, K] * W[N, K]^T for few rows of x (decode): a weight-streaming product on
// the fifth-generation tensor cores.
//
// With a handful of tokens the product is bound by reading W once, so the kernel is built
// around that stream.  The operands are swapped: 128 rows of W are the M side of the MMA and
// the tokens are its N side (16 to 128, zero-filled by the copy engine beyond M), so no tensor
// core row is wasted on padding.  One persistent block per SM:
//
//   warp 0   one thread issues TMA tile loads (W: 128 rows x 64 k, x: tokens x 64 k, both with
//            the 128-byte swizzle) into a ring of shared-memory stages; each load reports its
//            bytes to the stage's "full" mbarrier
//   warp 1   one thread issues tcgen05.mma (M 128, N tokens, K 16; four per stage) with the
//            accumulator in tensor memory; tcgen05.commit frees the stage ("empty") and, at the
//            end of a tile's k range, hands the accumulator to the epilogue
//   warps 2-5  read the accumulator (tcgen05.ld, one TMEM lane = one row of W per thread),
//            convert and store y, coalesced along N
//
// Work is cut stream-K fashion: the (tile, k chunk) units are numbered tile-major and every
// block takes an equal contiguous range, so all SMs stream the same number of bytes whatever
// N and K are.  A block whose range covers only part of a tile's k parks an fp32 partial
// tile; the block that arrives last at a tile (a counter per tile) adds the partials in block
// order and stores the result, so the sum's order is fixed and nobody waits for anybody.
//
// The weights are read with an evict-first mark (they pass once per step and are far larger than
// the L2), so that the small tensors the step's kernels hand to one another stay there.  For up to
// 16 tokens the kernel has a second instance whose epilogue also does a decoder block's additions
// and norms (EpilogueFusion below): the plain instance keeps its registers.
//
// Every mbarrier wait is bounded: a wait that gives up sets a status word, the block leaves
// its loops, frees its tensor memory and returns (the output is then wrong and the host finds
// the status set).
#include "common.cuh"

#include <cuda.h>

MI_DEFINE_ERROR_API()

#define TILE_ROWS 128   // rows of W per tile: the MMA's M
#define TILE_K 64       // k elements per stage: 128 bytes of bf16, one swizzle row
#define UMMA_K 16
#define GT_THREADS 192
#define MAX_TOKENS 128
#define SMEM_BUDGET (200 * 1024)   // ring of stages; about 100 KB per SM must be in flight to keep memory busy
#define ALIGNED_GRID_MIN_PCT 85     // use a block count that divides into the tiles if it keeps this share of the SMs
#define BOXES_PER_STAGE 2          // k boxes per stage: one box per stage leaves the issuing threads behind
#define WIDE_BOXES_PER_STAGE 4     // ... and four where they fit (see mi_gemm_tma_fused)
#define SMEM_BUDGET_WIDE (221 * 1024)
#define MAX_STAGES 12
#define SPIN_LIMIT (1 << 22)

static __device__ int g_gemm_tma_status;
// Where a give-up is reported: this library's own word above, or a word the host shares among
// its kernel libraries (mi_set_status_word) so that one small copy per step tells it about all.
static __device__ int* g_status_word;
#define MI_MAX_DEVICES 64
static int* g_status_word_host[MI_MAX_DEVICES];
__device__ __forceinline__ void report_give_up() { atomicExch(g_status_word ? g_status_word : &g_gemm_tma_status, 1); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* give_up) {
  for (int it = 0; it < SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023) == 1023 && *give_up) return false;   // another role of this block gave up
  }
  report_give_up();
  *give_up = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// The same loads with an L2 eviction policy.  Weights are read once per step and are far larger
// than the L2, so they are marked to be evicted first: what the step's kernels hand to one another
// (activations, the residual stream, partial tiles) then stays resident between them.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, "
      "%4}], [%2], %5;\n" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, "
      "%4, %5}], [%2], %6;\n" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the
// 128-byte swizzle in groups of 8 rows (1024 bytes apart).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)(1024 >> 4) << 32;              // stride between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                        // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M x N as given.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The units [u0, u1) of block c out of G, and the block that holds unit u.
__device__ __forceinline__ long long first_unit(long long total, int c, int G) { return total * c / G; }
__device__ __forceinline__ int block_of_unit(long long total, long long u, int G) {
  return (int)(((u + 1) * G - 1) / total);
}

// A block's range of units cut into segments, one per tile it touches.  In natural order the
// first and the last segment may cover only part of their tile's k range.  They are processed
// first and the whole tiles after them: the exchange of partial tiles then runs beside the
// block's remaining stream instead of at the kernel's end.
struct Segments {
  int nseg, tile_begin, kc_begin, first_len, last_len, kchunks;
  __device__ Segments(long long u0, long long u1, int kchunks_) : kchunks(kchunks_) {
    const int n_units = (int)(u1 - u0);
    tile_begin = (int)(u0 / kchunks);
    kc_begin = (int)(u0 - (long long)tile_begin * kchunks);
    first_len = min(kchunks - kc_begin, n_units);
    const int rest = n_units - first_len;
    nseg = 1 + (rest + kchunks - 1) / kchunks;
    last_len = nseg > 1 ? rest - (nseg - 2) * kchunks : first_len;
  }
  // the i-th segment to process: its natural index, tile, first k chunk and length
  __device__ __forceinline__ void get(int i, int& natural, int& tile, int& kc0, int& len) const {
    natural = i;
    if (nseg >= 3) natural = i == 0 ? 0 : (i == 1 ? nseg - 1 : i - 1);
    tile = tile_begin + natural;
    kc0 = natural == 0 ? kc_begin : 0;
    len = natural == 0 ? first_len : (natural == nseg - 1 ? last_len : kchunks);
  }
};

// What the epilogue may do beside storing the product, for a decoder block whose additions and
// norms ride on its products (at most 16 tokens).  Two halves that do not depend on each other:
//
//   stats_in   the input x was multiplied by the norm's gain but not yet divided by the root mean
//              square of its row: stats_in[t][token] are the sums of squares over 128 features
//              each, written by the product before; every accumulator of a token is scaled by
//              rsqrt(sum_t stats_in[t][token] / width + eps) before anything else happens to it
//   residual   the product is a branch's output: h = product + residual is stored back to the fp32
//              stream, y becomes h * gain[feature] (bf16, the next product's input), and
//              stats_out[tile][token] the sum of h^2 over the tile's features, added in a fixed
//              order (lanes by butterfly, then the four warps)
struct EpilogueFusion {
  const float* stats_in;
  int n_stat_tiles;
  float inv_width, eps;
  float* residual;
  const float* gain;
  float* stats_out;
};
#define FUSED_MAX_TOKENS 16

template <typename OutT, bool kFused>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tma_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                OutT* __restrict__ y, int ldy, int M, int N, int K, int n_tok, int stages, int kb, int chunked, int swiglu,
                float* __restrict__ partials, int* __restrict__ counters, const EpilogueFusion fus, int w_evict_first) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // stage s: kb W boxes [128][64] bf16 (16 KB each), then kb x boxes [n_tok][64] bf16
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t w_bytes = TILE_ROWS * TILE_K * 2, x_bytes = (uint32_t)n_tok * TILE_K * 2;
  const uint32_t stage_bytes = (w_bytes + x_bytes) * kb;
  __shared__ __align__(8) uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_full, acc_empty, inputs_ready;
  __shared__ uint32_t tmem_base_holder;
  __shared__ int give_up, is_last, epilogue_stop;
  __shared__ float row_scale[FUSED_MAX_TOKENS], square_sums[4][FUSED_MAX_TOKENS];

  // The kernel that follows in the stream may start its blocks now; it waits for this grid's
  // results itself before it touches them.
  mi_pdl_launch_dependents();

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kchunks = (K + TILE_K * kb - 1) / (TILE_K * kb);   // a unit of work: kb boxes along k
  const int n_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
  const long long total = (long long)n_tiles * kchunks;
  const int G = gridDim.x;
  const Segments segs(first_unit(total, blockIdx.x, G), first_unit(total, blockIdx.x + 1, G), kchunks);
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)n_tok) tmem_cols <<= 1;
  volatile int* gu = &give_up;

  if (warp == 0) {
    // The producer starts at once: it sets up the barriers, tells the other warps (without
    // waiting for them) and streams W.  Weights do not depend on the kernel before this one,
    // so the ring is filled with them before the wait for that kernel; x follows after it.
    if (lane == 0) {
      for (int i = 0; i < stages; ++i) {
        mbar_init(&full[i], 1);
        mbar_init(&empty[i], 1);
      }
      mbar_init(&acc_full, 1);
      mbar_init(&acc_empty, 4);
      mbar_init(&inputs_ready, 1);
      give_up = 0;
      epilogue_stop = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
      asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&map_x)) : "memory");
    }
    __syncwarp();
    asm volatile("bar.arrive 2, 192;\n" ::: "memory");
    if (lane == 0) {
      // the x boxes of unit kc (kb boxes along k), to the x part of a stage
      auto load_x = [&](unsigned char* xdst, int kc, uint64_t* bar) {
        if (chunked) {
          tma_load_3d(xdst, &map_x, 0, 0, kc * kb, bar);
        } else {
          for (int b = 0; b < kb; ++b) tma_load_2d(xdst + b * x_bytes, &map_x, (kc * kb + b) * TILE_K, 0, bar);
        }
      };
      int st = 0, round = 0, issued = 0;
      bool waited = false, ok = true;
      const uint64_t w_policy = l2_policy_evict_first();
      for (int i = 0; i < segs.nseg && ok; ++i) {
        int natural, tile, kc0, len;
        segs.get(i, natural, tile, kc0, len);
        for (int kc = kc0; kc < kc0 + len; ++kc) {
          if (!waited && issued == stages) {
            // the ring is full of weights: now the kernel before this one must be done
            mi_pdl_wait();
            if (kFused) mbar_arrive(&inputs_ready);   // the epilogue warps may read the kernels' before results
            waited = true;
            int st2 = 0, i2 = 0, kc2 = 0, nat2, tile2, kc02, len2 = 0;
            for (int n = 0; n < issued; ++n) {   // x for the stages already under way
              while (kc2 == len2) { segs.get(i2++, nat2, tile2, kc02, len2); kc2 = 0; }
              unsigned char* dst2 = smem + (size_t)st2 * stage_bytes + kb * w_bytes;
              load_x(dst2, kc02 + kc2, &full[st2]);
              ++kc2;
              ++st2;
            }
          }
          if (round > 0 && !mbar_wait(&empty[st], (round - 1) & 1, gu)) { ok = false; break; }
          unsigned char* dst = smem + (size_t)st * stage_bytes;
          mbar_expect_tx(&full[st], stage_bytes);
          if (!w_evict_first) {
            if (chunked) {
              tma_load_3d(dst, &map_w, 0, tile * TILE_ROWS, kc * kb, &full[st]);
            } else {
              for (int b = 0; b < kb; ++b)
                tma_load_2d(dst + b * w_bytes, &map_w, (kc * kb + b) * TILE_K, tile * TILE_ROWS, &full[st]);
            }
          } else if (chunked) {
            tma_load_3d_hint(dst, &map_w, 0, tile * TILE_ROWS, kc * kb, &full[st], w_policy);
          } else {
            for (int b = 0; b < kb; ++b)
              tma_load_2d_hint(dst + b * w_bytes, &map_w, (kc * kb + b) * TILE_K, tile * TILE_ROWS, &full[st], w_policy);
          }
          if (waited) load_x(dst + kb * w_bytes, kc, &full[st]);
          ++issued;
          if (++st == stages) { st = 0; ++round; }
        }
      }
      if (!waited && ok) {   // fewer units than stages: everything is under way, x still to come
        mi_pdl_wait();
        if (kFused) mbar_arrive(&inputs_ready);
        int st2 = 0, i2 = 0, kc2 = 0, nat2, tile2, kc02, len2 = 0;
        for (int n = 0; n < issued; ++n) {
          while (kc2 == len2) { segs.get(i2++, nat2, tile2, kc02, len2); kc2 = 0; }
          unsigned char* dst2 = smem + (size_t)st2 * stage_bytes + kb * w_bytes;
          load_x(dst2, kc02 + kc2, &full[st2]);
          ++kc2;
          ++st2;
        }
      }
    }
  } else {
    if (warp == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_holder)),
                   "r"(tmem_cols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    asm volatile("bar.sync 2, 192;\n" ::: "memory");   // barriers initialised (warp 0 arrived), TMEM allocated
    tc_fence_after();
  }
  const uint32_t tmem_acc = warp == 0 ? 0u : tmem_base_holder;

  if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(TILE_ROWS, n_tok);
      int st = 0, round = 0;
      bool ok = true;
      for (int i = 0; i < segs.nseg && ok; ++i) {
        int natural, tile, kc0, len;
        segs.get(i, natural, tile, kc0, len);
        if (i > 0) {   // the epilogue must have drained the previous accumulator
          if (!mbar_wait(&acc_empty, (i - 1) & 1, gu)) break;
          tc_fence_after();
        }
        for (int kc = 0; kc < len; ++kc) {
          if (!mbar_wait(&full[st], round & 1, gu)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a0 = smem_u32(smem + (size_t)st * stage_bytes), b0 = a0 + kb * w_bytes;
          for (int b = 0; b < kb; ++b) {
            const uint64_t da = umma_desc_sw128(a0 + b * w_bytes), db = umma_desc_sw128(b0 + b * x_bytes);
#pragma unroll
            for (int k = 0; k < TILE_K / UMMA_K; ++k)   // 32 bytes further along k: 2 in the address field
              umma_bf16(tmem_acc, da + 2 * k, db + 2 * k, idesc, (kc == 0 && b == 0 && k == 0) ? 0u : 1u);
          }
          umma_commit(&empty[st]);           // the stage is free once these MMAs have read it
          if (++st == stages) { st = 0; ++round; }
        }
        if (ok) umma_commit(&acc_full);      // the accumulator of this segment is complete
      }
    }
  } else if (warp >= 2) {
    // epilogue: TMEM lane quarter (warp & 3), one row of W per thread
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const int etid = (warp - 2) * 32 + lane;   // 0..127 among the epilogue threads
    // The last word on a tile's values v (16 tokens from c0, this thread's row n of W): scale, add
    // to the stream, store.  `res` holds the stream's values where fus.residual is set.
    auto store_final = [&](float (&v)[16], const float (&res)[16], float g, int c0, int tile, int n) {
      if (kFused && fus.stats_in) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= row_scale[j];
      }
      if (kFused && fus.residual) {
        float sq[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float h = 0.f;
          if (n < N && c0 + j < M) {
            h = v[j] + res[j];
            fus.residual[(size_t)(c0 + j) * N + n] = h;
            y[(size_t)(c0 + j) * ldy + n] = mi_from_float<OutT>(h * g);
          }
          sq[j] = h * h;
        }
        // Sixteen sums over the warp's 32 rows in 16 shuffles: at every step a lane passes on the
        // half of its values that its partner keeps, so lane l ends with the sum of token (l >> 1) & 15.
#pragma unroll
        for (int half = 8, off = 16; half >= 1; half >>= 1, off >>= 1) {
          const bool upper = (lane & off) != 0;
#pragma unroll
          for (int j = 0; j < half; ++j) {
            const float give = upper ? sq[j] : sq[j + half];
            const float keep = upper ? sq[j + half] : sq[j];
            sq[j] = keep + __shfl_xor_sync(0xffffffffu, give, off);
          }
        }
        sq[0] += __shfl_xor_sync(0xffffffffu, sq[0], 1);
        if (!(lane & 1)) square_sums[quarter][(lane >> 1) & 15] = sq[0];
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (etid < FUSED_MAX_TOKENS)
          fus.stats_out[tile * FUSED_MAX_TOKENS + etid] =
              (square_sums[0][etid] + square_sums[1][etid]) + (square_sums[2][etid] + square_sums[3][etid]);
        asm volatile("bar.sync 1, 128;\n" ::: "memory");   // the sums are read before the next tile writes them
      } else if (swiglu) {
        // rows alternate gate, up: the even lane of a pair has the gate, its neighbour the up
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          if (!(row & 1) && n < N && c0 + j < M)
            y[(size_t)(c0 + j) * ldy + (n >> 1)] = mi_from_float<OutT>((v[j] / (1.f + expf(-v[j]))) * other);
        }
      } else if (n < N) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < M) y[(size_t)(c0 + j) * ldy + n] = mi_from_float<OutT>(v[j]);
      }
    };
    auto load_stream = [&](float (&res)[16], int c0, int n) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        res[j] = (kFused && fus.residual && n < N && c0 + j < M) ? __ldcg(fus.residual + (size_t)(c0 + j) * N + n) : 0.f;
    };
    for (int i = 0; i < segs.nseg; ++i) {
      int natural, tile, kc0, len;
      segs.get(i, natural, tile, kc0, len);
      const bool whole = (len == kchunks);
      const int n = tile * TILE_ROWS + row;
      // who shares this tile (worked out while the MMAs still run: the divisions are slow)
      const long long t0 = (long long)tile * kchunks;
      int c_first = 0, c_last = 0, first_slot = 0;
      if (!whole) {
        c_first = block_of_unit(total, t0, G);
        c_last = block_of_unit(total, t0 + kchunks - 1, G);
        // Every block after the tile's first one begins inside the tile, so the tile is its
        // first segment (slot 0); the first block's is slot 0 only if it begins with the tile.
        first_slot = c_first * 2 + (first_unit(total, c_first, G) == t0 ? 0 : 1);
      }
      float stream_vals[16] = {};
      const float gain_n = (kFused && fus.residual && n < N) ? __ldg(fus.gain + n) : 0.f;   // needed last, asked for first
      if (kFused && i == 0) {
        // What the kernels before this one wrote may be read once the copy thread's wait for them is
        // over: it says so through a barrier of the block, which orders these warps' loads behind it
        // (measured: no faster and no slower than every warp waiting for the grids itself).
        // (a wait that gives up here makes the wait for the accumulator below give up as well)
        const bool ready = mbar_wait(&inputs_ready, 0, gu);
        if (fus.stats_in && ready && etid < FUSED_MAX_TOKENS) {
          // every token's scale from the sums the product before left, tile by tile
          float sum = 0.f;
          for (int t = 0; t < fus.n_stat_tiles; ++t) sum += __ldcg(fus.stats_in + t * FUSED_MAX_TOKENS + etid);
          row_scale[etid] = rsqrtf(sum * fus.inv_width + fus.eps);
        }
        // row_scale is read after the barrier that follows the wait for the accumulator
      }
      if (kFused && whole) load_stream(stream_vals, 0, n);   // asked for while the MMAs still run
      // the four warps leave together or not at all (they meet at named barriers below)
      if (!mbar_wait(&acc_full, i & 1, gu)) epilogue_stop = 1;
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (epilogue_stop) break;
      tc_fence_after();
      // partial tiles of this block: slot 0 for its first segment (natural order), 1 for its last
      const int slot = blockIdx.x * 2 + (natural == 0 ? 0 : 1);
      float* part = partials + (size_t)slot * n_tok * TILE_ROWS;
      for (int c0 = 0; c0 < n_tok; c0 += 16) {
        float v[16];
        tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        if (whole) {
          store_final(v, stream_vals, gain_n, c0, tile, n);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < M) part[(size_t)(c0 + j) * TILE_ROWS + row] = v[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty);
      if (!whole) {
        // count this block in; the last one to arrive adds the partial tiles in block order
        __threadfence();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (etid == 0) is_last = (atomicAdd(&counters[tile], 1) == c_last - c_first) ? 1 : 0;
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (is_last) {
          __threadfence();
          {
            // sixteen tokens and four blocks' partial tiles at a time: 64 independent loads are in
            // flight per thread; the additions still run in block order
            for (int j0 = 0; j0 < M; j0 += 16) {
              float acc[16];
              if (kFused) load_stream(stream_vals, j0, n);   // in flight beside the partial tiles
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = 0.f;
              for (int cb = c_first; cb <= c_last; cb += 4) {
                float v[4][16];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                  const int c = cb + cc;
                  const int s = c == c_first ? first_slot : c * 2;
                  const float* p = partials + ((size_t)s * n_tok + j0) * TILE_ROWS + row;
#pragma unroll
                  for (int j = 0; j < 16; ++j)   // only rows below M were written
                    v[cc][j] = (c <= c_last && j0 + j < M && n < N) ? __ldcg(p + (size_t)j * TILE_ROWS) : 0.f;
                }
#pragma unroll
                for (int cc = 0; cc < 4; ++cc)
#pragma unroll
                  for (int j = 0; j < 16; ++j) acc[j] += v[cc][j];
              }
              store_final(acc, stream_vals, gain_n, j0, tile, n);
            }
          }
          if (etid == 0) counters[tile] = 0;   // ready for the next call
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");   // is_last is read before it is written again
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_holder), "r"(tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// A [rows, cols] bf16 matrix with `ld` elements between rows, read in boxes of box_rows x 64
// with the 128-byte swizzle; out-of-range elements read as zero.
// The same matrix seen as [cols / 64 chunks][rows][64] (cols a multiple of 64): one copy then
// brings `chunks` consecutive boxes, laid out one after the other.
static bool make_map_chunked(CUtensorMap* map, const void* base, int rows, int cols, long long ld, int box_rows,
                             int chunks) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {TILE_K, (cuuint64_t)rows, (cuuint64_t)(cols / TILE_K)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, TILE_K * 2};
  cuuint32_t box[3] = {TILE_K, (cuuint32_t)box_rows, (cuuint32_t)chunks};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Report give-ups of this library's kernels on the current device into `device_word` (an int in
// device memory that the caller owns and keeps alive; null: back to the library's own word).
extern "C" int mi_set_status_word(int* device_word) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MI_MAX_DEVICES) MI_REFUSE("status word: bad device");
  cudaError_t e = cudaMemcpyToSymbol(g_status_word, &device_word, sizeof(int*));
  if (e != cudaSuccess) return (int)e;
  g_status_word_host[dev] = device_word;
  return 0;
}

// Non-zero when a block gave up a bounded wait since the last reset (synchronises the device).
extern "C" int mi_gemm_tma_status(int reset) {
  int dev = -1, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MI_MAX_DEVICES) return -1;
  int* word = g_status_word_host[dev];
  if (!word && cudaGetSymbolAddress((void**)&word, g_gemm_tma_status) != cudaSuccess) return -1;
  if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v) cudaMemset(word, 0, sizeof(int));
  return v;
}

// floats of `partials` and ints of `counters` a call with these sizes needs
extern "C" int mi_gemm_tma_workspace(int M, int N, int blocks, long long* partial_floats, int* counter_ints) {
  const int n_tok = ((M < 1 ? 1 : M) + 15) / 16 * 16;
  *partial_floats = (long long)blocks * 2 * n_tok * TILE_ROWS;
  *counter_ints = (N + TILE_ROWS - 1) / TILE_ROWS;
  return 0;
}

// x [M, K] bf16 (row stride ldx), w [N, K] bf16 contiguous, y [M, N] (row stride ldy) bf16 or
// fp32.  With `swiglu` the rows of w alternate gate, up and y is [M, N / 2]:
// y[m, i] = silu(x w[2i]) * (x w[2i+1]), computed on the fp32 accumulators.  `blocks` is the number of persistent blocks (the number of SMs); `partials` and
// `counters` (zero before the first call; the kernel leaves them zero) as mi_gemm_tma_workspace
// says.
//
// The fused forms (at most 16 rows of x), see EpilogueFusion: with `stats_in` ([stat_tiles][16] sums
// of squares, `width` features in all) every row of the product is scaled by
// rsqrt(sum / width + eps) first; with `residual` ([M, N] fp32, updated in place) the product is
// added to it, y = (product + residual) * gain[n], and `stats_out` ([ceil(N / 128)][16]) receives
// the sums of squares of the new residual per 128 features.  Null pointers switch a half off.
extern "C" int mi_gemm_tma_fused(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N,
                                 int K, int out_dtype, int swiglu, int blocks, float* partials, int* counters,
                                 const float* stats_in, int stat_tiles, int width, float eps, float* residual,
                                 const float* gain, float* stats_out, cudaStream_t stream) {
  EpilogueFusion fus = {stats_in, stat_tiles, width > 0 ? 1.f / (float)width : 0.f, eps, residual, gain, stats_out};
  if (stats_in || residual) {
    if (M > FUSED_MAX_TOKENS)
      MI_REFUSE("gemm_tma: the fused epilogues take at most %d rows of x, got %d", FUSED_MAX_TOKENS, M);
    if (stats_in && (stat_tiles <= 0 || width <= 0))
      MI_REFUSE("gemm_tma: row statistics need their tile count and width (%d, %d)", stat_tiles, width);
    if (residual && (!gain || !stats_out || swiglu))
      MI_REFUSE("gemm_tma: the residual epilogue needs a gain and room for its statistics, and no gate/up pairs");
    if (residual && !mi_aligned(residual, 4)) MI_REFUSE("gemm_tma: misaligned residual stream");
  }
  if (swiglu && (N % 2)) MI_REFUSE("gemm_tma: the gate/up epilogue needs an even number of rows of W, got %d", N);
  if (M <= 0 || N <= 0) return 0;
  if (M > MAX_TOKENS) MI_REFUSE("gemm_tma: %d rows of x; this kernel takes at most %d", M, MAX_TOKENS);
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0)
    MI_REFUSE("gemm_tma: K (%d) and the row stride of x (%lld) must be multiples of 8 (16-byte rows)", K, ldx);
  if (!mi_aligned(x, 16) || !mi_aligned(w, 16)) MI_REFUSE("gemm_tma: operands must be 16-byte aligned");
  if (blocks <= 0) MI_REFUSE("gemm_tma: bad block count %d", blocks);
  if (out_dtype != MI_DTYPE_BF16 && out_dtype != MI_DTYPE_F32) MI_REFUSE("gemm_tma: unknown output dtype %d", out_dtype);
  const int n_tok = (M + 15) / 16 * 16;
  // Four boxes along k per stage where three such stages fit (up to 16 tokens) and K is a whole
  // number of them: every row of W then contributes 512 contiguous bytes to a copy instead of 256
  // (inside a captured decode step of Llama 3.1 8B sizes: 3.762 -> 3.733 ms; three boxes: 3.736).
  int kb = BOXES_PER_STAGE;
  int budget = SMEM_BUDGET;
  if (K >= 2048 && K % (TILE_K * WIDE_BOXES_PER_STAGE) == 0 &&
      (TILE_ROWS * TILE_K * 2 + n_tok * TILE_K * 2) * WIDE_BOXES_PER_STAGE * 3 <= SMEM_BUDGET_WIDE) {
    kb = WIDE_BOXES_PER_STAGE;
    budget = SMEM_BUDGET_WIDE;
  }
  const long long total = (long long)((N + TILE_ROWS - 1) / TILE_ROWS) * ((K + TILE_K * kb - 1) / (TILE_K * kb));
  int grid = (int)(total < blocks ? total : blocks);
  {
    // With fewer tiles than blocks, a block count that is a multiple of the tile count gives every
    // block one stretch of one tile (one partial tile to exchange instead of two for the blocks
    // that would straddle a tile boundary), at the price of leaving a few SMs idle.
    const int n_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
    if (n_tiles < blocks && total >= blocks) {
      const int aligned = n_tiles * (blocks / n_tiles);
      if (aligned * 100 >= blocks * ALIGNED_GRID_MIN_PCT) grid = aligned;
    }
  }
  const int stage_bytes = (TILE_ROWS * TILE_K * 2 + n_tok * TILE_K * 2) * kb;
  int stages = budget / stage_bytes;
  if (stages < 2) stages = 2;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  const size_t smem = (size_t)stages * stage_bytes + 1024;
  CUtensorMap map_w, map_x;
  const int chunked = (K % TILE_K == 0 && kb > 1) ? 1 : 0;   // else the k tail needs the 2-D view's zero fill
  const bool maps_ok = chunked ? (make_map_chunked(&map_w, w, N, K, K, TILE_ROWS, kb) &&
                                  make_map_chunked(&map_x, x, M, K, ldx, n_tok, kb))
                               : (make_map(&map_w, w, N, K, K, TILE_ROWS) && make_map(&map_x, x, M, K, ldx, n_tok));
  if (!maps_ok)
    MI_REFUSE("gemm_tma: the driver refused a tensor map (N %d, K %d, M %d)", N, K, M);
  cudaError_t e;
#define GT_LAUNCH(T, FUSED)                                                                                        \
  {                                                                                                                \
    auto kern = gemm_tma_kernel<T, FUSED>;                                                                         \
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                        \
    if (e != cudaSuccess) return (int)e;                                                                           \
    MI_LAUNCH((kern), grid, GT_THREADS, smem, stream, map_w, map_x, (T*)y, (int)ldy, M, N, K, n_tok, stages, kb,   \
              chunked, swiglu ? 1 : 0, partials, counters, fus, w_evict_first);                                                   \
  }
  const bool fused = stats_in || residual;
  const int w_evict_first = mi_l2_hints_enabled() ? 1 : 0;
  if (out_dtype == MI_DTYPE_BF16) {
    if (fused) GT_LAUNCH(bf16, true) else GT_LAUNCH(bf16, false)
  } else {
    if (fused) GT_LAUNCH(float, true) else GT_LAUNCH(float, false)
  }
#undef GT_LAUNCH
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_gemm_tma(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
                           int out_dtype, int swiglu, int blocks, float* partials, int* counters, cudaStream_t stream) {
  return mi_gemm_tma_fused(x, ldx, w, y, ldy, M, N, K, out_dtype, swiglu, blocks, partials, counters, nullptr, 0, 0,
                           0.f, nullptr, nullptr, nullptr, stream);
}
