// Prefill attention over the paged cache on the fifth-generation tensor cores.
//
// One block takes NTILE tiles of 128 rows (tokens x the query heads that share one key/value
// head) and walks the request's keys in chunks of 64.  As built (NTILE 1) a block has one tile
// and eight warps and two blocks share an SM, each with half of the tensor memory; with NTILE 2
// one block of sixteen warps has two tiles and loads every chunk once for both (measured
// slower: 676 against 594 us at 8192 tokens).  Per tile:
//
//   two copy warps  issue TMA copies of key and value pages into a ring of stages.  The
//            cache stores every row with its 16-byte chunks permuted by the key's in-page
//            offset, which is exactly the 128-byte-swizzle pattern of the tensor cores' shared
//            memory operands, so un-swizzled box copies of [page_size keys x 64 dims] land in
//            the canonical layout: K as a K-major operand, V as an MN-major one.
//   two issuer warps  one thread each issues the tcgen05.mma of one product: S = Q K^T (128 x 64,
//            fp32 in tensor memory, two buffers so that the next chunk's scores are computed
//            while this one's softmax runs) and O += P V (128 x d, fp32 in tensor memory; P is
//            the A operand and is read from tensor memory, where the softmax warps leave it as
//            bf16 over the first half of the chunk's score buffer).
//   four softmax warps  one row per thread: read the row of S from tensor memory, mask what
//            the row must not see, keep the running maximum and sum in registers (fp32, log2
//            domain), rescale O in tensor memory when the maximum moved, write P (bf16) back
//            into tensor memory.  They are what the kernel waits for (64 exponentials a row and
//            chunk on the special-function unit, about 1,800 cycles a chunk), so they get the
//            registers of the other warps (setmaxnreg) and the two-wide fp32 instructions.
//
// Takes head sizes 64 and 128, power-of-two page sizes from 8 to 64, any group size that
// divides 128; the mma.sync kernel of attention_mma.cu takes everything else.
// Every mbarrier wait is bounded: a wait that gives up sets a status word, the block leaves
// its loops, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

MI_DEFINE_ERROR_API()

#define ROWS 128
#define KC 64            // keys per chunk
#define SPIN_LIMIT (1 << 22)
#define LOG2E 1.4426950408889634f
#define RESCALE_LOG2 8.0f   // how far (in powers of two) a score may exceed the running reference before O is rescaled

static __device__ int g_tc_status;
// Where a give-up is reported: this library's own word above, or a word the host shares among
// its kernel libraries (mi_set_status_word) so that one small copy per step tells it about all.
static __device__ int* g_status_word;
#define MI_MAX_DEVICES 64
static int* g_status_word_host[MI_MAX_DEVICES];
__device__ __forceinline__ void report_give_up() { atomicExch(g_status_word ? g_status_word : &g_tc_status, 1); }

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
// One try: the thread sleeps in hardware until the phase completes (it is woken at once) or
// until about WAIT_HINT_NS have passed.  Without the hint a try comes back after a few hundred
// cycles and the waiting warps' polling takes issue slots from the warps that work.
#define WAIT_HINT_NS 20000u
#define WAIT_LIMIT_NS 2000000000ull   // a wait gives up after two seconds
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* give_up) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (int it = 0; it < SPIN_LIMIT; ++it) {   // bounded both in tries and in time
    if (mbar_try_wait(bar, parity)) return true;
    if (*give_up) return false;   // another role of this block gave up
    if (global_ns() - t0 > WAIT_LIMIT_NS) break;
  }
  report_give_up();
  *give_up = 1;
  return false;
}
// the same for a whole warp: every lane waits, and they leave together
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* give_up) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, give_up));
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Shared-memory operand descriptors, 128-byte swizzle, 8-row groups 1024 bytes apart.
// K-major: rows are 128 bytes of k.  MN-major: rows are 128 bytes (64 elements) of m/n, one row
// per k; `lbo` is the distance to the next 64 elements of m/n.
__device__ __forceinline__ uint64_t desc_sw128(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> fp32; b_mn: the B operand is MN-major
__device__ __forceinline__ uint32_t idesc_bf16(int m, int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(a), "l"(b), "r"(idesc), "r"(accumulate));
}
// the same with the A operand in tensor memory (row i in lane i, two 16-bit elements of k per column)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// 32 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// the same without waiting: the registers are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
      "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
      "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
      "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st32_bits(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
      "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
      "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The softmax warps are bound by the number of instructions they issue, so the row's arithmetic
// uses the two-wide fp32 instructions and the three-input maximum of this architecture.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
  uint64_t p;
  asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "f"(lo), "f"(hi));
  return p;
}
__device__ __forceinline__ void unpair(uint64_t p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {   // a * b + c on both halves
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// barriers of the block, in one array
#ifndef NTILE
#define NTILE 1    // query tiles of 128 rows per block
#endif
#define NSTAGE (NTILE == 1 ? 2 : 3)   // chunks of keys and values in flight
// Warps come in groups of four (registers move between whole groups): per tile one group of
// softmax warps and one group of copy and issuer warps.
#define TC_THREADS (256 * NTILE)
#define W_SOFT (4 * NTILE)      // the softmax warps are 0 .. W_SOFT - 1, four per tile
#define W_KCOPY (W_SOFT + 0)
#define W_QK0 (W_SOFT + 1)      // also allocates and frees the tensor memory
#define W_VCOPY (W_SOFT + 2)
#define W_PV0 (W_SOFT + 3)
#define W_QK1 (W_SOFT + 4)      // with two tiles
#define W_PV1 (W_SOFT + 5)
#define TM_COLS (256 * NTILE)   // tensor memory columns: per tile two score buffers of 64 and O of 128
#define TM_O (128 * NTILE)      // O of tile t at TM_O + 128 t
enum {
  B_KFULL = 0, B_VFULL = NSTAGE, B_KEMPTY = 2 * NSTAGE, B_VEMPTY = 3 * NSTAGE,
  B_SFULL = 4 * NSTAGE,               // [tile][2 buffers]: the scores of a chunk are in tensor memory
  B_PFULL = 4 * NSTAGE + 4,           // [tile][2 buffers]: its probabilities are (the four softmax warps arrive)
  B_PVDONE = 4 * NSTAGE + 8,          // [tile][2 buffers]: its second product has finished, the buffer is free
  B_COUNT = 4 * NSTAGE + 12
};

__global__ void __launch_bounds__(TC_THREADS, 2 / NTILE)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ table_rows,
                            int page_size, int page_shift,
                            const int* __restrict__ q_start, const int* __restrict__ q_len,
                            const int* __restrict__ kv_len, const int* __restrict__ tile_req,
                            const int* __restrict__ tile_tok0, int nq, int nkv, int d, float scale, int window,
                            int gb, int tt) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int halves = d >> 6;                       // 64-element (128-byte) column blocks of a row
  const uint32_t tile_bytes = KC * 128 * halves;   // one K or V chunk: [half][64 keys][128 B]
  const uint32_t q_bytes = ROWS * 128 * halves;    // one query tile: [half][128 rows][128 B]
  unsigned char* Qs = smem;                        // [NTILE][q tile]
  unsigned char* Ks = Qs + NTILE * q_bytes;        // [NSTAGE][tile]
  unsigned char* Vs = Ks + NSTAGE * tile_bytes;    // [NSTAGE][tile]
  __shared__ __align__(8) uint64_t bars[B_COUNT];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int give_up;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  const int hi = p_first + ntok;                   // one past the last key any row of the block sees
  const int lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int heads_here = min(gb, g - hb * gb);
  const int c0 = lo / KC, c1 = (hi + KC - 1) / KC;
  const int n_chunks = c1 - c0;
  volatile int* gu = &give_up;

  if (tid == 0) {
    for (int i = 0; i < B_COUNT; ++i)   // the softmax warps arrive one thread each
      mbar_init(&bars[i], (i >= B_PFULL && i < B_PVDONE) ? 4 : (i >= B_KEMPTY && i < B_SFULL) ? NTILE : 1);
    give_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == W_QK0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_holder)),
                 "r"(TM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // the query tiles, row R of the block = (token tok0 + R / gb, head kvh * g + hb * gb + R % gb),
  // rows 0..127 in tile 0 and 128..255 in tile 1, into the swizzled K-major layout; rows that
  // do not exist are zero
  {
    // every thread keeps one 16-byte column u and walks the rows: all of its loads are in flight
    // before the first store (d and the group size are powers of two, so the indices are shifts)
    const int ushift = d == 128 ? 4 : 3, gshift = __ffs(gb) - 1;
    const int u = tid & ((1 << ushift) - 1), r0 = tid >> ushift, rstep = TC_THREADS >> ushift;
    const int half = u >> 3, c = u & 7;
    constexpr int PASSES = NTILE * ROWS / (TC_THREADS >> 4);   // with d 128; half as many with d 64
    uint4 v[PASSES];
#pragma unroll
    for (int k = 0; k < PASSES; ++k) {
      const int R = r0 + k * rstep;
      const int tk = R >> gshift, mem = R & (gb - 1);
      v[k] = make_uint4(0u, 0u, 0u, 0u);
      if (R < NTILE * ROWS && tk < ntok && mem < heads_here)
        v[k] = *reinterpret_cast<const uint4*>(q + (size_t)(qs + tok0 + tk) * q_stride +
                                               (size_t)(kvh * g + hb * gb + mem) * d + u * 8);
    }
#pragma unroll
    for (int k = 0; k < PASSES; ++k) {
      const int R = r0 + k * rstep;
      if (R < NTILE * ROWS) {
        const int t = R / ROWS, r = R & (ROWS - 1);
        *reinterpret_cast<uint4*>(Qs + t * q_bytes + half * (ROWS * 128) + r * 128 + ((c ^ (r & 7)) << 4)) = v[k];
      }
    }
    fence_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_holder;
  // Registers: the launch gives every thread 128; the softmax warps, which hold a row of 64 scores
  // each, take 192, the copy and issuer warps keep 64 (whole groups of four warps at a time).
#define REGS_GIVE() asm volatile("setmaxnreg.dec.sync.aligned.u32 64;\n")
#define REGS_TAKE() asm volatile("setmaxnreg.inc.sync.aligned.u32 192;\n")
  // tensor memory: S of tile t, buffer sb at columns (2 t + sb) * 64, whose first 32 columns then
  // hold the chunk's probabilities as bf16 pairs (the second product reads them from there: they
  // never pass through shared memory); O of tile t at TM_O + 128 t

  if (warp == W_KCOPY || warp == W_VCOPY) {
    // The copy warps, one for keys and one for values: lane p owns page p of the chunk (its id
    // is fetched one chunk ahead, all lanes at once) and issues that page's boxes, so a chunk
    // costs one round trip to the block table, not one per page.  A key stage is free as soon
    // as its scores are computed, a value stage only after the second product: the two rings
    // run independently, each as far ahead as its own stages allow.
    REGS_GIVE();
    const bool is_v = warp == W_VCOPY;
    const int* table = block_table + (size_t)(table_rows ? table_rows[b] : b) * bt_stride;
    const int ppc = KC >> page_shift;   // pages per chunk
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    unsigned char* ring = is_v ? Vs : Ks;
    const int full0 = is_v ? B_VFULL : B_KFULL, empty0 = is_v ? B_VEMPTY : B_KEMPTY;
    auto page_of = [&](int it) -> int {
      const int key = (c0 + it) * KC + (lane << page_shift);
      return (it < n_chunks && lane < ppc && key < hi) ? table[key >> page_shift] : -1;
    };
    int page = page_of(0);
    for (int it = 0; it < n_chunks; ++it) {
      const int st = it % NSTAGE, round = it / NSTAGE;
      const int next_page = page_of(it + 1);
      if (round > 0 && !warp_wait(&bars[empty0 + st], (round - 1) & 1, gu)) break;
      // pages of the chunk that hold a key below hi (the others are never touched: their
      // scores are masked and their value rows are cleared by the softmax warps)
      const int key0 = (c0 + it) * KC;
      const int n_pages = min(ppc, (hi - key0 + page_size - 1) >> page_shift);
      if (lane == 0) mbar_expect_tx(&bars[full0 + st], (uint32_t)n_pages * page_size * 128u * halves);
      __syncwarp();
      if (lane < n_pages) {
        const int row = (page * nkv + kvh) * page_size;
        for (int h = 0; h < halves; ++h)
          tma_load_2d(ring + st * tile_bytes + h * (KC * 128) + lane * page_size * 128, map, h * 64, row,
                      &bars[full0 + st]);
      }
      page = next_page;
    }
  } else if (warp == W_QK0 || warp == W_QK1) {
    // The first product's issuers, one thread per tile: S[t][it & 1] = Q_t K^T, ahead of the
    // softmax.  One thread issues a tcgen05.mma every 60 to 120 cycles whatever its shape; a
    // thread per tile and product keeps the tensor pipe fed and lets the tiles run out of step.
    // Operand descriptors are built once; a stage, a half or a k step only adds to the address.
    REGS_GIVE();
    if (lane == 0) {
      const int t = warp == W_QK0 ? 0 : 1;
      const uint32_t idesc_qk = idesc_bf16(ROWS, KC, 0);
      const uint64_t qd = desc_sw128(smem_u32(Qs + t * q_bytes), 0), k_desc = desc_sw128(smem_u32(Ks), 0);
      for (int it = 0; it < n_chunks; ++it) {
        const int st = it % NSTAGE, round = it / NSTAGE, sb = it & 1, sround = it >> 1;
        if (!mbar_wait(&bars[B_KFULL + st], round & 1, gu)) break;
        // the score buffer also held the probabilities of chunk it - 2: free once their product is done
        if (sround > 0 && !mbar_wait(&bars[B_PVDONE + 2 * t + sb], (sround - 1) & 1, gu)) break;
        tc_fence_after();
        const uint64_t kd = k_desc + ((st * tile_bytes) >> 4);
        for (int h = 0; h < halves; ++h)
#pragma unroll
          for (int k = 0; k < 4; ++k)   // 16 of the 64 dims of a half per MMA: 32 bytes along the row
            umma(tmem + (2 * t + sb) * KC, qd + ((h * (ROWS * 128) + k * 32) >> 4),
                 kd + ((h * (KC * 128) + k * 32) >> 4), idesc_qk, (h | k) ? 1u : 0u);
        umma_commit(&bars[B_SFULL + 2 * t + sb]);
        umma_commit(&bars[B_KEMPTY + st]);   // the stage is free when both tiles' issuers have said so
      }
    }
  } else if (warp == W_PV0 || warp == W_PV1) {
    // The second product's issuers, one thread per tile: O_t += P_t V as soon as the tile's
    // probabilities are published (A operand: the probabilities in tensor memory, 8 columns for
    // 16 keys).
    REGS_GIVE();
    if (lane == 0) {
      const int t = warp == W_PV0 ? 0 : 1;
      const uint32_t idesc_pv = idesc_bf16(ROWS, d, 1);
      const uint64_t v_desc = desc_sw128(smem_u32(Vs), KC * 128);
      for (int it = 0; it < n_chunks; ++it) {
        const int st = it % NSTAGE, round = it / NSTAGE, sb = it & 1, sround = it >> 1;
        if (!mbar_wait(&bars[B_VFULL + st], round & 1, gu)) break;
        if (!mbar_wait(&bars[B_PFULL + 2 * t + sb], sround & 1, gu)) break;
        tc_fence_after();
        const uint64_t vd = v_desc + ((st * tile_bytes) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k)   // 16 keys per MMA: 8 columns of P, two 8-key groups of V
          umma_ts(tmem + TM_O + t * 128, tmem + (2 * t + sb) * KC + k * 8, vd + ((k * 2048) >> 4), idesc_pv,
                  (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(&bars[B_PVDONE + 2 * t + sb]);
        umma_commit(&bars[B_VEMPTY + st]);
      }
    }
  } else if (warp >= W_SOFT) {
    // two warps without a role: they fill the fourth group of four, which hands over its registers
    REGS_GIVE();
  } else {
    // softmax: warps 0-3 own tile 0, warps 4-7 tile 1; one thread per row (TMEM lane).  The two
    // groups run out of step with each other, so one computes exponentials while the other
    // waits for its scores or publishes its probabilities.
    REGS_TAKE();
    const int t = warp >> 2, r = tid & (ROWS - 1), R = t * ROWS + r;
    const int tk = R / gb, mem = R - tk * gb;
    const bool rvalid = tk < ntok && mem < heads_here;
    const int prow = p_first + tk;
    const int lorow = window > 0 ? max(0, prow - window + 1) : 0;
    // the tile's own range of tokens: chunks past its last row's position are skipped wholesale
    const int t_first = p_first + (t * ROWS) / gb, t_last = min(hi - 1, p_first + (t * ROWS + ROWS - 1) / gb);
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tmem_o = tmem + TM_O + t * 128;
    const float sc = scale * LOG2E;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int it = 0; it < n_chunks; ++it) {
      const int c = c0 + it, sb = it & 1, sround = it >> 1, st = it % NSTAGE, round = it / NSTAGE;
      const int key0 = c * KC;
      if (!warp_wait(&bars[B_SFULL + 2 * t + sb], sround & 1, gu)) { ok = false; break; }
      tc_fence_after();
      float s[64];
      {
        uint32_t ra[32], rb[32];
        tmem_ld32_issue(tmem + lane_addr + (2 * t + sb) * KC, ra);
        tmem_ld32_issue(tmem + lane_addr + (2 * t + sb) * KC + 32, rb);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(ra[i]);
          s[32 + i] = __uint_as_float(rb[i]);
        }
      }
      const bool interior = key0 + KC - 1 <= t_first && key0 >= (window > 0 ? max(0, t_last - window + 1) : 0) && key0 >= lo;
      if (!interior || !rvalid) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (!(rvalid && key0 + j <= prow && key0 + j >= lorow)) s[j] = -INFINITY;
      }
      // The exponents are taken relative to m_run, which follows the true running maximum
      // lazily: it moves (and O and l are rescaled) only when some row of the warp found a
      // score more than 2^RESCALE_LOG2 above it.  Probabilities may then exceed 1 by that
      // factor, which fp32 sums and bf16 products hold without loss; the result is the same
      // quotient, and rescaling O in tensor memory becomes rare instead of the rule.
      // So the exponentials need not wait for the chunk's maximum: they are computed against
      // the reference as it stands while the maximum is being found (the two streams of
      // instructions use different pipes and interleave), and only when the reference has to
      // move, or a row has none yet, are they computed again against the new one.
      const uint64_t sc2 = pair_of(sc, sc);
      uint32_t pk[32];   // the probabilities as bf16 pairs: column j of this thread's lane holds keys 2j and 2j + 1
      float sum = 0.f, mx4[4];
      const bool ahead = __all_sync(0xffffffffu, m_run != -INFINITY);
      if (ahead) {
        const uint64_t mneg2 = pair_of(-m_run, -m_run);
        uint64_t acc[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          float x0, x1;
          unpair(fma2(pair_of(s[j], s[j + 1]), sc2, mneg2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          acc[(j >> 1) & 1] = add2(acc[(j >> 1) & 1], pair_of(p0, p1));
          pk[j >> 1] = pack_bf16(p0, p1);
          mx4[j >> 4] = (j & 15) ? max3(mx4[j >> 4], s[j], s[j + 1]) : fmaxf(s[j], s[j + 1]);
        }
        float a0, a1;
        unpair(add2(acc[0], acc[1]), a0, a1);
        sum = a0 + a1;
      } else {
#pragma unroll
        for (int j = 0; j < 64; j += 2)   // four independent chains of three-input maxima
          mx4[j >> 4] = (j & 15) ? max3(mx4[j >> 4], s[j], s[j + 1]) : fmaxf(s[j], s[j + 1]);
      }
      const float mx = fmaxf(max3(mx4[0], mx4[1], mx4[2]), mx4[3]) * sc;   // sc > 0
      const bool moved = __any_sync(0xffffffffu, mx > m_run + RESCALE_LOG2);
      const float m_new = moved ? fmaxf(m_run, mx) : m_run;
      float alpha = 1.f;
      if (!ahead || moved) {   // (the same for the whole warp)
        sum = 0.f;
        if (m_new != -INFINITY) {
          alpha = fast_exp2(m_run - m_new);
          const uint64_t mneg2 = pair_of(-m_new, -m_new);
          uint64_t acc[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
#pragma unroll
          for (int j = 0; j < 64; j += 2) {
            float x0, x1;
            unpair(fma2(pair_of(s[j], s[j + 1]), sc2, mneg2), x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            acc[(j >> 1) & 1] = add2(acc[(j >> 1) & 1], pair_of(p0, p1));
            pk[j >> 1] = pack_bf16(p0, p1);
          }
          float a0, a1;
          unpair(add2(acc[0], acc[1]), a0, a1);
          sum = a0 + a1;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) pk[j] = 0u;
        }
      }
      m_run = m_new;
      l_run = l_run * alpha + sum;
      // O may be touched once the tile's previous second product has finished (the probabilities
      // go into this chunk's own score buffer, which nothing else uses until its product is done)
      if (it > 0 && moved) {
        if (!warp_wait(&bars[B_PVDONE + 2 * t + (sb ^ 1)], ((it - 1) >> 1) & 1, gu)) { ok = false; break; }
        tc_fence_after();
        for (int c32 = 0; c32 < d; c32 += 32) {
          float o32[32];
          tmem_ld32(tmem_o + lane_addr + c32, o32);
#pragma unroll
          for (int i = 0; i < 32; ++i) o32[i] *= alpha;
          tmem_st32(tmem_o + lane_addr + c32, o32);
        }
        tmem_st_wait();
      }
      // P over the first 32 columns of the chunk's score buffer
      tmem_st32_bits(tmem + lane_addr + (2 * t + sb) * KC, pk);
      tmem_st_wait();
      // value rows of keys nobody may see can hold anything (pages never written, stale rows):
      // clear them, 0 * NaN is NaN.  Only a request's first and last chunks have such rows.  Each
      // tile does it before it publishes its probabilities (the tiles' second products are
      // issued independently; both write the same zeros).
      if (key0 < lo || key0 + KC > hi) {
        if (!warp_wait(&bars[B_VFULL + st], round & 1, gu)) { ok = false; break; }
        unsigned char* vt = Vs + st * tile_bytes;
        for (int idx = r; idx < KC * halves * 8; idx += ROWS) {
          const int j = idx / (halves * 8), rest = idx - j * (halves * 8);
          if (key0 + j < lo || key0 + j >= hi)
            *reinterpret_cast<uint4*>(vt + (rest >> 3) * (KC * 128) + j * 128 + ((rest & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_async_smem();   // plain stores that the tensor core reads
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[B_PFULL + 2 * t + sb]);
    }
    // the output: O / l
    if (ok && n_chunks > 0 && warp_wait(&bars[B_PVDONE + 2 * t + ((n_chunks - 1) & 1)], ((n_chunks - 1) >> 1) & 1, gu)) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* orow = out + (size_t)(qs + tok0 + tk) * out_stride + (size_t)(kvh * g + hb * gb + mem) * d;
      for (int c32 = 0; c32 < d; c32 += 32) {
        float o32[32];
        tmem_ld32(tmem_o + lane_addr + c32, o32);   // every thread of the warp takes part in the load
        if (rvalid && l_run > 0.f) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack_bf16(o32[i] * inv, o32[i + 1] * inv);
            v.y = pack_bf16(o32[i + 2] * inv, o32[i + 3] * inv);
            v.z = pack_bf16(o32[i + 4] * inv, o32[i + 5] * inv);
            v.w = pack_bf16(o32[i + 6] * inv, o32[i + 7] * inv);
            *reinterpret_cast<uint4*>(orow + c32 + i) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == W_QK0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base_holder), "r"(TM_COLS) : "memory");
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

// A cache [rows, d] bf16 read in boxes of page_size rows x 64 elements, bytes copied as they are
// (the rows are already stored in the swizzled order).
static bool make_cache_map(CUtensorMap* map, const void* base, long long rows, int d, int page_size) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)page_size};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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
extern "C" int mi_attention_tc_status(int reset) {
  int dev = -1, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MI_MAX_DEVICES) return -1;
  int* word = g_status_word_host[dev];
  if (!word && cudaGetSymbolAddress((void**)&word, g_tc_status) != cudaSuccess) return -1;
  if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (reset && v) cudaMemset(word, 0, sizeof(int));
  return v;
}

// 1 if the kernel takes these sizes (the caller uses the mma.sync kernel otherwise)
extern "C" int mi_attention_prefill_tc_supported(int nq, int nkv, int d, int page_size) {
  if (d != 64 && d != 128) return 0;
  if (page_size < 8 || page_size > KC || (page_size & (page_size - 1))) return 0;
  if (nq <= 0 || nkv <= 0 || nq % nkv) return 0;
  const int g = nq / nkv, gb = g < ROWS ? g : ROWS;
  return ROWS % gb == 0 ? 1 : 0;
}

// Tokens per tile the kernel wants for a group of g query heads per key/value head (a block
// takes NTILE * ROWS rows).
extern "C" int mi_attention_prefill_tc_tile_tokens(int g) {
  const int gb = g < ROWS ? g : ROWS;
  return NTILE * ROWS / gb;
}

// Same arguments as mi_attention_prefill (attention_mma.cu) plus the number of pages of the
// cache; tiles are mi_attention_prefill_tc_tile_tokens(g) tokens.
extern "C" int mi_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                       const void* vcache, long long n_pages, const int* block_table, int bt_stride,
                                       const int* table_rows, int page_size, const int* q_start, const int* q_len, const int* kv_len,
                                       const int* tile_req, const int* tile_tok0, int n_tiles, int tile_tokens,
                                       int nq, int nkv, int d, float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!mi_attention_prefill_tc_supported(nq, nkv, d, page_size))
    MI_REFUSE("attention_tc: sizes not taken (heads %d/%d, head size %d, pages of %d)", nq, nkv, d, page_size);
  if (!(scale > 0.f)) MI_REFUSE("attention_tc: the score scale must be positive");
  if (window < 0) MI_REFUSE("attention_tc: bad window %d", window);
  if (!mi_aligned(q, 16) || q_stride % 8 != 0) MI_REFUSE("attention_tc: queries must be 16-byte aligned rows");
  if (!mi_aligned(out, 16) || out_stride % 8 != 0) MI_REFUSE("attention_tc: output rows must be 16-byte aligned");
  if (!mi_aligned(kcache, 128) || !mi_aligned(vcache, 128)) MI_REFUSE("attention_tc: the cache must be 128-byte aligned");
  const int g = nq / nkv, gb = g < ROWS ? g : ROWS;
  if (tile_tokens != NTILE * ROWS / gb)
    MI_REFUSE("attention_tc: tiles of %d tokens, the kernel wants %d", tile_tokens, NTILE * ROWS / gb);
  const int hblocks = (g + gb - 1) / gb;
  if (nkv * hblocks > 65535) MI_REFUSE("attention_tc: too many heads for one launch");
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap map_k, map_v;
  const long long rows = n_pages * nkv * page_size;
  if (!make_cache_map(&map_k, kcache, rows, d, page_size) || !make_cache_map(&map_v, vcache, rows, d, page_size))
    MI_REFUSE("attention_tc: the driver refused a tensor map");
  const int halves = d / 64;
  const size_t smem = (size_t)NTILE * ROWS * 128 * halves + 2 * NSTAGE * (size_t)KC * 128 * halves + 1024;
  auto kern = attention_prefill_tc_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const long long n_blocks = (long long)n_tiles * nkv * hblocks;
  if (n_blocks > 0x7fffffffLL) MI_REFUSE("attention_tc: too many blocks for one launch");
  dim3 grid((unsigned)n_blocks);
  MI_LAUNCH((kern), grid, TC_THREADS, smem, stream, map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, out_stride,
            block_table, bt_stride, table_rows, page_size, page_shift, q_start, q_len, kv_len, tile_req, tile_tok0, nq, nkv, d, scale,
            window, gb, NTILE * ROWS / gb);
  MI_RETURN_LAUNCH_STATUS();
}
