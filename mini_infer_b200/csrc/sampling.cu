// Next-token choice on the device, one block per logits row.
//
//   temperature == 0            greedy: the lowest index among the largest logits
//   temperature  > 0            s_i = logit_i / temperature, optionally filtered by
//       top_k  (0 = off): keep s_i >= the k-th largest s (ties kept)
//       top_p  (1 = off): among those, keep token i while the probability mass of the
//                         strictly larger tokens is <= top_p (the boundary token is kept)
//     then draw from softmax over the kept set as argmax(s_i + g_i), g_i Gumbel noise.
//
// The noise is counter-based: g_i = -log(-log(u_i)), u_i from Philox4x32-10 with the
// row's 64-bit seed as key and (i, draw index, 0, 0) as counter, so a request's draws do
// not depend on which other rows share the batch or on the order of execution.  Filters
// are found by radix selection over order-preserving 32-bit keys; probability masses are
// accumulated in 64-bit fixed point (2^-40 of the largest probability), which makes the
// selection independent of the order of atomic additions.
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define SAMPLE_THREADS 512

__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t philox_first_word(uint32_t c0, uint32_t c1, uint32_t k0, uint32_t k1) {
  uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

__device__ __forceinline__ float gumbel_noise(uint32_t i, uint32_t draw, uint32_t k0, uint32_t k1) {
  const uint32_t x = philox_first_word(i, draw, k0, k1);
  const float u = ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1), 24 bits
  return -logf(-logf(u));
}

struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  if (b.i >= 0 && (a.i < 0 || b.v > a.v || (b.v == a.v && b.i < a.i))) return b;
  return a;
}
__device__ __forceinline__ ArgBest block_best(ArgBest x, ArgBest* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  ArgBest r;
  r.v = 0.f;
  r.i = -1;
  if (lane < (blockDim.x >> 5)) r = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, y);
  }
  return r;
}

// Calls f(i, logit_i) for the elements [begin, end) of a row that this thread owns.  With
// `vec` (row start 16-byte aligned, begin a multiple of 4) elements are fetched four at a time,
// two such loads in flight per thread: a pass over a row is bound by the latency of its loads,
// not by their bytes.  Which thread sees which element does not matter to any caller (all
// reductions here are order-independent).
template <typename F>
__device__ __forceinline__ void scan_row(const float* __restrict__ lg, int begin, int end, bool vec, int tid,
                                         int nthreads, F f) {
  if (vec) {
    const int n4 = (end - begin) >> 2;
    const float4* p = reinterpret_cast<const float4*>(lg + begin);
    for (int j = tid; j < n4; j += 2 * nthreads) {
      const int j2 = j + nthreads;
      const float4 a = p[j];
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j2 < n4) b = p[j2];
      const int ia = begin + 4 * j, ib = begin + 4 * j2;
      f(ia, a.x); f(ia + 1, a.y); f(ia + 2, a.z); f(ia + 3, a.w);
      if (j2 < n4) { f(ib, b.x); f(ib + 1, b.y); f(ib + 2, b.z); f(ib + 3, b.w); }
    }
    for (int i = begin + (n4 << 2) + tid; i < end; i += nthreads) f(i, lg[i]);
  } else {
    for (int i = begin + tid; i < end; i += nthreads) f(i, lg[i]);
  }
}

// Greedy choice with a row cut across ARGMAX_SPLITS blocks: each block finds the best of its
// slice, parks it, and the block that arrives last at the row picks the best of the slices
// (lowest index among equals, as everywhere) and resets the row's counter.  The scratch is a
// file-scope array: calls on different streams of one device must not overlap.
#define ARGMAX_SPLITS 16
#define ARGMAX_MAX_ROWS 4096
static __device__ ArgBest g_argmax_part[ARGMAX_MAX_ROWS * ARGMAX_SPLITS];
static __device__ int g_argmax_count[ARGMAX_MAX_ROWS];

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_split_kernel(const float* __restrict__ logits, int ld, int V, int vec, int* __restrict__ out) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  __shared__ ArgBest best_scratch[32];
  __shared__ int is_last;
  const int row = blockIdx.y, part = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)row * ld;
  const int per = ((V + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS + 3) & ~3;   // slices begin at multiples of 4
  const int begin = min(V, part * per), end = min(V, begin + per);
  ArgBest b;
  b.v = 0.f;
  b.i = -1;
  scan_row(lg, begin, end, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
    ArgBest c;
    c.v = x;
    c.i = i;
    if (x == x) b = better(b, c);  // NaN never wins
  });
  b = block_best(b, best_scratch);
  if (tid == 0) {
    g_argmax_part[row * ARGMAX_SPLITS + part] = b;
    __threadfence();
    is_last = atomicAdd(&g_argmax_count[row], 1) == ARGMAX_SPLITS - 1;
  }
  __syncthreads();
  if (!is_last) return;
  if (tid < 32) {
    __threadfence();
    ArgBest r;
    r.v = 0.f;
    r.i = -1;
    if (tid < ARGMAX_SPLITS) {
      r.v = __ldcg(&g_argmax_part[row * ARGMAX_SPLITS + tid].v);
      r.i = __ldcg(&g_argmax_part[row * ARGMAX_SPLITS + tid].i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgBest y;
      y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
      y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
      r = better(r, y);
    }
    if (tid == 0) {
      out[row] = r.i;
      g_argmax_count[row] = 0;
    }
  }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const uint32_t* __restrict__ seed_lo, const uint32_t* __restrict__ seed_hi,
              const uint32_t* __restrict__ draw_index, int vec, int* __restrict__ out) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  __shared__ ArgBest best_scratch[32];
  __shared__ unsigned int hist_cnt[256];
  __shared__ unsigned long long hist_mass[256];
  __shared__ uint32_t sh_prefix;
  __shared__ unsigned int sh_krem;
  __shared__ unsigned long long sh_above, sh_total;
  __shared__ int sh_flag;

  const int row = blockIdx.x, tid = threadIdx.x;
  const float* lg = logits + (size_t)row * ld;
  const float T = temperature ? temperature[row] : 0.f;

  if (!(T > 0.f)) {
    ArgBest b;
    b.v = 0.f;
    b.i = -1;
    scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
      ArgBest c;
      c.v = x;
      c.i = i;
      if (x == x) b = better(b, c);  // NaN never wins
    });
    b = block_best(b, best_scratch);
    if (tid == 0) out[row] = b.i;
    return;
  }

  const int k = top_k ? top_k[row] : 0;
  const float p = top_p ? top_p[row] : 1.f;
  uint32_t kmin = 0u;

  if (k > 0 && k < V) {
    uint32_t prefix = 0u, mask = 0u;
    if (tid == 0) sh_krem = (unsigned int)k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int b = tid; b < 256; b += SAMPLE_THREADS) hist_cnt[b] = 0u;
      __syncthreads();
      scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
        const uint32_t key = order_key(x / T);
        if ((key & mask) == prefix) atomicAdd(&hist_cnt[(key >> shift) & 255u], 1u);
      });
      __syncthreads();
      if (tid == 0) {
        unsigned int rem = sh_krem, cum = 0u;
        int sel = 0;
        for (int b = 255; b >= 0; --b) {
          if (cum + hist_cnt[b] >= rem) {
            sel = b;
            break;
          }
          cum += hist_cnt[b];
        }
        sh_krem = rem - cum;
        sh_prefix = prefix | ((uint32_t)sel << shift);
      }
      __syncthreads();
      prefix = sh_prefix;
      mask |= 255u << shift;
    }
    kmin = prefix;
  }

  if (p < 1.f) {
    // largest s for a stable exponent
    float mx = -INFINITY;
    scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) { mx = fmaxf(mx, x / T); });
    mx = mi_warp_max(mx);
    __shared__ float sh_max[32];
    __syncthreads();
    if ((tid & 31) == 0) sh_max[tid >> 5] = mx;
    __syncthreads();
    mx = sh_max[0];
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w) mx = fmaxf(mx, sh_max[w]);

    uint32_t prefix = 0u, mask = 0u;
    if (tid == 0) {
      sh_above = 0ull;
      sh_total = 0ull;
      sh_flag = 0;
    }
    __syncthreads();
    // total mass of the kept set
    unsigned long long part = 0ull;
    scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
      const float s = x / T;
      if (order_key(s) >= kmin) part += __float2ull_rd(expf(s - mx) * 1099511627776.f);
    });
    atomicAdd(&sh_total, part);
    __syncthreads();
    const unsigned long long target = (unsigned long long)((double)p * (double)sh_total);
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int b = tid; b < 256; b += SAMPLE_THREADS) hist_mass[b] = 0ull;
      __syncthreads();
      scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
        const float s = x / T;
        const uint32_t key = order_key(s);
        if (key >= kmin && (key & mask) == prefix)
          atomicAdd(&hist_mass[(key >> shift) & 255u], __float2ull_rd(expf(s - mx) * 1099511627776.f));
      });
      __syncthreads();
      if (tid == 0) {
        unsigned long long above = sh_above;
        int sel = -1;
        for (int b = 255; b >= 0; --b) {
          if (above + hist_mass[b] > target) {
            sel = b;
            break;
          }
          above += hist_mass[b];
        }
        if (sel < 0) {
          sh_flag = 1;  // the whole set stays
          sel = 0;
        }
        sh_above = above;
        sh_prefix = prefix | ((uint32_t)sel << shift);
      }
      __syncthreads();
      prefix = sh_prefix;
      mask |= 255u << shift;
      if (sh_flag) break;
    }
    if (!sh_flag && prefix > kmin) kmin = prefix;
  }

  const uint32_t k0 = seed_lo[row], k1 = seed_hi[row], draw = draw_index[row];
  ArgBest b;
  b.v = 0.f;
  b.i = -1;
  scan_row(lg, 0, V, vec != 0, tid, SAMPLE_THREADS, [&](int i, float x) {
    const float s = x / T;
    if (s == s && order_key(s) >= kmin) {
      ArgBest c;
      c.v = s + gumbel_noise((uint32_t)i, draw, k0, k1);
      c.i = i;
      b = better(b, c);
    }
  });
  b = block_best(b, best_scratch);
  if (tid == 0) out[row] = b.i;
}

// Any of temperature / top_k / top_p may be null (greedy / off / off).  seed_* and
// draw_index are required when any temperature may be positive.
extern "C" int mi_sample(const float* logits, int ld, int B, int V, const float* temperature,
                         const int* top_k, const float* top_p, const uint32_t* seed_lo,
                         const uint32_t* seed_hi, const uint32_t* draw_index, int* out,
                         cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0 || ld < V) MI_REFUSE("sample: bad vocabulary %d (row stride %d)", V, ld);
  if (temperature && (!seed_lo || !seed_hi || !draw_index))
    MI_REFUSE("sample: seeds and draw indices are required with a temperature");
  const int vec = (mi_aligned(logits, 16) && ld % 4 == 0) ? 1 : 0;
  if (!temperature && B <= ARGMAX_MAX_ROWS && V >= 4096) {   // all greedy: rows cut across blocks
    MI_LAUNCH((argmax_split_kernel), dim3(ARGMAX_SPLITS, B), SAMPLE_THREADS, 0, stream, logits, ld, V, vec, out);
    MI_RETURN_LAUNCH_STATUS();
  }
  MI_LAUNCH((sample_kernel), B, SAMPLE_THREADS, 0, stream, logits, ld, V, temperature, top_k, top_p, seed_lo,
                                                  seed_hi, draw_index, vec, out);
  MI_RETURN_LAUNCH_STATUS();
}
