// Attention over the paged key/value cache, any portion length, CUDA cores, fp32 math.
//
// This is the kernel of the 32-bit path and the plain twin of the tensor-core
// kernels.  One block takes 16 consecutive query tokens of one request and one query
// head, walks that request's keys in chunks of 32 (always cut at absolute multiples of
// 32, so a row's arithmetic never depends on what else is in the batch), and keeps an
// online softmax in fp32.  Keys and values are fetched through the block table; a
// query at absolute position p sees keys j with  max(0, p - window + 1) <= j <= p
// (window = 0: all keys up to p).
//
// Layouts
//   q    [tokens, q_stride]   head h at columns [h*d, (h+1)*d)
//   out  [tokens, out_stride] same head layout
//   kcache, vcache [pages, nkv, page_size, d]: the page_size keys of a page lie together
//                  per key/value head; the 16-byte chunks of a row are permuted by the key's
//                  in-page offset (mi_swizzled in common.cuh)
//   block_table [rows, bt_stride] page ids; request b uses row table_rows[b] (row b when
//                  table_rows is null);  q_start / q_len / kv_len [requests]
//   tile_req / tile_tok0 [tiles]: request and first token (within the portion) of a tile
#include "common.cuh"

MI_DEFINE_ERROR_API()

#define BQ 16
#define BK 32
#define NTHREADS 128

template <typename T, int DMAX>
__global__ void __launch_bounds__(NTHREADS)
attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                         const T* __restrict__ kcache, const T* __restrict__ vcache,
                         const int* __restrict__ block_table, int bt_stride,
                         const int* __restrict__ table_rows, int page_size,
                         const int* __restrict__ q_start, const int* __restrict__ q_len,
                         const int* __restrict__ kv_len, const int* __restrict__ tile_req,
                         const int* __restrict__ tile_tok0, int nq, int nkv, int d, float scale,
                         int window) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ __align__(16) float smem[];
  float* Vs = smem;                       // [BK][d]
  float* Qs = Vs + BK * d;                // [BQ][d]
  float* Ks = Qs + BQ * d;                // [BK][d + 1]
  float* Ss = Ks + BK * (d + 1);          // [BQ][BK]
  int* rowbase = reinterpret_cast<int*>(Ss + BQ * BK);  // [BK] element offset / d of each key row, -1: none
  int* rowswz = rowbase + BK;                            // [BK] chunk permutation of each key row
  constexpr int EPC = 16 / (int)sizeof(T);
  const int swz_mask = mi_swizzle_mask(d, (int)sizeof(T));

  const int tid = threadIdx.x;
  const int tile = blockIdx.x / nq, h = blockIdx.x - tile * nq;   // all heads of a tile, then the next tile (the caller lists long tiles first)
  const int kvh = h / (nq / nkv);
  const int b = tile_req[tile], tok0 = tile_tok0[tile];
  const int ql = q_len[b], kl = kv_len[b], qs = q_start[b];
  const int trow = table_rows ? table_rows[b] : b;   // the request's row of the block table
  const int rows = min(BQ, ql - tok0);
  const int p0 = kl - ql + tok0;  // absolute position of the tile's first query
  const int j_end = p0 + rows;    // one past the last visible key
  const int j_lo = window > 0 ? max(0, p0 - window + 1) : 0;
  const int dp = d + 1;

  for (int idx = tid; idx < BQ * d; idx += NTHREADS) {
    const int r = idx / d, k = idx - r * d;
    Qs[idx] = r < rows ? mi_to_float(q[(size_t)(qs + tok0 + r) * q_stride + h * d + k]) : 0.f;
  }

  const int r = tid >> 3, c = tid & 7;
  const int prow = p0 + r;
  const int lo_r = window > 0 ? max(0, prow - window + 1) : 0;
  float m_i = -INFINITY, l_i = 0.f;
  float acc[DMAX / 8];
#pragma unroll
  for (int e = 0; e < DMAX / 8; ++e) acc[e] = 0.f;
  const int ne = d >> 3;  // d is a multiple of 16

  for (int j0 = (j_lo / BK) * BK; j0 < j_end; j0 += BK) {
    __syncthreads();  // previous chunk fully consumed (and Qs written, first time)
    if (tid < BK) {
      const int j = j0 + tid;
      int base = -1;
      if (j >= j_lo && j < j_end) {
        const int page = block_table[(size_t)trow * bt_stride + j / page_size];
        base = (page * nkv + kvh) * page_size + j % page_size;
      }
      rowbase[tid] = base;
      rowswz[tid] = (j % page_size) & swz_mask;
    }
    __syncthreads();
    const int d4 = d >> 2;
    for (int idx = tid; idx < BK * d4; idx += NTHREADS) {
      const int jj = idx / d4, k4 = (idx - jj * d4) << 2;
      const int base = rowbase[jj];
      float kf[4] = {0.f, 0.f, 0.f, 0.f}, vf[4] = {0.f, 0.f, 0.f, 0.f};
      if (base >= 0) {
        const size_t off = (size_t)base * d + ((((k4 / EPC) ^ rowswz[jj]) * EPC) + (k4 % EPC));
        Vec4<T> kv, vv;
        kv.load(kcache + off);
        vv.load(vcache + off);
        kv.get(kf);
        vv.get(vf);
      }
      float* kd = Ks + jj * dp + k4;
      kd[0] = kf[0]; kd[1] = kf[1]; kd[2] = kf[2]; kd[3] = kf[3];
      *reinterpret_cast<float4*>(Vs + jj * d + k4) = make_float4(vf[0], vf[1], vf[2], vf[3]);
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* qrow = Qs + r * d;
    for (int k = 0; k < d; ++k) {
      const float qv = qrow[k];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) s[jj] = fmaf(qv, Ks[(c + 8 * jj) * dp + k], s[jj]);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = j0 + c + 8 * jj;
      const bool ok = (r < rows) && (j <= prow) && (j >= lo_r);
      s[jj] = ok ? s[jj] * scale : -INFINITY;
      mx = fmaxf(mx, s[jj]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    const float m_new = fmaxf(m_i, mx);
    float alpha = 1.f, psum = 0.f;
    float p[4] = {0.f, 0.f, 0.f, 0.f};
    if (m_new != -INFINITY) {
      alpha = expf(m_i - m_new);  // m_i = -inf gives 0
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        p[jj] = expf(s[jj] - m_new);  // masked entries give 0
        psum += p[jj];
      }
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    psum += __shfl_xor_sync(0xffffffffu, psum, 4);
    l_i = l_i * alpha + psum;
    m_i = m_new;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) Ss[r * BK + c + 8 * jj] = p[jj];
#pragma unroll
    for (int e = 0; e < DMAX / 8; ++e) acc[e] *= alpha;
    __syncthreads();
    for (int j = 0; j < BK; ++j) {
      const float pj = Ss[r * BK + j];
      const float* vrow = Vs + j * d + c;
#pragma unroll
      for (int e = 0; e < DMAX / 8; ++e)
        if (e < ne) acc[e] = fmaf(pj, vrow[8 * e], acc[e]);
    }
  }
  if (r < rows && l_i > 0.f) {
    const float inv = 1.f / l_i;
    T* orow = out + (size_t)(qs + tok0 + r) * out_stride + h * d + c;
#pragma unroll
    for (int e = 0; e < DMAX / 8; ++e)
      if (e < ne) orow[8 * e] = mi_from_float<T>(acc[e] * inv);
  }
}

template <typename T, int DMAX>
static int launch(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                  const void* vcache, const int* block_table, int bt_stride, const int* table_rows, int page_size,
                  const int* q_start, const int* q_len, const int* kv_len, const int* tile_req,
                  const int* tile_tok0, int n_tiles, int nq, int nkv, int d, float scale, int window,
                  cudaStream_t stream) {
  const size_t smem = ((size_t)BK * d + (size_t)BQ * d + (size_t)BK * (d + 1) + BQ * BK) * sizeof(float) +
                      2 * BK * sizeof(int);
  auto kern = attention_generic_kernel<T, DMAX>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((unsigned)(n_tiles * nq));
  MI_LAUNCH((kern), grid, NTHREADS, smem, stream, (const T*)q, q_stride, (T*)out, out_stride, (const T*)kcache,
                                         (const T*)vcache, block_table, bt_stride, table_rows, page_size, q_start,
                                         q_len, kv_len, tile_req, tile_tok0, nq, nkv, d, scale, window);
  return 0;
}

extern "C" int mi_attention_generic_tile_tokens() { return BQ; }

extern "C" int mi_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                    const void* kcache, const void* vcache, const int* block_table,
                                    int bt_stride, const int* table_rows, int page_size, const int* q_start,
                                    const int* q_len, const int* kv_len, const int* tile_req,
                                    const int* tile_tok0, int n_tiles, int nq, int nkv, int d,
                                    float scale, int window, int dtype, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (d <= 0 || d % 16 != 0 || d > 256)
    MI_REFUSE("attention: head size %d is not a multiple of 16 in [16, 256]", d);
  if (nq <= 0 || nkv <= 0 || nq % nkv != 0)
    MI_REFUSE("attention: %d query heads cannot share %d key/value heads", nq, nkv);
  if ((long long)n_tiles * nq > 0x7fffffffLL) MI_REFUSE("attention: too many blocks for one launch");
  if (page_size <= 0 || window < 0) MI_REFUSE("attention: bad page size %d or window %d", page_size, window);
  if (!mi_aligned(kcache, 16) || !mi_aligned(vcache, 16)) MI_REFUSE("attention: cache must be 16-byte aligned");
  int rc;
#define MI_GO(T, DMAX)                                                                              \
  rc = launch<T, DMAX>(q, q_stride, out, out_stride, kcache, vcache, block_table, bt_stride,        \
                       table_rows, page_size, q_start, q_len, kv_len, tile_req, tile_tok0, n_tiles, nq, nkv, d, \
                       scale, window, stream)
  if (dtype == MI_DTYPE_F32) {
    if (d <= 64) MI_GO(float, 64);
    else if (d <= 128) MI_GO(float, 128);
    else MI_GO(float, 256);
  } else if (dtype == MI_DTYPE_BF16) {
    if (d <= 64) MI_GO(bf16, 64);
    else if (d <= 128) MI_GO(bf16, 128);
    else MI_GO(bf16, 256);
  } else {
    MI_REFUSE("attention: unknown dtype %d", dtype);
  }
#undef MI_GO
  if (rc) return rc;
  MI_RETURN_LAUNCH_STATUS();
}
