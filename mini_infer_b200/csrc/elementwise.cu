// Row-wise kernels of the decoder: token embedding, (residual add +) RMS norm,
// rotary position encoding fused with the key/value page write, SiLU-and-multiply; and the
// scatter of new page ids into the block tables.
//
// All arithmetic is fp32; T is the storage type of activations (float or bf16).
// The residual stream is always stored in fp32.  Each kernel accepts any width;
// widths that are a multiple of 4 with 16-byte aligned rows take the vector path.
#include "common.cuh"

MI_DEFINE_ERROR_API()

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :].  An id outside [0, V) writes NaN rows
// (the step function validates ids on the host; this keeps a fault visible).
// ---------------------------------------------------------------------------
template <typename T, int VEC>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 T* __restrict__ out, int H, int V) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  const int t = blockIdx.x;
  const int id = ids[t];
  T* dst = out + (size_t)t * H;
  if ((unsigned)id >= (unsigned)V) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = mi_from_float<T>(__int_as_float(0x7fc00000));
    return;
  }
  const T* src = table + (size_t)id * H;
  if (VEC == 4) {
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      Vec4<T> v;
      v.load(src + i);
      v.store(dst + i);
    }
  } else {
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
  }
}

extern "C" int mi_embedding(const void* table, const int* ids, void* out, int M, int H, int V,
                            int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0 || V <= 0) MI_REFUSE("embedding: bad sizes H=%d V=%d", H, V);
  const size_t es = dtype == MI_DTYPE_F32 ? 4 : 2;
  const bool vec = (H % 4 == 0) && mi_aligned(table, 16) && mi_aligned(out, 16) && ((H * es) % 16 == 0 || es == 4);
  int threads = H / 4 >= 256 ? 256 : (H / 4 >= 128 ? 128 : 64);
  if (dtype == MI_DTYPE_F32) {
    if (vec) MI_LAUNCH((embedding_kernel<float, 4>), M, threads, 0, stream, (const float*)table, ids, (float*)out, H, V);
    else MI_LAUNCH((embedding_kernel<float, 1>), M, threads, 0, stream, (const float*)table, ids, (float*)out, H, V);
  } else if (dtype == MI_DTYPE_BF16) {
    const bool vecb = vec && (H % 8 == 0);
    if (vecb) MI_LAUNCH((embedding_kernel<bf16, 4>), M, threads, 0, stream, (const bf16*)table, ids, (bf16*)out, H, V);
    else MI_LAUNCH((embedding_kernel<bf16, 1>), M, threads, 0, stream, (const bf16*)table, ids, (bf16*)out, H, V);
  } else {
    MI_REFUSE("embedding: unknown dtype %d", dtype);
  }
  MI_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Block-table updates: table[slot, index] = page for each of *count triples (slot, index,
// page) in `updates` (at most `capacity` of them; a negative slot is skipped).  A step runs
// this before its first kernel, with the pages the host has just handed out.
//
// Kernels further down the stream may read the block tables before they wait for the
// kernels ahead of them (decode attention starts its copies early), so this kernel lets its
// dependents start only when its writes are done and visible, not at its beginning as the
// other kernels do.
// ---------------------------------------------------------------------------
__global__ void table_update_kernel(int* __restrict__ table, int stride, int rows,
                                    const int* __restrict__ updates, const int* __restrict__ count,
                                    int capacity) {
  mi_pdl_wait();
  const int n = min(*count, capacity);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int slot = updates[3 * i], index = updates[3 * i + 1];
    if (slot >= 0 && slot < rows && index >= 0 && index < stride) table[(size_t)slot * stride + index] = updates[3 * i + 2];
  }
  __threadfence();
  __syncthreads();
  mi_pdl_launch_dependents();
}

extern "C" int mi_table_update(int* table, int stride, int rows, const int* updates, const int* count,
                               int capacity, cudaStream_t stream) {
  if (capacity <= 0) return 0;
  if (stride <= 0 || rows <= 0) MI_REFUSE("table_update: bad table shape %d x %d", rows, stride);
  MI_LAUNCH((table_update_kernel), 1, 256, 0, stream, table, stride, rows, updates, count, capacity);
  MI_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// (Residual add +) RMS norm.
//   r      = float(x[src]) + (res_in ? res_in[src] : 0)        src = rows ? rows[i] : i
//   res_out[i] = r                                              (if res_out)
//   out[i] = T( w * r * rsqrt(mean(r^2) + eps) )
// One block per output row.  r is kept in shared memory when the row fits,
// else it is recomputed from the inputs in the second pass (same value).
// ---------------------------------------------------------------------------
template <typename T, typename WT, int VEC>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, const float* __restrict__ res_in,
                                   float* __restrict__ res_out, const WT* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, int H,
                                   float eps, int cache_row) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ float smem[];
  float* red = smem;         // 32 floats
  float* rbuf = smem + 32;   // H floats when cache_row
  const int i = blockIdx.x;
  const int src = rows ? rows[i] : i;
  const T* xr = x + (size_t)src * H;
  const float* rr = res_in ? res_in + (size_t)src * H : nullptr;
  float* ro = res_out ? res_out + (size_t)i * H : nullptr;
  T* orow = out + (size_t)i * H;

  float ss = 0.f;
  if (VEC == 4) {
    for (int k = threadIdx.x * 4; k < H; k += blockDim.x * 4) {
      Vec4<T> xv;
      xv.load(xr + k);
      float f[4];
      xv.get(f);
      if (rr) {
        float4 rv = *reinterpret_cast<const float4*>(rr + k);
        f[0] += rv.x; f[1] += rv.y; f[2] += rv.z; f[3] += rv.w;
      }
      ss += f[0] * f[0];
      ss += f[1] * f[1];
      ss += f[2] * f[2];
      ss += f[3] * f[3];
      if (ro) *reinterpret_cast<float4*>(ro + k) = make_float4(f[0], f[1], f[2], f[3]);
      if (cache_row) *reinterpret_cast<float4*>(rbuf + k) = make_float4(f[0], f[1], f[2], f[3]);
    }
  } else {
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
      float f = mi_to_float(xr[k]);
      if (rr) f += rr[k];
      ss += f * f;
      if (ro) ro[k] = f;
      if (cache_row) rbuf[k] = f;
    }
  }
  const float total = mi_block_sum(ss, red);
  const float inv = rsqrtf(total / (float)H + eps);
  // (the block sum's __syncthreads also orders the rbuf writes before these reads)
  if (VEC == 4) {
    for (int k = threadIdx.x * 4; k < H; k += blockDim.x * 4) {
      float f[4];
      if (cache_row) {
        float4 rv = *reinterpret_cast<const float4*>(rbuf + k);
        f[0] = rv.x; f[1] = rv.y; f[2] = rv.z; f[3] = rv.w;
      } else {
        Vec4<T> xv;
        xv.load(xr + k);
        xv.get(f);
        if (rr) {
          float4 rv = *reinterpret_cast<const float4*>(rr + k);
          f[0] += rv.x; f[1] += rv.y; f[2] += rv.z; f[3] += rv.w;
        }
      }
      float o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = mi_to_float(w[k + j]) * (f[j] * inv);
      Vec4<T> ov;
      ov.set(o);
      ov.store(orow + k);
    }
  } else {
    for (int k = threadIdx.x; k < H; k += blockDim.x) {
      float f;
      if (cache_row) {
        f = rbuf[k];
      } else {
        f = mi_to_float(xr[k]);
        if (rr) f += rr[k];
      }
      orow[k] = mi_from_float<T>(mi_to_float(w[k]) * (f * inv));
    }
  }
}

template <typename T, typename WT>
static int launch_add_rmsnorm(const void* x, const float* res_in, float* res_out, const void* w,
                              void* out, const int* rows, int M, int H, float eps,
                              cudaStream_t stream) {
  const size_t es = sizeof(T);
  bool vec = (H % 4 == 0) && ((H * es) % (es == 2 ? 8 : 16) == 0) && mi_aligned(x, 16) &&
             mi_aligned(out, 16) && (!res_in || mi_aligned(res_in, 16)) &&
             (!res_out || mi_aligned(res_out, 16));
  int threads = 32;
  while (threads < 512 && threads * 8 < H) threads <<= 1;
  const size_t row_bytes = (size_t)H * sizeof(float);
  const int cache_row = row_bytes <= 160 * 1024 ? 1 : 0;
  const size_t smem = 32 * sizeof(float) + (cache_row ? row_bytes : 0);
  auto kern = vec ? add_rmsnorm_kernel<T, WT, 4> : add_rmsnorm_kernel<T, WT, 1>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  MI_LAUNCH((kern), M, threads, smem, stream, (const T*)x, res_in, res_out, (const WT*)w, (T*)out, rows, H, eps,
                                     cache_row);
  return 0;
}

// w_dtype: dtype of the gain vector (a gain stored in 32-bit stays 32-bit even when
// activations are bf16).
extern "C" int mi_add_rmsnorm(const void* x, const float* res_in, float* res_out, const void* w,
                              void* out, const int* rows, int M, int H, float eps, int dtype,
                              int w_dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0) MI_REFUSE("rmsnorm: bad width %d", H);
  int rc;
  if (dtype == MI_DTYPE_F32 && w_dtype == MI_DTYPE_F32)
    rc = launch_add_rmsnorm<float, float>(x, res_in, res_out, w, out, rows, M, H, eps, stream);
  else if (dtype == MI_DTYPE_BF16 && w_dtype == MI_DTYPE_BF16)
    rc = launch_add_rmsnorm<bf16, bf16>(x, res_in, res_out, w, out, rows, M, H, eps, stream);
  else if (dtype == MI_DTYPE_BF16 && w_dtype == MI_DTYPE_F32)
    rc = launch_add_rmsnorm<bf16, float>(x, res_in, res_out, w, out, rows, M, H, eps, stream);
  else
    MI_REFUSE("rmsnorm: unsupported dtype pair (%d, %d)", dtype, w_dtype);
  if (rc) return rc;
  MI_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Rotary position encoding of q and k (half layout: dim j pairs with j + rot/2),
// fused with the write of k and v into cache pages.
//   qkv      [M, (nq + 2 nkv) * d]   q heads, then k heads, then v heads
//   pos      [M]  absolute positions;  inv_freq [rot/2] fp32
//   slot     [M]  flat cache slot (page * page_size + offset) of each token, < 0: no write
//   kcache, vcache  [pages, nkv, page_size, d]  (may be null: rotate only); a slot's row for
//                   key/value head h lies at ((page * nkv + h) * page_size + offset) * d, with its
//                   16-byte chunks permuted by the in-page offset (mi_swizzled in common.cuh)
// q is rotated in place.  k is rotated in place too (so that a later reader of the
// buffer sees what the cache holds) and stored; v is copied.  Angles, sine and cosine
// are fp32; each output is rounded once.  rot = 0 means no rotation (store only).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_write_kernel(T* __restrict__ qkv, const int* __restrict__ pos,
                                  const float* __restrict__ inv_freq, const int* __restrict__ slot,
                                  T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv,
                                  int d, int rot, int page_size) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  // one block per (token, head); heads are q heads, then k heads, then v heads
  const int t = blockIdx.x, h = blockIdx.y;
  const int width = (nq + 2 * nkv) * d;
  T* head = qkv + (size_t)t * width + (size_t)h * d;
  const int sl = (slot && kcache) ? slot[t] : -1;
  const int half = rot >> 1;
  constexpr int EPC = 16 / (int)sizeof(T);
  const int mask = mi_swizzle_mask(d, (int)sizeof(T));
  const int page = sl >= 0 ? sl / page_size : 0, off = sl >= 0 ? sl - page * page_size : 0;
  if (h < nq + nkv) {
    const bool is_k = h >= nq;
    T* dst = nullptr;
    if (is_k && sl >= 0) dst = kcache + (((size_t)page * nkv + (h - nq)) * page_size + off) * d;
    if (half > 0) {
      const float p = (float)pos[t];
      for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(p * inv_freq[i], &s, &c);
        const float x1 = mi_to_float(head[i]);
        const float x2 = mi_to_float(head[i + half]);
        float r1, r2;
        mi_rotate(x1, x2, s, c, r1, r2);
        const T y1 = mi_from_float<T>(r1);
        const T y2 = mi_from_float<T>(r2);
        head[i] = y1;
        head[i + half] = y2;
        if (dst) {
          dst[mi_swizzled(i, off, mask, EPC)] = y1;
          dst[mi_swizzled(i + half, off, mask, EPC)] = y2;
        }
      }
    }
    if (dst)  // un-rotated tail of k (rot < d)
      for (int i = rot + threadIdx.x; i < d; i += blockDim.x) dst[mi_swizzled(i, off, mask, EPC)] = head[i];
  } else if (sl >= 0) {
    T* dst = vcache + (((size_t)page * nkv + (h - nq - nkv)) * page_size + off) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[mi_swizzled(i, off, mask, EPC)] = head[i];
  }
}

// The same work in 16-byte chunks: a block takes one token and some consecutive heads;
// sine and cosine of the token's angles are computed once per block into shared memory, then
// every thread rotates one pair of chunks (elements [j, j + E) of both halves) or copies one
// chunk of an un-rotated tail or of v.  Needs rot / 2 to be a multiple of the chunk's E
// elements; other sizes take the element-wise kernel above.
#define ROPE_HEADS 8
template <typename T>
struct Chunk16 {
  static constexpr int E = 16 / (int)sizeof(T);
  uint4 raw;
  __device__ __forceinline__ void load(const T* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[E]) const {
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < E; ++i) f[i] = mi_to_float(e[i]);
  }
  __device__ __forceinline__ void set(const float (&f)[E]) {
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < E; ++i) e[i] = mi_from_float<T>(f[i]);
  }
};

template <typename T>
__global__ void rope_write_chunks_kernel(T* __restrict__ qkv, const int* __restrict__ pos,
                                         const float* __restrict__ inv_freq, const int* __restrict__ slot,
                                         T* __restrict__ kcache, T* __restrict__ vcache, int nq, int nkv,
                                         int d, int rot, int page_size, int heads, int heads_per_block) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  extern __shared__ float rope_sc[];   // [half] sines, [half] cosines
  constexpr int E = Chunk16<T>::E;
  const int t = blockIdx.x, h0 = blockIdx.y * heads_per_block;
  const int half = rot >> 1;
  if (half > 0 && h0 < nq + nkv) {
    const float p = (float)pos[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &rope_sc[i], &rope_sc[half + i]);
  }
  __syncthreads();
  const int width = (nq + 2 * nkv) * d;
  const int sl = (slot && kcache) ? slot[t] : -1;
  const int page = sl >= 0 ? sl / page_size : 0, off = sl >= 0 ? sl - page * page_size : 0;
  const int swz = off & mi_swizzle_mask(d, (int)sizeof(T));
  const int cpr = d / E;                     // chunks per head row; also the items per head
  const int n_rot = half / E, n_tail = (d - rot) / E;
  const int n_heads = min(heads_per_block, heads - h0);
  for (int item = threadIdx.x; item < n_heads * cpr; item += blockDim.x) {
    const int h = h0 + item / cpr, j = item % cpr;
    T* head = qkv + (size_t)t * width + (size_t)h * d;
    if (h < nq + nkv) {
      T* dst = (h >= nq && sl >= 0) ? kcache + (((size_t)page * nkv + (h - nq)) * page_size + off) * d : nullptr;
      if (j < n_rot) {
        Chunk16<T> a, b;
        a.load(head + j * E);
        b.load(head + half + j * E);
        float x1[E], x2[E], y1[E], y2[E];
        a.get(x1);
        b.get(x2);
#pragma unroll
        for (int i = 0; i < E; ++i) {
          mi_rotate(x1[i], x2[i], rope_sc[j * E + i], rope_sc[half + j * E + i], y1[i], y2[i]);
        }
        a.set(y1);
        b.set(y2);
        a.store(head + j * E);
        b.store(head + half + j * E);
        if (dst) {
          a.store(dst + ((j ^ swz) * E));
          b.store(dst + (((n_rot + j) ^ swz) * E));
        }
      } else if (j < n_rot + n_tail && dst) {   // un-rotated tail of k
        const int c = 2 * n_rot + (j - n_rot);
        Chunk16<T> a;
        a.load(head + c * E);
        a.store(dst + ((c ^ swz) * E));
      }
    } else if (sl >= 0) {
      T* dst = vcache + (((size_t)page * nkv + (h - nq - nkv)) * page_size + off) * d;
      Chunk16<T> a;
      a.load(head + j * E);
      a.store(dst + ((j ^ swz) * E));
    }
  }
}

// Sines and cosines of every token's rotary angles, for kernels that rotate on their own (decode
// attention rotates its query and the new key itself): out [M, 2 half] fp32, row t = [half]
// sines then [half] cosines of pos[t] * inv_freq[i], computed as the kernels above compute them.
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ out, int half) {
  mi_pdl_enter();
  const float p = (float)pos[blockIdx.x];
  float* row = out + (size_t)blockIdx.x * 2 * half;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(p * inv_freq[i], &row[i], &row[half + i]);
}

extern "C" int mi_rope_table(const int* pos, const float* inv_freq, float* out, int M, int half, cudaStream_t stream) {
  if (M <= 0 || half <= 0) return 0;
  if (!pos || !inv_freq || !out) MI_REFUSE("rope table: positions, frequencies and the output are required");
  MI_LAUNCH((rope_table_kernel), M, half < 128 ? ((half + 31) / 32 * 32) : 128, 0, stream, pos, inv_freq, out, half);
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_rope_write(void* qkv, const int* pos, const float* inv_freq, const int* slot,
                             void* kcache, void* vcache, int M, int nq, int nkv, int d, int rot,
                             int page_size, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nq < 0 || nkv < 0 || d <= 0) MI_REFUSE("rope: bad sizes nq=%d nkv=%d d=%d", nq, nkv, d);
  if (rot < 0 || rot > d || (rot & 1)) MI_REFUSE("rope: rotary width %d must be even and <= head size %d", rot, d);
  if (rot > 0 && (!pos || !inv_freq)) MI_REFUSE("rope: positions and frequencies are required");
  if ((kcache == nullptr) != (vcache == nullptr)) MI_REFUSE("rope: key and value cache go together");
  if (kcache && page_size <= 0) MI_REFUSE("rope: bad page size %d", page_size);
  const int heads = nq + nkv + (kcache ? nkv : 0);   // v heads only matter when they are stored
  if (heads <= 0) return 0;
  if (heads > 65535) MI_REFUSE("rope: too many heads (%d)", heads);
  const int es = dtype == MI_DTYPE_F32 ? 4 : 2, epc = 16 / es;
  if ((dtype == MI_DTYPE_F32 || dtype == MI_DTYPE_BF16) && (rot / 2) % epc == 0 && d % epc == 0 &&
      mi_aligned(qkv, 16) && (!kcache || (mi_aligned(kcache, 16) && mi_aligned(vcache, 16)))) {
    // Few tokens (decode): many small blocks, the kernel is bound by latency.  Many tokens
    // (prefill): one block per token, so the angles are computed once and every thread has
    // several independent chunks in flight.
    const int hpb = M < 256 ? ROPE_HEADS : heads;
    const int threads = M < 256 ? 128 : 256;
    dim3 cgrid(M, (heads + hpb - 1) / hpb);
    const size_t smem = (size_t)rot * sizeof(float);
    if (dtype == MI_DTYPE_F32)
      MI_LAUNCH((rope_write_chunks_kernel<float>), cgrid, threads, smem, stream, (float*)qkv, pos, inv_freq, slot,
                (float*)kcache, (float*)vcache, nq, nkv, d, rot, page_size, heads, hpb);
    else
      MI_LAUNCH((rope_write_chunks_kernel<bf16>), cgrid, threads, smem, stream, (bf16*)qkv, pos, inv_freq, slot,
                (bf16*)kcache, (bf16*)vcache, nq, nkv, d, rot, page_size, heads, hpb);
    MI_RETURN_LAUNCH_STATUS();
  }
  int threads = 32;
  while (threads < 128 && threads * 2 <= d) threads <<= 1;
  dim3 grid(M, heads);
  if (dtype == MI_DTYPE_F32)
    MI_LAUNCH((rope_write_kernel<float>), grid, threads, 0, stream, (float*)qkv, pos, inv_freq, slot, (float*)kcache,
                                                           (float*)vcache, nq, nkv, d, rot, page_size);
  else if (dtype == MI_DTYPE_BF16)
    MI_LAUNCH((rope_write_kernel<bf16>), grid, threads, 0, stream, (bf16*)qkv, pos, inv_freq, slot, (bf16*)kcache,
                                                          (bf16*)vcache, nq, nkv, d, rot, page_size);
  else
    MI_REFUSE("rope: unknown dtype %d", dtype);
  MI_RETURN_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// SiLU-and-multiply: out[m, i] = silu(gu[m, i]) * gu[m, I + i], silu(g) = g / (1 + e^-g).
// ---------------------------------------------------------------------------
template <typename T, int VEC>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  const int m = blockIdx.x;
  const T* g = gu + (size_t)m * 2 * I;
  const T* u = g + I;
  T* o = out + (size_t)m * I;
  const int i0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (i0 >= I) return;
  if (VEC == 4) {
    Vec4<T> gv, uv, ov;
    gv.load(g + i0);
    uv.load(u + i0);
    float gf[4], uf[4], of[4];
    gv.get(gf);
    uv.get(uf);
#pragma unroll
    for (int j = 0; j < 4; ++j) of[j] = (gf[j] / (1.f + expf(-gf[j]))) * uf[j];
    ov.set(of);
    ov.store(o + i0);
  } else {
    const float gf = mi_to_float(g[i0]), uf = mi_to_float(u[i0]);
    o[i0] = mi_from_float<T>((gf / (1.f + expf(-gf))) * uf);
  }
}

// The same with gate and up interleaved: out[m, i] = silu(gu[m, 2 i]) * gu[m, 2 i + 1] (the
// layout of a merged gate/up projection whose rows alternate, so that a matrix product's
// epilogue finds both halves of a pair side by side).
template <typename T, int VEC>
__global__ void silu_mul_pairs_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  const int m = blockIdx.x;
  const T* in = gu + (size_t)m * 2 * I;
  T* o = out + (size_t)m * I;
  const int i0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (i0 >= I) return;
  if (VEC == 4) {
    Vec4<T> a, b, ov;
    a.load(in + 2 * i0);
    b.load(in + 2 * i0 + 4);
    float af[4], bf[4], of[4];
    a.get(af);
    b.get(bf);
    of[0] = (af[0] / (1.f + expf(-af[0]))) * af[1];
    of[1] = (af[2] / (1.f + expf(-af[2]))) * af[3];
    of[2] = (bf[0] / (1.f + expf(-bf[0]))) * bf[1];
    of[3] = (bf[2] / (1.f + expf(-bf[2]))) * bf[3];
    ov.set(of);
    ov.store(o + i0);
  } else {
    const float gf = mi_to_float(in[2 * i0]), uf = mi_to_float(in[2 * i0 + 1]);
    o[i0] = mi_from_float<T>((gf / (1.f + expf(-gf))) * uf);
  }
}

// bfloat16, eight outputs per thread: two 16-byte loads, one 16-byte store
__global__ void silu_mul_pairs8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I) {
  mi_pdl_enter();   // inputs come from the kernels before this one
  const int m = blockIdx.x;
  const int i0 = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (i0 >= I) return;
  const uint4* in = reinterpret_cast<const uint4*>(gu + (size_t)m * 2 * I + 2 * i0);
  const uint4 a = in[0], b = in[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};   // each word: (gate, up) of one output
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j]));
    const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[2 * j + 1]));
    const __nv_bfloat162 o = __floats2bfloat162_rn((p0.x / (1.f + expf(-p0.x))) * p0.y,
                                                   (p1.x / (1.f + expf(-p1.x))) * p1.y);
    r[j] = *reinterpret_cast<const uint32_t*>(&o);
  }
  *reinterpret_cast<uint4*>(out + (size_t)m * I + i0) = make_uint4(r[0], r[1], r[2], r[3]);
}

extern "C" int mi_silu_mul_pairs(const void* gu, void* out, int M, int I, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (I <= 0) MI_REFUSE("silu_mul: bad width %d", I);
  const size_t es = dtype == MI_DTYPE_F32 ? 4 : 2;
  const bool vec = (I % 4 == 0) && mi_aligned(gu, 16) && mi_aligned(out, 16);
  const int threads = 256;
  if (dtype != MI_DTYPE_F32 && dtype != MI_DTYPE_BF16) MI_REFUSE("silu_mul: unknown dtype %d", dtype);
  (void)es;
  if (vec && dtype == MI_DTYPE_BF16 && I % 8 == 0) {
    dim3 grid(M, (I / 8 + threads - 1) / threads);
    MI_LAUNCH((silu_mul_pairs8_kernel), grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
    MI_RETURN_LAUNCH_STATUS();
  }
  if (vec) {
    dim3 grid(M, (I / 4 + threads - 1) / threads);
    if (dtype == MI_DTYPE_F32) MI_LAUNCH((silu_mul_pairs_kernel<float, 4>), grid, threads, 0, stream, (const float*)gu, (float*)out, I);
    else MI_LAUNCH((silu_mul_pairs_kernel<bf16, 4>), grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
  } else {
    dim3 grid(M, (I + threads - 1) / threads);
    if (dtype == MI_DTYPE_F32) MI_LAUNCH((silu_mul_pairs_kernel<float, 1>), grid, threads, 0, stream, (const float*)gu, (float*)out, I);
    else MI_LAUNCH((silu_mul_pairs_kernel<bf16, 1>), grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
  }
  MI_RETURN_LAUNCH_STATUS();
}

extern "C" int mi_silu_mul(const void* gu, void* out, int M, int I, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (I <= 0) MI_REFUSE("silu_mul: bad width %d", I);
  const size_t es = dtype == MI_DTYPE_F32 ? 4 : 2;
  const bool vec = (I % 4 == 0) && ((I * es) % (es == 2 ? 8 : 16) == 0) && mi_aligned(gu, 16) && mi_aligned(out, 16);
  const int threads = 256;
  if (vec) {
    dim3 grid(M, (I / 4 + threads - 1) / threads);
    if (dtype == MI_DTYPE_F32) MI_LAUNCH((silu_mul_kernel<float, 4>), grid, threads, 0, stream, (const float*)gu, (float*)out, I);
    else if (dtype == MI_DTYPE_BF16) MI_LAUNCH((silu_mul_kernel<bf16, 4>), grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
    else MI_REFUSE("silu_mul: unknown dtype %d", dtype);
  } else {
    dim3 grid(M, (I + threads - 1) / threads);
    if (dtype == MI_DTYPE_F32) MI_LAUNCH((silu_mul_kernel<float, 1>), grid, threads, 0, stream, (const float*)gu, (float*)out, I);
    else if (dtype == MI_DTYPE_BF16) MI_LAUNCH((silu_mul_kernel<bf16, 1>), grid, threads, 0, stream, (const bf16*)gu, (bf16*)out, I);
    else MI_REFUSE("silu_mul: unknown dtype %d", dtype);
  }
  MI_RETURN_LAUNCH_STATUS();
}
