// Shared helpers of the kernel libraries.
//
// Every library is a plain shared object with `extern "C"` entry points that take
// device pointers, sizes and a CUDA stream, launch on that stream and return a
// status: 0 = launched, > 0 = a cudaError_t, < 0 = the arguments were refused
// (the reason is then available from mi_error_message()).  Nothing here allocates
// device memory and nothing synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define MI_DTYPE_F32 0
#define MI_DTYPE_BF16 1

#define MI_REFUSED (-1)

#define MI_DEFINE_ERROR_API()                                              \
  static thread_local char g_mi_error[512] = "";                           \
  extern "C" const char* mi_error_message() { return g_mi_error; }

#define MI_REFUSE(...)                                                     \
  do {                                                                     \
    snprintf(g_mi_error, sizeof(g_mi_error), __VA_ARGS__);                 \
    return MI_REFUSED;                                                     \
  } while (0)

#define MI_RETURN_LAUNCH_STATUS()                                          \
  do {                                                                     \
    cudaError_t e__ = cudaGetLastError();                                  \
    if (e__ != cudaSuccess) {                                              \
      snprintf(g_mi_error, sizeof(g_mi_error), "CUDA: %s",                 \
               cudaGetErrorString(e__));                                   \
      return (int)e__;                                                     \
    }                                                                      \
    return 0;                                                              \
  } while (0)

typedef __nv_bfloat16 bf16;

// ---- programmatic dependent launch
//
// Every kernel of the engine is launched with programmatic stream serialization (MI_LAUNCH):
// its blocks may be scheduled while the kernel before it in the stream still runs, which hides
// the launch latency and lets a kernel do work that does not depend on its predecessors (set
// up barriers, stream weights into shared memory) ahead of time.  The contract: a kernel calls
// mi_pdl_wait() before it reads or writes anything that an earlier kernel may write or read;
// before that it touches only immutable data (weights) and its own shared or tensor memory.
// mi_pdl_launch_dependents() lets the next kernel's blocks be scheduled; it is called first
// thing, so the look-ahead is limited only by what fits on the SMs.  Kernels launched by
// other libraries take part as ordinary stream work: they start after everything before them
// has finished, and a kernel after them waits for all of them.
__device__ __forceinline__ void mi_pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
__device__ __forceinline__ void mi_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
// for kernels with nothing to do before their inputs are ready
__device__ __forceinline__ void mi_pdl_enter() {
  mi_pdl_launch_dependents();
  mi_pdl_wait();
}

#ifdef __CUDACC__
#include <stdlib.h>
// MINI_INFER_L2_HINTS=0 in the environment leaves out the evict-first marks on data that a step
// reads once (the weights of the streaming product, the keys and values of decode attention).
static inline bool mi_l2_hints_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("MINI_INFER_L2_HINTS");
    enabled = (e && e[0] == '0' && e[1] == 0) ? 0 : 1;
  }
  return enabled != 0;
}
// MINI_INFER_PDL=0 in the environment launches kernels the ordinary way (for comparisons).
static inline bool mi_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("MINI_INFER_PDL");
    enabled = (e && e[0] == '0') ? 0 : 1;
  }
  return enabled != 0;
}
template <typename... KArgs, typename... Args>
static inline cudaError_t mi_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = mi_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}
#define MI_LAUNCH(kernel, grid, block, smem, stream, ...) \
  mi_launch(kernel, dim3(grid), dim3(block), (size_t)(smem), stream, __VA_ARGS__)
#endif

__device__ __forceinline__ float mi_to_float(float x) { return x; }
__device__ __forceinline__ float mi_to_float(bf16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T mi_from_float(float x);
template <>
__device__ __forceinline__ float mi_from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ bf16 mi_from_float<bf16>(float x) { return __float2bfloat16_rn(x); }

// Four consecutive elements, loaded/stored as one access where T allows.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  float4 v;
  __device__ __forceinline__ void load(const float* p) { v = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ void get(float (&f)[4]) const { f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ __forceinline__ void set(const float (&f)[4]) { v = make_float4(f[0], f[1], f[2], f[3]); }
};
template <>
struct Vec4<bf16> {
  uint2 v;
  __device__ __forceinline__ void load(const bf16* p) { v = *reinterpret_cast<const uint2*>(p); }
  __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint2*>(p) = v; }
  __device__ __forceinline__ void get(float (&f)[4]) const {
    __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    f[0] = fa.x; f[1] = fa.y; f[2] = fb.x; f[3] = fb.y;
  }
  __device__ __forceinline__ void set(const float (&f)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f[2], f[3]);
    v.x = *reinterpret_cast<uint32_t*>(&a);
    v.y = *reinterpret_cast<uint32_t*>(&b);
  }
};

__device__ __forceinline__ float mi_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float mi_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; `scratch` holds 32 floats.  Every thread gets the result.
// The order of additions depends only on blockDim, never on the data.
__device__ __forceinline__ float mi_block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = mi_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = mi_warp_sum(t);
  return t;
}

// Cache rows are stored with their 16-byte chunks permuted: chunk c of the row of the token at
// in-page offset t sits at chunk position c ^ (t & mask).  A linear copy of a page into shared
// memory then lands in a layout whose 8-row ldmatrix reads touch all banks.  mask depends on
// the row size only: chunks per row n = d * elem_size / 16; mask = min(n, 8) - 1 when n is a
// power of two, else 0 (no permutation).
__host__ __device__ inline int mi_swizzle_mask(int d, int elem_size) {
  const int n = d * elem_size / 16;
  if (n < 2 || (n & (n - 1))) return 0;
  return (n < 8 ? n : 8) - 1;
}
// Physical element index within a row of logical element k (epc = elements per 16-byte chunk).
__device__ __forceinline__ int mi_swizzled(int k, int t, int mask, int epc) {
  return (((k / epc) ^ (t & mask)) * epc) + (k % epc);
}

// One rotation of the rotary encoding in fp32, every operation rounded on its own (never
// contracted into a fused multiply-add), so that every kernel that rotates gives the same bits:
// (y1, y2) = (x1 c - x2 s, x2 c + x1 s).
__device__ __forceinline__ void mi_rotate(float x1, float x2, float s, float c, float& y1, float& y2) {
  y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
  y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

static inline bool mi_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
