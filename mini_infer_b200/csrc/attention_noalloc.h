// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project.  It exists for hosts that
// hand a kernel library its inputs and outputs and nothing else: a serving process that pins
// its whole memory budget at start-up and treats any later cudaMalloc as a fault (an
// allocation can synchronise the device, fragment the pool or simply fail under load), or a
// plug-in running on a thread that is not allowed to touch the allocator.  The regular entry
// point, mi_attention_decode, asks its caller for scratch memory when the keys are cut into
// several slices; this one brings its own.
//
// The scratch is one file-scope `static __device__` array of
// MI_ATTENTION_NOALLOC_MAX_FLOATS floats (4 MiB).  Every GPU on which the library is loaded
// holds that array until the process exits.  A call needs B * nq * n_splits * (d + 2) floats
// of it plus one arrival counter per (request, key/value head, group of 8 query heads), the
// counters rounded up to a multiple of four so that everything behind them stays aligned, and
// is refused, with a message, when that is more than the array holds.
//
// What a caller has to know:
//   * The first call on a device looks up the array's device address (with that device
//     current) and remembers it.  Make that first call during set-up, before any stream
//     capture is begun.
//   * All calls share the one array and it keeps the previous call's contents.  Only the
//     arrival counters have to start at zero, and the entry point clears them on the stream
//     before it launches; every other slot a call reads it has written earlier in the same call.
//     Two calls that overlap on the GPU (different streams, or concurrent replays) race on it;
//     keep calls on one stream or serialise them yourself.
//   * No cudaMalloc, cudaFree or allocating library routine is called.  Inputs and outputs are
//     the caller's, exactly as for mi_attention_decode.
#pragma once

#include <cuda_runtime.h>

#define MI_ATTENTION_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and status codes as mi_attention_decode, without the two scratch pointers.
int mi_attention_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* kcache,
                                const void* vcache, const int* block_table, int bt_stride, int page_size,
                                const int* q_start, const int* kv_len, int B, int nq, int nkv, int d,
                                float scale, int window, int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
