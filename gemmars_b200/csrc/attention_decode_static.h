// gb_attention_decode_static: decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for hosts of this
// library that may not call cudaMalloc themselves or let a library do it for them: code that
// runs inside someone else's memory plan, such as a serving process that handed all device
// memory to its own pool at start-up, or a plug-in loaded into such a process, where a
// cudaMalloc would fail or break the host's accounting.  Such callers own q, out, the cache and
// the index arrays already; what they lack is the scratch buffer that gb_attention_decode wants
// when the keys are split over several CTAs ("shares" > 1).
//
// Here that scratch is a fixed array in the library's own device data segment,
// GB_ATTENTION_DECODE_STATIC_FLOATS float32 values (4 MiB).  The array belongs to one built
// library: attention_decode is built once per head size (and once more for the variant whose
// kernels start under their predecessor), and each of those builds that a process loads carries
// an array of its own.  Every GPU on which such a build is loaded holds its 4 MiB from the
// moment the build's module is loaded there until the process ends, whether or not this
// function is ever called.
//
// Arguments and result are those of gb_attention_decode (attention_decode.cu) without the
// scratch pointer.  The library is built for one head size; `hd` must be that size.
//
//  * Limit: ntok * nh * shares * (hd + 2) must not exceed GB_ATTENTION_DECODE_STATIC_FLOATS when
//    shares > 1, else GB_ERR_STATIC_SCRATCH (-5) is returned and nothing is launched.  With
//    hd = 128 that is, for instance, 64 tokens x 32 heads x 3 shares, or 8 tokens x 32 heads x 31.
//  * It calls no cudaMalloc, cudaFree or other allocating routine, and launches on `stream`.
//  * The first call with shares > 1 on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it; make that first call
//    before any stream capture begins.  A call with shares == 1 needs no scratch and looks
//    nothing up.
//  * All calls on a device share the one array and it keeps what the last call left.  Nothing in
//    it needs clearing between calls, but two calls whose kernels may run at the same time
//    (different streams without an ordering between them) race on it: order them.
#pragma once

#include <cuda_runtime.h>

#define GB_ATTENTION_DECODE_STATIC_FLOATS (1u << 20)
#define GB_ERR_STATIC_SCRATCH (-5)

#ifdef __cplusplus
extern "C" {
#endif
int gb_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                          const void* kcache, const void* vcache, const int* page_table,
                                          int table_width, int page_size, int nkv, int hd, const int* tok_pos,
                                          const int* tok_seq, const int* seq_slot, int ntok, int nh, int window,
                                          int shares, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
