// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in AntoineBut/TileInfer.jl; it exists for hosts of this
// library, not for the model. ti_attention_decode() needs a 32-bit work space for the partial
// results of its key splits, which its caller allocates. Some callers cannot do that: a program
// whose own memory pool already holds every byte of the device, so that cudaMalloc fails; or code
// that runs where an allocation call is not allowed because it synchronises the device, such as the
// inner loop of a latency-bound server. For them the work space is a fixed array inside the library.
//
// What to know before using it:
//  * The array is TI_DECODE_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory per GPU; every GPU that
//    loads this library holds it until the process exits.
//  * A call needs B * nq * splits * (D + 2) floats (nothing when splits == 1). A call that needs
//    more than the array holds is refused with an error text; it never writes outside the array.
//  * The first call on a device looks up the array's device address (once per device, with that
//    device current). Make that first call before any stream capture is begun.
//  * All calls share the one array, and it keeps the previous call's contents. The kernels write
//    every element they later read, so nothing has to be cleared between calls; but two calls whose
//    kernels overlap on the GPU (different streams, no ordering between them) race on it. Keep the
//    calls of one device on one stream, or order them with events.
//  * The array that is used is the CURRENT device's (cudaGetDevice at the time of the call): make the
//    device of `stream` current before calling, or the kernels are handed another GPU's array.
//  * The per-device table of looked-up addresses is not guarded by a lock: do the first call on each
//    device from one thread before other threads use that device (later calls only read the table).
//  * A sequence whose kv_lens entry is 0 gets an output of zeros.
//  * It calls no cudaMalloc, cudaFree or any routine that allocates.
//
// Arguments and results are those of ti_attention_decode() without the two work-space pointers:
// 0 on success; 2 when the sizes are outside what the kernel takes; 1 on any other error, with
// ti_last_error() giving the text.
#pragma once
#include <cuda_runtime.h>

#define TI_DECODE_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int ti_attention_decode_noalloc(void* out, const void* q, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* seq_slots, const int* kv_lens,
                                float scale, int B, int nq, int nkv, int D, int page_size, int splits, int window,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
