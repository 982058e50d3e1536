// Split decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which has no native code
// and lets PyTorch allocate whatever its attention needs).
//
// Who needs it: a host that gave this library no allocator.  Examples are a serving
// process that carved up all device memory at start-up and treats a later
// cudaMalloc as a bug (it can fail, or stall the device while the driver maps
// memory); a plug-in living inside another runtime's memory pool; a control loop
// with a latency bound that an allocator call would break.  The ordinary entry
// point, ss_attn_decode_mma, takes its scratch memory (the partial results of the
// key slices) from the caller, who usually gets it from an allocator.  This variant
// instead keeps that scratch in a fixed array inside the library.
//
// What it does: the same attention as ss_attn_decode_mma for the same arguments; the
// inputs and the output are still the caller's.  The slices always meet in the scratch
// array and the block that finishes a group of heads last adds them up in slice order.
// ss_attn_decode_mma takes that route only for more than 8 slices (with 2 to 8 it
// combines them inside a thread-block cluster, a different order of additions), so the
// two agree bit for bit above 8 slices and to rounding below.  It calls no cudaMalloc,
// cudaFree or any allocating library routine.
//
// Limits and rules:
//  * n_slices is at most SS_NOALLOC_MAX_SLICES (64); more is refused with
//    SS_NOALLOC_BAD_ARGUMENT before anything is launched.
//  * One GPU per call: the device that is current when the call is made.  Every device
//    has its own copy of the array, and the per-device set-up (the array's address, the
//    kernel's shared-memory opt-in) happens at the first call on that device.  First
//    calls on one device from two host threads at once must not overlap.
//  * The scratch array holds SS_NOALLOC_SCRATCH_FLOATS floats (8 MiB) per GPU, from
//    the moment the library is loaded on that GPU until the process exits.  A call
//    needs n_requests * n_q * n_slices * (HEAD_DIM + 1) floats; a call that needs
//    more is refused with SS_NOALLOC_TOO_LARGE and launches nothing.
//  * The first call on each device looks up the array's device address (with that
//    device current).  Make that first call during set-up, before any stream capture.
//  * Beside the floats there are SS_NOALLOC_COUNTERS small counters (one per request and
//    block of 16 heads of a kv group); a call with more of those is refused the same way.
//  * All calls share the one array, and it keeps what the last call left in it.
//    Nothing in the float part has to start at zero: every slice of every head writes its
//    whole partial result before the merge reads it.  The counters must be zero between
//    calls; the kernel itself puts them back to zero (the last slice to finish does it).  Two calls that overlap on the GPU
//    (different streams) would race on the array: run them in one stream or order
//    them with events.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define SS_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define SS_NOALLOC_COUNTERS 16384u
#define SS_NOALLOC_MAX_SLICES 64
#define SS_NOALLOC_TOO_LARGE (-1001)   // the call needs more scratch than the array holds
#define SS_NOALLOC_BAD_ARGUMENT (-1002)
#define SS_NOALLOC_SETUP_FAILED (-1003)  // cudaGetDevice / cudaGetSymbolAddress failed

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as ss_attn_decode_mma without the two scratch pointers.  Returns 0, a CUDA error code
// (> 0) from the launch, or one of the negative codes above.
int ss_attn_decode_noalloc(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* kv,
                           const int32_t* block_tables, int max_blocks, int n_requests,
                           const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv, int page_size,
                           int64_t num_pages, float scale, int window, int n_slices, int* err,
                           cudaStream_t stream);

// Floats of scratch the call above would need, and a sentence for a return code.
int64_t ss_attn_decode_noalloc_floats(int n_requests, int n_q, int n_slices);
const char* ss_attn_decode_noalloc_message(int code);

#ifdef __cplusplus
}
#endif
