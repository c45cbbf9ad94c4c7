// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for this
// library's own users.  Some of them run where cudaMalloc is off limits: inside a
// stream capture or a real-time loop where an allocation would stall or fail, in a
// plug-in whose host owns all device memory and hands out none, or under a memory
// budget that was fixed before this library was loaded.  The ordinary entry point
// (qd_decode_attention in attention_flash.cu) needs two scratch buffers from its
// caller when it splits the keys of a request over several CTAs; here that scratch
// is a fixed array that lives inside the library's device image, so the call
// allocates nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
// What it costs: QD_NOALLOC_SCRATCH_FLOATS floats (8 MiB) of device memory on every
// GPU on which this library is loaded, held until the process exits.
//
// Limits and rules
//  * T * H * splits * (d + 2) must not exceed QD_NOALLOC_SCRATCH_FLOATS; larger calls are
//    refused with QD_NOALLOC_TOO_LARGE and nothing is launched.  (64 requests x 16 heads
//    x 8 splits x head size 128 needs about 1.07 M floats.)
//  * The first call on a device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first
//    call outside any stream capture.
//  * All calls share the one array, and it keeps what the last call left in it.  Nothing
//    in it has to start at zero: every partial result is written by the call before the
//    same call reads it.  Two calls that overlap on the GPU (different streams, or
//    graphs replayed concurrently) race on the array; keep calls on one device ordered.
//  * The kernels are launched so that they may begin while the kernel before them on the stream
//    is still finishing (programmatic stream serialization), and they read `positions`,
//    `token_req`, `block_table` and the cache rows of earlier positions before they wait for that
//    kernel.  So the kernel that precedes this call on the stream must not still be writing
//    those when it lets its dependents start early.  Kernels that never trigger their dependents
//    early (every ordinary launch) are always safe; `q` and the newest cache row of each request
//    may be written by the preceding kernel in any case: they are read after the wait.
//  * Everything else (arguments, sizes accepted, result) is as qd_decode_attention.
#pragma once
#include <cuda_runtime.h>

#define QD_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)

#define QD_NOALLOC_OK 0
#define QD_NOALLOC_TOO_LARGE 20001     // the call needs more scratch than the fixed array holds
#define QD_NOALLOC_BAD_ARGUMENT 20002  // sizes or types the kernel does not take
#define QD_NOALLOC_SETUP_FAILED 20003  // the array's device address could not be looked up
// any other non-zero value is a CUDA error code from the launch

#ifdef __cplusplus
extern "C" {
#endif

// out[t, h, :] = attention of query token t (one per request) over the cached keys of its request.
// q: bfloat16, rows q_stride elements apart; out: bfloat16 [T, H*d]; kv: bfloat16
// [pages, 2, G, page_size, d]; block_table: int32 [*, max_blocks]; token_req, positions: int32 [T].
int qd_decode_attention_noalloc(const void* q, long long q_stride, void* out, const void* kv,
                                const int* block_table, int max_blocks, const int* token_req,
                                const int* positions, int T, int H, int G, int d, int page_size,
                                float scale, int window, int splits, cudaStream_t stream);

// Floats of scratch a call would need (to compare with QD_NOALLOC_SCRATCH_FLOATS beforehand).
long long qd_decode_attention_noalloc_scratch_floats(int T, int H, int d, int splits);

// A sentence for a return code of qd_decode_attention_noalloc.
const char* qd_decode_attention_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
