// An entry point of the kernel library that allocates nothing.  It has no counterpart in the
// reference (acvram reaches its kernels through torch and lets torch's allocator serve them).
//
// Who it is for.  Every other attention entry point of this library takes its scratch memory from
// the caller, who gets it from an allocator.  Some callers have none to ask: a C or C++ host that
// links the library without torch; a serving process that gave all of the device's memory to a pool
// of its own at start-up, so that a later cudaMalloc fails; a latency-bound loop that must not enter
// cudaMalloc or cudaFree because those calls stall the whole device.  For them the split-KV decode
// attention is offered once more with its scratch inside the library.
//
//   acv_attention_decode_static(...)   same arguments as acv_attention_decode, without the three
//                                      scratch pointers and their sizes
//
// The scratch is one file-scope device array of 4 MiB (2^20 floats;
// acv_attention_decode_static_capacity() returns that number).  Each GPU on which the library is
// loaded holds it until the process exits.  It has to hold, for n_splits > 1,
//     n_dec * NKV * n_splits * (NH/NKV) * (D + 2)  floats   (partial results of the splits)
//   + n_dec * NKV                                  ints     (one arrival counter per request and kv-head)
// and a call that needs more is refused with ACV_ERR_SCRATCH (-5) before anything is launched.
// Example: 64 requests, 8 kv-heads, 4 query heads per kv-head, head size 128, 3 splits: 0.8 M floats.
//
// The call itself makes no cudaMalloc, cudaFree or other allocating call: it clears its counters
// with cudaMemsetAsync on the given stream and launches the kernel there.  The first call on a
// device also asks the runtime for the array's device address (cudaGetSymbolAddress, with that
// device current) and remembers it; make that first call on each device outside any stream capture.
//
// All calls share the one array, and it keeps what the last call left.  Calls on the same stream
// follow one another and are safe.  Two calls that can run on the GPU at the same time (different
// streams, different host threads) race on the scratch and give wrong results: serialise them.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long acv_attention_decode_static_capacity(void);

int acv_attention_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, const int* dec_tokens, const int* dec_seqs, int n_dec,
                                const int* kv_len, const int* block_table, int bt_stride, int NH, int NKV, int D,
                                int page_size, int num_pages, float scale, int window, int n_splits, int max_kv,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
