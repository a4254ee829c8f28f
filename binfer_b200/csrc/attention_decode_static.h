// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (bwasti/binfer); it is an
// addition of this library.
//
// Who needs it: a program that drives this library through its C symbols and
// has no allocator to offer it.  Examples: a serving process whose own pool took
// all device memory at start-up, so that a later cudaMalloc would fail; a
// latency-bound loop that must not pay cudaMalloc's device-wide synchronisation;
// a host written in another language that can pass pointers it already owns but
// cannot call the CUDA runtime (or torch's allocator) for more.  The ordinary
// entry point, bf_decode_attention, needs two scratch buffers from its caller
// for the partial results of the key splits; here that scratch is a fixed array
// inside the library instead.
//
// The array is BF_DECODE_STATIC_SCRATCH_BYTES (8 MiB) of device memory.  Every
// GPU on which the library is loaded holds it from load until the process exits.
//
// Size limit: n_rows * nh * max_splits * (d + 2) * 4 bytes must fit the array
// (for instance 8 rows x 32 heads x 32 splits at head size 128).  A larger call
// is refused with BF_STATIC_ERR_TOO_LARGE and nothing is launched.
//
// First call on a device: the entry point looks up the array's device address
// once per device (cudaGetSymbolAddress, with that device current) and keeps
// it.  Make this first call outside any stream capture.
//
// Sharing: all calls use the same array, and it keeps what the last call left.
// Nothing in it has to start at zero: each call writes every partial result it
// later reads.  Two calls that overlap on the GPU (different streams, or one
// stream on two host threads without ordering) race on the array; order them.
//
// The function calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once
#include <cuda_runtime.h>

#define BF_DECODE_STATIC_SCRATCH_BYTES (8u << 20)

#define BF_STATIC_ERR_TOO_LARGE (-1)   // the splits' partial results exceed the array
#define BF_STATIC_ERR_HEAD_DIM (-2)    // head size not one of 32, 64, 96, 128, 256
#define BF_STATIC_ERR_ARGUMENT (-3)    // a null pointer or a non-positive size
#define BF_STATIC_ERR_DEVICE (-4)      // device index beyond what the library tracks

#ifdef __cplusplus
extern "C" {
#endif

// Same computation and arguments as bf_decode_attention, minus the scratch pointers:
// q [tokens, nh, d] bf16; k_cache, v_cache [pages, nkv, page_size, d] bf16;
// rows (may be null: rows 0..n_rows-1), seq_of_token, positions: int32 per token;
// block_tables int32 [requests, table_stride]; out [tokens, nh, d] bf16;
// max_splits >= ceil(longest context / 128); err: int32 error word on the device.
// A row whose keys need more splits than max_splits says is not a fault: the kernels set
// bit 16 of the error word, leave the splits without room out of that row's result, and
// neither read nor write past the part of the array that the call was sized for.
// Returns 0, a BF_STATIC_ERR_* code (negative), or a cudaError_t (positive).
int bf_decode_attention_static(const void* q, const void* k_cache, const void* v_cache,
                               const int* rows, const int* seq_of_token, const int* positions,
                               const int* block_tables, int table_stride, void* out, int n_rows,
                               int nh, int nkv, int d, int page_size, int num_pages, int window,
                               int max_splits, float scale, int* err, cudaStream_t stream);

// A sentence for each code that bf_decode_attention_static can return.
const char* bf_decode_attention_static_error(int code);

#ifdef __cplusplus
}
#endif
