// Allocation-free entry point of libtahb200.  It has no counterpart in the reference code base.
//
// Who needs it: callers that are not allowed to create device memory at the moment they need
// attention results.  Examples are a serving loop that runs under a fixed, pre-negotiated memory
// budget (another framework owns the allocator and hands this library only input and output
// buffers), a plug-in loaded into a host process whose policy forbids cudaMalloc after start-up,
// and latency-critical code for which the implicit device synchronisation of cudaMalloc / cudaFree
// is unacceptable.  The regular split-KV decode attention needs a scratch buffer for the partial
// results of the splits and expects the caller to allocate it; this variant brings its own.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch area, in floats.  A call needs
// rows * nq * n_split * (hd + 2) floats when n_split > 1 and none when n_split == 1.
long long tahb_decode_attn_noalloc_capacity(void);

// Split-KV paged decode attention with the scratch held inside the library.
//
// Same arguments and results as tahb_decode_attn, minus the workspace pointer: the caller passes
// only inputs (q, the paged caches, page tables, lengths, depths) and the output buffer.  The
// partial results of the n_split splits go to a file-scope device array of
// tahb_decode_attn_noalloc_capacity() floats (4 MiB) that every GPU which loads the library keeps
// until the process exits.  The function calls neither cudaMalloc nor cudaFree nor any routine
// that allocates.
//
// Returns 0 on success; -7 when the request needs more scratch than the built-in area holds
// (lower n_split or the number of rows, or use tahb_decode_attn with your own buffer); -8 when the
// address of the scratch array could not be obtained; otherwise the codes of tahb_decode_attn.
//
// First call on a device: the function looks up the device address of the scratch array (with that
// device current) and remembers it.  Make this first call before starting any stream capture.
//
// All calls on one device share the one scratch area, and it keeps the previous call's contents.
// Nothing in it has to start at zero (every slot that is read is written first by the same call),
// but two calls whose kernels may overlap on the GPU - different streams without an ordering
// between them, or several host threads - race on it and must be serialised by the caller.
int tahb_decode_attn_noalloc(const void* q, void* out, void* const* caches, const int* const* page_tables,
                             const int* const* lens, const int* max_pages, int n_caches, const int* depth,
                             int rows, int nq, int nkv, int hd, int page_size, float scale, int n_split,
                             int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
