// Declaration of the one entry point of this library that allocates nothing.  It has no counterpart in
// mashbox-labs/mashbox: it exists for callers of these kernels that cannot allocate device memory.
//
// Who cannot allocate, and why.  The engine of this repository sizes its cache pool once and keeps a workspace for its
// scratch, so it never needs this.  Other programs that link the kernels directly may be in a different position: a
// host that has given every remaining byte of the GPU to its own pools at start-up (a later cudaMalloc fails or
// fragments), a real-time loop that must not take the driver's allocation lock, or a plug-in that runs under another
// program's memory manager and is forbidden to call cudaMalloc / cudaFree at all.  For them mb_sample_noalloc runs the
// sampling kernel with its scratch (the processed logits of every row) in a fixed array that is part of the library
// image: `static __device__ __align__(256) float[MB_NOALLOC_MAX_ROWS * MB_NOALLOC_MAX_VOCAB]`, 2 MiB, held by every GPU
// that loads the library until the process exits.
//
// Contract.
//   * logits, params, cnt, seen and out are the caller's, exactly as for mb_sample; only `work` is gone.  cnt and
//     seen come together or not at all (one without the other is MB_NOALLOC_BAD_ARGUMENT).  What stands INSIDE params
//     is not checked: each row's `logits_row` must be a row of `logits`, and its `slot` -1 or a row of cnt / seen (and
//     -1 when those are null); a wrong value there makes the kernel read or write outside the caller's arrays.
//   * n_rows <= MB_NOALLOC_MAX_ROWS and vocab <= MB_NOALLOC_MAX_VOCAB, else MB_NOALLOC_TOO_LARGE is returned and nothing
//     is launched.  mb_noalloc_strerror() gives the words for a return code.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, once per device, with that
//     device current) and keeps it; make that first call before any stream capture begins.  That first call is also
//     when the driver loads this library's image on the device, which is when the 2 MiB of the array are taken.
//   * Every call shares the one array and finds the previous call's contents in it.  Nothing in it has to start at
//     zero: the kernel writes each row's V values before it reads them.  Two calls that overlap on the GPU (different
//     streams, no dependency) race on the array; order them.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#define MB_NOALLOC_MAX_ROWS 4
#define MB_NOALLOC_MAX_VOCAB 131072

#define MB_NOALLOC_TOO_LARGE (-3)      // n_rows or vocab beyond the maximum above
#define MB_NOALLOC_BAD_ARGUMENT (-4)   // a null pointer, a non-positive size, or only one of cnt and seen
#define MB_NOALLOC_NO_SYMBOL (-5)      // the scratch array's address could not be looked up on this device

#ifdef __cplusplus
extern "C" {
#endif
int mb_sample_noalloc(const float* logits, const void* params, int* cnt, unsigned char* seen, int n_rows, int vocab,
                      int* out, cudaStream_t stream);
const char* mb_noalloc_strerror(int code);
int mb_noalloc_max_rows(void);
int mb_noalloc_max_vocab(void);
#ifdef __cplusplus
}
#endif
