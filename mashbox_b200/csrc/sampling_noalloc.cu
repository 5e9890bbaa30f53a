// mb_sample_noalloc: the sampling kernel with its scratch in a fixed device array instead of caller-supplied memory,
// for callers that cannot allocate (see sampling_noalloc.h, which states the contract).  The kernel itself is the one
// of sampling.cu, compiled into this library a second time; only the launcher differs.
#define MB_SAMPLING_KERNELS_ONLY
#include "sampling.cu"
#include "sampling_noalloc.h"
#include <mutex>

// The scratch: processed logits of up to MB_NOALLOC_MAX_ROWS rows of up to MB_NOALLOC_MAX_VOCAB values (2 MiB).
// In host code this name is only a stand-in for the symbol; a kernel must be given the address that
// cudaGetSymbolAddress returns for the current device.
static __device__ __align__(256) float mb_noalloc_scratch[(size_t)MB_NOALLOC_MAX_ROWS * MB_NOALLOC_MAX_VOCAB];

#define MB_NOALLOC_MAX_DEVICES 64
static float* scratch_of_device[MB_NOALLOC_MAX_DEVICES];       // filled on the first call on each device
static std::once_flag scratch_looked_up[MB_NOALLOC_MAX_DEVICES];  // two threads may make a device's first call together

static int scratch_address(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MB_NOALLOC_MAX_DEVICES) return MB_NOALLOC_NO_SYMBOL;
    std::call_once(scratch_looked_up[dev], [dev]() {
        void* p = nullptr;                  // a failed lookup leaves the entry null, and every call reports it
        if (cudaGetSymbolAddress(&p, mb_noalloc_scratch) == cudaSuccess) scratch_of_device[dev] = static_cast<float*>(p);
    });
    if (scratch_of_device[dev] == nullptr) return MB_NOALLOC_NO_SYMBOL;
    *out = scratch_of_device[dev];
    return 0;
}

extern "C" __attribute__((visibility("default")))
int mb_sample_noalloc(const float* logits, const void* params, int* cnt, unsigned char* seen, int n_rows, int vocab,
                      int* out, cudaStream_t stream) {
    if (!logits || !params || !out || n_rows <= 0 || vocab <= 0) return MB_NOALLOC_BAD_ARGUMENT;
    if ((cnt == nullptr) != (seen == nullptr)) return MB_NOALLOC_BAD_ARGUMENT;      // the penalty state comes as a pair
    if (n_rows > MB_NOALLOC_MAX_ROWS || vocab > MB_NOALLOC_MAX_VOCAB) return MB_NOALLOC_TOO_LARGE;
    float* work = nullptr;
    const int rc = scratch_address(&work);
    if (rc != 0) return rc;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, work, (const RowParams*)params, cnt, seen, vocab, out);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" __attribute__((visibility("default")))
const char* mb_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case MB_NOALLOC_TOO_LARGE: return "mb_sample_noalloc: n_rows or vocab is beyond the fixed scratch (4 rows of 131072 values)";
        case MB_NOALLOC_BAD_ARGUMENT: return "mb_sample_noalloc: a null pointer, a non-positive size, or only one of cnt and seen";
        case MB_NOALLOC_NO_SYMBOL: return "mb_sample_noalloc: the scratch array's device address could not be looked up";
        default: return "mb_sample_noalloc: CUDA error at launch";
    }
}

extern "C" __attribute__((visibility("default"))) int mb_noalloc_max_rows(void) { return MB_NOALLOC_MAX_ROWS; }
extern "C" __attribute__((visibility("default"))) int mb_noalloc_max_vocab(void) { return MB_NOALLOC_MAX_VOCAB; }
