// Shared helpers of the sm_100a kernels: storage types, warp/block reductions with a fixed shape, error codes.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define MB_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// Codes a kernel leaves in the engine's error word (first one wins); the host reads the word after a step.
enum MbDeviceError {
    MB_ERR_NONE = 0,
    MB_ERR_TOKEN_RANGE = 1,     // a token id outside [0, vocab)
    MB_ERR_PAGE_MISSING = 2,    // a position whose page the block table does not hold
    MB_ERR_PAGE_RANGE = 3,      // a page id outside the pool
    MB_ERR_WAIT_TIMEOUT = 4,    // a bounded wait inside a kernel ran out
};

__device__ __forceinline__ void mb_set_error(int* err, int code) {
    if (err) atomicCAS(err, 0, code);
}

template <typename T> __device__ __forceinline__ float mb_load(const T* p);
template <> __device__ __forceinline__ float mb_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float mb_load<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void mb_store(T* p, float v);
template <> __device__ __forceinline__ void mb_store<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void mb_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float mb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float mb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024): warp trees, then one tree over the warp sums.
// The shape of the reduction depends on the block size only, so a row's result does not depend on the batch.
__device__ __forceinline__ float mb_block_sum(float v, float* scratch /* 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = mb_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : 0.0f;
    return mb_warp_sum(t);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// two floats rounded to bf16 in one 32-bit word, the first in the low half
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---- programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may start while
// the kernel before it in the stream still runs.  It must call pdl_wait() -- every thread that goes on to touch global
// memory -- before it reads anything another kernel of the step wrote and before it writes anything at all; what it
// does before that (setting barriers up, fetching weights, which no kernel writes) overlaps with the tail of the kernel
// before.  Data that a kernel before it produced is read around the L1 (TMA, cp.async.cg, ld.global.cg), never through
// the read-only path: a line may have reached an SM's L1 before its producer had finished.  pdl_launch_dependents()
// lets the kernel AFTER this one start; without the attribute on the launch both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// Every kernel library has one switch: MB_PDL_SWITCH(mb_<library>_set_pdl) defines it and the function that sets it.
#define MB_PDL_SWITCH(name) static int mb_pdl = 0; MB_API int name(int on) { mb_pdl = on; return 0; }

// kernel<<<grid, block, smem, st>>>(args...), with the programmatic-serialization attribute when pdl is set
template <typename... Params, typename... Args>
static inline cudaError_t mb_launch(bool pdl, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t st, Args... args) {
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// the same as a launch of thread-block clusters of cluster_x blocks along x (1: no clusters)
template <typename... Params, typename... Args>
static inline cudaError_t mb_launch_cluster(bool pdl, unsigned cluster_x, void (*kernel)(Params...), dim3 grid, dim3 block,
                                            size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

#define MB_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)
