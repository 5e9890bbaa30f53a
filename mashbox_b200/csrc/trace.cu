// Tracing of logits: per row an order-independent hash and the gap between the two largest logits.
//
// hash(row) = sum over v of bits(lg[v]) * (2 v + 1) mod 2^32, as mashbox-labs/mashbox records it per generated token
// (src/mashbox/runtime/engine.py:80-84): an integer sum, so it does not depend on the order of the reduction, and any
// single changed bit of any logit changes it.  Two runs whose rows have equal hashes computed bit-identical logits:
// the cheap way to check that a request's logits do not depend on how it was batched or cut into steps.
// gap(row) = largest - second largest logit in float32 (engine.py:87-89; two equal maxima give 0): how close the greedy
// choice was to a tie.
#include "common.cuh"

#define TRACE_THREADS 1024

// out: n_rows pairs (hash as uint32, gap as float bits)
__global__ void __launch_bounds__(TRACE_THREADS)
logit_trace_kernel(const float* __restrict__ logits, int V, uint32_t* __restrict__ out) {
    __shared__ uint32_t sh_hash[32];
    __shared__ float sh_a[32], sh_b[32];
    const float* lg = logits + (size_t)blockIdx.x * V;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t h = 0u;
    float a = -INFINITY, b = -INFINITY;                 // the largest and the second largest seen (b <= a)
    for (int v = threadIdx.x; v < V; v += TRACE_THREADS) {
        const float x = lg[v];
        h += __float_as_uint(x) * (2u * (uint32_t)v + 1u);
        if (x > a) { b = a; a = x; } else if (x > b) b = x;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        h += __shfl_xor_sync(0xffffffffu, h, o);
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        // the two largest of {a, b, oa, ob} with a >= b and oa >= ob
        const float hi = fmaxf(a, oa), lo = fmaxf(fminf(a, oa), fmaxf(b, ob));
        a = hi; b = lo;
    }
    if (lane == 0) { sh_hash[warp] = h; sh_a[warp] = a; sh_b[warp] = b; }
    __syncthreads();
    if (warp == 0) {
        h = sh_hash[lane]; a = sh_a[lane]; b = sh_b[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            h += __shfl_xor_sync(0xffffffffu, h, o);
            const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
            const float hi = fmaxf(a, oa), lo = fmaxf(fminf(a, oa), fmaxf(b, ob));
            a = hi; b = lo;
        }
        if (lane == 0) {
            out[2 * blockIdx.x] = h;
            out[2 * blockIdx.x + 1] = __float_as_uint(V > 1 ? a - b : 0.0f);
        }
    }
}

MB_API int mb_logit_trace(const float* logits, int n_rows, int V, uint32_t* out, cudaStream_t st) {
    if (n_rows == 0) return 0;
    if (V < 1) return -2;
    logit_trace_kernel<<<n_rows, TRACE_THREADS, 0, st>>>(logits, V, out);
    MB_LAUNCH_CHECK();
    return 0;
}
