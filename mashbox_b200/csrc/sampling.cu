// Sampling on the device, one block per row of logits.  Order, as mashbox-labs/mashbox's sampler: repetition penalty
// (prompt + generated tokens; positive logits divided, negative multiplied) -> frequency penalty -> presence penalty ->
// temperature -> top_k -> top_p -> min_p -> one draw.  temperature <= 0 is greedy: the lowest index of the maximum of
// the penalised logits.  Ties at a top_k or top_p cut are kept; the cuts are found by bisection on order-preserving
// integer keys.  The draw is argmax(x + Gumbel noise) with Philox4x32-10 keyed by the row's 64-bit seed and counted by
// (vocabulary index, index of the token in the row's answer), so a row's tokens depend on nothing else in the batch.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ int f32_key(float x) {
    int b = __float_as_int(x);
    return b < 0 ? b ^ 0x7FFFFFFF : b;
}

__device__ __forceinline__ uint32_t philox_word(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1) {
    uint32_t c2 = 0u, c3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c0;
}

__device__ __forceinline__ float gumbel(uint32_t word) {
    const float u = ((float)(word >> 8) + 0.5f) * (1.0f / 16777216.0f);      // in (0, 1), 24 bits
    return -logf(-logf(u));
}

struct ArgMax { float v; int i; };

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) sh[warp] = a;
    __syncthreads();
    ArgMax r = sh[0];
    for (int w = 1; w < nwarp; w++) r = better(r, sh[w]);
    return r;
}

__device__ float block_sum_f(float v, float* sh) { return mb_block_sum(v, sh); }

__device__ int block_sum_i(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int t = 0;
    for (int w = 0; w < nwarp; w++) t += sh[w];
    return t;
}

__device__ int block_min_i(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int t = sh[0];
    for (int w = 1; w < nwarp; w++) t = min(t, sh[w]);
    return t;
}

__device__ int block_max_i(int v, int* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    int t = sh[0];
    for (int w = 1; w < nwarp; w++) t = max(t, sh[w]);
    return t;
}

struct RowParams {          // one per row, filled on the host
    float temperature, top_p, min_p, rep, freq, pres;
    int top_k;
    int slot;               // row of the penalty state, -1 = the row has none
    uint32_t seed_lo, seed_hi;
    int step;               // index of the token in the row's answer
    int logits_row;         // row of the logits matrix
};

// logits (n_logit_rows, V) float; work (n_rows, V) float scratch; cnt (slots, V) int32 counts of generated tokens;
// seen (slots, V) uint8 prompt + generated tokens.  The chosen token is added to the row's penalty state.
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits, float* __restrict__ work,
                                                                 const RowParams* __restrict__ params, int* __restrict__ cnt,
                                                                 unsigned char* __restrict__ seen, int V,
                                                                 int* __restrict__ out) {
    __shared__ ArgMax sh_a[32];
    __shared__ float sh_f[32];
    __shared__ int sh_i[32];
    const int row = blockIdx.x;
    const RowParams P = params[row];
    const float* lg = logits + (size_t)P.logits_row * V;
    float* x = work + (size_t)row * V;
    int* rc = (P.slot >= 0 && cnt) ? cnt + (size_t)P.slot * V : nullptr;
    unsigned char* rs = (P.slot >= 0 && seen) ? seen + (size_t)P.slot * V : nullptr;
    const bool pen = rc && (P.rep != 1.0f || P.freq != 0.0f || P.pres != 0.0f);
    const bool greedy = P.temperature <= 0.0f;
    const float invT_div = greedy ? 1.0f : P.temperature;

    // pass 0: penalties, the greedy token, temperature
    ArgMax best = {-INFINITY, 0x7FFFFFFF};
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
        float a = lg[v];
        if (pen) {
            if (rs[v]) a = a > 0.0f ? a / P.rep : a * P.rep;
            const float c = (float)rc[v];
            a = a - P.freq * c;
            a = a - P.pres * (c > 0.0f ? 1.0f : 0.0f);
        }
        ArgMax cand = {a, v};
        best = better(best, cand);
        x[v] = a / invT_div;
    }
    best = block_argmax(best, sh_a);
    int token = best.i;
    if (!greedy) {
        __syncthreads();
        if (P.top_k > 0 && P.top_k < V) {
            int kmin = 0x7FFFFFFF, kmax = (int)0x80000000;
            for (int v = threadIdx.x; v < V; v += blockDim.x) { const int k = f32_key(x[v]); kmin = min(kmin, k); kmax = max(kmax, k); }
            int lo = block_min_i(kmin, sh_i);
            int hi = block_max_i(kmax, sh_i);
            for (int it = 0; it < 33; it++) {
                const int mid = (lo >> 1) + (hi >> 1) + ((lo | hi) & 1);
                int c = 0;
                for (int v = threadIdx.x; v < V; v += blockDim.x) c += f32_key(x[v]) >= mid;
                c = block_sum_i(c, sh_i);
                if (c >= P.top_k) lo = mid; else hi = mid - 1;
            }
            for (int v = threadIdx.x; v < V; v += blockDim.x) if (f32_key(x[v]) < lo) x[v] = -INFINITY;
            __syncthreads();
        }
        if (P.top_p < 1.0f) {
            float mx = -INFINITY;
            int kmin = 0x7FFFFFFF, kmax = (int)0x80000000;
            for (int v = threadIdx.x; v < V; v += blockDim.x) {
                const float a = x[v]; mx = fmaxf(mx, a);
                const int k = f32_key(a); kmin = min(kmin, k); kmax = max(kmax, k);
            }
            ArgMax am = {mx, (int)threadIdx.x};
            mx = block_argmax(am, sh_a).v;
            float z = 0.0f;
            for (int v = threadIdx.x; v < V; v += blockDim.x) z += expf(x[v] - mx);
            z = block_sum_f(z, sh_f);
            int lo = block_min_i(kmin, sh_i);
            int hi = block_max_i(kmax, sh_i);
            for (int it = 0; it < 33; it++) {
                const int mid = (lo >> 1) + (hi >> 1) + (lo & hi & 1);
                float mass = 0.0f;
                for (int v = threadIdx.x; v < V; v += blockDim.x) { const float a = x[v]; if (f32_key(a) > mid) mass += expf(a - mx); }
                mass = block_sum_f(mass, sh_f);
                if (mass < P.top_p * z) hi = mid; else lo = mid + 1;
            }
            for (int v = threadIdx.x; v < V; v += blockDim.x) if (f32_key(x[v]) < hi) x[v] = -INFINITY;
            __syncthreads();
        }
        if (P.min_p > 0.0f) {
            float mx = -INFINITY;
            for (int v = threadIdx.x; v < V; v += blockDim.x) mx = fmaxf(mx, x[v]);
            ArgMax am = {mx, (int)threadIdx.x};
            mx = block_argmax(am, sh_a).v;
            for (int v = threadIdx.x; v < V; v += blockDim.x) if (expf(x[v] - mx) < P.min_p) x[v] = -INFINITY;
            __syncthreads();
        }
        ArgMax d = {-INFINITY, 0x7FFFFFFF};
        for (int v = threadIdx.x; v < V; v += blockDim.x) {
            const float a = x[v];
            if (a == -INFINITY) continue;
            ArgMax cand = {a + gumbel(philox_word(P.seed_lo, P.seed_hi, (uint32_t)v, (uint32_t)P.step)), v};
            d = better(d, cand);
        }
        d = block_argmax(d, sh_a);
        token = d.i;
    }
    if (threadIdx.x == 0) {
        out[row] = token;
        if (rc && token >= 0 && token < V) { rc[token] += 1; rs[token] = 1; }
    }
}

// Rebuilds one row of the penalty state: seen = prompt + generated tokens, cnt = counts of the generated tokens.
__global__ void penalty_fill_kernel(int* __restrict__ cnt_row, unsigned char* __restrict__ seen_row,
                                    const int* __restrict__ tokens, int n_prompt, int n_total, int V) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_total) return;
    const int t = tokens[i];
    if (t < 0 || t >= V) return;
    seen_row[t] = 1;
    if (i >= n_prompt) atomicAdd(cnt_row + t, 1);
}

// first index of the maximum of each row (the greedy token without any other processing), in two stages so that a few
// rows still fill the GPU: blocks (chunk, row) reduce a chunk of the row each, then one block per row reduces the chunks
#define ARGMAX_CHUNKS 32
__global__ void __launch_bounds__(256) argmax_partial_kernel(const float* __restrict__ logits, int V,
                                                              float* __restrict__ pval, int* __restrict__ pidx) {
    __shared__ ArgMax sh_a[32];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = chunk * per, hi = min(V, lo + per);
    const float* lg = logits + (size_t)row * V;
    ArgMax best = {-INFINITY, 0x7FFFFFFF};
    for (int v = lo + threadIdx.x; v < hi; v += blockDim.x) { ArgMax c = {lg[v], v}; best = better(best, c); }
    best = block_argmax(best, sh_a);
    if (threadIdx.x == 0) { pval[row * ARGMAX_CHUNKS + chunk] = best.v; pidx[row * ARGMAX_CHUNKS + chunk] = best.i; }
}

__global__ void argmax_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx, int* __restrict__ out) {
    const int row = blockIdx.x, lane = threadIdx.x;                    // 32 threads, one chunk each
    ArgMax a = {pval[row * ARGMAX_CHUNKS + lane], pidx[row * ARGMAX_CHUNKS + lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    if (lane == 0) out[row] = a.i;
}

#ifndef MB_SAMPLING_KERNELS_ONLY
MB_API int mb_sample(const float* logits, float* work, const void* params, int* cnt, unsigned char* seen, int n_rows,
                     int V, int* out, cudaStream_t st) {
    if (n_rows == 0) return 0;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, st>>>(logits, work, (const RowParams*)params, cnt, seen, V, out);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_penalty_fill(int* cnt_row, unsigned char* seen_row, const int* tokens, int n_prompt, int n_total, int V,
                           cudaStream_t st) {
    if (n_total == 0) return 0;
    penalty_fill_kernel<<<(n_total + 255) / 256, 256, 0, st>>>(cnt_row, seen_row, tokens, n_prompt, n_total, V);
    MB_LAUNCH_CHECK();
    return 0;
}

// scratch: n_rows * 32 floats and as many ints, given by the caller (pval, pidx)
MB_API int mb_argmax(const float* logits, int n_rows, int V, float* pval, int* pidx, int* out, cudaStream_t st) {
    if (n_rows == 0) return 0;
    if (n_rows > 65535) return -2;
    argmax_partial_kernel<<<dim3(ARGMAX_CHUNKS, n_rows), 256, 0, st>>>(logits, V, pval, pidx);
    argmax_final_kernel<<<n_rows, 32, 0, st>>>(pval, pidx, out);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_sample_params_size() { return (int)sizeof(RowParams); }
#endif  // MB_SAMPLING_KERNELS_ONLY
