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

// ------------------------------------------------------------------------------------------------ the fast path
// The kernel above walks the whole row once per step of its bisections (33 for top_k, 33 more for top_p, an
// exponential per value each time): a millisecond for 8 rows of 128,256 logits.  Serving uses three short kernels
// instead, with the same cuts:
//   sample_cut_kernel    one block per row that has a cut.  Every cut is a threshold on the order-preserving key of the
//                        processed logit (top_k: the k-th largest key; top_p: the smallest key t with mass(key > t) <
//                        top_p * mass; min_p: a test against the row's maximum), so the kernel only has to find the
//                        thresholds.  It bisects over the whole row only until the bracket [lo, hi] that holds the
//                        threshold has few enough values to fit in shared memory -- taking the middle of the bracket's
//                        VALUES, not of their bit patterns, which gets there in one to four passes -- gathers those
//                        values and finishes the bisection there.  What lies above the bracket is carried as a count
//                        (top_k) or a weight (top_p).  Weights are fixed-point (2^-40 of the largest), so sums are exact
//                        and do not depend on the order in which values were gathered.
//   sample_draw_partial  (chunk of the vocabulary, row): recomputes the processed logits of its chunk, applies the
//                        thresholds, and takes the best of value + Gumbel noise (or of the bare value: greedy rows).
//   sample_draw_final    reduces a row's chunks, writes the token and counts it in the penalty state.
#define CUT_THREADS 1024
#define CUT_CAPACITY 16384             // values of a bracket in shared memory: key and value, 4 + 4 bytes
#define DRAW_CHUNKS 32
#define WEIGHT_ONE 1099511627776.0f    // 2^40: fixed-point weight of the row's largest value

struct RowCut {            // what sample_cut_kernel leaves for the draw
    int threshold;         // keep key >= threshold (INT_MIN: keep all)
    float mx;              // the row's maximum (for min_p)
};

__device__ __forceinline__ float processed(const float* lg, const int* rc, const unsigned char* rs, bool pen,
                                           const RowParams& P, float divisor, int v) {
    float a = lg[v];
    if (pen) {
        if (rs[v]) a = a > 0.0f ? a / P.rep : a * P.rep;
        const float c = (float)rc[v];
        a = a - P.freq * c;
        a = a - P.pres * (c > 0.0f ? 1.0f : 0.0f);
    }
    return a / divisor;
}

__device__ __forceinline__ float key_f32(int k) { return __int_as_float(k < 0 ? k ^ 0x7FFFFFFF : k); }

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    unsigned long long t = 0;
    for (int w = 0; w < nwarp; w++) t += sh[w];
    return t;
}

__device__ __forceinline__ unsigned long long weight_of(float x, float mx) {
    return __float2ull_rn(expf(x - mx) * WEIGHT_ONE);
}

// a key strictly inside (lo, hi]: on even turns the key of the middle of the two VALUES (what narrows real logits
// fastest), on odd turns, or when that is no such key, the middle of the keys themselves (which bounds the number of
// turns whatever the values are: an outlier of 1e30 would otherwise be halved a hundred times)
__device__ __forceinline__ int middle_key(int lo, int hi, int turn) {
    int mid = lo;
    if ((turn & 1) == 0) {
        const float m = 0.5f * key_f32(lo) + 0.5f * key_f32(hi);
        if (m == m && fabsf(m) < INFINITY) mid = f32_key(m);
    }
    if (mid <= lo || mid > hi) mid = (lo >> 1) + (hi >> 1) + ((lo | hi) & 1);      // the ceiling of the keys' middle
    return mid;
}

// f(value, index) for every value of a row of floats, four at a time when the row allows it (several 16-byte loads in
// flight per thread: one block walking a row of 128k values with 4-byte loads is bound by their latency)
template <typename F>
__device__ __forceinline__ void for_each_value(const float* __restrict__ x, int V, F f) {
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const int n4 = V >> 2;
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
            const float4 a = x4[i];
            f(a.x, 4 * i); f(a.y, 4 * i + 1); f(a.z, 4 * i + 2); f(a.w, 4 * i + 3);
        }
    } else {
        for (int v = threadIdx.x; v < V; v += blockDim.x) f(x[v], v);
    }
}

__global__ void __launch_bounds__(CUT_THREADS) sample_cut_kernel(const float* __restrict__ logits, float* __restrict__ work,
                                                                 const RowParams* __restrict__ params,
                                                                 const int* __restrict__ cnt,
                                                                 const unsigned char* __restrict__ seen, int V,
                                                                 RowCut* __restrict__ cuts) {
    extern __shared__ __align__(16) unsigned char cut_smem[];
    int* ckey = reinterpret_cast<int*>(cut_smem);                    // [CUT_CAPACITY]
    float* cval = reinterpret_cast<float*>(ckey + CUT_CAPACITY);     // [CUT_CAPACITY]
    __shared__ int sh_i[32];
    __shared__ unsigned long long sh_u[32];
    __shared__ int n_cand;
    const int row = blockIdx.x;
    const RowParams P = params[row];
    const bool top_k = P.top_k > 0 && P.top_k < V, top_p = P.top_p < 1.0f;
    if (P.temperature <= 0.0f || !(top_k || top_p || P.min_p > 0.0f)) {
        if (threadIdx.x == 0) { cuts[row].threshold = (int)0x80000000; cuts[row].mx = 0.0f; }
        return;
    }
    const float* lg = logits + (size_t)P.logits_row * V;
    float* x = work + (size_t)row * V;
    const int* rc = (P.slot >= 0 && cnt) ? cnt + (size_t)P.slot * V : nullptr;
    const unsigned char* rs = (P.slot >= 0 && seen) ? seen + (size_t)P.slot * V : nullptr;
    const bool pen = rc && (P.rep != 1.0f || P.freq != 0.0f || P.pres != 0.0f);

    // the processed logits, once, into the row's scratch; the smallest and the largest key
    int kmin = 0x7FFFFFFF, kmax = (int)0x80000000;
    if (!pen && (V & 3) == 0 && ((reinterpret_cast<uintptr_t>(lg) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        const float4* l4 = reinterpret_cast<const float4*>(lg);
        float4* x4 = reinterpret_cast<float4*>(x);
#pragma unroll 4
        for (int i = threadIdx.x; i < (V >> 2); i += blockDim.x) {
            float4 a = l4[i];
            a.x /= P.temperature; a.y /= P.temperature; a.z /= P.temperature; a.w /= P.temperature;
            x4[i] = a;
            const int k0 = f32_key(a.x), k1 = f32_key(a.y), k2 = f32_key(a.z), k3 = f32_key(a.w);
            kmin = min(min(kmin, min(k0, k1)), min(k2, k3));
            kmax = max(max(kmax, max(k0, k1)), max(k2, k3));
        }
    } else {
#pragma unroll 4
        for (int v = threadIdx.x; v < V; v += blockDim.x) {
            const float a = processed(lg, rc, rs, pen, P, P.temperature, v);
            x[v] = a;
            const int k = f32_key(a);
            kmin = min(kmin, k); kmax = max(kmax, k);
        }
    }
    kmin = block_min_i(kmin, sh_i);
    kmax = block_max_i(kmax, sh_i);
    const float mx = key_f32(kmax);
    __syncthreads();
    int threshold = (int)0x80000000;

    // gathers the values with lo <= key <= hi into shared memory (the caller knows there are at most CUT_CAPACITY)
    auto gather = [&](int lo, int hi) -> int {
        if (threadIdx.x == 0) n_cand = 0;
        __syncthreads();
        for_each_value(x, V, [&](float a, int) {
            const int k = f32_key(a);
            if (k >= lo && k <= hi) { const int s = atomicAdd(&n_cand, 1); if (s < CUT_CAPACITY) { ckey[s] = k; cval[s] = a; } }
        });
        __syncthreads();
        return min(n_cand, CUT_CAPACITY);
    };

    if (top_k) {
        // the largest key t with count(key >= t) >= k: t stays in [lo, hi]; `above` counts the keys above hi
        int lo = kmin, hi = kmax, above = 0, inside = V;
        for (int turn = 0; lo < hi && inside > CUT_CAPACITY; turn++) {
            const int mid = middle_key(lo, hi, turn);               // lo < mid <= hi
            int upper = 0;
            for_each_value(x, V, [&](float a, int) { const int k = f32_key(a); upper += (k >= mid && k <= hi); });
            upper = block_sum_i(upper, sh_i);
            if (above + upper >= P.top_k) { lo = mid; inside = upper; }
            else { hi = mid - 1; above += upper; inside -= upper; }
        }
        if (lo < hi) {
            const int n = gather(lo, hi);
            while (lo < hi) {
                const int mid = (lo >> 1) + (hi >> 1) + ((lo | hi) & 1);
                int mine = 0;
                for (int i = threadIdx.x; i < n; i += blockDim.x) mine += ckey[i] >= mid;
                mine = block_sum_i(mine, sh_i);
                if (above + mine >= P.top_k) lo = mid; else hi = mid - 1;
            }
        }
        threshold = lo;
    }

    if (top_p) {
        // the smallest key t with weight(key > t) < top_p * weight(all kept): t stays in [lo, hi]; `above` is the weight
        // of the keys above hi.  Only keys at or above the top_k threshold count.
        int lo = max(kmin, threshold), hi = kmax, inside = 0;
        unsigned long long total = 0, above = 0;
        {
            unsigned long long w = 0;
            int c = 0;
            for_each_value(x, V, [&](float a, int) { if (f32_key(a) >= lo) { w += weight_of(a, mx); c++; } });
            total = block_sum_u64(w, sh_u);
            inside = block_sum_i(c, sh_i);
        }
        const unsigned long long target = (unsigned long long)((double)P.top_p * (double)total);
        for (int turn = 0; lo < hi && inside > CUT_CAPACITY; turn++) {
            const int mid = middle_key(lo, hi, turn) - 1;           // lo <= mid < hi
            unsigned long long w = 0;
            int c = 0;
            for_each_value(x, V, [&](float a, int) {
                const int k = f32_key(a);
                if (k > mid && k <= hi) { w += weight_of(a, mx); c++; }
            });
            w = block_sum_u64(w, sh_u);
            c = block_sum_i(c, sh_i);
            if (above + w < target) { hi = mid; above += w; inside -= c; }
            else { lo = mid + 1; inside = c; }
        }
        if (lo < hi) {
            const int n = gather(lo, hi);
            while (lo < hi) {
                const int mid = (lo >> 1) + (hi >> 1) + (lo & hi & 1);
                unsigned long long w = 0;
                for (int i = threadIdx.x; i < n; i += blockDim.x) if (ckey[i] > mid) w += weight_of(cval[i], mx);
                w = block_sum_u64(w, sh_u);
                if (above + w < target) hi = mid; else lo = mid + 1;
            }
        }
        threshold = max(threshold, lo);
    }
    if (threadIdx.x == 0) { cuts[row].threshold = threshold; cuts[row].mx = mx; }
}

// grid (DRAW_CHUNKS, rows).  out_work: when given, the processed logits after the cuts (cut values -inf) are written.
__global__ void __launch_bounds__(256) sample_draw_partial_kernel(const float* __restrict__ logits,
                                                                   const RowParams* __restrict__ params,
                                                                   const int* __restrict__ cnt,
                                                                   const unsigned char* __restrict__ seen, int V,
                                                                   const RowCut* __restrict__ cuts, float* __restrict__ out_work,
                                                                   float* __restrict__ pval, int* __restrict__ pidx) {
    __shared__ ArgMax sh_a[32];
    const int row = blockIdx.y, chunk = blockIdx.x;
    const RowParams P = params[row];
    const float* lg = logits + (size_t)P.logits_row * V;
    const int* rc = (P.slot >= 0 && cnt) ? cnt + (size_t)P.slot * V : nullptr;
    const unsigned char* rs = (P.slot >= 0 && seen) ? seen + (size_t)P.slot * V : nullptr;
    const bool pen = rc && (P.rep != 1.0f || P.freq != 0.0f || P.pres != 0.0f);
    const bool greedy = P.temperature <= 0.0f;
    const float divisor = greedy ? 1.0f : P.temperature;
    RowCut cut = {(int)0x80000000, 0.0f};                               // no cut kernel ran: no row has a cut
    if (cuts) cut = cuts[row];
    const bool min_p = !greedy && P.min_p > 0.0f;
    const int per = (V + DRAW_CHUNKS - 1) / DRAW_CHUNKS;
    const int lo = chunk * per, hi = min(V, lo + per);
    ArgMax best = {-INFINITY, 0x7FFFFFFF};
#pragma unroll 4
    for (int v = lo + threadIdx.x; v < hi; v += blockDim.x) {
        const float a = processed(lg, rc, rs, pen, P, divisor, v);
        bool keep = f32_key(a) >= cut.threshold;
        if (keep && min_p) keep = !(expf(a - cut.mx) < P.min_p);
        if (out_work) out_work[(size_t)row * V + v] = keep ? a : -INFINITY;
        if (!keep || a == -INFINITY) continue;
        ArgMax c = {greedy ? a : a + gumbel(philox_word(P.seed_lo, P.seed_hi, (uint32_t)v, (uint32_t)P.step)), v};
        best = better(best, c);
    }
    best = block_argmax(best, sh_a);
    if (threadIdx.x == 0) { pval[row * DRAW_CHUNKS + chunk] = best.v; pidx[row * DRAW_CHUNKS + chunk] = best.i; }
}

__global__ void sample_draw_final_kernel(const float* __restrict__ pval, const int* __restrict__ pidx,
                                         const RowParams* __restrict__ params, int* __restrict__ cnt,
                                         unsigned char* __restrict__ seen, int V, int* __restrict__ out) {
    const int row = blockIdx.x, lane = threadIdx.x;                    // 32 threads, one chunk each
    ArgMax a = {pval[row * DRAW_CHUNKS + lane], pidx[row * DRAW_CHUNKS + lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    if (lane == 0) {
        const int token = a.i;
        out[row] = token;
        const int slot = params[row].slot;
        if (slot >= 0 && cnt && seen && token >= 0 && token < V) {
            cnt[(size_t)slot * V + token] += 1;
            seen[(size_t)slot * V + token] = 1;
        }
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
    const int per = ((V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS + 3) & ~3;        // a multiple of four: chunks start on 16 bytes
    const int lo = min(V, chunk * per), hi = min(V, lo + per);
    const float* lg = logits + (size_t)row * V;
    ArgMax best = {-INFINITY, 0x7FFFFFFF};
    if (V % 4 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
        // four values a load, all of a thread's loads in flight before the first comparison (one value a load and
        // turn left the kernel waiting on sixteen trips to the L2: 10 us for 8 rows of 128,256)
        const float4* lg4 = reinterpret_cast<const float4*>(lg);
        for (int q0 = lo / 4 + threadIdx.x; q0 < hi / 4; q0 += 4 * blockDim.x) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int q = q0 + u * blockDim.x;
                x[u] = q < hi / 4 ? lg4[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int v = 4 * (q0 + u * blockDim.x);
                ArgMax c0 = {x[u].x, v}, c1 = {x[u].y, v + 1}, c2 = {x[u].z, v + 2}, c3 = {x[u].w, v + 3};
                best = better(best, c0); best = better(best, c1); best = better(best, c2); best = better(best, c3);
            }
        }
    } else {
        for (int v = lo + threadIdx.x; v < hi; v += blockDim.x) { ArgMax c = {lg[v], v}; best = better(best, c); }
    }
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

// The three-kernel path.  work: (n_rows, V) floats of scratch for the rows with cuts; cuts: n_rows RowCut (8 bytes each);
// pval, pidx: n_rows * 32 floats / ints; out_work: null, or (n_rows, V) floats that receive the processed logits after
// the cuts.  any_cut: 0 when no row has a top_k, top_p or min_p (the first kernel is skipped).
MB_API int mb_sample_fast(const float* logits, float* work, const void* params, int* cnt, unsigned char* seen, int n_rows,
                          int V, void* cuts, float* pval, int* pidx, float* out_work, int any_cut, int* out,
                          cudaStream_t st) {
    if (n_rows == 0) return 0;
    if (n_rows > 65535) return -2;
    const size_t smem = (size_t)CUT_CAPACITY * 8;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(sample_cut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (any_cut)
        sample_cut_kernel<<<n_rows, CUT_THREADS, smem, st>>>(logits, work, (const RowParams*)params, cnt, seen, V, (RowCut*)cuts);
    sample_draw_partial_kernel<<<dim3(DRAW_CHUNKS, n_rows), 256, 0, st>>>(logits, (const RowParams*)params, cnt, seen, V,
                                                                          any_cut ? (const RowCut*)cuts : nullptr, out_work,
                                                                          pval, pidx);
    sample_draw_final_kernel<<<n_rows, 32, 0, st>>>(pval, pidx, (const RowParams*)params, cnt, seen, V, out);
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
