// Memory-bound kernels of the step: embedding gather, residual-add + RMSNorm, rotation + K/V page write, SwiGLU.
// T is the activation / cache storage type (float on the 32-bit path, bf16 to serve); all arithmetic is float.
#include "common.cuh"

// ------------------------------------------------------------------------------------------------ 8-wide access
// Eight consecutive values as floats, read and written with 128-bit accesses (the address must be 16-byte aligned for
// bf16 and 32-byte aligned rows are not needed: two float4 for float storage).
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------------------------------------ embedding
// x[n, :] = table[tok[n], :] into the float residual stream.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tok, const T* __restrict__ table, float* __restrict__ x,
                             int D, int V, int* err) {
    const int n = blockIdx.x;
    int t = tok[n];
    if (t < 0 || t >= V) {
        if (threadIdx.x == 0) mb_set_error(err, MB_ERR_TOKEN_RANGE);
        for (int d = threadIdx.x; d < D; d += blockDim.x) x[(size_t)n * D + d] = 0.0f;
        return;
    }
    const T* row = table + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) x[(size_t)n * D + d] = mb_load(row + d);
}


// the same with 128-bit accesses, for widths that are a multiple of 8
template <typename T>
__global__ void embed_vec_kernel(const int* __restrict__ tok, const T* __restrict__ table, float* __restrict__ x,
                                 int D, int V, int* err) {
    const int n = blockIdx.x;
    const int t = tok[n];
    const bool ok = t >= 0 && t < V;
    if (!ok && threadIdx.x == 0) mb_set_error(err, MB_ERR_TOKEN_RANGE);
    const T* row = table + (size_t)(ok ? t : 0) * D;
    for (int c = threadIdx.x; c < D / 8; c += blockDim.x) {
        float v[8];
        if (ok) load8(row + c * 8, v);
        else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.0f;
        }
        store8(x + (size_t)n * D + c * 8, v);
    }
}

// ------------------------------------------------------------------------------------------------ add + RMSNorm
// v = x[r] (+ delta[r] (+ dbias));  if rows == nullptr the sum is written back to x (the residual stream);
// out[i] = v * rsqrt(mean(v^2) + eps) * w.  r = rows ? rows[i] : i.  One block per output row.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ dbias,
                                   const int* __restrict__ rows, const float* __restrict__ w, float eps,
                                   T* __restrict__ out, int D) {
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float* xr = x + r * D;
    const T* dr = delta ? delta + r * D : nullptr;
    float ss = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = xr[d];
        if (dr) {
            float a = mb_load(dr + d);
            if (dbias) a += dbias[d];
            v += a;
            if (!rows) xr[d] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = mb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)D + eps);
    T* o = out + (size_t)i * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = xr[d];
        if (dr && rows) {
            float a = mb_load(dr + d);
            if (dbias) a += dbias[d];
            v += a;
        }
        mb_store(o + d, v * inv * w[d]);
    }
}


// The same for widths that are a multiple of 8 and at most 256 * 8 * NORM_MAX_CHUNKS: every thread keeps its values in
// registers between the two passes and all accesses are 128 bits wide.
#define NORM_MAX_CHUNKS 4
template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                             const float* __restrict__ dbias,
                                                             const int* __restrict__ rows, const float* __restrict__ w,
                                                             float eps, T* __restrict__ out, int D) {
    __shared__ float scratch[32];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float* xr = x + r * D;
    const T* dr = delta ? delta + r * D : nullptr;
    const int chunks = D / 8;
    float v[NORM_MAX_CHUNKS][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NORM_MAX_CHUNKS; j++) {
        const int c = threadIdx.x + j * 256;
        if (c < chunks) {
            load8(xr + c * 8, v[j]);
            if (dr) {
                float a[8];
                load8(dr + c * 8, a);
                if (dbias) {
                    float b[8];
                    load8(dbias + c * 8, b);
#pragma unroll
                    for (int e = 0; e < 8; e++) a[e] += b[e];
                }
#pragma unroll
                for (int e = 0; e < 8; e++) v[j][e] += a[e];
                if (!rows) store8(xr + c * 8, v[j]);
            }
#pragma unroll
            for (int e = 0; e < 8; e++) ss = fmaf(v[j][e], v[j][e], ss);
        }
    }
    ss = mb_block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)D + eps);
    T* o = out + (size_t)i * D;
#pragma unroll
    for (int j = 0; j < NORM_MAX_CHUNKS; j++) {
        const int c = threadIdx.x + j * 256;
        if (c < chunks) {
            float g[8];
            load8(w + c * 8, g);
#pragma unroll
            for (int e = 0; e < 8; e++) g[e] = v[j][e] * inv * g[e];
            store8(o + c * 8, g);
        }
    }
}

// ------------------------------------------------------------------------------------------------ rotation + K/V write
// qkv[n] = [q (H*HD) | k (KV*HD) | v (KV*HD)] (+ bias).  q is rotated in place; k is rotated and written to its page,
// v is written to its page (when pools are given).  freqs[i] is the angle per position step of pair i (RD/2 values);
// pairing 0 rotates (2i, 2i+1), pairing 1 rotates (i, i + RD/2); dims from RD on pass through.  freqs == nullptr
// means no rotation.  Page of position p of sequence s: table[s * max_blocks + p / page].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ bias,
                                     const int* __restrict__ positions, const int* __restrict__ tok_seq,
                                     const int* __restrict__ table, int max_blocks, T* __restrict__ kpool,
                                     T* __restrict__ vpool, const float* __restrict__ freqs, int H, int KV, int HD,
                                     int RD, int pairing, int page, int num_pages, int* err) {
    const int n = blockIdx.x;
    const int half = HD / 2, rhalf = RD / 2;
    const int per = blockDim.x / half;               // heads handled at once by one block; gridDim.y blocks share a token
    const int lane = threadIdx.x % half, sub = threadIdx.x / half;
    const int pos = positions[n];
    T* row = qkv + (size_t)n * (H + 2 * KV) * HD;
    const float* brow = bias;
    size_t slot = 0;
    bool store = kpool != nullptr;
    if (store) {
        const int pg = table[(size_t)tok_seq[n] * max_blocks + pos / page];
        if (pg < 0 || pg >= num_pages) {
            if (threadIdx.x == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            store = false;
        } else {
            slot = (size_t)pg * KV * page + (pos % page);       // + kvh * page, then * HD
        }
    }
    if (sub >= per) return;
    // the pair this thread owns inside every head: element indices e0, e1 and whether it is rotated
    int e0, e1;
    bool rot;
    if (pairing == 0) {
        e0 = 2 * lane; e1 = e0 + 1; rot = lane < rhalf;
    } else if (lane < rhalf) {
        e0 = lane; e1 = lane + rhalf; rot = true;
    } else {                                          // the passthrough dims RD .. HD-1, two per thread
        e0 = RD + 2 * (lane - rhalf); e1 = e0 + 1; rot = false;
    }
    float c = 1.0f, s = 0.0f;
    if (rot && freqs) {
        const float ang = (float)pos * freqs[lane];
        sincosf(ang, &s, &c);
    } else {
        rot = false;
    }
    for (int h = sub + blockIdx.y * per; h < H + 2 * KV; h += per * gridDim.y) {
        T* p = row + (size_t)h * HD;
        float a = mb_load(p + e0), b = mb_load(p + e1);
        if (brow) { a += brow[(size_t)h * HD + e0]; b += brow[(size_t)h * HD + e1]; }
        if (h < H + KV && rot) {
            const float ra = a * c - b * s, rb = a * s + b * c;
            a = ra; b = rb;
        }
        if (h < H) {
            mb_store(p + e0, a); mb_store(p + e1, b);
        } else if (store) {
            const int kvh = (h - H) % KV;
            T* pool = (h < H + KV) ? kpool : vpool;
            T* dst = pool + (slot + (size_t)kvh * page) * HD;
            mb_store(dst + e0, a); mb_store(dst + e1, b);
        }
    }
}

// The same for bf16 with eight values (16 bytes) per thread and the token's cosines and sines computed once per block:
// HD a multiple of 8, RD a multiple of 16.  A q head that is neither rotated nor biased is left alone; with the halves
// pairing a thread takes a chunk of the first half together with its partner chunk in the second.
__global__ void rope_kv_write_vec_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ bias,
                                         const int* __restrict__ positions, const int* __restrict__ tok_seq,
                                         const int* __restrict__ table, int max_blocks, __nv_bfloat16* __restrict__ kpool,
                                         __nv_bfloat16* __restrict__ vpool, const float* __restrict__ freqs, int H, int KV,
                                         int HD, int RD, int pairing, int page, int num_pages, int* err) {
    extern __shared__ float2 rope_cs[];                              // (cos, sin) of the token's RD/2 pairs
    // What comes before pdl_wait() reads the step's own arrays and the frequency table only (no kernel writes them) and
    // may run while the q/k/v product before this kernel still does; q, k and v are read after it, around the L1.
    pdl_launch_dependents();
    const int n = blockIdx.x, pos = positions[n];
    __nv_bfloat16* row = qkv + (size_t)n * (H + 2 * KV) * HD;
    size_t slot = 0;
    bool store = kpool != nullptr;
    if (store) {
        const int pg = table[(size_t)tok_seq[n] * max_blocks + pos / page];
        if (pg < 0 || pg >= num_pages) {
            if (threadIdx.x == 0 && blockIdx.y == 0) mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            store = false;
        } else {
            slot = (size_t)pg * KV * page + (pos % page);
        }
    }
    const bool rot = freqs != nullptr;
    if (rot) {
        for (int i = threadIdx.x; i < RD / 2; i += blockDim.x) {
            float s, c;
            sincosf((float)pos * freqs[i], &s, &c);
            rope_cs[i] = make_float2(c, s);
        }
        __syncthreads();
    }
    pdl_wait();
    const int cph = HD / 8, rhalf = RD / 2, total = (H + 2 * KV) * cph;
    for (int w = threadIdx.x + blockIdx.y * blockDim.x; w < total; w += blockDim.x * gridDim.y) {
        const int h = w / cph, e0 = (w % cph) * 8;
        const bool is_q = h < H, is_v = h >= H + KV;
        const bool rotates = rot && !is_v && e0 < RD;
        if (is_q ? (!rotates && !bias) : !store) continue;
        const bool paired = rotates && pairing == 1;
        if (paired && e0 >= rhalf) continue;                         // done by the thread of the partner chunk
        __nv_bfloat16* src = row + (size_t)h * HD + e0;
        __nv_bfloat16* dst = src;
        if (!is_q) dst = (is_v ? vpool : kpool) + (slot + (size_t)((h - H) % KV) * page) * HD + e0;
        float a[8], b[8];
        {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src));
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; i++) { const float2 x = __bfloat1622float2(p2[i]); a[2 * i] = x.x; a[2 * i + 1] = x.y; }
        }
        if (bias) {
#pragma unroll
            for (int i = 0; i < 8; i++) a[i] += bias[(size_t)h * HD + e0 + i];
        }
        if (paired) {
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + rhalf));
            const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int i = 0; i < 4; i++) { const float2 x = __bfloat1622float2(p2[i]); b[2 * i] = x.x; b[2 * i + 1] = x.y; }
            if (bias) {
#pragma unroll
                for (int i = 0; i < 8; i++) b[i] += bias[(size_t)h * HD + e0 + rhalf + i];
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float2 cs = rope_cs[e0 + i];
                const float ra = a[i] * cs.x - b[i] * cs.y, rb = a[i] * cs.y + b[i] * cs.x;
                a[i] = ra; b[i] = rb;
            }
            uint4 o;
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; i++) o2[i] = __floats2bfloat162_rn(b[2 * i], b[2 * i + 1]);
            *reinterpret_cast<uint4*>(dst + rhalf) = o;
        } else if (rotates) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 cs = rope_cs[e0 / 2 + i];
                const float ra = a[2 * i] * cs.x - a[2 * i + 1] * cs.y, rb = a[2 * i] * cs.y + a[2 * i + 1] * cs.x;
                a[2 * i] = ra; a[2 * i + 1] = rb;
            }
        }
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; i++) o2[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
        *reinterpret_cast<uint4*>(dst) = o;
    }
}

// ------------------------------------------------------------------------------------------------ token feedback
// dst[pairs[2i]] = src[pairs[2i + 1]]: the ids sampled in one step become input tokens of the next without a trip
// through the host (the next step is laid out and queued while this one still runs).
__global__ void patch_tokens_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ pairs, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[pairs[2 * i]] = src[pairs[2 * i + 1]];
}
MB_API int mb_patch_tokens(int* dst, const int* src, const int* pairs, int n, cudaStream_t st) {
    if (n <= 0) return 0;
    patch_tokens_kernel<<<(n + 127) / 128, 128, 0, st>>>(dst, src, pairs, n);
    MB_LAUNCH_CHECK();
    return 0;
}

// ------------------------------------------------------------------------------------------------ SwiGLU
// gu[n] = [gate (F) | up (F)] -> out[n, f] = silu(gate) * up
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t n = i / F, f = i % F;
    const float g = mb_load(gu + n * 2 * F + f), u = mb_load(gu + n * 2 * F + F + f);
    mb_store(out + i, (g / (1.0f + expf(-g))) * u);
}


// the same, eight values per thread, for F a multiple of 8: block (x: chunks of a row), grid.y: rows
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int F) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= F / 8) return;
    const size_t n = blockIdx.y;
    float g[8], u[8];
    load8(gu + n * 2 * F + c * 8, g);
    load8(gu + n * 2 * F + F + c * 8, u);
#pragma unroll
    for (int e = 0; e < 8; e++) g[e] = (g[e] / (1.0f + expf(-g[e]))) * u[e];
    store8(out + n * F + c * 8, g);
}

// ------------------------------------------------------------------------------------------------ launchers
template <typename T>
static int embed_launch(const int* tok, const void* table, float* x, int N, int D, int V, int* err, cudaStream_t st) {
    if (N == 0) return 0;
    if (D % 8 == 0) embed_vec_kernel<T><<<N, 128, 0, st>>>(tok, (const T*)table, x, D, V, err);
    else embed_kernel<T><<<N, 256, 0, st>>>(tok, (const T*)table, x, D, V, err);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_embed_f32(const int* tok, const void* table, float* x, int N, int D, int V, int* err, cudaStream_t st) {
    return embed_launch<float>(tok, table, x, N, D, V, err, st);
}
MB_API int mb_embed_bf16(const int* tok, const void* table, float* x, int N, int D, int V, int* err, cudaStream_t st) {
    return embed_launch<__nv_bfloat16>(tok, table, x, N, D, V, err, st);
}

template <typename T>
static int add_rmsnorm_launch(float* x, const void* delta, const float* dbias, const int* rows, const float* w,
                              float eps, void* out, int n_out, int D, cudaStream_t st) {
    if (n_out == 0) return 0;
    if (D % 8 == 0 && D <= 256 * 8 * NORM_MAX_CHUNKS)
        add_rmsnorm_vec_kernel<T><<<n_out, 256, 0, st>>>(x, (const T*)delta, dbias, rows, w, eps, (T*)out, D);
    else
        add_rmsnorm_kernel<T><<<n_out, 256, 0, st>>>(x, (const T*)delta, dbias, rows, w, eps, (T*)out, D);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_add_rmsnorm_f32(float* x, const void* delta, const float* dbias, const int* rows, const float* w,
                              float eps, void* out, int n_out, int D, cudaStream_t st) {
    return add_rmsnorm_launch<float>(x, delta, dbias, rows, w, eps, out, n_out, D, st);
}
MB_API int mb_add_rmsnorm_bf16(float* x, const void* delta, const float* dbias, const int* rows, const float* w,
                               float eps, void* out, int n_out, int D, cudaStream_t st) {
    return add_rmsnorm_launch<__nv_bfloat16>(x, delta, dbias, rows, w, eps, out, n_out, D, st);
}

MB_PDL_SWITCH(mb_elementwise_set_pdl)

template <typename T>
static int rope_kv_write_launch(void* qkv, const float* bias, const int* positions, const int* tok_seq,
                                const int* table, int max_blocks, void* kpool, void* vpool, const float* freqs, int N,
                                int H, int KV, int HD, int RD, int pairing, int page, int num_pages, int* err,
                                cudaStream_t st) {
    if (N == 0) return 0;
    if (HD % 2 || RD % 2 || RD > HD || HD / 2 > 1024) return -2;
    if (sizeof(T) == 2 && HD % 8 == 0 && RD % 16 == 0 && N <= 0x7fffffff / ((H + 2 * KV) * HD) &&
        (((uintptr_t)qkv | (uintptr_t)kpool | (uintptr_t)vpool) & 15) == 0) {
        const int items = (H + 2 * KV) * (HD / 8);
        int split = N >= 512 ? 1 : (items + 255) / 256;
        if (split > 16) split = 16;
        const cudaError_t e = mb_launch(mb_pdl != 0, rope_kv_write_vec_kernel, dim3(N, split), dim3(256),
                                        (RD / 2) * sizeof(float2), st, (__nv_bfloat16*)qkv, bias, positions, tok_seq, table,
                                        max_blocks, (__nv_bfloat16*)kpool, (__nv_bfloat16*)vpool, freqs, H, KV, HD, RD,
                                        pairing, page, num_pages, err);
        return e == cudaSuccess ? 0 : (int)e;
    }
    int threads = 256;
    if (HD / 2 > threads) threads = ((HD / 2 + 31) / 32) * 32;
    const int per = threads / (HD / 2);
    int split = (H + 2 * KV + per - 1) / per;       // blocks per token: enough to fill the GPU when tokens are few
    if (split > 16) split = 16;
    if (N >= 512) split = 1;
    rope_kv_write_kernel<T><<<dim3(N, split), threads, 0, st>>>((T*)qkv, bias, positions, tok_seq, table, max_blocks, (T*)kpool,
                                                    (T*)vpool, freqs, H, KV, HD, RD, pairing, page, num_pages, err);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_rope_kv_write_f32(void* qkv, const float* bias, const int* positions, const int* tok_seq,
                                const int* table, int max_blocks, void* kpool, void* vpool, const float* freqs, int N,
                                int H, int KV, int HD, int RD, int pairing, int page, int num_pages, int* err,
                                cudaStream_t st) {
    return rope_kv_write_launch<float>(qkv, bias, positions, tok_seq, table, max_blocks, kpool, vpool, freqs, N, H, KV,
                                       HD, RD, pairing, page, num_pages, err, st);
}
MB_API int mb_rope_kv_write_bf16(void* qkv, const float* bias, const int* positions, const int* tok_seq,
                                 const int* table, int max_blocks, void* kpool, void* vpool, const float* freqs, int N,
                                 int H, int KV, int HD, int RD, int pairing, int page, int num_pages, int* err,
                                 cudaStream_t st) {
    return rope_kv_write_launch<__nv_bfloat16>(qkv, bias, positions, tok_seq, table, max_blocks, kpool, vpool, freqs,
                                               N, H, KV, HD, RD, pairing, page, num_pages, err, st);
}

template <typename T>
static int swiglu_launch(const void* gu, void* out, int N, int F, cudaStream_t st) {
    const size_t total = (size_t)N * F;
    if (total == 0) return 0;
    if (F % 8 == 0 && N <= 65535)
        swiglu_vec_kernel<T><<<dim3((F / 8 + 127) / 128, N), 128, 0, st>>>((const T*)gu, (T*)out, F);
    else
        swiglu_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)gu, (T*)out, F, total);
    MB_LAUNCH_CHECK();
    return 0;
}
MB_API int mb_swiglu_f32(const void* gu, void* out, int N, int F, cudaStream_t st) {
    return swiglu_launch<float>(gu, out, N, F, st);
}
MB_API int mb_swiglu_bf16(const void* gu, void* out, int N, int F, cudaStream_t st) {
    return swiglu_launch<__nv_bfloat16>(gu, out, N, F, st);
}
