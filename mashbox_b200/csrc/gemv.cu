// Matrix-vector products for decode steps with at most 4 tokens: out[n, m] = sum_k act[n, k] * W[m, k].
//
// With one to four tokens the product is a pure stream of W and needs no tensor core: a warp owns two rows of W from
// end to end, each lane reads 16 bytes of both rows at a time (four chunks ahead), multiplies them with the matching
// 16 bytes of every token's activations (read through L1) in float32, and one shuffle tree per (row, token) finishes
// the sums.  No shared memory, no partial sums across blocks: 2,048 independent warps for a 4,096-row matrix, so every
// SM has loads in flight all the time.  A token's result does not depend on how many tokens share the call.
//
// Modes: plain (bf16 out), float32 out (the output head), SwiGLU (W = [gate rows | up rows]: a warp takes a gate row and
// the up row of the same feature and writes silu(gate) * up).  K must be a multiple of 8.
#include "common.cuh"

typedef __nv_bfloat16 bf16;

#define GV_WARPS 8
#define GV_ROWS 2
#define GV_MAX_TOKENS 4

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float dot8(const uint4& w, const uint4& x, float acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        acc = fmaf(__uint_as_float(wv[i] << 16), __uint_as_float(xv[i] << 16), acc);
        acc = fmaf(__uint_as_float(wv[i] & 0xffff0000u), __uint_as_float(xv[i] & 0xffff0000u), acc);
    }
    return acc;
}

// What a decode step of one token is made of beside the products is folded into them, so that a layer is six kernels
// instead of ten:
//   NORM   the activations are not read but made: every block normalises the token's row of the float32 residual
//          stream (x * rsqrt(mean(x^2) + eps) * w, as the norm kernel does, rounded to bf16) into shared memory once
//          and then walks its share of the rows of W;
//   MODE 3 the product is added into the float32 residual stream in place (plus a bias), every element by the one
//          thread that owns it.
struct GemvNorm { const float* x; const float* w; float eps; };

// MODE 4: the rows of W are the q, k and v heads of an attention layer.  The product's epilogue is the rotate-and-store
// step: bias, rotation of the q and k heads by the token's position, q into the output, k and v into their cache pages.
// A warp takes the two rows of a rotated pair, so the pair meets in one lane.
struct GemvRope {
    const int* positions; const int* tok_row; const int* table; int max_blocks;
    bf16* kpool; bf16* vpool; const float* freqs; const float* bias;
    int H, KV, HD, RD, pairing, page, num_pages;
    int* err;
};

// The activations: from global memory, or from the block's shared memory.  What the kernel before this one wrote (the
// activations, the residual stream) is read around the L1 (ld.global.cg): launched with the programmatic-serialization
// attribute this kernel's blocks may be resident before that kernel has finished, and an SM's L1 may hold lines of its
// output from before it was complete.
template <bool SHARED> __device__ __forceinline__ uint4 gv_act(const bf16* p) {
    return *reinterpret_cast<const uint4*>(p);
}

__device__ __forceinline__ void gv_load8(const float* p, float (&v)[8]) {                 // a norm's weight
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void gv_load8_stream(const float* p, float (&v)[8]) {          // the residual stream
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p)), b = __ldcg(reinterpret_cast<const float4*>(p + 4));
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// NT tokens (1..4).  MODE 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out; 3: out is
// the float32 residual stream (N, M), added to.
template <int NT, int MODE, int PRE>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_kernel(const bf16* __restrict__ act, const bf16* __restrict__ W,
                                                             void* __restrict__ out, int M, int K, GemvNorm nrm,
                                                             const float* __restrict__ bias, GemvRope rope) {
    extern __shared__ __align__(16) unsigned char gv_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // The q/k/v products let the kernel after them start at once: the attention kernel, launched with the
    // programmatic-serialization attribute, fetches its first cached keys and values while this product still runs
    // (and waits for it by itself before it reads what it writes): a one-token step of the 8B shape at 8,192 tokens of
    // context 3.26 against 3.31 ms.  (These kernels themselves are launched plainly: see below.)
    if (MODE == 0 || MODE == 4) pdl_launch_dependents();
    // These kernels are launched plainly.  With the programmatic-serialization attribute (wait at the top, dependents
    // let go at the start or at the end of a block's work) a one-token step of the 8B shape took 4.3 ms against 3.7
    // ms.  Tried again with the L2 asked for the first 4 KB of every warp's rows before the wait: one request on the
    // 1B shape 1,399 against 1,378 tokens/s, on the 3B shape 535 against 605, on the 8B shape 286 against 328 (blocks
    // that are resident early take the places of blocks of the kernel that is still running).
    constexpr bool NORM = PRE == 1;
    if (PRE == 2) {
        // the activations once per block into shared memory (16 bytes a thread and turn), instead of once per warp from
        // the L2
        bf16* hs = reinterpret_cast<bf16*>(gv_smem);
        for (int c = threadIdx.x; c < NT * (K / 8); c += GV_WARPS * 32)
            *reinterpret_cast<uint4*>(hs + (size_t)c * 8) = *reinterpret_cast<const uint4*>(act + (size_t)c * 8);
        __syncthreads();
        act = hs;
    }
    if (NORM) {
        __shared__ float scratch[32];
        bf16* hs = reinterpret_cast<bf16*>(gv_smem);                 // [NT][K]
        const int chunks8 = K / 8;
#pragma unroll
        for (int n = 0; n < NT; n++) {
            float v[4][8];                                           // K <= 8,192: at most four chunks of eight per thread
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int c = threadIdx.x + j * GV_WARPS * 32;
                if (c < chunks8) {
                    gv_load8_stream(nrm.x + (size_t)n * K + c * 8, v[j]);
#pragma unroll
                    for (int e = 0; e < 8; e++) ss = fmaf(v[j][e], v[j][e], ss);
                }
            }
            ss = mb_block_sum(ss, scratch);
            const float inv = rsqrtf(ss / (float)K + nrm.eps);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int c = threadIdx.x + j * GV_WARPS * 32;
                if (c < chunks8) {
                    float g[8];
                    gv_load8(nrm.w + c * 8, g);
                    uint4 o;
                    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __nv_bfloat162 p = __floats2bfloat162_rn(v[j][2 * e] * inv * g[2 * e], v[j][2 * e + 1] * inv * g[2 * e + 1]);
                        ow[e] = *reinterpret_cast<const uint32_t*>(&p);
                    }
                    *reinterpret_cast<uint4*>(hs + (size_t)n * K + c * 8) = o;
                }
            }
        }
        __syncthreads();
        act = hs;
    }
    const int units = MODE == 1 ? M : (M + GV_ROWS - 1) / GV_ROWS;
    for (int unit = blockIdx.x * GV_WARPS + warp; unit < units; unit += gridDim.x * GV_WARPS) {
    int m0 = MODE == 1 ? unit : unit * GV_ROWS;                     // MODE 1: one feature (two rows); else two rows
    int m1 = MODE == 1 ? M + m0 : min(m0 + 1, M - 1);
    int pair = 0;                                                    // MODE 4: index of the rotated pair, -1: not rotated
    if (MODE == 4) {
        const int hh = rope.HD / 2, rh = rope.RD / 2, head = unit / hh, i = unit % hh;
        int e0, e1;
        if (rope.pairing == 0) { e0 = 2 * i; e1 = e0 + 1; pair = i < rh ? i : -1; }
        else if (i < rh) { e0 = i; e1 = i + rh; pair = i; }
        else { e0 = rope.RD + 2 * (i - rh); e1 = e0 + 1; pair = -1; }
        m0 = head * rope.HD + e0;
        m1 = head * rope.HD + e1;
    }
    const bf16* rows[GV_ROWS];
    rows[0] = W + (size_t)m0 * K;
    rows[1] = W + (size_t)m1 * K;
    float acc[GV_ROWS][NT];
#pragma unroll
    for (int r = 0; r < GV_ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) acc[r][n] = 0.0f;
    // MODE 3: the stream's old values are sent for before the rows of W.  Asked for at the end, behind everything the
    // other warps have in flight, they took 6 us to arrive (a 2,048 x 2,048 product: 11.6 us against 5.8 for the plain
    // form).
    float old[GV_ROWS][NT];
    if (MODE == 3 && lane == 0) {
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++)
#pragma unroll
            for (int n = 0; n < NT; n++)
                old[r][n] = m0 + r < M ? __ldcg(reinterpret_cast<const float*>(out) + (size_t)n * M + m0 + r) : 0.0f;
    }
    const int chunks = K / 8;
    int c = lane;
    // eight chunks of both rows ahead (16 loads of 16 bytes in flight per lane): with four, a matrix of long rows
    // (K = 14,336) streamed at half the rate of one with short rows
    for (; c + 224 < chunks; c += 256) {
        uint4 w[8][GV_ROWS];
#pragma unroll
        for (int u = 0; u < 8; u++)
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) w[u][r] = ld_stream16(rows[r] + (size_t)(c + 32 * u) * 8);
#pragma unroll
        for (int u = 0; u < 8; u++)
#pragma unroll
            for (int n = 0; n < NT; n++) {
                const uint4 x = gv_act<PRE != 0>(act + (size_t)n * K + (size_t)(c + 32 * u) * 8);
#pragma unroll
                for (int r = 0; r < GV_ROWS; r++) acc[r][n] = dot8(w[u][r], x, acc[r][n]);
            }
    }
    for (; c + 96 < chunks; c += 128) {
        uint4 w[4][GV_ROWS];
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) w[u][r] = ld_stream16(rows[r] + (size_t)(c + 32 * u) * 8);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int n = 0; n < NT; n++) {
                const uint4 x = gv_act<PRE != 0>(act + (size_t)n * K + (size_t)(c + 32 * u) * 8);
#pragma unroll
                for (int r = 0; r < GV_ROWS; r++) acc[r][n] = dot8(w[u][r], x, acc[r][n]);
            }
    }
    for (; c < chunks; c += 32) {
        uint4 w[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++) w[r] = ld_stream16(rows[r] + (size_t)c * 8);
#pragma unroll
        for (int n = 0; n < NT; n++) {
            const uint4 x = gv_act<PRE != 0>(act + (size_t)n * K + (size_t)c * 8);
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) acc[r][n] = dot8(w[r], x, acc[r][n]);
        }
    }
#pragma unroll
    for (int r = 0; r < GV_ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) acc[r][n] = mb_warp_sum(acc[r][n]);
    if (lane != 0) continue;
#pragma unroll
    for (int n = 0; n < NT; n++) {
        if (MODE == 4) {
            // as the separate kernels do it: the product rounded to bf16, then bias and rotation in float, then bf16
            float a = __bfloat162float(__float2bfloat16_rn(acc[0][n])), b = __bfloat162float(__float2bfloat16_rn(acc[1][n]));
            if (rope.bias) { a += rope.bias[m0]; b += rope.bias[m1]; }
            const int head = m0 / rope.HD, pos = rope.positions[n];
            if (pair >= 0 && rope.freqs && head < rope.H + rope.KV) {
                float s, c;
                sincosf((float)pos * rope.freqs[pair], &s, &c);
                const float ra = a * c - b * s, rb = a * s + b * c;
                a = ra; b = rb;
            }
            if (head < rope.H) {
                reinterpret_cast<bf16*>(out)[(size_t)n * M + m0] = __float2bfloat16_rn(a);
                reinterpret_cast<bf16*>(out)[(size_t)n * M + m1] = __float2bfloat16_rn(b);
            } else if (rope.kpool) {
                const int pg = rope.table[(size_t)rope.tok_row[n] * rope.max_blocks + pos / rope.page];
                if (pg < 0 || pg >= rope.num_pages) {
                    mb_set_error(rope.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
                } else {
                    const int kvh = (head - rope.H) % rope.KV;
                    bf16* pool = head < rope.H + rope.KV ? rope.kpool : rope.vpool;
                    bf16* dst = pool + (((size_t)pg * rope.KV + kvh) * rope.page + pos % rope.page) * rope.HD;
                    dst[m0 % rope.HD] = __float2bfloat16_rn(a);
                    dst[m1 % rope.HD] = __float2bfloat16_rn(b);
                }
            }
        } else if (MODE == 1) {
            // gate and up pass through bf16 as they do when the products are separate kernels
            const float g = __bfloat162float(__float2bfloat16_rn(acc[0][n])), up = __bfloat162float(__float2bfloat16_rn(acc[1][n]));
            reinterpret_cast<bf16*>(out)[(size_t)n * M + m0] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * up);
        } else {
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) {
                if (m0 + r >= M) continue;
                if (MODE == 3) {
                    float* xo = reinterpret_cast<float*>(out) + (size_t)n * M + m0 + r;
                    *xo = old[r][n] + (acc[r][n] + (bias ? bias[m0 + r] : 0.0f));
                }
                else if (MODE == 2) reinterpret_cast<float*>(out)[(size_t)n * M + m0 + r] = acc[r][n];
                else reinterpret_cast<bf16*>(out)[(size_t)n * M + m0 + r] = __float2bfloat16_rn(acc[r][n]);
            }
        }
    }
    }   // units
}

// The same product for matrices of long rows (K >= GV_LONG_K): the eight warps of a block share two rows, warp w
// taking the 512-byte pieces w, w + 8, ... of both, so a block reads 4 KB of a row at a time and the number of rows in
// flight is an eighth; the warps' partial sums meet in shared memory.  (With a warp per pair of rows a 4,096 x 14,336
// matrix streamed at 3.8 TB/s against 6 TB/s for 28,672 x 4,096.)
template <int NT, int MODE>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_long_kernel(const bf16* __restrict__ act, const bf16* __restrict__ W,
                                                                  void* __restrict__ out, int M, int K,
                                                                  const float* __restrict__ bias) {
    __shared__ float part[GV_WARPS][GV_ROWS][NT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x;
    const int m0 = MODE == 1 ? unit : unit * GV_ROWS;
    const bf16* rows[GV_ROWS];
    rows[0] = W + (size_t)m0 * K;
    rows[1] = MODE == 1 ? W + (size_t)(M + m0) * K : W + (size_t)min(m0 + 1, M - 1) * K;
    float acc[GV_ROWS][NT];
#pragma unroll
    for (int r = 0; r < GV_ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) acc[r][n] = 0.0f;
    // MODE 3: the stream's old value of the thread that will write it, sent for before the rows of W (see gemv_kernel)
    float old = 0.0f;
    if (MODE == 3 && threadIdx.x < GV_ROWS * NT && m0 + threadIdx.x / NT < M)
        old = __ldcg(reinterpret_cast<const float*>(out) + (size_t)(threadIdx.x % NT) * M + m0 + threadIdx.x / NT);
    const int chunks = K / 8;
    constexpr int STEP = GV_WARPS * 32;
    int c = warp * 32 + lane;
    for (; c + 3 * STEP < chunks; c += 4 * STEP) {
        uint4 w[4][GV_ROWS];
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) w[u][r] = ld_stream16(rows[r] + (size_t)(c + STEP * u) * 8);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int n = 0; n < NT; n++) {
                const uint4 x = *(reinterpret_cast<const uint4*>(act + (size_t)n * K + (size_t)(c + STEP * u) * 8));
#pragma unroll
                for (int r = 0; r < GV_ROWS; r++) acc[r][n] = dot8(w[u][r], x, acc[r][n]);
            }
    }
    for (; c < chunks; c += STEP) {
        uint4 w[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++) w[r] = ld_stream16(rows[r] + (size_t)c * 8);
#pragma unroll
        for (int n = 0; n < NT; n++) {
            const uint4 x = *(reinterpret_cast<const uint4*>(act + (size_t)n * K + (size_t)c * 8));
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) acc[r][n] = dot8(w[r], x, acc[r][n]);
        }
    }
#pragma unroll
    for (int r = 0; r < GV_ROWS; r++)
#pragma unroll
        for (int n = 0; n < NT; n++) {
            const float s = mb_warp_sum(acc[r][n]);
            if (lane == 0) part[warp][r][n] = s;
        }
    __syncthreads();
    if (threadIdx.x >= GV_ROWS * NT) return;
    const int r = threadIdx.x / NT, n = threadIdx.x % NT;
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < GV_WARPS; w++) s += part[w][r][n];            // a fixed order: the result does not depend on timing
    if (MODE == 1) {
        part[0][r][n] = s;
        __syncwarp();
        if (r == 0) {
            const float g = __bfloat162float(__float2bfloat16_rn(part[0][0][n])), up = __bfloat162float(__float2bfloat16_rn(part[0][1][n]));
            reinterpret_cast<bf16*>(out)[(size_t)n * M + m0] = __float2bfloat16_rn((g / (1.0f + expf(-g))) * up);
        }
    } else if (m0 + r < M) {
        if (MODE == 3) {
            float* xo = reinterpret_cast<float*>(out) + (size_t)n * M + m0 + r;
            *xo = old + (s + (bias ? bias[m0 + r] : 0.0f));
        }
        else if (MODE == 2) reinterpret_cast<float*>(out)[(size_t)n * M + m0 + r] = s;
        else reinterpret_cast<bf16*>(out)[(size_t)n * M + m0 + r] = __float2bfloat16_rn(s);
    }
}

#define GV_LONG_K 8192

template <int MODE, bool NORM>
static int gemv_launch(const void* act, const void* W, void* out, int N, int M, int K, GemvNorm nrm, const float* bias,
                       cudaStream_t st, GemvRope rope = GemvRope{}) {
    if (N == 0 || M == 0) return 0;
    if (N > GV_MAX_TOKENS || K % 8 || K < 8 || (reinterpret_cast<uintptr_t>(W) & 15) ||
        (!NORM && (reinterpret_cast<uintptr_t>(act) & 15)))
        return -2;
    const int units = MODE == 1 ? M : (M + GV_ROWS - 1) / GV_ROWS;
    const bf16* a = (const bf16*)act;
    const bf16* w = (const bf16*)W;
    if (K >= GV_LONG_K) {
        if (NORM || MODE == 4) return -2;                            // the normalised row is kept for K < GV_LONG_K only
        const unsigned g2 = (unsigned)units;
        cudaError_t le = cudaSuccess;
        switch (N) {
            case 1: le = mb_launch(false, gemv_long_kernel<1, MODE>, dim3(g2), dim3(GV_WARPS * 32), 0, st, a, w, out, M, K, bias); break;
            case 2: le = mb_launch(false, gemv_long_kernel<2, MODE>, dim3(g2), dim3(GV_WARPS * 32), 0, st, a, w, out, M, K, bias); break;
            case 3: le = mb_launch(false, gemv_long_kernel<3, MODE>, dim3(g2), dim3(GV_WARPS * 32), 0, st, a, w, out, M, K, bias); break;
            default: le = mb_launch(false, gemv_long_kernel<4, MODE>, dim3(g2), dim3(GV_WARPS * 32), 0, st, a, w, out, M, K, bias); break;
        }
        return le == cudaSuccess ? 0 : (int)le;
    }
    unsigned grid = (unsigned)((units + GV_WARPS - 1) / GV_WARPS);
    size_t smem = 0;
    // without a norm: the activations are copied into shared memory once per block when they fit, else read from global
    const bool copy = !NORM && (size_t)N * K * sizeof(bf16) <= 48 * 1024;
    if (NORM || copy) {
        // every block makes (or copies) the rows once: a few blocks per SM that walk the rows of W, not one block per
        // 16 rows
        if (NORM && ((reinterpret_cast<uintptr_t>(nrm.x) & 15) || (reinterpret_cast<uintptr_t>(nrm.w) & 15))) return -2;
        smem = (size_t)N * K * sizeof(bf16);
        if (smem > 48 * 1024) return -2;
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        if (grid > (unsigned)(4 * sms)) grid = (unsigned)(4 * sms);
    }
    cudaError_t le = cudaSuccess;
#define GV_GO(NT_, PRE_) le = mb_launch(false, gemv_kernel<NT_, MODE, PRE_>, dim3(grid), dim3(GV_WARPS * 32), smem, st, a, w, out, M, K, nrm, bias, rope)
#define GV_PRE(NT_) do { if (NORM) GV_GO(NT_, 1); else if (copy) GV_GO(NT_, 2); else GV_GO(NT_, 0); } while (0)
    switch (N) {
        case 1: GV_PRE(1); break;
        case 2: GV_PRE(2); break;
        case 3: GV_PRE(3); break;
        default: GV_PRE(4); break;
    }
#undef GV_PRE
#undef GV_GO
    return le == cudaSuccess ? 0 : (int)le;
}

MB_API int mb_gemv_bf16(const void* act, const void* W, void* out, int N, int M, int K, cudaStream_t st) {
    return gemv_launch<0, false>(act, W, out, N, M, K, GemvNorm{nullptr, nullptr, 0.0f}, nullptr, st);
}
MB_API int mb_gemv_swiglu_bf16(const void* act, const void* W, void* out, int N, int M, int K, cudaStream_t st) {
    return gemv_launch<1, false>(act, W, out, N, M, K, GemvNorm{nullptr, nullptr, 0.0f}, nullptr, st);
}
MB_API int mb_gemv_f32out(const void* act, const void* W, void* out, int N, int M, int K, cudaStream_t st) {
    return gemv_launch<2, false>(act, W, out, N, M, K, GemvNorm{nullptr, nullptr, 0.0f}, nullptr, st);
}
// x (N, M) float32 += act W^T + bias (bias may be null)
MB_API int mb_gemv_residual(const void* act, const void* W, float* x, const float* bias, int N, int M, int K, cudaStream_t st) {
    return gemv_launch<3, false>(act, W, x, N, M, K, GemvNorm{nullptr, nullptr, 0.0f}, bias, st);
}
// out = rmsnorm(x; norm_w, eps) W^T, x (N, K) float32; the SwiGLU form as mb_gemv_swiglu_bf16.  K < 8,192.
MB_API int mb_gemv_normed_bf16(const float* x, const float* norm_w, float eps, const void* W, void* out, int N, int M,
                               int K, cudaStream_t st) {
    return gemv_launch<0, true>(nullptr, W, out, N, M, K, GemvNorm{x, norm_w, eps}, nullptr, st);
}
MB_API int mb_gemv_normed_swiglu_bf16(const float* x, const float* norm_w, float eps, const void* W, void* out, int N,
                                      int M, int K, cudaStream_t st) {
    return gemv_launch<1, true>(nullptr, W, out, N, M, K, GemvNorm{x, norm_w, eps}, nullptr, st);
}
// out (N, M) = the q part of rmsnorm(x) W^T + bias, rotated; the k and v parts go rotated / as they are into the pages
// of the tokens' positions (kpool null: they are dropped).  M = (H + 2 KV) HD, K < 8,192.
MB_API int mb_gemv_normed_qkv_bf16(const float* x, const float* norm_w, float eps, const void* W, void* out, int N, int M,
                                   int K, const float* bias, const int* positions, const int* tok_row, const int* table,
                                   int max_blocks, void* kpool, void* vpool, const float* freqs, int H, int KV, int HD,
                                   int RD, int pairing, int page, int num_pages, int* err, cudaStream_t st) {
    if (HD % 2 || RD % 2 || RD > HD || M != (H + 2 * KV) * HD || page < 1) return -2;
    GemvRope r;
    r.positions = positions; r.tok_row = tok_row; r.table = table; r.max_blocks = max_blocks;
    r.kpool = (bf16*)kpool; r.vpool = (bf16*)vpool; r.freqs = freqs; r.bias = bias;
    r.H = H; r.KV = KV; r.HD = HD; r.RD = RD; r.pairing = pairing; r.page = page; r.num_pages = num_pages; r.err = err;
    return gemv_launch<4, true>(nullptr, W, out, N, M, K, GemvNorm{x, norm_w, eps}, nullptr, st, r);
}
