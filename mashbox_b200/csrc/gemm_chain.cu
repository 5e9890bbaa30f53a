// A chain of weight-streaming products (the forms of gemm_stream.cu: at most 16 tokens, bound by reading W once) in
// ONE launch: product p + 1 reads what product p wrote, so between two products every block passes a grid-wide
// barrier, but the weights of product p + 1 -- which no kernel writes -- are sent for as soon as the stages of the
// ring come free, while the block finishes product p, meets the others and fetches the new activations.
//
// Why: a decode step is a chain of such products, each a few to 40 us long, and between two launches an SM idles for
// 3 to 4 us (its block ends, the next kernel's block starts, sets itself up, and its first bytes arrive 2 us later),
// even with programmatic dependent launch, because a streaming block takes the SM's whole shared memory and its
// successor cannot be resident beside it.  Here the ring never runs dry: the epilogue of product p, the barrier and
// the first activations of product p + 1 take about 3 us, during which up to 200 KB of the next weights arrive.
//
// Every product is cut as gemm_stream.cu cuts it when there are no more row tiles than SMs: a block per row tile of TH
// rows (128, 64 or 32), all of K; products that would need shared tiles are refused (they are launched by
// themselves).  The grid is the largest number of tiles of a product; a block without a tile in a product only takes
// part in the barriers.  All blocks are resident at once (one per SM by shared memory, at most as many as SMs), which
// the barrier needs; the kernel after this one is launched only when every block has started.
//
// The barrier: a counter and a generation in global memory.  One consumer thread per block adds 1 to the counter
// (acq_rel) after the block's stores; the block that brings it to G x (p + 1) adds 1 to the generation (release; after
// the last barrier of a launch it sets the counter back to 0 first).  Who waits reads the generation (acquire) until it
// has grown by p + 1 since the kernel started; every wait has an iteration limit, after which the error word is set and
// the thread goes on.  Data that another block wrote is read by TMA (after fence.proxy.async) or ld.global.cg.
//
// Roles of the 192 threads as in gemm_stream.cu: warp 0 producer, warps 1-4 consumers (ldmatrix + mma.sync m16n8k16),
// warp 5 the 1 / rms of products of a normalised stream.  The stage size differs from product to product; the
// mbarriers of the ring keep their phases across products, and the producer lays the first stages of a product over
// those of the one before only where the consumers have left them.
#include <cstring>
#include "gemm_stream.cuh"

#define C_MAX 4                                            // products in one launch
#define C_MEET (16 * 1024)                                 // where the consumer warps' sums meet (the largest form)
#define C_SMALL 1024                                       // barriers, flags, 1 / rms, warp sums
#define C_RING (S_SMEM - 1024 - C_SMALL - C_MEET)          // bytes of the ring of stages
#define C_MAX_STAGES 6
#define C_SPIN_LIMIT (1 << 22)

struct ChainProduct {
    CUtensorMap wmap, xmap;
    void* out;
    const float* bias;
    StreamNorm nrm;
    StreamAfter after;
    int N, M, K, tiles, kind;                              // kind = EPI * 6 + SCALED * 3 + (0: TH 32, 1: 64, 2: 128)
};
struct ChainArgs {
    ChainProduct prod[C_MAX];
    int n;
    int* sync;                                             // [0] arrivals of this launch, [1] generation
    int* err;
};

template <int EPI, int TH> struct ChainShape : StreamShape<EPI, TH> {
    using B = StreamShape<EPI, TH>;
    static constexpr int FIT_C = C_RING / B::STAGE;
    static constexpr int STAGES_C = FIT_C > C_MAX_STAGES ? C_MAX_STAGES : FIT_C;
    static_assert(STAGES_C >= 2, "a ring of at least two stages");
    static_assert(B::RED <= C_MEET, "the meeting area holds the largest form");
};

// where the ring stands, carried from product to product
struct ChainPipe {
    uint32_t fpar = 0;                  // consumers: parity of the next completion of full[s], bit s
    uint32_t epar = 0;                  // producer: parity of the next completion of empty[s], bit s
    uint32_t pend = 0, pend_old = 0;    // producer: stages filled whose emptying it has not waited for (this product's / the one before's)
    int old_stage = 0;                  // stage size of the product before
};

__device__ __forceinline__ bool chain_wait(const int* gen, int gen0, int n, int* err) {
    for (int it = 0; it < C_SPIN_LIMIT; it++) {
        int g;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(g) : "l"(gen) : "memory");
        if (g - gen0 >= n) return true;
        __nanosleep(32);
    }
    mb_set_error(err, MB_ERR_WAIT_TIMEOUT);
    return false;
}

// one thread of a block, after the block's stores have been fenced: arrival at barrier p of n_bar
__device__ __forceinline__ void chain_arrive(int* sync, int p, int n_bar, int G) {
    asm volatile("fence.proxy.async.global;\n" ::: "memory");
    int before;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;\n" : "=r"(before) : "l"(sync) : "memory");
    if (before == G * (p + 1) - 1) {
        if (p == n_bar - 1) asm volatile("st.relaxed.gpu.global.s32 [%0], %1;\n" ::"l"(sync), "r"(0) : "memory");
        asm volatile("red.release.gpu.global.add.s32 [%0], 1;\n" ::"l"(sync + 1) : "memory");
    }
}

// the producer waits until nothing lies any more where stage s of a product with stages of STAGE bytes goes
template <int STAGE>
__device__ __forceinline__ bool chain_free_stage(ChainPipe& pp, int s, uint32_t empty0, int* err) {
    uint32_t need = (pp.pend | pp.pend_old) & (1u << s);
    if (pp.pend_old) {
        const int lo = s * STAGE, hi = lo + STAGE;
#pragma unroll
        for (int i = 0; i < C_MAX_STAGES; i++)
            if (((pp.pend_old >> i) & 1) && i * pp.old_stage < hi && (i + 1) * pp.old_stage > lo) need |= 1u << i;
    }
    if (need) {
#pragma unroll
        for (int i = 0; i < C_MAX_STAGES; i++)
            if ((need >> i) & 1) {
                if (!mbar_wait(empty0 + 8 * i, (pp.epar >> i) & 1, err)) return false;
                pp.epar ^= 1u << i;
            }
        pp.pend &= ~need;
        pp.pend_old &= ~need;
    }
    return true;
}

// the TMA copies of item `it` of the block's tile: the weights (WHAT = 1), the activations that go with them (2), or both
template <int EPI, int TH, int WHAT>
__device__ __forceinline__ void chain_copies(const CUtensorMap* wmap, const CUtensorMap* xmap, int M, int it, int row,
                                             uint32_t stage0, uint32_t full0) {
    using SH = ChainShape<EPI, TH>;
    const int s = it % SH::STAGES_C;
    const uint32_t fb = full0 + 8 * s, dst = stage0 + s * SH::STAGE;
    if (WHAT & 1) mbar_expect_tx(fb, SH::STAGE);
#pragma unroll
    for (int b = 0; b < SH::NB; b++) {
        const int k = it * SH::KS + b * 64;
        if (WHAT & 1) {
            tma_load_2d(dst + b * SH::BOX, wmap, k, row, fb);
            if (EPI == 1) tma_load_2d(dst + S_W_BYTES + b * SH::BOX, wmap, k, M + row, fb);
        }
        if (WHAT & 2) tma_load_2d(dst + SH::SETS * S_W_BYTES + b * S_XBOX, xmap, k, 0, fb);
    }
}

// The producer's part of product p (one thread).  part 1: the weights of the first ring, as the stages come free, then
// -- once the inputs are there -- their activations; part 2: the rest of the items.  (Product 0 runs part 1 before the
// block's first __syncthreads, so they are two calls.)
template <int EPI, int TH>
__device__ __forceinline__ bool chain_produce(const ChainProduct& P, int p, int part, bool has_tile, ChainPipe& pp,
                                              uint32_t stage0, uint32_t full0, uint32_t empty0, const int* gen,
                                              int* gen0_smem, int* err) {
    using SH = ChainShape<EPI, TH>;
    const CUtensorMap* wmap = &P.wmap;
    const CUtensorMap* xmap = &P.xmap;
    const int M = P.M;
    const int items = has_tile ? (P.K + SH::KS - 1) / SH::KS : 0;
    const int row = blockIdx.x * TH;
    const int n_pre = items < SH::STAGES_C ? items : SH::STAGES_C;
    if (part & 1) {
        for (int it = 0; it < n_pre; it++) {
            if (!chain_free_stage<SH::STAGE>(pp, it, empty0, err)) return false;
            chain_copies<EPI, TH, 1>(wmap, xmap, M, it, row, stage0, full0);
            pp.pend |= 1u << it;
        }
        if (p == 0) {
            pdl_wait();                                     // the grid before this launch is done: its outputs stand
        } else {
            chain_wait(gen, *gen0_smem, p, err);
            asm volatile("fence.proxy.async.global;\n" ::: "memory");
        }
        for (int it = 0; it < n_pre; it++) chain_copies<EPI, TH, 2>(wmap, xmap, M, it, row, stage0, full0);
        // ... and so does the barrier's generation (read after the copies are on their way: nobody needs it before
        // the block's first __syncthreads)
        if (p == 0) *gen0_smem = *reinterpret_cast<const volatile int*>(gen);
    }
    if (part & 2) {
        for (int it = n_pre; it < items; it++) {
            const int s = it % SH::STAGES_C;
            if (pp.pend_old) {
                if (!chain_free_stage<SH::STAGE>(pp, s, empty0, err)) return false;
            } else {
                if (!mbar_wait(empty0 + 8 * s, (pp.epar >> s) & 1, err)) return false;
                pp.epar ^= 1u << s;
            }
            chain_copies<EPI, TH, 3>(wmap, xmap, M, it, row, stage0, full0);
            pp.pend |= 1u << s;
        }
        // whatever of the product before this one was never overlaid has long been read: its phases are taken now, so
        // that every completion of an empty barrier has been waited for exactly once
#pragma unroll
        for (int i = 0; i < C_MAX_STAGES; i++)
            if ((pp.pend_old >> i) & 1) {
                if (!mbar_wait(empty0 + 8 * i, (pp.epar >> i) & 1, err)) return false;
                pp.epar ^= 1u << i;
            }
        pp.pend_old = pp.pend;
        pp.pend = 0;
        pp.old_stage = SH::STAGE;
    }
    return true;
}

// The consumers' part of product p: the block's row tile over all of K, then the form's last step (gemm_stream.cu).
template <int EPI, bool SCALED, int TH>
__device__ __forceinline__ bool chain_consume(const ChainProduct& P, bool has_tile, ChainPipe& pp, uint32_t stage0,
                                              uint32_t full0, uint32_t empty0, float* inv_rms, float* red, float* meet,
                                              int* err) {
    using SH = ChainShape<EPI, TH>;
    constexpr int SETS = SH::SETS, MG = SH::MG, KG = SH::KG, BOX = SH::BOX, STAGE = SH::STAGE, STAGES = SH::STAGES_C;
    if (!has_tile) return true;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cw = warp - 1, t128 = cw * 32 + lane, g = lane >> 2, t = lane & 3;
    const int mg = cw % MG, kg = cw / MG, mi = lane >> 3, l7 = lane & 7;
    const bool active = kg == 0;
    const int tile = blockIdx.x, N = P.N, M = P.M;
    const int kblocks = (P.K + SH::KS - 1) / SH::KS;
    float acc[SETS][2][2][4];
    float* accf = &acc[0][0][0][0];
#pragma unroll
    for (int a = 0; a < SETS * 16; a++) accf[a] = 0.0f;
    float old[16];
    float row_b[4] = {0.0f, 0.0f, 0.0f, 0.0f}, row_w[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (EPI == 3 && active) {
        // the stream's old values (another block of the product before may have written them: the barrier has been
        // passed by now) are on their way while the tile's weights arrive
#pragma unroll
        for (int a = 0; a < 16; a++) {
            const int n = 8 * ((a >> 2) & 1) + 2 * t + (a & 1), m = tile * TH + mg * 32 + ((a >> 3) & 1) * 16 + g + ((a >> 1) & 1) * 8;
            old[a] = (m < M && n < N) ? __ldcg(reinterpret_cast<const float*>(P.out) + (size_t)n * M + m) : 0.0f;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int m = tile * TH + mg * 32 + (q >> 1) * 16 + g + (q & 1) * 8;
            if (m < M) {
                if (P.bias) row_b[q] = __ldg(P.bias + m);
                if (P.after.scaled) row_w[q] = __ldg(P.after.w + m);
            }
        }
    }
    for (int kb = 0; kb < kblocks; kb++) {
        const int s = kb % STAGES;
        if (!mbar_wait(full0 + 8 * s, (pp.fpar >> s) & 1, err)) return false;
        pp.fpar ^= 1u << s;
        const uint32_t w_addr = stage0 + s * STAGE, x_addr = w_addr + SETS * S_W_BYTES;
#pragma unroll
        for (int bk = 0; bk < 8; bk++) {                      // this warp's two boxes, four k steps of 16 in each
            const int b = (bk >> 2) * KG + kg, ks = bk & 3;
            uint32_t xb[4];
            ldsm4(x_addr + b * S_XBOX + ((mi >> 1) * 8 + l7) * 128 + (((ks * 2 + (mi & 1)) ^ l7) << 4), xb);
#pragma unroll
            for (int set = 0; set < SETS; set++)
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    uint32_t wa[4];
                    ldsm4(w_addr + set * S_W_BYTES + b * BOX + (mg * 32 + mt * 16 + (mi & 1) * 8 + l7) * 128 +
                              (((ks * 2 + (mi >> 1)) ^ l7) << 4), wa);
                    mma16816(acc[set][mt][0], wa, xb[0], xb[1]);
                    mma16816(acc[set][mt][1], wa, xb[2], xb[3]);
                }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
    }
    if (KG > 1) {
        // the warps that shared the k of these rows add their sums, in the order of the warps
        if (!active) {
#pragma unroll
            for (int a = 0; a < SETS * 16; a++) meet[(cw * SETS * 16 + a) * 32 + lane] = accf[a];
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (active) {
#pragma unroll
            for (int q = 1; q < KG; q++)
#pragma unroll
                for (int a = 0; a < SETS * 16; a++) accf[a] += meet[((q * MG + mg) * SETS * 16 + a) * 32 + lane];
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
    if (SCALED) asm volatile("bar.sync 2, 160;\n" ::: "memory");       // warp 5 has the tokens' 1 / rms
#define C_ROW(a) (mg * 32 + (((a) >> 3) & 1) * 16 + g + (((a) >> 1) & 1) * 8)
#define C_TOK(a) (8 * (((a) >> 2) & 1) + 2 * t + ((a) & 1))
    if (active) {
#pragma unroll
        for (int a = 0; a < 16; a++) {
            const int n = C_TOK(a), m = tile * TH + C_ROW(a);
            if (m >= M || n >= N) continue;
            float v = accf[a];
            if (SCALED) v *= inv_rms[n];
            if (EPI == 3) {
                v += old[a] + row_b[((a >> 3) & 1) * 2 + ((a >> 1) & 1)];
                reinterpret_cast<float*>(P.out)[(size_t)n * M + m] = v;
                if (P.after.scaled) P.after.scaled[(size_t)n * M + m] = __float2bfloat16_rn(v * row_w[((a >> 3) & 1) * 2 + ((a >> 1) & 1)]);
                accf[a] = v;
            } else if (EPI == 1) {
                float up = accf[(SETS - 1) * 16 + a];
                if (SCALED) up *= inv_rms[n];
                const float gt = bf16_round(v);
                reinterpret_cast<bf16*>(P.out)[(size_t)n * M + m] = __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * bf16_round(up));
            } else {
                reinterpret_cast<bf16*>(P.out)[(size_t)n * M + m] = __float2bfloat16_rn(v);
            }
        }
    }
    if (EPI == 3 && P.after.ssq) {
        if (active) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int nt = q >> 1, par = q & 1, n = 8 * nt + 2 * t + par;
                float ss = 0.0f;
#pragma unroll
                for (int mt = 0; mt < 2; mt++)
#pragma unroll
                    for (int hi8 = 0; hi8 < 2; hi8++) {
                        const int m = tile * TH + mg * 32 + mt * 16 + g + hi8 * 8;
                        const float v = acc[0][mt][nt][hi8 * 2 + par];
                        if (m < M && n < N) ss = fmaf(v, v, ss);
                    }
                ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                ss += __shfl_xor_sync(0xffffffffu, ss, 8);
                ss += __shfl_xor_sync(0xffffffffu, ss, 16);
                if (g == 0) red[mg * S_NT + n] = ss;
            }
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (t128 < MG * S_NT && (tile * MG + t128 / S_NT) * 32 < M)
            P.after.ssq[((size_t)tile * MG + t128 / S_NT) * S_NT + t128 % S_NT] = red[t128];
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
#undef C_ROW
#undef C_TOK
    return true;
}

// warp 5: 1 / rms of every token's row from the sums of squares by 32 columns, in a fixed order (gemm_stream.cu)
__device__ __forceinline__ void chain_rms(const ChainProduct& P, float* inv_rms) {
    const int lane = threadIdx.x & 31, quad = lane & 3, part = lane >> 2;
    float4 ss = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float4* rows = reinterpret_cast<const float4*>(P.nrm.ssq);
#pragma unroll 16
    for (int tl = part; tl < P.nrm.ssq_tiles; tl += 8) {
        const float4 v = __ldcg(rows + tl * 4 + quad);
        ss.x += v.x; ss.y += v.y; ss.z += v.z; ss.w += v.w;
    }
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o); ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
        ss.z += __shfl_xor_sync(0xffffffffu, ss.z, o); ss.w += __shfl_xor_sync(0xffffffffu, ss.w, o);
    }
    if (part == 0) {
        const float k = (float)P.K;
        inv_rms[4 * quad] = rsqrtf(ss.x / k + P.nrm.eps); inv_rms[4 * quad + 1] = rsqrtf(ss.y / k + P.nrm.eps);
        inv_rms[4 * quad + 2] = rsqrtf(ss.z / k + P.nrm.eps); inv_rms[4 * quad + 3] = rsqrtf(ss.w / k + P.nrm.eps);
    }
    __syncwarp();
    asm volatile("bar.arrive 2, 160;\n" ::: "memory");
}

// kind -> the compile-time form; f is called with an instance of ChainForm<EPI, SCALED, TH>
template <int EPI_, bool SCALED_, int TH_> struct ChainForm {
    static constexpr int EPI = EPI_, TH = TH_;
    static constexpr bool SCALED = SCALED_;
};
#define C_KIND(epi, scaled, thc) ((epi) * 6 + (scaled) * 3 + (thc))
template <class F>
__device__ __forceinline__ bool chain_dispatch(int kind, F&& f) {
    switch (kind) {
#ifdef C_FEW
        case C_KIND(0, 1, 1): return f(ChainForm<0, true, 64>{});
        case C_KIND(1, 1, 2): return f(ChainForm<1, true, 128>{});
        case C_KIND(3, 0, 0): return f(ChainForm<3, false, 32>{});
#else
        case C_KIND(0, 0, 0): return f(ChainForm<0, false, 32>{});
        case C_KIND(0, 0, 1): return f(ChainForm<0, false, 64>{});
        case C_KIND(0, 0, 2): return f(ChainForm<0, false, 128>{});
        case C_KIND(0, 1, 0): return f(ChainForm<0, true, 32>{});
        case C_KIND(0, 1, 1): return f(ChainForm<0, true, 64>{});
        case C_KIND(0, 1, 2): return f(ChainForm<0, true, 128>{});
        case C_KIND(1, 0, 0): return f(ChainForm<1, false, 32>{});
        case C_KIND(1, 0, 1): return f(ChainForm<1, false, 64>{});
        case C_KIND(1, 0, 2): return f(ChainForm<1, false, 128>{});
        case C_KIND(1, 1, 0): return f(ChainForm<1, true, 32>{});
        case C_KIND(1, 1, 1): return f(ChainForm<1, true, 64>{});
        case C_KIND(1, 1, 2): return f(ChainForm<1, true, 128>{});
        case C_KIND(3, 0, 0): return f(ChainForm<3, false, 32>{});
        case C_KIND(3, 0, 1): return f(ChainForm<3, false, 64>{});
        case C_KIND(3, 0, 2): return f(ChainForm<3, false, 128>{});
#endif
    }
    return false;
}
// the producer's code depends on the form only through EPI (one or two sets of W) and TH
template <class F>
__device__ __forceinline__ bool chain_dispatch_shape(int kind, F&& f) {
    const int epi = kind / 6, thc = kind % 3;
    if (epi == 1) {
        if (thc == 0) return f(ChainForm<1, false, 32>{});
        if (thc == 1) return f(ChainForm<1, false, 64>{});
        return f(ChainForm<1, false, 128>{});
    }
    if (thc == 0) return f(ChainForm<0, false, 32>{});
    if (thc == 1) return f(ChainForm<0, false, 64>{});
    return f(ChainForm<0, false, 128>{});
}

__global__ void __launch_bounds__(S_THREADS, 1) gemm_chain_kernel(const __grid_constant__ ChainArgs A) {
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C_RING);
    int* gen0_smem = reinterpret_cast<int*>(bars + 2 * C_MAX_STAGES);
    float* inv_rms = reinterpret_cast<float*>(gen0_smem + 4);                      // [S_NT]
    float* red = inv_rms + S_NT;                                                     // [4][S_NT] warp sums
    float* meet = reinterpret_cast<float*>(smem + C_RING + C_SMALL);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * C_MAX_STAGES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, n = A.n;
    int* err = A.err;
    const int* gen = A.sync + 1;
    ChainPipe pp;
    bool ok = true;

    if (tid == 0) {
        for (int p = 0; p < n; p++) asm volatile("prefetch.tensormap [%0];\n" ::"l"(&A.prod[p].wmap) : "memory");
        for (int s = 0; s < C_MAX_STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        const ChainProduct& P = A.prod[0];
        const bool has_tile = (int)blockIdx.x < P.tiles;
        ok = chain_dispatch_shape(P.kind, [&](auto f) {
            using F = decltype(f);
            return chain_produce<F::EPI, F::TH>(P, 0, 1, has_tile, pp, stage0, full0, empty0, gen, gen0_smem, err);
        });
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();                         // every thread, before it reads anything the grid before wrote
    const int gen0 = *gen0_smem;

    if (warp == 0) {
        if (lane == 0) {
            for (int p = 0; p < n && ok; p++) {
                const ChainProduct& P = A.prod[p];
                const bool has_tile = (int)blockIdx.x < P.tiles;
                ok = chain_dispatch_shape(P.kind, [&](auto f) {
                    using F = decltype(f);
                    return chain_produce<F::EPI, F::TH>(P, p, p == 0 ? 2 : 3, has_tile, pp, stage0, full0, empty0, gen,
                                                        gen0_smem, err);
                });
            }
        }
    } else if (warp < 5) {
        const int t128 = (warp - 1) * 32 + lane;
        for (int p = 0; p < n && ok; p++) {
            const ChainProduct& P = A.prod[p];
            const bool has_tile = (int)blockIdx.x < P.tiles;
            if (p > 0) {
                // what the product before wrote, in whichever block, is there when the barrier has been passed
                if (t128 == 0) chain_wait(gen, gen0, p, err);
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
            }
            ok = chain_dispatch(P.kind, [&](auto f) {
                using F = decltype(f);
                return chain_consume<F::EPI, F::SCALED, F::TH>(P, has_tile, pp, stage0, full0, empty0, inv_rms, red, meet, err);
            });
            if (p + 1 < n) {
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (t128 == 0) chain_arrive(A.sync, p, n - 1, G);
            }
        }
    } else {
        for (int p = 0; p < n; p++) {
            const ChainProduct& P = A.prod[p];
            const bool scaled = (P.kind / 3) % 2 == 1;
            if (!scaled || (int)blockIdx.x >= P.tiles) continue;
            if (p > 0) chain_wait(gen, gen0, p, err);
            chain_rms(P, inv_rms);
        }
    }
}

// ------------------------------------------------------------------------------------------------ host side
static int chain_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

// the height of a row tile as gemm_stream.cu chooses it, or 0 when that product would be dealt in shares (more tiles
// than SMs, or too few even at 32 rows): such a product is not chained
static int chain_tile_height(int M) {
    const int sms = chain_sms();
    int th = 32;
    for (int h = 128; h > 32; h /= 2)
        if ((M + h - 1) / h >= (sms * 3 + 4) / 5) { th = h; break; }
    const int tiles = (M + th - 1) / th;
    return tiles <= sms && tiles >= (sms * 3 + 4) / 5 ? th : 0;
}

MB_PDL_SWITCH(mb_gemm_chain_set_pdl)

// 1 when a product of M output features (mode as mb_gemm_chain's) can be a member of a chain
MB_API int mb_gemm_chain_takes(int M, int K, int mode) {
    return (mode == 0 || mode == 1 || mode == 3) && K >= 8 && K % 8 == 0 && chain_tile_height(M) != 0;
}

// ints of the barrier's state, zero before the first launch (the kernel leaves the counter zero)
MB_API int mb_gemm_chain_sync_ints() { return 2; }

// One member of a chain.  mode 0: out (N, M) bf16 = act W^T; 1: SwiGLU, W has 2 M rows, out (N, M) bf16; 3: out is the
// float32 residual stream (N, M), added to in place (+ bias), with ssq_out / next_w / scaled_out as in
// mb_gemm_stream_residual.  ssq (modes 0 and 1): act is a normalised stream's rows times the norm's weight, as in
// mb_gemm_stream.
struct ChainMember {
    const void* act; const float* ssq; float eps; const void* W; void* out; const float* bias;
    float* ssq_out; const float* next_w; void* scaled_out; int N, M, K, mode;
};

// members[0 .. n): each reads what the ones before it wrote.  sync: mb_gemm_chain_sync_ints() ints, zero at first.
MB_API int mb_gemm_chain(const ChainMember* members, int n, int* sync, int* err, cudaStream_t st) {
    if (n < 1 || n > C_MAX || !sync) return -2;
    ChainArgs A;
    memset(&A, 0, sizeof(A));
    A.n = n; A.sync = sync; A.err = err;
    int grid = 0;
    for (int p = 0; p < n; p++) {
        const ChainMember& m = members[p];
        ChainProduct& P = A.prod[p];
        if (m.N < 1 || m.N > S_NT || !mb_gemm_chain_takes(m.M, m.K, m.mode) || (reinterpret_cast<uintptr_t>(m.W) & 15) ||
            (reinterpret_cast<uintptr_t>(m.act) & 15) || (m.ssq && (reinterpret_cast<uintptr_t>(m.ssq) & 15)) ||
            (m.mode == 3 && m.ssq) || ((m.next_w == nullptr) != (m.scaled_out == nullptr)))
            return -2;
        const int th = chain_tile_height(m.M), sets = m.mode == 1 ? 2 : 1;
        int rc = matrix_map(m.W, (long long)sets * m.M, m.K, th, &P.wmap);
        if (rc) return rc;
        if ((rc = matrix_map(m.act, m.N, m.K, S_NT, &P.xmap))) return rc;
        P.out = m.out; P.bias = m.bias;
        P.nrm = StreamNorm{m.ssq, (m.K + 31) / 32, m.eps};
        P.after = m.mode == 3 ? StreamAfter{m.ssq_out, m.next_w, (bf16*)m.scaled_out} : StreamAfter{};
        P.N = m.N; P.M = m.M; P.K = m.K;
        P.tiles = (m.M + th - 1) / th;
        P.kind = C_KIND(m.mode, m.ssq ? 1 : 0, th == 32 ? 0 : th == 64 ? 1 : 2);
        if (P.tiles > grid) grid = P.tiles;
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S_SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const cudaError_t e = mb_launch(mb_pdl != 0, gemm_chain_kernel, dim3((unsigned)grid), dim3(S_THREADS), (size_t)S_SMEM, st, A);
    return e == cudaSuccess ? 0 : (int)e;
}
