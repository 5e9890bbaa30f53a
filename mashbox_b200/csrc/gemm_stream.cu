// bf16 matrix products for decode batches (at most 16 tokens), bound by reading W once:
// out[n, m] = sum_k act[n, k] * W[m, k].
//
// W is cut into row tiles of TH rows (128, 64 or 32) and k blocks of 16,384 / TH, so an item (row tile, k block) is 32
// KB of W.  stream_plan() picks the height and the number of blocks: a matrix of 4,096 rows is 128 tiles of 32 rows
// with a block each and no tile is shared; a matrix with few tiles and long rows gets two or three blocks per tile.
// In general the items, row tile major, are dealt in equal shares: block b of G takes [T b / G, T (b + 1) / G), which
// covers the end of one row tile, whole row tiles, and the start of another; a tile that several blocks share is
// finished by the block that arrives last (a counter per tile counts k blocks; it resets itself): every sharer leaves
// its partial sums in its own slot of a workspace and the last one adds the slots in the order of the blocks, so the
// result does not depend on which block was last.  A block works on its two shared tiles first, so that its
// neighbours' sums meet while its whole tiles are still streaming.
//
// Roles of the 192 threads:
//   warp 0     producer: TMA boxes of W (TH rows x 64 k, 128-byte swizzle; for SwiGLU the gate rows and the up rows)
//              and the 2 KB of activations that go with each, four to six stages of 36 to 48 KB in flight (three of
//              68 KB for SwiGLU); the first ring is issued before the block has set itself up;
//   warps 1-4  consumers: ldmatrix from the swizzled tiles, mma.sync m16n8k16 with W as the row operand and the 16
//              token columns as the other, sums in registers; side by side along the rows of a tile and, for tiles of
//              fewer than 128 rows, along k (their sums then meet in shared memory); then the form's last step.  The
//              product is a few percent of the tensor pipe at these sizes; the tcgen05 path was measured here too and
//              its tensor-memory allocation alone cost 1 to 2 us per launch, a fifth of the smaller products;
//   warp 5     (SCALED) turns the sums of squares into every token's 1/rms meanwhile.
//
// Forms (EPI): 0 bf16 out; 1 SwiGLU (W = [gate rows | up rows], out = silu(gate) * up); 2 float out; 3 the float32
// residual stream is added to in place (+ bias), and on request the product leaves what the norm after it needs: the
// sums of squares of the new rows by 32 columns and the new rows times that norm's weight, in bf16.  (Rotation and the
// cache write stay a kernel of their own after the q/k/v product: as an epilogue here, sixteen values per thread on
// the few warps that finish a tile, they cost 9 to 15 us against its 3.)  SCALED: the input is such a pair (rows
// times the norm's weight in bf16, sums of squares): the token's 1/rms, computed in float from the sums, scales the
// float sums of the product, which makes it the product of rmsnorm(x) without a norm kernel.
//
// PDL (programmatic dependent launch): a decode step is a chain of such products, each waiting for the one before, and
// between two launches the memory system idles for about 3 us (the grid drains, the next one starts, its first bytes
// arrive).  Launched with the programmatic-serialization attribute, a block sets its barriers up and sends for its
// first ring of W -- which no kernel of the step writes -- and only then waits for the grid before it
// (griddepcontrol.wait); the activations, the residual stream and the sums of squares are read after that wait, by TMA
// or ld.global.cg.  Measured on the four products of the 8B shape at 8 tokens, launch to launch inside a graph: 1.0 to
// 2.4 us less per launch (o 9.3 -> 8.3, q/k/v 11.8 -> 10.5, down 24.3 -> 23.2, gate/up 40.5 -> 38.1).  A variant with
// half the shared memory and at most 168 registers, so that the next product's block is resident beside this one's
// and its ring already full when this grid ends, was slower than no overlap at all: the shorter ring costs 1.8 to 3.5
// us per launch, the overlap brings back 1.4.
//
// Sizes: K a multiple of 8; N <= 16; any M.  Every wait on an mbarrier is bounded; on a timeout the roles fall through
// to the end of the kernel.
#include "tcgen05.cuh"

#define S_NT 16                       // token columns of the accumulator
#define S_W_BYTES (32 * 1024)         // a set of W per stage: TH rows x (16,384 / TH) k, as boxes of TH rows x 64 k
#define S_XBOX (S_NT * 64 * 2)        // the activations that go with one box: 16 token rows x 64 k
#define S_SMEM (225 * 1024)           // what a block may use
#define S_THREADS 192

// the input of a SCALED product: sums of squares of the rows of x by 32 columns ([ssq_tiles][16]) and eps
struct StreamNorm { const float* ssq; int ssq_tiles; float eps; };
// what form 3 leaves for the norm after it (all null: nothing): sums of squares, the norm's weight, rows times weight
struct StreamAfter { float* ssq; const float* w; bf16* scaled; };

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// A block's range [lo, hi) of items as segments (row tile, k blocks k_lo..k_hi), in the order it works through them:
// the row tile its range starts in, the one it ends in, then the whole tiles between.  The two it shares with its
// neighbours come first, so the neighbours' partial sums meet while the whole tiles are still streaming.
struct StreamSeg { int tile, k_lo, k_hi; };
struct StreamRange {
    long long lo, hi;
    int kblocks, t_first, n_seg;
    __device__ __forceinline__ StreamRange(long long lo_, long long hi_, int kblocks_) : lo(lo_), hi(hi_), kblocks(kblocks_) {
        t_first = (int)(lo / kblocks);
        n_seg = hi > lo ? (int)((hi - 1) / kblocks) - t_first + 1 : 0;
    }
    __device__ __forceinline__ StreamSeg seg(int j) const {
        const int tile = j == 0 ? t_first : (j == 1 ? t_first + n_seg - 1 : t_first + j - 1);
        const long long t0 = (long long)tile * kblocks;
        const long long s = lo > t0 ? lo : t0, e = hi < t0 + kblocks ? hi : t0 + kblocks;
        return StreamSeg{tile, (int)(s - t0), (int)(e - t0)};
    }
};
// walks a range's items in working order
struct StreamWalk {
    const StreamRange& r;
    int j, tile, kb, k_hi;
    __device__ __forceinline__ StreamWalk(const StreamRange& r_) : r(r_), j(0), tile(0), kb(0), k_hi(0) { load(); }
    __device__ __forceinline__ void load() {
        if (j < r.n_seg) { const StreamSeg g = r.seg(j); tile = g.tile; kb = g.k_lo; k_hi = g.k_hi; }
    }
    __device__ __forceinline__ void next() { if (++kb == k_hi) { j++; load(); } }
    __device__ __forceinline__ void skip(int n) { for (; n > 0; n--) next(); }
};

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// compile-time shape of a kernel: TH rows of W per tile (128, 64 or 32)
template <int EPI, int TH> struct StreamShape {
    static constexpr int SETS = EPI == 1 ? 2 : 1;
    static constexpr int MG = TH / 32;                  // consumer warps side by side along the rows of a tile
    static constexpr int KG = 4 / MG;                   // ... and along k: warp w takes the boxes b with b % KG == w / MG
    static constexpr int NB = 2 * KG;                   // boxes of 64 k per set and stage
    static constexpr int KS = 64 * NB;                  // k per item
    static constexpr int BOX = TH * 128;                // bytes of a box of W
    static constexpr int STAGE = SETS * S_W_BYTES + NB * S_XBOX;
    static constexpr int RED = KG > 1 ? 4 * 32 * SETS * 16 * 4 : 0;        // the warps' sums meet here
    static constexpr int SMALL = 1024;                  // barriers, flags, 1 / rms, warp sums
    static constexpr int FIT = (S_SMEM - 1024 - SMALL - RED) / STAGE;
    static constexpr int STAGES = FIT > 6 ? 6 : FIT;
    static constexpr size_t BYTES = 1024 + (size_t)STAGES * STAGE + SMALL + RED;
};

template <int EPI, bool SCALED, int TH>
__global__ void __launch_bounds__(S_THREADS, 1) gemm_stream_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                    const __grid_constant__ CUtensorMap xmap,
                                                                    void* __restrict__ out, int N, int M, int K, int tiles,
                                                                    float* __restrict__ partial, int* __restrict__ tile_done,
                                                                    StreamNorm nrm, const float* __restrict__ bias,
                                                                    StreamAfter after, int* err) {
    using SH = StreamShape<EPI, TH>;
    constexpr int SETS = SH::SETS, MG = SH::MG, KG = SH::KG, NB = SH::NB, KS = SH::KS, BOX = SH::BOX;
    constexpr int STAGE = SH::STAGE, STAGES = SH::STAGES;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE);
    int* last_flag = reinterpret_cast<int*>(bars + 2 * STAGES);
    float* inv_rms = reinterpret_cast<float*>(last_flag + 4);                    // [S_NT]
    float* red = inv_rms + S_NT;                                                   // [4][S_NT] warp sums
    float* meet = reinterpret_cast<float*>(smem + (size_t)STAGES * STAGE + SH::SMALL);   // [4 warps][SETS * 16][32 lanes]
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = (K + KS - 1) / KS;
    const long long T = (long long)tiles * kblocks;
    const long long lo = T * blockIdx.x / gridDim.x, hi = T * (blockIdx.x + 1) / gridDim.x;
    const StreamRange range(lo, hi, kblocks);
    const long long items = hi - lo;
    // the TMA copies of an item of this block: the weights (what = 1), the activations that go with them (2), or both
    auto produce = [&](long long it, int tile, int kb, int what) {
        const int s = (int)(it % STAGES), row = tile * TH;
        const uint32_t fb = full0 + 8 * s, dst = stage0 + s * STAGE;
        if (what & 1) mbar_expect_tx(fb, STAGE);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int k = kb * KS + b * 64;
            if (what & 1) {
                tma_load_2d(dst + b * BOX, &wmap, k, row, fb);
                if (EPI == 1) tma_load_2d(dst + S_W_BYTES + b * BOX, &wmap, k, M + row, fb);
            }
            if (what & 2) tma_load_2d(dst + SETS * S_W_BYTES + b * S_XBOX, &xmap, k, 0, fb);
        }
    };
    StreamWalk pw(range);                                             // the producer's place (thread 0 only)
    long long p_it = 0;
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&wmap) : "memory");
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        // The first ring of copies is on its way before the block has set itself up: the weights first (nobody writes
        // them), then, once the grid before this one is done, the activations it produced.
        StreamWalk w2(range);
        long long i2 = 0;
        for (; i2 < items && i2 < STAGES; i2++, w2.next()) produce(i2, w2.tile, w2.kb, 1);
        pdl_wait();
        for (; p_it < items && p_it < STAGES; p_it++, pw.next()) produce(p_it, pw.tile, pw.kb, 2);
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();                         // every thread, before it reads anything the grid before wrote

    if (warp == 0) {
        if (lane == 0) {
            for (; p_it < items; p_it++, pw.next()) {
                if (!mbar_wait(empty0 + 8 * (int)(p_it % STAGES), (uint32_t)(p_it / STAGES - 1) & 1, err)) break;
                produce(p_it, pw.tile, pw.kb, 3);
            }
        }
    } else if (warp < 5) {
        // consumers: warp cw = (mg, kg) owns rows 32 mg .. 32 mg + 31 of a tile and the boxes b with b % KG == kg; sums in
        // registers: acc[set][mt][nt][i] is row 32 mg + 16 mt + g + 8 (i >> 1), token 8 nt + 2 t + (i & 1)
        // (g = lane / 4, t = lane % 4).  The warps with kg == 0 finish a tile ("active"); all take part in the barriers.
        const int cw = warp - 1, t128 = cw * 32 + lane, g = lane >> 2, t = lane & 3;
        const int mg = cw % MG, kg = cw / MG, mi = lane >> 3, l7 = lane & 7;
        const bool active = kg == 0;
        const int tact = mg * 32 + lane;                              // this thread's column of the slots and of meet
        int it = 0;
        bool ok = true, have_rms = false;
        for (int j = 0; j < range.n_seg && ok; j++) {
            const StreamSeg sg = range.seg(j);
            const int tile = sg.tile, k_lo = sg.k_lo, k_hi = sg.k_hi;
            float acc[SETS][2][2][4];
            float* accf = &acc[0][0][0][0];
#pragma unroll
            for (int a = 0; a < SETS * 16; a++) accf[a] = 0.0f;
            float old[16];
            if (EPI == 3 && active) {
                // the stream's old values are on their way while the tile's weights arrive
#pragma unroll
                for (int a = 0; a < 16; a++) {
                    const int n = 8 * ((a >> 2) & 1) + 2 * t + (a & 1), m = tile * TH + mg * 32 + ((a >> 3) & 1) * 16 + g + ((a >> 1) & 1) * 8;
                    old[a] = (m < M && n < N) ? __ldcg(reinterpret_cast<const float*>(out) + (size_t)n * M + m) : 0.0f;
                }
            }
            float row_b[4] = {0.0f, 0.0f, 0.0f, 0.0f}, row_w[4] = {0.0f, 0.0f, 0.0f, 0.0f};      // bias and next norm's weight of this thread's rows
            if (EPI == 3 && active) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int m = tile * TH + mg * 32 + (q >> 1) * 16 + g + (q & 1) * 8;
                    if (m < M) {
                        if (bias) row_b[q] = __ldg(bias + m);
                        if (after.scaled) row_w[q] = __ldg(after.w + m);
                    }
                }
            }
            for (int kb = k_lo; kb < k_hi; kb++, it++) {
                const int s = it % STAGES, round = it / STAGES;
                if (!mbar_wait(full0 + 8 * s, round & 1, err)) { ok = false; break; }
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
                if (lane == 0) mbar_arrive(empty0 + 8 * s);           // this warp has read the stage
            }
            if (!ok) break;
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
                asm volatile("bar.sync 1, 128;\n" ::: "memory");      // meet may be written again
            }
            bool finish = true;
            if (k_lo > 0 || k_hi < kblocks) {
                // this block holds a part of the row tile's sum: slot 0 when the tile is the one its range starts in
                const int slot = tile == range.t_first ? 0 : 1;
                float* mine = partial + ((size_t)blockIdx.x * 2 + slot) * (SETS * S_NT * 128);
                if (active) {
#pragma unroll
                    for (int a = 0; a < SETS * 16; a++)
                        if (8 * ((a >> 2) & 1) + 2 * t + (a & 1) < N) mine[a * 128 + tact] = accf[a];
                }
                // the warps' stores, then one thread's release: who brings the count to the tile's k blocks acquires
                // what the others released
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (t128 == 0) {
                    int before;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;\n" : "=r"(before) : "l"(tile_done + tile), "r"(k_hi - k_lo) : "memory");
                    *last_flag = before + (k_hi - k_lo) == kblocks;
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                finish = *last_flag != 0;
                if (finish) {
                    const long long first_item = (long long)tile * kblocks, last_item = first_item + kblocks - 1;
                    const int c_first = (int)(((first_item + 1) * gridDim.x + T - 1) / T) - 1;
                    const int c_last = (int)(((last_item + 1) * gridDim.x + T - 1) / T) - 1;
#pragma unroll
                    for (int a = 0; a < SETS * 16; a++) accf[a] = 0.0f;
                    if (active) {
#pragma unroll 4
                        for (int c = c_first; c <= c_last; c++) {
                            const int c_slot = (int)((T * c / gridDim.x) / kblocks) == tile ? 0 : 1;
                            const float* theirs = partial + ((size_t)c * 2 + c_slot) * (SETS * S_NT * 128);
#pragma unroll
                            for (int a = 0; a < SETS * 16; a++)
                                if (8 * ((a >> 2) & 1) + 2 * t + (a & 1) < N) accf[a] += __ldcg(theirs + a * 128 + tact);
                        }
                    }
                    if (t128 == 0) tile_done[tile] = 0;                // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");      // last_flag may be written again
            }
            if (!finish) continue;
            // the first tile this block finishes waits for warp 5's 1 / rms (its loads queue behind the TMA copies, so
            // not earlier than needed: a wait here while tiles are still to come would stall the ring)
            if (SCALED && !have_rms) { asm volatile("bar.sync 2, 160;\n" ::: "memory"); have_rms = true; }
            // row r of the tile and token n of sum a of this thread
#define S_ROW(a) (mg * 32 + (((a) >> 3) & 1) * 16 + g + (((a) >> 1) & 1) * 8)
#define S_TOK(a) (8 * (((a) >> 2) & 1) + 2 * t + ((a) & 1))
            {
                if (active) {
#pragma unroll
                    for (int a = 0; a < 16; a++) {
                        const int n = S_TOK(a), m = tile * TH + S_ROW(a);
                        if (m >= M || n >= N) continue;
                        float v = accf[a];
                        if (SCALED) v *= inv_rms[n];
                        if (EPI == 2) {
                            reinterpret_cast<float*>(out)[(size_t)n * M + m] = v;
                        } else if (EPI == 3) {
                            v += old[a] + row_b[((a >> 3) & 1) * 2 + ((a >> 1) & 1)];
                            reinterpret_cast<float*>(out)[(size_t)n * M + m] = v;
                            if (after.scaled) after.scaled[(size_t)n * M + m] = __float2bfloat16_rn(v * row_w[((a >> 3) & 1) * 2 + ((a >> 1) & 1)]);
                            accf[a] = v;
                        } else if (EPI == 1) {
                            // gate and up pass through bf16 as they do when the products are separate kernels
                            float up = accf[(SETS - 1) * 16 + a];
                            if (SCALED) up *= inv_rms[n];
                            const float gt = bf16_round(v);
                            reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * bf16_round(up));
                        } else {
                            reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(v);
                        }
                    }
                }
                if (EPI == 3 && after.ssq) {
                    // the sums of squares of the new rows over this tile's columns, for the norm that follows
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
                    // one row of sums per 32 columns of x, whatever the tile's height
                    if (t128 < MG * S_NT && (tile * MG + t128 / S_NT) * 32 < M)
                        after.ssq[((size_t)tile * MG + t128 / S_NT) * S_NT + t128 % S_NT] = red[t128];
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");  // red may be written again
                }
            }
        }
    } else if (SCALED && warp == 5) {
        // 1 / rms of every token's row, in float, from the sums of squares by 32 columns in a fixed order, while the
        // consumers are at work: lane (part, quad) adds the rows part, part + 8, ... of the sums for the tokens
        // 4 quad .. 4 quad + 3, then the eight parts meet in a tree of shuffles
        const int quad = lane & 3, part = lane >> 2;
        float4 ss = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float4* rows = reinterpret_cast<const float4*>(nrm.ssq);
#pragma unroll 16
        for (int tl = part; tl < nrm.ssq_tiles; tl += 8) {
            const float4 v = __ldcg(rows + tl * 4 + quad);
            ss.x += v.x; ss.y += v.y; ss.z += v.z; ss.w += v.w;
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o); ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
            ss.z += __shfl_xor_sync(0xffffffffu, ss.z, o); ss.w += __shfl_xor_sync(0xffffffffu, ss.w, o);
        }
        if (part == 0) {
            const float k = (float)K;
            inv_rms[4 * quad] = rsqrtf(ss.x / k + nrm.eps); inv_rms[4 * quad + 1] = rsqrtf(ss.y / k + nrm.eps);
            inv_rms[4 * quad + 2] = rsqrtf(ss.z / k + nrm.eps); inv_rms[4 * quad + 3] = rsqrtf(ss.w / k + nrm.eps);
        }
        __syncwarp();
        asm volatile("bar.arrive 2, 160;\n" ::: "memory");
    }
#undef S_ROW
#undef S_TOK
}

// ------------------------------------------------------------------------------------------------ host side
static int stream_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

// floats of workspace (two slots of partial sums per block) and ints of counters (one per 32 rows of W, zero before
// the first call; the kernels leave them zero) that a product with M output features needs
MB_API long long mb_gemm_stream_workspace() { return (long long)stream_sms() * 2 * 2 * S_NT * 128; }
MB_API long long mb_gemm_stream_counters(int M) { return (M + 31) / 32; }

// What was measured about the pace of these kernels (8B shapes, launch to launch inside a graph).  With the weights
// resident in L2 they take almost as long as from DRAM (o 7.8 against 8.5 us, q/k/v 9.4 against 11.4, down 23.0 against
// 23.0); one token takes as long as sixteen; leaving out the products of the token columns 8..15 when there are at most
// 8 tokens, or asking for the fragments of the next k step before the products of this one are issued, changed nothing;
// a kernel that only streams the matrix into shared memory takes as long as the product.  So neither DRAM nor the
// consumer warps set it: about 2.5 us per launch before the first bytes and after the last, and an intake of some 50
// GB/s per SM in between.  More blocks did not help either way: cutting the same matrices into more tiles than SMs and
// dealing equal shares (q/k/v as 192 tiles of 32 rows: 14.4 us against 11.5; gate/up as 224 of 64: 42.5 against 38.7)
// loses more to the tiles that blocks share than the idle SMs cost, and tiles of 48 rows for q/k/v (128 blocks instead
// of 96) and of 112 rows for gate/up (128 instead of 112), one block each, were slower as well (12.6 against 11.4).
// Nor did it help to have a product's producer warp, once its own last weights are on their way, ask the L2 for the
// first ring of the product that follows (cp.async.bulk.prefetch.tensor with that product's tensor map): a layer's four
// products took 85.3 us against 82.2.
// The height of a row tile: the largest of 128, 64, 32 that gives at least 0.6 tiles per SM, so that a matrix of few
// rows still has a tile for most SMs and no tile is shared (then the grid is one block per tile); matrices with more
// tiles than SMs, or too few even at 32 rows, are cut into equal shares of items.  least: the smallest height allowed.
static int stream_tile_height(int M, int sms, int least) {
    for (int th = 128; th > least; th /= 2)
        if ((M + th - 1) / th >= (sms * 3 + 4) / 5) return th;
    return least;
}

// How a product is cut: the height of a row tile and the number of blocks.  Of the heights that give no more tiles
// than SMs and of the numbers of blocks per tile (1 to as many as fit, at most one per k block; the same for every
// tile, so that a tile's sharers finish together), the pair that this estimate puts first: 4 us, the matrix's bytes
// at the rate the blocks take them in (60 GB/s a block, 6 TB/s in all), and 1.5 us + 0.5 us per sharer when blocks
// share a tile (their partial sums meet through global memory, behind whatever else is in flight).  Measured alone
// (8 tokens, launch to launch in a graph), us: 2,048 x 2,048 as 64 blocks 4.2, as 128 blocks that share 5.5, dealt
// unevenly over all SMs as before 7.7; 2,048 x 8,192: 12.8 / 10.5 / 11.3; 5,120 x 3,072 as 80 tiles of 64 rows 8.9,
// unevenly 10.6; 6,144 x 4,096 as 96 tiles of 64 rows 11.3, as 48 tiles of 128 rows shared by three 11.6 -- and inside
// a model the shared form cost 7 us more than that.  With more tiles than SMs at every height (the output head)
// stream_tile_height() decides and all SMs take equal shares.
struct StreamPlan { int th; long long grid; };
static StreamPlan stream_plan(int M, int K, int sets, int sms, int least) {
    StreamPlan best{0, 0};
    double best_t = 0.0;
    const double bytes = (double)sets * M * K * 2.0;
    for (int th = least; th <= 128; th *= 2) {                       // at equal cost the lower tile: fewer sharers
        const long long tiles = (M + th - 1) / th;
        if (tiles > sms) continue;
        const long long ks = 16384 / th, kblocks = (K + ks - 1) / ks;
        for (long long per = 1; per <= kblocks && tiles * per <= sms; per++) {
            const double blocks = (double)(tiles * per);
            const double stream = bytes / 6e6 > bytes / (blocks * 60e3) ? bytes / 6e6 : bytes / (blocks * 60e3);
            const double t = 4.0 + stream + (per > 1 ? 1.5 + 0.5 * (double)per : 0.0);
            if (best.th == 0 || t < best_t - 1e-9) { best = StreamPlan{th, tiles * per}; best_t = t; }
        }
    }
    if (best.th == 0) best = StreamPlan{stream_tile_height(M, sms, least), sms};
    return best;
}

MB_PDL_SWITCH(mb_gemm_stream_set_pdl)

template <int EPI, bool SCALED, int TH>
static int stream_launch_th(const void* act, const void* W, void* out, int N, int M, int K, float* workspace, int* counters,
                            StreamNorm nrm, const float* bias, StreamAfter after, int* err, cudaStream_t st, long long grid) {
    using SH = StreamShape<EPI, TH>;
    static_assert(SH::STAGES >= 2, "a ring of at least two stages");
    CUtensorMap wmap, xmap;
    int rc = matrix_map(W, (long long)SH::SETS * M, K, TH, &wmap);
    if (rc) return rc;
    if ((rc = matrix_map(act, N, K, S_NT, &xmap))) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<EPI, SCALED, TH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SH::BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = (M + TH - 1) / TH;
    const long long T = (long long)tiles * ((K + SH::KS - 1) / SH::KS);
    if (grid > T) grid = T;
    const cudaError_t e = mb_launch(mb_pdl != 0, gemm_stream_kernel<EPI, SCALED, TH>, dim3((unsigned)grid), dim3(S_THREADS),
                                    SH::BYTES, st, wmap, xmap, out, N, M, K, tiles, workspace, counters, nrm, bias, after, err);
    return e == cudaSuccess ? 0 : (int)e;
}

template <int EPI, bool SCALED>
static int stream_launch(const void* act, const void* W, void* out, int N, int M, int K, float* workspace, int* counters,
                         StreamNorm nrm, const float* bias, StreamAfter after, int* err, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    if (N > S_NT || K % 8 || K < 8 || !workspace || !counters || (reinterpret_cast<uintptr_t>(W) & 15) ||
        (reinterpret_cast<uintptr_t>(act) & 15) || (SCALED && (!nrm.ssq || (reinterpret_cast<uintptr_t>(nrm.ssq) & 15))))
        return -2;
    const StreamPlan plan = stream_plan(M, K, EPI == 1 ? 2 : 1, stream_sms(), 32);
    switch (plan.th) {
        case 128: return stream_launch_th<EPI, SCALED, 128>(act, W, out, N, M, K, workspace, counters, nrm, bias, after, err, st, plan.grid);
        case 64: return stream_launch_th<EPI, SCALED, 64>(act, W, out, N, M, K, workspace, counters, nrm, bias, after, err, st, plan.grid);
        default: return stream_launch_th<EPI, SCALED, 32>(act, W, out, N, M, K, workspace, counters, nrm, bias, after, err, st, plan.grid);
    }
}

// mode 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out (N, M).
// ssq (or null): act holds rows of a residual stream times a norm's weight and ssq ([ceil(K / 32)][16]) the sums of
// squares of those rows by 32 columns, as mb_gemm_stream_residual leaves them: out is then the product of
// rmsnorm(x; weight, eps).
MB_API int mb_gemm_stream(const void* act, const float* ssq, float eps, const void* W, void* out, int N, int M, int K,
                          int mode, float* workspace, int* counters, int* err, cudaStream_t st) {
    const StreamNorm nn{ssq, (K + 31) / 32, eps};
    const StreamAfter na{};
    if (ssq) {
        if (mode == 0) return stream_launch<0, true>(act, W, out, N, M, K, workspace, counters, nn, nullptr, na, err, st);
        if (mode == 1) return stream_launch<1, true>(act, W, out, N, M, K, workspace, counters, nn, nullptr, na, err, st);
        return -2;
    }
    switch (mode) {
        case 0: return stream_launch<0, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, na, err, st);
        case 1: return stream_launch<1, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, na, err, st);
        case 2: return stream_launch<2, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, na, err, st);
    }
    return -2;
}

// x (N, M) float32 += act (N, K) bf16 @ W (M, K)^T (+ bias (M) float32 or null), in place.  ssq_out (or null):
// [ceil(M / 32)][16] floats that receive the sums of squares of the new rows of x by 32 columns; next_w and scaled_out
// (or null): the weight (M) of the norm that reads x next, and (N, M) bf16 that receives the new rows times it
MB_API int mb_gemm_stream_residual(const void* act, const void* W, float* x, const float* bias, int N, int M, int K,
                                   float* ssq_out, const float* next_w, void* scaled_out, float* workspace, int* counters,
                                   int* err, cudaStream_t st) {
    if ((next_w == nullptr) != (scaled_out == nullptr)) return -2;
    return stream_launch<3, false>(act, W, x, N, M, K, workspace, counters, StreamNorm{}, bias,
                                   StreamAfter{ssq_out, next_w, (bf16*)scaled_out}, err, st);
}
