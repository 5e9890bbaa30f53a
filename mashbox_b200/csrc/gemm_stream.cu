// bf16 matrix products for decode batches (at most 16 tokens), bound by reading W once:
// out[n, m] = sum_k act[n, k] * W[m, k].
//
// The work is the list of (row tile of 128 rows, k block of 64) items, row tile major, and block b of G takes the items
// [T b / G, T (b + 1) / G): every SM streams the same number of bytes whatever the matrix's shape.  A block's range
// covers the end of one row tile, whole row tiles, and the start of another; a row tile that several blocks share is
// finished by the block that arrives last (a counter per row tile counts k blocks; it resets itself): every sharer
// leaves its partial sums in its own slot of a workspace and the last one adds the slots in the order of the blocks,
// so the result does not depend on which block was last.  A block works on its two shared tiles first, so that its
// neighbours' sums meet while its whole tiles are still streaming.
//
// Roles of the 288 threads:
//   warp 0     producer: one TMA box of W (128 rows x 64 k, 16 KB, 128-byte swizzle; two for SwiGLU: gate rows and up
//              rows) and the 2 KB of activations that go with it per stage, ten stages in flight (six for SwiGLU); the
//              first ring is issued before the block has set itself up;
//   warps 1-4  consumers: ldmatrix from the swizzled tiles, mma.sync m16n8k16 with W as the row operand (32 rows per
//              warp) and the 16 token columns as the other, sums in registers, then the sharing protocol above and
//              the form's last step.  The product is a few percent of the tensor pipe at these sizes; the tcgen05
//              path was measured here too and its tensor-memory allocation alone cost 1 to 2 us per launch, a fifth
//              of the smaller products;
//   warps 5-8  (normalising forms) make the activations themselves: x[n, k] * g[k] from the float32 residual stream,
//              rounded to bf16, written into the stage in the layout the TMA would have produced.
//
// Forms (EPI): 0 bf16 out; 1 SwiGLU (W = [gate rows | up rows], out = silu(gate) * up); 2 float out; 3 the float32
// residual stream is added to in place (+ bias); 4 the fused q/k/v product with rotation and the write of k and v into
// the pages of the cache.  NORM: the input is rmsnorm(x) of the float32 residual stream: the product runs on
// bf16(x * g) and the token's 1/rms, which the consumer warps compute in float while the first tiles arrive, scales
// the sums.
//
// Sizes: K a multiple of 8; N <= 16; any M.  Form 4 wants a head size that divides 128.  Every wait on an mbarrier is
// bounded; on a timeout the roles fall through to the end of the kernel.
#include "tcgen05.cuh"

#define S_NT 16                       // token columns of the accumulator
#define S_BK 128                      // k per item: two 128-byte swizzle spans ("halves") of 64
#define S_W_BYTES (2 * 128 * 64 * 2)  // a set of W per stage: two boxes of 128 rows x 64 k
#define S_X_BYTES (2 * S_NT * 64 * 2) // the activations per stage: two tiles of 16 token rows x 64 k
#define S_THREADS 288
#define S_CONV_WARPS 4

// ssq: sums of squares of the rows of x by row tile ([tiles][16], from the product that last added into x), or null
struct StreamNorm { const float* x; const float* w; float eps; const float* ssq; int ssq_tiles; };
struct StreamRope {
    const int* positions; const int* tok_row; const int* table; int max_blocks;
    bf16* kpool; bf16* vpool; const float* freqs;
    int H, KV, HD, RD, pairing, page, num_pages;
};

#ifdef S_TRACE
__device__ unsigned long long* s_trace_buf;
__device__ __forceinline__ void s_mark(int ev) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    if (s_trace_buf) s_trace_buf[blockIdx.x * 8 + ev] = t;
}
MB_API int mb_gemm_stream_trace(unsigned long long* buf) { return (int)cudaMemcpyToSymbol(s_trace_buf, &buf, sizeof(buf)); }
#else
#define s_mark(ev)
#endif

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

template <int EPI, bool NORM>
__global__ void __launch_bounds__(S_THREADS, 1) gemm_stream_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                    const __grid_constant__ CUtensorMap xmap,
                                                                    void* __restrict__ out, int N, int M, int K,
                                                                    float* __restrict__ partial, int* __restrict__ tile_done,
                                                                    StreamNorm nrm, const float* __restrict__ bias,
                                                                    StreamRope rope, float* __restrict__ ssq_out, int* err) {
    constexpr int SETS = EPI == 1 ? 2 : 1;
    constexpr int STAGE = SETS * S_W_BYTES + S_X_BYTES;
    constexpr int STAGES = EPI == 1 ? 3 : 6;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE);
    int* last_flag = reinterpret_cast<int*>(bars + 2 * STAGES);
    float* inv_rms = reinterpret_cast<float*>(last_flag + 4);                    // [S_NT]
    float* red = inv_rms + S_NT;                                                   // [4][S_NT] warp sums
    float* xch = red + 4 * S_NT;                                                   // [S_NT][128], form 4 only
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_tiles = (M + 127) / 128, kblocks = (K + S_BK - 1) / S_BK;
    const long long T = (long long)row_tiles * kblocks;
    const long long lo = T * blockIdx.x / gridDim.x, hi = T * (blockIdx.x + 1) / gridDim.x;
    const StreamRange range(lo, hi, kblocks);
    const long long items = hi - lo;

    auto produce = [&](long long it, int tile, int kb) {              // the TMA copies of an item of this block
        const int s = (int)(it % STAGES);
        const uint32_t fb = full0 + 8 * s, dst = stage0 + s * STAGE;
        mbar_expect_tx(fb, NORM ? SETS * S_W_BYTES : STAGE);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            tma_load_2d(dst + h * (S_W_BYTES / 2), &wmap, kb * S_BK + h * 64, tile * 128, fb);
            if (EPI == 1) tma_load_2d(dst + S_W_BYTES + h * (S_W_BYTES / 2), &wmap, kb * S_BK + h * 64, M + tile * 128, fb);
            if (!NORM) tma_load_2d(dst + SETS * S_W_BYTES + h * (S_X_BYTES / 2), &xmap, kb * S_BK + h * 64, 0, fb);
        }
    };
    StreamWalk pw(range);                                             // the producer's place (thread 0 only)
    long long p_it = 0;
    if (tid == 0) {
        s_mark(0);
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&wmap) : "memory");
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, NORM ? 3 : 1); mbar_init(empty0 + 8 * s, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        // the first ring of copies is on its way before the block has set itself up
        for (; p_it < items && p_it < STAGES; p_it++, pw.next()) produce(p_it, pw.tile, pw.kb);
        s_mark(1);
    }
    if (NORM && warp >= 5) {
        // the token rows that no token fills stay zero in every stage
        for (int s = 0; s < STAGES; s++) {
            uint32_t* xs = reinterpret_cast<uint32_t*>(smem + (size_t)s * STAGE + SETS * S_W_BYTES);
            for (int i = tid - 160; i < S_X_BYTES / 4; i += 32 * S_CONV_WARPS) xs[i] = 0u;
        }
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) {
            for (; p_it < items; p_it++, pw.next()) {
                if (!mbar_wait(empty0 + 8 * (int)(p_it % STAGES), (uint32_t)(p_it / STAGES - 1) & 1, err)) break;
                produce(p_it, pw.tile, pw.kb);
            }
        }
    } else if (warp < 5) {
        // consumers: warp cw owns rows 32 cw .. 32 cw + 31 of every row tile, the sums stay in its registers:
        // acc[set][mt][nt][i] is row 32 cw + 16 mt + g + 8 (i >> 1), token 8 nt + 2 t + (i & 1)  (g = lane / 4, t = lane % 4)
        const int cw = warp - 1, t128 = cw * 32 + lane, g = lane >> 2, t = lane & 3;
        const int mi = lane >> 3, l7 = lane & 7;
        if (NORM) {
            // 1 / rms of every token's row of the residual stream, in float, summed in a fixed order: from the sums by
            // row tile that the product before left, or over the rows themselves
            if (nrm.ssq) {
                if (t128 < N) {
                    float ss = 0.0f;
                    for (int tl = 0; tl < nrm.ssq_tiles; tl++) ss += __ldcg(nrm.ssq + tl * S_NT + t128);
                    inv_rms[t128] = rsqrtf(ss / (float)K + nrm.eps);
                }
            } else {
                for (int n = 0; n < N; n++) {
                    float ss = 0.0f;
                    const float4* row = reinterpret_cast<const float4*>(nrm.x + (size_t)n * K);
#pragma unroll 8
                    for (int c = t128; c < K / 4; c += 128) {
                        const float4 v = __ldg(row + c);
                        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
                    }
                    ss = mb_warp_sum(ss);
                    if (lane == 0) red[cw * S_NT + n] = ss;
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (t128 < N) {
                    const float ss = (red[t128] + red[S_NT + t128]) + (red[2 * S_NT + t128] + red[3 * S_NT + t128]);
                    inv_rms[t128] = rsqrtf(ss / (float)K + nrm.eps);
                }
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
        }
        int it = 0;
        bool ok = true;
        if (t128 == 0) s_mark(2);
        for (int j = 0; j < range.n_seg && ok; j++) {
            const StreamSeg sg = range.seg(j);
            const int tile = sg.tile, k_lo = sg.k_lo, k_hi = sg.k_hi;
            float acc[SETS][2][2][4];
#pragma unroll
            for (int a = 0; a < SETS * 16; a++) (&acc[0][0][0][0])[a] = 0.0f;
            for (int kb = k_lo; kb < k_hi; kb++, it++) {
                const int s = it % STAGES, round = it / STAGES;
                if (!mbar_wait(full0 + 8 * s, round & 1, err)) { ok = false; break; }
                if (t128 == 0 && it == 0) s_mark(3);
                if (t128 == 0 && it == items - 1) s_mark(4);
                const uint32_t w_addr = stage0 + s * STAGE, x_addr = w_addr + SETS * S_W_BYTES;
#pragma unroll
                for (int hk = 0; hk < S_BK / 16; hk++) {
                    const int h = hk >> 2, ks = hk & 3;               // half of the stage, k step of 16 inside it
                    uint32_t b[4];
                    ldsm4(x_addr + h * (S_X_BYTES / 2) + ((mi >> 1) * 8 + l7) * 128 + (((ks * 2 + (mi & 1)) ^ l7) << 4), b);
#pragma unroll
                    for (int set = 0; set < SETS; set++)
#pragma unroll
                        for (int mt = 0; mt < 2; mt++) {
                            uint32_t a[4];
                            ldsm4(w_addr + set * S_W_BYTES + h * (S_W_BYTES / 2) + (cw * 32 + mt * 16 + (mi & 1) * 8 + l7) * 128 +
                                      (((ks * 2 + (mi >> 1)) ^ l7) << 4), a);
                            mma16816(acc[set][mt][0], a, b[0], b[1]);
                            mma16816(acc[set][mt][1], a, b[2], b[3]);
                        }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);           // this warp has read the stage
            }
            if (!ok) break;
            bool finish = true;
            if (t128 == 0 && j == range.n_seg - 1) s_mark(5);
            if (k_lo > 0 || k_hi < kblocks) {
                // this block holds a part of the row tile's sum: slot 0 when the tile is the one its range starts in
                const int slot = tile == range.t_first ? 0 : 1;
                float* mine = partial + ((size_t)blockIdx.x * 2 + slot) * (SETS * S_NT * 128);
#pragma unroll
                for (int a = 0; a < SETS * 16; a++)
                    if (8 * ((a >> 2) & 1) + 2 * t + (a & 1) < N) mine[a * 128 + t128] = (&acc[0][0][0][0])[a];
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
                    for (int a = 0; a < SETS * 16; a++) (&acc[0][0][0][0])[a] = 0.0f;
#pragma unroll 4
                    for (int c = c_first; c <= c_last; c++) {
                        const int c_slot = (int)((T * c / gridDim.x) / kblocks) == tile ? 0 : 1;
                        const float* theirs = partial + ((size_t)c * 2 + c_slot) * (SETS * S_NT * 128);
#pragma unroll
                        for (int a = 0; a < SETS * 16; a++)
                            if (8 * ((a >> 2) & 1) + 2 * t + (a & 1) < N) (&acc[0][0][0][0])[a] += __ldcg(theirs + a * 128 + t128);
                    }
                    if (t128 == 0) tile_done[tile] = 0;                // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");      // last_flag may be written again
            }
            if (t128 == 0 && j == range.n_seg - 1) s_mark(6);
            if (!finish) continue;
            if (EPI == 4) {
                // rotation pairs two rows of a head: the rows of the tile meet in shared memory
#pragma unroll
                for (int a = 0; a < 16; a++) {
                    const int r = cw * 32 + ((a >> 3) & 1) * 16 + g + ((a >> 1) & 1) * 8, n = 8 * ((a >> 2) & 1) + 2 * t + (a & 1);
                    const int m = tile * 128 + r;
                    // as the separate kernels do it: the product rounded to bf16, then bias and rotation in float
                    float v = (&acc[0][0][0][0])[a];
                    if (NORM && n < N) v *= inv_rms[n];
                    v = bf16_round(v) + ((bias && m < M) ? bias[m] : 0.0f);
                    (&acc[0][0][0][0])[a] = v;
                    xch[n * 128 + r] = v;
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
                for (int a = 0; a < 16; a++) {
                    const int r = cw * 32 + ((a >> 3) & 1) * 16 + g + ((a >> 1) & 1) * 8, n = 8 * ((a >> 2) & 1) + 2 * t + (a & 1);
                    const int m = tile * 128 + r;
                    if (m >= M || n >= N) continue;
                    const int head = m / rope.HD, e = m % rope.HD, rh = rope.RD / 2;
                    int pe = e, pair = -1;
                    bool first = true;
                    if (rope.pairing == 0) { pe = e ^ 1; first = !(e & 1); pair = (e >> 1) < rh ? (e >> 1) : -1; }
                    else if (e < rope.RD) { first = e < rh; pe = first ? e + rh : e - rh; pair = first ? e : e - rh; }
                    float v = (&acc[0][0][0][0])[a];
                    const int pos = rope.positions[n];
                    if (pair >= 0 && rope.freqs && head < rope.H + rope.KV) {
                        const float p = xch[n * 128 + r - e + pe];
                        const float c0 = first ? v : p, c1 = first ? p : v;      // the pair in its order
                        float sn, cs;
                        sincosf((float)pos * rope.freqs[pair], &sn, &cs);
                        const float r0 = c0 * cs - c1 * sn, r1 = c0 * sn + c1 * cs;
                        v = first ? r0 : r1;
                    }
                    if (head < rope.H) {
                        reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(v);
                    } else if (rope.kpool) {
                        const int pg = rope.table[(size_t)rope.tok_row[n] * rope.max_blocks + pos / rope.page];
                        if (pg < 0 || pg >= rope.num_pages) {
                            mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
                        } else {
                            const int kvh = (head - rope.H) % rope.KV;
                            bf16* pool = head < rope.H + rope.KV ? rope.kpool : rope.vpool;
                            pool[(((size_t)pg * rope.KV + kvh) * rope.page + pos % rope.page) * rope.HD + e] = __float2bfloat16_rn(v);
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");      // xch may be written again
            } else {
#pragma unroll
                for (int a = 0; a < 16; a++) {
                    const int r = cw * 32 + ((a >> 3) & 1) * 16 + g + ((a >> 1) & 1) * 8, n = 8 * ((a >> 2) & 1) + 2 * t + (a & 1);
                    const int m = tile * 128 + r;
                    if (m >= M || n >= N) continue;
                    float v = acc[0][(a >> 3) & 1][(a >> 2) & 1][a & 3];
                    if (NORM) v *= inv_rms[n];
                    if (EPI == 2) {
                        reinterpret_cast<float*>(out)[(size_t)n * M + m] = v;
                    } else if (EPI == 3) {
                        float* dst = reinterpret_cast<float*>(out) + (size_t)n * M + m;
                        v += *dst + (bias ? bias[m] : 0.0f);
                        *dst = v;
                        acc[0][(a >> 3) & 1][(a >> 2) & 1][a & 3] = v;
                    } else if (EPI == 1) {
                        // gate and up pass through bf16 as they do when the products are separate kernels
                        float up = acc[SETS - 1][(a >> 3) & 1][(a >> 2) & 1][a & 3];
                        if (NORM) up *= inv_rms[n];
                        const float gt = bf16_round(v);
                        reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * bf16_round(up));
                    } else {
                        reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(v);
                    }
                }
                if (EPI == 3 && ssq_out) {
                    // the sums of squares of the new rows over this tile's 128 columns, for the norm that follows
                    float sq[2][2];                                   // [nt][token parity]
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int nt = q >> 1, par = q & 1, n = 8 * nt + 2 * t + par;
                        float ss = 0.0f;
#pragma unroll
                        for (int mt = 0; mt < 2; mt++)
#pragma unroll
                            for (int hi8 = 0; hi8 < 2; hi8++) {
                                const int m = tile * 128 + cw * 32 + mt * 16 + g + hi8 * 8;
                                const float v = acc[0][mt][nt][hi8 * 2 + par];
                                if (m < M && n < N) ss = fmaf(v, v, ss);
                            }
                        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 8);
                        ss += __shfl_xor_sync(0xffffffffu, ss, 16);
                        sq[nt][par] = ss;
                    }
                    if (g == 0) {
#pragma unroll
                        for (int q = 0; q < 4; q++) red[cw * S_NT + 8 * (q >> 1) + 2 * t + (q & 1)] = sq[q >> 1][q & 1];
                    }
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    if (t128 < S_NT)
                        ssq_out[tile * S_NT + t128] = (red[t128] + red[S_NT + t128]) + (red[2 * S_NT + t128] + red[3 * S_NT + t128]);
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");  // red may be written again
                }
            }
            if (t128 == 0 && j == range.n_seg - 1) s_mark(7);
        }
    } else if (NORM) {
        // converter w makes half h = w & 1 of the activations of the items w / 2, w / 2 + 2, ...; the values of its
        // next item are on their way while it waits for the stage of this one
        const int cw = warp - 5, h = cw & 1;
        float2 cur[S_NT], nxt[S_NT];
        StreamWalk cwalk(range);
        auto fetch = [&](float2 (&dst)[S_NT]) {
            const int k = cwalk.kb * S_BK + h * 64 + 2 * lane;
            float2 gw = make_float2(0.0f, 0.0f);
            if (k < K) gw = __ldg(reinterpret_cast<const float2*>(nrm.w + k));
#pragma unroll
            for (int n = 0; n < S_NT; n++) {
                float2 x = make_float2(0.0f, 0.0f);
                if (n < N && k < K) x = __ldg(reinterpret_cast<const float2*>(nrm.x + (size_t)n * K + k));
                dst[n] = make_float2(x.x * gw.x, x.y * gw.y);
            }
        };
        long long it = cw >> 1;
        if (it < items) { cwalk.skip((int)it); fetch(cur); }
        for (; it < items; it += S_CONV_WARPS / 2) {
            if (it + S_CONV_WARPS / 2 < items) { cwalk.skip(S_CONV_WARPS / 2); fetch(nxt); }
            const int s = (int)(it % STAGES), round = (int)(it / STAGES);
            if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1, err)) break;
            unsigned char* xs = smem + (size_t)s * STAGE + SETS * S_W_BYTES + h * (S_X_BYTES / 2);
#pragma unroll
            for (int n = 0; n < S_NT; n++)
                if (n < N)
                    *reinterpret_cast<uint32_t*>(xs + n * 128 + (((lane >> 2) ^ (n & 7)) << 4) + ((lane & 3) << 2)) =
                        pack2(cur[n].x, cur[n].y);
            __syncwarp();
            if (lane == 0) mbar_arrive(full0 + 8 * s);
#pragma unroll
            for (int n = 0; n < S_NT; n++) cur[n] = nxt[n];
        }
    }
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

// floats of workspace (two slots of partial sums per block) and ints of counters (one per 128 rows of W, zero before
// the first call; the kernels leave them zero) that a product with M output features needs
MB_API long long mb_gemm_stream_workspace() { return (long long)stream_sms() * 2 * 2 * S_NT * 128; }
MB_API long long mb_gemm_stream_counters(int M) { return (M + 127) / 128; }

template <int EPI, bool NORM>
static int stream_launch(const void* act, const void* W, void* out, int N, int M, int K, float* workspace, int* counters,
                         StreamNorm nrm, const float* bias, StreamRope rope, float* ssq_out, int* err, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    if (N > S_NT || K % 8 || K < 8 || !workspace || !counters || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
    if (NORM ? ((reinterpret_cast<uintptr_t>(nrm.x) & 15) || (reinterpret_cast<uintptr_t>(nrm.w) & 7))
             : (reinterpret_cast<uintptr_t>(act) & 15) != 0)
        return -2;
    if (EPI == 4 && (rope.HD <= 0 || 128 % rope.HD || rope.RD % 2 || rope.RD > rope.HD || M != (rope.H + 2 * rope.KV) * rope.HD))
        return -2;
    constexpr int SETS = EPI == 1 ? 2 : 1;
    constexpr int STAGES = EPI == 1 ? 3 : 6;
    CUtensorMap wmap, xmap;
    int rc = matrix_map(W, (long long)SETS * M, K, 128, &wmap);
    if (rc) return rc;
    if (NORM) xmap = wmap;                                                        // not used
    else if ((rc = matrix_map(act, N, K, S_NT, &xmap))) return rc;
    const size_t smem = 1024 + (size_t)STAGES * (SETS * S_W_BYTES + S_X_BYTES) + 2 * STAGES * 8 + 16 +
                        (S_NT + 4 * S_NT) * 4 + (EPI == 4 ? S_NT * 128 * 4 : 0);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<EPI, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long T = (long long)((M + 127) / 128) * ((K + S_BK - 1) / S_BK);
    const int sms = stream_sms();
    gemm_stream_kernel<EPI, NORM><<<(unsigned)(T < sms ? T : sms), S_THREADS, smem, st>>>(
        wmap, xmap, out, N, M, K, workspace, counters, nrm, bias, rope, ssq_out, err);
    MB_LAUNCH_CHECK();
    return 0;
}

// mode 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out (N, M)
MB_API int mb_gemm_stream(const void* act, const void* W, void* out, int N, int M, int K, int mode, float* workspace,
                          int* counters, int* err, cudaStream_t st) {
    const StreamNorm nn{};
    const StreamRope nr{};
    switch (mode) {
        case 0: return stream_launch<0, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, nr, nullptr, err, st);
        case 1: return stream_launch<1, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, nr, nullptr, err, st);
        case 2: return stream_launch<2, false>(act, W, out, N, M, K, workspace, counters, nn, nullptr, nr, nullptr, err, st);
    }
    return -2;
}

// x (N, M) float32 += act (N, K) bf16 @ W (M, K)^T (+ bias (M) float32 or null), in place.  ssq_out (or null):
// [ceil(M / 128)][16] floats that receive, by row tile, the sums of squares of the new rows of x
MB_API int mb_gemm_stream_residual(const void* act, const void* W, float* x, const float* bias, int N, int M, int K,
                                   float* ssq_out, float* workspace, int* counters, int* err, cudaStream_t st) {
    return stream_launch<3, false>(act, W, x, N, M, K, workspace, counters, StreamNorm{}, bias, StreamRope{}, ssq_out, err, st);
}

// out (N, M) bf16 = rmsnorm(x; norm_w, eps) @ W^T for the float32 residual stream x (N, K); mode 1: SwiGLU.
// ssq (or null): what mb_gemm_stream_residual left for this x, ceil(K / 128) row tiles
MB_API int mb_gemm_stream_normed(const float* x, const float* norm_w, float eps, const float* ssq, const void* W, void* out,
                                 int N, int M, int K, int mode, float* workspace, int* counters, int* err, cudaStream_t st) {
    const StreamNorm nn{x, norm_w, eps, ssq, (K + 127) / 128};
    const StreamRope nr{};
    if (mode == 0) return stream_launch<0, true>(nullptr, W, out, N, M, K, workspace, counters, nn, nullptr, nr, nullptr, err, st);
    if (mode == 1) return stream_launch<1, true>(nullptr, W, out, N, M, K, workspace, counters, nn, nullptr, nr, nullptr, err, st);
    return -2;
}

// the fused q/k/v product of rmsnorm(x) with bias, rotation and the cache write in its epilogue: out (N, M) bf16
// receives the rotated q heads (M = (H + 2 KV) HD), k and v go into the pages of the tokens' positions (kpool null:
// they are dropped)
MB_API int mb_gemm_stream_normed_qkv(const float* x, const float* norm_w, float eps, const float* ssq, const void* W,
                                     void* out, int N, int M, int K, const float* bias, const int* positions,
                                     const int* tok_row, const int* table, int max_blocks, void* kpool, void* vpool,
                                     const float* freqs, int H, int KV, int HD, int RD, int pairing, int page,
                                     int num_pages, float* workspace, int* counters, int* err, cudaStream_t st) {
    StreamRope r;
    r.positions = positions; r.tok_row = tok_row; r.table = table; r.max_blocks = max_blocks;
    r.kpool = (bf16*)kpool; r.vpool = (bf16*)vpool; r.freqs = freqs;
    r.H = H; r.KV = KV; r.HD = HD; r.RD = RD; r.pairing = pairing; r.page = page; r.num_pages = num_pages;
    return stream_launch<4, true>(nullptr, W, out, N, M, K, workspace, counters, StreamNorm{x, norm_w, eps, ssq, (K + 127) / 128},
                                  bias, r, nullptr, err, st);
}
