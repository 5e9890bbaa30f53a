// Paged flash attention with the K/V tiles brought in by the Tensor Memory Accelerator.
//
// Same work decomposition and arithmetic as attention_mma.cu (rows = (token, head-in-group) of one sequence and kv head;
// PREFILL form with 64 rows per block, DECODE form with at most 16 rows and the 64 keys of a tile split over the warps;
// splits over blocks merged by attn_merge_kernel of that file).  What changes is how keys and values reach shared
// memory: one producer warp walks the block table and issues one cp.async.bulk.tensor.2d per (page, 128-byte half of a
// head row) with the 128-byte swizzle, completing on an mbarrier per stage; four consumer warps wait on that barrier,
// run ldmatrix + mma.sync on the tile and hand the stage back through a second mbarrier.  The consumer warps execute
// no address arithmetic and no load instructions for K and V, which is what bounded the cp.async kernel (its decode
// form spent most of its issue slots on them).  Every wait on an mbarrier is bounded: when it runs out the thread
// records MB_ERR_WAIT_TIMEOUT in the engine's error word and returns.
//
// It takes head sizes 64 and 128 and page sizes 8, 16, 32 and 64 (a page's box must cover whole 8-row swizzle atoms and
// a 64-key tile must cover whole pages); other sizes go to attention_mma.cu.  No cluster, no multicast.
#include <cuda.h>
#include <cstdio>
#include <cstring>
#include "attention_common.cuh"

#define TMA_WAIT_LIMIT (1 << 20)

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// false when the wait ran out (the error word is set)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    for (int it = 0; it < TMA_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    mb_set_error(err, MB_ERR_WAIT_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

// thread-block clusters: the barrier over all threads of the cluster that have not exited (a hardware barrier, no
// spinning), and reads of another block's shared memory
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// element offset of 16-byte chunk c of key row `row` in a K or V stage as the TMA lays it out: halves of 64 columns,
// each 64 rows x 128 bytes, 16-byte chunks XORed with the row (the 128-byte swizzle)
template <int HD> __device__ __forceinline__ int kv_off(int row, int c) {
    return (c >> 3) * (64 * 64) + row * 64 + (((c & 7) ^ (row & 7)) << 3);
}

// bias and rotation of the pair (e0, e1) of a head's row: pair i of HD / 2; rotated pairs are (2i, 2i + 1) or, with the
// halves pairing, (i, i + RD / 2); the pairs past the rotated part pass through.  The arithmetic of
// rope_kv_write_vec_kernel (elementwise.cu): float from bf16, + bias, rotation by pos * freq, back to bf16.
struct RopePair { int e0, e1, pair; };
__device__ __forceinline__ RopePair rope_pair(int i, int rd, int pairing) {
    const int rh = rd / 2;
    if (pairing == 0) return RopePair{2 * i, 2 * i + 1, i < rh ? i : -1};
    if (i < rh) return RopePair{i, i + rh, i};
    return RopePair{rd + 2 * (i - rh), rd + 2 * (i - rh) + 1, -1};
}
__device__ __forceinline__ void rope_apply(float& a, float& b, int pair, int pos, const float* __restrict__ freqs) {
    if (pair < 0 || freqs == nullptr) return;
    float s, c;
    sincosf((float)pos * freqs[pair], &s, &c);
    const float ra = a * c - b * s, rb = a * s + b * c;
    a = ra; b = rb;
}

template <int HD, bool DECODE, int STAGES, bool ROPE>
__global__ void __launch_bounds__(160, 2) attn_tma_kernel(const AttnParams P, const __grid_constant__ CUtensorMap kmap,
                                                        const __grid_constant__ CUtensorMap vmap) {
    constexpr int BM = DECODE ? 16 : 64, BN = 64, CH = HD / 8;
    constexpr int NT = DECODE ? 2 : 8;
    constexpr int KS = HD / 16;
    constexpr int DT = HD / 8;
    constexpr int HALVES = HD / 64;
    constexpr int TILE = BN * HD;                        // elements of one K (or V) tile
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem_raw = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    bf16* kvs = reinterpret_cast<bf16*>(smem_raw);                       // STAGES x (K tile, V tile), 1024-byte aligned
    bf16* qs = kvs + (size_t)STAGES * 2 * TILE;                          // BM x HD, swizzled as in attention_mma.cu
    uint64_t* bars = reinterpret_cast<uint64_t*>(qs + BM * HD);          // full[STAGES], empty[STAGES], the merge's flag
    bf16* newkv = reinterpret_cast<bf16*>(bars + 2 * STAGES + 2);         // ROPE: the token's own key and value rows
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);

    // Up to pdl_wait() the kernel reads the step's own arrays only (which no kernel writes); the queries, the pages --
    // the step's own keys and values among them -- and the splits' partial results come after it, by TMA, cp.async.cg
    // and ld.global.cg.
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int4 item = P.items[blockIdx.x];
    const int seq = item.x, m_tile = item.y, split = item.z, n_splits = item.w;
    const int kvh = blockIdx.y;
    const int G = P.G, R = P.q_len[seq] * G, pos0 = P.pos0[seq], tok0 = P.q_start[seq];
    const int row0 = m_tile * BM;
    if (row0 >= R) return;
    const int row_last = min(R, row0 + BM) - 1;
    const int pos_min = pos0 + row0 / G, pos_max = pos0 + row_last / G;
    const int hi = pos_max + 1;
    const int lo = (P.window > 0 && pos_min - P.window + 1 > 0) ? pos_min - P.window + 1 : 0;
    const int lo_al = (lo / BN) * BN;
    const int n_tiles = (hi - lo_al + BN - 1) / BN;
    const int tps = (n_tiles + n_splits - 1) / n_splits;
    const int t_begin = split * tps, t_end = min(n_tiles, t_begin + tps);
    const int* tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
    // With the rotation folded in, nothing the producer warp reads is written by a kernel of this step: the pages hold
    // the keys and values of earlier steps (the token's own rows never come from the page, see below) and the block table
    // is the step's input.  So it does not wait: the first tiles are on their way while the q/k/v product still runs.
    if (!ROPE || warp != 4) pdl_wait();

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        // Every copy of a tile is issued by a lane of its own: lane = (K or V, page of the tile, 64-column half).  One
        // thread issuing them one after the other took thousands of cycles per tile and bounded the whole block.  The
        // lane's page id is read from the block table one tile ahead.
        const int shift = P.page_shift, page = P.page;
        const int boxes = (BN >> shift) * HALVES;                   // per operand: 1 .. 16
        const int which = lane / boxes, b = lane % boxes;           // which: 0 = K, 1 = V (lanes past 2 * boxes idle)
        const int p = b / HALVES, h = b % HALVES;
        const bool active = lane < 2 * boxes;
        auto page_of = [&](int t) -> int {
            const int key0 = lo_al + t * BN + p * page, block = key0 >> shift;
            const bool live = active && key0 < hi && key0 + page > lo && block < P.max_blocks;
            return live ? __ldg(tb + block) : 0;
        };
        int pg = (t_begin < t_end) ? page_of(t_begin) : 0;
        for (int t = t_begin; t < t_end; t++) {
            const int i = t - t_begin, s = i % STAGES, round = i / STAGES;
            const int pg_next = (t + 1 < t_end) ? page_of(t + 1) : 0;
            const bool ok = round == 0 || mbar_wait(empty0 + 8 * s, (round - 1) & 1, P.err);
            if (!__all_sync(0xffffffffu, ok)) return;
            const uint32_t fb = full0 + 8 * s;
            if (lane == 0) mbar_expect_tx(fb, 2u * TILE * 2u);
            __syncwarp();
            if (active) {
                const int key0 = lo_al + t * BN + p * page;
                if (pg < 0 || pg >= P.num_pages) {
                    if (key0 < hi && key0 + page > lo) mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
                    pg = 0;                                            // any page: every key of it is masked
                }
                const uint32_t dst = smem_u32(kvs + (size_t)s * 2 * TILE) + which * TILE * 2 +
                                     (uint32_t)(h * 64 * 64 + p * page * 64) * 2u;
                tma_load_2d(dst, which ? &vmap : &kmap, h * 64, (pg * P.KV + kvh) * page, fb);
            }
            pg = pg_next;
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    for (int cid = tid; cid < BM * CH; cid += 128) {
        const int row = cid / CH, c = cid % CH, r = row0 + row;
        const bf16* src = P.q;
        int bytes = 0;
        if (r < R) {
            src = P.q + (size_t)(tok0 + r / G) * P.q_stride + (size_t)(kvh * G + r % G) * HD + c * 8;
            bytes = 16;
        }
        cp_async16(qs + swz<HD>(row, c), src, bytes);
    }
    cp_async_commit();

    const int m0 = DECODE ? 0 : warp * 16;
    const int nbase = DECODE ? warp * 16 : 0;
    int rpos[2], rlo[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = row0 + m0 + g + i * 8;
        if (r < R) {
            rpos[i] = pos0 + r / G;
            rlo[i] = (P.window > 0 && rpos[i] - P.window + 1 > 0) ? rpos[i] - P.window + 1 : 0;
        } else {
            rpos[i] = -1; rlo[i] = 0;
        }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; d++) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.0f; }

    cp_async_wait<0>();
    consumer_sync();
    if (ROPE) {
        // The rotate-and-store step of a one-token sequence, folded in.  Every block rotates the G query rows it has
        // just fetched, in shared memory.  The block whose splits hold the token's own key tile also makes the token's
        // key and value rows (bias, rotation), writes them to the token's page for the steps to come, and keeps them in
        // shared memory: when that tile arrives it holds whatever the page held before at the token's slot, and the warp
        // that owns the slot's keys puts the new rows there before it reads the tile.
        const int pos = pos0, rd = P.rope_rd, pairing = P.rope_pairing;
        for (int idx = tid; idx < G * (HD / 2); idx += 128) {
            const int row = idx / (HD / 2);
            const RopePair rp = rope_pair(idx % (HD / 2), rd, pairing);
            bf16* p0 = qs + swz<HD>(row, rp.e0 >> 3) + (rp.e0 & 7);
            bf16* p1 = qs + swz<HD>(row, rp.e1 >> 3) + (rp.e1 & 7);
            float a = __bfloat162float(*p0), b = __bfloat162float(*p1);
            if (P.rope_bias) {
                const float* bh = P.rope_bias + (size_t)(kvh * G + row) * HD;
                a += bh[rp.e0]; b += bh[rp.e1];
            }
            rope_apply(a, b, rp.pair, pos, P.rope_freqs);
            *p0 = __float2bfloat16_rn(a);
            *p1 = __float2bfloat16_rn(b);
        }
        if (t_begin <= n_tiles - 1 && n_tiles - 1 < t_end) {
            const int pg = tb[pos / P.page];
            const bool paged = pg >= 0 && pg < P.num_pages;
            if (!paged && tid == 0) mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            const size_t slot = (((size_t)(paged ? pg : 0) * P.KV + kvh) * P.page + pos % P.page) * HD;
            const unsigned short* raw = reinterpret_cast<const unsigned short*>(P.q + (size_t)tok0 * P.q_stride);
            for (int idx = tid; idx < HD; idx += 128) {
                const bool is_v = idx >= HD / 2;
                const RopePair rp = is_v ? RopePair{2 * (idx - HD / 2), 2 * (idx - HD / 2) + 1, -1} : rope_pair(idx, rd, pairing);
                const int head = is_v ? P.H + P.KV + kvh : P.H + kvh;
                float a = __uint_as_float((uint32_t)__ldcg(raw + (size_t)head * HD + rp.e0) << 16);
                float b = __uint_as_float((uint32_t)__ldcg(raw + (size_t)head * HD + rp.e1) << 16);
                if (P.rope_bias) { a += P.rope_bias[(size_t)head * HD + rp.e0]; b += P.rope_bias[(size_t)head * HD + rp.e1]; }
                rope_apply(a, b, rp.pair, pos, P.rope_freqs);
                const bf16 ra = __float2bfloat16_rn(a), rb = __float2bfloat16_rn(b);
                bf16* mine = newkv + (is_v ? HD : 0);
                mine[rp.e0] = ra; mine[rp.e1] = rb;
                if (paged) {
                    bf16* pool = const_cast<bf16*>(is_v ? P.vpool : P.kpool) + slot;
                    pool[rp.e0] = ra; pool[rp.e1] = rb;
                }
            }
        }
        consumer_sync();
    }
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        ldmatrix_x4(qf[ks], qs + swz<HD>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));

    for (int t = t_begin; t < t_end; t++) {
        const int i = t - t_begin, s = i % STAGES, round = i / STAGES;
        if (!mbar_wait(full0 + 8 * s, round & 1, P.err)) return;
        const bf16* kt = kvs + (size_t)s * 2 * TILE;
        const bf16* vt = kt + TILE;
        const int kb = lo_al + t * BN;
        if (ROPE && DECODE && t == n_tiles - 1 && pos0 - kb >= nbase && pos0 - kb < nbase + 16) {
            // the token's own slot is among this warp's keys of the tile: its new key and value rows go in
            const int rowk = pos0 - kb;
            for (int c = lane; c < 2 * CH; c += 32) {
                bf16* tile = const_cast<bf16*>(c < CH ? kt : vt);
                *reinterpret_cast<uint4*>(tile + kv_off<HD>(rowk, c % CH)) =
                    *reinterpret_cast<const uint4*>(newkv + (c < CH ? 0 : HD) + (c % CH) * 8);
            }
            __syncwarp();
        }

        float sc[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + kv_off<HD>(nbase + np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(sc[2 * np], qf[ks], b[0], b[1]);
                mma_bf16(sc[2 * np + 1], qf[ks], b[2], b[3]);
            }
        }
        // a tile whose keys every row of the block may read needs no mask (all tiles but the last and, with a window,
        // the first ones); rows past the end of the block then get finite scores, and they are never written
        const bool full_tile = kb + BN - 1 <= pos_min && kb >= ((P.window > 0) ? pos_max - P.window + 1 : 0);
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int ii = e >> 1;
                float v = sc[j][e] * P.scale_log2;
                if (!full_tile) {
                    const int key = kb + nbase + j * 8 + 2 * tig + (e & 1);
                    if (!(key <= rpos[ii] && key >= rlo[ii])) v = -INFINITY;
                }
                sc[j][e] = v;
                tmax[ii] = fmaxf(tmax[ii], v);
            }
        }
        float corr[2], muse[2];
#pragma unroll
        for (int ii = 0; ii < 2; ii++) {
            tmax[ii] = fmaxf(tmax[ii], __shfl_xor_sync(0xffffffffu, tmax[ii], 1));
            tmax[ii] = fmaxf(tmax[ii], __shfl_xor_sync(0xffffffffu, tmax[ii], 2));
            const float m_new = fmaxf(m_run[ii], tmax[ii]);
            muse[ii] = (m_new == -INFINITY) ? 0.0f : m_new;
            corr[ii] = exp2f(m_run[ii] - muse[ii]);
            m_run[ii] = m_new;
            l_run[ii] *= corr[ii];
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(sc[j][e] - muse[e >> 1]);
                l_run[e >> 1] += p;
                sc[j][e] = p;
            }
        }
        // the running maximum rarely moves after the first tiles: rescale the accumulators only when it did
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
            for (int d = 0; d < DT; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
        }
#pragma unroll
        for (int kk = 0; kk < NT / 2; kk++) {
            uint32_t a[4];
            a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
            a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
            a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
            a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; dp++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + kv_off<HD>(nbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);           // this warp is done with the stage
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    const int H = P.H;
    if (!DECODE) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = row0 + m0 + g + i * 8;
            if (r >= R) continue;
            const int tq = r / G, h = kvh * G + r % G;
            if (n_splits == 1) {
                const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
                bf16* dst = P.out + ((size_t)(tok0 + tq) * H + h) * HD + 2 * tig;
#pragma unroll
                for (int d = 0; d < DT; d++)
                    *reinterpret_cast<uint32_t*>(dst + d * 8) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
            } else {
                const size_t base = ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits + split;
                float* dst = P.part_o + base * HD + 2 * tig;
#pragma unroll
                for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
                if (tig == 0) { P.part_ml[base * 2] = m_run[i]; P.part_ml[base * 2 + 1] = l_run[i]; }
            }
        }
    } else {
        consumer_sync();                                    // every consumer warp is done with the K/V stages
        float* mo = reinterpret_cast<float*>(kvs);          // [4 warps][16 rows][HD]
        float* sm_m = mo + 4 * 16 * HD;
        float* sm_l = sm_m + 4 * 16;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int row = g + i * 8;
            float* dst = mo + ((size_t)(warp * 16 + row)) * HD + 2 * tig;
#pragma unroll
            for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
            if (tig == 0) { sm_m[warp * 16 + row] = m_run[i]; sm_l[warp * 16 + row] = l_run[i]; }
        }
        consumer_sync();
        for (int idx = tid; idx < 16 * HD; idx += 128) {
            const int row = idx / HD, d = idx % HD, r = row0 + row;
            if (r >= R) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w * 16 + row]);
            float acc = 0.0f, L = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float mw = sm_m[w * 16 + row];
                const float scl = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
                acc += mo[((size_t)(w * 16 + row)) * HD + d] * scl;
                L += sm_l[w * 16 + row] * scl;
            }
            const int tq = r / G, h = kvh * G + r % G;
            if (n_splits == 1) {
                P.out[((size_t)(tok0 + tq) * H + h) * HD + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
            } else if (P.cluster > 1) {
                // the split's result stays in this block's shared memory (behind the warps' partial results)
                float* fin = mo + 4 * 16 * HD + 2 * 4 * 16;             // [16 rows][HD], then [16 rows][2]
                fin[row * HD + d] = acc;
                if (d == 0) { fin[16 * HD + 2 * row] = M; fin[16 * HD + 2 * row + 1] = L; }
            } else {
                const size_t base = ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits + split;
                P.part_o[base * HD + d] = acc;
                if (d == 0) { P.part_ml[base * 2] = M; P.part_ml[base * 2 + 1] = L; }
            }
        }
    }
    // Launched as clusters (one block per split of a sequence and kv head), the splits meet in shared memory: after a
    // barrier over the cluster every block reads, for its share of the head's columns, all splits' sums in the order of
    // the splits and writes the rows; a second barrier keeps a block's memory alive until its neighbours have read it.
    // (The producer warp has exited by now; the barrier counts the threads that have not.)
    if (DECODE && n_splits > 1 && P.cluster > 1) {
        cluster_sync();
        const float* fin = reinterpret_cast<const float*>(kvs) + 4 * 16 * HD + 2 * 4 * 16;
        const uint32_t fin_addr = smem_u32(fin);
        const int rows = min(BM, R - row0), per = (HD + n_splits - 1) / n_splits;      // columns of a row this block writes
        for (int it = tid; it < rows * per; it += 128) {
            const int row = it / per, d = split * per + it % per, r = row0 + row;
            if (d >= HD) continue;
            float M = -INFINITY;
            for (int s = 0; s < n_splits; s++) M = fmaxf(M, cluster_ld(cluster_map(fin_addr + (16 * HD + 2 * row) * 4, s)));
            float acc = 0.0f, L = 0.0f;
            for (int s = 0; s < n_splits; s++) {                      // in the order of the splits
                const uint32_t base = cluster_map(fin_addr, s);
                const float ms = cluster_ld(base + (16 * HD + 2 * row) * 4);
                const float sc = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
                L += cluster_ld(base + (16 * HD + 2 * row + 1) * 4) * sc;
                acc += cluster_ld(base + (row * HD + d) * 4) * sc;
            }
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;
            P.out[((size_t)(tok0 + r / G) * H + kvh * G + r % G) * HD + d] = __float2bfloat16_rn(acc * inv);
        }
        cluster_sync();
        return;
    }
    // The splits of a tile are merged by whichever of their blocks finishes last: every block publishes its partial
    // result, then draws a ticket; the one that draws the last ticket reads all of them back (in the order of the
    // splits, so the sum does not depend on who came last), writes the rows and sets the counter back to zero for the
    // next launch.  Without counters a separate kernel does the merge.
    if (n_splits > 1 && P.counters != nullptr) {
        int* flag = reinterpret_cast<int*>(bars + 2 * STAGES);
        __threadfence();
        consumer_sync();
        if (tid == 0) {
            int* counter = P.counters + (size_t)(blockIdx.x - split) * P.KV + kvh;
            const int ticket = atomicAdd(counter, 1);
            *flag = ticket == n_splits - 1;
            if (ticket == n_splits - 1) *counter = 0;
        }
        consumer_sync();
        if (*flag) {
            __threadfence();
            // the K/V stages are free by now: the splits' (maximum, sum) pairs go there, then their weights
            float* sm_w = reinterpret_cast<float*>(kvs);              // [rows][n_splits]: maxima, then weights 2^(m - M)
            float* sm_l = sm_w + BM * n_splits;                       // [rows][n_splits]: sums
            float* sm_tot = sm_l + BM * n_splits;                     // [rows]: the total of a row
            const int rows = min(BM, R - row0);
            for (int i = tid; i < rows * n_splits; i += 128) {
                const int r = row0 + i / n_splits, s = i % n_splits;
                const size_t base = ((size_t)(P.part_base[seq] + r / G) * H + kvh * G + r % G) * P.max_splits + s;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(P.part_ml + base * 2));
                sm_w[i] = ml.x;
                sm_l[i] = ml.y;
            }
            consumer_sync();
            if (tid < rows) {
                float M = -INFINITY, L = 0.0f;
                for (int s = 0; s < n_splits; s++) M = fmaxf(M, sm_w[tid * n_splits + s]);
                for (int s = 0; s < n_splits; s++) {
                    const float ms = sm_w[tid * n_splits + s];
                    const float sc = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
                    sm_w[tid * n_splits + s] = sc;
                    L += sm_l[tid * n_splits + s] * sc;
                }
                sm_tot[tid] = L;
            }
            consumer_sync();
            for (int it = tid; it < rows * (HD / 4); it += 128) {
                const int row = it / (HD / 4), d = (it % (HD / 4)) * 4, r = row0 + row;
                const int tq = r / G, h = kvh * G + r % G;
                const float* src = P.part_o + ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits * HD + d;
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
                for (int s = 0; s < n_splits; s++) {                  // in the order of the splits, whoever came last
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)s * HD));
                    const float sc = sm_w[row * n_splits + s];
                    acc.x += v.x * sc; acc.y += v.y * sc; acc.z += v.z * sc; acc.w += v.w * sc;
                }
                const float L = sm_tot[row], inv = L > 0.0f ? 1.0f / L : 0.0f;
                uint2 o;
                o.x = pack_bf16(acc.x * inv, acc.y * inv);
                o.y = pack_bf16(acc.z * inv, acc.w * inv);
                *reinterpret_cast<uint2*>(P.out + ((size_t)(tok0 + tq) * H + h) * HD + d) = o;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

struct MapKey { const void* ptr; long long rows; int hd, page; };
struct MapEntry { MapKey key; CUtensorMap map; };
#define MAP_CACHE 512
static MapEntry map_cache[MAP_CACHE];
static int map_count = 0;

// the pool [pages][KV][page][HD] seen as a matrix of (pages * KV * page) rows of HD values; box = one page of one kv
// head, 64 columns wide, 128-byte swizzle
static int pool_map(const void* pool, long long rows, int HD, int page, CUtensorMap* out) {
    for (int i = 0; i < map_count; i++) {
        const MapKey& k = map_cache[i].key;
        if (k.ptr == pool && k.rows == rows && k.hd == HD && k.page == page) { *out = map_cache[i].map; return 0; }
    }
    EncodeTiled enc = encode_fn();
    if (!enc) return -6;
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)page};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -6;
    if (map_count < MAP_CACHE) {
        map_cache[map_count].key = MapKey{pool, rows, HD, page};
        map_cache[map_count].map = m;
        map_count++;
    }
    *out = m;
    return 0;
}

MB_PDL_SWITCH(mb_attn_tma_set_pdl)

template <int HD, bool DECODE, int STAGES, bool ROPE = false>
static int launch_tma(const AttnParams& P, const CUtensorMap& kmap, const CUtensorMap& vmap, int n_items, cudaStream_t st) {
    constexpr int BM = DECODE ? 16 : 64;
    const size_t smem = 1024 + (size_t)STAGES * 2 * 64 * HD * 2 + (size_t)BM * HD * 2 + 2 * STAGES * 8 + 16 + (ROPE ? 4 * HD : 0);
    static bool configured = false;
    static int max_cluster = 1;         // the largest cluster of these blocks the device can place (a power of two up to 8)
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tma_kernel<HD, DECODE, STAGES, ROPE>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        // two blocks per SM need most of the SM's memory as shared memory: ask for the largest carve-out
        cudaFuncSetAttribute(attn_tma_kernel<HD, DECODE, STAGES, ROPE>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
        if (DECODE) {
            // Clusters of up to 8 blocks (the portable size).  Clusters of 16 can be placed too, but were slower wherever
            // they applied (two sequences of 8,192 keys: 29.5 us against 18.6 us for 16 splits that meet through global
            // memory): a cluster of 16 of these blocks needs eight SMs of one GPC free at once.
            for (int c = 8; c > 1; c /= 2) {
                cudaLaunchAttribute attr;
                attr.id = cudaLaunchAttributeClusterDimension;
                attr.val.clusterDim.x = c; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(c, 1); cfg.blockDim = dim3(160); cfg.dynamicSmemBytes = smem; cfg.attrs = &attr; cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, attn_tma_kernel<HD, DECODE, STAGES, ROPE>, &cfg) == cudaSuccess && n >= 1) {
                    max_cluster = c;
                    break;
                }
                cudaGetLastError();
            }
        }
        configured = true;
    }
    if (n_items == -1) return max_cluster;               // a query (mb_attn_tma_max_cluster)
    if (n_items < -1) {                                  // a query: how many clusters of -n_items blocks the device holds at once
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = -n_items; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(-n_items, 1); cfg.blockDim = dim3(160); cfg.dynamicSmemBytes = smem; cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, attn_tma_kernel<HD, DECODE, STAGES, ROPE>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        return n;
    }
    if (P.cluster > max_cluster || (P.cluster > 1 && n_items % P.cluster)) return -2;
    const cudaError_t e = mb_launch_cluster(mb_pdl != 0, P.cluster > 1 ? P.cluster : 1, attn_tma_kernel<HD, DECODE, STAGES, ROPE>,
                                            dim3(n_items, P.KV), dim3(160), smem, st, P, kmap, vmap);
    return e == cudaSuccess ? 0 : (int)e;
}

MB_API int mb_attn_tma_supports(int HD, int page) {
    return (HD == 64 || HD == 128) && (page == 8 || page == 16 || page == 32 || page == 64);
}

// fuse: 0, or 1 for the decode form with the rotate-and-store step folded in (then every sequence of the step brings ONE
// token, q points at the rows [q | k | v] the q/k/v product left, and bias / freqs / RD / pairing are those of
// mb_rope_kv_write_bf16)
static int attn_tma_run(const void* q, int q_stride, void* out, const void* kpool, const void* vpool,
                        const void* items, int n_items, int decode, const int* q_start, const int* q_len,
                        const int* pos0, const int* part_base, const int* seq_row, const int* table, int max_blocks,
                        float* part_o, float* part_ml, int max_splits, int H, int KV, int HD, int page, int num_pages,
                        int window, float scale, int* counters, int* err, cudaStream_t st, int fuse, const float* bias,
                        const float* freqs, int RD, int pairing, int cluster = 0) {
    if (n_items == 0) return 0;
    if (cluster > 1 && (!decode || cluster > 8)) return -2;
    if (!mb_attn_tma_supports(HD, page) || KV < 1 || H % KV || KV > 65535) return -2;
    if (fuse && (!decode || H / KV > 16 || RD % 2 || RD > HD || RD < 0 || !kpool || !vpool)) return -2;
    AttnParams P;
    P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out;
    P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = (const int4*)items;
    P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.part_base = part_base; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.part_o = part_o; P.part_ml = part_ml; P.max_splits = max_splits; P.counters = counters;
    P.H = H; P.KV = KV; P.G = H / KV; P.page = page; P.num_pages = num_pages; P.window = window;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    P.cluster = cluster > 1 ? cluster : 0;
    P.fuse_rope = fuse; P.rope_bias = bias; P.rope_freqs = freqs; P.rope_rd = freqs ? RD : 0; P.rope_pairing = pairing;
    CUtensorMap kmap, vmap;
    const long long rows = (long long)num_pages * KV * page;
    int rc = pool_map(kpool, rows, HD, page, &kmap);
    if (rc) return rc;
    rc = pool_map(vpool, rows, HD, page, &vmap);
    if (rc) return rc;
    if (fuse) return HD == 128 ? launch_tma<128, true, 3, true>(P, kmap, vmap, n_items, st)
                               : launch_tma<64, true, 4, true>(P, kmap, vmap, n_items, st);
    if (HD == 128) return decode ? launch_tma<128, true, 3>(P, kmap, vmap, n_items, st)
                                 : launch_tma<128, false, 2>(P, kmap, vmap, n_items, st);
    return decode ? launch_tma<64, true, 4>(P, kmap, vmap, n_items, st)
                  : launch_tma<64, false, 3>(P, kmap, vmap, n_items, st);
}

MB_API int mb_attn_tma_bf16(const void* q, int q_stride, void* out, const void* kpool, const void* vpool,
                            const void* items, int n_items, int decode, const int* q_start, const int* q_len,
                            const int* pos0, const int* part_base, const int* seq_row, const int* table, int max_blocks,
                            float* part_o, float* part_ml, int max_splits, int H, int KV, int HD, int page, int num_pages,
                            int window, float scale, int* counters, int* err, cudaStream_t st) {
    return attn_tma_run(q, q_stride, out, kpool, vpool, items, n_items, decode, q_start, q_len, pos0, part_base, seq_row,
                        table, max_blocks, part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale,
                        counters, err, st, 0, nullptr, nullptr, 0, 0);
}

// The decode form for a step in which every sequence brings one token, with the rotate-and-store step folded in: qkv
// (N, (H + 2 KV) HD) as the q/k/v product left it.  The result equals mb_rope_kv_write_bf16 followed by
// mb_attn_tma_bf16 bit for bit (qkv itself is left as it was: the rotated queries exist in shared memory only).
MB_API int mb_attn_tma_rope_bf16(const void* qkv, int q_stride, void* out, void* kpool, void* vpool, const void* items,
                                 int n_items, const int* q_start, const int* q_len, const int* pos0, const int* part_base,
                                 const int* seq_row, const int* table, int max_blocks, float* part_o, float* part_ml,
                                 int max_splits, int H, int KV, int HD, int page, int num_pages, int window, float scale,
                                 int* counters, int* err, const float* bias, const float* freqs, int RD, int pairing,
                                 cudaStream_t st) {
    return attn_tma_run(qkv, q_stride, out, kpool, vpool, items, n_items, 1, q_start, q_len, pos0, part_base, seq_row, table,
                        max_blocks, part_o, part_ml, max_splits, H, KV, HD, page, num_pages, window, scale, counters,
                        err, st, 1, bias, freqs, RD, pairing);
}

// The decode form launched as thread-block clusters: every sequence of the launch is cut into `cluster` splits (2 to
// 8; the items of a sequence in the order of the splits), a cluster is the splits of one sequence and kv head, and
// their results meet in the cluster's shared memory instead of global memory: no partial buffers, no counters.  rope:
// as mb_attn_tma_rope_bf16 (bias / freqs may be null), 0: q is the rotated queries as for mb_attn_tma_bf16.
MB_API int mb_attn_tma_cluster_bf16(const void* q, int q_stride, void* out, void* kpool, void* vpool, const void* items,
                                    int n_items, const int* q_start, const int* q_len, const int* pos0, const int* seq_row,
                                    const int* table, int max_blocks, int cluster, int H, int KV, int HD, int page,
                                    int num_pages, int window, float scale, int* err, int rope, const float* bias,
                                    const float* freqs, int RD, int pairing, cudaStream_t st) {
    if (cluster < 2) return -2;
    return attn_tma_run(q, q_stride, out, kpool, vpool, items, n_items, 1, q_start, q_len, pos0, nullptr, seq_row, table,
                        max_blocks, nullptr, nullptr, cluster, H, KV, HD, page, num_pages, window, scale, nullptr, err, st,
                        rope, bias, freqs, RD, pairing, cluster);
}

static int attn_tma_query(int HD, int rope, int what) {
    AttnParams P{};
    CUtensorMap m{};
    if (HD == 128) return rope ? launch_tma<128, true, 3, true>(P, m, m, what, nullptr) : launch_tma<128, true, 3>(P, m, m, what, nullptr);
    return rope ? launch_tma<64, true, 4, true>(P, m, m, what, nullptr) : launch_tma<64, true, 4>(P, m, m, what, nullptr);
}

// the largest cluster mb_attn_tma_cluster_bf16 can be given on this device for this head size (1: none)
MB_API int mb_attn_tma_max_cluster(int HD, int rope) {
    if (HD != 64 && HD != 128) return 1;
    return attn_tma_query(HD, rope, -1);
}

// how many clusters of `cluster` (2 to 8) such blocks the device holds at the same time (0: none)
MB_API int mb_attn_tma_active_clusters(int HD, int rope, int cluster) {
    if ((HD != 64 && HD != 128) || cluster < 2 || cluster > 8) return 0;
    return attn_tma_query(HD, rope, -cluster);
}
