// Paged flash attention for prompt portions on the 5th-generation tensor cores, head sizes 64 and 128.
//
// A work unit is 256 packed query rows -- (token, head-in-group) of one sequence and one kv head -- as TWO query tiles
// of 128 rows that share the K and V tiles, against the keys up to the last row's position, 128 keys at a time.  A
// block of 384 threads walks a static list of units (sorted heaviest first, dealt back and forth over the blocks):
//   warps 0-3, 4-7  softmax, one warpgroup per query tile, thread = row.  tcgen05.ld brings the row's 128 scores with one
//              wait; maximum and sum need no shuffle; the probabilities go back as bf16 pairs into the first 64 columns
//              of their own scores in tensor memory, where the output product reads them as its A operand.  The output
//              accumulator stays in tensor memory over all tiles; a row rescales its lane of it (tcgen05.ld / st) only
//              when its running maximum has grown by more than 8.  At the end the row is normalised and written.  The
//              warpgroup also fetches its query tile of the NEXT unit before this unit's output is written.
//   warp 8     producer: walks the block table and brings each K and V tile in with one cp.async.bulk.tensor.2d per
//              page and 64-column half (128-byte swizzle), one lane per box, page ids read one tile ahead; two stages.
//   warp 9     one thread issues the products, for the two query tiles in turn: O_g += P_g V (M = 128 rows, N = head
//              size, 8 k-steps over the keys; V is the MN-major operand, read as the TMA laid it out), then
//              S_g = Q_g K^T of the next key tile (M = 128, N = 128 keys, head size / 16 k-steps), so the products of
//              one query tile run under the softmax of the other.
// Tensor memory (512 columns): scores of tile g in columns g * 128, outputs of tile g from column 256 + g * head size.
// The roles keep their barriers and phase counts from unit to unit; nothing is handed out at run time and there is
// no block-wide barrier between units.  Softmax, scale and running sums are float32.  Every mbarrier wait is bounded;
// every role reaches the common exit, where the tensor memory is given back.  Page sizes 8..128 (powers of two); other
// sizes and head sizes go to the mma.sync kernels.
#include "tcgen05.cuh"
#include "attention_common.cuh"

#define T5_BM 128                              // rows of one query tile: one softmax warpgroup, thread = row
#define T5_QT 2                                // query tiles of a block, sharing the K and V tiles
#define T5_ROWS (T5_BM * T5_QT)
#define T5_THREADS (T5_QT * T5_BM + 128)       // two softmax warpgroups; a third holds the producer warp and the product warp
#define T5_BN 128
#define T5_HALF (128 * 128)                    // bytes of 128 rows of 64 bf16: what one 128-byte-swizzled column half of a tile takes
#ifndef T5_POLY
#define T5_POLY 0                              // pairs in eight whose 2^x is a polynomial on the FMA units (it paid at
#endif                                         // neither head size: 938 us -> 994 / 1,016 / 1,082 us with 2 / 4 / 6 at 64)
// 2^x with the special-function unit (ex2.approx.ftz: 2 ulp; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Two floats in one 64-bit register pair and the packed arithmetic on them (one issue slot for two results); a maximum
// of three.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fsub2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x for two values without the special-function unit, which a softmax over 128 x 128 scores keeps as busy as the
// tensor cores: x = n + f with n the nearest integer (taken from the low mantissa bits of x + 1.5 * 2^23) and f in
// [-1/2, 1/2]; 2^f by a cubic (relative error 7.5e-5, a thirtieth of a bf16 rounding step); n goes into the exponent.
// x is clamped at -126, so masked scores (-inf) come out as 2^-126 instead of 0.
__device__ __forceinline__ void poly_exp2_pair(uint64_t x2, float& ra, float& rb) {
    float xa, xb;
    unpack2(x2, xa, xb);
    const uint64_t xc = pack2(fmaxf(xa, -126.0f), fmaxf(xb, -126.0f));
    const uint64_t magic = pack2(12582912.0f, 12582912.0f);
    const uint64_t fi = fadd2(xc, magic);
    const uint64_t fr = fsub2(xc, fsub2(fi, magic));
    uint64_t p = ffma2(pack2(0.0551716685f, 0.0551716685f), fr, pack2(0.2426111251f, 0.2426111251f));
    p = ffma2(p, fr, pack2(0.6932609677f, 0.6932609677f));
    p = ffma2(p, fr, pack2(0.9999280572f, 0.9999280572f));
    float pa, pb, ia, ib;
    unpack2(p, pa, pb);
    unpack2(fi, ia, ib);
    ra = __uint_as_float(__float_as_uint(pa) + (__float_as_uint(ia) << 23));
    rb = __uint_as_float(__float_as_uint(pb) + (__float_as_uint(ib) << 23));
}

// The shared-memory matrix descriptor (128-byte swizzle, version 1) in two halves.  Only the low word changes from product to product (start address in bits 0-13,
// leading byte offset in bits 16-29), so the issuing thread keeps one low word per operand and adds a constant: built
// whole for every product, the descriptors cost that one thread more time than the products take to run.
constexpr uint32_t T5_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);       // stride byte offset 1024, version 1, 128-byte swizzle
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t addr, uint32_t lbo) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ uint64_t umma_desc_join(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(d) : "r"(lo), "r"(T5_DESC_HI));
    return d;
}

// One work unit: 256 packed rows of one sequence and one kv head, as two query tiles, and the key tiles they read.
struct T5Unit {
    int kvh, row0, R, G, pos0, tok0, lo, lo_al, T, hi;
    int T0, T1, pmin0, pmin1, pmax0, pmax1;                         // per query tile: key tiles, first and last position
    const int* tb;
    __device__ __forceinline__ int tiles(int g) const { return g == 0 ? T0 : T1; }
    __device__ __forceinline__ int pmin(int g) const { return g == 0 ? pmin0 : pmin1; }
    __device__ __forceinline__ int pmax(int g) const { return g == 0 ? pmax0 : pmax1; }
};
__device__ __forceinline__ bool t5_unit(const AttnParams& P, int unit, T5Unit& U) {
    const int4 item = P.items[unit / P.KV];
    const int seq = item.x;
    U.kvh = unit % P.KV;
    U.G = P.G; U.R = P.q_len[seq] * P.G; U.pos0 = P.pos0[seq]; U.tok0 = P.q_start[seq];
    U.row0 = item.y * T5_ROWS;
    if (U.row0 >= U.R) return false;
    const int pos_min = U.pos0 + U.row0 / U.G;
    U.lo = (P.window > 0 && pos_min - P.window + 1 > 0) ? pos_min - P.window + 1 : 0;
    U.lo_al = (U.lo / T5_BN) * T5_BN;
    U.pmin0 = pos_min;
    U.pmax0 = U.pos0 + (min(U.R, U.row0 + T5_BM) - 1) / U.G;
    U.T0 = (U.pmax0 + 1 - U.lo_al + T5_BN - 1) / T5_BN;             // at least one
    const int r1 = U.row0 + T5_BM;
    if (r1 < U.R) {
        U.pmin1 = U.pos0 + r1 / U.G;
        U.pmax1 = U.pos0 + (min(U.R, r1 + T5_BM) - 1) / U.G;
        U.T1 = (U.pmax1 + 1 - U.lo_al + T5_BN - 1) / T5_BN;
    } else {
        U.pmin1 = U.pmax1 = 0;
        U.T1 = 0;
    }
    U.T = max(U.T0, U.T1);
    U.hi = max(U.pmax0, U.pmax1) + 1;
    U.tb = P.table + (size_t)P.seq_row[seq] * P.max_blocks;
    return true;
}
// The units are sorted heaviest first; block b takes units b, 2g-1-b, 2g+b, 4g-1-b, ... (g blocks): back and forth over
// the sorted list, so the block with the heaviest unit of one round gets the lightest of the next.  Every role of the
// block walks the same list by itself: nothing is handed out at run time and no role waits for another between units.
__device__ __forceinline__ int t5_unit_at(int k, int n_units) {
    const int g = gridDim.x, b = blockIdx.x;
    const int u = k * g + ((k & 1) ? g - 1 - b : b);
    return u < n_units ? u : -1;
}

template <int HD>
__global__ void __launch_bounds__(T5_THREADS, 1) attn_tc5_kernel(const AttnParams P, const __grid_constant__ CUtensorMap kmap,
                                                                  const __grid_constant__ CUtensorMap vmap, int n_units) {
    constexpr int HALVES = HD / 64;                 // 64-column halves of a row of a tile (one TMA box wide each)
    constexpr int TILE = T5_BN * HD * 2;            // bytes of one K or V tile, and of one query tile
    constexpr int OC = HD / 32;                     // 32-column groups of a row of the output
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    // 2 x Q tile | 2 stages x K tile | 2 stages x V tile (32 KB each at head size 128, 16 KB at 64) | barriers
    const uint32_t q_s0 = smem_u32(smem), k_s0 = q_s0 + T5_QT * TILE, v_s0 = k_s0 + 2 * TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T5_QT * TILE + 4 * TILE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    const uint32_t k_full0 = smem_u32(bars), k_empty0 = k_full0 + 16, v_full0 = k_full0 + 32, v_empty0 = k_full0 + 48,
                   s_full0 = k_full0 + 64, p_full0 = k_full0 + 80, o_done0 = k_full0 + 96, q_ready0 = k_full0 + 112;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 8 * 32) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&kmap) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&vmap) : "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    // The barriers live as long as the block: every role counts the tiles and units it has been through and takes the
    // stage and the phase of a barrier from its own count, so the roles run on from one unit into the next (the producer
    // fetches the first keys of the next unit while the last products of this one run).
    if (tid == 0) {
        for (int s = 0; s < 2; s++) {
            mbar_init(k_full0 + 8 * s, 1); mbar_init(k_empty0 + 8 * s, 1); mbar_init(v_full0 + 8 * s, 1);
            mbar_init(v_empty0 + 8 * s, 1); mbar_init(s_full0 + 8 * s, 1); mbar_init(p_full0 + 8 * s, T5_BM);
            mbar_init(o_done0 + 8 * s, 1); mbar_init(q_ready0 + 8 * s, T5_BM);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // tensor memory: scores of tile g in columns g*128 .. +127 (its probabilities go back into the first 64 of them as
    // bf16 pairs), output accumulator of tile g in columns 256 + g*HD .. +HD-1
    const uint32_t tm_s0 = tmem_base, tm_o0 = tmem_base + 256;

    // The block is compiled for 168 registers a thread; a softmax thread keeps a row of 128 scores in registers and wants
    // more, the third warpgroup needs few: it hands its share over.
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;\n");
    if (warp == 8) {
        // ---------------------------------------------------------------- producer
        // Every copy of a tile is issued by a lane of its own: lane = (page of the tile, 64-column half).  One thread
        // issuing them one after the other took 3,000 to 4,000 cycles per 32 KB tile and was what the whole block
        // waited for.  The lane's page id is read from the block table one tile ahead.
        const int shift = P.page_shift, page = P.page;
        const int boxes = (T5_BN >> shift) * HALVES;                 // 1 .. 32
        const int p = lane / HALVES, h = lane % HALVES;
        T5Unit U;
        int k = 0, unit = t5_unit_at(0, n_units);
        bool live = unit >= 0 && t5_unit(P, unit, U);
        int kt = 0;                                                  // key tiles loaded so far
        bool ok = true;
        for (; ok && unit >= 0; k++, unit = t5_unit_at(k, n_units), live = unit >= 0 && t5_unit(P, unit, U)) {
            if (!live) continue;
            auto page_of = [&](int t) -> int {
                const int key0 = U.lo_al + t * T5_BN + p * page, block = key0 >> shift;
                const bool live = lane < boxes && key0 < U.hi && key0 + page > U.lo && block < P.max_blocks;
                return live ? __ldg(U.tb + block) : 0;
            };
            // K of tile t+1 goes out before V of tile t: the key stage is free as soon as the score products that read
            // it are done, the value stage only after the output products, one tile later
            auto load = [&](int t, bool keys, int pg) -> bool {
                const int n = kt + t, s = n & 1, round = n >> 1;
                const uint32_t empty = (keys ? k_empty0 : v_empty0) + 8 * s, fb = (keys ? k_full0 : v_full0) + 8 * s;
                bool got = round == 0 || mbar_wait(empty, (round - 1) & 1, P.err);
                if (!__all_sync(0xffffffffu, got)) return false;
                if (lane == 0) mbar_expect_tx(fb, TILE);
                __syncwarp();
                if (lane < boxes) {
                    const int key0 = U.lo_al + t * T5_BN + p * page;
                    if (pg < 0 || pg >= P.num_pages) {
                        if (key0 < U.hi && key0 + page > U.lo) mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
                        pg = 0;                                      // any page: every key of it is masked
                    }
                    const uint32_t dst = (keys ? k_s0 : v_s0) + s * TILE + h * T5_HALF + p * page * 128;
                    tma_load_2d(dst, keys ? &kmap : &vmap, h * 64, (pg * P.KV + U.kvh) * page, fb);
                }
                return true;
            };
            int pg_cur = page_of(0);
            ok = load(0, true, pg_cur);
            for (int t = 0; t < U.T && ok; t++) {
                int pg_next = 0;
                if (t + 1 < U.T) { pg_next = page_of(t + 1); ok = load(t + 1, true, pg_next); }
                if (ok) ok = load(t, false, pg_cur);
                pg_cur = pg_next;
            }
            kt += U.T;
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- products
        // One thread issues, for the two query tiles in turn: O_g += P_g(t) V(t), then S_g = Q_g K(t+1)^T.  While the
        // softmax warps of one tile work, the tensor cores run the products of the other.  The score product of a tile
        // overwrites the buffer its probabilities lay in; it is issued after the output product that read them, and the
        // products run in the order they were issued.
        if (lane == 0) {
            // D float, A and B bf16, M = 128; scores N = 128 keys, outputs N = HD with B MN-major (bit 16)
            constexpr uint32_t idesc_qk = umma_idesc(T5_BM, T5_BN);
            constexpr uint32_t idesc_pv = umma_idesc(T5_BM, HD) | (1u << 16);
            T5Unit U;
            int k = 0, unit = t5_unit_at(0, n_units);
            bool live = unit >= 0 && t5_unit(P, unit, U);
            int kt = 0, nu0 = 0, nu1 = 0, nt0 = 0, nt1 = 0;           // key tiles; per query tile: units and tiles so far
            bool ok = true;
            for (; ok && unit >= 0; k++, unit = t5_unit_at(k, n_units), live = unit >= 0 && t5_unit(P, unit, U)) {
                if (!live) continue;
                auto last_reader = [&](int g, int t) -> bool {      // no later query tile reads key tile t
                    return g == T5_QT - 1 || t >= U.T1;
                };
                auto scores = [&](int g, int t) -> bool {           // S_g = Q_g K_t^T
                    const int n = kt + t, s = n & 1;
                    if (!mbar_wait(k_full0 + 8 * s, (n >> 1) & 1, P.err)) return false;
                    tc_fence_after();
                    const uint32_t k_lo = umma_desc_lo(k_s0 + s * TILE, 0), q_lo = umma_desc_lo(q_s0 + g * TILE, 0);
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        constexpr uint32_t half = T5_HALF >> 4;
                        const uint32_t off = (ks >> 2) * half + (ks & 3) * 2;             // in 16-byte units
                        umma_f16(tm_s0 + g * 128, umma_desc_join(q_lo + off), umma_desc_join(k_lo + off), idesc_qk, ks > 0);
                    }
                    if (last_reader(g, t)) umma_commit(k_empty0 + 8 * s);
                    umma_commit(s_full0 + 8 * g);
                    return true;
                };
                auto outputs = [&](int g, int t) -> bool {          // O_g += P_g V_t
                    const int n = kt + t, s = n & 1;
                    if (!mbar_wait(p_full0 + 8 * g, ((g == 0 ? nt0 : nt1) + t) & 1, P.err)) return false;
                    if (!mbar_wait(v_full0 + 8 * s, (n >> 1) & 1, P.err)) return false;
                    tc_fence_after();
                    const uint32_t v_lo = umma_desc_lo(v_s0 + s * TILE, T5_HALF);
#pragma unroll
                    for (int kk = 0; kk < 8; kk++)                  // 16 keys per step: 2,048 bytes further in the tile
                        umma_f16_ts(tm_o0 + g * HD, tm_s0 + g * 128 + kk * 8, umma_desc_join(v_lo + kk * 128), idesc_pv,
                                    (t > 0 || kk > 0) ? 1u : 0u);
                    if (last_reader(g, t)) umma_commit(v_empty0 + 8 * s);
                    if (t == U.tiles(g) - 1) umma_commit(o_done0 + 8 * g);
                    return true;
                };
#pragma unroll
                for (int g = 0; g < T5_QT; g++)
                    if (ok && U.tiles(g) > 0) ok = mbar_wait(q_ready0 + 8 * g, (g == 0 ? nu0 : nu1) & 1, P.err) && scores(g, 0);
                for (int t = 0; t < U.T && ok; t++) {
#pragma unroll
                    for (int g = 0; g < T5_QT; g++) {
                        if (ok && t < U.tiles(g)) ok = outputs(g, t);
                        if (ok && t + 1 < U.tiles(g)) ok = scores(g, t + 1);
                    }
                }
                kt += U.T;
                if (U.T0 > 0) { nu0++; nt0 += U.T0; }
                if (U.T1 > 0) { nu1++; nt1 += U.T1; }
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;\n");
        // ---------------------------------------------------------------- softmax: warpgroup = query tile, thread = row
        const int g = warp >> 2, q = warp & 3, r_loc = q * 32 + lane;
        const int st = tid - g * T5_BM;                             // 0..127 within the warpgroup
        const uint32_t q_s = q_s0 + g * TILE;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const uint32_t s_addr = tm_s0 + g * 128 + lane_addr, o_addr = tm_o0 + g * HD + lane_addr;
        T5Unit U;
        int k = 0, unit = t5_unit_at(0, n_units);
        bool live = unit >= 0 && t5_unit(P, unit, U);
        int nu = 0, nt = 0;                                         // units and tiles this query tile has been through
        bool ok = true;
        // the block's next unit in which this query tile has rows (-1: none left)
        auto advance = [&]() {
            for (;;) {
                k++;
                unit = t5_unit_at(k, n_units);
                if (unit < 0) return;
                if (t5_unit(P, unit, U) && U.tiles(g) > 0) return;
            }
        };
        // the unit's query tile goes into shared memory (asynchronous copies, waited for in publish_q)
        auto fetch_q = [&]() {
            const int row_g = U.row0 + g * T5_BM;
            for (int cid = st; cid < T5_BM * (HD / 8); cid += T5_BM) {
                const int row = cid / (HD / 8), c = cid % (HD / 8), rr = row_g + row;
                const bf16* src = P.q;
                int bytes = 0;
                if (rr < U.R) {
                    src = P.q + (size_t)(U.tok0 + rr / U.G) * P.q_stride + (size_t)(U.kvh * U.G + rr % U.G) * HD + c * 8;
                    bytes = 16;
                }
                const uint32_t dst = q_s + (c >> 3) * T5_HALF + (row >> 3) * 1024 + (row & 7) * 128 + (((c & 7) ^ (row & 7)) << 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
            }
            cp_async_commit();
        };
        auto publish_q = [&]() {
            cp_async_wait<0>();
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbar_arrive(q_ready0 + 8 * g);
        };
        if (unit >= 0 && !(live && U.tiles(g) > 0)) advance();
        if (unit >= 0) { fetch_q(); publish_q(); }
        while (ok && unit >= 0) {
            const int Tq = U.tiles(g), pos_min_g = U.pmin(g), pos_max_g = U.pmax(g);
            const int G = U.G, R = U.R, r = U.row0 + g * T5_BM + r_loc;
            const int tok0 = U.tok0, kvh = U.kvh, lo_al = U.lo_al, pos0 = U.pos0;
            int rpos = -1, rlo = 0;
            if (r < R) {
                rpos = pos0 + r / G;
                rlo = (P.window > 0 && rpos - P.window + 1 > 0) ? rpos - P.window + 1 : 0;
            }
            float m_run = -INFINITY, l_run = 0.0f;
            for (int t = 0; t < Tq && ok; t++) {
                // the scores of this tile are complete -- and so is every product issued before them: the output product
                // of the tile before, which read the probabilities in this buffer and wrote the accumulator
                if (!mbar_wait(s_full0 + 8 * g, (nt + t) & 1, P.err)) { ok = false; break; }
                tc_fence_after();
                const int kb = lo_al + t * T5_BN;
                const bool full_tile = kb + T5_BN - 1 <= pos_min_g && kb >= ((P.window > 0) ? pos_max_g - P.window + 1 : 0);
                // the row's 128 scores come from tensor memory with four loads and ONE wait (a load and its wait are a
                // round trip of several hundred cycles) and stay in registers for both passes
                uint32_t sv[4][32];
#pragma unroll
                for (int c = 0; c < 4; c++) tmem_ld32(s_addr + c * 32, sv[c]);
                tmem_ld_wait();
                // eight running maxima (and eight partial sums below): one chain of 128 dependent operations would cost
                // its latency 128 times over
                float mxs[8];
#pragma unroll
                for (int i = 0; i < 8; i++) mxs[i] = -INFINITY;
                if (full_tile) {
#pragma unroll
                    for (int c = 0; c < 4; c++)
#pragma unroll
                        for (int i = 0; i < 32; i += 2)
                            mxs[(i >> 1) & 7] = fmax3(mxs[(i >> 1) & 7], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
                } else {
                    // masked keys become -inf once, here; 2^(-inf) = 0 does the rest
#pragma unroll
                    for (int c = 0; c < 4; c++)
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            const int key = kb + c * 32 + i;
                            if (!(key <= rpos && key >= rlo)) sv[c][i] = 0xff800000u;
                            mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(sv[c][i]));
                        }
                }
                float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])), fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
                mx *= P.scale_log2;                                   // the scale is positive: max(scale * s) = scale * max(s)
                // The reference point of the exponentials follows the running maximum lazily: it moves only when the
                // maximum has grown by more than 8 (a factor of 256), so probabilities stay below 256 and the output
                // accumulator is rescaled a few times per row instead of at almost every tile.  The result is the same:
                // the sums and the output use one reference point at any time and the final division cancels it.
                const float m_new = (m_run == -INFINITY || mx > m_run + 8.0f) ? fmaxf(m_run, mx) : m_run;
                const float muse = (m_new == -INFINITY) ? 0.0f : m_new;
                const float corr = fast_exp2(m_run - muse);
                // a row whose running maximum moved rescales its lane of the output; the loads and stores are warp-wide
                // instructions, so the whole warp goes when any of its rows has to (the others multiply by one)
                const bool rescale = t > 0 && __any_sync(0xffffffffu, m_new != m_run);
                if (rescale) {
#pragma unroll 1
                    for (int c = 0; c < OC; c++) {
                        uint32_t ov[32];
                        tmem_ld32(o_addr + c * 32, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
                        tmem_st32(o_addr + c * 32, ov);
                    }
                }
                m_run = m_new;
                // probabilities = 2^(scale * s - reference); as bf16 pairs they go back into the first 64 columns of the
                // score buffer, where the output product reads them as its A operand.  T5_POLY pairs in eight take the
                // polynomial, the others the special-function unit.
                uint64_t sums2[4];
#pragma unroll
                for (int i = 0; i < 4; i++) sums2[i] = 0ull;
                const uint64_t scale2 = pack2(P.scale_log2, P.scale_log2), nm2 = pack2(-muse, -muse);
                uint32_t pk[2][32];
#pragma unroll
                for (int c = 0; c < 4; c++) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {                   // 8 keys = four packed columns
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const uint64_t x2 = ffma2(pack2(__uint_as_float(sv[c][j * 8 + 2 * e]), __uint_as_float(sv[c][j * 8 + 2 * e + 1])),
                                                      scale2, nm2);
                            float pa, pb;
                            const int pair = (j * 4 + e) & 7;
                            if ((pair * 3 & 7) < T5_POLY) {         // pairs 0, 3, 6, 1, ... of eight
                                poly_exp2_pair(x2, pa, pb);
                            } else {
                                unpack2(x2, pa, pb);
                                pa = fast_exp2(pa);
                                pb = fast_exp2(pb);
                            }
                            sums2[e] = fadd2(sums2[e], pack2(pa, pb));
                            pk[c >> 1][(c & 1) * 16 + j * 4 + e] = pack_bf16(pa, pb);
                        }
                    }
                    if (c == 1) tmem_st32(s_addr, pk[0]);
                }
                tmem_st32(s_addr + 32, pk[1]);
                tmem_st_wait();
                float sums[8];
#pragma unroll
                for (int i = 0; i < 4; i++) unpack2(sums2[i], sums[2 * i], sums[2 * i + 1]);
                const float sum = ((sums[0] + sums[1]) + (sums[2] + sums[3])) + ((sums[4] + sums[5]) + (sums[6] + sums[7]));
                l_run = l_run * corr + sum;
                tc_fence_before();
                mbar_arrive(p_full0 + 8 * g);
            }
            if (!ok) break;
            // Every score product of this unit is done (the last tile's scores were read above), so the query tile of
            // the next unit can come in now, while the last output product runs; it is handed to the product thread
            // before this unit's output is written, so the first scores of the next unit are computed meanwhile.
            advance();
            if (unit >= 0) fetch_q();
            if (!mbar_wait(o_done0 + 8 * g, nu & 1, P.err)) { ok = false; break; }
            tc_fence_after();
            if (unit >= 0) publish_q();
            {
                const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                const bool live_row = r < R;                        // rows past the end take part in the loads only
                bf16* dst = P.out + (live_row ? ((size_t)(tok0 + r / G) * P.H + (kvh * G + r % G)) * HD : 0);
#pragma unroll 1
                for (int c = 0; c < OC; c++) {
                    uint32_t ov[32];
                    tmem_ld32(o_addr + c * 32, ov);
                    tmem_ld_wait();
                    if (live_row) {
#pragma unroll
                        for (int i = 0; i < 32; i += 16) {          // 16 values = 32 bytes, a whole sector, per store
                            uint32_t w[8];
#pragma unroll
                            for (int e = 0; e < 8; e++)
                                w[e] = pack_bf16(__uint_as_float(ov[i + 2 * e]) * inv, __uint_as_float(ov[i + 2 * e + 1]) * inv);
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"l"(dst + c * 32 + i),
                                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
                        }
                    }
                }
            }
            nu++;
            nt += Tq;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(*tmem_slot), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ host side
// tensor maps of the cache pools: a pool is (pages * kv heads * page) rows of HD bf16; a box is one page of one kv head,
// 64 columns wide, with the 128-byte swizzle
struct PoolMap { const void* ptr; long long rows; int hd, page; CUtensorMap map; };
#define POOL_MAPS 512
static PoolMap pool_maps[POOL_MAPS];
static int pool_map_count = 0;

static int pool_map(const void* pool, long long rows, int HD, int page, CUtensorMap* out) {
    for (int i = 0; i < pool_map_count; i++) {
        const PoolMap& k = pool_maps[i];
        if (k.ptr == pool && k.rows == rows && k.hd == HD && k.page == page) { *out = k.map; return 0; }
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
    if (pool_map_count < POOL_MAPS) pool_maps[pool_map_count++] = PoolMap{pool, rows, HD, page, m};
    *out = m;
    return 0;
}

MB_API int mb_attn_tc5_rows() { return T5_ROWS; }

MB_API int mb_attn_tc5_supports(int HD, int page) {
    return (HD == 64 || HD == 128) && (page == 8 || page == 16 || page == 32 || page == 64 || page == 128);
}

template <int HD>
static int launch_tc5(const AttnParams& P, const CUtensorMap& kmap, const CUtensorMap& vmap, int n_units, cudaStream_t st) {
    constexpr size_t smem = 1024 + (T5_QT + 4) * (size_t)(T5_BN * HD * 2) + 16 * 8 + 16;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc5_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    attn_tc5_kernel<HD><<<n_units < sms ? n_units : sms, T5_THREADS, smem, st>>>(P, kmap, vmap, n_units);
    MB_LAUNCH_CHECK();
    return 0;
}

// items: (sequence, tile of T5_ROWS = 256 packed rows, 0, 1), heaviest first -- this kernel does not split the keys over blocks.
MB_API int mb_attn_tc5_bf16(const void* q, int q_stride, void* out, const void* kpool, const void* vpool,
                            const void* items, int n_items, const int* q_start, const int* q_len, const int* pos0,
                            const int* seq_row, const int* table, int max_blocks, int H, int KV, int HD, int page,
                            int num_pages, int window, float scale, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (!mb_attn_tc5_supports(HD, page) || KV < 1 || H % KV || KV > 65535) return -2;
    AttnParams P;
    P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out;
    P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = (const int4*)items;
    P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.part_base = nullptr; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.part_o = nullptr; P.part_ml = nullptr; P.max_splits = 1; P.counters = nullptr;
    P.H = H; P.KV = KV; P.G = H / KV; P.page = page; P.num_pages = num_pages; P.window = window;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    CUtensorMap kmap, vmap;
    const long long rows = (long long)num_pages * KV * page;
    int rc = pool_map(kpool, rows, HD, page, &kmap);
    if (rc) return rc;
    rc = pool_map(vpool, rows, HD, page, &vmap);
    if (rc) return rc;
    const int n_units = n_items * KV;
    return HD == 64 ? launch_tc5<64>(P, kmap, vmap, n_units, st) : launch_tc5<128>(P, kmap, vmap, n_units, st);
}
