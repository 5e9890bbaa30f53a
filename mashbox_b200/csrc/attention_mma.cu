// Paged flash attention on tensor cores for the bf16 path: prompt portions and decode tokens in one launch each.
//
// The query rows of one sequence and one KV head are packed as (token, head-in-group): all G = H / KV query heads that
// read the same KV head share each K/V tile that is loaded.  A work item is (sequence, tile of rows, split of the keys);
// the grid is (items, KV heads).  K and V tiles of 64 keys are gathered page by page through the block table with
// cp.async into XOR-swizzled shared memory (several stages in flight), scores and the weighted sum run on
// mma.sync.m16n8k16 with float accumulators, the softmax is online in float with exp2.
//   * PREFILL form: 64 rows per block, each of the 4 warps owns 16 rows and all 64 keys of a tile.
//   * DECODE form: at most 16 rows per block (one or a few tokens of one sequence), the 4 warps split the 64 keys of a
//     tile and are merged through shared memory at the end.
// With more than one split an item writes its unnormalised partial (o, m, l) to scratch memory and a second kernel
// merges the splits; with one split it writes the output directly.
#include "attention_common.cuh"

template <int HD, int BN>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const AttnParams& P, const int* tb, int kvh, int kb,
                                             int lo, int hi, int tid) {
    constexpr int CH = HD / 8;
    const int shift = P.page_shift, mask = P.page - 1;
    int last_block = -1, pg = -1;
#pragma unroll
    for (int cid = tid; cid < BN * CH; cid += 128) {
        const int row = cid / CH, c = cid % CH;
        const int kp = kb + row;
        const bf16 *ksrc = P.kpool, *vsrc = P.vpool;
        int bytes = 0;
        if (kp >= lo && kp < hi) {                       // below lo a window may have given the pages back
            int block, slot;
            if (shift >= 0) { block = kp >> shift; slot = kp & mask; }
            else { block = kp / P.page; slot = kp - block * P.page; }
            if (block != last_block) { pg = tb[block]; last_block = block; }
            if (pg >= 0 && pg < P.num_pages) {
                const size_t off = (((size_t)pg * P.KV + kvh) * P.page + slot) * HD + c * 8;
                ksrc += off; vsrc += off; bytes = 16;
            } else {
                mb_set_error(P.err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            }
        }
        const int so = swz<HD>(row, c);
        cp_async16(ks + so, ksrc, bytes);
        cp_async16(vs + so, vsrc, bytes);
    }
}

template <int HD, bool DECODE, int STAGES>
__global__ void __launch_bounds__(128) attn_mma_kernel(const AttnParams P) {
    constexpr int BM = DECODE ? 16 : 64, BN = 64, CH = HD / 8;
    constexpr int NT = DECODE ? 2 : 8;      // 8-key tiles per warp per key tile
    constexpr int KS = HD / 16;             // k steps of q k^T
    constexpr int DT = HD / 8;              // 8-wide tiles of the output
    constexpr int ROW = tile_row<HD>();     // elements of a tile's row in shared memory
    constexpr bool QREG = HD <= 128;        // the query fragments stay in registers (above: read again for every key tile)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* kvs = qs + BM * ROW;

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
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (t_begin + s < t_end)
            load_kv_tile<HD, BN>(kvs + (size_t)s * 2 * BN * ROW, kvs + (size_t)s * 2 * BN * ROW + BN * ROW, P, tb, kvh,
                                 lo_al + (t_begin + s) * BN, lo, hi, tid);
        cp_async_commit();
    }

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

    cp_async_wait<STAGES - 1>();
    __syncthreads();
    uint32_t qf[QREG ? KS : 1][4];
    if (QREG) {
#pragma unroll
        for (int ks = 0; ks < KS; ks++)
            ldmatrix_x4(qf[QREG ? ks : 0], qs + swz<HD>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
    }

    for (int t = t_begin; t < t_end; t++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int tn = t + STAGES - 1;
            if (tn < t_end) {
                bf16* st = kvs + (size_t)((tn - t_begin) % STAGES) * 2 * BN * ROW;
                load_kv_tile<HD, BN>(st, st + BN * ROW, P, tb, kvh, lo_al + tn * BN, lo, hi, tid);
            }
            cp_async_commit();
        }
        const bf16* kt = kvs + (size_t)((t - t_begin) % STAGES) * 2 * BN * ROW;
        const bf16* vt = kt + BN * ROW;
        const int kb = lo_al + t * BN;

        float s[NT][4];
#pragma unroll
        for (int j = 0; j < NT; j++) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            if (!QREG) ldmatrix_x4(qf[0], qs + swz<HD>(m0 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
            for (int np = 0; np < NT / 2; np++) {
                uint32_t b[4];
                ldmatrix_x4(b, kt + swz<HD>(nbase + np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)));
                mma_bf16(s[2 * np], qf[QREG ? ks : 0], b[0], b[1]);
                mma_bf16(s[2 * np + 1], qf[QREG ? ks : 0], b[2], b[3]);
            }
        }
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = e >> 1;
                const int key = kb + nbase + j * 8 + 2 * tig + (e & 1);
                const bool ok = key <= rpos[i] && key >= rlo[i];
                const float v = ok ? s[j][e] * P.scale_log2 : -INFINITY;
                s[j][e] = v;
                tmax[i] = fmaxf(tmax[i], v);
            }
        }
        float corr[2], muse[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 1));
            tmax[i] = fmaxf(tmax[i], __shfl_xor_sync(0xffffffffu, tmax[i], 2));
            const float m_new = fmaxf(m_run[i], tmax[i]);
            muse[i] = (m_new == -INFINITY) ? 0.0f : m_new;
            corr[i] = exp2f(m_run[i] - muse[i]);
            m_run[i] = m_new;
            l_run[i] *= corr[i];
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float p = exp2f(s[j][e] - muse[e >> 1]);
                l_run[e >> 1] += p;
                s[j][e] = p;
            }
        }
#pragma unroll
        for (int d = 0; d < DT; d++) { o[d][0] *= corr[0]; o[d][1] *= corr[0]; o[d][2] *= corr[1]; o[d][3] *= corr[1]; }
#pragma unroll
        for (int kk = 0; kk < NT / 2; kk++) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; dp++) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vt + swz<HD>(nbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dp * 2 + (lane >> 4)));
                mma_bf16(o[2 * dp], a, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
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
        __syncthreads();                                    // every warp is done with the K/V stages
        float* mo = reinterpret_cast<float*>(kvs);          // [4 warps][16 rows][HD]
        float* sm_m = mo + 4 * 16 * HD;                     // [4][16]
        float* sm_l = sm_m + 4 * 16;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int row = g + i * 8;
            float* dst = mo + ((size_t)(warp * 16 + row)) * HD + 2 * tig;
#pragma unroll
            for (int d = 0; d < DT; d++) { dst[d * 8] = o[d][2 * i]; dst[d * 8 + 1] = o[d][2 * i + 1]; }
            if (tig == 0) { sm_m[warp * 16 + row] = m_run[i]; sm_l[warp * 16 + row] = l_run[i]; }
        }
        __syncthreads();
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
                const float sc = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
                acc += mo[((size_t)(w * 16 + row)) * HD + d] * sc;
                L += sm_l[w * 16 + row] * sc;
            }
            const int tq = r / G, h = kvh * G + r % G;
            if (n_splits == 1) {
                P.out[((size_t)(tok0 + tq) * H + h) * HD + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
            } else {
                const size_t base = ((size_t)(P.part_base[seq] + tq) * H + h) * P.max_splits + split;
                P.part_o[base * HD + d] = acc;
                if (d == 0) { P.part_ml[base * 2] = M; P.part_ml[base * 2 + 1] = L; }
            }
        }
    }
}

// Merges the splits of the tokens that were split: one block per (split token, head).
// part_tok[i] = (token index in the batch, number of splits of its sequence)
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  const int2* __restrict__ part_tok, bf16* __restrict__ out, int H, int HD,
                                  int max_splits) {
    const int pt = blockIdx.x, h = blockIdx.y;
    const int n = part_tok[pt].x, ns = part_tok[pt].y;
    const size_t base = ((size_t)pt * H + h) * max_splits;
    float M = -INFINITY;
    for (int s = 0; s < ns; s++) M = fmaxf(M, part_ml[(base + s) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.0f, L = 0.0f;
        for (int s = 0; s < ns; s++) {
            const float ms = part_ml[(base + s) * 2];
            const float sc = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
            acc += part_o[(base + s) * HD + d] * sc;
            L += part_ml[(base + s) * 2 + 1] * sc;
        }
        out[((size_t)n * H + h) * HD + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
    }
}

template <int HD, bool DECODE, int STAGES>
static int launch_one(const AttnParams& P, int n_items, cudaStream_t st) {
    constexpr int BM = DECODE ? 16 : 64;
    constexpr int ROW = tile_row<HD>();
    size_t smem = (size_t)BM * ROW * 2 + (size_t)STAGES * 2 * 64 * ROW * 2;
    const size_t merge = (size_t)(4 * 16 * HD + 2 * 4 * 16) * 4 + (size_t)BM * ROW * 2;
    if (DECODE && merge > smem) smem = merge;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_mma_kernel<HD, DECODE, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    attn_mma_kernel<HD, DECODE, STAGES><<<dim3(n_items, P.KV), 128, smem, st>>>(P);
    MB_LAUNCH_CHECK();
    return 0;
}

// 1 when the tensor-core kernel takes this head size
// 1 when this library's tensor-core kernel takes the head size.  The source builds two libraries: the common head
// sizes (16, 32, 64, 128), and with -DMB_ATTN_WIDE every other multiple of 16 up to 256 (a model needs one of them,
// and each takes a while to compile).
static bool common_head_size(int HD) { return HD == 16 || HD == 32 || HD == 64 || HD == 128; }
#ifdef MB_ATTN_WIDE
MB_API int mb_attn_mma_supports(int HD) { return HD >= 16 && HD <= 256 && HD % 16 == 0 && !common_head_size(HD); }
#else
MB_API int mb_attn_mma_supports(int HD) { return common_head_size(HD); }
#endif

// decode != 0: items are tiles of at most 16 rows; else tiles of 64 rows.
MB_API int mb_attn_mma_bf16(const void* q, int q_stride, void* out, const void* kpool, const void* vpool,
                            const void* items, int n_items, int decode, const int* q_start, const int* q_len,
                            const int* pos0, const int* part_base, const int* seq_row, const int* table, int max_blocks,
                            float* part_o,
                            float* part_ml, int max_splits, int H, int KV, int HD, int page, int num_pages, int window,
                            float scale, int* err, cudaStream_t st) {
    if (n_items == 0) return 0;
    if (!mb_attn_mma_supports(HD) || KV < 1 || H % KV || KV > 65535) return -2;
    AttnParams P;
    P.q = (const bf16*)q; P.q_stride = q_stride; P.out = (bf16*)out;
    P.kpool = (const bf16*)kpool; P.vpool = (const bf16*)vpool;
    P.items = (const int4*)items;
    P.q_start = q_start; P.q_len = q_len; P.pos0 = pos0; P.part_base = part_base; P.seq_row = seq_row;
    P.table = table; P.max_blocks = max_blocks;
    P.part_o = part_o; P.part_ml = part_ml; P.max_splits = max_splits; P.counters = nullptr;
    P.H = H; P.KV = KV; P.G = H / KV; P.page = page; P.num_pages = num_pages; P.window = window;
    P.page_shift = -1;
    for (int sft = 0; sft < 31; sft++) if ((1 << sft) == page) P.page_shift = sft;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.err = err;
    // head sizes in steps of 16 up to 256; above 128 two stages of K/V tiles (a stage is 64 KB at 256)
#define MB_ATTN_CASE(hd)                                                                   \
    case hd:                                                                               \
        return decode ? launch_one<hd, true, (hd > 128 ? 2 : 3)>(P, n_items, st) : launch_one<hd, false, 2>(P, n_items, st);
    switch (HD) {
#ifdef MB_ATTN_WIDE
        MB_ATTN_CASE(48) MB_ATTN_CASE(80) MB_ATTN_CASE(96) MB_ATTN_CASE(112) MB_ATTN_CASE(144) MB_ATTN_CASE(160)
        MB_ATTN_CASE(176) MB_ATTN_CASE(192) MB_ATTN_CASE(208) MB_ATTN_CASE(224) MB_ATTN_CASE(240) MB_ATTN_CASE(256)
#else
        MB_ATTN_CASE(16) MB_ATTN_CASE(32) MB_ATTN_CASE(64) MB_ATTN_CASE(128)
#endif
    }
    return -2;
}

MB_API int mb_attn_merge_bf16(const float* part_o, const float* part_ml, const void* part_tok, int n_part, void* out,
                              int H, int HD, int max_splits, cudaStream_t st) {
    if (n_part == 0) return 0;
    attn_merge_kernel<<<dim3(n_part, H), 128, 0, st>>>(part_o, part_ml, (const int2*)part_tok, (bf16*)out, H, HD,
                                                       max_splits);
    MB_LAUNCH_CHECK();
    return 0;
}
