// bf16 matrix product for prompt portions on the 5th-generation tensor cores: out[n, m] = sum_k act[n, k] * W[m, k].
//
// One persistent block per SM, warp-specialised:
//   warp 0   producer: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings a 128-token x 64-k tile of the
//            activations and a 256-row x 64-k tile of W per stage into a ring of 4 stages (48 KB each);
//   warp 1   issues tcgen05.mma (cta_group::1, kind::f16, M = 128 tokens, N = 256 features, K = 16 per instruction,
//            4 per stage) from shared-memory descriptors into an accumulator of 256 float columns in tensor memory,
//            and hands stages back / accumulators on with tcgen05.commit on mbarriers; it also owns the TMEM allocation
//            (all 512 columns: two accumulators, so the epilogue of one tile overlaps the products of the next);
//   warps 2-5  epilogue: tcgen05.ld (32 lanes x 32 columns per warp and instruction) -> bf16 or float -> global memory.
// Tiles are walked with the token tile running fastest, so the blocks that run together share a tile of W in L2 and
// every weight is read from HBM once.
//
// Fused SwiGLU mode: W = [gate rows | up rows]; the 256 rows of a stage are 128 gate rows and the 128 up rows of the
// same features, the accumulator holds gate in columns 0..127 and up in 128..255, and the epilogue writes
// silu(gate) * up -- the gate/up activations never reach memory.
//
// Sizes: K a multiple of 8, M a multiple of 8; anything else, and batches under 128 tokens, go to the library product.
// Every wait on an mbarrier is bounded; on a timeout the roles fall through to the common exit, where the tensor memory
// is given back.
#include <cuda.h>
#include "common.cuh"

typedef __nv_bfloat16 bf16;

#define G_BM 128            // tokens per tile (UMMA M)
#define G_BN 256            // features per tile (UMMA N)
#define G_BK 64             // k per stage (one 128-byte swizzle span)
#define G_STAGES 4
#define G_WAIT_LIMIT (1 << 22)
#define G_A_BYTES (G_BM * G_BK * 2)
#define G_B_BYTES (G_BN * G_BK * 2)
#define G_STAGE_BYTES (G_A_BYTES + G_B_BYTES)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    for (int it = 0; it < G_WAIT_LIMIT; it++) {
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

// ---- tensor memory and tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes with the 128-byte swizzle: start address,
// stride between 8-row groups 1024 bytes, descriptor version 1, layout type 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// instruction descriptor, kind::f16: D float (1 << 4), A and B bf16 (1 << 7, 1 << 10), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// MODE 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out (N, M)
template <int MODE>
__global__ void __launch_bounds__(192, 1) gemm_tc5_kernel(const __grid_constant__ CUtensorMap amap,
                                                           const __grid_constant__ CUtensorMap wmap,
                                                           void* __restrict__ out, int N, int M, int K, int* err) {
    constexpr int FEATS = MODE == 1 ? 128 : 256;          // output features of one tile
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)G_STAGES * G_STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * G_STAGES + 4);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * G_STAGES;
    const uint32_t tfull0 = empty0 + 8 * G_STAGES, tempty0 = tfull0 + 16;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tok_tiles = (N + G_BM - 1) / G_BM, m_tiles = (M + FEATS - 1) / FEATS;
    const int tiles = tok_tiles * m_tiles, kblocks = (K + G_BK - 1) / G_BK;

    if (tid == 0) {
        for (int s = 0; s < G_STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;                                               // stages issued so far
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const int tok0 = (tile % tok_tiles) * G_BM, m0 = (tile / tok_tiles) * FEATS;
                bool ok = true;
                for (int kb = 0; kb < kblocks && ok; kb++, it++) {
                    const int s = it % G_STAGES, round = it / G_STAGES;
                    if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1, err)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * s, a_dst = stage0 + s * G_STAGE_BYTES, b_dst = a_dst + G_A_BYTES;
                    mbar_expect_tx(fb, G_STAGE_BYTES);
                    tma_load_2d(a_dst, &amap, kb * G_BK, tok0, fb);
                    tma_load_2d(b_dst, &wmap, kb * G_BK, m0, fb);
                    tma_load_2d(b_dst + G_B_BYTES / 2, &wmap, kb * G_BK, MODE == 1 ? M + m0 : m0 + 128, fb);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(G_BM, G_BN);
            int it = 0, j = 0;                                        // stages consumed, tiles done by this block
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, j++) {
                const int acc = j & 1, use = j >> 1;
                if (use > 0 && !mbar_wait(tempty0 + 8 * acc, (use - 1) & 1, err)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * G_BN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; kb++, it++) {
                    const int s = it % G_STAGES, round = it / G_STAGES;
                    if (!mbar_wait(full0 + 8 * s, round & 1, err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = stage0 + s * G_STAGE_BYTES;
                    const uint64_t adesc = umma_desc(a_addr), bdesc = umma_desc(a_addr + G_A_BYTES);
#pragma unroll
                    for (int k = 0; k < G_BK / 16; k++)
                        umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);                     // the stage is free when these products are done
                }
                if (!ok) break;
                umma_commit(tfull0 + 8 * acc);                       // the accumulator is complete
            }
        }
    } else {
        const int q = warp & 3;                                       // the 32 TMEM lanes this warp may read
        int j = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, j++) {
            const int acc = j & 1, use = j >> 1;
            if (!mbar_wait(tfull0 + 8 * acc, use & 1, err)) break;
            tc_fence_after();
            const int tok = (tile % tok_tiles) * G_BM + q * 32 + lane, m0 = (tile / tok_tiles) * FEATS;
            const uint32_t taddr = tmem_base + acc * G_BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < FEATS; c += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + c, r);
                if (MODE == 1) {
                    uint32_t u[32];
                    tmem_ld32(taddr + 128 + c, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        // gate and up pass through bf16 as they do when the products are separate kernels
                        const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
                        const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[i])));
                        // fast exponential and division: no slow path for huge or tiny gate values
                        r[i] = __float_as_uint(__fdividef(g, 1.0f + __expf(-g)) * up);
                    }
                } else {
                    tmem_ld_wait();
                }
                if (tok < N) {
                    if (MODE == 2) {
                        float* dst = reinterpret_cast<float*>(out) + (size_t)tok * M + m0 + c;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (m0 + c + i + 4 <= M)
                                *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                                  __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)tok * M + m0 + c;
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            if (m0 + c + i + 8 <= M) {
                                uint4 v;
                                v.x = pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                                v.y = pack2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                                v.z = pack2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                                v.w = pack2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                                *reinterpret_cast<uint4*>(dst + i) = v;
                            }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
        }
    }
    // common exit: every role comes here, also after a wait that ran out; then the tensor memory is given back
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------ decode batches
// The same machinery turned around for at most 16 tokens ("swap AB"): the 128 rows of a tile of W are the M side of the
// product, the tokens (padded to 16 by the TMA's zero fill) the N side, and the accumulator is 16 float columns.  The
// product is bound by reading W once, so the kernel is a deep stream: stages of one 128-row x 64-k box of W (16 KB, one
// TMA copy) plus the 2 KB of activations that go with it, ten stages in flight per SM.  Matrices with few row tiles are
// also cut along K so that every SM has work; the split that finishes last for a row tile adds the partial sums in a
// fixed order and writes the result (a counter per row tile in global memory tells which one is last; it resets itself).
#define S_STAGE_K 64
#define S_W_BYTES (128 * 64 * 2)
#define S_X_BYTES (16 * 64 * 2)

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

// MODE 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out (N, M).  N <= 16.
template <int MODE>
__global__ void __launch_bounds__(192, 1) gemm_tc5_stream_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                  const __grid_constant__ CUtensorMap xmap,
                                                                  void* __restrict__ out, int N, int M, int K, int splits,
                                                                  int kb_per, float* __restrict__ partial,
                                                                  int* __restrict__ tile_done, int* err) {
    constexpr int SETS = MODE == 1 ? 2 : 1;
    constexpr int STAGE = SETS * S_W_BYTES + S_X_BYTES;
    constexpr int STAGES = MODE == 1 ? 5 : 10;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row_tiles = (M + 127) / 128, units = row_tiles * splits, kblocks = (K + S_STAGE_K - 1) / S_STAGE_K;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 64);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int u = blockIdx.x; u < units; u += gridDim.x) {
                const int m0 = (u / splits) * 128, k_lo = (u % splits) * kb_per, k_hi = min(kblocks, k_lo + kb_per);
                bool ok = true;
                for (int kb = k_lo; kb < k_hi; kb++, it++) {
                    const int s = it % STAGES, round = it / STAGES;
                    if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1, err)) { ok = false; break; }
                    const uint32_t fb = full0 + 8 * s, dst = stage0 + s * STAGE;
                    mbar_expect_tx(fb, STAGE);
                    tma_load_2d(dst, &wmap, kb * S_STAGE_K, m0, fb);
                    if (MODE == 1) tma_load_2d(dst + S_W_BYTES, &wmap, kb * S_STAGE_K, M + m0, fb);
                    tma_load_2d(dst + SETS * S_W_BYTES, &xmap, kb * S_STAGE_K, 0, fb);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(128, 16);
            int it = 0, j = 0;
            for (int u = blockIdx.x; u < units; u += gridDim.x, j++) {
                const int acc = j & 1, use = j >> 1;
                const int k_lo = (u % splits) * kb_per, k_hi = min(kblocks, k_lo + kb_per);
                if (use > 0 && !mbar_wait(tempty0 + 8 * acc, (use - 1) & 1, err)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 32;
                bool ok = true;
                for (int kb = k_lo; kb < k_hi; kb++, it++) {
                    const int s = it % STAGES, round = it / STAGES;
                    if (!mbar_wait(full0 + 8 * s, round & 1, err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t w_addr = stage0 + s * STAGE, x_addr = w_addr + SETS * S_W_BYTES;
                    const uint64_t xdesc = umma_desc(x_addr);
#pragma unroll
                    for (int set = 0; set < SETS; set++) {
                        const uint64_t wdesc = umma_desc(w_addr + set * S_W_BYTES);
#pragma unroll
                        for (int k = 0; k < S_STAGE_K / 16; k++)
                            umma_f16(d_tmem + set * 16, wdesc + 2 * k, xdesc + 2 * k, idesc, (kb > k_lo || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);
                }
                if (!ok) break;
                umma_commit(tfull0 + 8 * acc);
            }
        }
    } else {
        const int q = warp & 3, et = q * 32 + lane;                   // et: this thread's row of the tile (TMEM lane)
        int j = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, j++) {
            const int acc = j & 1, use = j >> 1;
            const int row_tile = u / splits, split = u % splits, m = row_tile * 128 + et;
            if (!mbar_wait(tfull0 + 8 * acc, use & 1, err)) break;
            tc_fence_after();
            uint32_t v[SETS][16];
#pragma unroll
            for (int set = 0; set < SETS; set++) tmem_ld16(tmem_base + acc * 32 + set * 16 + ((uint32_t)(q * 32) << 16), v[set]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);            // the accumulator may be written again
            bool finish = true;
            if (splits > 1) {
                // partial[split][set][n][m]; the last split to arrive for this row tile adds them up
                if (m < M) {
#pragma unroll
                    for (int set = 0; set < SETS; set++)
#pragma unroll
                        for (int n = 0; n < 16; n++)
                            if (n < N) partial[(((size_t)split * SETS + set) * 16 + n) * M + m] = __uint_as_float(v[set][n]);
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                if (et == 0) *last_flag = (atomicAdd(tile_done + row_tile, 1) == splits - 1);
                asm volatile("bar.sync 1, 128;\n" ::: "memory");
                finish = *last_flag != 0;
                if (finish) {
                    __threadfence();
                    if (m < M) {
#pragma unroll
                        for (int set = 0; set < SETS; set++)
#pragma unroll
                            for (int n = 0; n < 16; n++) {
                                float t = 0.0f;
                                if (n < N)
                                    for (int sp = 0; sp < splits; sp++)
                                        t += __ldcg(partial + (((size_t)sp * SETS + set) * 16 + n) * M + m);
                                v[set][n] = __float_as_uint(t);
                            }
                    }
                    if (et == 0) tile_done[row_tile] = 0;             // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;\n" ::: "memory");      // last_flag may be written again
            }
            if (finish && m < M) {
#pragma unroll
                for (int n = 0; n < 16; n++) {
                    if (n >= N) continue;
                    const float a = __uint_as_float(v[0][n]);
                    if (MODE == 2) {
                        reinterpret_cast<float*>(out)[(size_t)n * M + m] = a;
                    } else if (MODE == 1) {
                        const float g = __bfloat162float(__float2bfloat16_rn(a));
                        const float up = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[SETS - 1][n])));
                        reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g)) * up);
                    } else {
                        reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(a);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 64);
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

struct MapEntry { const void* ptr; long long rows; int cols, box_rows; CUtensorMap map; };
#define MAP_CACHE 1024
static MapEntry map_cache[MAP_CACHE];
static int map_count = 0;

// a row-major bf16 matrix (rows, K); box = box_rows rows x 64 columns with the 128-byte swizzle; outside reads give 0
static int matrix_map(const void* base, long long rows, int K, int box_rows, CUtensorMap* out) {
    for (int i = 0; i < map_count; i++)
        if (map_cache[i].ptr == base && map_cache[i].rows == rows && map_cache[i].cols == K &&
            map_cache[i].box_rows == box_rows) { *out = map_cache[i].map; return 0; }
    EncodeTiled enc = encode_fn();
    if (!enc) return -6;
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -6;
    if (map_count < MAP_CACHE) {
        map_cache[map_count].ptr = base; map_cache[map_count].rows = rows; map_cache[map_count].cols = K;
        map_cache[map_count].box_rows = box_rows; map_cache[map_count].map = m;
        map_count++;
    }
    *out = m;
    return 0;
}

template <int MODE>
static int tc5_launch(const void* act, const void* W, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    if (K % 8 || M % 8 || K < 8 || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(act) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        return -2;
    CUtensorMap amap, wmap;
    int rc = matrix_map(act, N, K, 128, &amap);
    if (rc) return rc;
    rc = matrix_map(W, (long long)(MODE == 1 ? 2 : 1) * M, K, 128, &wmap);
    if (rc) return rc;
    const size_t smem = 1024 + (size_t)G_STAGES * G_STAGE_BYTES + (2 * G_STAGES + 4) * 8 + 16;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    const int feats = MODE == 1 ? 128 : 256;
    const int tiles = ((N + G_BM - 1) / G_BM) * ((M + feats - 1) / feats);
    gemm_tc5_kernel<MODE><<<tiles < sms ? tiles : sms, 192, smem, st>>>(amap, wmap, out, N, M, K, err);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_gemm_tc5_supports(int N, int M, int K) { return N >= 1 && K >= 8 && K % 8 == 0 && M % 8 == 0; }

MB_API int mb_gemm_tc5_bf16(const void* act, const void* W, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    return tc5_launch<0>(act, W, out, N, M, K, err, st);
}
// W holds 2 * M rows: gate rows then up rows; out (N, M) = silu(gate) * up
MB_API int mb_gemm_tc5_swiglu_bf16(const void* act, const void* W, void* out, int N, int M, int K, int* err,
                                   cudaStream_t st) {
    return tc5_launch<1>(act, W, out, N, M, K, err, st);
}
MB_API int mb_gemm_tc5_f32out(const void* act, const void* W, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    return tc5_launch<2>(act, W, out, N, M, K, err, st);
}

// k splits of the stream kernels for a (M, K) matrix: about two units per SM, at least four k blocks per split
static int stream_splits(int M, int K, int sms) {
    const int row_tiles = (M + 127) / 128, kblocks = (K + S_STAGE_K - 1) / S_STAGE_K;
    int splits = (2 * sms + row_tiles - 1) / row_tiles;
    if (splits > 16) splits = 16;
    if (splits > kblocks / 4) splits = kblocks / 4;
    if (splits < 1) splits = 1;
    const int kb_per = (kblocks + splits - 1) / splits;
    return (kblocks + kb_per - 1) / kb_per;
}

// ---- decode batches (at most 16 tokens): workspace = float scratch for the partial sums of the k splits
// (mb_gemm_tc5_stream_workspace says how many floats), counters = one int per 128 rows of W, zero
// before the first call (the kernel leaves them zero)
template <int MODE>
static int stream_launch(const void* act, const void* W, void* out, int N, int M, int K, float* workspace, int* counters,
                         int* err, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    if (N > 16 || K % 8 || K < 8 || (reinterpret_cast<uintptr_t>(W) & 15) || (reinterpret_cast<uintptr_t>(act) & 15)) return -2;
    constexpr int SETS = MODE == 1 ? 2 : 1;
    constexpr int STAGES = MODE == 1 ? 5 : 10;
    CUtensorMap wmap, xmap;
    int rc = matrix_map(W, (long long)SETS * M, K, 128, &wmap);
    if (rc) return rc;
    rc = matrix_map(act, N, K, 16, &xmap);
    if (rc) return rc;
    const size_t smem = 1024 + (size_t)STAGES * (SETS * S_W_BYTES + S_X_BYTES) + (2 * STAGES + 4) * 8 + 16;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_stream_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        configured = true;
    }
    const int row_tiles = (M + 127) / 128, kblocks = (K + S_STAGE_K - 1) / S_STAGE_K;
    int splits = stream_splits(M, K, sms);
    if (!workspace || !counters) splits = 1;
    const int kb_per = (kblocks + splits - 1) / splits;
    splits = (kblocks + kb_per - 1) / kb_per;
    const int units = row_tiles * splits;
    gemm_tc5_stream_kernel<MODE><<<units < sms ? units : sms, 192, smem, st>>>(wmap, xmap, out, N, M, K, splits, kb_per,
                                                                               workspace, counters, err);
    MB_LAUNCH_CHECK();
    return 0;
}

// floats of workspace the stream kernels may use for an output of M features (SwiGLU: M = the gate's width)
MB_API long long mb_gemm_tc5_stream_workspace(int M, int K, int sets) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int splits = stream_splits(M, K, sms > 0 ? sms : 148);
    return splits > 1 ? (long long)splits * sets * 16 * M : 0;
}

MB_API int mb_gemm_tc5_stream_bf16(const void* act, const void* W, void* out, int N, int M, int K, float* workspace,
                                   int* counters, int* err, cudaStream_t st) {
    return stream_launch<0>(act, W, out, N, M, K, workspace, counters, err, st);
}
MB_API int mb_gemm_tc5_stream_swiglu_bf16(const void* act, const void* W, void* out, int N, int M, int K, float* workspace,
                                          int* counters, int* err, cudaStream_t st) {
    return stream_launch<1>(act, W, out, N, M, K, workspace, counters, err, st);
}
MB_API int mb_gemm_tc5_stream_f32out(const void* act, const void* W, void* out, int N, int M, int K, float* workspace,
                                     int* counters, int* err, cudaStream_t st) {
    return stream_launch<2>(act, W, out, N, M, K, workspace, counters, err, st);
}
