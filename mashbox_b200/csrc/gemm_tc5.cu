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
#include "tcgen05.cuh"

#define G_BM 128            // tokens per tile (UMMA M)
#define G_BN 256            // features per tile (UMMA N)
#define G_BK 64             // k per stage (one 128-byte swizzle span)
#define G_STAGES 4
#define G_A_BYTES (G_BM * G_BK * 2)
#define G_B_BYTES (G_BN * G_BK * 2)
#define G_STAGE_BYTES (G_A_BYTES + G_B_BYTES)

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
                                v.x = pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                                v.y = pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                                v.z = pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                                v.w = pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
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

