// Weight-streaming matrix product for decode steps: out[n, m] = sum_k act[n, k] * W[m, k] for at most 16 tokens (n).
//
// With so few tokens the product is bound by reading W once from HBM, so the kernel is a deep TMA stream with a little
// tensor-core work hanging off it.  A block owns 16 rows of W over all of K.  One producer warp issues
// cp.async.bulk.tensor.2d copies of 16 x 64 boxes (128-byte swizzle) into a ring of stages of 256 columns, about
// 96 KB per block and two blocks per SM, so close to 200 KB per SM are in flight whatever the registers hold.  Four
// consumer warps each take one box of a stage: ldmatrix brings the rows of W in as the A operand of
// mma.sync.m16n8k16 -- W is the 16-row side, the tokens the 8-wide side ("swap AB") -- the activations come from global
// memory through L1 as the B operand.  Accumulation is float32; the four warps' partial sums are added in a fixed order
// through shared memory.  Columns past K and rows past the matrix are filled with zeros by the TMA itself.
//
// Modes: plain (bf16 out), float32 out (the output head), and SwiGLU: W = [gate rows | up rows], the block streams the
// same 16 rows of both and writes silu(gate) * up, so the gate/up activations never travel through memory.
// K must be a multiple of 8 (16-byte rows); larger batches go to the library product.  Waits are bounded.
#include <cuda.h>
#include "common.cuh"

typedef __nv_bfloat16 bf16;

#define SK_MAX_TOKENS 16
#define SK_STAGE_K 256
#define SK_WAIT_LIMIT (1 << 20)

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
    for (int it = 0; it < SK_WAIT_LIMIT; it++) {
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
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT: 8-token tiles (1 or 2).  MODE 0: bf16 out (N, M); 1: SwiGLU, W has 2 * M rows, bf16 out (N, M); 2: float out.
template <int NT, int MODE, int STAGES>
__global__ void __launch_bounds__(160) gemm_skinny_kernel(const __grid_constant__ CUtensorMap wmap,
                                                           const bf16* __restrict__ act, void* __restrict__ out, int N,
                                                           int M, int K, int* err) {
    constexpr int SETS = MODE == 1 ? 2 : 1;
    constexpr int BOX = 16 * 64 * 2;                       // bytes of one 16-row x 64-column box
    constexpr int STAGE = SETS * 4 * BOX;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)STAGES * STAGE);
    float* red = reinterpret_cast<float*>(bars + 2 * STAGES);          // [4 warps][SETS][NT][16][8]
    const uint32_t stage0 = smem_u32(smem), full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int steps = (K + SK_STAGE_K - 1) / SK_STAGE_K;
    const int tiles = (M + 15) / 16;
    const int my_tiles = ((int)blockIdx.x < tiles) ? (tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total = my_tiles * steps;                    // stages this block streams, over all its row tiles

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

    if (warp == 4) {
        if (lane != 0) return;
        for (int i = 0; i < total; i++) {
            const int s = i % STAGES, round = i / STAGES;
            if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1, err)) return;
            const int m0 = ((int)blockIdx.x + (i / steps) * (int)gridDim.x) * 16, step = i % steps;
            const uint32_t fb = full0 + 8 * s;
            mbar_expect_tx(fb, STAGE);
#pragma unroll
            for (int set = 0; set < SETS; set++)
#pragma unroll
                for (int b = 0; b < 4; b++)
                    tma_load_2d(stage0 + s * STAGE + (set * 4 + b) * BOX, &wmap, step * SK_STAGE_K + b * 64, set * M + m0, fb);
        }
        return;
    }

    const bf16* ap[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) ap[j] = act + (size_t)min(j * 8 + g, N - 1) * K + 2 * tig;
    // ldmatrix address of this lane inside a box: row = lane % 8 + 8 * ((lane / 8) % 2), 16-byte chunk = 2 * ks + lane / 16
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8, lchunk = lane >> 4;
    const uint32_t lbase = lrow * 128;

    // the activations of a stage are fetched one stage ahead, so that their latency hides behind the stage before
    uint32_t bq[4][NT][2];
    auto fetch = [&](int step) {
        const int k0 = step * SK_STAGE_K + warp * 64;
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const int k = k0 + ks * 16 + 2 * tig;                 // columns past K hold zeros in W: any finite value does
                bq[ks][j][0] = (k < K) ? __ldg(reinterpret_cast<const uint32_t*>(ap[j] + k0 + ks * 16)) : 0u;
                bq[ks][j][1] = (k + 8 < K) ? __ldg(reinterpret_cast<const uint32_t*>(ap[j] + k0 + ks * 16 + 8)) : 0u;
            }
    };
    float acc[SETS][NT][4];
    if (total > 0) fetch(0);
    for (int i = 0; i < total; i++) {
        const int s = i % STAGES, round = i / STAGES, step = i % steps;
        if (step == 0) {
#pragma unroll
            for (int st = 0; st < SETS; st++)
#pragma unroll
                for (int j = 0; j < NT; j++) acc[st][j][0] = acc[st][j][1] = acc[st][j][2] = acc[st][j][3] = 0.0f;
        }
        uint32_t bc[4][NT][2];
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
#pragma unroll
            for (int j = 0; j < NT; j++) { bc[ks][j][0] = bq[ks][j][0]; bc[ks][j][1] = bq[ks][j][1]; }
        if (i + 1 < total) fetch((i + 1) % steps);
        if (!mbar_wait(full0 + 8 * s, round & 1, err)) return;
        if (step * SK_STAGE_K + warp * 64 < K) {
#pragma unroll
            for (int set = 0; set < SETS; set++) {
                const uint32_t box = stage0 + s * STAGE + (set * 4 + warp) * BOX + lbase;
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    uint32_t a[4];
                    ldmatrix_x4(a, box + ((((ks * 2 + lchunk) ^ (lrow & 7))) << 4));
#pragma unroll
                    for (int j = 0; j < NT; j++) mma16816(acc[set][j], a, bc[ks][j][0], bc[ks][j][1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);
        if (step != steps - 1) continue;

        // ---- the row tile is complete: add the four warps' sums in a fixed order and write
        const int m0 = ((int)blockIdx.x + (i / steps) * (int)gridDim.x) * 16;
        asm volatile("bar.sync 1, 128;\n" ::: "memory");               // the tile before has been written out of `red`
#pragma unroll
        for (int st = 0; st < SETS; st++)
#pragma unroll
            for (int j = 0; j < NT; j++) {
                float* r = red + (((size_t)(warp * SETS + st) * NT + j) * 16) * 8;
                r[g * 8 + 2 * tig] = acc[st][j][0];
                r[g * 8 + 2 * tig + 1] = acc[st][j][1];
                r[(g + 8) * 8 + 2 * tig] = acc[st][j][2];
                r[(g + 8) * 8 + 2 * tig + 1] = acc[st][j][3];
            }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        // tokens past N were computed from the last token's activations and are dropped here
        for (int idx = tid; idx < NT * 16 * 8; idx += 128) {
            const int j = idx / 128, row = (idx / 8) % 16, col = idx % 8;
            const int n = j * 8 + col, m = m0 + row;
            if (n >= N || m >= M) continue;
            float v[SETS];
#pragma unroll
            for (int st = 0; st < SETS; st++) {
                float t = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; w++) t += red[(((size_t)(w * SETS + st) * NT + j) * 16 + row) * 8 + col];
                v[st] = t;
            }
            if (MODE == 2) {
                reinterpret_cast<float*>(out)[(size_t)n * M + m] = v[0];
            } else if (MODE == 1) {
                // the gate and up sums pass through bf16 as they do when the two products are separate kernels
                const float gt = __bfloat162float(__float2bfloat16_rn(v[0])), up = __bfloat162float(__float2bfloat16_rn(v[SETS - 1]));
                reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn((gt / (1.0f + expf(-gt))) * up);
            } else {
                reinterpret_cast<bf16*>(out)[(size_t)n * M + m] = __float2bfloat16_rn(v[0]);
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

struct MapEntry { const void* ptr; long long rows; int cols; CUtensorMap map; };
#define MAP_CACHE 1024
static MapEntry map_cache[MAP_CACHE];
static int map_count = 0;

// W (rows, K) row-major bf16; box = 16 rows x 64 columns with the 128-byte swizzle; reads outside give zeros
static int weight_map(const void* W, long long rows, int K, CUtensorMap* out) {
    for (int i = 0; i < map_count; i++)
        if (map_cache[i].ptr == W && map_cache[i].rows == rows && map_cache[i].cols == K) { *out = map_cache[i].map; return 0; }
    EncodeTiled enc = encode_fn();
    if (!enc) return -6;
    CUtensorMap m;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {64u, 16u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(W), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -6;
    if (map_count < MAP_CACHE) {
        map_cache[map_count].ptr = W; map_cache[map_count].rows = rows; map_cache[map_count].cols = K;
        map_cache[map_count].map = m;
        map_count++;
    }
    *out = m;
    return 0;
}

template <int NT, int MODE>
static int launch_one(const CUtensorMap& map, const void* act, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    constexpr int SETS = MODE == 1 ? 2 : 1;
    constexpr int STAGES = MODE == 1 ? 6 : 12;
    const size_t smem = 1024 + (size_t)STAGES * SETS * 4 * 2048 + 2 * STAGES * 8 + (size_t)4 * SETS * NT * 16 * 8 * 4;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NT, MODE, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    static int slots = 0;                                  // blocks the device holds at once: two per SM
    if (!slots) {
        int dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        slots = 2 * (sms > 0 ? sms : 148);
    }
    const int tiles = (M + 15) / 16;
    gemm_skinny_kernel<NT, MODE, STAGES><<<(unsigned)(tiles < slots ? tiles : slots), 160, smem, st>>>(
        map, (const bf16*)act, out, N, M, K, err);
    MB_LAUNCH_CHECK();
    return 0;
}

template <int MODE>
static int skinny_launch(const void* act, const void* W, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    if (N == 0 || M == 0) return 0;
    if (N > SK_MAX_TOKENS || K % 8 || K < 8 || (reinterpret_cast<uintptr_t>(W) & 15)) return -2;
    CUtensorMap map;
    const int rc = weight_map(W, (long long)(MODE == 1 ? 2 : 1) * M, K, &map);
    if (rc) return rc;
    return N <= 8 ? launch_one<1, MODE>(map, act, out, N, M, K, err, st) : launch_one<2, MODE>(map, act, out, N, M, K, err, st);
}

MB_API int mb_gemm_skinny_supports(int N, int K) { return N >= 1 && N <= SK_MAX_TOKENS && K >= 8 && K % 8 == 0; }

MB_API int mb_gemm_skinny_bf16(const void* act, const void* W, void* out, int N, int M, int K, int* err, cudaStream_t st) {
    return skinny_launch<0>(act, W, out, N, M, K, err, st);
}
// W holds 2 * M rows: gate rows then up rows; out (N, M) = silu(gate) * up
MB_API int mb_gemm_skinny_swiglu_bf16(const void* act, const void* W, void* out, int N, int M, int K, int* err,
                                      cudaStream_t st) {
    return skinny_launch<1>(act, W, out, N, M, K, err, st);
}
MB_API int mb_gemm_skinny_f32out(const void* act, const void* W, void* out, int N, int M, int K, int* err,
                                 cudaStream_t st) {
    return skinny_launch<2>(act, W, out, N, M, K, err, st);
}
