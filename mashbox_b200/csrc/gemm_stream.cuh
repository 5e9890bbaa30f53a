// What the weight-streaming products share (gemm_stream.cu: one product per launch; gemm_chain.cu: several products in
// one launch with a grid-wide barrier between them): sizes, the structs a product's epilogue takes, the fragment loads
// and the compile-time shape of a kernel.
#pragma once
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

