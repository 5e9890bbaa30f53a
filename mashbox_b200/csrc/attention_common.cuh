// What the two tensor-core attention kernels share: the launch parameters, the PTX wrappers (cp.async, ldmatrix,
// mma.sync m16n8k16 bf16) and the XOR swizzle of a tile whose rows hold HD bf16 values.
#pragma once
#include "common.cuh"

struct AttnParams {
    const bf16* q; int q_stride;            // q[n * q_stride + h * HD + d]
    bf16* out;                              // out[n * H * HD + h * HD + d]
    const bf16* kpool; const bf16* vpool;   // [page][KV][slot][HD]
    const int4* items;                      // (sequence, row tile, split, number of splits)
    const int* q_start; const int* q_len; const int* pos0; const int* part_base;   // per sequence
    const int* seq_row;                     // row of the block table of each sequence
    const int* table; int max_blocks;
    float* part_o; float* part_ml; int max_splits;
    int* counters;                          // one per (first item of a split group, kv head), zero between launches; or null
    int H, KV, G, page, num_pages, window;
    int page_shift;                         // log2(page) when the page size is a power of two, else -1
    float scale_log2;
    int* err;
    // the decode form of the TMA kernel with the rotate-and-store step folded in (every sequence brings ONE token): q
    // points at rows [q heads | k heads | v heads] as the q/k/v product left them; the kernel adds rope_bias ((H + 2 KV)
    // HD floats, or null), rotates q and k by the token's position (rope_freqs: rope_rd / 2 angles per position step,
    // or null; rope_pairing 0 adjacent pairs, 1 halves) and writes k and v into the token's page
    // the decode form of the TMA kernel launched as thread-block clusters of `cluster` blocks, one per split of a
    // sequence (every sequence of the launch has that many splits): the splits' results meet in shared memory
    int cluster = 0;
    int fuse_rope = 0;
    const float* rope_bias = nullptr;
    const float* rope_freqs = nullptr;
    int rope_rd = 0, rope_pairing = 0;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Rows of a tile in shared memory hold HD bf16 values in 16-byte chunks, swizzled against bank conflicts by XOR with
// row bits.  2 and 4 chunks (head sizes 16, 32) have swizzles of their own; every other head size is laid out in
// groups of 8 chunks, the row padded to a whole number of groups (the XOR stays inside a group).
template <int HD> __host__ __device__ constexpr int tile_row() {               // elements of a row in shared memory
    return (HD / 8 == 2 || HD / 8 == 4) ? HD : ((HD / 8 + 7) / 8) * 64;
}
// element offset of 16-byte chunk c of row `row`
template <int HD> __device__ __forceinline__ int swz(int row, int c) {
    constexpr int CH = HD / 8;
    if (CH == 4) return (row * CH + (c ^ ((row >> 1) & 3))) * 8;
    if (CH == 2) return (row * CH + (c ^ ((row >> 2) & 1))) * 8;
    return row * tile_row<HD>() + (c ^ (row & 7)) * 8;
}

