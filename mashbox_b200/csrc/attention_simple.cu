// Paged attention, plain form: one warp per (token, query head), keys in ascending position through the block table.
// It serves the whole float32 path and, on the bf16 path, every head size the tensor-core kernel does not take.
// Scores, softmax and the weighted sum are float.  The order of every sum depends only on the query's position and
// the window, never on how tokens were cut into steps or which pages hold the keys.
#include "common.cuh"

#define SIMPLE_MAX_HD 256
#define WARPS 4

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attn_simple_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, const int* __restrict__ positions,
    const int* __restrict__ tok_seq, const int* __restrict__ table, int max_blocks, const T* __restrict__ kpool,
    const T* __restrict__ vpool, int N, int H, int KV, int HD, int page, int num_pages, int window, float scale,
    int* err) {
    __shared__ float qs[WARPS][SIMPLE_MAX_HD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)N * H) return;
    const int n = (int)(item / H), h = (int)(item % H);
    const int kvh = h / (H / KV);
    const int pos = positions[n];
    const int* tb = table + (size_t)tok_seq[n] * max_blocks;
    const T* qr = q + (size_t)n * q_stride + (size_t)h * HD;
    for (int d = lane; d < HD; d += 32) qs[warp][d] = mb_load(qr + d);
    __syncwarp();
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.0f;
    float acc[SIMPLE_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < SIMPLE_MAX_HD / 32; i++) acc[i] = 0.0f;
    for (int base = lo; base <= pos; base += 32) {
        const int kp = base + lane;
        const bool valid = kp <= pos;
        long long off = -1;
        float s = -INFINITY;
        if (valid) {
            const int pg = tb[kp / page];
            if (pg < 0 || pg >= num_pages) {
                mb_set_error(err, pg < 0 ? MB_ERR_PAGE_MISSING : MB_ERR_PAGE_RANGE);
            } else {
                off = (((long long)pg * KV + kvh) * page + (kp % page)) * HD;
                const T* kr = kpool + off;
                float a = 0.0f;
                for (int d = 0; d < HD; d++) a = fmaf(qs[warp][d], mb_load(kr + d), a);
                s = a * scale;
            }
        }
        const float tmax = mb_warp_max(s);
        const float m_new = fmaxf(m, tmax);
        if (m_new == -INFINITY) continue;                      // only after a table error: nothing to add
        const float p = (off >= 0) ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + mb_warp_sum(p);
#pragma unroll
        for (int i = 0; i < SIMPLE_MAX_HD / 32; i++) acc[i] *= corr;
        const int cnt = min(32, pos - base + 1);
        for (int j = 0; j < cnt; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            if (oj < 0) continue;
            const T* vr = vpool + oj;
#pragma unroll
            for (int i = 0; i < SIMPLE_MAX_HD / 32; i++) {
                const int d = lane + 32 * i;
                if (d < HD) acc[i] = fmaf(pj, mb_load(vr + d), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    T* o = out + (size_t)n * H * HD + (size_t)h * HD;
#pragma unroll
    for (int i = 0; i < SIMPLE_MAX_HD / 32; i++) {
        const int d = lane + 32 * i;
        if (d < HD) mb_store(o + d, acc[i] * inv);
    }
}

template <typename T>
static int attn_simple_launch(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                              const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                              int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                              cudaStream_t st) {
    if (N == 0) return 0;
    if (HD > SIMPLE_MAX_HD || HD < 1 || KV < 1 || H % KV) return -2;
    const long long items = (long long)N * H;
    attn_simple_kernel<T><<<(unsigned)((items + WARPS - 1) / WARPS), WARPS * 32, 0, st>>>(
        (const T*)q, q_stride, (T*)out, positions, tok_seq, table, max_blocks, (const T*)kpool, (const T*)vpool, N, H,
        KV, HD, page, num_pages, window, scale, err);
    MB_LAUNCH_CHECK();
    return 0;
}

MB_API int mb_attn_simple_f32(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                              const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                              int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                              cudaStream_t st) {
    return attn_simple_launch<float>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N, H, KV,
                                     HD, page, num_pages, window, scale, err, st);
}
MB_API int mb_attn_simple_bf16(const void* q, int q_stride, void* out, const int* positions, const int* tok_seq,
                               const int* table, int max_blocks, const void* kpool, const void* vpool, int N, int H,
                               int KV, int HD, int page, int num_pages, int window, float scale, int* err,
                               cudaStream_t st) {
    return attn_simple_launch<__nv_bfloat16>(q, q_stride, out, positions, tok_seq, table, max_blocks, kpool, vpool, N,
                                             H, KV, HD, page, num_pages, window, scale, err, st);
}
