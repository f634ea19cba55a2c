// Causal grouped-query attention over the paged cache, CUDA cores, fp32 arithmetic.
//
// One kernel serves prompts and decoding, fp32 and bf16 storage, every head size up
// to 256 (any multiple of 2), any number of heads and groups, full and windowed
// layers, windows that keep a sequence's first keys in sight, and values whose size
// differs from the keys'.  A warp owns one (query row, head, split): it walks its range of keys with
// an online softmax (running maximum m, sum l, weighted values o), the head's
// dimensions spread over the lanes.  With more than one split the warps write
// (m, l, o) to a scratch buffer and a second kernel merges them; that keeps many
// warps busy when a few rows face long contexts (decoding).
//
// It is the true 32-bit path's attention and the bf16 path's fallback.  Reference:
// decodeAttentionKernel and the split/combine pair (attention_kernels.cu:29-111,
// 131-235), prefillAttentionKernel (:513-645); mask by range as there (j <= position).
//
// Geometry of a step: every row carries its sequence (row_seq, an index into the step's
// block table) and its position (row_pos); it sees the keys of its sequence up to that
// position.  Keys and values of position j are in page block_table[seq][j / page], row
// j % page, of pools laid out [pages][page][nkv][hd] (keys) and [pages][page][nkv][vd] (values).
//
// With a window W and `keep_first` F, row i sees key j if j <= i and (i - j < W or j < F): the keys
// a warp walks are the kept ones below the window's start followed by the window's.
#include <math.h>

#include "attention_merge.cuh"
#include "common.cuh"

FR_EXPORT const char* attention_simt_last_error() { return fr_error_text; }

namespace {

constexpr int MAX_PER_LANE = 8;   // head sizes up to 256

struct AttnArgs {
    const void* q;        // [rows][q_stride] ; head h at h*hd
    void* out;            // [rows][nq*hd]
    const void* k_pool;
    const void* v_pool;
    const int* block_table;
    const int* row_seq;   // [rows] sequence of the row, < 0: padding row (output zeros)
    const int* row_pos;   // [rows] position of the row
    float* part;          // [rows][nq][splits][hd + 2] when splits > 1
    int table_width, page, rows, nq, nkv, hd, q_stride, window, splits;
    float scale;
    int vd, keep_first;   // size of a value head; keys below keep_first stay visible behind a window
    float out_scale;      // the result is multiplied by this
};

template <typename T>
__global__ void __launch_bounds__(128) attention_kernel(AttnArgs p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;          // (row, head)
    if (item >= p.rows * p.nq) return;
    const int row = item / p.nq, h = item - row * p.nq;
    const int split = blockIdx.y;
    const int seq = p.row_seq[row];
    T* o_row = (T*)p.out + (size_t)row * p.nq * p.vd + (size_t)h * p.vd;
    float* part = p.splits > 1 ? p.part + ((size_t)item * p.splits + split) * (p.vd + 2) : nullptr;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    if (seq >= 0) {
        const int pos = p.row_pos[row];
        const int kvh = h / (p.nq / p.nkv);
        const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const int kept = min(p.keep_first, lo);         // kept keys below the window's start
        const int n = kept + pos - lo + 1;
        const int chunk = (n + p.splits - 1) / p.splits;
        const int i0 = split * chunk;
        const int i1 = min(i0 + chunk, n);
        const T* q = (const T*)p.q + (size_t)row * p.q_stride + (size_t)h * p.hd;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            qv[i] = d < p.hd ? fr_load(q + d) * p.scale : 0.f;
        }
        const int* table = p.block_table + (size_t)seq * p.table_width;
        // four keys at a time: their loads are issued together, so that a warp waits for memory once per four keys
        for (int i = i0; i < i1; i += 4) {
            const T* kr[4];
            const T* vr[4];
            float s4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int iu = min(i + u, i1 - 1);           // past the end: the last key again (its weight is set to zero)
                const int j = iu < kept ? iu : lo + (iu - kept);
                const size_t at = ((size_t)table[j / p.page] * p.page + j % p.page) * p.nkv + kvh;
                kr[u] = (const T*)p.k_pool + at * p.hd;
                vr[u] = (const T*)p.v_pool + at * p.vd;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float s = 0.f;
#pragma unroll
                for (int c = 0; c < MAX_PER_LANE; ++c) {
                    const int d = lane + 32 * c;
                    if (d < p.hd) s = fmaf(qv[c], fr_load(kr[u] + d), s);
                }
                s4[u] = s;
            }
            float vv[4][MAX_PER_LANE];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int c = 0; c < MAX_PER_LANE; ++c) {
                    const int d = lane + 32 * c;
                    vv[u][c] = d < p.vd ? fr_load(vr[u] + d) : 0.f;
                }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) s4[u] += __shfl_xor_sync(0xffffffffu, s4[u], o);
            float m_new = m;
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + u < i1) m_new = fmaxf(m_new, s4[u]);
            const float alpha = expf(m - m_new);      // exp(-inf) = 0 on the first keys
            float e4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) e4[u] = i + u < i1 ? expf(s4[u] - m_new) : 0.f;
            l = l * alpha + ((e4[0] + e4[1]) + (e4[2] + e4[3]));
#pragma unroll
            for (int c = 0; c < MAX_PER_LANE; ++c) {
                const int d = lane + 32 * c;
                if (d < p.vd)
                    acc[c] = acc[c] * alpha + ((e4[0] * vv[0][c] + e4[1] * vv[1][c]) + (e4[2] * vv[2][c] + e4[3] * vv[3][c]));
            }
            m = m_new;
        }
    }
    if (part == nullptr) {
        const float inv = l > 0.f ? p.out_scale / l : 0.f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < p.vd) fr_store(o_row + d, acc[i] * inv);
        }
    } else {
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < p.vd) part[d] = acc[i];
        }
        if (lane == 0) {
            part[p.vd] = m;
            part[p.vd + 1] = l;
        }
    }
}

}  // namespace

// Scratch floats needed for `splits` > 1 (vd: the size of a value head).
FR_EXPORT long long attention_simt_scratch_floats(int rows, int nq, int vd, int splits) {
    return splits > 1 ? (long long)rows * nq * splits * (vd + 2) : 0;
}

// vd: size of a value head (the result is [rows][nq * vd]); keep_first: keys below it stay visible behind a window;
// out_scale multiplies the result.
FR_EXPORT int attention_simt_masked(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                                    const int* block_table, int table_width, int page, const int* row_seq,
                                    const int* row_pos, int rows, int nq, int nkv, int hd, int vd, int window, int keep_first,
                                    float scale, float out_scale, int splits, float* scratch, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (hd <= 0 || hd > 32 * MAX_PER_LANE) FR_REFUSE("attention: head size %d is outside 1..%d", hd, 32 * MAX_PER_LANE);
    if (vd <= 0 || vd > 32 * MAX_PER_LANE) FR_REFUSE("attention: value size %d is outside 1..%d", vd, 32 * MAX_PER_LANE);
    if (nkv <= 0 || nq % nkv != 0) FR_REFUSE("attention: %d heads cannot share %d key/value heads", nq, nkv);
    if (splits < 1 || splits > 65535) FR_REFUSE("attention: %d splits", splits);
    if (splits > 1 && scratch == nullptr) FR_REFUSE("attention: splits need a scratch buffer");
    if (keep_first < 0) FR_REFUSE("attention: keep_first = %d", keep_first);
    AttnArgs p{q, out, k_pool, v_pool, block_table, row_seq, row_pos, scratch, table_width, page, rows, nq, nkv, hd,
               q_stride, window, splits, scale, vd, window > 0 ? keep_first : 0, out_scale};
    const int items = rows * nq;
    MergeArgs mp{scratch, out, rows, nq, vd, splits, out_scale};
    dim3 grid((items + 3) / 4, splits);
    if (dtype == FR_F32) {
        attention_kernel<float><<<grid, 128, 0, stream>>>(p);
        FR_CHECK_LAUNCH("attention");
        if (splits > 1) attention_merge_kernel<float><<<(items + 3) / 4, 128, 0, stream>>>(mp);
    } else if (dtype == FR_BF16) {
        attention_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(p);
        FR_CHECK_LAUNCH("attention");
        if (splits > 1) attention_merge_kernel<__nv_bfloat16><<<(items + 3) / 4, 128, 0, stream>>>(mp);
    } else {
        FR_REFUSE("attention: unknown dtype %d", dtype);
    }
    FR_CHECK_LAUNCH("attention merge");
    return FR_OK;
}

FR_EXPORT int attention_simt(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                             const int* block_table, int table_width, int page, const int* row_seq,
                             const int* row_pos, int rows, int nq, int nkv, int hd, int window, float scale,
                             int splits, float* scratch, int dtype, cudaStream_t stream) {
    return attention_simt_masked(q, q_stride, out, k_pool, v_pool, block_table, table_width, page, row_seq, row_pos, rows, nq,
                                 nkv, hd, hd, window, 0, scale, 1.0f, splits, scratch, dtype, stream);
}
