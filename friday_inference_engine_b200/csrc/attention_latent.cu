// Attention whose keys and values are expanded from one small latent per token.
//
// Every token leaves a latent c [rank] (RMS-normed) and one rotated key part r [rot] that all heads share; head h has
// key [W_uk,h c ; r] and value W_uv,h c.  Nothing but c and r is cached.  The expansion is never materialised: with
//     qc_h = W_uk,h^T q_h(unrotated part)                       [rank]
// the score of query i and key j is (qc_h(i) . c(j) + qr_h(i) . r(j)) * scale, and the head's result is
//     W_uv,h (sum_j p_ij c(j)) ,
// so every head attends over the same rows [c ; r] of the cache (read once per key for score and value alike).
// The softmax may have a sink per head: a logit that takes part in the denominator only (no key, no value, not scaled).
//
//   rotate_pairs   interleaved rotary encoding in place: (x[2i], x[2i+1]) of the chosen dimensions of every head turn by
//                  pos * freq[i]; cos and sin are multiplied by `mult` (frequency tables that stretch long wavelengths
//                  carry such a multiplier)
//   prepare        per row of the stacked projection [q | dkv | ...]: c = rmsnorm(dkv[:rank]) * w and the rotated r go to
//                  `ckr` [rows][rank + rot] (what the cache stores), the rotated query parts go to qf [rows][heads][rank + rot]
//                  (fp32) behind the place of qc
//   head_linear    a product per head: out[row][h][n] = sum_k x[row][h][k] W_h[k][n] (weights [heads * k][n], layout 0) or
//                  sum_k x[row][h][k] W_h[n][k] (weights [heads * n][k], layout 1), optionally times sigmoid(gate[row][h])
//   attention      a warp per (row, head, split of the keys): online softmax in fp32 over the paged cache
//                  (c in the key pool [pages][page][rank], r in the value pool [pages][page][rot]); a merge kernel when the
//                  keys were split; the sink joins the denominator at the end
//
// Scores, weights, norms, positions and angles are fp32; the angle is fp32(pos) * freq[i], sine and cosine by sincosf.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* attention_latent_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

// ------------------------------------------------------------------ rotation
struct RotateArgs {
    void* x;                  // [rows][ld]
    const int* row_seq;       // may be null
    const int* row_pos;
    const float* freq;        // [dims / 2]
    float mult;
    int ld, rows, heads, head_stride, first, dims;
};

template <typename T>
__global__ void rotate_pairs_kernel(RotateArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    if (p.row_seq != nullptr && p.row_seq[row] < 0) return;
    const float pos = (float)p.row_pos[row];
    const int half = p.dims / 2;
    T* x = (T*)p.x + (size_t)row * p.ld;
    for (int idx = threadIdx.x; idx < p.heads * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        float s, c;
        sincosf(pos * p.freq[i], &s, &c);
        s *= p.mult;
        c *= p.mult;
        T* at = x + (size_t)h * p.head_stride + p.first + 2 * i;
        float a, b;
        fr_rotate(fr_load(at), fr_load(at + 1), c, s, a, b);
        fr_store(at, a);
        fr_store(at + 1, b);
    }
}

// ------------------------------------------------------------------ prepare
struct PrepareArgs {
    const void* x;            // [rows][ld]: queries [heads][dim + rot] at q_off, [latent rank | key part rot] at kv_off
    void* ckr;                // [rows][rank + rot] in x's dtype
    float* qf;                // [rows][heads][rank + rot] fp32: this kernel fills the last rot of every head
    const void* norm_w;       // [rank]
    int norm_dtype;
    const int* row_seq;
    const int* row_pos;
    const float* freq;        // [rot / 2]
    float mult, eps;
    int ld, q_off, kv_off, heads, dim, rot, rank;
    int rot_dims;             // the first rot_dims of the rot numbers turn, the rest pass unchanged
};

template <typename T>
__global__ void __launch_bounds__(256) prepare_kernel(PrepareArgs p) {
    __shared__ float partial[8];
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    if (p.row_seq != nullptr && p.row_seq[row] < 0) return;
    const T* x = (const T*)p.x + (size_t)row * p.ld;
    T* ckr = (T*)p.ckr + (size_t)row * (p.rank + p.rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x) {
        const float v = fr_load(x + p.kv_off + i);
        ss = fmaf(v, v, ss);
    }
    ss = fr_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += partial[i];
    const float inv = 1.0f / sqrtf(total / (float)p.rank + p.eps);
    const FrVec w{p.norm_w, p.norm_dtype};
    for (int i = threadIdx.x; i < p.rank; i += blockDim.x) fr_store(ckr + i, fr_load(x + p.kv_off + i) * inv * w.at(i));
    const float pos = (float)p.row_pos[row];
    const int half = p.rot_dims / 2;
    // what does not turn passes as it is
    const int still = p.rot - p.rot_dims;
    for (int idx = threadIdx.x; idx < (p.heads + 1) * still; idx += blockDim.x) {
        const int item = idx / still, e = p.rot_dims + (idx - item * still);
        if (item == 0) ckr[p.rank + e] = x[p.kv_off + p.rank + e];
        else p.qf[((size_t)row * p.heads + item - 1) * (p.rank + p.rot) + p.rank + e] = fr_load(x + p.q_off + (size_t)(item - 1) * (p.dim + p.rot) + p.dim + e);
    }
    // the key part (item 0) and every head's rotated query part
    for (int idx = threadIdx.x; idx < (p.heads + 1) * half; idx += blockDim.x) {
        const int item = idx / half, i = idx - item * half;
        float s, c;
        sincosf(pos * p.freq[i], &s, &c);
        s *= p.mult;
        c *= p.mult;
        float a, b;
        if (item == 0) {
            fr_rotate(fr_load(x + p.kv_off + p.rank + 2 * i), fr_load(x + p.kv_off + p.rank + 2 * i + 1), c, s, a, b);
            fr_store(ckr + p.rank + 2 * i, a);
            fr_store(ckr + p.rank + 2 * i + 1, b);
        } else {
            const int h = item - 1;
            const T* q = x + p.q_off + (size_t)h * (p.dim + p.rot) + p.dim + 2 * i;
            fr_rotate(fr_load(q), fr_load(q + 1), c, s, a, b);
            float* o = p.qf + ((size_t)row * p.heads + h) * (p.rank + p.rot) + p.rank + 2 * i;
            o[0] = a;
            o[1] = b;
        }
    }
}

// ------------------------------------------------------------------ a product per head
struct HeadLinearArgs {
    const void* x;            // [rows][ld_x], head h at x_off + h * x_stride, k numbers
    const void* w;            // layout 0: [heads * k][n]; layout 1: [heads * n][k]
    void* out;                // [rows][ld_out], head h at h * out_stride, n numbers
    const void* gate;         // [rows][ld_gate] at gate_off + h: the result is multiplied by its sigmoid (or null)
    const int* row_seq;
    int rows, heads, k, n, ld_x, x_off, x_stride, ld_out, out_stride, ld_gate, gate_off;
};

constexpr int HL_ROWS = 8;        // rows per block

// layout 0: a thread owns output column n of head blockIdx.y for HL_ROWS rows; x staged in shared memory
template <typename TX, typename TW, typename TO, typename TG>
__global__ void __launch_bounds__(128) head_linear_kn_kernel(HeadLinearArgs p) {
    extern __shared__ float sx[];            // [HL_ROWS][k]
    fr_pdl_wait();
    fr_pdl_launch();
    const int h = blockIdx.y, row0 = blockIdx.z * HL_ROWS;
    const int nr = min(HL_ROWS, p.rows - row0);
    for (int idx = threadIdx.x; idx < nr * p.k; idx += blockDim.x) {
        const int r = idx / p.k, i = idx - r * p.k;
        sx[r * p.k + i] = fr_load((const TX*)p.x + (size_t)(row0 + r) * p.ld_x + p.x_off + (size_t)h * p.x_stride + i);
    }
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= p.n) return;
    float acc[HL_ROWS];
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
    const TW* w = (const TW*)p.w + (size_t)h * p.k * p.n + n;
    for (int i = 0; i < p.k; ++i) {
        const float wv = fr_load(w + (size_t)i * p.n);
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r)
            if (r < nr) acc[r] = fmaf(sx[r * p.k + i], wv, acc[r]);
    }
#pragma unroll
    for (int r = 0; r < HL_ROWS; ++r) {
        if (r >= nr) continue;
        const int row = row0 + r;
        if (p.row_seq != nullptr && p.row_seq[row] < 0) continue;
        float v = acc[r];
        if (p.gate != nullptr) {
            const float g = fr_load((const TG*)p.gate + (size_t)row * p.ld_gate + p.gate_off + h);
            v *= 1.0f / (1.0f + expf(-g));
        }
        fr_store((TO*)p.out + (size_t)row * p.ld_out + (size_t)h * p.out_stride + n, v);
    }
}

// layout 1: a warp owns output column n of head blockIdx.y for HL_ROWS rows; the lanes share k
template <typename TX, typename TW, typename TO, typename TG>
__global__ void __launch_bounds__(128) head_linear_nk_kernel(HeadLinearArgs p) {
    extern __shared__ float sx[];            // [HL_ROWS][k]
    fr_pdl_wait();
    fr_pdl_launch();
    const int h = blockIdx.y, row0 = blockIdx.z * HL_ROWS;
    const int nr = min(HL_ROWS, p.rows - row0);
    for (int idx = threadIdx.x; idx < nr * p.k; idx += blockDim.x) {
        const int r = idx / p.k, i = idx - r * p.k;
        sx[r * p.k + i] = fr_load((const TX*)p.x + (size_t)(row0 + r) * p.ld_x + p.x_off + (size_t)h * p.x_stride + i);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int n = blockIdx.x * 16 + warp; n < min(p.n, (int)(blockIdx.x + 1) * 16); n += 4) {
        float acc[HL_ROWS];
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r) acc[r] = 0.f;
        const TW* w = (const TW*)p.w + ((size_t)h * p.n + n) * p.k;
        for (int i = lane; i < p.k; i += 32) {
            const float wv = fr_load(w + i);
#pragma unroll
            for (int r = 0; r < HL_ROWS; ++r)
                if (r < nr) acc[r] = fmaf(sx[r * p.k + i], wv, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < HL_ROWS; ++r) acc[r] = fr_warp_sum(acc[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < HL_ROWS; ++r) {
                if (r >= nr) continue;
                const int row = row0 + r;
                if (p.row_seq != nullptr && p.row_seq[row] < 0) continue;
                float v = acc[r];
                if (p.gate != nullptr) {
                    const float g = fr_load((const TG*)p.gate + (size_t)row * p.ld_gate + p.gate_off + h);
                    v *= 1.0f / (1.0f + expf(-g));
                }
                fr_store((TO*)p.out + (size_t)row * p.ld_out + (size_t)h * p.out_stride + n, v);
            }
        }
    }
}

template <typename TX, typename TW, typename TO>
int launch_head_linear(const HeadLinearArgs& p, int layout, cudaStream_t stream) {
    const size_t smem = (size_t)HL_ROWS * p.k * sizeof(float);
    if (smem > 48 * 1024) FR_REFUSE("head_linear: %d inputs per head (at most %d)", p.k, 48 * 1024 / (HL_ROWS * 4));
    const int row_blocks = (p.rows + HL_ROWS - 1) / HL_ROWS;
    if (layout == 0) {
        const dim3 grid((p.n + 127) / 128, p.heads, row_blocks);
        FR_CUDA(fr_launch(head_linear_kn_kernel<TX, TW, TO, TO>, grid, dim3(128), smem, stream, p));
    } else {
        const dim3 grid((p.n + 15) / 16, p.heads, row_blocks);
        FR_CUDA(fr_launch(head_linear_nk_kernel<TX, TW, TO, TO>, grid, dim3(128), smem, stream, p));
    }
    FR_CHECK_LAUNCH("head_linear");
    return FR_OK;
}

// ------------------------------------------------------------------ attention
constexpr int C_PER_LANE = 16;    // latent sizes up to 512
constexpr int R_PER_LANE = 4;     // rotated key parts up to 128

struct AttnArgs {
    const float* q;           // [rows][heads][rank + rot]
    float* out;               // [rows][heads][rank]
    const void* c_pool;       // [pages][page][rank]
    const void* r_pool;       // [pages][page][rot]
    const int* block_table;
    const int* row_seq;
    const int* row_pos;
    const void* sink;         // [heads] or null
    int sink_dtype;
    float* part;              // [rows * heads][splits][rank + 2] when splits > 1
    int table_width, page, rows, heads, rank, rot, splits;
    float scale;
};

// V numbers per lane and load: lane l owns dimensions V l + e + 32 V i (e < V).  V = 2 needs an even latent size and an
// even rotated part (rows of the pools then start on 4-byte boundaries).
template <typename T, int V> struct Pack;
template <> struct Pack<float, 1> { static __device__ __forceinline__ void load(const float* p, float* o) { o[0] = *p; } };
template <> struct Pack<bf16, 1> { static __device__ __forceinline__ void load(const bf16* p, float* o) { o[0] = __bfloat162float(*p); } };
template <> struct Pack<float, 2> {
    static __device__ __forceinline__ void load(const float* p, float* o) { const float2 v = *(const float2*)p; o[0] = v.x; o[1] = v.y; }
};
template <> struct Pack<bf16, 2> {
    static __device__ __forceinline__ void load(const bf16* p, float* o) {
        const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)p);
        o[0] = v.x; o[1] = v.y;
    }
};

template <typename T, int V>
__global__ void __launch_bounds__(128) latent_attention_kernel(AttnArgs p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;          // (row, head)
    if (item >= p.rows * p.heads) return;
    const int row = item / p.heads, h = item - row * p.heads;
    const int split = blockIdx.y;
    fr_pdl_wait();
    fr_pdl_launch();
    const int seq = p.row_seq[row];
    constexpr int CI = C_PER_LANE / V, RI = R_PER_LANE / V;
    float qc[C_PER_LANE], qr[R_PER_LANE], acc[C_PER_LANE];
#pragma unroll
    for (int i = 0; i < C_PER_LANE; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (seq >= 0) {
        const int n = p.row_pos[row] + 1;
        const int chunk = (n + p.splits - 1) / p.splits;
        const int i0 = split * chunk, i1 = min(i0 + chunk, n);
        const float* q = p.q + (size_t)item * (p.rank + p.rot);
#pragma unroll
        for (int i = 0; i < CI; ++i)
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const int d = V * lane + 32 * V * i + e;
                qc[V * i + e] = d < p.rank ? q[d] * p.scale : 0.f;
            }
#pragma unroll
        for (int i = 0; i < RI; ++i)
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const int d = V * lane + 32 * V * i + e;
                qr[V * i + e] = d < p.rot ? q[p.rank + d] * p.scale : 0.f;
            }
        const int* table = p.block_table + (size_t)seq * p.table_width;
        // two keys at a time: their loads are issued together
        for (int j = i0; j < i1; j += 2) {
            float cv[2][C_PER_LANE], s2[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int ju = min(j + u, i1 - 1);
                const size_t at = (size_t)table[ju / p.page] * p.page + ju % p.page;
                const T* cr = (const T*)p.c_pool + at * p.rank;
                const T* rr = (const T*)p.r_pool + at * p.rot;
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < CI; ++i) {
                    const int d = V * lane + 32 * V * i;
#pragma unroll
                    for (int e = 0; e < V; ++e) cv[u][V * i + e] = 0.f;
                    if (d < p.rank) Pack<T, V>::load(cr + d, &cv[u][V * i]);
#pragma unroll
                    for (int e = 0; e < V; ++e) s = fmaf(qc[V * i + e], cv[u][V * i + e], s);
                }
#pragma unroll
                for (int i = 0; i < RI; ++i) {
                    const int d = V * lane + 32 * V * i;
                    float rv[V];
#pragma unroll
                    for (int e = 0; e < V; ++e) rv[e] = 0.f;
                    if (d < p.rot) Pack<T, V>::load(rr + d, rv);
#pragma unroll
                    for (int e = 0; e < V; ++e) s = fmaf(qr[V * i + e], rv[e], s);
                }
                s2[u] = s;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                s2[0] += __shfl_xor_sync(0xffffffffu, s2[0], o);
                s2[1] += __shfl_xor_sync(0xffffffffu, s2[1], o);
            }
            const bool two = j + 1 < i1;
            const float m_new = fmaxf(m, two ? fmaxf(s2[0], s2[1]) : s2[0]);
            const float alpha = expf(m - m_new);
            const float e0 = expf(s2[0] - m_new), e1 = two ? expf(s2[1] - m_new) : 0.f;
            l = l * alpha + (e0 + e1);
#pragma unroll
            for (int i = 0; i < C_PER_LANE; ++i) acc[i] = acc[i] * alpha + (e0 * cv[0][i] + e1 * cv[1][i]);
            m = m_new;
        }
    }
    if (p.splits > 1) {
        float* part = p.part + ((size_t)item * p.splits + split) * (p.rank + 2);
#pragma unroll
        for (int i = 0; i < CI; ++i)
#pragma unroll
            for (int e = 0; e < V; ++e) {
                const int d = V * lane + 32 * V * i + e;
                if (d < p.rank) part[d] = acc[V * i + e];
            }
        if (lane == 0) {
            part[p.rank] = m;
            part[p.rank + 1] = l;
        }
        return;
    }
    float* o = p.out + (size_t)item * p.rank;
    float denom = l;
    float f = 1.f;
    if (p.sink != nullptr && seq >= 0) {
        const float sk = FrVec{p.sink, p.sink_dtype}.at(h);
        const float top = fmaxf(m, sk);
        f = expf(m - top);
        denom = l * f + expf(sk - top);
    }
    const float inv = denom > 0.f ? f / denom : 0.f;
#pragma unroll
    for (int i = 0; i < CI; ++i)
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const int d = V * lane + 32 * V * i + e;
            if (d < p.rank) o[d] = acc[V * i + e] * inv;
        }
}

__global__ void __launch_bounds__(128) latent_merge_kernel(AttnArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= p.rows * p.heads) return;
    const int h = item % p.heads;
    const float* part = p.part + (size_t)item * p.splits * (p.rank + 2);
    // every lane takes the maximum and the sum of some splits: their loads are in flight together
    float top = -INFINITY;
    for (int s = lane; s < p.splits; s += 32) top = fmaxf(top, part[(size_t)s * (p.rank + 2) + p.rank]);
    top = fr_warp_max(top);
    const bool live = p.row_seq[item / p.heads] >= 0;
    float sk = -INFINITY;
    if (p.sink != nullptr && live) {
        sk = FrVec{p.sink, p.sink_dtype}.at(h);
        top = fmaxf(top, sk);
    }
    float l = 0.f;
    for (int s = lane; s < p.splits; s += 32) {
        const float ls = part[(size_t)s * (p.rank + 2) + p.rank + 1];
        if (ls > 0.f) l += ls * expf(part[(size_t)s * (p.rank + 2) + p.rank] - top);
    }
    l = fr_warp_sum(l);
    float acc[C_PER_LANE];
#pragma unroll
    for (int i = 0; i < C_PER_LANE; ++i) acc[i] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
        const float* ps = part + (size_t)s * (p.rank + 2);
        const float ls = ps[p.rank + 1];
        const float f = ls > 0.f ? expf(ps[p.rank] - top) : 0.f;
#pragma unroll
        for (int i = 0; i < C_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < p.rank) acc[i] += ps[d] * f;
        }
    }
    if (p.sink != nullptr && live) l += expf(sk - top);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    float* o = p.out + (size_t)item * p.rank;
#pragma unroll
    for (int i = 0; i < C_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < p.rank) o[d] = acc[i] * inv;
    }
}

// ------------------------------------------------------------------ prompts: the pieces between tensor-core products
// Rows [0, n) of one sequence's cached latents and key parts, gathered from the pages into contiguous rows; rows
// [n, n_pad) are zero.  The latents are written twice, [2 n_pad][rank] with row n_pad + j equal to row j: the values
// expanded from them then stand side by side twice, once for each half of the split weights.
template <typename T>
__global__ void gather_kernel(const T* __restrict__ c_pool, const T* __restrict__ r_pool, const int* __restrict__ table, int page,
                              int n, int n_pad, int rank, int rot, T* __restrict__ c_all, T* __restrict__ r_all) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int j = blockIdx.x;
    T* c = c_all + (size_t)j * rank;
    T* c2 = c_all + (size_t)(n_pad + j) * rank;
    T* r = r_all + (size_t)j * rot;
    if (j >= n) {
        for (int i = threadIdx.x; i < rank; i += blockDim.x) { fr_store(c + i, 0.f); fr_store(c2 + i, 0.f); }
        for (int i = threadIdx.x; i < rot; i += blockDim.x) fr_store(r + i, 0.f);
        return;
    }
    const size_t at = (size_t)table[j / page] * page + j % page;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) { const T v = c_pool[at * rank + i]; c[i] = v; c2[i] = v; }
    for (int i = threadIdx.x; i < rot; i += blockDim.x) r[i] = r_pool[at * rot + i];
}

// Every head's key [unrotated part from kn [rows][heads * dim] | the shared rotated part r [rows][rot]] side by side:
// out [rows][heads][dim + rot]
template <typename T>
__global__ void key_concat_kernel(const T* __restrict__ kn, const T* __restrict__ r, int heads, int dim, int rot, T* __restrict__ out) {
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t j = blockIdx.x;
    const int hd = dim + rot;
    for (int idx = threadIdx.x; idx < heads * hd; idx += blockDim.x) {
        const int h = idx / hd, e = idx - h * hd;
        out[j * heads * hd + idx] = e < dim ? kn[j * heads * dim + (size_t)h * dim + e] : r[j * rot + (e - dim)];
    }
}

// Row r of scores [rows][ld] (fp32, unscaled) belongs to position pos0 + r and sees keys 0 .. pos0 + r.  Its softmax
// (scores times scale, the sink in the denominator) is written as two bf16 numbers per weight, p = hi + lo, so that the
// product with the values keeps the weights' 32-bit precision in effect; keys out of sight get zeros.
__global__ void __launch_bounds__(256) softmax_split_kernel(const float* __restrict__ s, int ld, int n_pad, int pos0, float scale,
                                                            const void* sink, int sink_dtype, int head, bf16* __restrict__ hi,
                                                            bf16* __restrict__ lo, int ld_p) {
    __shared__ float red[8];
    __shared__ float bc;
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int n = min(pos0 + row + 1, n_pad);
    const float* sr = s + (size_t)row * ld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float m = -INFINITY;
    for (int j = threadIdx.x; j < n; j += blockDim.x) m = fmaxf(m, sr[j] * scale);
    m = fr_warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int i = 1; i < 8; ++i) t = fmaxf(t, red[i]);
        if (sink != nullptr) t = fmaxf(t, FrVec{sink, sink_dtype}.at(head));
        bc = t;
    }
    __syncthreads();
    m = bc;
    float l = 0.f;
    for (int j = threadIdx.x; j < n; j += blockDim.x) l += expf(sr[j] * scale - m);
    l = fr_warp_sum(l);
    __syncthreads();
    if (lane == 0) red[warp] = l;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; ++i) t += red[i];
        if (sink != nullptr) t += expf(FrVec{sink, sink_dtype}.at(head) - m);
        bc = 1.0f / t;
    }
    __syncthreads();
    const float inv = bc;
    bf16* h = hi + (size_t)row * ld_p;
    bf16* o = lo + (size_t)row * ld_p;
    for (int j = threadIdx.x; j < n_pad; j += blockDim.x) {
        const float p = j < n ? expf(sr[j] * scale - m) * inv : 0.f;
        const bf16 ph = __float2bfloat16_rn(p);
        h[j] = ph;
        o[j] = __float2bfloat16_rn(p - __bfloat162float(ph));
    }
}

// out[row][h * vd + n] = x[row][h * vd + n] * sigmoid(gate[row][gate_off + h]) (gate null: 1), fp32 -> T
template <typename T>
__global__ void gate_cast_kernel(const float* __restrict__ x, const T* __restrict__ gate, int ld_gate, int gate_off, int heads, int vd,
                                 T* __restrict__ out) {
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t row = blockIdx.x;
    for (int i = threadIdx.x; i < heads * vd; i += blockDim.x) {
        float v = x[row * heads * vd + i];
        if (gate != nullptr) v *= 1.0f / (1.0f + expf(-fr_load(gate + row * ld_gate + gate_off + i / vd)));
        fr_store(out + row * heads * vd + i, v);
    }
}

}  // namespace

FR_EXPORT int attention_latent_rotate_pairs(void* x, int ld, const int* row_seq, const int* row_pos, const float* freq, float mult,
                                            int rows, int heads, int head_stride, int first, int dims, int dtype,
                                            cudaStream_t stream) {
    if (rows <= 0 || heads <= 0 || dims <= 0) return FR_OK;
    if (dims % 2) FR_REFUSE("rotate_pairs: %d rotated dimensions (must be even)", dims);
    RotateArgs p{x, row_seq, row_pos, freq, mult, ld, rows, heads, head_stride, first, dims};
    if (dtype == FR_F32) FR_CUDA(fr_launch(rotate_pairs_kernel<float>, dim3(rows), dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(rotate_pairs_kernel<bf16>, dim3(rows), dim3(128), 0, stream, p));
    else FR_REFUSE("rotate_pairs: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("rotate_pairs");
    return FR_OK;
}

FR_EXPORT int attention_latent_prepare(const void* x, int ld, int q_off, int kv_off, void* ckr, float* qf, const void* norm_w,
                                       int norm_dtype, float eps, const int* row_seq, const int* row_pos, const float* freq,
                                       float mult, int rows, int heads, int dim, int rot, int rot_dims, int rank, int dtype,
                                       cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (rot_dims % 2 || rot_dims < 0 || rot_dims > rot || rank <= 0 || heads <= 0)
        FR_REFUSE("latent prepare: rank %d, rotated part %d of which %d turn, %d heads", rank, rot, rot_dims, heads);
    PrepareArgs p{x, ckr, qf, norm_w, norm_dtype, row_seq, row_pos, freq, mult, eps, ld, q_off, kv_off, heads, dim, rot, rank, rot_dims};
    if (dtype == FR_F32) FR_CUDA(fr_launch(prepare_kernel<float>, dim3(rows), dim3(256), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(prepare_kernel<bf16>, dim3(rows), dim3(256), 0, stream, p));
    else FR_REFUSE("latent prepare: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("latent prepare");
    return FR_OK;
}

// x_dtype / w_dtype / out_dtype: FR_F32 or FR_BF16 each; the gate (if any) is stored in the result's dtype.
FR_EXPORT int attention_latent_head_linear(const void* x, int x_dtype, int ld_x, int x_off, int x_stride, const void* w, int w_dtype,
                                           int layout, void* out, int out_dtype, int ld_out, int out_stride, const void* gate,
                                           int ld_gate, int gate_off, const int* row_seq, int rows, int heads, int k, int n,
                                           cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (heads <= 0 || k <= 0 || n <= 0) FR_REFUSE("head_linear: %d heads, k %d, n %d", heads, k, n);
    HeadLinearArgs p{x, w, out, gate, row_seq, rows, heads, k, n, ld_x, x_off, x_stride, ld_out, out_stride, ld_gate, gate_off};
    const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch_head_linear<float, float, float>(p, layout, stream);
        case 4 + 2 + 0: return launch_head_linear<bf16, bf16, float>(p, layout, stream);
        case 0 + 2 + 1: return launch_head_linear<float, bf16, bf16>(p, layout, stream);
        case 0 + 2 + 0: return launch_head_linear<float, bf16, float>(p, layout, stream);
        case 4 + 2 + 1: return launch_head_linear<bf16, bf16, bf16>(p, layout, stream);
        default: FR_REFUSE("head_linear: dtypes x %d, weights %d, out %d are not a combination that is built", x_dtype, w_dtype, out_dtype);
    }
}

FR_EXPORT int attention_latent(const float* q, float* out, const void* c_pool, const void* r_pool, const int* block_table,
                               int table_width, int page, const int* row_seq, const int* row_pos, const void* sink, int sink_dtype,
                               int rows, int heads, int rank, int rot, float scale, int splits, float* scratch, int dtype,
                               cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (rank <= 0 || rank > 32 * C_PER_LANE) FR_REFUSE("latent attention: latent size %d is outside 1..%d", rank, 32 * C_PER_LANE);
    if (rot < 0 || rot > 32 * R_PER_LANE) FR_REFUSE("latent attention: rotated part %d is outside 0..%d", rot, 32 * R_PER_LANE);
    if (splits < 1 || splits > 65535) FR_REFUSE("latent attention: %d splits", splits);
    if (splits > 1 && scratch == nullptr) FR_REFUSE("latent attention: splits need a scratch buffer");
    AttnArgs p{q, out, c_pool, r_pool, block_table, row_seq, row_pos, sink, sink_dtype, scratch, table_width, page, rows, heads, rank,
               rot, splits, scale};
    const int items = rows * heads;
    const dim3 grid((items + 3) / 4, splits);
    const bool pairs = rank % 2 == 0 && rot % 2 == 0 && (((uintptr_t)c_pool | (uintptr_t)r_pool) & 7) == 0;
    if (dtype == FR_F32 && pairs) FR_CUDA(fr_launch(latent_attention_kernel<float, 2>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_F32) FR_CUDA(fr_launch(latent_attention_kernel<float, 1>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16 && pairs) FR_CUDA(fr_launch(latent_attention_kernel<bf16, 2>, grid, dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(latent_attention_kernel<bf16, 1>, grid, dim3(128), 0, stream, p));
    else FR_REFUSE("latent attention: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("latent attention");
    if (splits > 1) {
        FR_CUDA(fr_launch(latent_merge_kernel, dim3((items + 3) / 4), dim3(128), 0, stream, p));
        FR_CHECK_LAUNCH("latent attention merge");
    }
    return FR_OK;
}

// One sequence's cached rows 0 .. n-1 (table: the sequence's row of the block table) as contiguous [2 n_pad][rank] (the
// latents twice, one below the other) and [n_pad][rot]; rows from n on are zero.
FR_EXPORT int attention_latent_gather(const void* c_pool, const void* r_pool, const int* table, int page, int n, int n_pad, int rank,
                                      int rot, void* c_all, void* r_all, int dtype, cudaStream_t stream) {
    if (n_pad <= 0) return FR_OK;
    if (dtype == FR_F32) FR_CUDA(fr_launch(gather_kernel<float>, dim3(n_pad), dim3(128), 0, stream, (const float*)c_pool, (const float*)r_pool, table, page, n, n_pad, rank, rot, (float*)c_all, (float*)r_all));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(gather_kernel<bf16>, dim3(n_pad), dim3(128), 0, stream, (const bf16*)c_pool, (const bf16*)r_pool, table, page, n, n_pad, rank, rot, (bf16*)c_all, (bf16*)r_all));
    else FR_REFUSE("latent gather: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("latent gather");
    return FR_OK;
}

// hi and lo: rows of ld_p numbers each (the two may be halves of one buffer's rows)
FR_EXPORT int attention_latent_softmax_split(const float* scores, int ld, int rows, int n_pad, int pos0, float scale, const void* sink,
                                             int sink_dtype, int head, void* hi, void* lo, int ld_p, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    FR_CUDA(fr_launch(softmax_split_kernel, dim3(rows), dim3(256), 0, stream, scores, ld, n_pad, pos0, scale, sink, sink_dtype, head,
                      (bf16*)hi, (bf16*)lo, ld_p));
    FR_CHECK_LAUNCH("softmax_split");
    return FR_OK;
}

FR_EXPORT int attention_latent_gate_cast(const float* x, const void* gate, int ld_gate, int gate_off, int rows, int heads, int vd,
                                         void* out, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (dtype == FR_F32) FR_CUDA(fr_launch(gate_cast_kernel<float>, dim3(rows), dim3(256), 0, stream, x, (const float*)gate, ld_gate, gate_off, heads, vd, (float*)out));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(gate_cast_kernel<bf16>, dim3(rows), dim3(256), 0, stream, x, (const bf16*)gate, ld_gate, gate_off, heads, vd, (bf16*)out));
    else FR_REFUSE("gate_cast: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("gate_cast");
    return FR_OK;
}

FR_EXPORT int attention_latent_key_concat(const void* kn, const void* r, int rows, int heads, int dim, int rot, void* out, int dtype,
                                          cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (dtype == FR_F32) FR_CUDA(fr_launch(key_concat_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)kn, (const float*)r, heads, dim, rot, (float*)out));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(key_concat_kernel<bf16>, dim3(rows), dim3(256), 0, stream, (const bf16*)kn, (const bf16*)r, heads, dim, rot, (bf16*)out));
    else FR_REFUSE("key_concat: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("key_concat");
    return FR_OK;
}
