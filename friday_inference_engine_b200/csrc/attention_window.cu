// Prompt attention for layers whose keys and values differ in size and whose window keeps a sequence's first keys in
// sight: bf16 operands on the tensor cores (mma.sync.m16n8k16, fp32 sums), softmax in fp32.
//
// Row i of a sequence sees key j if j <= i and (window == 0 or i - j < window or j < keep_first).  A CTA owns 64
// consecutive rows of one sequence and one query head; it walks the blocks of 64 keys (a page of the cache each) that
// any of its rows can see: the blocks that hold kept keys, then those of the window.  Per block: K [64][dk] and V
// transposed [dv][64] are staged in shared memory, S = Q K^T (fp32), mask, running maximum and sum per row, and
// O += P V.  The weights P stay 32-bit in effect: P is split into a bf16 head and a bf16 remainder (P = hi + lo to
// 2^-17) and both go through the tensor cores, so the second product sums what an fp32 P would give to 16 bits more than
// bf16 keeps.  Scores are exact products of bf16 numbers summed in fp32, scaled in fp32.
//
// Head sizes are rounded up to 32, 64 or 128 (zero filled); anything larger, and one-token steps, run on the CUDA-core
// kernel (attention_simt.cu).
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* attention_window_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 64, BN = 64, PAD = 8;

struct WinArgs {
    const bf16* q;        // [rows][q_stride], head h at h * dk
    bf16* out;            // [rows][nq * dv]
    const bf16* k_pool;   // [pages][64][nkv][dk]
    const bf16* v_pool;   // [pages][64][nkv][dv]
    const int* block_table;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_pos0;
    int table_width, q_stride, nq, nkv, dk, dv, window, keep_first;
    float scale, out_scale;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *(const uint32_t*)&v;
}

// head and remainder of two fp32 weights as packed bf16 pairs
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const bf16 hx = __float2bfloat16_rn(x), hy = __float2bfloat16_rn(y);
    const __nv_bfloat162 h = __halves2bfloat162(hx, hy);
    hi = *(const uint32_t*)&h;
    lo = pack2(x - __bfloat162float(hx), y - __bfloat162float(hy));
}

template <int DK, int DV>
__global__ void __launch_bounds__(128, 3) window_prefill_kernel(WinArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* sq = (bf16*)smem_raw;                           // [BM][DK + PAD]
    bf16* sk = sq + BM * (DK + PAD);                      // [BN][DK + PAD]
    bf16* svt = sk + BN * (DK + PAD);                     // [DV][BN + PAD]
    const int seq = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
    const int qlen = p.seq_qlen[seq];
    if (q0 >= qlen) return;
    const int row0 = p.seq_start[seq] + q0, pos0 = p.seq_pos0[seq] + q0;
    const int n_rows = min(BM, qlen - q0);
    const int kvh = h / (p.nq / p.nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    fr_pdl_wait();
    fr_pdl_launch();

    // ---- Q tile, zero filled beyond the rows and the head size
    for (int idx = tid; idx < BM * (DK / 8); idx += 128) {
        const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rows) {
            const bf16* src = p.q + (size_t)(row0 + r) * p.q_stride + (size_t)h * p.dk + c;
            if (c + 8 <= p.dk && (((uintptr_t)src) & 15) == 0) v = *(const uint4*)src;
            else {
                bf16* e = (bf16*)&v;
                for (int i = 0; i < 8; ++i) e[i] = c + i < p.dk ? src[i] : __float2bfloat16_rn(0.f);
            }
        }
        *(uint4*)(sq + r * (DK + PAD) + c) = v;
    }
    __syncthreads();
    uint32_t qa[DK / 16][4];
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
        const bf16* base = sq + (warp * 16 + g) * (DK + PAD) + ks * 16 + 2 * t;
        qa[ks][0] = *(const uint32_t*)base;
        qa[ks][1] = *(const uint32_t*)(base + 8 * (DK + PAD));
        qa[ks][2] = *(const uint32_t*)(base + 8);
        qa[ks][3] = *(const uint32_t*)(base + 8 * (DK + PAD) + 8);
    }

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int my_pos[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};

    // ---- the key blocks: those with kept keys below the window's start, then the window's
    const int last_pos = pos0 + n_rows - 1;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;             // earliest key of the window of the first row
    const int kept = p.window > 0 ? min(p.keep_first, lo) : 0;
    const int kept_blocks = (kept + BN - 1) / BN;
    const int first_window_block = lo / BN, last_block = last_pos / BN;
    const int* table = p.block_table + (size_t)seq * p.table_width;
    for (int b = 0; b <= last_block; ++b) {
        if (b >= kept_blocks && b < first_window_block) {
            b = first_window_block - 1;
            continue;
        }
        const int page = table[b];
        __syncthreads();                                   // the block before is done with sk and svt
        const bf16* kp = p.k_pool + ((size_t)page * BN * p.nkv + kvh) * p.dk;
        for (int idx = tid; idx < BN * (DK / 8); idx += 128) {
            const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
            const bf16* src = kp + (size_t)r * p.nkv * p.dk + c;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (b * BN + r <= last_pos) {
                if (c + 8 <= p.dk && (((uintptr_t)src) & 15) == 0) v = *(const uint4*)src;
                else {
                    bf16* e = (bf16*)&v;
                    for (int i = 0; i < 8; ++i) e[i] = c + i < p.dk ? src[i] : __float2bfloat16_rn(0.f);
                }
            }
            *(uint4*)(sk + r * (DK + PAD) + c) = v;
        }
        const bf16* vp = p.v_pool + ((size_t)page * BN * p.nkv + kvh) * p.dv;
        for (int idx = tid; idx < BN * (DV / 8); idx += 128) {
            // consecutive threads take consecutive keys of one piece of 8 channels: the transposed 2-byte stores below then
            // fall into different banks (consecutive pieces of one key's row, which would read memory in longer runs, put
            // sixteen threads on one bank and made the kernel a third slower)
            const int r = idx % BN, c = (idx / BN) * 8;
            const bf16* src = vp + (size_t)r * p.nkv * p.dv + c;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (b * BN + r <= last_pos) {
                if (c + 8 <= p.dv && (((uintptr_t)src) & 15) == 0) v = *(const uint4*)src;
                else {
                    bf16* e = (bf16*)&v;
                    for (int i = 0; i < 8; ++i) e[i] = c + i < p.dv ? src[i] : __float2bfloat16_rn(0.f);
                }
            }
            const bf16* e = (const bf16*)&v;
#pragma unroll
            for (int i = 0; i < 8; ++i) svt[(c + i) * (BN + PAD) + r] = e[i];
        }
        __syncthreads();

        // ---- S = Q K^T for this warp's 16 rows and the block's 64 keys
        float s[BN / 8][4];
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                const bf16* kb = sk + (nt * 8 + g) * (DK + PAD) + ks * 16 + 2 * t;
                mma_16816(s[nt], qa[ks], *(const uint32_t*)kb, *(const uint32_t*)(kb + 8));
            }
        }
        // ---- mask, running maximum and sum
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = b * BN + nt * 8 + 2 * t + (e & 1), half = e >> 1;
                const int pos = my_pos[half];
                const bool seen = j <= pos && pos <= last_pos && (p.window <= 0 || pos - j < p.window || j < p.keep_first);
                s[nt][e] = seen ? s[nt][e] * p.scale : -INFINITY;
                m_new[half] = fmaxf(m_new[half], s[nt][e]);
            }
        }
        float corr[2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 1));
            m_new[half] = fmaxf(m_new[half], __shfl_xor_sync(0xffffffffu, m_new[half], 2));
            corr[half] = m_new[half] == -INFINITY ? 1.f : expf(m_run[half] - m_new[half]);
            m_run[half] = m_new[half];
            l_run[half] *= corr[half];
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        float l_add[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int half = e >> 1;
                const float w = m_new[half] == -INFINITY ? 0.f : expf(s[nt][e] - m_new[half]);
                s[nt][e] = w;
                l_add[half] += w;
            }
        }
        l_run[0] += l_add[0];
        l_run[1] += l_add[1];
        // ---- O += P V, P as head and remainder
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t hi[4], lw[4];
            split2(s[2 * kk][0], s[2 * kk][1], hi[0], lw[0]);
            split2(s[2 * kk][2], s[2 * kk][3], hi[1], lw[1]);
            split2(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lw[2]);
            split2(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lw[3]);
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) {
                const bf16* vb = svt + (nt * 8 + g) * (BN + PAD) + kk * 16 + 2 * t;
                const uint32_t b0 = *(const uint32_t*)vb, b1 = *(const uint32_t*)(vb + 8);
                mma_16816(o[nt], hi, b0, b1);
                mma_16816(o[nt], lw, b0, b1);
            }
        }
    }
    // ---- the rows' sums over the four lanes that share a row, then the result
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 1);
        l_run[half] += __shfl_xor_sync(0xffffffffu, l_run[half], 2);
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int r = warp * 16 + g + 8 * half;
        if (r >= n_rows) continue;
        const float inv = l_run[half] > 0.f ? p.out_scale / l_run[half] : 0.f;
        bf16* dst = p.out + (size_t)(row0 + r) * p.nq * p.dv + (size_t)h * p.dv;
#pragma unroll
        for (int nt = 0; nt < DV / 8; ++nt) {
            const int c = nt * 8 + 2 * t;
            const float x = o[nt][2 * half] * inv, y = o[nt][2 * half + 1] * inv;
            if (c + 1 < p.dv && (((uintptr_t)(dst + c)) & 3) == 0) *(uint32_t*)(dst + c) = pack2(x, y);
            else {
                if (c < p.dv) dst[c] = __float2bfloat16_rn(x);
                if (c + 1 < p.dv) dst[c + 1] = __float2bfloat16_rn(y);
            }
        }
    }
}

template <int DK, int DV>
int launch(const WinArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    const size_t smem = ((size_t)(BM + BN) * (DK + PAD) + (size_t)DV * (BN + PAD)) * sizeof(bf16);
    static bool set = false;
    if (!set) {
        FR_CUDA(cudaFuncSetAttribute(window_prefill_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    const dim3 grid((max_q_len + BM - 1) / BM, p.nq, n_seqs);
    FR_CUDA(fr_launch(window_prefill_kernel<DK, DV>, grid, dim3(128), smem, stream, p));
    FR_CHECK_LAUNCH("attention_window");
    return FR_OK;
}

template <int DK>
int by_value_size(const WinArgs& p, int n_seqs, int max_q_len, cudaStream_t stream) {
    if (p.dv <= 32) return launch<DK, 32>(p, n_seqs, max_q_len, stream);
    if (p.dv <= 64) return launch<DK, 64>(p, n_seqs, max_q_len, stream);
    return launch<DK, 128>(p, n_seqs, max_q_len, stream);
}

}  // namespace

// 1 if the kernel takes these sizes (bf16 only; pages of 64)
FR_EXPORT int attention_window_fits(int dk, int dv, int page) { return dk >= 1 && dk <= 128 && dv >= 1 && dv <= 128 && page == 64; }

// q [rows][q_stride] bf16; out [rows][nq * dv] bf16; pools of pages of 64 positions.  Sequences bring seq_qlen rows from
// row seq_start, the first at position seq_pos0; their keys are in the cache already.
FR_EXPORT int attention_window(const void* q, int q_stride, void* out, const void* k_pool, const void* v_pool,
                               const int* block_table, int table_width, int page, const int* seq_start, const int* seq_qlen,
                               const int* seq_pos0, int n_seqs, int max_q_len, int nq, int nkv, int dk, int dv, int window,
                               int keep_first, float scale, float out_scale, cudaStream_t stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return FR_OK;
    if (!attention_window_fits(dk, dv, page)) FR_REFUSE("attention_window: head sizes %d and %d (1 to 128), pages of %d (64)", dk, dv, page);
    if (nkv <= 0 || nq % nkv != 0) FR_REFUSE("attention_window: %d heads cannot share %d key/value heads", nq, nkv);
    if (n_seqs > 65535 || nq > 65535) FR_REFUSE("attention_window: %d sequences, %d heads", n_seqs, nq);
    WinArgs p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool;
    p.block_table = block_table; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_pos0 = seq_pos0;
    p.table_width = table_width; p.q_stride = q_stride; p.nq = nq; p.nkv = nkv; p.dk = dk; p.dv = dv; p.window = window;
    p.keep_first = window > 0 ? keep_first : 0; p.scale = scale; p.out_scale = out_scale;
    if (dk <= 32) return by_value_size<32>(p, n_seqs, max_q_len, stream);
    if (dk <= 64) return by_value_size<64>(p, n_seqs, max_q_len, stream);
    return by_value_size<128>(p, n_seqs, max_q_len, stream);
}
