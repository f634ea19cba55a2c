// Mixers that carry a matrix-valued state per head from token to token (gated linear attention,
// token-shift time mixing with a data-dependent decay): the kernels around their products.
//
//   shift_mix        s-th mix of a row with the row before it: h + (h_prev - h) * mu_s; the row before a
//                    step's first row comes from the sequence's state
//   tanh_rows        x = tanh(x) in place
//   scan             per (sequence, head): the state S [dk][dv] walks the step's rows in order, starting from
//                    the sequence's stored state and ending there
//                        decay-first (bonus null):  S = diag(a_t) S + k_t v_t^T;   o_t = S^T q_t
//                        bonus (u given):            o_t = (S + diag(u) k_t v_t^T)^T q_t;   S = diag(a_t) S + k_t v_t^T
//                    a_t is formed here, in fp32, from the raw projection z_t (+ bias):
//                        mode 0:  a = sigmoid(z)^(1/tau) = exp(-softplus(-z) / tau)
//                        mode 1:  a = exp(-exp(z))
//   head_norm_gate   o / sqrt(mean_head(o^2) + eps) * weight * act(gate) * out_scale, per (row, head); act is silu or sigmoid
//
// The state, the decays, their logarithms and exponentials, the outer products and the unit norms are fp32
// whatever the activations' dtype; q, k, v and the gate come from products in the activation dtype.
//
// Long steps (prompts) are cut into segments that run side by side: the recurrence is linear in the state, so a
// segment that starts from zero yields U and the product D of its decays with S_end = diag(D) S_start + U; a second
// kernel walks the segments of a sequence in order (a few elementwise operations each) and leaves every segment's true
// starting state and the sequence's final state; a third runs the segments again from their true starts and writes the
// outputs.  The arithmetic is the recurrence's own, only grouped differently; everything stays fp32.
//
// A block of the scan owns `cols` value channels of one head: a thread keeps its column of S (dk numbers) in
// registers, the step's q, k and decays are staged through shared memory some tokens at a time.  Columns of S
// never mix, so any split of the value channels over blocks is exact.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* recurrence_last_error() { return fr_error_text; }

typedef __nv_bfloat16 bf16;

namespace {

struct MixArgs {
    const void* h;            // [rows][width]
    void* out;                // [n_mix][rows][width]
    const void* mu[8];        // n_mix vectors [width]
    int mu_dtype;
    const float* state;       // [slots][state_stride]: the last row of the step before, at offset 0
    long long state_stride;
    const int* row_seq;
    const int* seq_start;
    const int* seq_slots;
    int rows, width, n_mix;
};

template <typename T>
__global__ void shift_mix_kernel(MixArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int seq = p.row_seq[row];
    if (seq < 0) return;
    const T* h = (const T*)p.h + (size_t)row * p.width;
    const bool first = row == p.seq_start[seq];
    const float* sp = p.state + (size_t)p.seq_slots[seq] * p.state_stride;
    const T* hp = h - p.width;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < p.width; c += gridDim.y * blockDim.x) {
        const float x = fr_load(h + c);
        const float prev = first ? sp[c] : fr_load(hp + c);
        const float d = prev - x;
        for (int s = 0; s < p.n_mix; ++s) {
            const FrVec mu{p.mu[s], p.mu_dtype};
            fr_store((T*)p.out + ((size_t)s * p.rows + row) * p.width + c, fmaf(d, mu.at(c), x));
        }
    }
}

template <typename T>
__global__ void tanh_rows_kernel(T* x, long long n) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        fr_store(x + i, tanhf(fr_load(x + i)));
}

struct ScanArgs {
    const void* q;            // [rows][ld_q]   head h at h * dk      (the "receptance" of a time-mix layer)
    const void* k;            // [rows][ld_k]   head h at h * dk
    const void* v;            // [rows][ld_v]   head h at h * dv
    const float* z;           // [rows][heads * dk] raw decay projection, fp32
    const void* z_bias;       // [heads * dk] or null
    int z_bias_dtype;
    const void* bonus;        // [heads * dk] or null
    int bonus_dtype;
    float* out;               // [rows][heads * dv] fp32
    float* state;             // [slots][state_stride]
    long long state_stride, s_off;     // S of head h at state + slot * stride + s_off + h * dk * dv, laid out [dk][dv]
    const void* carry;        // rows [rows][carry_width] whose last one per sequence is kept at offset 0 of the state (or null)
    int carry_width;
    const int* row_seq;
    const int* seq_start;
    const int* seq_qlen;
    const int* seq_slots;
    int ld_q, ld_k, ld_v, heads, dk, dv, cols, mode;
    float q_scale, inv_tau;
    // segments (0: the whole step in one go)
    int seg_len, max_segs;
    float* seg_u;             // [n_seqs][max_segs][heads][dk][dv]: U of each segment, then its true starting state
    float* seg_d;             // [n_seqs][max_segs][heads][dk]: product of the segment's decays
};

constexpr int SCAN_TOKENS = 8;      // tokens staged at a time

__device__ __forceinline__ float decay_of(float z, int mode, float inv_tau) {
    if (mode == 0) {
        // sigmoid(z)^(1/tau) = exp(log_sigmoid(z) / tau); log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
        const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
        return expf(ls * inv_tau);
    }
    return expf(-expf(z));
}

// PHASE 0: the whole step from the stored state, outputs, state stored.  1: a segment from zero, no outputs, U and D
// stored.  2: a segment from its true start (seg_u), outputs.
template <typename T, int DK, int PHASE>
__global__ void scan_kernel(ScanArgs p) {
    extern __shared__ float sm[];
    float* sq = sm;                                   // [SCAN_TOKENS][DK]
    float* sk = sq + SCAN_TOKENS * DK;
    float* sa = sk + SCAN_TOKENS * DK;
    float* su = sa + SCAN_TOKENS * DK;                // [DK] bonus
    float* sd = su + DK;                              // [DK] product of the decays (PHASE 1)
    float* sv = sd + DK;                              // [SCAN_TOKENS][threads] each thread's value channel
    const int seq = PHASE == 0 ? blockIdx.x : blockIdx.x / p.max_segs, seg = PHASE == 0 ? 0 : blockIdx.x % p.max_segs;
    const int head = blockIdx.y;
    const int col = blockIdx.z * p.cols + threadIdx.x;
    const bool live_col = threadIdx.x < p.cols && col < p.dv;
    const int seq_r0 = p.seq_start[seq], seq_n = p.seq_qlen[seq];
    fr_pdl_wait();
    fr_pdl_launch();
    if (p.row_seq[seq_r0] < 0 || seq_n <= 0) return;
    if (PHASE != 0 && seg * p.seg_len >= seq_n) return;
    const int r0 = PHASE == 0 ? seq_r0 : seq_r0 + seg * p.seg_len;
    const int n = PHASE == 0 ? seq_n : min(p.seg_len, seq_n - seg * p.seg_len);
    float* slot = p.state + (size_t)p.seq_slots[seq] * p.state_stride;
    float* S = PHASE == 0 ? slot + p.s_off + (size_t)head * p.dk * p.dv
                          : p.seg_u + (((size_t)seq * p.max_segs + seg) * p.heads + head) * p.dk * p.dv;
    float s[DK];
#pragma unroll
    for (int i = 0; i < DK; ++i) s[i] = (PHASE != 1 && live_col && i < p.dk) ? S[(size_t)i * p.dv + col] : 0.f;
    if (PHASE == 1)
        for (int i = threadIdx.x; i < DK; i += blockDim.x) sd[i] = 1.f;
    const bool has_bonus = p.bonus != nullptr;
    for (int i = threadIdx.x; i < DK; i += blockDim.x)
        su[i] = (has_bonus && i < p.dk) ? FrVec{p.bonus, p.bonus_dtype}.at(head * p.dk + i) : 0.f;
    const FrVec zb{p.z_bias, p.z_bias_dtype};
    for (int t0 = 0; t0 < n; t0 += SCAN_TOKENS) {
        const int nt = min(SCAN_TOKENS, n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * DK; idx += blockDim.x) {
            const int t = idx / DK, i = idx - t * DK;
            float qv = 0.f, kv = 0.f, av = 0.f;
            if (i < p.dk) {
                const size_t row = (size_t)(r0 + t0 + t);
                if (PHASE != 1) qv = fr_load((const T*)p.q + row * p.ld_q + head * p.dk + i) * p.q_scale;
                kv = fr_load((const T*)p.k + row * p.ld_k + head * p.dk + i);
                float z = p.z[row * ((size_t)p.heads * p.dk) + head * p.dk + i];
                if (p.z_bias != nullptr) z += zb.at(head * p.dk + i);
                av = decay_of(z, p.mode, p.inv_tau);
            }
            sq[idx] = qv;
            sk[idx] = kv;
            sa[idx] = av;
        }
        // this thread's value channel of the staged tokens: loaded together, ahead of the chain that uses them
#pragma unroll
        for (int t = 0; t < SCAN_TOKENS; ++t)
            if (live_col && t < nt)
                sv[t * blockDim.x + threadIdx.x] = fr_load((const T*)p.v + (size_t)(r0 + t0 + t) * p.ld_v + head * p.dv + col);
        __syncthreads();
        if (PHASE == 1 && blockIdx.z == 0)
            for (int i = threadIdx.x; i < p.dk; i += blockDim.x) {
                float d = sd[i];
                for (int t = 0; t < nt; ++t) d *= sa[t * DK + i];
                sd[i] = d;
            }
        if (live_col) {
            for (int t = 0; t < nt; ++t) {
                const size_t row = (size_t)(r0 + t0 + t);
                const float vv = sv[t * blockDim.x + threadIdx.x];
                const float4* q4 = (const float4*)(sq + t * DK);
                const float4* k4 = (const float4*)(sk + t * DK);
                const float4* a4 = (const float4*)(sa + t * DK);
                const float4* u4 = (const float4*)su;
                float o = 0.f;
                if (PHASE == 1) {
#pragma unroll
                    for (int i = 0; i < DK / 4; ++i) {
                        const float4 k = k4[i], a = a4[i];
                        s[4 * i] = fmaf(a.x, s[4 * i], k.x * vv);
                        s[4 * i + 1] = fmaf(a.y, s[4 * i + 1], k.y * vv);
                        s[4 * i + 2] = fmaf(a.z, s[4 * i + 2], k.z * vv);
                        s[4 * i + 3] = fmaf(a.w, s[4 * i + 3], k.w * vv);
                    }
                    continue;
                }
                float o1 = 0.f, o2 = 0.f, o3 = 0.f;            // four chains instead of one
                if (has_bonus) {
#pragma unroll
                    for (int i = 0; i < DK / 4; ++i) {
                        const float4 q = q4[i], k = k4[i], a = a4[i], u = u4[i];
                        float kv;
                        kv = k.x * vv; o = fmaf(q.x, fmaf(u.x, kv, s[4 * i]), o);       s[4 * i] = fmaf(a.x, s[4 * i], kv);
                        kv = k.y * vv; o1 = fmaf(q.y, fmaf(u.y, kv, s[4 * i + 1]), o1); s[4 * i + 1] = fmaf(a.y, s[4 * i + 1], kv);
                        kv = k.z * vv; o2 = fmaf(q.z, fmaf(u.z, kv, s[4 * i + 2]), o2); s[4 * i + 2] = fmaf(a.z, s[4 * i + 2], kv);
                        kv = k.w * vv; o3 = fmaf(q.w, fmaf(u.w, kv, s[4 * i + 3]), o3); s[4 * i + 3] = fmaf(a.w, s[4 * i + 3], kv);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < DK / 4; ++i) {
                        const float4 q = q4[i], k = k4[i], a = a4[i];
                        s[4 * i] = fmaf(a.x, s[4 * i], k.x * vv);         o = fmaf(q.x, s[4 * i], o);
                        s[4 * i + 1] = fmaf(a.y, s[4 * i + 1], k.y * vv); o1 = fmaf(q.y, s[4 * i + 1], o1);
                        s[4 * i + 2] = fmaf(a.z, s[4 * i + 2], k.z * vv); o2 = fmaf(q.z, s[4 * i + 2], o2);
                        s[4 * i + 3] = fmaf(a.w, s[4 * i + 3], k.w * vv); o3 = fmaf(q.w, s[4 * i + 3], o3);
                    }
                }
                o = (o + o1) + (o2 + o3);
                p.out[row * ((size_t)p.heads * p.dv) + head * p.dv + col] = o;
            }
        }
    }
    if (PHASE != 2 && live_col) {
#pragma unroll
        for (int i = 0; i < DK; ++i)
            if (i < p.dk) S[(size_t)i * p.dv + col] = s[i];
    }
    if (PHASE == 1 && blockIdx.z == 0) {
        __syncthreads();
        float* D = p.seg_d + (((size_t)seq * p.max_segs + seg) * p.heads + head) * p.dk;
        for (int i = threadIdx.x; i < p.dk; i += blockDim.x) D[i] = sd[i];
    }
    // the step's last row becomes the row before the next step's first
    if (PHASE == 0 && p.carry != nullptr && head == 0 && blockIdx.z == 0) {
        const T* last = (const T*)p.carry + (size_t)(r0 + n - 1) * p.carry_width;
        for (int c = threadIdx.x; c < p.carry_width; c += blockDim.x) slot[c] = fr_load(last + c);
    }
}

// Walks a sequence's segments in order: seg_u[seg] becomes the segment's true starting state, the state after the last
// segment goes to the sequence's slot.  One thread per element of a head's matrix.
__global__ void __launch_bounds__(256) scan_combine_kernel(ScanArgs p, int carry_dtype) {
    const int seq = blockIdx.x, head = blockIdx.y;
    const int r0 = p.seq_start[seq], n = p.seq_qlen[seq];
    fr_pdl_wait();
    fr_pdl_launch();
    if (p.row_seq[r0] < 0 || n <= 0) return;
    const int segs = (n + p.seg_len - 1) / p.seg_len;
    float* slot = p.state + (size_t)p.seq_slots[seq] * p.state_stride;
    float* S = slot + p.s_off + (size_t)head * p.dk * p.dv;
    const int per = p.dk * p.dv;
    for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < per; e += gridDim.z * blockDim.x) {
        const int i = e / p.dv;
        float r = S[e];
        for (int s0 = 0; s0 < segs; s0 += 8) {              // eight segments' numbers are loaded together, then chained
            float u[8], d[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const size_t at = ((size_t)seq * p.max_segs + min(s0 + k, segs - 1)) * p.heads + head;
                u[k] = p.seg_u[at * per + e];
                d[k] = p.seg_d[at * p.dk + i];
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (s0 + k < segs) {
                    const size_t at = ((size_t)seq * p.max_segs + s0 + k) * p.heads + head;
                    p.seg_u[at * per + e] = r;
                    r = fmaf(d[k], r, u[k]);
                }
            }
        }
        S[e] = r;
    }
    if (p.carry != nullptr && head == 0 && blockIdx.z == 0) {
        for (int c = threadIdx.x; c < p.carry_width; c += blockDim.x) {
            const size_t at = (size_t)(r0 + n - 1) * p.carry_width + c;
            slot[c] = carry_dtype == FR_F32 ? ((const float*)p.carry)[at] : __bfloat162float(((const bf16*)p.carry)[at]);
        }
    }
}

struct NormGateArgs {
    const float* o;           // [rows][heads * dv]
    const void* gate;         // [rows][ld_gate], before its silu
    void* out;                // [rows][heads * dv]
    const void* weight;       // [dv] (shared by the heads) or [heads * dv]
    int weight_dtype, weight_per_head;
    const int* row_seq;
    int rows, heads, dv, ld_gate;
    float eps, out_scale;
    int gate_act;             // 0: silu(gate), 1: sigmoid(gate)
};

template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(NormGateArgs p) {
    fr_pdl_wait();
    fr_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * 4 + warp;
    if (item >= p.rows * p.heads) return;
    const int row = item / p.heads, head = item - row * p.heads;
    if (p.row_seq != nullptr && p.row_seq[row] < 0) return;
    const float* o = p.o + (size_t)row * p.heads * p.dv + (size_t)head * p.dv;
    float ss = 0.f;
    for (int c = lane; c < p.dv; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = fr_warp_sum(ss);
    const float inv = p.out_scale / sqrtf(ss / (float)p.dv + p.eps);
    const FrVec w{p.weight, p.weight_dtype};
    const T* g = (const T*)p.gate + (size_t)row * p.ld_gate + (size_t)head * p.dv;
    T* out = (T*)p.out + (size_t)row * p.heads * p.dv + (size_t)head * p.dv;
    for (int c = lane; c < p.dv; c += 32) {
        const float gv = fr_load(g + c);
        const float sg = 1.0f / (1.0f + expf(-gv));
        const float act = p.gate_act == 1 ? sg : gv * sg;
        fr_store(out + c, o[c] * inv * w.at(p.weight_per_head ? head * p.dv + c : c) * act);
    }
}

template <typename T, int DK>
int launch_scan(const ScanArgs& p, int n_seqs, int splits, int threads, cudaStream_t stream) {
    const size_t smem = ((size_t)(3 * SCAN_TOKENS + 2) * DK + (size_t)SCAN_TOKENS * threads) * sizeof(float);
    if (p.seg_len <= 0) {
        FR_CUDA(fr_launch(scan_kernel<T, DK, 0>, dim3(n_seqs, p.heads, splits), dim3(threads), smem, stream, p));
        FR_CHECK_LAUNCH("scan");
        return FR_OK;
    }
    const dim3 grid(n_seqs * p.max_segs, p.heads, splits);
    FR_CUDA(fr_launch(scan_kernel<T, DK, 1>, grid, dim3(threads), smem, stream, p));
    FR_CHECK_LAUNCH("scan (segments)");
    int zs = (p.dk * p.dv + 255) / 256;
    if (zs > 16) zs = 16;
    FR_CUDA(fr_launch(scan_combine_kernel, dim3(n_seqs, p.heads, zs), dim3(256), 0, stream, p,
                      (int)(sizeof(T) == 4 ? FR_F32 : FR_BF16)));
    FR_CHECK_LAUNCH("scan (combine)");
    FR_CUDA(fr_launch(scan_kernel<T, DK, 2>, grid, dim3(threads), smem, stream, p));
    FR_CHECK_LAUNCH("scan (outputs)");
    return FR_OK;
}

template <typename T>
int scan_by_size(const ScanArgs& p, int n_seqs, int splits, int threads, cudaStream_t stream) {
    if (p.dk <= 16) return launch_scan<T, 16>(p, n_seqs, splits, threads, stream);
    if (p.dk <= 32) return launch_scan<T, 32>(p, n_seqs, splits, threads, stream);
    if (p.dk <= 64) return launch_scan<T, 64>(p, n_seqs, splits, threads, stream);
    if (p.dk <= 128) return launch_scan<T, 128>(p, n_seqs, splits, threads, stream);
    if (p.dk <= 256) return launch_scan<T, 256>(p, n_seqs, splits, threads, stream);
    FR_REFUSE("scan: %d key channels per head (at most 256)", p.dk);
}

}  // namespace

FR_EXPORT int recurrence_shift_mix(const void* h, void* out, const void* const* mu, int n_mix, int mu_dtype, const float* state,
                                   long long state_stride, const int* row_seq, const int* seq_start, const int* seq_slots,
                                   int rows, int width, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    if (n_mix < 1 || n_mix > 8) FR_REFUSE("shift_mix: %d mixes (1 to 8)", n_mix);
    MixArgs p;
    p.h = h; p.out = out; p.mu_dtype = mu_dtype; p.state = state; p.state_stride = state_stride; p.row_seq = row_seq;
    p.seq_start = seq_start; p.seq_slots = seq_slots; p.rows = rows; p.width = width; p.n_mix = n_mix;
    for (int i = 0; i < 8; ++i) p.mu[i] = i < n_mix ? mu[i] : nullptr;
    const int tiles = rows < 256 ? (width + 255) / 256 : 1;       // few rows: spread a row's columns over blocks
    if (dtype == FR_F32) FR_CUDA(fr_launch(shift_mix_kernel<float>, dim3(rows, tiles), dim3(256), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(shift_mix_kernel<bf16>, dim3(rows, tiles), dim3(256), 0, stream, p));
    else FR_REFUSE("shift_mix: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("shift_mix");
    return FR_OK;
}

FR_EXPORT int recurrence_tanh_rows(void* x, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
    if (dtype == FR_F32) FR_CUDA(fr_launch(tanh_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)x, n));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(tanh_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, n));
    else FR_REFUSE("tanh_rows: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("tanh_rows");
    return FR_OK;
}

// How long a segment should be for a step whose longest sequence brings max_q_len rows (0: do not cut), and the
// floats of scratch that cutting needs.
FR_EXPORT int recurrence_scan_plan(int n_seqs, int max_q_len, int heads, int dk, int dv, long long* scratch_floats) {
    *scratch_floats = 0;
    if (max_q_len < 128) return 0;
    const int sms = fr_sm_count() > 0 ? fr_sm_count() : 128;
    // The chain of a segment waits on memory between its staged tokens, and only other warps hide that: a profile of
    // 7 warps per SM showed them stalled on loads three cycles of four.  So the segments are made short enough for
    // some 24 warps per SM (a warp owns 32 value channels of one head), 32 tokens at least and 256 at most.
    const long long base = (long long)n_seqs * heads * ((dv + 31) / 32);
    int seg = 256;
    while (seg > 32 && base * ((max_q_len + seg - 1) / seg) < 24LL * sms) seg >>= 1;
    const long long segs = (max_q_len + seg - 1) / seg;
    if (segs < 2) return 0;
    *scratch_floats = (long long)n_seqs * segs * heads * ((long long)dk * dv + dk);
    return seg;
}

// mode 0: a = sigmoid(z + bias)^(1/tau), mode 1: a = exp(-exp(z + bias)).  seg_len > 0 with seg_scratch (see
// recurrence_scan_plan) cuts long steps into segments that run side by side.  bonus null: the state is updated before it is
// read; otherwise it is read first, with bonus * k v^T added for the present token.  carry: see ScanArgs.
FR_EXPORT int recurrence_scan(const void* q, int ld_q, const void* k, int ld_k, const void* v, int ld_v, const float* z,
                              const void* z_bias, int z_bias_dtype, const void* bonus, int bonus_dtype, float* out, float* state,
                              long long state_stride, long long s_off, const void* carry, int carry_width, const int* row_seq,
                              const int* seq_start, const int* seq_qlen, const int* seq_slots, int n_seqs, int max_q_len,
                              int heads, int dk, int dv, int mode, float q_scale, float tau, int seg_len, float* seg_scratch,
                              int dtype, cudaStream_t stream) {
    if (n_seqs <= 0) return FR_OK;
    if (heads <= 0 || dk <= 0 || dv <= 0) FR_REFUSE("scan: heads %d, dk %d, dv %d", heads, dk, dv);
    if (mode == 0 && !(tau > 0.f)) FR_REFUSE("scan: tau must be positive");
    ScanArgs p;
    p.q = q; p.k = k; p.v = v; p.z = z; p.z_bias = z_bias; p.z_bias_dtype = z_bias_dtype; p.bonus = bonus; p.bonus_dtype = bonus_dtype;
    p.out = out; p.state = state; p.state_stride = state_stride; p.s_off = s_off; p.carry = carry; p.carry_width = carry_width;
    p.row_seq = row_seq; p.seq_start = seq_start; p.seq_qlen = seq_qlen; p.seq_slots = seq_slots;
    p.ld_q = ld_q; p.ld_k = ld_k; p.ld_v = ld_v; p.heads = heads; p.dk = dk; p.dv = dv; p.mode = mode;
    p.q_scale = q_scale; p.inv_tau = mode == 0 ? 1.0f / tau : 0.f;
    p.seg_len = 0; p.max_segs = 0; p.seg_u = nullptr; p.seg_d = nullptr;
    if (seg_len > 0 && seg_scratch != nullptr && max_q_len > seg_len) {
        p.seg_len = seg_len;
        p.max_segs = (max_q_len + seg_len - 1) / seg_len;
        p.seg_u = seg_scratch;
        p.seg_d = seg_scratch + (size_t)n_seqs * p.max_segs * heads * dk * dv;
    }
    // value channels per block: 32 where the device would otherwise stay empty, up to 128
    const int sms = fr_sm_count() > 0 ? fr_sm_count() : 128;
    int cols = 128;
    const long long segs = p.max_segs > 0 ? p.max_segs : 1;
    while (cols > 32 && (long long)n_seqs * segs * heads * ((dv + cols - 1) / cols) < 2LL * sms) cols >>= 1;
    if (cols > ((dv + 31) / 32) * 32) cols = ((dv + 31) / 32) * 32;
    p.cols = cols;
    const int splits = (dv + cols - 1) / cols;
    const int threads = cols < 64 ? 64 : cols;       // at least two warps stage the tokens
    (void)max_q_len;
    if (dtype == FR_F32) return scan_by_size<float>(p, n_seqs, splits, threads, stream);
    if (dtype == FR_BF16) return scan_by_size<bf16>(p, n_seqs, splits, threads, stream);
    FR_REFUSE("scan: unknown dtype %d", dtype);
}

FR_EXPORT int recurrence_head_norm_gate(const float* o, const void* gate, int ld_gate, void* out, const void* weight,
                                        int weight_dtype, int weight_per_head, const int* row_seq, int rows, int heads, int dv,
                                        float eps, float out_scale, int gate_act, int dtype, cudaStream_t stream) {
    if (rows <= 0) return FR_OK;
    NormGateArgs p;
    p.gate_act = gate_act;
    p.o = o; p.gate = gate; p.out = out; p.weight = weight; p.weight_dtype = weight_dtype; p.weight_per_head = weight_per_head;
    p.row_seq = row_seq; p.rows = rows; p.heads = heads; p.dv = dv; p.ld_gate = ld_gate; p.eps = eps; p.out_scale = out_scale;
    const int blocks = (rows * heads + 3) / 4;
    if (dtype == FR_F32) FR_CUDA(fr_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, stream, p));
    else if (dtype == FR_BF16) FR_CUDA(fr_launch(head_norm_gate_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, p));
    else FR_REFUSE("head_norm_gate: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("head_norm_gate");
    return FR_OK;
}
