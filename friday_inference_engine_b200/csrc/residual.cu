// Row-wise kernels for models whose residual stream is kept in 32-bit floats while their
// products run in the activation dtype: a norm that reads one dtype and writes another (with
// weights stored around zero or around one), [a; b] side by side in the activation dtype, the
// sum residual + alpha * y, the store of keys and values whose sizes differ, and the
// per-layer token input (a gated, normed projection of a small per-token table).
//
// All arithmetic is fp32; rounding happens only where a result is stored in bf16.
#include <math.h>

#include "common.cuh"

FR_EXPORT const char* residual_last_error() { return fr_error_text; }

namespace {

__device__ __forceinline__ float block_sum(float v, float* partial) {
    v = fr_warp_sum(v);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
    const int warps = (blockDim.x + 31) >> 5;
    for (int i = 0; i < warps; ++i) total += partial[i];
    __syncthreads();
    return total;
}

// y = x / sqrt(mean(x^2) + eps) * (offset + w), one block per row; x and y may differ in dtype.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
norm_cast_kernel(const TI* __restrict__ x, FrVec w, float offset, TO* __restrict__ y, int width, float eps) {
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const TI* xr = x + (size_t)blockIdx.x * width;
    TO* yr = y + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = fr_load(xr + i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) fr_store(yr + i, fr_load(xr + i) * inv * (offset + w.at(i)));
}

// out[r] = [a[r], b[r]] in the dtype of out
template <typename TI, typename TO>
__global__ void concat_cast_kernel(const TI* __restrict__ a, const TI* __restrict__ b, TO* __restrict__ out, int wa, int wb) {
    fr_pdl_wait();
    fr_pdl_launch();
    const size_t r = blockIdx.x;
    TO* o = out + r * (size_t)(wa + wb);
    for (int i = threadIdx.x; i < wa; i += blockDim.x) fr_store(o + i, fr_load(a + r * wa + i));
    for (int i = threadIdx.x; i < wb; i += blockDim.x) fr_store(o + wa + i, fr_load(b + r * wb + i));
}

// out = residual + alpha * y (+ beta * z)
template <typename TY>
__global__ void add_scaled_kernel(const float* __restrict__ residual, const TY* __restrict__ y, float alpha,
                                  const TY* __restrict__ z, float beta, float* __restrict__ out, long long n) {
    fr_pdl_wait();
    fr_pdl_launch();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = fmaf(alpha, fr_load(y + i), residual[i]);
        if (z != nullptr) v = fmaf(beta, fr_load(z + i), v);
        out[i] = v;
    }
}

// Keys [nkv][kd] at src + k_off and values [nkv][vd] at src + v_off of every live row go to the row of the paged
// cache that holds the row's position: pools [pages][page][nkv][kd] and [pages][page][nkv][vd].
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ src, int ld, int k_off, int v_off, int nkv, int kd, int vd,
                                const int* __restrict__ row_seq, const int* __restrict__ row_pos, T* __restrict__ k_pool,
                                T* __restrict__ v_pool, const int* __restrict__ block_table, int table_width, int page) {
    const int row = blockIdx.x;
    const int seq = row_seq[row];
    fr_pdl_wait();
    fr_pdl_launch();
    if (seq < 0) return;
    const int pos = row_pos[row];
    const int pg = block_table[(size_t)seq * table_width + pos / page];
    const size_t at = (size_t)pg * page + pos % page;
    const T* s = src + (size_t)row * ld;
    T* kd_ = k_pool + at * nkv * kd;
    T* vd_ = v_pool + at * nkv * vd;
    for (int i = threadIdx.x; i < nkv * kd; i += blockDim.x) kd_[i] = s[k_off + i];
    for (int i = threadIdx.x; i < nkv * vd; i += blockDim.x) vd_[i] = s[v_off + i];
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// The per-layer token input, one block per row, in place on the 32-bit residual stream:
//   e = table[token][col0 .. col0 + dim);  g = gelu_tanh(gate x) * e;  y = proj g;
//   x += y / sqrt(mean(y^2) + eps) * norm
// gate [dim][width], proj [width][dim], norm [width], table [vocab][table_ld] in the dtype TW.
template <typename TW>
__global__ void __launch_bounds__(256)
token_input_kernel(float* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ row_seq,
                   const TW* __restrict__ table, int table_ld, int col0, int vocab, const TW* __restrict__ gate,
                   const TW* __restrict__ proj, FrVec norm, int width, int dim, float eps) {
    extern __shared__ float sm[];
    float* g = sm;                // [dim]
    float* y = sm + dim;          // [width]
    __shared__ float partial[32];
    fr_pdl_wait();
    fr_pdl_launch();
    const int row = blockIdx.x;
    const int token = tokens[row];
    if ((row_seq != nullptr && row_seq[row] < 0) || token < 0 || token >= vocab) return;
    float* xr = x + (size_t)row * width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int d = warp; d < dim; d += warps) {
        const TW* gr = gate + (size_t)d * width;
        float s = 0.f;
        for (int c = lane; c < width; c += 32) s = fmaf(xr[c], fr_load(gr + c), s);
        s = fr_warp_sum(s);
        if (lane == 0) g[d] = gelu_tanh(s) * fr_load(table + (size_t)token * table_ld + col0 + d);
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const TW* pr = proj + (size_t)c * dim;
        float s = 0.f;
        for (int d = 0; d < dim; ++d) s = fmaf(g[d], fr_load(pr + d), s);
        y[c] = s;
        ss = fmaf(s, s, ss);
    }
    ss = block_sum(ss, partial);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) xr[c] += y[c] * inv * norm.at(c);
}

inline int blocks_for(long long n) {
    const long long cap = (long long)(fr_sm_count() > 0 ? fr_sm_count() : 128) * 16;
    const long long want = (n + 255) / 256;
    return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

}  // namespace

typedef __nv_bfloat16 bf16;

FR_EXPORT int residual_norm_cast(const void* x, int in_dtype, const void* w, int w_dtype, float offset, void* y, int out_dtype,
                                 int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    FrVec wv{w, w_dtype};
    const int key = in_dtype * 2 + out_dtype;
    switch (key) {
        case 0: FR_CUDA(fr_launch(norm_cast_kernel<float, float>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, offset, (float*)y, width, eps)); break;
        case 1: FR_CUDA(fr_launch(norm_cast_kernel<float, bf16>, dim3(n_rows), dim3(256), 0, stream, (const float*)x, wv, offset, (bf16*)y, width, eps)); break;
        case 2: FR_CUDA(fr_launch(norm_cast_kernel<bf16, float>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, offset, (float*)y, width, eps)); break;
        case 3: FR_CUDA(fr_launch(norm_cast_kernel<bf16, bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)x, wv, offset, (bf16*)y, width, eps)); break;
        default: FR_REFUSE("norm_cast: unknown dtypes %d -> %d", in_dtype, out_dtype);
    }
    FR_CHECK_LAUNCH("norm_cast");
    return FR_OK;
}

FR_EXPORT int residual_concat_cast(const void* a, const void* b, int in_dtype, void* out, int out_dtype, int n_rows, int wa,
                                   int wb, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const int key = in_dtype * 2 + out_dtype;
    switch (key) {
        case 0: FR_CUDA(fr_launch(concat_cast_kernel<float, float>, dim3(n_rows), dim3(256), 0, stream, (const float*)a, (const float*)b, (float*)out, wa, wb)); break;
        case 1: FR_CUDA(fr_launch(concat_cast_kernel<float, bf16>, dim3(n_rows), dim3(256), 0, stream, (const float*)a, (const float*)b, (bf16*)out, wa, wb)); break;
        case 2: FR_CUDA(fr_launch(concat_cast_kernel<bf16, float>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, (float*)out, wa, wb)); break;
        case 3: FR_CUDA(fr_launch(concat_cast_kernel<bf16, bf16>, dim3(n_rows), dim3(256), 0, stream, (const bf16*)a, (const bf16*)b, (bf16*)out, wa, wb)); break;
        default: FR_REFUSE("concat_cast: unknown dtypes %d -> %d", in_dtype, out_dtype);
    }
    FR_CHECK_LAUNCH("concat_cast");
    return FR_OK;
}

// out [n] fp32 = residual [n] fp32 + alpha * y [n] (+ beta * z [n]); y and z in y_dtype; out may be residual.
FR_EXPORT int residual_add_scaled(const float* residual, const void* y, float alpha, const void* z, float beta, int y_dtype,
                                  float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return FR_OK;
    if (y_dtype == FR_F32)
        FR_CUDA(fr_launch(add_scaled_kernel<float>, dim3(blocks_for(n)), dim3(256), 0, stream, residual, (const float*)y, alpha,
                          (const float*)z, beta, out, n));
    else if (y_dtype == FR_BF16)
        FR_CUDA(fr_launch(add_scaled_kernel<bf16>, dim3(blocks_for(n)), dim3(256), 0, stream, residual, (const bf16*)y, alpha,
                          (const bf16*)z, beta, out, n));
    else
        FR_REFUSE("add_scaled: unknown dtype %d", y_dtype);
    FR_CHECK_LAUNCH("add_scaled");
    return FR_OK;
}

FR_EXPORT int residual_kv_store(const void* src, int ld, int k_off, int v_off, int nkv, int kd, int vd, const int* row_seq,
                                const int* row_pos, void* k_pool, void* v_pool, const int* block_table, int table_width,
                                int page, int n_rows, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    if (k_pool == nullptr || v_pool == nullptr || block_table == nullptr) FR_REFUSE("kv_store: no cache to write to");
    if (dtype == FR_F32)
        FR_CUDA(fr_launch(kv_store_kernel<float>, dim3(n_rows), dim3(128), 0, stream, (const float*)src, ld, k_off, v_off, nkv, kd,
                          vd, row_seq, row_pos, (float*)k_pool, (float*)v_pool, block_table, table_width, page));
    else if (dtype == FR_BF16)
        FR_CUDA(fr_launch(kv_store_kernel<bf16>, dim3(n_rows), dim3(128), 0, stream, (const bf16*)src, ld, k_off, v_off, nkv, kd,
                          vd, row_seq, row_pos, (bf16*)k_pool, (bf16*)v_pool, block_table, table_width, page));
    else
        FR_REFUSE("kv_store: unknown dtype %d", dtype);
    FR_CHECK_LAUNCH("kv_store");
    return FR_OK;
}

FR_EXPORT int residual_token_input(float* x, const int* tokens, const int* row_seq, const void* table, int table_ld, int col0,
                                   int vocab, const void* gate, const void* proj, const void* norm, int norm_dtype, int n_rows,
                                   int width, int dim, float eps, int w_dtype, cudaStream_t stream) {
    if (n_rows <= 0) return FR_OK;
    const size_t smem = (size_t)(dim + width) * sizeof(float);
    if (smem > 200 * 1024) FR_REFUSE("token_input: width %d and dim %d need more shared memory than an SM has", width, dim);
    FrVec nv{norm, norm_dtype};
    if (w_dtype == FR_F32) {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(token_input_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(token_input_kernel<float>, dim3(n_rows), dim3(256), smem, stream, x, tokens, row_seq, (const float*)table,
                          table_ld, col0, vocab, (const float*)gate, (const float*)proj, nv, width, dim, eps));
    } else if (w_dtype == FR_BF16) {
        if (smem > 48 * 1024) FR_CUDA(cudaFuncSetAttribute(token_input_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        FR_CUDA(fr_launch(token_input_kernel<bf16>, dim3(n_rows), dim3(256), smem, stream, x, tokens, row_seq, (const bf16*)table,
                          table_ld, col0, vocab, (const bf16*)gate, (const bf16*)proj, nv, width, dim, eps));
    } else {
        FR_REFUSE("token_input: unknown dtype %d", w_dtype);
    }
    FR_CHECK_LAUNCH("token_input");
    return FR_OK;
}
