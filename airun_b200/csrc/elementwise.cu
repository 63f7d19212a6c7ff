// Embedding gather, RMSNorm with the residual add (and a row gather) fused in,
// and the SwiGLU product.  All arithmetic is float32; storage may be bfloat16.
//
// Formulas as the reference computes them:
//   embedding  x[t] = E[token[t]], an id outside the table reads row 0
//              (crates/airun-cuda/kernels/ops.cu:227-252);
//   RMSNorm    out = x * rsqrt(sum(x^2)/n + eps) * w   (ops.cu:12-41);
//   add+norm   x += delta, then the norm of the sum    (ops.cu:47-78);
//   SwiGLU     out = g / (1 + exp(-g)) * u             (ops.cu:191-200).
#include "common.cuh"

template <typename TTab>
__global__ void embed_kernel(const TTab* __restrict__ table, const int32_t* __restrict__ ids,
                             float* __restrict__ out, int H, int V, int* __restrict__ err) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && err) atomicOr(err, AIRUN_DEV_BAD_TOKEN);
        id = 0;
    }
    const TTab* src = table + (size_t)id * H;
    float* dst = out + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32<TTab>(src[i]);
}

AIRUN_EXPORT int airun_embed(const void* table, int table_dtype, const int32_t* ids, float* out,
                             int T, int H, int V, int* err, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == AIRUN_DT_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>((const float*)table, ids, out, H, V, err);
    else if (table_dtype == AIRUN_DT_BF16)
        embed_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, H, V, err);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// One block per output row.  Source row = rows ? rows[r] : r.  With `delta` the
// sum x + delta is normed; it is written back to x only when write_back is set
// (a gathered final norm leaves x alone).
template <typename TOut>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                               const float* __restrict__ w, TOut* __restrict__ out,
                               const int32_t* __restrict__ rows, int n, float eps, int write_back) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * n;
    const float* dr = delta ? delta + (size_t)src * n : nullptr;
    TOut* outr = out + (size_t)r * n;

    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (dr) {
            v += dr[i];
            if (write_back) xr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (dr && !write_back) v += dr[i];
        outr[i] = from_f32<TOut>(v * inv * (w ? w[i] : 1.0f));
    }
}

AIRUN_EXPORT int airun_rmsnorm(float* x, const float* delta, const float* w, void* out, int out_dtype,
                               const int32_t* rows, int n_rows, int n, float eps, int write_back,
                               cudaStream_t stream) {
    if (n_rows < 0 || n <= 0) return AIRUN_ERR_ARG;
    if (rows && write_back) return AIRUN_ERR_ARG;
    if (n_rows == 0) return AIRUN_OK;
    int threads = ((n + 3) / 4 + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    if (out_dtype == AIRUN_DT_F32)
        rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>(x, delta, w, (float*)out, rows, n, eps, write_back);
    else if (out_dtype == AIRUN_DT_BF16)
        rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(x, delta, w, (__nv_bfloat16*)out, rows, n, eps, write_back);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// in: [T][2*I] where blocks of `group` gate columns alternate with blocks of
// `group` up columns (group == I means plain [gate | up] halves).  out: [T][I].
template <typename TIn, typename TOut>
__global__ void swiglu_kernel(const TIn* __restrict__ in, TOut* __restrict__ out,
                              long long total, int I, int group) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / I;
    const int i = (int)(idx - t * I);
    const int b = i / group, o = i - b * group;
    const TIn* row = in + t * 2 * (long long)I;
    const float g = to_f32<TIn>(row[(size_t)(2 * b) * group + o]);
    const float u = to_f32<TIn>(row[(size_t)(2 * b + 1) * group + o]);
    out[idx] = from_f32<TOut>(g / (1.0f + expf(-g)) * u);
}

AIRUN_EXPORT int airun_swiglu(const void* in, int in_dtype, void* out, int out_dtype,
                              int T, int I, int group, cudaStream_t stream) {
    if (T < 0 || I <= 0 || group <= 0 || I % group != 0) return AIRUN_ERR_ARG;
    const long long total = (long long)T * I;
    if (total == 0) return AIRUN_OK;
    const int threads = 256;
    const int blocks = ceil_div_i(total, threads);
    if (in_dtype == AIRUN_DT_F32 && out_dtype == AIRUN_DT_F32)
        swiglu_kernel<float, float><<<blocks, threads, 0, stream>>>((const float*)in, (float*)out, total, I, group);
    else if (in_dtype == AIRUN_DT_F32 && out_dtype == AIRUN_DT_BF16)
        swiglu_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, total, I, group);
    else if (in_dtype == AIRUN_DT_BF16 && out_dtype == AIRUN_DT_BF16)
        swiglu_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, I, group);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// out[r] = in[rows[r]] for rows of n elements of `elt` bytes (n*elt a multiple of 4).
__global__ void gather_rows_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                   const int32_t* __restrict__ rows, int words) {
    const uint32_t* s = in + (size_t)rows[blockIdx.x] * words;
    uint32_t* d = out + (size_t)blockIdx.x * words;
    for (int i = threadIdx.x; i < words; i += blockDim.x) d[i] = s[i];
}

AIRUN_EXPORT int airun_gather_rows(const void* in, void* out, const int32_t* rows, int n_rows,
                                   int row_bytes, cudaStream_t stream) {
    if (n_rows < 0 || row_bytes <= 0 || row_bytes % 4 != 0) return AIRUN_ERR_ARG;
    if (n_rows == 0) return AIRUN_OK;
    gather_rows_kernel<<<n_rows, 256, 0, stream>>>((const uint32_t*)in, (uint32_t*)out, rows, row_bytes / 4);
    return airun_launch_status();
}
