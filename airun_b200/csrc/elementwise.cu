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
#include <type_traits>

template <typename TTab>
__global__ void embed_kernel(const TTab* __restrict__ table, const int32_t* __restrict__ ids,
                             float* __restrict__ out, int H, int V, float scale, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0 && err) atomicOr(err, AIRUN_DEV_BAD_TOKEN);
        id = 0;
    }
    const TTab* src = table + (size_t)id * H;
    float* dst = out + (size_t)t * H;
    // scale 1 (no scaling, as the reference) leaves the value as it is: x * 1.0f is exact
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32<TTab>(src[i]) * scale;
}

AIRUN_EXPORT int airun_embed(const void* table, int table_dtype, const int32_t* ids, float* out,
                             int T, int H, int V, float scale, int* err, cudaStream_t stream) {
    if (T < 0 || H <= 0 || V <= 0) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == AIRUN_DT_F32)
        airun_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, out, H, V, scale, err);
    else if (table_dtype == AIRUN_DT_BF16)
        airun_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, out, H, V, scale, err);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// One block per output row.  Source row = rows ? rows[r] : r.  With `delta` the
// sum x + delta is normed; it is written back to x only when write_back is set
// (a gathered final norm leaves x alone).  VEC = 4 reads float4 (n % 4 == 0) and keeps up to
// KEEP vectors per thread in registers between the two passes; longer rows are read again.
#define KEEP 4
template <typename TOut, int VEC>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                               const float* __restrict__ w, TOut* __restrict__ out,
                               const int32_t* __restrict__ rows, int n, float eps, int write_back) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * n;
    const float* dr = delta ? delta + (size_t)src * n : nullptr;
    TOut* outr = out + (size_t)r * n;
    const int nv = n / VEC;                       // vectors in the row
    float keep[KEEP][VEC];
    float ss = 0.0f;
    // All loads of x and delta first, then the sums and the stores: a load issued after a store through the
    // same pointer waits for it, and four such round trips in turn were most of this kernel's time at a
    // few rows (3.9 us of a decode layer's two norms each).
    float dk[KEEP][VEC];
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
#pragma unroll
        for (int e = 0; e < VEC; ++e) { keep[k][e] = 0.0f; dk[k][e] = 0.0f; }
        if (i < nv) {
            if (VEC == 4) {
                const float4 v = reinterpret_cast<const float4*>(xr)[i];
                keep[k][0] = v.x; keep[k][1 % VEC] = v.y; keep[k][2 % VEC] = v.z; keep[k][3 % VEC] = v.w;
                if (dr) {
                    const float4 d = reinterpret_cast<const float4*>(dr)[i];
                    dk[k][0] = d.x; dk[k][1 % VEC] = d.y; dk[k][2 % VEC] = d.z; dk[k][3 % VEC] = d.w;
                }
            } else {
                keep[k][0] = xr[i];
                if (dr) dk[k][0] = dr[i];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nv) {
            if (dr) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) keep[k][e] += dk[k][e];
                if (write_back) {
                    if (VEC == 4) reinterpret_cast<float4*>(xr)[i] = make_float4(keep[k][0], keep[k][1 % VEC], keep[k][2 % VEC], keep[k][3 % VEC]);
                    else xr[i] = keep[k][0];
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) ss = fmaf(keep[k][e], keep[k][e], ss);
        }
    }
    for (int i = threadIdx.x + KEEP * blockDim.x; i < nv; i += blockDim.x) {       // the rest of a long row
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float v = xr[i * VEC + e];
            if (dr) { v += dr[i * VEC + e]; if (write_back) xr[i * VEC + e] = v; }
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)n + eps);
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nv) {
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                outr[i * VEC + e] = from_f32<TOut>(keep[k][e] * inv * (w ? w[i * VEC + e] : 1.0f));
        }
    }
    for (int i = threadIdx.x + KEEP * blockDim.x; i < nv; i += blockDim.x) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float v = xr[i * VEC + e];
            if (dr && !write_back) v += dr[i * VEC + e];
            outr[i * VEC + e] = from_f32<TOut>(v * inv * (w ? w[i * VEC + e] : 1.0f));
        }
    }
}

// Many rows: one warp per row, no block-wide synchronisation.  The loads of a batch of RB float4 per
// lane (and as many of delta) are all issued before the first of them is used or anything is stored:
// a load after a store through the same pointer would otherwise wait for it.  The sum x + delta is
// written back and read again (from cache) for the second pass.
#define RB 8
template <typename TOut>
__global__ __launch_bounds__(256) void rmsnorm_rows_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                           const float* __restrict__ w, TOut* __restrict__ out,
                                                           int n_rows, int n, float eps, int write_back) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    float4* xr = reinterpret_cast<float4*>(x + (size_t)row * n);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + (size_t)row * n) : nullptr;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    TOut* outr = out + (size_t)row * n;
    const int nv = n >> 2;
    float ss = 0.0f;
    const bool rewrite = dr && write_back;
    for (int i0 = lane; i0 < nv; i0 += 32 * RB) {
        float4 v[RB], d[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = i0 + 32 * u;
            v[u] = i < nv ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (dr) {
#pragma unroll
            for (int u = 0; u < RB; ++u) {
                const int i = i0 + 32 * u;
                d[u] = i < nv ? dr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int u = 0; u < RB; ++u) { v[u].x += d[u].x; v[u].y += d[u].y; v[u].z += d[u].z; v[u].w += d[u].w; }
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = i0 + 32 * u;
            if (rewrite && i < nv) xr[i] = v[u];
            ss = fmaf(v[u].x, v[u].x, fmaf(v[u].y, v[u].y, fmaf(v[u].z, v[u].z, fmaf(v[u].w, v[u].w, ss))));
        }
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i0 = lane; i0 < nv; i0 += 32 * RB) {
        float4 v[RB], g[RB];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = i0 + 32 * u;
            v[u] = i < nv ? xr[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            g[u] = (w && i < nv) ? w4[i] : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        }
        if (dr && !rewrite) {
#pragma unroll
            for (int u = 0; u < RB; ++u) {
                const int i = i0 + 32 * u;
                if (i < nv) { const float4 d = dr[i]; v[u].x += d.x; v[u].y += d.y; v[u].z += d.z; v[u].w += d.w; }
            }
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int i = i0 + 32 * u;
            if (i >= nv) continue;
            const float a = v[u].x * inv * g[u].x, b = v[u].y * inv * g[u].y, c = v[u].z * inv * g[u].z, d2 = v[u].w * inv * g[u].w;
            if (sizeof(TOut) == 4) {
                reinterpret_cast<float4*>(outr)[i] = make_float4(a, b, c, d2);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d2);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(outr)[i] = pk;
            }
        }
    }
}

AIRUN_EXPORT int airun_rmsnorm(float* x, const float* delta, const float* w, void* out, int out_dtype,
                               const int32_t* rows, int n_rows, int n, float eps, int write_back,
                               cudaStream_t stream) {
    if (n_rows < 0 || n <= 0) return AIRUN_ERR_ARG;
    if (rows && write_back) return AIRUN_ERR_ARG;
    if (n_rows == 0) return AIRUN_OK;
    const bool vec = n % 4 == 0 && (((uintptr_t)x | (uintptr_t)delta) & 15) == 0;
    if (vec && !rows && n_rows >= 256 && n >= 512 && (((uintptr_t)out | (uintptr_t)w) & 15) == 0) {
        // enough warps per block that the blocks still cover the SMs twice
        const int wpb = n_rows >= 2368 ? 8 : n_rows >= 1184 ? 4 : 2;
        const int blocks = (n_rows + wpb - 1) / wpb;
        if (out_dtype == AIRUN_DT_F32)
            airun_launch(rmsnorm_rows_kernel<float>, dim3(blocks), dim3(32 * wpb), 0, stream, x, delta, w, (float*)out, n_rows, n, eps, write_back);
        else if (out_dtype == AIRUN_DT_BF16)
            airun_launch(rmsnorm_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(32 * wpb), 0, stream, x, delta, w, (__nv_bfloat16*)out, n_rows, n, eps, write_back);
        else
            return AIRUN_ERR_UNSUPPORTED;
        return airun_launch_status();
    }
    const int nv = vec ? n / 4 : n;
    int threads = (nv + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    if (n_rows <= 64 && threads > 256 && vec) threads = 256;      // few rows: more loads in flight per thread
#define LAUNCH(TOut, VEC) \
    airun_launch(rmsnorm_kernel<TOut, VEC>, dim3(n_rows), dim3(threads), 0, stream, x, delta, w, (TOut*)out, rows, n, eps, write_back)
    if (out_dtype == AIRUN_DT_F32) { if (vec) LAUNCH(float, 4); else LAUNCH(float, 1); }
    else if (out_dtype == AIRUN_DT_BF16) { if (vec) LAUNCH(__nv_bfloat16, 4); else LAUNCH(__nv_bfloat16, 1); }
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}

// in: [T][2*I] where blocks of `group` gate columns alternate with blocks of
// `group` up columns (group == I means plain [gate | up] halves).  out: [T][I].
template <typename TIn, typename TOut>
__global__ void swiglu_kernel(const TIn* __restrict__ in, TOut* __restrict__ out,
                              long long total, int I, int group) {
    pdl_trigger();
    pdl_wait();
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
        airun_launch(swiglu_kernel<float, float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, total, I, group);
    else if (in_dtype == AIRUN_DT_F32 && out_dtype == AIRUN_DT_BF16)
        airun_launch(swiglu_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (__nv_bfloat16*)out, total, I, group);
    else if (in_dtype == AIRUN_DT_BF16 && out_dtype == AIRUN_DT_BF16)
        airun_launch(swiglu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, total, I, group);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// out[r] = in[rows[r]] for rows of n elements of `elt` bytes (n*elt a multiple of 4).
__global__ void gather_rows_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                   const int32_t* __restrict__ rows, int words) {
    pdl_trigger();
    pdl_wait();
    const uint32_t* s = in + (size_t)rows[blockIdx.x] * words;
    uint32_t* d = out + (size_t)blockIdx.x * words;
    for (int i = threadIdx.x; i < words; i += blockDim.x) d[i] = s[i];
}

AIRUN_EXPORT int airun_gather_rows(const void* in, void* out, const int32_t* rows, int n_rows,
                                   int row_bytes, cudaStream_t stream) {
    if (n_rows < 0 || row_bytes <= 0 || row_bytes % 4 != 0) return AIRUN_ERR_ARG;
    if (n_rows == 0) return AIRUN_OK;
    airun_launch(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, (const uint32_t*)in, (uint32_t*)out, rows, row_bytes / 4);
    return airun_launch_status();
}

// Random weights from a counter: element i of a tensor with key k is a function of (k, i) alone, so
// the host and the device fill the same tensor bit for bit and no generator state is carried.
//   h(c)  = mix(k + c * 0x9E3779B97F4A7C15), mix = the finaliser of splitmix64;
//   z     = (sum of the twelve 16-bit fields of h(3i), h(3i+1), h(3i+2) - 393210) / 65536:
//           integers up to there, so exact; mean 0, variance 1 - 2^-32, |z| <= 6;
//   kind 0: w = z * scale            (one float32 product)
//   kind 1: w = 1 + z * scale        (product, then sum: two roundings, never fused)
//   kind 2: w = h(3i) & 0x7fff       (int32)
// The reference has no random-weights mode; its benchmark makes token ids from a seeded xorshift the
// same stateless way (crates/airun-cli/src/bench.rs:177-187).
__device__ __forceinline__ unsigned long long fill_mix(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename TOut>
__global__ void fill_random_kernel(TOut* __restrict__ out, long long n, unsigned long long key, int kind, float scale) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned long long c = 3ull * (unsigned long long)i;
    const unsigned long long h0 = fill_mix(key + c * 0x9E3779B97F4A7C15ull);
    if constexpr (std::is_same<TOut, int32_t>::value) {
        out[i] = (int32_t)(h0 & 0x7fffull);
    } else {
        const unsigned long long h1 = fill_mix(key + (c + 1) * 0x9E3779B97F4A7C15ull);
        const unsigned long long h2 = fill_mix(key + (c + 2) * 0x9E3779B97F4A7C15ull);
        int s = 0;
#pragma unroll
        for (int f = 0; f < 4; ++f)
            s += (int)((h0 >> (16 * f)) & 0xffff) + (int)((h1 >> (16 * f)) & 0xffff) + (int)((h2 >> (16 * f)) & 0xffff);
        const float z = (float)(s - 393210) * (1.0f / 65536.0f);
        float w = __fmul_rn(z, scale);
        if (kind == 1) w = __fadd_rn(1.0f, w);
        out[i] = from_f32<TOut>(w);
    }
}

AIRUN_EXPORT int airun_fill_random(void* out, int out_dtype, long long n, unsigned long long key, int kind, float scale,
                                   cudaStream_t stream) {
    if (n < 0 || kind < 0 || kind > 2) return AIRUN_ERR_ARG;
    if (n == 0) return AIRUN_OK;
    const int threads = 256;
    const long long blocks = (n + threads - 1) / threads;
    if (blocks > 0x7fffffffll) return AIRUN_ERR_ARG;
    if (kind == 2) {
        if (out_dtype != 2) return AIRUN_ERR_UNSUPPORTED;
        fill_random_kernel<int32_t><<<(unsigned)blocks, threads, 0, stream>>>((int32_t*)out, n, key, kind, scale);
    } else if (out_dtype == AIRUN_DT_F32) {
        fill_random_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((float*)out, n, key, kind, scale);
    } else if (out_dtype == AIRUN_DT_BF16) {
        fill_random_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>((__nv_bfloat16*)out, n, key, kind, scale);
    } else {
        return AIRUN_ERR_UNSUPPORTED;
    }
    return airun_launch_status();
}


// x = cap * tanh(x / cap), in place: a soft limit on logits.  The dense Qwen3 head has none (the
// reference applies no cap, crates/airun-core/src/runtime.rs:2632-2651); a head part may ask for one.
__global__ void soft_cap_kernel(float* __restrict__ x, long long n, float cap) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

AIRUN_EXPORT int airun_soft_cap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n < 0 || !(cap > 0.0f)) return AIRUN_ERR_ARG;
    if (n == 0) return AIRUN_OK;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffll) return AIRUN_ERR_ARG;
    airun_launch(soft_cap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, cap);
    return airun_launch_status();
}

// Copies whole cache pages inside the pools of one cache group: for every pair (src, dst) and every
// owner layer, page dst = page src.  pool: [owners][pages][page_words] 16-byte words.  Pairs whose
// ids are outside the pool set the bad-page bit and are skipped.
__global__ void copy_pages_kernel(uint4* __restrict__ pool, long long owner_words, long long page_words,
                                  const int32_t* __restrict__ pairs, int num_pages, int* __restrict__ err) {
    const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
    if (src < 0 || src >= num_pages || dst < 0 || dst >= num_pages) {
        if (threadIdx.x == 0 && err) atomicOr(err, AIRUN_DEV_BAD_PAGE);
        return;
    }
    const uint4* s = pool + (long long)blockIdx.y * owner_words + (long long)src * page_words;
    uint4* d = pool + (long long)blockIdx.y * owner_words + (long long)dst * page_words;
    for (long long i = threadIdx.x; i < page_words; i += blockDim.x) d[i] = s[i];
}

AIRUN_EXPORT int airun_copy_pages(void* pool, int owners, int num_pages, long long page_bytes, const int32_t* pairs,
                                  int n_pairs, int* err, cudaStream_t stream) {
    if (owners <= 0 || num_pages <= 0 || page_bytes <= 0 || page_bytes % 16 != 0 || n_pairs < 0 || ((uintptr_t)pool & 15))
        return AIRUN_ERR_ARG;
    if (n_pairs == 0) return AIRUN_OK;
    if (owners > 65535) return AIRUN_ERR_ARG;
    copy_pages_kernel<<<dim3(n_pairs, owners), 256, 0, stream>>>((uint4*)pool, (long long)num_pages * (page_bytes / 16),
                                                                 page_bytes / 16, pairs, num_pages, err);
    return airun_launch_status();
}
