// Everything between the q/k/v projection and attention, in one launch:
// per-head RMSNorm of q and k, rotary position encoding of both, q out in the
// attention kernel's input type, and k and v into their cache pages.
//
// Formulas as the reference computes them
// (crates/airun-cuda/kernels/ops.cu:422-501, crates/airun-cuda/kernels/airun.cuh:147-163):
//   per head row h of head_dim values: h = h * rsqrt(sum(h^2)/head_dim + eps) * w
//   (one weight vector shared by all heads, same eps as the layer norms, before
//   the rotation; v is not normed);
//   rotation: pair i couples dims lo and hi, theta = rpos * inv_freq[i],
//   x'_lo = x_lo cos - x_hi sin,  x'_hi = x_lo sin + x_hi cos; dims >= r are left alone; the accurate
//   sincosf is used on purpose (angles reach thousands of radians).  NeoX pairing: lo = i, hi = i + r/2;
//   interleaved (GPT-J) pairing: lo = 2i, hi = 2i + 1 (ops.cu:154-157, :176-179 keeps both as a kernel
//   parameter).  rpos is the token's cache position unless the caller gives rotation positions of
//   their own (the reference's shift / mpos indirection, airun.cuh:121-143).
// inv_freq[i] = theta_base^(-2i/r) is computed on the host in double precision
// and rounded once to float32, so the device and a plain implementation multiply
// the position by the very same constant.
//
// Cache layout of one layer: [num_pages][2 (K,V)][n_kv_heads][page_size][head_dim];
// the token at position p of request r lives in page block_table[r][p / page_size],
// row p % page_size.  A block-table entry outside [0, num_pages) sets an error
// bit and the store is skipped; nothing traps.
#include "common.cuh"

#define ROPE_NONE 0
#define ROPE_NEOX 1
#define ROPE_INTERLEAVED 2
#define MAX_PER_LANE 8   // head_dim <= 256

// DPL: values of a head per lane, ceil(head_dim / 32) rounded up to 1, 2, 4 or 8.
template <typename TQ, typename TKV, int DPL>
__global__ __launch_bounds__(256) void qkv_post_kernel(
    const float* __restrict__ qkv, long long ld_qkv,
    TQ* __restrict__ q_out,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token,
    int rope_kind, int rotary_dim, const float* __restrict__ inv_freq, const int32_t* __restrict__ rope_positions,
    TKV* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks,
    int num_reqs, int num_pages, int page_size, int do_store, int kv_from_qkv,
    int nh, int nkv, int hd, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarp = blockDim.x >> 5;
    float* row = smem + (size_t)warp * hd;
    float* cs = smem + (size_t)nwarp * hd;          // cos[half], sin[half] of this token, shared by its heads
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int req = req_of_token[t];
    const int total_heads = kv_from_qkv ? nh + 2 * nkv : nh;
    const int half = rotary_dim / 2;
    if (rope_kind != ROPE_NONE) {
        const int rpos = rope_positions ? rope_positions[t] : pos;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float s, c;
            sincosf((float)rpos * inv_freq[i], &s, &c);
            cs[i] = c;
            cs[half + i] = s;
        }
        __syncthreads();
    }

    for (int h = blockIdx.y * nwarp + warp; h < total_heads; h += gridDim.y * nwarp) {
        const bool is_q = h < nh;
        const bool is_k = !is_q && h < nh + nkv;
        const float* src = qkv + (size_t)t * ld_qkv + (size_t)h * hd;
        float x[DPL];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + i * 32;
            x[i] = d < hd ? src[d] : 0.0f;
            ss = fmaf(x[i], x[i], ss);
        }
        const float* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
        if (w) {
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)hd + eps);
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + i * 32;
                if (d < hd) x[i] = x[i] * inv * w[d];
            }
        }
        if (rope_kind != ROPE_NONE && (is_q || is_k)) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + i * 32;
                if (d < hd) row[d] = x[i];
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + i * 32;
                if (d < rotary_dim && d < hd) {
                    const bool neox = rope_kind == ROPE_NEOX;
                    const bool first = neox ? d < half : (d & 1) == 0;
                    const int pair = neox ? (first ? d : d - half) : d >> 1;
                    const int other = neox ? (first ? d + half : d - half) : d ^ 1;
                    const float c = cs[pair], s = cs[half + pair];
                    const float x0 = first ? row[d] : row[other];
                    const float x1 = first ? row[other] : row[d];
                    x[i] = first ? x0 * c - x1 * s : x0 * s + x1 * c;
                }
            }
        }
        if (is_q) {
            TQ* dst = q_out + ((size_t)t * nh + h) * hd;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + i * 32;
                if (d < hd) dst[d] = from_f32<TQ>(x[i]);
            }
        } else if (do_store && req >= 0 && pos >= 0) {
            if (req >= num_reqs) {
                if (lane == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
                continue;
            }
            const int blk = pos / page_size;
            const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
            if (page < 0 || page >= num_pages) {
                if (lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
                continue;
            }
            const int kvh = is_k ? h - nh : h - nh - nkv;
            TKV* dst = pool + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size
                               + (pos % page_size)) * hd;
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + i * 32;
                if (d < hd) dst[d] = from_f32<TKV>(x[i]);
            }
        }
    }
}

// The same for head_dim 128 with a full-width NeoX rotation (the benchmark's shape): a lane holds four
// neighbouring values, loads them as one float4 and stores them as one 8- or 16-byte word; the
// rotation partner of dims 4l .. 4l+3 sits in lane l ^ 16, so it comes by shuffle and not through
// shared memory.  Same arithmetic, in the same order, as the kernel above.
template <typename TQ, typename TKV>
__global__ __launch_bounds__(256) void qkv_post_hd128_kernel(
    const float* __restrict__ qkv, long long ld_qkv,
    TQ* __restrict__ q_out,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token,
    const float* __restrict__ inv_freq,
    TKV* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks,
    int num_reqs, int num_pages, int page_size, int do_store, int kv_from_qkv,
    int nh, int nkv, int* __restrict__ err) {
    pdl_trigger();
    constexpr int HD = 128, HALF = 64;
    __shared__ float cs[2 * HALF];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarp = blockDim.x >> 5;
    const int t = blockIdx.x;
    // positions and requests of the batch were copied to the device before the step began: the
    // angles are worked out while the product in front of this kernel is still finishing
    const int pos = positions[t];
    const int req = req_of_token[t];
    const int total_heads = kv_from_qkv ? nh + 2 * nkv : nh;
    for (int i = threadIdx.x; i < HALF; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[HALF + i] = s;
    }
    __syncthreads();
    pdl_wait();
    const bool first = lane < 16;
    const int pair = 4 * (lane & 15);
    const float4 c4 = *reinterpret_cast<const float4*>(cs + pair);
    const float4 s4 = *reinterpret_cast<const float4*>(cs + HALF + pair);

    for (int h = blockIdx.y * nwarp + warp; h < total_heads; h += gridDim.y * nwarp) {
        const bool is_q = h < nh;
        const bool is_k = !is_q && h < nh + nkv;
        float4 v = *reinterpret_cast<const float4*>(qkv + (size_t)t * ld_qkv + (size_t)h * HD + 4 * lane);
        const float* w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
        if (w) {
            float ss = fmaf(v.x, v.x, 0.0f);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)HD + eps);
            const float4 g = *reinterpret_cast<const float4*>(w + 4 * lane);
            v.x = v.x * inv * g.x; v.y = v.y * inv * g.y; v.z = v.z * inv * g.z; v.w = v.w * inv * g.w;
            float4 o;
            o.x = __shfl_xor_sync(0xffffffffu, v.x, 16);
            o.y = __shfl_xor_sync(0xffffffffu, v.y, 16);
            o.z = __shfl_xor_sync(0xffffffffu, v.z, 16);
            o.w = __shfl_xor_sync(0xffffffffu, v.w, 16);
            // first half: x_i cos - x_{i+64} sin; second half: x_i sin + x_{i+64} cos (x_i is the partner's)
            if (first) {
                v.x = v.x * c4.x - o.x * s4.x; v.y = v.y * c4.y - o.y * s4.y;
                v.z = v.z * c4.z - o.z * s4.z; v.w = v.w * c4.w - o.w * s4.w;
            } else {
                v.x = o.x * s4.x + v.x * c4.x; v.y = o.y * s4.y + v.y * c4.y;
                v.z = o.z * s4.z + v.z * c4.z; v.w = o.w * s4.w + v.w * c4.w;
            }
        }
        if (is_q) {
            TQ* dst = q_out + ((size_t)t * nh + h) * HD + 4 * lane;
            if (sizeof(TQ) == 4) {
                *reinterpret_cast<float4*>(dst) = v;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = pk;
            }
        } else if (do_store && req >= 0 && pos >= 0) {
            if (req >= num_reqs) {
                if (lane == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
                continue;
            }
            const int blk = pos / page_size;
            const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
            if (page < 0 || page >= num_pages) {
                if (lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
                continue;
            }
            const int kvh = is_k ? h - nh : h - nh - nkv;
            TKV* dst = pool + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size
                               + (pos % page_size)) * HD + 4 * lane;
            if (sizeof(TKV) == 4) {
                *reinterpret_cast<float4*>(dst) = v;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = pk;
            }
        }
    }
}

// kv_from_qkv = 0: the row holds q only (the layer reads another layer's cache).
AIRUN_EXPORT int airun_qkv_post(
    const float* qkv, long long ld_qkv, void* q_out, int q_dtype,
    const float* q_norm_w, const float* k_norm_w, float eps,
    const int32_t* positions, const int32_t* req_of_token, int T,
    int rope_kind, int rotary_dim, const float* inv_freq, const int32_t* rope_positions,
    void* pool, int kv_dtype, const int32_t* block_table, int max_blocks, int num_reqs,
    int num_pages, int page_size, int do_store, int kv_from_qkv,
    int nh, int nkv, int hd, int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || hd > 32 * MAX_PER_LANE) return AIRUN_ERR_ARG;
    if (rope_kind != ROPE_NONE && rope_kind != ROPE_NEOX && rope_kind != ROPE_INTERLEAVED) return AIRUN_ERR_UNSUPPORTED;
    if (rope_kind != ROPE_NONE && (rotary_dim <= 0 || rotary_dim > hd || rotary_dim % 2 != 0 || !inv_freq))
        return AIRUN_ERR_ARG;
    if (do_store && (page_size <= 0 || num_pages <= 0 || !pool || !block_table || !err)) return AIRUN_ERR_ARG;
    if (q_dtype != kv_dtype) return AIRUN_ERR_UNSUPPORTED;
    if (T == 0) return AIRUN_OK;
    const int heads = kv_from_qkv ? nh + 2 * nkv : nh;
    // few tokens: one head per warp and many small blocks, so a decode step is not a handful of
    // blocks each walking all heads; many tokens: eight heads per block
    int warps = T <= 64 ? (heads < 2 ? heads : 2) : (heads < 8 ? heads : 8);
    const int blocks_y = T <= 64 ? (heads + warps - 1) / warps : 1;
    const size_t smem = ((size_t)warps * hd + (rope_kind != ROPE_NONE ? rotary_dim : 0)) * sizeof(float);
    // head_dim 128, both norms, the rotation over the whole head, 16-byte aligned rows: the vector kernel
    const bool vec128 = hd == 128 && rope_kind == ROPE_NEOX && rotary_dim == 128 && !rope_positions && q_norm_w && k_norm_w &&
                        ld_qkv % 4 == 0 && (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pool |
                                             (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 15) == 0;
    if (vec128) {
#define LAUNCH128(TQ, TKV) \
    airun_launch(qkv_post_hd128_kernel<TQ, TKV>, dim3(T, blocks_y), dim3(warps * 32), 0, stream, qkv, ld_qkv, (TQ*)q_out, \
        q_norm_w, k_norm_w, eps, positions, req_of_token, inv_freq, (TKV*)pool, block_table, max_blocks, num_reqs, \
        num_pages, page_size, do_store, kv_from_qkv, nh, nkv, err)
        if (q_dtype == AIRUN_DT_F32) LAUNCH128(float, float);
        else if (q_dtype == AIRUN_DT_BF16) LAUNCH128(__nv_bfloat16, __nv_bfloat16);
        else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH128
        return airun_launch_status();
    }
#define LAUNCH(TQ, TKV, DPL) \
    airun_launch(qkv_post_kernel<TQ, TKV, DPL>, dim3(T, blocks_y), dim3(warps * 32), smem, stream, qkv, ld_qkv, (TQ*)q_out, q_norm_w, k_norm_w, eps, \
        positions, req_of_token, rope_kind, rotary_dim, inv_freq, rope_positions, (TKV*)pool, block_table, max_blocks, num_reqs, \
        num_pages, page_size, do_store, kv_from_qkv, nh, nkv, hd, err)
#define LAUNCH_DPL(TQ, TKV) \
    do { if (hd <= 32) LAUNCH(TQ, TKV, 1); else if (hd <= 64) LAUNCH(TQ, TKV, 2); \
         else if (hd <= 128) LAUNCH(TQ, TKV, 4); else LAUNCH(TQ, TKV, 8); } while (0)
    if (q_dtype == AIRUN_DT_F32) LAUNCH_DPL(float, float);
    else if (q_dtype == AIRUN_DT_BF16) LAUNCH_DPL(__nv_bfloat16, __nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH_DPL
#undef LAUNCH
    return airun_launch_status();
}
