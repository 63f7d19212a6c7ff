// Causal attention over cache pages, any sizes, float32 arithmetic.
//
// One block per (token, query head).  Each warp walks every ATTN_WARPS-th
// visible key with a running maximum and sum (online softmax), lanes hold the
// head dimensions; the warps' partial results are merged at the end.  This is
// the shape of the reference's generic streaming kernel
// (crates/airun-cuda/kernels/ops.cu:524-645): head h reads KV head
// h / (n_heads / n_kv_heads); s_j = scale * (q . K_j); key j is visible iff
// j <= pos and, with a window w > 0, pos - j < w (ops.cu:573-576); a row that
// sees nothing yields 0 (ops.cu:626).  The accurate expf is used.
//
// It is the attention of the true 32-bit path (float32 q and pages) and, with
// bfloat16 storage, the plain twin of the tensor-core kernels.  The result for
// a token depends only on its own q, position and the keys it sees, not on the
// batch around it.
#include "common.cuh"

#define ATTN_WARPS 4
#define MAX_PER_LANE 8   // head_dim <= 256

template <typename TQ, typename TKV>
__global__ __launch_bounds__(32 * ATTN_WARPS) void attention_generic_kernel(
    const TQ* __restrict__ q, TQ* __restrict__ out,
    const TKV* __restrict__ pool, const int32_t* __restrict__ block_table, int max_blocks,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ req_of_token,
    int num_reqs, int num_pages, int page_size, int nh, int nkv, int hd,
    float scale, int window, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* s_max = smem;
    float* s_sum = smem + ATTN_WARPS;
    float* s_acc = smem + 2 * ATTN_WARPS;

    const int t = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int req = req_of_token[t];
    TQ* dst = out + ((size_t)t * nh + head) * hd;
    if (req < 0 || pos < 0 || req >= num_reqs) {     // a padding row
        if (req >= num_reqs && threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        for (int d = threadIdx.x; d < hd; d += blockDim.x) dst[d] = from_f32<TQ>(0.0f);
        return;
    }
    const int kvh = head / (nh / nkv);
    const TQ* qv = q + ((size_t)t * nh + head) * hd;
    float qreg[MAX_PER_LANE], acc[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        qreg[i] = d < hd ? to_f32<TQ>(qv[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float run_max = -INFINITY, run_sum = 0.0f;
    const int32_t* bt = block_table + (size_t)req * max_blocks;
    const int begin = window > 0 ? max(0, pos - window + 1) : 0;
    bool bad = false;
    for (int j = begin + warp; j <= pos; j += ATTN_WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const TKV* kj = pool + (((size_t)page * 2 * nkv + kvh) * page_size + (j % page_size)) * hd;
        const TKV* vj = kj + (size_t)nkv * page_size * hd;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < hd) dot = fmaf(qreg[i], to_f32<TKV>(kj[d]), dot);
        }
        dot = warp_sum(dot) * scale;
        const float new_max = fmaxf(run_max, dot);
        const float corr = expf(run_max - new_max);    // exactly 0 on the first key
        const float p = expf(dot - new_max);
        run_sum = run_sum * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < hd) acc[i] = fmaf(p, to_f32<TKV>(vj[d]), acc[i] * corr);
        }
        run_max = new_max;
    }
    if (bad && lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
    if (lane == 0) { s_max[warp] = run_max; s_sum[warp] = run_sum; }
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < hd) s_acc[(size_t)warp * hd + d] = acc[i];
    }
    __syncthreads();
    if (warp != 0) return;
    float gmax = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) gmax = fmaxf(gmax, s_max[w]);
    float weight[ATTN_WARPS], gsum = 0.0f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) {
        weight[w] = s_sum[w] > 0.0f ? expf(s_max[w] - gmax) : 0.0f;
        gsum += s_sum[w] * weight[w];
    }
    const float inv = gsum > 0.0f ? 1.0f / gsum : 0.0f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d >= hd) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < ATTN_WARPS; ++w) v = fmaf(s_acc[(size_t)w * hd + d], weight[w], v);
        dst[d] = from_f32<TQ>(v * inv);
    }
}

AIRUN_EXPORT int airun_attention_generic(
    const void* q, void* out, int q_dtype, const void* pool, int kv_dtype,
    const int32_t* block_table, int max_blocks,
    const int32_t* positions, const int32_t* req_of_token, int T, int num_reqs,
    int num_pages, int page_size, int nh, int nkv, int hd, float scale, int window,
    int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || hd > 32 * MAX_PER_LANE ||
        page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || !err)
        return AIRUN_ERR_ARG;
    if (q_dtype != kv_dtype) return AIRUN_ERR_UNSUPPORTED;
    if (T == 0) return AIRUN_OK;
    if (nh > 65535) return AIRUN_ERR_ARG;
    dim3 grid(T, nh);
    const size_t smem = (size_t)ATTN_WARPS * (2 + hd) * sizeof(float);
#define LAUNCH(TQ, TKV) \
    airun_launch(attention_generic_kernel<TQ, TKV>, dim3(grid), dim3(32 * ATTN_WARPS), smem, stream, (const TQ*)q, (TQ*)out, (const TKV*)pool, \
        block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, nh, nkv, hd, scale, window, err)
    if (q_dtype == AIRUN_DT_F32) LAUNCH(float, float);
    else if (q_dtype == AIRUN_DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}
