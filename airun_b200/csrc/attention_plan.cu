// The work lists of the attention kernels, made on the device from the batch's layout.
//
// A step's batch is a flat list of tokens; request r owns tokens cu_tokens[r] .. cu_tokens[r+1]-1
// and holds context_lens[r] tokens after the step.  A request that brings one token goes to the
// decode kernel's row list; a longer portion is cut into tiles of per_tile tokens for the prefill
// kernels, {request, first token row, tokens, keys its last token sees}, the tiles with the most
// keys first (CTAs are handed out in order and the longest must not start last).  The host makes
// the same lists when a step runs kernel by kernel; this kernel exists so that a step whose shape
// is only known on the device (a replayed CUDA graph of a padded batch) needs no host in between.
// The reference sizes its captured attention the same way, from a device-side count
// (crates/airun-cuda/kernels/ops.cu:660-676).
#include "common.cuh"

#define PLAN_THREADS 256
#define PLAN_SORT_MAX 1024

__global__ __launch_bounds__(PLAN_THREADS) void attn_plan_kernel(
    const int* __restrict__ cu_tokens, const int* __restrict__ context_lens, int num_reqs, int per_tile,
    int4* __restrict__ tiles, int max_tiles, int* __restrict__ rows, int max_rows, int* __restrict__ counts,
    int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ int s_off[];                   // [num_reqs + 1] first tile, [num_reqs + 1] first row
    __shared__ int4 s_tiles[PLAN_SORT_MAX];
    int* t_off = s_off;
    int* r_off = s_off + num_reqs + 1;
    for (int r = threadIdx.x; r < num_reqs; r += PLAN_THREADS) {
        const int n = cu_tokens[r + 1] - cu_tokens[r];
        t_off[r] = n > 1 ? (n + per_tile - 1) / per_tile : 0;
        r_off[r] = n == 1 ? 1 : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0, q = 0;
        for (int r = 0; r < num_reqs; ++r) {
            const int a = t_off[r], b = r_off[r];
            t_off[r] = t;
            r_off[r] = q;
            t += a;
            q += b;
        }
        t_off[num_reqs] = t;
        r_off[num_reqs] = q;
    }
    __syncthreads();
    const int nt = t_off[num_reqs], nr = r_off[num_reqs];
    if (nt > max_tiles || nr > max_rows) {           // the lists are too short: run nothing and say so
        if (threadIdx.x == 0) {
            atomicOr(err, AIRUN_DEV_BAD_REQ);
            counts[0] = 0;
            counts[1] = 0;
        }
        return;
    }
    const bool sorted = nt <= PLAN_SORT_MAX;
    for (int r = threadIdx.x; r < num_reqs; r += PLAN_THREADS) {
        const int t0 = cu_tokens[r], n = cu_tokens[r + 1] - t0;
        if (n == 1) {
            rows[r_off[r]] = t0;
        } else if (n > 1) {
            const int c = context_lens[r];
            int4* dst = (sorted ? s_tiles : tiles) + t_off[r];
            for (int s = 0, i = 0; s < n; s += per_tile, ++i) {
                const int k = min(per_tile, n - s);
                dst[i] = make_int4(r, t0 + s, k, c - n + s + k);
            }
        }
    }
    __syncthreads();
    if (sorted) {
        for (int i = threadIdx.x; i < nt; i += PLAN_THREADS) {
            const int4 me = s_tiles[i];
            int rank = 0;
            for (int j = 0; j < nt; ++j) {
                const int w = s_tiles[j].w;
                rank += (w > me.w || (w == me.w && j < i)) ? 1 : 0;
            }
            tiles[rank] = me;
        }
    }
    if (threadIdx.x == 0) {
        counts[0] = nt;
        counts[1] = nr;
    }
}

// tiles: int32 [max_tiles][4]; rows: int32 [max_rows]; counts: int32 [2] = {tiles, rows} written.
AIRUN_EXPORT int airun_attn_plan(const int32_t* cu_tokens, const int32_t* context_lens, int num_reqs, int per_tile,
                                 void* tiles, int max_tiles, int32_t* rows, int max_rows, int32_t* counts,
                                 int* err, cudaStream_t stream) {
    if (!cu_tokens || !context_lens || !tiles || !rows || !counts || !err) return AIRUN_ERR_ARG;
    if (num_reqs <= 0 || per_tile <= 0 || max_tiles <= 0 || max_rows <= 0) return AIRUN_ERR_ARG;
    const size_t smem = 2 * (size_t)(num_reqs + 1) * sizeof(int);
    if (smem > 30 * 1024) return AIRUN_ERR_UNSUPPORTED;
    airun_launch(attn_plan_kernel, dim3(1), dim3(PLAN_THREADS), (int)smem, stream, cu_tokens, context_lens, num_reqs,
                 per_tile, (int4*)tiles, max_tiles, rows, max_rows, counts, err);
    return airun_launch_status();
}
