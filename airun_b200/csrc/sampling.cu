// Picking the next token on the device: greedy and temperature sampling.
//
// Greedy follows the reference's rule (crates/airun-core/src/sample.rs:639-649,
// device twin crates/airun-cuda/kernels/ops.cu:118-149): the FIRST maximum wins
// (strictly greater replaces), NaN never wins, a row of -inf yields 0.
// Temperature T > 0 draws from p_i ~ exp((l_i - max) / T)
// (crates/airun-core/src/sample.rs:406-418) by inverting the cumulative sum at
// u * total, u in [0,1) supplied per row by the host's seeded generator
// (sample.rs:778-798), so a row's draw does not depend on the batch around it.
// The cumulative sum runs in vocabulary order.  T <= 0 is greedy.
#include "common.cuh"

#define SAMPLE_THREADS 1024

struct BestPair { float v; int i; };

__device__ __forceinline__ BestPair better(BestPair a, BestPair b) {
    // larger value wins; on a tie the smaller index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ BestPair block_best(BestPair p, BestPair* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        BestPair q;
        q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
        q.i = __shfl_xor_sync(0xffffffffu, p.i, o);
        p = better(p, q);
    }
    __syncthreads();
    if (lane == 0) sh[warp] = p;
    __syncthreads();
    if (warp == 0) {
        const int nwarp = (blockDim.x + 31) >> 5;
        BestPair q = lane < nwarp ? sh[lane] : BestPair{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            BestPair r;
            r.v = __shfl_xor_sync(0xffffffffu, q.v, o);
            r.i = __shfl_xor_sync(0xffffffffu, q.i, o);
            q = better(q, r);
        }
        if (lane == 0) sh[32] = q;
    }
    __syncthreads();
    return sh[32];
}

// One block per row.  Each thread owns one contiguous slice of the vocabulary so
// that the per-thread sums, scanned in thread order, form the cumulative sum in
// vocabulary order.
// First stage of the argmax over a large vocabulary: block (c, r) finds the first maximum of its
// slice of row r.  The reference splits its device argmax the same way
// (crates/airun-cuda/kernels/ops.cu:118-149: 128 partial blocks, then one final block).
#define ARGMAX_CHUNKS 64
__global__ __launch_bounds__(256) void argmax_partial_kernel(
    const float* __restrict__ logits, long long ld, int V, BestPair* __restrict__ partial) {
    pdl_trigger();
    pdl_wait();
    __shared__ BestPair sh_best[33];
    const int r = blockIdx.y, c = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = min(V, c * per), hi = min(V, lo + per);
    BestPair best{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v) { best.v = v; best.i = i; }
    }
    best = block_best(best, sh_best);
    if (threadIdx.x == 0) partial[(size_t)r * ARGMAX_CHUNKS + c] = best;
}

__global__ __launch_bounds__(SAMPLE_THREADS) void sample_kernel(
    const float* __restrict__ logits, long long ld, int V,
    const float* __restrict__ temperature, const float* __restrict__ uniform,
    int32_t* __restrict__ out, const BestPair* __restrict__ partial) {
    pdl_trigger();
    pdl_wait();
    __shared__ BestPair sh_best[33];
    __shared__ float sh_sum[SAMPLE_THREADS];
    __shared__ float red[33];
    __shared__ int sh_pick;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;

    BestPair best{-INFINITY, 0x7fffffff};
    if (partial) {
        if (threadIdx.x < ARGMAX_CHUNKS) best = partial[(size_t)r * ARGMAX_CHUNKS + threadIdx.x];
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > best.v) { best.v = v; best.i = i; }     // NaN compares false: never wins
        }
    }
    best = block_best(best, sh_best);
    if (best.i == 0x7fffffff) best.i = 0;               // all -inf or NaN
    const float T = temperature ? temperature[r] : 0.0f;
    if (!(T > 0.0f) || best.v == -INFINITY) {
        if (threadIdx.x == 0) out[r] = best.i;
        return;
    }
    const float inv_t = 1.0f / T;
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
    float s = 0.0f;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += expf((v - best.v) * inv_t);
    }
    sh_sum[threadIdx.x] = s;
    const float total = block_sum(s, red);
    if (threadIdx.x == 0) {
        sh_pick = -1;
        float target = uniform[r] * total;
        // find the slice the target falls in (sequential over <= 1024 sums)
        int tsel = blockDim.x - 1;
        for (int tt = 0; tt < (int)blockDim.x; ++tt) {
            if (target < sh_sum[tt]) { tsel = tt; break; }
            target -= sh_sum[tt];
        }
        const int l2 = min(V, tsel * chunk), h2 = min(V, l2 + chunk);
        int pick = -1, last_ok = -1;
        for (int i = l2; i < h2; ++i) {
            const float v = row[i];
            if (!(v == v)) continue;
            const float p = expf((v - best.v) * inv_t);
            if (p > 0.0f) last_ok = i;
            target -= p;
            if (target < 0.0f && p > 0.0f) { pick = i; break; }
        }
        if (pick < 0) pick = last_ok >= 0 ? last_ok : best.i;   // rounding left the target beyond the slice
        sh_pick = pick;
        out[r] = pick;
    }
}

// scratch: rows * 64 * 8 bytes for the first stage of the argmax, or null (one block per row then
// walks the whole row, which is fine for small vocabularies).
AIRUN_EXPORT int airun_sample(const float* logits, long long ld, int rows, int V,
                              const float* temperature, const float* uniform,
                              int32_t* out, void* scratch, cudaStream_t stream) {
    if (rows < 0 || V <= 0 || ld < V) return AIRUN_ERR_ARG;
    if (temperature && !uniform) return AIRUN_ERR_ARG;
    if (rows == 0) return AIRUN_OK;
    if (rows > 65535) return AIRUN_ERR_ARG;
    BestPair* partial = nullptr;
    if (scratch && V >= 8192) {
        partial = (BestPair*)scratch;
        airun_launch(argmax_partial_kernel, dim3(dim3(ARGMAX_CHUNKS, rows)), dim3(256), 0, stream, logits, ld, V, partial);
    }
    airun_launch(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature, uniform, out, partial);
    return airun_launch_status();
}
