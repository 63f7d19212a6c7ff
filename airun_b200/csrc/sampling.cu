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

// ------------------------------------------------------------------ the largest logits of a row
// For requests whose sampling chain cuts to the k largest logits anyway (top-k, the reference's default), only those
// candidates have to travel to the host: the chain's earlier stages can only LOWER logits (repetition, presence and
// frequency penalties over the last n tokens), so the k largest after them are among the k + n largest before.
// Row rows[r] of logits -> its n_cand largest values with their ids, the largest first, equal values by ascending
// id (the order the host's top-k uses, so that a tie at the cut falls the same way).  NaN never wins.
// One block per row: every thread keeps the CAND_PER_THREAD largest of its strided share in registers as 64-bit keys
// (orderable value bits, then the inverted id), the 4,096 keys are sorted in shared memory (bitonic), the first
// n_cand leave.  If a thread's share held more than CAND_PER_THREAD of the row's n_cand largest, one of them may be
// missing: the row's flag says so and the host takes the whole row instead (with ids strided over 1,024 threads the
// chance is about one in ten thousand for 105 of 151,936).
#define CAND_THREADS 1024
#define CAND_PER_THREAD 4
#define CAND_MAX 512

__device__ __forceinline__ unsigned long long cand_key(float v, int id) {
    if (v != v) return 0ull;                                     // NaN: no candidate at all
    unsigned u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);              // ascending order of the floats
    return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)id);
}

__global__ __launch_bounds__(CAND_THREADS) void largest_logits_kernel(
    const float* __restrict__ logits, long long ld, int V, const int32_t* __restrict__ rows, int n_cand,
    int32_t* __restrict__ out_ids, float* __restrict__ out_vals, int32_t* __restrict__ out_flags) {
    pdl_trigger();
    extern __shared__ unsigned long long s_keys[];               // CAND_THREADS * CAND_PER_THREAD
    __shared__ int s_flag;
    pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)rows[r] * ld;
    unsigned long long best[CAND_PER_THREAD];                     // descending
#pragma unroll
    for (int i = 0; i < CAND_PER_THREAD; ++i) best[i] = 0ull;
    int seen = 0;
    for (int j = threadIdx.x; j < V; j += CAND_THREADS, ++seen) {
        unsigned long long k = cand_key(row[j], j);
        if (k > best[CAND_PER_THREAD - 1]) {
#pragma unroll
            for (int i = 0; i < CAND_PER_THREAD; ++i) {          // insertion into the sorted few
                if (k > best[i]) { const unsigned long long t = best[i]; best[i] = k; k = t; }
            }
        }
    }
    if (threadIdx.x == 0) s_flag = 0;
#pragma unroll
    for (int i = 0; i < CAND_PER_THREAD; ++i) s_keys[threadIdx.x * CAND_PER_THREAD + i] = best[i];
    __syncthreads();
    constexpr int N = CAND_THREADS * CAND_PER_THREAD;
    for (int k = 2; k <= N; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < N; i += CAND_THREADS) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = s_keys[i], b = s_keys[ixj];
                    const bool descending = (i & k) == 0;
                    if (descending ? a < b : a > b) { s_keys[i] = b; s_keys[ixj] = a; }
                }
            }
            __syncthreads();
        }
    }
    // a thread that kept as many as it can and whose last is among the row's n_cand largest may have dropped one that is too
    const unsigned long long cut = s_keys[n_cand - 1];
    if (seen > CAND_PER_THREAD && best[CAND_PER_THREAD - 1] >= cut && cut != 0ull) s_flag = 1;
    __syncthreads();
    for (int i = threadIdx.x; i < n_cand; i += CAND_THREADS) {
        const unsigned long long k = s_keys[i];
        const int id = (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull));
        const bool real = k != 0ull && id >= 0 && id < V;
        out_ids[(size_t)r * n_cand + i] = real ? id : -1;
        out_vals[(size_t)r * n_cand + i] = real ? row[id] : -INFINITY;
    }
    if (threadIdx.x == 0) out_flags[r] = s_flag;
}

// rows: [n] int32 row indices into logits (on the device); out_ids / out_vals: [n][n_cand]; out_flags: [n].
AIRUN_EXPORT int airun_largest_logits(const float* logits, long long ld, int V, const int32_t* rows, int n, int n_cand,
                                      int32_t* out_ids, float* out_vals, int32_t* out_flags, cudaStream_t stream) {
    if (n < 0 || V <= 0 || ld < V || n_cand < 1 || n_cand > CAND_MAX || !rows || !out_ids || !out_vals || !out_flags) return AIRUN_ERR_ARG;
    if (n == 0) return AIRUN_OK;
    if (n > 65535) return AIRUN_ERR_ARG;
    constexpr int SMEM = CAND_THREADS * CAND_PER_THREAD * 8;
    static unsigned long long configured = 0;                    // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(largest_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(largest_logits_kernel, dim3(n), dim3(CAND_THREADS), SMEM, stream, logits, ld, V, rows, n_cand, out_ids, out_vals, out_flags);
    return airun_launch_status();
}
