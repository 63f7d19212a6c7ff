// bfloat16 matrix product on the 5th-generation tensor cores:
//   out[M][N] = x[M][K] * W[N][K]^T, float32 accumulation in tensor memory.
//
// One CTA computes one 128 x BN tile D = A * B^T of two K-major operands
// ("rows of K contiguous values"), over one slice of K:
//   warp 0   : one thread issues TMA loads (cp.async.bulk.tensor, 128-byte
//              swizzle) of A and B blocks of 64 k-values into a ring of stages;
//   warp 1   : allocates tensor memory; one thread issues tcgen05.mma
//              (M=128, N=BN, K=16, four per block) and commits to mbarriers;
//   warps 2-5: read the accumulator with tcgen05.ld, apply the epilogue, store.
// Which operand is A decides the mode:
//   normal (prompt portions): A = activations (128 tokens), B = weights (BN rows);
//   swapped (few tokens)    : A = weights (128 rows), B = activations (BN >= tokens),
//                             so a decode step streams each weight once and wastes
//                             no tensor-core rows on padding.
// With ksplit > 1 the CTAs of one tile each write a float32 partial tile to a
// scratch buffer; the last one to finish (a counter per tile) adds the partials
// in slice order and runs the epilogue, so the result does not depend on timing.
// Epilogues: float32 store, bfloat16 store, SwiGLU (columns alternate between
// blocks of 16 gate and 16 up values; out = silu(g) * u as bfloat16).
//
// Every wait on an mbarrier is bounded: when it runs out the kernel sets an
// error bit, skips the rest of its work, frees its tensor memory and returns.
// From 17 tokens on the K slices of a tile run as one thread-block cluster and add up through distributed
// shared memory (see cluster_reduce); no TMA load uses multicast.
//
// The reference's counterparts are its wmma prefill GEMM and its half-precision
// matvec kernels (crates/airun-cuda/kernels/matmul.cu:518-636, :1498-1563); its
// fused gate/up/SwiGLU decode kernel is matmul.cu:150-214.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <string>
#include <cstring>

#define BM 128
#define BK 64
#define EPI_F32 0
#define EPI_BF16 1
#define EPI_SWIGLU 2
#define EPI_RESID 3
#define GEMM_THREADS 192
#define WAIT_LIMIT_NS 2000000000ull

// AIRUN_FOLD_NORM=1 builds the variant with the RMSNorm folded into the products (token scales on the
// input, the residual + norm epilogue).  The plain build leaves that code out: the engine does not use it
// unless asked to, and the leaner kernels run a decode step 0.5 to 1 % faster.
#ifndef AIRUN_FOLD_NORM
#define AIRUN_FOLD_NORM 0
#endif

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait; false when about two seconds have passed without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// ---- thread-block clusters: the rank of this CTA, a barrier over all threads of all CTAs, and loads
// from a peer's shared memory
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) with the
// 128-byte swizzle: 8-row groups 1024 bytes apart, version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

struct GemmParams {
    int a_rows, b_rows, K;        // extents of the A and B operands
    int k_blocks_per_split;       // blocks of 64 k-values per slice
    int ksplit;
    void* out;
    long long ldc;                // output row stride in elements
    float* scratch;               // [tiles][ksplit][BN][128] partial tiles
    int* counters;                // [tiles], zero between launches
    int* err;
    // RMSNorm folded into two products.  The product that ENDS a sub-layer (EPI_RESID) adds its result to
    // the residual stream x, writes h' = bfloat16(x * w_norm) for the next product and the sums of x^2
    // per token in parts; the product that STARTS the next sub-layer reads h' and multiplies each
    // token's results by rsqrt(sum of the parts / n + eps): (s * h') W^T = s * (h' W^T).
    const float* ssq_in;          // [ssq_parts][ssq_ld] or null: token scales of the input
    int ssq_parts, ssq_ld;
    float eps_in, inv_n_in;       // 1 / (size of the normed row)
    float* resid;                 // [tokens][ld_resid] float32 residual stream (EPI_RESID)
    long long ld_resid;
    const float* norm_w;          // [weight rows] weight of the norm that follows (EPI_RESID)
    float* ssq_out;               // [parts][ssq_out_ld] (EPI_RESID)
    int ssq_out_ld;
    int cluster_reduce;           // the ksplit CTAs of a tile are one cluster and add their slices through
                                  // distributed shared memory instead of the scratch
};

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;   // + alignment slack
};

// Epilogue for 16 consecutive accumulator columns [c0, c0+16) of this thread's row.
template <int EPI, bool SWAP>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const float* v, int a_row, int b0, int c0) {
    // normal: out[a_row][b0 + c0 + i];  swapped: out[b0 + c0 + i][a_row]
    if (!SWAP) {
        if (a_row >= p.a_rows) return;
        const int n0 = b0 + c0;
        if (EPI == EPI_F32) {
            float* o = (float*)p.out + (size_t)a_row * p.ldc + n0;
            if (n0 + 16 <= p.b_rows && (((size_t)o) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) if (n0 + i < p.b_rows) o[i] = v[i];
            }
        } else {
            __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)a_row * p.ldc + n0;
            if (n0 + 16 <= p.b_rows && (((size_t)o) & 15) == 0) {
                uint32_t w[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                    w[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(o + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) if (n0 + i < p.b_rows) o[i] = __float2bfloat16_rn(v[i]);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int tok = b0 + c0 + i;
            if (tok < p.b_rows && a_row < p.a_rows) {
                if (EPI == EPI_F32) ((float*)p.out)[(size_t)tok * p.ldc + a_row] = v[i];
                else ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldc + a_row] = __float2bfloat16_rn(v[i]);
            }
        }
    }
}

// SwiGLU, normal mode: g = columns [c0, c0+16), u = columns [c0+16, c0+32) of this row.
__device__ __forceinline__ void store_swiglu_normal(const GemmParams& p, const float* g, const float* u,
                                                    int a_row, int b0, int c0) {
    if (a_row >= p.a_rows) return;
    const int n_out = (b0 + c0) / 2;
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)a_row * p.ldc + n_out;
    if (b0 + c0 + 32 <= p.b_rows && (((size_t)o) & 15) == 0) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul(g[2 * i], u[2 * i]), silu_mul(g[2 * i + 1], u[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(o + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        return;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (b0 + c0 + 16 + i < p.b_rows) o[i] = __float2bfloat16_rn(silu_mul(g[i], u[i]));
}

// SwiGLU, swapped mode: this lane's row is a gate row when (a_row / 16) is even, and lane + 16
// holds the matching up row.  v: 16 columns (tokens).
__device__ __forceinline__ void store_swiglu_swapped(const GemmParams& p, const float* v, int a_row, int b0, int c0) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float up = __shfl_down_sync(0xffffffffu, v[i], 16);
        const int tok = b0 + c0 + i;
        if (lane < 16 && tok < p.b_rows && a_row < p.a_rows) {
            const int n_out = (a_row / 32) * 16 + (a_row % 32);
            ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldc + n_out] = __float2bfloat16_rn(silu_mul(v[i], up));
        }
    }
}

// rsqrt(sum of the parts / n + eps) of one token
__device__ __forceinline__ float token_scale(const GemmParams& p, int tok) {
    float s = 0.0f;
    for (int i = 0; i < p.ssq_parts; ++i) s += __ldcg(p.ssq_in + (size_t)i * p.ssq_ld + tok);
    return rsqrtf(s * p.inv_n_in + p.eps_in);
}

// EPI_RESID, normal mode: this thread's token row, 16 weight rows from n0.  Returns the sum of squares.
__device__ __forceinline__ float store_resid_normal(const GemmParams& p, const float* v, int a_row, int n0) {
    if (a_row >= p.a_rows) return 0.0f;
    float* xr = p.resid + (size_t)a_row * p.ld_resid + n0;
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)a_row * p.ldc + n0;
    float sq = 0.0f;
    if (n0 + 16 <= p.b_rows && ((((size_t)xr) | ((size_t)(p.norm_w + n0))) & 15) == 0 && (((size_t)o) & 15) == 0) {
        uint32_t w[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float4 x4 = *reinterpret_cast<float4*>(xr + 4 * q);
            const float4 g = *reinterpret_cast<const float4*>(p.norm_w + n0 + 4 * q);
            x4.x += v[4 * q]; x4.y += v[4 * q + 1]; x4.z += v[4 * q + 2]; x4.w += v[4 * q + 3];
            *reinterpret_cast<float4*>(xr + 4 * q) = x4;
            sq = fmaf(x4.x, x4.x, fmaf(x4.y, x4.y, fmaf(x4.z, x4.z, fmaf(x4.w, x4.w, sq))));
            __nv_bfloat162 lo = __floats2bfloat162_rn(x4.x * g.x, x4.y * g.y), hi = __floats2bfloat162_rn(x4.z * g.z, x4.w * g.w);
            w[2 * q] = *reinterpret_cast<uint32_t*>(&lo);
            w[2 * q + 1] = *reinterpret_cast<uint32_t*>(&hi);
        }
        *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(o + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (n0 + i < p.b_rows) {
                const float xn = xr[i] + v[i];
                xr[i] = xn;
                sq = fmaf(xn, xn, sq);
                o[i] = __float2bfloat16_rn(xn * p.norm_w[n0 + i]);
            }
        }
    }
    return sq;
}

// EPI_RESID, swapped mode: this lane's weight row a_row, 16 tokens from b0 + c0.  The sums of squares
// over the warp's 32 weight rows go to ssq_warp[c0 + token] in shared memory; the caller adds the four
// warps of the tile and stores one part per tile and token.
__device__ __forceinline__ void store_resid_swapped(const GemmParams& p, const float* v, int a_row, int b0, int c0,
                                                    float* ssq_warp) {
    const int lane = threadIdx.x & 31;
    const bool row_ok = a_row < p.a_rows;
    const float g = row_ok ? p.norm_w[a_row] : 0.0f;
    // the residual's values of all 16 tokens first: sixteen loads in flight, not sixteen round trips in turn
    float xv[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int tok = b0 + c0 + i;
        xv[i] = (row_ok && tok < p.b_rows) ? __ldcg(p.resid + (size_t)tok * p.ld_resid + a_row) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int tok = b0 + c0 + i;
        float sq = 0.0f;
        if (row_ok && tok < p.b_rows) {
            const float xn = xv[i] + v[i];
            p.resid[(size_t)tok * p.ld_resid + a_row] = xn;
            sq = xn * xn;
            ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldc + a_row] = __float2bfloat16_rn(xn * g);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) ssq_warp[c0 + i] = sq;
    }
}

// CLUSTER: the build that can add up the slices of a tile through distributed shared memory.  It is a
// build of its own because the extra code made the plain one slower inside a decode step (by 2 % at
// batch 8) although nothing of it ran there.
template <int BN, int STAGES, int EPI, bool SWAP, bool CLUSTER>
__global__ __launch_bounds__(GEMM_THREADS, 1) void gemm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + L::BAR_OFFSET);
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    __shared__ int s_ticket;
    __shared__ int s_abort;

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a0 = blockIdx.x * BM;            // first A row of the tile
    const int b0 = blockIdx.y * BN;            // first B row of the tile
    const int split = blockIdx.z;
    const int kb_total = (p.K + BK - 1) / BK;
    const int kb_begin = split * p.k_blocks_per_split;
    int kb_end = kb_begin + p.k_blocks_per_split;
    if (kb_end > kb_total) kb_end = kb_total;
    const int n_kb = kb_end > kb_begin ? kb_end - kb_begin : 0;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), accum = smem_u32(bars + 2 * STAGES);
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // The weight operand (A when swapped, B otherwise) is written by no kernel, so the first stages'
    // weight blocks are requested before waiting for the kernel before this one: the weights keep
    // streaming across the boundary between two kernels.
    const int n_pre = n_kb < STAGES ? n_kb : STAGES;
    if (warp == 0 && lane == 0) {
        for (int i = 0; i < n_pre; ++i) {
            mbar_expect_tx(full0 + 8 * i, L::STAGE_BYTES);
            const uint32_t sa = smem_u32(smem + i * L::STAGE_BYTES);
            const int k = (kb_begin + i) * BK;
            if (SWAP) tma_load_2d(sa, &map_a, full0 + 8 * i, k, a0);
            else tma_load_2d(sa + L::A_BYTES, &map_b, full0 + 8 * i, k, b0);
        }
    }
    // from here on the results of earlier kernels are read and their buffers written
    pdl_wait();

    // what the epilogue warps (2..5) share between their two phases
    const int quad = warp & 3;
    const int a_row = a0 + quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    __shared__ float s_scale[SWAP ? BN : 1];
    __shared__ float s_ssq[4][(SWAP && AIRUN_FOLD_NORM) ? BN : 1];       // per epilogue warp: sums of squares per token
    float row_scale = 1.0f;
    bool ok = true;
    const bool direct = p.ksplit == 1;
    const bool clustered = CLUSTER && !direct;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    // Sums the slices of the tile (or takes the accumulator as it is), applies the epilogue and stores.
    // rank < 0: all columns, slices from tensor memory (one slice) or from the scratch; rank >= 0: the
    // chunks of columns that fall to this CTA of the cluster, slices from the peers' shared memory.
    auto finish_tile = [&](int rank) {
        float ssq_acc = 0.0f;
        const float* all = (direct || rank >= 0) ? nullptr : p.scratch + (size_t)tile * p.ksplit * (BN * BM);
        const uint32_t mine = smem_u32(smem);
        constexpr int STEP = (EPI == EPI_SWIGLU && !SWAP) ? 32 : 16;
        for (int c = 0; c < BN; c += STEP) {
            if (rank >= 0 && (c / STEP) % p.ksplit != rank) continue;
            float v[16], u[16];
            if (direct) {
                if (n_kb > 0) {
                    tmem_ld16(lane_addr + c, v);
                    if (STEP == 32) tmem_ld16(lane_addr + c + 16, u);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) { v[i] = 0.0f; u[i] = 0.0f; }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) { v[i] = 0.0f; u[i] = 0.0f; }
                // slices are added in order; loads of four slices are in flight at a time
                for (int s0 = 0; s0 < p.ksplit; s0 += 4) {
                    float t[4][STEP];
#pragma unroll
                    for (int d = 0; d < 4; ++d) {
                        if (CLUSTER && rank >= 0) {
                            const uint32_t peer = s0 + d < p.ksplit ? map_to_cta(mine, (uint32_t)(s0 + d)) : 0u;
#pragma unroll
                            for (int i = 0; i < STEP; ++i)
                                t[d][i] = (s0 + d < p.ksplit)
                                              ? ld_cluster_f32(peer + 4u * (uint32_t)((c + i) * BM + quad * 32 + lane)) : 0.0f;
                        } else {
                            const float* ps = all + (size_t)(s0 + d) * (BN * BM) + quad * 32 + lane;
#pragma unroll
                            for (int i = 0; i < STEP; ++i)
                                t[d][i] = (s0 + d < p.ksplit) ? __ldcg(ps + (size_t)(c + i) * BM) : 0.0f;
                        }
                    }
#pragma unroll
                    for (int d = 0; d < 4; ++d) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            v[i] += t[d][i];
                            if (STEP == 32) u[i] += t[d][(STEP == 32 ? 16 : 0) + i];
                        }
                    }
                }
            }
            if (AIRUN_FOLD_NORM && p.ssq_in) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float f = SWAP ? s_scale[c + i] : row_scale;
                    v[i] *= f;
                    if (STEP == 32) u[i] *= f;
                }
            }
            if (EPI == EPI_SWIGLU) {
                if (SWAP) store_swiglu_swapped(p, v, a_row, b0, c);
                else store_swiglu_normal(p, v, u, a_row, b0, c);
            } else if (EPI == EPI_RESID) {
                if (SWAP) store_resid_swapped(p, v, a_row, b0, c, s_ssq[quad]);
                else ssq_acc += store_resid_normal(p, v, a_row, b0 + c);
            } else {
                store_chunk<EPI, SWAP>(p, v, a_row, b0, c);
            }
        }
        if (EPI == EPI_RESID && !SWAP && a_row < p.a_rows) p.ssq_out[(size_t)blockIdx.y * p.ssq_out_ld + a_row] = ssq_acc;
        if (AIRUN_FOLD_NORM && EPI == EPI_RESID && SWAP) {
            // one part per tile of 128 weight rows: the four warps' sums, for the tokens this block has stored
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int j = threadIdx.x - 64; j < BN; j += 128) {
                const bool mine = rank < 0 || (j / STEP) % p.ksplit == rank;
                if (mine && b0 + j < p.b_rows)
                    p.ssq_out[(size_t)blockIdx.x * p.ssq_out_ld + b0 + j] = s_ssq[0][j] + s_ssq[1][j] + s_ssq[2][j] + s_ssq[3][j];
            }
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                if (i < n_pre) {                 // the weight half of this stage is already on its way
                    if (SWAP) tma_load_2d(sa + L::A_BYTES, &map_b, full0 + 8 * s, k, b0);
                    else tma_load_2d(sa, &map_a, full0 + 8 * s, k, a0);
                    continue;
                }
                const uint32_t phase = (i / STAGES) & 1;
                if (!mbar_wait(empty0 + 8 * s, phase ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); s_abort = 1; break; }
                mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                tma_load_2d(sa, &map_a, full0 + 8 * s, k, a0);
                tma_load_2d(sa + L::A_BYTES, &map_b, full0 + 8 * s, k, b0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t phase = (i / STAGES) & 1;
                if (!mbar_wait(full0 + 8 * s, phase)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); s_abort = 1; ok = false; break; }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + L::A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_bf16(tmem_base, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * s);      // the stage is free once these MMAs have read it
            }
            umma_commit(accum);                   // arrives when every MMA issued so far is complete
        }
    } else {
        // epilogue warps 2..5: warp w may touch the 32 TMEM lanes of quadrant w % 4
        // token scales of a normed input, while the MMAs run
        if (AIRUN_FOLD_NORM && p.ssq_in) {
            if (SWAP) {
                // the parts of 16 tokens at a time: every thread takes every 128th part, the warps add theirs up
                // and the four warp sums meet in shared memory (one round trip to L2 for all parts)
                const int t = threadIdx.x - 64;
                for (int j0 = 0; j0 < BN; j0 += 16) {
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
                    for (int part = t; part < p.ssq_parts; part += 128) {
                        const float* src = p.ssq_in + (size_t)part * p.ssq_ld + b0 + j0;
#pragma unroll
                        for (int i = 0; i < 16; ++i) acc[i] += (b0 + j0 + i < p.b_rows) ? __ldcg(src + i) : 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float a = acc[i];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                        if (lane == 0) s_ssq[quad][j0 + i] = a;
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int j = t; j < BN; j += 128)
                    s_scale[j] = b0 + j < p.b_rows
                        ? rsqrtf((s_ssq[0][j] + s_ssq[1][j] + s_ssq[2][j] + s_ssq[3][j]) * p.inv_n_in + p.eps_in) : 0.0f;
                asm volatile("bar.sync 1, 128;" ::: "memory");
            } else if (a_row < p.a_rows) {
                row_scale = token_scale(p, a_row);
            }
        }
        ok = n_kb == 0 ? true : mbar_wait(accum, 0);
        if (!ok) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); }
        tc_fence_after();
        bool last = true;
        if (!direct) {
            // the partial tile goes to this CTA's own shared memory (the stages are free: every MMA is
            // complete) when the slices of a tile form a cluster, else to the scratch in global memory
            float* part = clustered ? reinterpret_cast<float*>(smem)
                                    : p.scratch + ((size_t)tile * p.ksplit + split) * (BN * BM);
            if (ok) {
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    if (n_kb > 0) tmem_ld16(lane_addr + c, v);
                    else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) part[(size_t)(c + i) * BM + quad * 32 + lane] = v[i];
                }
            }
            if (clustered) {
                last = false;                     // the sums are formed after the cluster's barrier, below
            } else {
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) s_ticket = atomicAdd(p.counters + tile, 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                last = s_ticket == p.ksplit - 1;
                if (last) {
                    __threadfence();
                    if (threadIdx.x == 64) p.counters[tile] = 0;       // ready for the next launch
                }
            }
        }
        if (ok && last) finish_tile(-1);
    }
    if (CLUSTER && clustered) {
        // Every CTA of the cluster has its partial tile in shared memory.  CTA r takes every ksplit-th
        // chunk of 16 (or 32) columns, adds the slices in order through distributed shared memory
        // and stores the result; nobody leaves while a peer may still read its memory.
        __syncwarp();
        cluster_sync_all();
        if (warp >= 2) finish_tile((int)cluster_rank());
        __syncwarp();
        cluster_sync_all();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ persistent variant (prompt portions)
// One CTA per SM walks the tiles of the product (m fastest, so CTAs running side by side share a
// weight tile).  The stage ring runs on across tiles, and the accumulator is double-buffered in
// tensor memory (2 x 256 columns): while the epilogue warps drain tile i, the MMA thread is already
// filling tile i + 1.  Normal mode, BN = 256, no K slices.
#define PBN 256
#define PSTAGES 4
template <int EPI>
__global__ __launch_bounds__(GEMM_THREADS, 1) void gemm_tcgen05_persistent_kernel(
    const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p,
    int m_tiles, int n_tiles) {
    pdl_trigger();
    using L = SmemLayout<PBN, PSTAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + L::BAR_OFFSET);          // full[S], empty[S], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_slot_p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_total = (p.K + BK - 1) / BK;
    const int total_tiles = m_tiles * n_tiles;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + PSTAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * PSTAGES), acce0 = smem_u32(bars + 2 * PSTAGES + 2);
    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf0 + 8 * b, 1); mbar_init(acce0 + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot_p), 2 * PBN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot_p;
    // The weights (the B operand) are written by no kernel: the first stages of this CTA's first tile
    // ask for their weight blocks before waiting for the kernel in front.
    const int n_pre = (int)blockIdx.x < total_tiles ? (kb_total < PSTAGES ? kb_total : PSTAGES) : 0;
    if (warp == 0 && lane == 0) {
        const int b0 = ((int)blockIdx.x / m_tiles) * PBN;
        for (int i = 0; i < n_pre; ++i) {
            mbar_expect_tx(full0 + 8 * i, L::STAGE_BYTES);
            tma_load_2d(smem_u32(smem + i * L::STAGE_BYTES) + L::A_BYTES, &map_b, full0 + 8 * i, i * BK, b0);
        }
    }
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int a0 = (tile % m_tiles) * BM, b0 = (tile / m_tiles) * PBN;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    if (it < n_pre) {                // the weight half of this stage is already on its way
                        tma_load_2d(sa, &map_a, full0 + 8 * s, kb * BK, a0);
                        continue;
                    }
                    if (!mbar_wait(empty0 + 8 * s, ((it / PSTAGES) & 1) ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); ok = false; break; }
                    mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                    tma_load_2d(sa, &map_a, full0 + 8 * s, kb * BK, a0);
                    tma_load_2d(sa + L::A_BYTES, &map_b, full0 + 8 * s, kb * BK, b0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PBN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int it = 0, n = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++n) {
                const int buf = n & 1;
                if (!mbar_wait(acce0 + 8 * buf, ((n >> 1) & 1) ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + buf * PBN;
                for (int kb = 0; kb < kb_total; ++kb, ++it) {
                    const int s = it % PSTAGES;
                    if (!mbar_wait(full0 + 8 * s, (it / PSTAGES) & 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_bf16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty0 + 8 * s);
                }
                umma_commit(accf0 + 8 * buf);
            }
        }
    } else {
        const int quad = warp & 3;
        int n = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++n) {
            const int buf = n & 1;
            const int a0 = (tile % m_tiles) * BM, b0 = (tile / m_tiles) * PBN;
            const int a_row = a0 + quad * 32 + lane;
            const float row_scale = (AIRUN_FOLD_NORM && p.ssq_in && a_row < p.a_rows) ? token_scale(p, a_row) : 1.0f;   // while the MMAs run
            float ssq_acc = 0.0f;
            if (!mbar_wait(accf0 + 8 * buf, (n >> 1) & 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + buf * PBN + ((uint32_t)(quad * 32) << 16);
            constexpr int STEP = EPI == EPI_SWIGLU ? 32 : 16;
#pragma unroll 2
            for (int c = 0; c < PBN; c += STEP) {
                float v[16], u[16];
                tmem_ld16(lane_addr + c, v);
                if (STEP == 32) tmem_ld16(lane_addr + c + 16, u);
                if (c + STEP >= PBN) {                      // the last columns are in registers: hand the buffer back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acce0 + 8 * buf) : "memory");
                }
                if (AIRUN_FOLD_NORM && p.ssq_in) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) { v[i] *= row_scale; if (STEP == 32) u[i] *= row_scale; }
                }
                if (EPI == EPI_SWIGLU) store_swiglu_normal(p, v, u, a_row, b0, c);
                else if (EPI == EPI_RESID) ssq_acc += store_resid_normal(p, v, a_row, b0 + c);
                else store_chunk<EPI, false>(p, v, a_row, b0, c);
            }
            if (EPI == EPI_RESID && a_row < p.a_rows) p.ssq_out[(size_t)(tile / m_tiles) * p.ssq_out_ld + a_row] = ssq_acc;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * PBN);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)f;
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows, K, ld; int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        h = h * 1000003u ^ (size_t)k.rows;
        h = h * 1000003u ^ (size_t)k.K;
        h = h * 1000003u ^ (size_t)k.ld;
        h = h * 1000003u ^ (size_t)k.box_rows;
        return h;
    }
};

// A tensor map of a row-major [rows][K] bfloat16 matrix with boxes of box_rows x 64.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, K, ld, box_rows};
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return AIRUN_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return AIRUN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return AIRUN_ERR_ARG;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
    return AIRUN_OK;
}

// Stages of the clustered build: as many as fit in 200 KB, at most twice the plain build's.
constexpr int cluster_stages(int bn, int stages) {
    const int stage_bytes = (BM + bn) * BK * 2;
    const int fit = (200 * 1024) / stage_bytes;
    return fit < 2 * stages ? fit : 2 * stages;
}

template <int BN, int STAGES, int EPI, bool SWAP>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    constexpr bool CAN_CLUSTER = !(SWAP && BN < 32);          // see the call site of cluster_reduce
    if constexpr (CAN_CLUSTER) {
        if (p.cluster_reduce) {
            // clustered CTAs are placed one to an SM at most (ncu: launch__cluster_max_active), so each
            // may as well use the whole shared memory: twice the stages
            constexpr int CS = cluster_stages(BN, STAGES);
            using LC = SmemLayout<BN, CS>;
            static unsigned long long configured_c = 0;       // one bit per device: the attribute is the device's
            auto kern = gemm_tcgen05_kernel<BN, CS, EPI, SWAP, true>;
            if (first_on_device(configured_c)) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LC::TOTAL);
                if (e != cudaSuccess) return (int)e;
            }
            airun_launch_cluster(kern, dim3(grid), dim3(GEMM_THREADS), LC::TOTAL, stream, (unsigned)p.ksplit, ma, mb, p);
            return airun_launch_status();
        }
    }
    static unsigned long long configured = 0;
    auto kern = gemm_tcgen05_kernel<BN, STAGES, EPI, SWAP, false>;
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(kern, dim3(grid), dim3(GEMM_THREADS), L::TOTAL, stream, ma, mb, p);
    return airun_launch_status();
}

template <int EPI>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
    using L = SmemLayout<PBN, PSTAGES>;
    constexpr int SMEM = L::TOTAL + 64;
    static unsigned long long configured = 0;
    static int sms_of[64];
    auto kern = gemm_tcgen05_persistent_kernel<EPI>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return AIRUN_ERR_ARG;
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev);
    }
    const int n_sm = sms_of[dev];
    const int m_tiles = (p.a_rows + BM - 1) / BM, n_tiles = (p.b_rows + PBN - 1) / PBN;
    const int total = m_tiles * n_tiles;
    const int grid = total < n_sm ? total : n_sm;
    airun_launch(kern, dim3(grid), dim3(GEMM_THREADS), SMEM, stream, ma, mb, p, m_tiles, n_tiles);
    return airun_launch_status();
}

// How many clusters of `ks` CTAs of this kernel the GPU holds at once (0: unknown or none).  A product
// whose tiles outnumber them would run its last clusters alone in a second wave.
template <int BN, int STAGES, int EPI, bool SWAP>
int cluster_capacity(int ks) {
    static int per_device[64][9];                             // zero: not asked yet on that device
    int dev = 0;
    if (ks < 2 || ks > 8 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    int* cache = per_device[dev];
    if (cache[ks] == 0) {
        using L = SmemLayout<BN, cluster_stages(BN, STAGES)>;
        auto kern = gemm_tcgen05_kernel<BN, cluster_stages(BN, STAGES), EPI, SWAP, true>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, ks);
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = L::TOTAL;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = ks;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess) cudaGetLastError();
        cache[ks] = (e == cudaSuccess && n > 0) ? n : -1;
    }
    return cache[ks] > 0 ? cache[ks] : 0;
}

template <int EPI>
int cluster_capacity_for(bool swap, int bn, int ks) {
    if (!swap) return bn == 128 ? cluster_capacity<128, 6, EPI, false>(ks) : bn == 256 ? cluster_capacity<256, 4, EPI, false>(ks) : 0;
    if (bn == 32) return cluster_capacity<32, 5, EPI, true>(ks);
    if (bn == 64) return cluster_capacity<64, 4, EPI, true>(ks);
    if (bn == 128) return cluster_capacity<128, 3, EPI, true>(ks);
    return 0;
}

int cluster_capacity_any(int epi, bool swap, int bn, int ks) {
    if (epi == EPI_F32) return cluster_capacity_for<EPI_F32>(swap, bn, ks);
    if (epi == EPI_BF16) return cluster_capacity_for<EPI_BF16>(swap, bn, ks);
    if (epi == EPI_SWIGLU) return cluster_capacity_for<EPI_SWIGLU>(swap, bn, ks);
#if AIRUN_FOLD_NORM
    if (epi == EPI_RESID) return cluster_capacity_for<EPI_RESID>(swap, bn, ks);
#endif
    return 0;
}

template <int EPI>
int dispatch(bool swap, int bn, const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid,
             cudaStream_t stream) {
    if (!swap) {
        static const bool persistent_allowed = !(getenv("AIRUN_GEMM_PERSISTENT") && getenv("AIRUN_GEMM_PERSISTENT")[0] == '0');
        if (bn == 256 && p.ksplit == 1 && persistent_allowed) return launch_persistent<EPI>(ma, mb, p, stream);
        if (bn == 128) return launch<128, 6, EPI, false>(ma, mb, p, grid, stream);
        if (bn == 256) return launch<256, 4, EPI, false>(ma, mb, p, grid, stream);
        return AIRUN_ERR_UNSUPPORTED;
    }
    // stage counts that leave room for two CTAs on an SM (about 110 KB each)
    if (bn == 16) return launch<16, 6, EPI, true>(ma, mb, p, grid, stream);
    if (bn == 32) return launch<32, 5, EPI, true>(ma, mb, p, grid, stream);
    if (bn == 64) return launch<64, 4, EPI, true>(ma, mb, p, grid, stream);
    if (bn == 128) return launch<128, 3, EPI, true>(ma, mb, p, grid, stream);
    return AIRUN_ERR_UNSUPPORTED;
}

}  // namespace

// Scratch the caller must provide for ksplit > 1: floats and tile counters.
AIRUN_EXPORT long long airun_gemm_tcgen05_scratch_floats(int M, int N, int swap, int bn, int ksplit) {
    const long long a_rows = swap ? N : M, b_rows = swap ? M : N;
    const long long tiles = ((a_rows + BM - 1) / BM) * ((b_rows + bn - 1) / bn);
    return ksplit > 1 ? tiles * ksplit * bn * BM : 0;
}

// out[M][N] = x[M][K] * W[N][K]^T.  x, W bfloat16 row-major (K % 8 == 0, 16-byte aligned rows).
// epi: 0 float32 out [M][N]; 1 bfloat16 out [M][N]; 2 SwiGLU, bfloat16 out [M][N/2];
//      3 residual + norm: resid[M][N] += result, out[M][N] = bfloat16(resid * norm_w), ssq_out[parts][ssq_out_ld]
//        = sums of resid^2 per token; parts = ceil(N / 128) when swapped, ceil(N / bn) otherwise.
// swap: weights as the 128-row operand (bn >= M, one B tile per 'bn' tokens).
// counters: one int per tile, zero on entry when ksplit > 1 (the kernel leaves them zero).
// ssq_in: when not null, x is an un-normalised bfloat16(resid * norm_w) and every token's results are
//   multiplied by rsqrt(sum over ssq_parts of ssq_in[part][token] / norm_size + eps).
AIRUN_EXPORT int airun_gemm_tcgen05_ex(const void* x, const void* W, void* out, int M, int N, int K,
                                       long long ldx, long long ldw, long long ldc, int epi, int swap, int bn,
                                       int ksplit, float* scratch, int* counters, int* err, cudaStream_t stream,
                                       const float* ssq_in, int ssq_parts, int ssq_ld, float eps_in, int norm_size,
                                       float* resid, long long ld_resid, const float* norm_w, float* ssq_out,
                                       int ssq_out_ld) {
    if (M <= 0 || N <= 0 || K <= 0 || !err) return M == 0 ? AIRUN_OK : AIRUN_ERR_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return AIRUN_ERR_ARG;
    if (epi == EPI_SWIGLU && (N % 32 != 0)) return AIRUN_ERR_ARG;
    if (ksplit < 1 || (ksplit > 1 && (!scratch || !counters))) return AIRUN_ERR_ARG;
    if (!AIRUN_FOLD_NORM && (ssq_in || epi == EPI_RESID)) return AIRUN_ERR_UNSUPPORTED;      // the other build has it
    if (ssq_in && (ssq_parts <= 0 || ssq_ld < M || norm_size <= 0)) return AIRUN_ERR_ARG;
    if (epi == EPI_RESID && (!resid || !norm_w || !ssq_out || ssq_out_ld < M || ld_resid < N)) return AIRUN_ERR_ARG;
    const int kb_total = (K + BK - 1) / BK;
    if (ksplit > kb_total) ksplit = kb_total;
    // 2 to 8 slices of a tile run as one cluster and add up through distributed shared memory
    // (AIRUN_GEMM_CLUSTER=0: through the scratch, as more than 8 slices always do).  Not for the
    // narrowest tiles (up to 16 tokens): their partial tiles are small, and inside a decode step the
    // clusters, which need all their CTAs placed at once, overlapped less with the kernel before
    // them than single CTAs do (measured: 2 to 4 % slower steps at batch 1 and 8).  If the GPU cannot
    // hold a cluster for every tile at once, fewer slices are cut.
    static const bool cluster_allowed = !(getenv("AIRUN_GEMM_CLUSTER") && getenv("AIRUN_GEMM_CLUSTER")[0] == '0');
    bool clustered = cluster_allowed && ksplit >= 2 && ksplit <= 8 && !(swap && bn < 32) && !(epi == EPI_RESID && !swap);
    if (clustered) {
        const long long tiles = (long long)(((swap ? N : M) + BM - 1) / BM) * (((swap ? M : N) + bn - 1) / bn);
        int ks = ksplit;
        while (ks >= 2) {
            // the slices may come out fewer than asked for once they are whole K-steps
            const int per = (kb_total + ks - 1) / ks, real = (kb_total + per - 1) / per;
            if (real >= 2 && cluster_capacity_any(epi, swap != 0, bn, real) >= tiles) break;
            --ks;
        }
        if (ks >= 2) ksplit = ks;
        else clustered = false;
    }
    GemmParams p = {};
    p.a_rows = swap ? N : M;
    p.b_rows = swap ? M : N;
    p.K = K;
    p.k_blocks_per_split = (kb_total + ksplit - 1) / ksplit;
    p.ksplit = (kb_total + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.out = out;
    p.ldc = ldc;
    p.scratch = scratch;
    p.counters = counters;
    p.err = err;
    p.ssq_in = ssq_in; p.ssq_parts = ssq_parts; p.ssq_ld = ssq_ld; p.eps_in = eps_in;
    p.inv_n_in = norm_size > 0 ? 1.0f / (float)norm_size : 0.0f;
    p.resid = resid; p.ld_resid = ld_resid; p.norm_w = norm_w; p.ssq_out = ssq_out; p.ssq_out_ld = ssq_out_ld;
    p.cluster_reduce = (clustered && p.ksplit >= 2 && p.ksplit <= 8) ? 1 : 0;
    CUtensorMap ma, mb;
    int r;
    if (swap) {
        if ((r = make_map(&ma, W, N, K, ldw, BM)) != AIRUN_OK) return r;
        if ((r = make_map(&mb, x, M, K, ldx, bn)) != AIRUN_OK) return r;
    } else {
        if ((r = make_map(&ma, x, M, K, ldx, BM)) != AIRUN_OK) return r;
        if ((r = make_map(&mb, W, N, K, ldw, bn)) != AIRUN_OK) return r;
    }
    dim3 grid((p.a_rows + BM - 1) / BM, (p.b_rows + bn - 1) / bn, p.ksplit);
    if (grid.y > 65535 || grid.z > 65535) return AIRUN_ERR_ARG;
    if (epi == EPI_F32) return dispatch<EPI_F32>(swap != 0, bn, ma, mb, p, grid, stream);
    if (epi == EPI_BF16) return dispatch<EPI_BF16>(swap != 0, bn, ma, mb, p, grid, stream);
    if (epi == EPI_SWIGLU) return dispatch<EPI_SWIGLU>(swap != 0, bn, ma, mb, p, grid, stream);
#if AIRUN_FOLD_NORM
    if (epi == EPI_RESID) return dispatch<EPI_RESID>(swap != 0, bn, ma, mb, p, grid, stream);
#endif
    return AIRUN_ERR_UNSUPPORTED;
}

AIRUN_EXPORT int airun_gemm_tcgen05(const void* x, const void* W, void* out, int M, int N, int K,
                                    long long ldx, long long ldw, long long ldc, int epi, int swap, int bn,
                                    int ksplit, float* scratch, int* counters, int* err, cudaStream_t stream) {
    if (epi == EPI_RESID) return AIRUN_ERR_ARG;
    return airun_gemm_tcgen05_ex(x, W, out, M, N, K, ldx, ldw, ldc, epi, swap, bn, ksplit, scratch, counters, err, stream,
                                 nullptr, 0, 0, 0.0f, 0, nullptr, 0, nullptr, nullptr, 0);
}

// ------------------------------------------------------------------ no-allocation variant
// See gemm_tcgen05_static.h: the same kernel, with its split-K scratch in arrays that belong
// to this library instead of buffers the caller allocates.  Only the plain build of this file
// carries the arrays and the entry point: the build with the folded norm (AIRUN_FOLD_NORM=1) is a
// second library of the same process and would hold a second copy of them on every GPU.
#if !AIRUN_FOLD_NORM
#include "gemm_tcgen05_static.h"

static __device__ __align__(256) float g_static_scratch[AIRUN_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) int g_static_counters[AIRUN_STATIC_COUNTERS];

namespace {
constexpr int STATIC_MAX_DEVICES = 64;
float* g_static_scratch_addr[STATIC_MAX_DEVICES];
int* g_static_counters_addr[STATIC_MAX_DEVICES];
std::mutex g_static_mu;

// In host code the array names above are only stand-ins; the device addresses come from
// cudaGetSymbolAddress, once per device, with that device current.
int static_addresses(float** scratch, int** counters) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= STATIC_MAX_DEVICES) return AIRUN_ERR_STATIC_SETUP;
    std::lock_guard<std::mutex> g(g_static_mu);
    if (!g_static_scratch_addr[dev]) {
        float* s = nullptr;
        int* c = nullptr;
        if (cudaGetSymbolAddress((void**)&s, g_static_scratch) != cudaSuccess || !s) return AIRUN_ERR_STATIC_SETUP;
        if (cudaGetSymbolAddress((void**)&c, g_static_counters) != cudaSuccess || !c) return AIRUN_ERR_STATIC_SETUP;
        g_static_scratch_addr[dev] = s;
        g_static_counters_addr[dev] = c;
    }
    *scratch = g_static_scratch_addr[dev];
    *counters = g_static_counters_addr[dev];
    return AIRUN_OK;
}

// A tensor map made on the spot, without the cache (which lives on the host heap).
int make_map_uncached(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return AIRUN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? AIRUN_OK : AIRUN_ERR_ARG;
}
}  // namespace

AIRUN_EXPORT int airun_gemm_tcgen05_static(const void* x, const void* W, void* out, int M, int N, int K,
                                           long long ldx, long long ldw, long long ldc, int epi, int swap, int bn,
                                           int ksplit, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0 || !err) return M == 0 ? AIRUN_OK : AIRUN_ERR_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)W & 15)) return AIRUN_ERR_ARG;
    if (epi == EPI_SWIGLU && (N % 32 != 0)) return AIRUN_ERR_ARG;
    if (ksplit < 1) return AIRUN_ERR_ARG;
    if (swap ? !(bn == 16 || bn == 32 || bn == 64 || bn == 128) : !(bn == 128 || bn == 256)) return AIRUN_ERR_UNSUPPORTED;
    const int kb_total = (K + BK - 1) / BK;
    if (ksplit > kb_total) ksplit = kb_total;
    GemmParams p = {};
    p.a_rows = swap ? N : M;
    p.b_rows = swap ? M : N;
    p.K = K;
    p.k_blocks_per_split = (kb_total + ksplit - 1) / ksplit;
    p.ksplit = (kb_total + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.out = out;
    p.ldc = ldc;
    p.err = err;
    p.scratch = nullptr;
    p.counters = nullptr;
    const long long tiles = (long long)((p.a_rows + BM - 1) / BM) * ((p.b_rows + bn - 1) / bn);
    if (p.ksplit > 1) {
        if (tiles * p.ksplit * bn * BM > (long long)AIRUN_STATIC_SCRATCH_FLOATS || tiles > AIRUN_STATIC_COUNTERS)
            return AIRUN_ERR_STATIC_TOO_LARGE;
        const int r = static_addresses(&p.scratch, &p.counters);
        if (r != AIRUN_OK) return r;
        // the counters must start at zero whatever an earlier call left behind
        cudaError_t e = cudaMemsetAsync(p.counters, 0, (size_t)tiles * sizeof(int), stream);
        if (e != cudaSuccess) return (int)e;
    }
    CUtensorMap ma, mb;
    int r;
    if (swap) {
        if ((r = make_map_uncached(&ma, W, N, K, ldw, BM)) != AIRUN_OK) return r;
        if ((r = make_map_uncached(&mb, x, M, K, ldx, bn)) != AIRUN_OK) return r;
    } else {
        if ((r = make_map_uncached(&ma, x, M, K, ldx, BM)) != AIRUN_OK) return r;
        if ((r = make_map_uncached(&mb, W, N, K, ldw, bn)) != AIRUN_OK) return r;
    }
    dim3 grid((p.a_rows + BM - 1) / BM, (p.b_rows + bn - 1) / bn, p.ksplit);
    if (grid.y > 65535 || grid.z > 65535) return AIRUN_ERR_ARG;
    if (epi == EPI_F32) return dispatch<EPI_F32>(swap != 0, bn, ma, mb, p, grid, stream);
    if (epi == EPI_BF16) return dispatch<EPI_BF16>(swap != 0, bn, ma, mb, p, grid, stream);
    if (epi == EPI_SWIGLU) return dispatch<EPI_SWIGLU>(swap != 0, bn, ma, mb, p, grid, stream);
    return AIRUN_ERR_UNSUPPORTED;
}
#endif  // !AIRUN_FOLD_NORM
