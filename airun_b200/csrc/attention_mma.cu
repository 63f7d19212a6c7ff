// Tensor-core attention over cache pages for bfloat16 q and pages, one head size per
// build (-DHD=<head_dim>, a multiple of 16 up to 256).
//
// Both kernels pack the query heads that share a KV head into the rows of one
// matrix product, so every key and value row is read once for the whole group
// (the reference's decode kernel makes "the G query heads rows of the MMA",
// crates/airun-cuda/kernels/ops.cu:1167-1364; its prefill kernel is the FA-2 style
// crates/airun-cuda/kernels/ops.cu:1796-2078).  Scores are s = scale * q.K in float32
// from bfloat16 operands; the running maximum, the sum and the output accumulate
// in float32; probabilities are rounded to bfloat16 for the P.V product.  Key j is
// visible to a query at position p iff j <= p and (window == 0 or p - j < window).
//
//  attn_prefill: one CTA = 128 packed rows (128/G tokens x G heads) of one request and
//    KV head; 8 warps x 16 rows; K/V tiles of 64 keys gathered page by page with
//    cp.async into double-buffered, swizzled shared memory; tiles wholly hidden by
//    the causal rule or the window are skipped.  The blocks of the tiles with the most
//    keys, of all KV heads, start first.
//  attn_decode: one CTA = one token, one KV head (16 heads of its group at most),
//    one slice of the keys; its 4 warps take 16-key tiles in turn with private stages
//    (three, filled by cp.async.bulk.tensor, when pages are powers of two >= 16 and the
//    head size a multiple of 64; else two, filled by cp.async) and merge in shared
//    memory.  With more than one slice each CTA
//    writes (max, sum, acc) to scratch and the last CTA of the token and head (a
//    counter, no spinning) merges the slices in order.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <cstring>
#include <utility>

#ifndef HD
#error "compile with -DHD=<head_dim>"
#endif
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head_dim must be a multiple of 16 up to 256");

#define CHUNKS (HD / 8)                 // 16-byte chunks per row
#define SWZ (HD % 64 == 0)
#define NEG_BIG (-1.0e30f)
#define LOG2E 1.4426950408889634f

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ int swz(int row, int chunk) { return SWZ ? (chunk ^ (row & 7)) : chunk; }
// byte offset of (row, chunk) inside a [rows][HD] bf16 tile
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return (uint32_t)(row * CHUNKS + swz(row, chunk)) * 16u; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// ---- TMA pieces of the decode kernel (pages whose size is a multiple of 16, head_dim a multiple of 64)
// A 16-key K (or V) tile is HD/64 boxes of 16 rows x 128 bytes, landed with the 128-byte swizzle.
__device__ __forceinline__ uint32_t tile_off_tma(int row, int chunk) {
    return (uint32_t)((chunk >> 3) * 2048 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {     // bounded: about two seconds
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnParams {
    const __nv_bfloat16* q;        // [T][nh][HD]
    __nv_bfloat16* out;            // [T][nh][HD]
    const __nv_bfloat16* pool;     // [pages][2][nkv][page_size][HD]
    const int32_t* block_table;    // [R][max_blocks]
    const int32_t* positions;      // [T]
    const int32_t* req_of_token;   // [T]
    int max_blocks, num_reqs, num_pages, page_size, page_shift, nh, nkv, G;   // page_shift: log2(page_size) or -1
    float scale_log2;              // scale * log2(e)
    int window;
    int* err;
};

// Address of key j's row (K) of KV head kvh; V is v_off elements further.  Returns nullptr for a
// bad page (and records it).
__device__ __forceinline__ const __nv_bfloat16* key_row(const AttnParams& p, const int32_t* bt, int kvh, int j) {
    const int blk = p.page_shift >= 0 ? (j >> p.page_shift) : j / p.page_size;
    const int page = blk < p.max_blocks ? __ldg(bt + blk) : -1;
    if (page < 0 || page >= p.num_pages) { atomicOr(p.err, AIRUN_DEV_BAD_PAGE); return nullptr; }
    return p.pool + (((size_t)page * 2 * p.nkv + kvh) * p.page_size + (j - blk * p.page_size)) * HD;
}

// ------------------------------------------------------------------ prefill
#define PM 128         // packed rows per CTA (8 warps x 16 rows)
#define PTHREADS 256
#define PN 64          // keys per tile

struct PrefillTile { int req, tok0, n_tok, first_row; };   // tokens [tok0, tok0+n_tok) of the batch, all of request req

// SHARED: the same kernel over a prefix of keys that several decoded tokens have in common (their
// requests were forked from one: the first pages of their block tables are the same pages).  The
// tokens of the batch, PM / G to a CTA, are the packed rows; every key below *k_end_dev is visible to
// all of them; the keys are cut into gridDim.x slices; and instead of an output row the CTA writes
// each row's (maximum, sum, unnormalised output) into the slice's slot of the decode kernel's
// scratch, which merges them with the slices of the token's own keys.  The keys and values of the
// prefix are then read once for all the tokens, not once for each.
struct SharedArgs {
    const int32_t* k_end_dev;   // keys [0, *k_end_dev) are shared
    int n_tok;                  // tokens in the batch (rows 0 .. n_tok-1)
    float* scratch;             // the decode kernel's partial results
    int unit_stride, slot0;     // slots per (token, KV head, head group); first slot of this kernel's slices
};

// n_tiles_dev: null, or the number of tiles another kernel has written (the grid may be larger)
template <bool SHARED>
__global__ __launch_bounds__(PTHREADS, 2) void attn_prefill_kernel(const AttnParams p, const int4* __restrict__ tiles,
                                                                   const int* __restrict__ n_tiles_dev, const SharedArgs sh) {
    pdl_trigger();
    pdl_wait();
    // the KV heads of a tile before the next tile (blocks start in the order of their linear index): the
    // tiles with the most keys, of all heads, start first
    const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const int tile_idx = SHARED ? (int)blockIdx.x : lin / (int)gridDim.y;
    if (!SHARED && n_tiles_dev && tile_idx >= *n_tiles_dev) return;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* sQ = smem;                               // [PM][HD]
    uint8_t* sK = sQ + PM * HD * 2;                   // [2][PN][HD]
    uint8_t* sV = sK + 2 * PN * HD * 2;               // [2][PN][HD]
    const int G = p.G;
    int req, tok0, n_tok;
    if (SHARED) {
        const int per = PM / G;
        tok0 = blockIdx.z * per;
        n_tok = min(per, sh.n_tok - tok0);
        req = p.req_of_token[tok0];
    } else {
        const int4 t4 = tiles[tile_idx];
        req = t4.x; tok0 = t4.y; n_tok = t4.z;
    }
    const int kvh = SHARED ? (int)blockIdx.y : lin % (int)gridDim.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_rows = n_tok * G;                     // valid packed rows (<= PM)
    const bool req_ok = req >= 0 && req < p.num_reqs;  // (a padded batch: rows of no request)
    const int32_t* bt = p.block_table + (size_t)(req_ok ? req : 0) * p.max_blocks;
    const size_t v_off = (size_t)p.nkv * p.page_size * HD;

    // positions of the first and last token of the tile (tokens of a request are in position order);
    // SHARED: the last shared key stands for both
    const int k_end = SHARED ? (req_ok ? *sh.k_end_dev : 0) : 0;
    const int pos_lo = SHARED ? k_end - 1 : p.positions[tok0], pos_hi = SHARED ? k_end - 1 : p.positions[tok0 + n_tok - 1];

    // ---- Q tile -> shared memory
    for (int i = threadIdx.x; i < PM * CHUNKS; i += PTHREADS) {
        const int r = i / CHUNKS, c = i - r * CHUNKS;
        const bool valid = r < n_rows;
        const int tok = tok0 + (valid ? r / G : 0), head = kvh * G + (valid ? r % G : 0);
        cp_async16(smem_u32(sQ) + tile_off(r, c), p.q + ((size_t)tok * p.nh + head) * HD + c * 8, valid);
    }
    cp_commit();

    const int k_first = (!SHARED && p.window > 0) ? max(0, pos_lo - p.window + 1) : 0;
    int tile_first = k_first / PN;
    int n_tiles = pos_hi >= 0 ? pos_hi / PN - tile_first + 1 : 0;
    if (SHARED) {                                     // this CTA's slice of the shared tiles
        const int per_slice = (n_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
        tile_first = min(n_tiles, (int)blockIdx.x * per_slice);
        n_tiles = min(n_tiles, tile_first + per_slice) - tile_first;
    }

    auto load_kv = [&](int tile, int stage) {
        const int j0 = tile * PN;
        uint32_t kb = smem_u32(sK + stage * PN * HD * 2), vb = smem_u32(sV + stage * PN * HD * 2);
#pragma unroll 4
        for (int i = threadIdx.x; i < PN * CHUNKS; i += PTHREADS) {
            const int r = i / CHUNKS, c = i - r * CHUNKS;
            const int j = j0 + r;
            const __nv_bfloat16* src = (j <= pos_hi && j >= k_first) ? key_row(p, bt, kvh, j) : nullptr;
            const bool valid = src != nullptr;
            const __nv_bfloat16* s = valid ? src + c * 8 : p.pool;
            cp_async16(kb + tile_off(r, c), s, valid);
            cp_async16(vb + tile_off(r, c), valid ? s + v_off : s, valid);
        }
        cp_commit();
    };

    if (n_tiles > 0) load_kv(tile_first, 0);

    // this thread's two rows: warp*16 + g and + 8
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const int pos0 = r0 < n_rows ? (SHARED ? pos_hi : p.positions[tok0 + r0 / G]) : -1;
    const int pos1 = r1 < n_rows ? (SHARED ? pos_hi : p.positions[tok0 + r1 / G]) : -1;

    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.0f, l1 = 0.0f;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }

    for (int it = 0; it < n_tiles; ++it) {
        const int stage = it & 1;
        if (it + 1 < n_tiles) { load_kv(tile_first + it + 1, stage ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
        __syncthreads();
        const uint32_t kb = smem_u32(sK + stage * PN * HD * 2), vb = smem_u32(sV + stage * PN * HD * 2);
        const int j0 = (tile_first + it) * PN;

        float s[PN / 8][4];
#pragma unroll
        for (int n = 0; n < PN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f; }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
            uint32_t qf[4];                   // the Q fragment is read again for every tile: registers are scarcer than shared-memory reads
            ldsm4(qf, smem_u32(sQ) + tile_off(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * k + (lane >> 4)));
#pragma unroll
            for (int n2 = 0; n2 < PN / 16; ++n2) {
                uint32_t b[4];
                ldsm4(b, kb + tile_off(n2 * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * k + ((lane >> 3) & 1)));
                mma16816(s[2 * n2], qf, b[0], b[1]);
                mma16816(s[2 * n2 + 1], qf, b[2], b[3]);
            }
        }
        // mask, scale, running maximum
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int n = 0; n < PN / 8; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + n * 8 + 2 * t + (e & 1);
                const int pos = (e < 2) ? pos0 : pos1;
                const bool vis = j <= pos && (SHARED || p.window == 0 || pos - j < p.window);
                const float v = vis ? s[n][e] * p.scale_log2 : NEG_BIG;
                s[n][e] = v;
                if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);
        m0 = mx0; m1 = mx1;
        float rs0 = 0.0f, rs1 = 0.0f;
        uint32_t pf[PN / 16][4];
#pragma unroll
        for (int n = 0; n < PN / 8; ++n) {
            // a fully hidden row keeps m = NEG_BIG: exp2(NEG_BIG - NEG_BIG) would be 1, so test visibility by value
            const float p00 = s[n][0] > 0.5f * NEG_BIG ? exp2f(s[n][0] - mx0) : 0.0f;
            const float p01 = s[n][1] > 0.5f * NEG_BIG ? exp2f(s[n][1] - mx0) : 0.0f;
            const float p10 = s[n][2] > 0.5f * NEG_BIG ? exp2f(s[n][2] - mx1) : 0.0f;
            const float p11 = s[n][3] > 0.5f * NEG_BIG ? exp2f(s[n][3] - mx1) : 0.0f;
            rs0 += p00 + p01;
            rs1 += p10 + p11;
            pf[n >> 1][(n & 1) * 2 + 0] = pack_bf16(p00, p01);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
        if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {      // the maximum moved somewhere in the warp
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        }
#pragma unroll
        for (int kk = 0; kk < PN / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < HD / 16; ++n2) {
                uint32_t b[4];
                ldsm4t(b, vb + tile_off(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * n2 + (lane >> 4)));
                mma16816(o[2 * n2], pf[kk], b[0], b[1]);
                mma16816(o[2 * n2 + 1], pf[kk], b[2], b[3]);
            }
        }
        __syncthreads();       // everyone is done with this stage before it is refilled
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (SHARED) {
        if (n_tiles == 0) cp_wait<0>();               // (the Q tile was asked for and never used)
        // (maximum, sum, unnormalised output) of each row into this slice's slot of the row's unit
        const int hgroups = (G + 15) / 16;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r1 : r0;
            if (r >= n_rows) continue;
            const int tok = tok0 + r / G, hin = r % G;
            const int unit = tok * (p.nkv * hgroups) + kvh * hgroups + hin / 16;
            float* dst = sh.scratch + ((size_t)unit * sh.unit_stride + sh.slot0 + blockIdx.x) * (16 * (HD + 2))
                         + (hin % 16) * (HD + 2);
            if (t == 0) { dst[0] = half ? m1 : m0; dst[1] = half ? l1 : l0; }
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) {
                dst[2 + n * 8 + 2 * t] = o[n][2 * half];
                dst[2 + n * 8 + 2 * t + 1] = o[n][2 * half + 1];
            }
        }
        return;
    }
    const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
    if (r0 < n_rows) {
        __nv_bfloat16* dst = p.out + ((size_t)(tok0 + r0 / G) * p.nh + kvh * G + r0 % G) * HD;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][0] * i0, o[n][1] * i0);
    }
    if (r1 < n_rows) {
        __nv_bfloat16* dst = p.out + ((size_t)(tok0 + r1 / G) * p.nh + kvh * G + r1 % G) * HD;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][2] * i1, o[n][3] * i1);
    }
}

// ------------------------------------------------------------------ decode
#define DW 4                    // warps per CTA
#define DN 16                   // keys per tile
#define MAX_SPLITS 64

struct DecodeExtra {
    const int32_t* rows;        // [n] batch rows (tokens) this launch handles
    int n_splits;
    float* scratch;             // [n][nkv*hgroups][n_splits][16][HD + 2]
    int* counters;              // [n][nkv*hgroups], zero between launches
    const int32_t* n_rows_dev;  // null, or: the rows in use are read on the device (the grid may be larger) and
    int dyn_slots;              //   every row picks its own number of slices, at most n_splits, so that about
                                //   dyn_slots CTAs run and a slice has 128 keys or more
    const int32_t* k_begin_dev; // null, or: keys below *k_begin_dev are not this kernel's (a shared prefix, whose
    int extra_slices;           //   results another kernel has put into the extra_slices slots after this
                                //   kernel's n_splits; they are merged with this kernel's own slices)
    int early_ok;               // the caller vouches that every key but each token's newest was written before the
                                //   chain of launches this one belongs to began (a step replayed as one graph)
};

// TMA = true: K/V tiles arrive by cp.async.bulk.tensor (one lane of each warp issues HD/64 boxes per
// tile, three stages per warp, an mbarrier per stage); TMA = false: cp.async, two stages, any page size.
// WITH_PREFIX: the build that leaves a shared prefix to another kernel and merges its results
// (k_begin_dev, extra_slices); a build of its own so that the plain one carries none of that code.
template <bool TMA, bool WITH_PREFIX>
__global__ __launch_bounds__(32 * DW) void attn_decode_kernel(const AttnParams p, const DecodeExtra x,
                                                              const __grid_constant__ CUtensorMap kv_map) {
    pdl_trigger();
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // per warp: DSTAGES x (K tile + V tile); the Q tile [16][HD] and the mbarriers sit after them
    constexpr int DSTAGES = TMA ? 3 : 2;
    constexpr int TILE_BYTES = DN * HD * 2;
    constexpr int WARP_BYTES = DSTAGES * 2 * TILE_BYTES;
    uint8_t* sQ = smem + DW * WARP_BYTES;
    uint64_t* bars = (uint64_t*)(sQ + 16 * HD * 2) + (threadIdx.x >> 5) * DSTAGES;
    if (TMA && (threadIdx.x & 31) == 0) {
        for (int s = 0; s < DSTAGES; ++s) mbar_init(smem_u32(bars + s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // Keys and values of earlier positions were written by earlier steps, and the batch's layout was
    // copied to the device before the step began: with TMA, no row list from a kernel of this step and
    // the caller's word for it (early_ok), the first tiles are requested before waiting for the kernel
    // in front (which writes q and the newest key), so they stream in under its tail.  The tile that
    // holds the newest key waits.
    const bool early = TMA && x.n_rows_dev == nullptr && x.early_ok != 0;
    if (!early) pdl_wait();
    __shared__ float s_m[DW][16], s_l[DW][16];
    __shared__ int s_ticket;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x;
    const int hgroups = (p.G + 15) / 16;
    const int kvh = blockIdx.y / hgroups, hg = blockIdx.y - kvh * hgroups;
    const int n_rows_used = x.n_rows_dev ? *x.n_rows_dev : (int)gridDim.z;
    if ((int)blockIdx.z >= n_rows_used) return;
    const int tok = x.rows ? x.rows[blockIdx.z] : (int)blockIdx.z;     // no list: row i is token i
    const int pos = p.positions[tok];
    const int req = p.req_of_token[tok];
    const int heads = min(16, p.G - hg * 16);          // valid rows
    const int head0 = kvh * p.G + hg * 16;
    const bool live = req >= 0 && req < p.num_reqs && pos >= 0;
    const int32_t* bt = p.block_table + (size_t)(live ? req : 0) * p.max_blocks;
    const size_t v_off = (size_t)p.nkv * p.page_size * HD;
    const int k_begin = (WITH_PREFIX && x.k_begin_dev) ? *x.k_begin_dev : 0;
    const int k_first = live ? max(k_begin, p.window > 0 ? max(0, pos - p.window + 1) : 0) : 0;
    const int tile_first = k_first / DN;
    const int n_tiles_all = live ? pos / DN - tile_first + 1 : 0;
    int ns = x.n_splits, ns_stride = x.n_splits;       // slices of this row; slices the scratch has room for
    if (x.n_rows_dev) {
        const int fit = max(1, x.dyn_slots / max(1, n_rows_used * (int)gridDim.y));
        ns_stride = min(x.n_splits, fit);
        ns = max(1, min(ns_stride, (n_tiles_all + 7) / 8));
        if (split >= ns) return;
    }

    // key tiles of this token, this slice, this warp
    const int per_split = (n_tiles_all + ns - 1) / ns;
    const int tb = tile_first + split * per_split;
    const int te = min(tile_first + n_tiles_all, tb + per_split);
    const int my_n = te > tb + warp ? (te - tb - warp + DW - 1) / DW : 0;      // tiles tb+warp, tb+warp+DW, ...

    uint8_t* wbase = smem + warp * WARP_BYTES;
    // A 16-key tile lies inside one page when the page size is a multiple of 16: one block-table
    // lookup per tile, and the tile's K rows (and V rows) are one contiguous run of 16 * HD values.
    const bool one_page = p.page_shift >= 4;
    auto load_tile = [&](int tile, int stage) {
        const int j0 = tile * DN;
        const uint32_t kb = smem_u32(wbase + stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        if (one_page) {
            const __nv_bfloat16* base = key_row(p, bt, kvh, j0);
            const bool inside = j0 >= k_first && j0 + DN - 1 <= pos;
#pragma unroll
            for (int k = 0; k < DN * CHUNKS / 32; ++k) {
                const int i = lane + 32 * k;
                const int r = i / CHUNKS, c = i - r * CHUNKS;
                const bool valid = base != nullptr && (inside || (j0 + r <= pos && j0 + r >= k_first));
                const __nv_bfloat16* s = valid ? base + i * 8 : p.pool;
                cp_async16(kb + tile_off(r, c), s, valid);
                cp_async16(vb + tile_off(r, c), valid ? s + v_off : s, valid);
            }
        } else {
#pragma unroll 4
            for (int i = lane; i < DN * CHUNKS; i += 32) {
                const int r = i / CHUNKS, c = i - r * CHUNKS;
                const int j = j0 + r;
                const __nv_bfloat16* src = (j <= pos && j >= k_first) ? key_row(p, bt, kvh, j) : nullptr;
                const bool valid = src != nullptr;
                const __nv_bfloat16* s = valid ? src + c * 8 : p.pool;
                cp_async16(kb + tile_off(r, c), s, valid);
                cp_async16(vb + tile_off(r, c), valid ? s + v_off : s, valid);
            }
        }
        cp_commit();
    };
    // TMA: lane 0 arms the stage's barrier with the tile's bytes and issues its boxes.  Rows of the
    // page beyond the context hold older or zero data; those keys are masked below.
    auto issue_tile = [&](int tile, int stage) {
        const int j0 = tile * DN;
        const int blk = j0 >> p.page_shift;
        int page = blk < p.max_blocks ? __ldg(bt + blk) : -1;
        if (page < 0 || page >= p.num_pages) { atomicOr(p.err, AIRUN_DEV_BAD_PAGE); page = 0; }
        const int krow = (((page * 2) * p.nkv + kvh) << p.page_shift) + (j0 & (p.page_size - 1));
        const int vrow = krow + (p.nkv << p.page_shift);
        const uint32_t bar = smem_u32(bars + stage);
        const uint32_t kb = smem_u32(wbase + stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        mbar_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
        for (int h = 0; h < HD / 64; ++h) {
            tma_load_2d(kb + h * 2048, &kv_map, bar, h * 64, krow);
            tma_load_2d(vb + h * 2048, &kv_map, bar, h * 64, vrow);
        }
    };
    if (TMA) {
        int deferred = -1;
        if (lane == 0)
            for (int i = 0; i < DSTAGES - 1 && i < my_n; ++i) {
                const int tile = tb + warp + i * DW;
                if (early && tile == pos / DN) deferred = i;           // holds the key the kernel in front writes
                else issue_tile(tile, i);
            }
        if (early) {
            pdl_wait();
            if (deferred >= 0) issue_tile(tb + warp + deferred * DW, deferred);
        }
    }
    // Q rows -> shared memory (rows >= heads are zero)
    for (int i = threadIdx.x; i < 16 * CHUNKS; i += 32 * DW) {
        const int r = i / CHUNKS, c = i - r * CHUNKS;
        const bool valid = r < heads;
        cp_async16(smem_u32(sQ) + tile_off(r, c), p.q + ((size_t)tok * p.nh + head0 + (valid ? r : 0)) * HD + c * 8, valid);
    }
    cp_commit();

    if (!TMA && my_n > 0) load_tile(tb + warp, 0);

    float m0 = NEG_BIG, m1 = NEG_BIG, l0 = 0.0f, l1 = 0.0f;
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f; }

    cp_wait<0>();
    __syncthreads();                       // Q (and each warp's first tile) has landed
    uint32_t qf[HD / 16][4];
#pragma unroll
    for (int k = 0; k < HD / 16; ++k)
        ldsm4(qf[k], smem_u32(sQ) + tile_off((lane & 7) + ((lane >> 3) & 1) * 8, 2 * k + (lane >> 4)));

    bool timed_out = false;
    for (int it = 0; it < my_n; ++it) {
        const int stage = TMA ? it % DSTAGES : (it & 1);
        if (TMA) {
            if (lane == 0 && it + DSTAGES - 1 < my_n) {
                // the stage being refilled was read (by ldmatrix) in the iteration before this one
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                issue_tile(tb + warp + (it + DSTAGES - 1) * DW, (it + DSTAGES - 1) % DSTAGES);
            }
            if (!mbar_wait(smem_u32(bars + stage), (it / DSTAGES) & 1)) { timed_out = true; break; }
        } else {
            if (it + 1 < my_n) { load_tile(tb + warp + (it + 1) * DW, stage ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
            __syncwarp();
        }
        const uint32_t kb = smem_u32(wbase + stage * 2 * TILE_BYTES), vb = kb + TILE_BYTES;
        const int j0 = (tb + warp + it * DW) * DN;
        float s[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
            uint32_t b[4];
            ldsm4(b, kb + (TMA ? tile_off_tma(((lane >> 4) << 3) + (lane & 7), 2 * k + ((lane >> 3) & 1))
                               : tile_off(((lane >> 4) << 3) + (lane & 7), 2 * k + ((lane >> 3) & 1))));
            mma16816(s[0], qf[k], b[0], b[1]);
            mma16816(s[1], qf[k], b[2], b[3]);
        }
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + n * 8 + 2 * t + (e & 1);
                const bool vis = j <= pos && j >= k_first;
                const float v = vis ? s[n][e] * p.scale_log2 : NEG_BIG;
                s[n][e] = v;
                if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);
        m0 = mx0; m1 = mx1;
        uint32_t pf[4];
        float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
            const float p00 = s[n][0] > 0.5f * NEG_BIG ? exp2f(s[n][0] - mx0) : 0.0f;
            const float p01 = s[n][1] > 0.5f * NEG_BIG ? exp2f(s[n][1] - mx0) : 0.0f;
            const float p10 = s[n][2] > 0.5f * NEG_BIG ? exp2f(s[n][2] - mx1) : 0.0f;
            const float p11 = s[n][3] > 0.5f * NEG_BIG ? exp2f(s[n][3] - mx1) : 0.0f;
            rs0 += p00 + p01;
            rs1 += p10 + p11;
            pf[n * 2 + 0] = pack_bf16(p00, p01);
            pf[n * 2 + 1] = pack_bf16(p10, p11);
        }
        l0 = l0 * c0 + rs0;
        l1 = l1 * c1 + rs1;
        if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {      // the maximum moved somewhere in the warp
#pragma unroll
            for (int n = 0; n < HD / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        }
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
            uint32_t b[4];
            ldsm4t(b, vb + (TMA ? tile_off_tma((lane & 7) + ((lane >> 3) & 1) * 8, 2 * n2 + (lane >> 4))
                                : tile_off((lane & 7) + ((lane >> 3) & 1) * 8, 2 * n2 + (lane >> 4))));
            mma16816(o[2 * n2], pf, b[0], b[1]);
            mma16816(o[2 * n2 + 1], pf, b[2], b[3]);
        }
        __syncwarp();
    }
    if (timed_out && lane == 0) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    // ---- merge the warps: each warp's (m, l, o) -> shared memory (its own K/V stages are free now)
    __syncthreads();
    float* wo = reinterpret_cast<float*>(wbase);         // [16][HD] floats = 64*HD bytes <= WARP_BYTES
    if (t == 0) { s_m[warp][g] = m0; s_m[warp][g + 8] = m1; s_l[warp][g] = l0; s_l[warp][g + 8] = l1; }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        wo[g * HD + n * 8 + 2 * t] = o[n][0];
        wo[g * HD + n * 8 + 2 * t + 1] = o[n][1];
        wo[(g + 8) * HD + n * 8 + 2 * t] = o[n][2];
        wo[(g + 8) * HD + n * 8 + 2 * t + 1] = o[n][3];
    }
    __syncthreads();
    // thread i handles element(s) (row, d): row = e / HD
    const int unit = blockIdx.z * gridDim.y + blockIdx.y;
    const int extra = WITH_PREFIX ? x.extra_slices : 0;
    const int unit_stride = ns_stride + extra;
    float* part = ns + extra > 1 ? x.scratch + ((size_t)unit * unit_stride + split) * (16 * (HD + 2)) : nullptr;
    for (int e = threadIdx.x; e < heads * HD; e += 32 * DW) {
        const int r = e / HD, d = e - r * HD;
        float gm = NEG_BIG;
#pragma unroll
        for (int w = 0; w < DW; ++w) gm = fmaxf(gm, s_m[w][r]);
        float acc = 0.0f, sum = 0.0f;
#pragma unroll
        for (int w = 0; w < DW; ++w) {
            const float f = s_l[w][r] > 0.0f ? exp2f(s_m[w][r] - gm) : 0.0f;
            acc = fmaf(reinterpret_cast<float*>(smem + w * WARP_BYTES)[r * HD + d], f, acc);
            sum = fmaf(s_l[w][r], f, sum);
        }
        if (part) {
            part[r * (HD + 2) + 2 + d] = acc;
            if (d == 0) { part[r * (HD + 2)] = gm; part[r * (HD + 2) + 1] = sum; }
        } else {
            p.out[((size_t)tok * p.nh + head0 + r) * HD + d] = __float2bfloat16_rn(sum > 0.0f ? acc / sum : 0.0f);
        }
    }
    if (!part) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(x.counters + unit, 1);
    __syncthreads();
    if (s_ticket != ns - 1) return;
    __threadfence();
    if (threadIdx.x == 0) x.counters[unit] = 0;
    // The last CTA of this token and head group merges the slices, in slice order.  The loads of
    // several slices and elements are issued together: this part runs alone, so what it costs is
    // the number of dependent round trips to the L2 cache.
    const float* all = x.scratch + (size_t)unit * unit_stride * (16 * (HD + 2));
    const int nt = ns + extra;                                 // this kernel's slices, then the other kernel's
    auto slot = [&](int sp) { return sp < ns ? sp : ns_stride + (sp - ns); };
    __shared__ float s_f[MAX_SPLITS][16];
    __shared__ float s_l2[MAX_SPLITS][16];
    __shared__ float s_inv[16];
    for (int i = threadIdx.x; i < nt * 16; i += 32 * DW) {
        const int sp = i >> 4, r = i & 15;
        const float* ps = all + (size_t)slot(sp) * 16 * (HD + 2) + r * (HD + 2);
        s_f[sp][r] = r < heads ? __ldcg(ps) : NEG_BIG;          // the slice's maximum
        s_l2[sp][r] = r < heads ? __ldcg(ps + 1) : 0.0f;        // and its sum
    }
    __syncthreads();
    if (threadIdx.x < heads) {
        const int r = threadIdx.x;
        float gm = NEG_BIG;
        for (int sp = 0; sp < nt; ++sp) gm = fmaxf(gm, s_f[sp][r]);
        float sum = 0.0f;
        for (int sp = 0; sp < nt; ++sp) {
            const float l = s_l2[sp][r];
            const float f = l > 0.0f ? exp2f(s_f[sp][r] - gm) : 0.0f;
            s_f[sp][r] = f;
            sum = fmaf(l, f, sum);
        }
        s_inv[r] = sum > 0.0f ? 1.0f / sum : 0.0f;
    }
    __syncthreads();
    constexpr int EG = 4, SG = 8;                                // elements and slices per round of loads
    const int total = heads * HD;
    for (int e0 = threadIdx.x; e0 < total; e0 += 32 * DW * EG) {
        float acc[EG];
#pragma unroll
        for (int k = 0; k < EG; ++k) acc[k] = 0.0f;
        for (int s0 = 0; s0 < nt; s0 += SG) {
            float v[EG][SG];
#pragma unroll
            for (int k = 0; k < EG; ++k) {
                const int e = e0 + k * 32 * DW;
                const int r = e / HD, d = e - r * HD;
#pragma unroll
                for (int j = 0; j < SG; ++j)
                    v[k][j] = (e < total && s0 + j < nt)
                                  ? __ldcg(all + (size_t)slot(s0 + j) * 16 * (HD + 2) + r * (HD + 2) + 2 + d) : 0.0f;
            }
#pragma unroll
            for (int k = 0; k < EG; ++k) {
                const int e = e0 + k * 32 * DW;
                const int r = e < total ? e / HD : 0;
#pragma unroll
                for (int j = 0; j < SG; ++j)
                    if (s0 + j < nt) acc[k] = fmaf(v[k][j], s_f[s0 + j][r], acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < EG; ++k) {
            const int e = e0 + k * 32 * DW;
            if (e < total) {
                const int r = e / HD, d = e - r * HD;
                p.out[((size_t)tok * p.nh + head0 + r) * HD + d] = __float2bfloat16_rn(acc[k] * s_inv[r]);
            }
        }
    }
}

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

// Tensor map of one layer's pages seen as [rows][HD] bfloat16, boxes of 16 rows x 64 values.
int kv_map_for(CUtensorMap* out, const void* pool, long long rows) {
    static std::unordered_map<const void*, std::pair<long long, CUtensorMap>> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(pool);
    if (it != cache.end() && it->second.first == rows) { *out = it->second.second; return AIRUN_OK; }
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, DN};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return AIRUN_ERR_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[pool] = std::make_pair(rows, *out);
    return AIRUN_OK;
}

AttnParams make_params(const void* q, void* out, const void* pool, const int32_t* block_table, int max_blocks,
                       const int32_t* positions, const int32_t* req_of_token, int num_reqs, int num_pages,
                       int page_size, int nh, int nkv, float scale, int window, int* err) {
    AttnParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.pool = (const __nv_bfloat16*)pool;
    p.block_table = block_table; p.positions = positions; p.req_of_token = req_of_token;
    p.max_blocks = max_blocks; p.num_reqs = num_reqs; p.num_pages = num_pages; p.page_size = page_size;
    p.page_shift = -1;
    for (int sft = 0; sft < 20; ++sft) if ((1 << sft) == page_size) p.page_shift = sft;
    p.nh = nh; p.nkv = nkv; p.G = nh / nkv; p.scale_log2 = scale * LOG2E; p.window = window; p.err = err;
    return p;
}

}  // namespace

AIRUN_EXPORT int airun_attn_head_dim() { return HD; }

// Tokens per prefill tile for a group of G heads.
AIRUN_EXPORT int airun_attn_prefill_tokens_per_tile(int G) { return G > 0 && G <= PM ? PM / G : 0; }

// tiles: [n_tiles] int4 {request, first token row, token count (<= PM / G), 0}.  With n_tiles_dev the
// grid has n_tiles CTAs and those from *n_tiles_dev on (read on the device) leave at once.
AIRUN_EXPORT int airun_attn_prefill(const void* q, void* out, const void* pool, const int32_t* block_table,
                                    int max_blocks, const int32_t* positions, const int32_t* req_of_token,
                                    int num_reqs, int num_pages, int page_size, int nh, int nkv, float scale,
                                    int window, const void* tiles, int n_tiles, const int32_t* n_tiles_dev,
                                    int* err, cudaStream_t stream) {
    if (n_tiles < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > PM || page_size <= 0 || !err) return AIRUN_ERR_ARG;
    if (n_tiles == 0) return AIRUN_OK;
    if (nkv > 65535) return AIRUN_ERR_ARG;
    const AttnParams p = make_params(q, out, pool, block_table, max_blocks, positions, req_of_token, num_reqs,
                                     num_pages, page_size, nh, nkv, scale, window, err);
    const int smem = (PM + 4 * PN) * HD * 2;
    static unsigned long long configured = 0;            // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(attn_prefill_kernel<false>, dim3(n_tiles, nkv), dim3(PTHREADS), smem, stream, p, (const int4*)tiles, n_tiles_dev, SharedArgs{});
    return airun_launch_status();
}

// The shared prefix of a batch of decoded tokens (rows 0 .. n_tok-1 of the batch, whose block tables
// begin with the same pages): keys [0, *k_end_dev) in `slices` slices, results into slots
// n_splits .. n_splits+slices-1 of every (token, KV head, head group) unit of the decode kernel's
// scratch, which has n_splits + slices slots per unit.  airun_attn_decode with k_begin_dev = k_end_dev
// and extra_slices = slices, launched after this on the same stream, does the rest.
AIRUN_EXPORT int airun_attn_shared_prefix(const void* q, const void* pool, const int32_t* block_table, int max_blocks,
                                          const int32_t* positions, const int32_t* req_of_token, int num_reqs,
                                          int num_pages, int page_size, int nh, int nkv, float scale, int n_tok,
                                          const int32_t* k_end_dev, int slices, int n_splits, float* scratch, int* err,
                                          cudaStream_t stream) {
    if (n_tok <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > PM || page_size <= 0 || !err || !k_end_dev ||
        !scratch || slices < 1 || n_splits < 1 || slices + n_splits > MAX_SPLITS)
        return AIRUN_ERR_ARG;
    const AttnParams p = make_params(q, nullptr, pool, block_table, max_blocks, positions, req_of_token, num_reqs,
                                     num_pages, page_size, nh, nkv, scale, 0, err);
    const int per = PM / (nh / nkv);
    const int groups = (n_tok + per - 1) / per;
    if (nkv > 65535 || groups > 65535) return AIRUN_ERR_ARG;
    const int smem = (PM + 4 * PN) * HD * 2;
    static unsigned long long configured = 0;            // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    SharedArgs sh{k_end_dev, n_tok, scratch, n_splits + slices, n_splits};
    airun_launch(attn_prefill_kernel<true>, dim3(slices, nkv, groups), dim3(PTHREADS), smem, stream, p,
                 (const int4*)nullptr, (const int*)nullptr, sh);
    return airun_launch_status();
}

AIRUN_EXPORT long long airun_attn_decode_scratch_floats(int n_rows, int nh, int nkv, int n_splits) {
    const int hgroups = (nh / nkv + 15) / 16;
    return n_splits > 1 ? (long long)n_rows * nkv * hgroups * n_splits * 16 * (HD + 2) : 0;
}

// rows: [n_rows] batch rows (one decoded token each).  counters: [n_rows * nkv * hgroups] ints, zero on entry.
// With n_rows_dev the grid is made for n_rows rows and n_splits slices, but only the first *n_rows_dev rows
// (read on the device) are run, each with its own number of slices (see DecodeExtra); the scratch then needs
// min(n_splits, dyn_slots / (rows x head groups), at least 1) slices per row and head group.
AIRUN_EXPORT int airun_attn_decode(const void* q, void* out, const void* pool, const int32_t* block_table,
                                   int max_blocks, const int32_t* positions, const int32_t* req_of_token,
                                   int num_reqs, int num_pages, int page_size, int nh, int nkv, float scale,
                                   int window, const int32_t* rows, int n_rows, int n_splits, float* scratch,
                                   int* counters, const int32_t* n_rows_dev, int dyn_slots, const int32_t* k_begin_dev,
                                   int extra_slices, int early_ok, int* err, cudaStream_t stream) {
    if (n_rows_dev && (dyn_slots <= 0 || !rows)) return AIRUN_ERR_ARG;
    if (extra_slices < 0 || n_splits + extra_slices > MAX_SPLITS || (extra_slices > 0 && (n_rows_dev || !k_begin_dev || !scratch || !counters)))
        return AIRUN_ERR_ARG;
    if (n_rows < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || n_splits < 1 || n_splits > MAX_SPLITS || !err) return AIRUN_ERR_ARG;
    if (n_splits > 1 && (!scratch || !counters)) return AIRUN_ERR_ARG;
    if (n_rows == 0) return AIRUN_OK;
    const int hgroups = (nh / nkv + 15) / 16;
    if (nkv * hgroups > 65535 || n_rows > 65535) return AIRUN_ERR_ARG;
    const AttnParams p = make_params(q, out, pool, block_table, max_blocks, positions, req_of_token, num_reqs,
                                     num_pages, page_size, nh, nkv, scale, window, err);
    DecodeExtra x{rows, n_splits, scratch, counters, n_rows_dev, dyn_slots, k_begin_dev, extra_slices, early_ok};
    // TMA needs whole 16-key tiles inside one page and 128-byte boxes
    static const bool tma_allowed = !(getenv("AIRUN_ATTN_TMA") && getenv("AIRUN_ATTN_TMA")[0] == '0');
    const bool tma = tma_allowed && (HD % 64 == 0) && p.page_shift >= 4 && encode_fn() != nullptr;
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (tma) {
        const int r = kv_map_for(&map, pool, (long long)num_pages * 2 * nkv * page_size);
        if (r != AIRUN_OK) return r;
    }
    const int stages = tma ? 3 : 2;
    const int smem = DW * stages * 2 * DN * HD * 2 + 16 * HD * 2 + DW * 3 * 8 + 1024;
    static unsigned long long configured[4] = {0, 0, 0, 0};          // one bit per device each
    const bool prefix = extra_slices > 0 || k_begin_dev != nullptr;
    const int which = (tma ? 1 : 0) + (prefix ? 2 : 0);
    auto kern = which == 0 ? attn_decode_kernel<false, false> : which == 1 ? attn_decode_kernel<true, false>
              : which == 2 ? attn_decode_kernel<false, true> : attn_decode_kernel<true, true>;
    if (first_on_device(configured[which])) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(kern, dim3(n_splits, nkv * hgroups, n_rows), dim3(32 * DW), smem, stream, p, x, map);
    return airun_launch_status();
}
