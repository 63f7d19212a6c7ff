// Flash attention of prompt portions on the 5th-generation tensor cores, for bfloat16 q and
// pages, one head size per build (-DHD=64 or 128), page sizes that are a power of two >= 16.
//
// One CTA = 128 packed query rows (128/G tokens x the G heads of one KV head) of one request.
// Keys and values come in tiles of 128 keys:
//   warp 0   : one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the K and V
//              tiles, 16 keys (one page or a part of one) per box, into two stages each;
//   warp 1   : allocates tensor memory; one thread issues tcgen05.mma:
//                S_j = Q K_j^T   (M=128, N=128, K=HD)   into one of two S buffers in tensor memory,
//                O  += P_j V_j   (M=128, N=HD,  K=128)  into the O buffer, P_j read from shared memory,
//                                                        V_j as an MN-major operand straight from its tile;
//              S_{j+1} is issued before O_j so the tensor cores work while the softmax of tile j runs;
//   warps 2-9: two threads per query row (its lane of tensor memory), one for each half of the
//              keys of a tile and of the head dimensions: read S_j with tcgen05.ld, mask, running
//              maximum (agreed between the two through shared memory) and sum in float32 (exp2),
//              write P_j as bfloat16 into shared memory in the operand layout.  O accumulates in
//              tensor memory over the tiles; a row of it is rescaled only when the row's maximum
//              has to be raised (by more than 2^8), which is rare after the first tiles.
// Key j is visible to a query at position p iff j <= p and (window == 0 or p - j < window); tiles
// wholly hidden are skipped.  Formulas as the reference's prefill kernel computes them
// (crates/airun-cuda/kernels/ops.cu:1796-2078: scale * log2(e) folded, exp2, float32 statistics,
// probabilities rounded to 16 bits for the second product).
//
// Every mbarrier wait is bounded (about two seconds); on a time-out the kernel sets an error
// bit, stops working, frees its tensor memory and returns.  No cluster, no multicast.
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <utility>
#include <cstring>

#ifndef HD
#error "compile with -DHD=64 or -DHD=128"
#endif
static_assert(HD == 64 || HD == 128, "this kernel is built for head_dim 64 or 128");

#define QM 128                    // packed query rows per CTA
#define KN 128                    // keys per tile
#define HALVES (HD / 64)          // 64-value (128-byte) column blocks of a head
#define ROWBLK (128 * 128)        // bytes of one 128-row x 128-byte block
#define TC_THREADS 320
#define NEG_BIG (-1.0e30f)
#define LOG2E 1.4426950408889634f
#define WAIT_NS 2000000000ull

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t1 - t0 > WAIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
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
// the A operand in tensor memory (rows on the lanes, two 16-bit values per column)
__device__ __forceinline__ void umma_bf16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with each descriptor as (low word, high word).  The low word holds the start address in units of 16
// bytes (shared memory ends below 2^18, so adding an offset never carries out of the field): a step along K is
// one 32-bit add on a value computed once, which keeps the issuing thread, that shares its scheduler with two
// softmax warps, ahead of the tensor cores.
__device__ __forceinline__ void umma_bf16_lh(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_bf16_ta_lh(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 columns of this thread's lane -> tensor memory
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// two loads in flight, one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* v) {
    uint32_t r[64];
#define LD32(base, off) \
    asm volatile( \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 " \
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15," \
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];" \
        : "=r"(r[off + 0]), "=r"(r[off + 1]), "=r"(r[off + 2]), "=r"(r[off + 3]), "=r"(r[off + 4]), "=r"(r[off + 5]), \
          "=r"(r[off + 6]), "=r"(r[off + 7]), "=r"(r[off + 8]), "=r"(r[off + 9]), "=r"(r[off + 10]), "=r"(r[off + 11]), \
          "=r"(r[off + 12]), "=r"(r[off + 13]), "=r"(r[off + 14]), "=r"(r[off + 15]), "=r"(r[off + 16]), "=r"(r[off + 17]), \
          "=r"(r[off + 18]), "=r"(r[off + 19]), "=r"(r[off + 20]), "=r"(r[off + 21]), "=r"(r[off + 22]), "=r"(r[off + 23]), \
          "=r"(r[off + 24]), "=r"(r[off + 25]), "=r"(r[off + 26]), "=r"(r[off + 27]), "=r"(r[off + 28]), "=r"(r[off + 29]), \
          "=r"(r[off + 30]), "=r"(r[off + 31]) \
        : "r"(base))
    LD32(taddr, 0);
    LD32(taddr + 32, 32);
#undef LD32
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// K-major operand (rows of 128 bytes, 128-byte swizzle): 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand: 64 values of the N dimension are contiguous (128 bytes), the next 64 are a whole
// 128-row block further (leading byte offset); along K, rows are 128 bytes apart and 8-row groups 1024
// bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)(ROWBLK >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

struct TcParams {
    const __nv_bfloat16* q;        // [T][nh][HD]
    __nv_bfloat16* out;            // [T][nh][HD]
    const int32_t* block_table;    // [R][max_blocks]
    const int32_t* positions;      // [T]
    int max_blocks, num_pages, page_size, page_shift, nh, nkv, G;
    float scale_log2;
    int window;
    int* err;
};

// shared memory map (after 1024-byte alignment)
constexpr int Q_BYTES = HALVES * ROWBLK;           // Q tile, K-major
constexpr int KV_BYTES = HALVES * ROWBLK;          // one K or V tile
constexpr int P_BYTES = 2 * ROWBLK;                // P tile: 128 rows x 128 keys
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;             // 2 stages
constexpr int OFF_V = OFF_K + 2 * KV_BYTES;        // 2 stages
constexpr int OFF_P = OFF_V + 2 * KV_BYTES;
constexpr int OFF_XM = OFF_P + P_BYTES;             // row maxima exchanged between the two warpgroups
constexpr int OFF_BAR = OFF_XM + 2 * 2 * 128 * 4;
constexpr int N_BARS = 16;
constexpr int SMEM_TOTAL = OFF_BAR + N_BARS * 8 + 64 + 1024;
enum { B_KFULL = 0, B_KEMPTY = 2, B_VFULL = 4, B_VEMPTY = 6, B_SFULL = 8, B_SFREE = 10, B_PFULL = 12, B_OFULL = 13, B_OFREE = 14, B_XM = 15 };

// SHARED: the same loop over a prefix of keys that the decoded tokens of a batch have in common (their
// requests begin with the same pages).  The batch's tokens, 128 / G to a CTA (blockIdx.z), are the
// packed rows; all keys below *k_end_dev are visible to all of them; blockIdx.x picks one of gridDim.x
// slices of those keys; and instead of an output row each thread writes its row's (maximum, sum,
// unnormalised output) into the slice's slot of the decode kernel's scratch (attention_mma.cu), which
// merges them with the slices of each token's own keys.
struct TcShared {
    const int32_t* k_end_dev;   // keys [0, *k_end_dev) are shared
    const int32_t* req_of_token;
    int n_tok, num_reqs;        // tokens in the batch (rows 0 .. n_tok-1)
    float* scratch;             // the decode kernel's partial results: [unit][unit_stride][16][HD + 2]
    int unit_stride, slot0;     // slots per (token, KV head, head group); first slot of this kernel's slices
};

template <bool SHARED>
__global__ __launch_bounds__(TC_THREADS, 1) void attn_prefill_tc_kernel(
    const TcParams p, const int4* __restrict__ tiles, const __grid_constant__ CUtensorMap kv_map,
    const int* __restrict__ n_tiles_dev, const TcShared sh) {
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + OFF_BAR);
    uint32_t* tmem_slot = (uint32_t*)(bars + N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(BAR(i), 1);                 // K/V full and empty
        mbar_init(BAR(B_SFULL), 1); mbar_init(BAR(B_SFULL + 1), 1);
        mbar_init(BAR(B_SFREE), 8); mbar_init(BAR(B_SFREE + 1), 8);      // one arrival per softmax warp
        mbar_init(BAR(B_PFULL), 8);
        mbar_init(BAR(B_OFULL), 1);
        mbar_init(BAR(B_OFREE), 8);
        mbar_init(BAR(B_XM), 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    // Blocks are handed out in the order of their linear index, and the work list has the tiles with the most
    // keys first: so the linear index counts the KV heads of a tile before it moves on to the next tile, and
    // the long tiles of ALL heads start first (with the head as the slow index the long tiles of the last
    // heads started last, on top of a machine already half done).
    const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const int tile_idx = SHARED ? (int)blockIdx.x : lin / (int)gridDim.y;
    if (!SHARED && n_tiles_dev && tile_idx >= *n_tiles_dev) {       // a CTA beyond the tiles in use: nothing to do
        tc_fence_before();
        __syncthreads();
        if (warp == 1) {
            tc_fence_after();
            tmem_dealloc(tmem_base, 512);
        }
        return;
    }

    const int G = p.G;
    int req, tok0, n_tok;
    if (SHARED) {
        const int per = QM / G;
        tok0 = blockIdx.z * per;
        n_tok = min(per, sh.n_tok - tok0);
        req = sh.req_of_token[tok0];
    } else {
        const int4 t4 = tiles[tile_idx];
        req = t4.x; tok0 = t4.y; n_tok = t4.z;
    }
    const int kvh = SHARED ? (int)blockIdx.y : lin % (int)gridDim.y;
    const int n_rows = n_tok * G;
    const bool req_ok = !SHARED || (req >= 0 && req < sh.num_reqs);      // (a padded batch: rows of no request)
    const int32_t* bt = p.block_table + (size_t)(req_ok ? req : 0) * p.max_blocks;
    const int k_end = SHARED ? (req_ok ? *sh.k_end_dev : 0) : 0;
    const int pos_lo = SHARED ? k_end - 1 : p.positions[tok0], pos_hi = SHARED ? k_end - 1 : p.positions[tok0 + n_tok - 1];
    const int k_first = (!SHARED && p.window > 0) ? max(0, pos_lo - p.window + 1) : 0;
    int tile_first = k_first / KN;
    int n_tiles = pos_hi >= 0 ? pos_hi / KN - tile_first + 1 : 0;
    if (SHARED) {                                     // this CTA's slice of the shared tiles
        const int per_slice = (n_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
        tile_first = min(n_tiles, (int)blockIdx.x * per_slice);
        n_tiles = min(n_tiles, tile_first + per_slice) - tile_first;
    }

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const int j0 = (tile_first + it) * KN;
                // K tile
                if (!mbar_wait(BAR(B_KEMPTY + s), ph ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
                mbar_expect_tx(BAR(B_KFULL + s), KV_BYTES);
                const uint32_t kdst = smem_u32(smem + OFF_K + s * KV_BYTES);
                int rows[KN / 16];
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey) {
                    const int j = j0 + gkey * 16;
                    const int blk = j >> p.page_shift;
                    int page = (j <= pos_hi && blk < p.max_blocks) ? __ldg(bt + blk) : 0;
                    if (page < 0 || page >= p.num_pages) {
                        if (j >= k_first) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);      // a page the window has passed may be gone
                        page = 0;
                    }
                    rows[gkey] = (((page * 2) * p.nkv + kvh) << p.page_shift) + (j & (p.page_size - 1));
                }
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(kdst + h * ROWBLK + gkey * 2048, &kv_map, BAR(B_KFULL + s), h * 64, rows[gkey]);
                // V tile
                if (!mbar_wait(BAR(B_VEMPTY + s), ph ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
                mbar_expect_tx(BAR(B_VFULL + s), KV_BYTES);
                const uint32_t vdst = smem_u32(smem + OFF_V + s * KV_BYTES);
                const int vskip = p.nkv << p.page_shift;
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(vdst + h * ROWBLK + gkey * 2048, &kv_map, BAR(B_VFULL + s), h * 64, rows[gkey] + vskip);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KN >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
            const uint32_t q_addr = smem_u32(smem + OFF_Q), p_addr = smem_u32(smem + OFF_P);
            bool ok = mbar_wait(BAR(B_PFULL), 0);          // first phase of P_full: the Q tile is in shared memory
            auto issue_s = [&](int it) -> bool {
                const int s = it & 1;
                if (!mbar_wait(BAR(B_KFULL + s), (it >> 1) & 1)) return false;
                if (!mbar_wait(BAR(B_SFREE + s), ((it >> 1) & 1) ^ 1)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(smem + OFF_K + s * KV_BYTES);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (k >> 2) * ROWBLK + (k & 3) * 32;
                    umma_bf16(tmem_base + s * KN, desc_kmajor(q_addr + off), desc_kmajor(k_addr + off), idesc_s, k > 0 ? 1u : 0u);
                }
                umma_commit(BAR(B_KEMPTY + s));
                umma_commit(BAR(B_SFULL + s));
                return true;
            };
            if (ok && n_tiles > 0) ok = issue_s(0);          // (a slice of a shared prefix may be empty)
            for (int it = 0; it < n_tiles && ok; ++it) {
                if (it + 1 < n_tiles) { ok = issue_s(it + 1); if (!ok) break; }
                const int s = it & 1;
                // P_it is in shared memory (phase it + 1 of P_full) and the O buffer has been read
                if (!mbar_wait(BAR(B_PFULL), (it + 1) & 1)) { ok = false; break; }
                if (!mbar_wait(BAR(B_VFULL + s), (it >> 1) & 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(smem + OFF_V + s * KV_BYTES);
#pragma unroll
                for (int k = 0; k < KN / 16; ++k) {              // O accumulates over the tiles in tensor memory
                    const uint32_t poff = (k >> 2) * ROWBLK + (k & 3) * 32;
                    umma_bf16(tmem_base + 2 * KN, desc_kmajor(p_addr + poff), desc_mnmajor(v_addr + k * 2048), idesc_o,
                              (it > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(BAR(B_VEMPTY + s));
                umma_commit(BAR(B_OFULL));
            }
            if (!ok) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        }
    } else {
        // ------------------------------------------------ softmax, correction, epilogue
        // Two warpgroups share the 128 rows: thread (half, r) owns row r (its lane of tensor memory), the
        // keys [64*half, 64*half+64) of every S tile and the head dimensions [DPT*half, DPT*half+DPT) of
        // the output.  The two threads of a row agree on the row's maximum through shared memory.
        const int half = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const bool row_ok = r < n_rows;
        const int tok = tok0 + (row_ok ? r / G : 0);
        const int head = kvh * G + (row_ok ? r % G : 0);
        const int pos = row_ok ? (SHARED ? pos_hi : p.positions[tok]) : -1;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        constexpr int DPT = HD / 2;                               // head dimensions per thread
        float* xm = reinterpret_cast<float*>(smem + OFF_XM);      // [2 tiles][2 halves][128 rows]

        // this thread's part of the Q row -> shared memory in the K-major swizzled layout
        {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)tok * p.nh + head) * HD);
#pragma unroll
            for (int i = 0; i < DPT / 8; ++i) {
                const int c = half * (DPT / 8) + i;
                const uint4 v = row_ok ? src[c] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(smem + OFF_Q + (c >> 3) * ROWBLK + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B_PFULL));          // phase 0: Q is ready
        }

        // The output accumulates in tensor memory.  A row's running maximum is only raised when the
        // new maximum exceeds it by more than 2^8 (probabilities then stay below 256, harmless in
        // float32 and bfloat16); raising it means rescaling the row of O, which is rare after the
        // first tiles, so the product of one tile overlaps the softmax of the next.
        float m = NEG_BIG, l = 0.0f;
        bool ok = true;
        const float sc = p.scale_log2;
        for (int it = 0; it < n_tiles && ok; ++it) {
            const int s = it & 1;
            const int j0 = (tile_first + it) * KN + half * 64;           // first key of this thread's columns
            if (!mbar_wait(BAR(B_SFULL + s), (it >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            // every key of the tile is visible to every row: no masks
            const bool full = (SHARED || p.window == 0) && (tile_first + it) * KN + KN - 1 <= pos_lo;
            float v[64];
            tmem_ld64(lane_addr + s * KN + half * 64, v);
            // the S buffer is in registers: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B_SFREE + s));
            float raw = NEG_BIG;
            if (full) {
#pragma unroll
                for (int i = 0; i < 64; ++i) raw = fmaxf(raw, v[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int j = j0 + i;
                    const bool vis = j <= pos && (SHARED || p.window == 0 || pos - j < p.window);
                    v[i] = vis ? v[i] : NEG_BIG;
                    raw = fmaxf(raw, v[i]);
                }
            }
            // the row's maximum over both halves
            float* xmt = xm + (it & 1) * 256;
            xmt[half * 128 + r] = raw;
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B_XM));                   // a bounded wait, unlike bar.sync
            if (!mbar_wait(BAR(B_XM), it & 1)) { ok = false; break; }
            raw = fmaxf(raw, xmt[(half ^ 1) * 128 + r]);
            const float mx = raw > 0.5f * NEG_BIG ? raw * sc : NEG_BIG;
            const bool raise = mx > m + 8.0f;
            bool landed = it == 0;                                   // has the product of the tile before landed?
            if (it == 0) {
                m = mx;                                              // nothing accumulated yet
            } else if (__any_sync(0xffffffffu, raise)) {
                // rescale this warp's rows of O: the product of the tile before must have landed
                if (!mbar_wait(BAR(B_OFULL), (it - 1) & 1)) { ok = false; break; }
                landed = true;
                tc_fence_after();
                const float f = raise ? ex2(m - mx) : 1.0f;
#pragma unroll
                for (int c = 0; c < DPT; c += 32) {
                    float t[32];
                    tmem_ld32(lane_addr + 2 * KN + half * DPT + c, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) t[i] *= f;
                    tmem_st32(lane_addr + 2 * KN + half * DPT + c, t);
                }
                tmem_st_wait();
                l *= f;
                if (raise) m = mx;
            }
            // probabilities -> shared memory (operand layout), row sum.  The P buffer is free once the
            // product of the tile before, which reads it, has landed.
            if (!landed && !mbar_wait(BAR(B_OFULL), (it - 1) & 1)) { ok = false; break; }
            // exp2(v * scale - m) for two values at a time (packed float32 multiply-add and add of
            // sm_100).  A hidden key holds -1e30, which the product sends to exp2(-inf) = 0 without a
            // test; only a row that has seen no key at all (m = -1e30) must not add its -m.
            const float2 sc2 = make_float2(sc, sc);
            const float nm = m > 0.5f * NEG_BIG ? -m : 0.0f;
            const float2 nm2 = make_float2(nm, nm);
            float2 rs2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int q8 = 0; q8 < 8; ++q8) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 e = __ffma2_rn(make_float2(v[q8 * 8 + 2 * i], v[q8 * 8 + 2 * i + 1]), sc2, nm2);
                    const float2 pp = make_float2(ex2(e.x), ex2(e.y));
                    rs2 = __fadd2_rn(rs2, pp);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(pp.x, pp.y);
                    w[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(smem + OFF_P + half * ROWBLK + r * 128 + ((q8 ^ (r & 7)) << 4)) =
                    make_uint4(w[0], w[1], w[2], w[3]);
            }
            const float rs = rs2.x + rs2.y;
            l += rs;
            // P written (and O rescaled if need be): hand over to the MMA thread
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B_PFULL));
        }
        // the output row
        float o[DPT];
#pragma unroll
        for (int d = 0; d < DPT; ++d) o[d] = 0.0f;
        if (ok && n_tiles > 0) {
            if (mbar_wait(BAR(B_OFULL), (n_tiles - 1) & 1)) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < DPT; c += 32) tmem_ld32(lane_addr + 2 * KN + half * DPT + c, o + c);
            } else {
                ok = false;
            }
        }
        // the row's sum is the sum of its two halves
        float* xl = xm + (n_tiles & 1) * 256;
        xl[half * 128 + r] = l;
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(B_XM));
        if (ok && mbar_wait(BAR(B_XM), n_tiles & 1)) l += xl[(half ^ 1) * 128 + r];
        else ok = false;
        if (!ok) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        if (SHARED) {
            // (maximum, sum, unnormalised output) of the row into this slice's slot of the row's unit;
            // each of the row's two threads writes its half of the head dimensions
            if (row_ok) {
                const int hgroups = (G + 15) / 16, hin = r % G;
                const int unit = tok * (p.nkv * hgroups) + kvh * hgroups + hin / 16;
                float* dst = sh.scratch + ((size_t)unit * sh.unit_stride + sh.slot0 + blockIdx.x) * (16 * (HD + 2))
                             + (hin % 16) * (HD + 2);
                if (half == 0) { dst[0] = ok ? m : NEG_BIG; dst[1] = ok ? l : 0.0f; }
#pragma unroll
                for (int d = 0; d < DPT; ++d) dst[2 + half * DPT + d] = ok ? o[d] : 0.0f;
            }
        } else if (row_ok && ok) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)tok * p.nh + head) * HD + half * DPT);
#pragma unroll
            for (int c = 0; c < DPT / 8; ++c) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
                    w[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------------------------------
// The wide variant: one CTA = 256 packed query rows, two Q tiles (A: rows 0-127, B: rows 128-255) that
// share every K and V tile, so a key or value crosses from the L2 cache to the SM once for 256 rows (at
// 128 rows the load of the tiles, not the tensor cores, bounds a long prompt).  Tensor memory holds
// S_A, S_B (128 columns each) and O_A, O_B; P overwrites S in place as packed bfloat16 pairs and is the
// product's A operand from tensor memory, so shared memory holds only Q (two tiles) and two stages each
// of K and V.
//   warp 0    : TMA producer, as above;
//   warp 1    : the products, in the order S_A0 S_B0 | O_A0 S_A1 O_B0 S_B1 | O_A1 S_A2 ...  The tensor
//               cores run them in this order, so S_X(j+1) may overwrite P_X(j) right behind O_X(j), and
//               the barrier that reports S_X(j+1) reports O_X(j) too.  O_X(j) starts on keys 0-63 as soon
//               as their P stands (a barrier of its own), while the softmax still works on keys 64-127;
//   warps 2-5 : softmax of Q tile A, one thread per row (all 128 keys of a tile, all head dimensions);
//   warps 6-9 : the same for Q tile B.  While one warpgroup works on its S tile the tensor cores work
//               for the other.
// A tile of at most 128 rows runs with the B half idle.
constexpr int W_OFF_Q = 0;                              // two Q tiles
constexpr int W_OFF_K = 2 * Q_BYTES;                    // 2 stages
constexpr int W_OFF_V = W_OFF_K + 2 * KV_BYTES;         // 2 stages
constexpr int W_OFF_BAR = W_OFF_V + 2 * KV_BYTES;
constexpr int W_N_BARS = 15;
constexpr int W_SMEM_TOTAL = W_OFF_BAR + W_N_BARS * 8 + 64 + 1024;
enum { W_KFULL = 0, W_KEMPTY = 2, W_VFULL = 4, W_VEMPTY = 6, W_SFULL = 8, W_PFULL = 10, W_FINAL = 12, W_PHALF = 13 };

__global__ __launch_bounds__(TC_THREADS, 1) void attn_prefill_wide_kernel(
    const TcParams p, const int4* __restrict__ tiles, const __grid_constant__ CUtensorMap kv_map,
    const int* __restrict__ n_tiles_dev) {
    pdl_trigger();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + W_OFF_BAR);
    uint32_t* tmem_slot = (uint32_t*)(bars + W_N_BARS);
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(BAR(i), 1);                 // K/V full and empty
        mbar_init(BAR(W_SFULL), 1); mbar_init(BAR(W_SFULL + 1), 1);
        mbar_init(BAR(W_PFULL), 4); mbar_init(BAR(W_PFULL + 1), 4);      // one arrival per warp of the tile's warpgroup
        mbar_init(BAR(W_FINAL), 1);
        mbar_init(BAR(W_PHALF), 4); mbar_init(BAR(W_PHALF + 1), 4);      // P of keys 0-63 of a tile
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    // the KV heads of a tile before the next tile: the tiles with the most keys, of all heads, start first
    const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const int tile_idx = lin / (int)gridDim.y;
    if (n_tiles_dev && tile_idx >= *n_tiles_dev) {       // a CTA beyond the tiles in use: nothing to do
        tc_fence_before();
        __syncthreads();
        if (warp == 1) {
            tc_fence_after();
            tmem_dealloc(tmem_base, 512);
        }
        return;
    }

    const int G = p.G;
    const int4 t4 = tiles[tile_idx];
    const int req = t4.x, tok0 = t4.y, n_tok = t4.z;
    const int kvh = lin % (int)gridDim.y;
    const int n_rows = n_tok * G;
    const bool two = n_rows > QM;                       // is there a Q tile B?
    const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
    const int pos_lo = p.positions[tok0], pos_hi = p.positions[tok0 + n_tok - 1];
    const int k_first = p.window > 0 ? max(0, pos_lo - p.window + 1) : 0;
    const int tile_first = k_first / KN;
    const int n_tiles = pos_hi >= 0 ? pos_hi / KN - tile_first + 1 : 0;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it & 1;
                const uint32_t ph = (it >> 1) & 1;
                const int j0 = (tile_first + it) * KN;
                if (!mbar_wait(BAR(W_KEMPTY + s), ph ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
                mbar_expect_tx(BAR(W_KFULL + s), KV_BYTES);
                const uint32_t kdst = smem_u32(smem + W_OFF_K + s * KV_BYTES);
                int rows[KN / 16];
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey) {
                    const int j = j0 + gkey * 16;
                    const int blk = j >> p.page_shift;
                    int page = (j <= pos_hi && blk < p.max_blocks) ? __ldg(bt + blk) : 0;
                    if (page < 0 || page >= p.num_pages) {
                        if (j >= k_first) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);      // a page the window has passed may be gone
                        page = 0;
                    }
                    rows[gkey] = (((page * 2) * p.nkv + kvh) << p.page_shift) + (j & (p.page_size - 1));
                }
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(kdst + h * ROWBLK + gkey * 2048, &kv_map, BAR(W_KFULL + s), h * 64, rows[gkey]);
                if (!mbar_wait(BAR(W_VEMPTY + s), ph ^ 1)) { atomicOr(p.err, AIRUN_DEV_TIMEOUT); break; }
                mbar_expect_tx(BAR(W_VFULL + s), KV_BYTES);
                const uint32_t vdst = smem_u32(smem + W_OFF_V + s * KV_BYTES);
                const int vskip = p.nkv << p.page_shift;
#pragma unroll
                for (int gkey = 0; gkey < KN / 16; ++gkey)
#pragma unroll
                    for (int h = 0; h < HALVES; ++h)
                        tma_load_2d(vdst + h * ROWBLK + gkey * 2048, &kv_map, BAR(W_VFULL + s), h * 64, rows[gkey] + vskip);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KN >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
            constexpr uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QM >> 4) << 24);
            const int last_x = two ? 1 : 0;
            // descriptors of the first Q, K and V tiles; the others and the steps along K are offsets of the low word
            const uint64_t qd = desc_kmajor(smem_u32(smem + W_OFF_Q)), kd = desc_kmajor(smem_u32(smem + W_OFF_K)),
                           vd = desc_mnmajor(smem_u32(smem + W_OFF_V));
            const uint32_t q_lo = (uint32_t)qd, q_hi = (uint32_t)(qd >> 32), k_lo = (uint32_t)kd, k_hi = (uint32_t)(kd >> 32),
                           v_lo = (uint32_t)vd, v_hi = (uint32_t)(vd >> 32);
            // first phase of P_full: the Q tiles are in shared memory
            bool ok = mbar_wait(BAR(W_PFULL), 0) && (!two || mbar_wait(BAR(W_PFULL + 1), 0));
            auto issue_s = [&](int it, int x) -> bool {          // S of Q tile x and key tile it
                const int s = it & 1;
                if (x == 0) {
                    if (!mbar_wait(BAR(W_KFULL + s), (it >> 1) & 1)) return false;
                    tc_fence_after();
                }
                const uint32_t qx = q_lo + x * (Q_BYTES >> 4), ks = k_lo + s * (KV_BYTES >> 4), d = tmem_base + x * KN;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = ((k >> 2) * ROWBLK + (k & 3) * 32) >> 4;
                    umma_bf16_lh(d, qx + off, q_hi, ks + off, k_hi, idesc_s, k > 0 ? 1u : 0u);
                }
                if (x == last_x) umma_commit(BAR(W_KEMPTY + s));
                umma_commit(BAR(W_SFULL + x));
                return true;
            };
            auto issue_o = [&](int it, int x) -> bool {          // O of Q tile x += P V of key tile it
                const int s = it & 1;
                if (!mbar_wait(BAR(W_PHALF + x), it & 1)) return false;           // P of keys 0-63 stands where S stood
                if (x == 0 && !mbar_wait(BAR(W_VFULL + s), (it >> 1) & 1)) return false;
                tc_fence_after();
                const uint32_t vs = v_lo + s * (KV_BYTES >> 4), d = tmem_base + (2 + x) * KN, pa = tmem_base + x * KN;
                const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
                for (int k = 0; k < KN / 32; ++k)                // 16 keys of P = 8 columns of packed pairs
                    umma_bf16_ta_lh(d, pa + k * 8, vs + k * (2048 >> 4), v_hi, idesc_o, k > 0 ? 1u : acc0);
                if (!mbar_wait(BAR(W_PFULL + x), (it + 1) & 1)) return false;     // and of keys 64-127
                tc_fence_after();
#pragma unroll
                for (int k = KN / 32; k < KN / 16; ++k)
                    umma_bf16_ta_lh(d, pa + k * 8, vs + k * (2048 >> 4), v_hi, idesc_o, 1u);
                if (x == last_x) umma_commit(BAR(W_VEMPTY + s));
                return true;
            };
            if (ok && n_tiles > 0) {
                ok = issue_s(0, 0);
                if (ok && two) ok = issue_s(0, 1);
            }
            for (int it = 0; it < n_tiles && ok; ++it) {
                ok = issue_o(it, 0);
                if (ok && it + 1 < n_tiles) ok = issue_s(it + 1, 0);
                if (ok && two) {
                    ok = issue_o(it, 1);
                    if (ok && it + 1 < n_tiles) ok = issue_s(it + 1, 1);
                }
            }
            if (ok) umma_commit(BAR(W_FINAL));
            else atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        }
    } else if (two || warp < 6) {
        // ------------------------------------------------ softmax, correction, epilogue
        const int x = (warp - 2) >> 2;                    // this warpgroup's Q tile
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                   // the thread's lane of tensor memory
        const int row = x * QM + r;
        const bool row_ok = row < n_rows;
        const int tok = tok0 + (row_ok ? row / G : 0);
        const int head = kvh * G + (row_ok ? row % G : 0);
        const int pos = row_ok ? p.positions[tok] : -1;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_addr = lane_addr + x * KN, o_addr = lane_addr + (2 + x) * KN;

        // the Q row -> shared memory in the K-major swizzled layout
        {
            const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)tok * p.nh + head) * HD);
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                const uint4 v = row_ok ? src[c] : make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(smem + W_OFF_Q + x * Q_BYTES + (c >> 3) * ROWBLK + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(W_PFULL + x));          // phase 0: Q is ready
        }

        float m = NEG_BIG, l = 0.0f;
        bool ok = true;
        const float sc = p.scale_log2;
        for (int it = 0; it < n_tiles && ok; ++it) {
            // S of this key tile has landed, and with it the product of the tile before
            if (!mbar_wait(BAR(W_SFULL + x), it & 1)) { ok = false; break; }
            tc_fence_after();
            const int j0 = (tile_first + it) * KN;
            const bool full = p.window == 0 && j0 + KN - 1 <= pos_lo;       // every key visible to every row: no masks
            float v[64];
            // the row's maximum, as four chains that the scheduler can interleave: keys 64-127, then keys 0-63,
            // which stay in registers
            float r0 = NEG_BIG, r1 = NEG_BIG, r2 = NEG_BIG, r3 = NEG_BIG;
#pragma unroll
            for (int c = 1; c >= 0; --c) {
                tmem_ld64(s_addr + c * 64, v);
                if (!full) {
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int j = j0 + c * 64 + i;
                        const bool vis = j <= pos && (p.window == 0 || pos - j < p.window);
                        v[i] = vis ? v[i] : NEG_BIG;
                    }
                }
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    r0 = fmaxf(r0, v[i]); r1 = fmaxf(r1, v[i + 1]); r2 = fmaxf(r2, v[i + 2]); r3 = fmaxf(r3, v[i + 3]);
                }
            }
            const float raw = fmaxf(fmaxf(r0, r1), fmaxf(r2, r3));
            const float mx = raw > 0.5f * NEG_BIG ? raw * sc : NEG_BIG;
            const bool raise = mx > m + 8.0f;
            if (it == 0) {
                m = mx;                                              // nothing accumulated yet
            } else if (__any_sync(0xffffffffu, raise)) {
                // rescale this warp's rows of O
                const float f = raise ? ex2(m - mx) : 1.0f;
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    float t[32];
                    tmem_ld32(o_addr + c, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) t[i] *= f;
                    tmem_st32(o_addr + c, t);
                }
                l *= f;
                if (raise) m = mx;
            }
            // probabilities as pairs of bfloat16 over the S tile (keys 2c, 2c+1 in column c), row sum.
            // A hidden key holds -1e30, which the product sends to exp2(-inf) = 0 without a test; only a
            // row that has seen no key at all (m = -1e30) must not add its -m.
            const float2 sc2 = make_float2(sc, sc);
            const float nm = m > 0.5f * NEG_BIG ? -m : 0.0f;
            const float2 nm2 = make_float2(nm, nm);
            float2 rs2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                if (c == 1) {                                        // keys 64-127 again (their columns are untouched)
                    tmem_ld64(s_addr + 64, v);
                    if (!full) {
#pragma unroll
                        for (int i = 0; i < 64; ++i) {
                            const int j = j0 + 64 + i;
                            const bool vis = j <= pos && (p.window == 0 || pos - j < p.window);
                            v[i] = vis ? v[i] : NEG_BIG;
                        }
                    }
                }
                uint32_t pw[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float2 e = __ffma2_rn(make_float2(v[2 * i], v[2 * i + 1]), sc2, nm2);
                    const float2 pp = make_float2(ex2(e.x), ex2(e.y));
                    rs2 = __fadd2_rn(rs2, pp);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(pp.x, pp.y);
                    pw[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                tmem_st32u(s_addr + c * 32, pw);
                if (c == 0) {                                        // the product may start on keys 0-63
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(W_PHALF + x));
                }
            }
            tmem_st_wait();
            l += rs2.x + rs2.y;
            // P written (and O rescaled if need be): hand over to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(W_PFULL + x));
        }
        // the output row
        if (ok && n_tiles > 0 && !mbar_wait(BAR(W_FINAL), 0)) ok = false;
        if (!ok) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        tc_fence_after();
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        uint4* dst = reinterpret_cast<uint4*>(p.out + ((size_t)tok * p.nh + head) * HD);
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
            float o[32];
            if (ok && n_tiles > 0) {
                tmem_ld32(o_addr + c, o);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = 0.0f;
            }
            if (row_ok && ok) {
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[q8 * 8 + 2 * i] * inv, o[q8 * 8 + 2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&h2);
                    }
                    dst[c / 8 + q8] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
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
// One layer's pages seen as [rows][HD] bfloat16, boxes of 16 rows x 64 values.
int kv_map_for(CUtensorMap* out, const void* pool, long long rows) {
    static std::unordered_map<const void*, std::pair<long long, CUtensorMap>> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(pool);
    if (it != cache.end() && it->second.first == rows) { *out = it->second.second; return AIRUN_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return AIRUN_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, 16};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return AIRUN_ERR_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[pool] = std::make_pair(rows, *out);
    return AIRUN_OK;
}

}  // namespace

AIRUN_EXPORT int airun_attn_tc_head_dim() { return HD; }

// tiles: [n_tiles] int4 {request, first token row, token count (<= 128 / G), -}.  Pages must be a
// power of two >= 16 tokens; G = nh / nkv <= 128.  With n_tiles_dev the grid has n_tiles CTAs and
// those from *n_tiles_dev on (read on the device) leave at once.
AIRUN_EXPORT int airun_attn_prefill_tc(const void* q, void* out, const void* pool, const int32_t* block_table,
                                       int max_blocks, const int32_t* positions, int num_pages, int page_size,
                                       int nh, int nkv, float scale, int window, const void* tiles, int n_tiles,
                                       const int32_t* n_tiles_dev, int* err, cudaStream_t stream) {
    if (n_tiles < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > QM || !err) return AIRUN_ERR_ARG;
    int shift = -1;
    for (int s = 4; s < 20; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) return AIRUN_ERR_UNSUPPORTED;
    if (n_tiles == 0) return AIRUN_OK;
    if (nkv > 65535) return AIRUN_ERR_ARG;
    TcParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions;
    p.max_blocks = max_blocks; p.num_pages = num_pages; p.page_size = page_size; p.page_shift = shift;
    p.nh = nh; p.nkv = nkv; p.G = nh / nkv; p.scale_log2 = scale * LOG2E; p.window = window; p.err = err;
    CUtensorMap map;
    const int r = kv_map_for(&map, pool, (long long)num_pages * 2 * nkv * page_size);
    if (r != AIRUN_OK) return r;
    static unsigned long long configured = 0;            // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(attn_prefill_tc_kernel<false>, dim3(n_tiles, nkv), dim3(TC_THREADS), SMEM_TOTAL, stream, p, (const int4*)tiles, map, n_tiles_dev, TcShared{});
    return airun_launch_status();
}

// The same for tiles of up to 256 / G tokens (attn_prefill_wide_kernel).
AIRUN_EXPORT int airun_attn_prefill_wide(const void* q, void* out, const void* pool, const int32_t* block_table,
                                         int max_blocks, const int32_t* positions, int num_pages, int page_size,
                                         int nh, int nkv, float scale, int window, const void* tiles, int n_tiles,
                                         const int32_t* n_tiles_dev, int* err, cudaStream_t stream) {
    if (n_tiles < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > QM || !err) return AIRUN_ERR_ARG;
    int shift = -1;
    for (int s = 4; s < 20; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) return AIRUN_ERR_UNSUPPORTED;
    if (n_tiles == 0) return AIRUN_OK;
    if (nkv > 65535) return AIRUN_ERR_ARG;
    TcParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.positions = positions;
    p.max_blocks = max_blocks; p.num_pages = num_pages; p.page_size = page_size; p.page_shift = shift;
    p.nh = nh; p.nkv = nkv; p.G = nh / nkv; p.scale_log2 = scale * LOG2E; p.window = window; p.err = err;
    CUtensorMap map;
    const int r = kv_map_for(&map, pool, (long long)num_pages * 2 * nkv * page_size);
    if (r != AIRUN_OK) return r;
    static unsigned long long configured = 0;            // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(attn_prefill_wide_kernel, dim3(n_tiles, nkv), dim3(TC_THREADS), W_SMEM_TOTAL, stream, p, (const int4*)tiles, map, n_tiles_dev);
    return airun_launch_status();
}

// The shared prefix of a batch of decoded tokens on tcgen05: see TcShared.  Same contract as
// airun_attn_shared_prefix of attention_mma.cu (slots n_splits .. n_splits+slices-1 of every unit of the
// decode kernel's scratch, n_splits + slices slots per unit).
AIRUN_EXPORT int airun_attn_shared_prefix_tc(const void* q, const void* pool, const int32_t* block_table, int max_blocks,
                                             const int32_t* req_of_token, int num_reqs, int num_pages, int page_size,
                                             int nh, int nkv, float scale, int n_tok, const int32_t* k_end_dev,
                                             int slices, int n_splits, float* scratch, int* err, cudaStream_t stream) {
    if (n_tok <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || nh / nkv > QM || !err || !k_end_dev || !scratch ||
        !req_of_token || slices < 1 || n_splits < 1)
        return AIRUN_ERR_ARG;
    int shift = -1;
    for (int s = 4; s < 20; ++s) if ((1 << s) == page_size) shift = s;
    if (shift < 0) return AIRUN_ERR_UNSUPPORTED;
    TcParams p;
    p.q = (const __nv_bfloat16*)q; p.out = nullptr; p.block_table = block_table; p.positions = nullptr;
    p.max_blocks = max_blocks; p.num_pages = num_pages; p.page_size = page_size; p.page_shift = shift;
    p.nh = nh; p.nkv = nkv; p.G = nh / nkv; p.scale_log2 = scale * LOG2E; p.window = 0; p.err = err;
    const int per = QM / p.G;
    const int groups = (n_tok + per - 1) / per;
    if (nkv > 65535 || groups > 65535) return AIRUN_ERR_ARG;
    CUtensorMap map;
    const int r = kv_map_for(&map, pool, (long long)num_pages * 2 * nkv * page_size);
    if (r != AIRUN_OK) return r;
    static unsigned long long configured = 0;            // one bit per device
    if (first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    TcShared sh{k_end_dev, req_of_token, n_tok, num_reqs, scratch, n_splits + slices, n_splits};
    airun_launch(attn_prefill_tc_kernel<true>, dim3(slices, nkv, groups), dim3(TC_THREADS), SMEM_TOTAL, stream, p,
                 (const int4*)nullptr, map, (const int*)nullptr, sh);
    return airun_launch_status();
}
