// Shared helpers of the sm_100a kernels: status codes, typed loads and stores,
// warp and block reductions.  Every entry point is extern "C", takes raw device
// pointers plus sizes and a stream, checks its arguments on the host and returns
// a status the Python side turns into an exception; it never allocates.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>
#include <stdlib.h>

#define AIRUN_OK 0
#define AIRUN_ERR_ARG 1000        // a size or pointer the kernel refuses
#define AIRUN_ERR_UNSUPPORTED 1001

// Bits of the device-side error word kernels set instead of trapping.
#define AIRUN_DEV_BAD_PAGE 1      // a block-table entry outside [0, num_pages)
#define AIRUN_DEV_BAD_REQ 2       // a token naming a request outside the batch
#define AIRUN_DEV_BAD_TOKEN 4     // a token id outside the vocabulary
#define AIRUN_DEV_TIMEOUT 8       // a bounded wait ran out

#define AIRUN_DT_F32 0
#define AIRUN_DT_BF16 1

#define AIRUN_EXPORT extern "C" __attribute__((visibility("default")))

// Programmatic dependent launch: a kernel launched with the attribute may become resident while
// the kernel before it in the stream is still running; it must call pdl_wait() before it touches
// global memory that an earlier kernel writes or reads (the wait returns when the earlier kernels
// have finished and their writes are visible).  Every kernel calls pdl_trigger() first, which lets
// the kernel after it become resident as soon as room is free.  What a kernel does before
// pdl_wait() (shared-memory barriers, tensor-memory allocation, loads of WEIGHTS, which no kernel
// writes) overlaps the tail of the kernel before it.  AIRUN_PDL=0 in the environment turns it off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static thread_local int airun_launch_rc = 0;

static inline bool airun_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("AIRUN_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline void airun_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (airun_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess && airun_launch_rc == 0) airun_launch_rc = (int)e;
}

// The same with thread-block clusters of (1, 1, cluster_z) CTAs (grid.z must be a multiple of it).
template <typename... KArgs, typename... Args>
static inline void airun_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                        unsigned cluster_z, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z;
    ++n;
    if (airun_pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess && airun_launch_rc == 0) airun_launch_rc = (int)e;
}

static inline int airun_launch_status() {
    cudaError_t e = cudaGetLastError();
    int rc = airun_launch_rc;
    airun_launch_rc = 0;
    if (rc) return rc;
    return e == cudaSuccess ? AIRUN_OK : (int)e;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();               // `red` may still be read from an earlier call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

static inline int ceil_div_i(long long a, long long b) { return (int)((a + b - 1) / b); }

// True the first time it is asked on the current device (``mask``: one bit per device, of one kernel).
// cudaFuncSetAttribute holds for one device only, so each kernel is configured once on each.
static inline bool first_on_device(unsigned long long& mask) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if ((mask >> dev) & 1ull) return false;
    mask |= 1ull << dev;
    return true;
}
