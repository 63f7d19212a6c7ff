// Plain matrix product C[M][N] = A[M][K] * W[N][K]^T on the CUDA cores.
//
// This is the true 32-bit path of every projection (float32 operands, FFMA
// accumulation, no tensor cores, no reduced-precision mode) and, with bfloat16
// operands, the plain twin the tensor-core kernels are tested against.  The
// reference keeps exact f32 FMA matvecs for the same purpose
// (crates/airun-cuda/kernels/matmul.cu:59-141, switch at
// crates/airun-core/src/runtime.rs:5344-5352).  Every output element is one
// sequential sum over k, so a row's result does not depend on M.
#include "common.cuh"

#define TM 64
#define TN 64
#define TK 16
#define PAD 4

template <typename TA, typename TW, typename TC>
__global__ __launch_bounds__(256) void gemm_simt_kernel(
    const TA* __restrict__ A, const TW* __restrict__ W, TC* __restrict__ C,
    int M, int N, int K, long long lda, long long ldw, long long ldc) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float As[TK][TM + PAD];
    __shared__ __align__(16) float Ws[TK][TN + PAD];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            float a = 0.0f, w = 0.0f;
            if (k < K) {
                if (m0 + lr < M) a = to_f32<TA>(A[(size_t)(m0 + lr) * lda + k]);
                if (n0 + lr < N) w = to_f32<TW>(W[(size_t)(n0 + lr) * ldw + k]);
            }
            As[lk + j][lr] = a;
            Ws[lk + j][lr] = w;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
            const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
        }
    }
}

// dtypes: a_dtype == w_dtype in {f32, bf16}; c_dtype in {f32, bf16}.
AIRUN_EXPORT int airun_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype,
                                 void* C, int c_dtype, int M, int N, int K,
                                 long long lda, long long ldw, long long ldc, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N) return AIRUN_ERR_ARG;
    if (M == 0) return AIRUN_OK;
    dim3 grid(ceil_div_i(N, TN), ceil_div_i(M, TM));
    if (grid.y > 65535) return AIRUN_ERR_ARG;
#define LAUNCH(TA, TW, TC) \
    airun_launch(gemm_simt_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, stream, (const TA*)A, (const TW*)W, (TC*)C, M, N, K, lda, ldw, ldc)
    if (a_dtype == AIRUN_DT_F32 && w_dtype == AIRUN_DT_F32 && c_dtype == AIRUN_DT_F32) LAUNCH(float, float, float);
    else if (a_dtype == AIRUN_DT_BF16 && w_dtype == AIRUN_DT_BF16 && c_dtype == AIRUN_DT_F32) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
    else if (a_dtype == AIRUN_DT_BF16 && w_dtype == AIRUN_DT_BF16 && c_dtype == AIRUN_DT_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef LAUNCH
    return airun_launch_status();
}
