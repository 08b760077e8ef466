// gemm_f32.cu -- strided-batched fp32 GEMM, C_b = A_b · B_b, fp32 FMA accumulation in k order.
//
// The exact-arithmetic companion of the tcgen05 projections: what the reference's CPU classes compute
// with vedic_gemm (include/VedicGEMM.hpp, called from AttentionHead::forward, include/Attention.hpp:221-223,
// 262-266, and MultiHeadAttention::forward, :299) and its GPU model with cuda_gemm in full-precision mode.
// It serves the fp32 form of the multi-head forward (configuration "fp32, seq 512, d_model 1024"), whose
// sizes are small; the 16-bit path on the tensor cores is logos_qkv_project / logos_project(_heads).
//
// 64 x 64 output tile per CTA, 256 threads, 4 x 4 outputs per thread, k in steps of 16 through shared
// memory.  Any M, N, K, leading dimensions and batch strides (0 = operand shared by the whole batch).
#include "common.cuh"

namespace logos {
namespace {

constexpr int kT = 64, kTK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, int lda, int64_t sA, const float* __restrict__ B, int ldb, int64_t sB,
                float* __restrict__ C, int ldc, int64_t sC, int M, int N, int K) {
    __shared__ float As[kTK][kT + 1];     // [k][m]
    __shared__ float Bs[kTK][kT];         // [k][n]
    const int bz = blockIdx.z;
    A += (int64_t)bz * sA; B += (int64_t)bz * sB; C += (int64_t)bz * sC;
    const int m0 = blockIdx.y * kT, n0 = blockIdx.x * kT;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kTK) {
        // A tile: 64 rows x 16 k, thread -> (row = tid / 4, k = 4 (tid % 4) .. +3)
        {
            const int r = tid >> 2, kk = (tid & 3) * 4;
            const int m = m0 + r;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int k = k0 + kk + e;
                As[kk + e][r] = (m < M && k < K) ? A[(int64_t)m * lda + k] : 0.0f;
            }
        }
        // B tile: 16 k x 64 columns, thread -> (k = tid / 16, n = 4 (tid % 16) .. +3)
        {
            const int kk = tid >> 4, c = (tid & 15) * 4;
            const int k = k0 + kk;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = n0 + c + e;
                Bs[kk][c + e] = (k < K && n < N) ? B[(int64_t)k * ldb + n] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
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
            if (n < N) C[(int64_t)m * ldc + n] = acc[i][j];
        }
    }
}

}  // namespace

int gemm_f32(logos_ctx* ctx, const float* A, int lda, int64_t strideA, const float* B, int ldb, int64_t strideB,
             float* C, int ldc, int64_t strideC, int M, int N, int K, int batch) {
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0 || batch <= 0 || lda < K || ldb < N || ldc < N)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "gemm_f32: bad pointer, extent or leading dimension");
    if (batch > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "gemm_f32: more than 65535 matrices per call");
    dim3 grid((N + kT - 1) / kT, (M + kT - 1) / kT, batch);
    if (grid.y > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "gemm_f32: M too large");
    gemm_f32_kernel<<<grid, 256, 0, ctx->stream>>>(A, lda, strideA, B, ldb, strideB, C, ldc, strideC, M, N, K);
    LOGOS_LAUNCH_CHECK(ctx, "gemm_f32_kernel");
    return LOGOS_OK;
}

}  // namespace logos
