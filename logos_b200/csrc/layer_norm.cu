// layer_norm.cu -- the LayerNorm in front of a layer's projections (layernorm_kernel, cuda/VedicGEMM.cu:157-199,
// called per layer at cuda/ModelGPU.cu:772): y = gamma (x - mean) / sqrt(var + eps) + beta with the biased
// variance taken in a second pass over the row, fp32 arithmetic; here on 16-bit activations, one warp per row with
// the row held in registers.  A decode step has 32 rows, so the kernel is all latency: it lets the kernel after it
// start at once (a projection launched to overlap fetches its weights meanwhile) and, when launched to overlap the
// kernel before it, reads gamma and beta first and waits for that kernel before it touches the activations.
#include "common.cuh"

namespace logos {
namespace {

constexpr int kLnMaxChunks = 8;          // 8 x 256 = 2048 values per row at most
constexpr int kLnWarps = 4;

template <typename T> __device__ __forceinline__ float ln_to_f32(T v);
template <> __device__ __forceinline__ float ln_to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ln_to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T ln_from_f32(float v);
template <> __device__ __forceinline__ __half ln_from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 ln_from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_total(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// CHUNKS = ceil(D / 256): lane l owns values [256 c + 8 l, 256 c + 8 l + 8) of every chunk c
template <typename T, int CHUNKS>
__global__ void __launch_bounds__(32 * kLnWarps)
layer_norm_kernel(const T* __restrict__ X, const float* __restrict__ gamma, const float* __restrict__ beta,
                  T* __restrict__ Y, int rows, int D, float eps) {
    grid_release_dependents();
    const int lane = threadIdx.x & 31, row = blockIdx.x * kLnWarps + (threadIdx.x >> 5);
    float g[CHUNKS][8], b[CHUNKS][8];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int at = 256 * c + 8 * lane;
        if (at < D) {
            const float4 g0 = *reinterpret_cast<const float4*>(gamma + at), g1 = *reinterpret_cast<const float4*>(gamma + at + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(beta + at), b1 = *reinterpret_cast<const float4*>(beta + at + 4);
            g[c][0] = g0.x; g[c][1] = g0.y; g[c][2] = g0.z; g[c][3] = g0.w; g[c][4] = g1.x; g[c][5] = g1.y; g[c][6] = g1.z; g[c][7] = g1.w;
            b[c][0] = b0.x; b[c][1] = b0.y; b[c][2] = b0.z; b[c][3] = b0.w; b[c][4] = b1.x; b[c][5] = b1.y; b[c][6] = b1.z; b[c][7] = b1.w;
        }
    }
    grid_wait_for_earlier();
    if (row >= rows) return;
    const T* x = X + (size_t)row * D;
    float v[CHUNKS][8];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int at = 256 * c + 8 * lane;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[c][e] = 0.0f;
        if (at < D) {
            const uint4 w = *reinterpret_cast<const uint4*>(x + at);
            const T* t = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int e = 0; e < 8; ++e) { v[c][e] = ln_to_f32<T>(t[e]); sum += v[c][e]; }
        }
    }
    const float mean = warp_total(sum) / (float)D;
    float sq = 0.0f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        if (256 * c + 8 * lane < D) {
#pragma unroll
            for (int e = 0; e < 8; ++e) { const float d = v[c][e] - mean; sq += d * d; }
        }
    }
    const float inv = rsqrtf(warp_total(sq) / (float)D + eps);
    T* y = Y + (size_t)row * D;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int at = 256 * c + 8 * lane;
        if (at < D) {
            uint4 w;
            T* t = reinterpret_cast<T*>(&w);
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = ln_from_f32<T>(g[c][e] * ((v[c][e] - mean) * inv) + b[c][e]);
            *reinterpret_cast<uint4*>(y + at) = w;
        }
    }
}

template <typename T, int CHUNKS>
int launch_ln(logos_ctx* ctx, const void* X, const float* gamma, const float* beta, void* Y, int rows, int D, float eps) {
    const dim3 grid((rows + kLnWarps - 1) / kLnWarps), block(32 * kLnWarps);
    auto* fn = layer_norm_kernel<T, CHUNKS>;
    if (ctx->project_overlap) {
        LOGOS_CUDA_TRY(ctx, launch_overlapped(fn, grid, block, 0, ctx->stream, static_cast<const T*>(X), gamma, beta,
                                              static_cast<T*>(Y), rows, D, eps));
    } else {
        fn<<<grid, block, 0, ctx->stream>>>(static_cast<const T*>(X), gamma, beta, static_cast<T*>(Y), rows, D, eps);
    }
    LOGOS_LAUNCH_CHECK(ctx, "layer_norm_kernel");
    return LOGOS_OK;
}

template <typename T>
int dispatch_ln(logos_ctx* ctx, const void* X, const float* gamma, const float* beta, void* Y, int rows, int D, float eps) {
    const int chunks = (D + 255) / 256;
    if (chunks <= 1) return launch_ln<T, 1>(ctx, X, gamma, beta, Y, rows, D, eps);
    if (chunks <= 2) return launch_ln<T, 2>(ctx, X, gamma, beta, Y, rows, D, eps);
    if (chunks <= 4) return launch_ln<T, 4>(ctx, X, gamma, beta, Y, rows, D, eps);
    return launch_ln<T, kLnMaxChunks>(ctx, X, gamma, beta, Y, rows, D, eps);
}

}  // namespace

int layer_norm(logos_ctx* ctx, int dtype, const void* X, const float* gamma, const float* beta, void* Y, int rows,
               int D, float eps) {
    if (!X || !gamma || !beta || !Y || rows <= 0 || D <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "layer_norm: bad pointer or extent");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "layer_norm: activations are BF16 or FP16");
    if ((D % 8) != 0 || D > 256 * kLnMaxChunks)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "layer_norm: D = %d (a multiple of 8, at most %d)", D, 256 * kLnMaxChunks);
    if (!aligned16(X) || !aligned16(Y) || !aligned16(gamma) || !aligned16(beta))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "layer_norm: tensors must be 16-byte aligned");
    if (dtype == LOGOS_F16) return dispatch_ln<__half>(ctx, X, gamma, beta, Y, rows, D, eps);
    return dispatch_ln<__nv_bfloat16>(ctx, X, gamma, beta, Y, rows, D, eps);
}

}  // namespace logos
