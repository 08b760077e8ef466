// nikhilam.cu -- Nikhilam INT8 KV cache: batched absmax + quantize, dequantize and
// quantize-on-append.
//
// Arithmetic contract (bit-exact with cuda/ModelGPU.cu:293-386 of LOGOS read as
// IEEE fp32):  absmax = max|x| ;  scale = (absmax + 1e-8f) / 127.5f ;
// q = rne(clamp(x / (scale + 1e-8f), -127, 127)) ;  x' = (float)q * scale.
// One scale per tensor.  Everything stays on the device: the reference's blocking
// copy of absmax to the host between the two kernels is gone.
//
// Data movement: every thread moves 16 output bytes per step (one 16-byte store)
// from 16 source values (four 16-byte loads for fp32, two for 16-bit sources), so
// all global accesses are full 16-byte vectors on 16-byte boundaries.
#include "common.cuh"

namespace logos {
namespace {

constexpr int kThreads = 256;

template <typename T> struct Vec16;  // 16 source values as 16-byte vectors
template <> struct Vec16<float> {
    float4 v[4];
    __device__ void load(const float* p) {
        const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __ldg(q + i);
    }
    __device__ float get(int i) const { return reinterpret_cast<const float*>(v)[i]; }
};
template <typename T16> struct Vec16Half {
    uint4 v[2];
    __device__ void load(const T16* p) {
        const uint4* q = reinterpret_cast<const uint4*>(p);
        v[0] = __ldg(q);
        v[1] = __ldg(q + 1);
    }
    __device__ float get(int i) const { return to_f32<T16>(reinterpret_cast<const T16*>(v)[i]); }
};
template <> struct Vec16<__nv_bfloat16> : Vec16Half<__nv_bfloat16> {};
template <> struct Vec16<__half> : Vec16Half<__half> {};

// max|x| per tensor; partial maxima meet in one word per tensor.  Non-negative
// floats order like their bit patterns, so an integer atomicMax is exact, and max
// is order-independent, so any reduction tree gives the reference's value.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const T* __restrict__ src, int64_t src_stride, int64_t elems,
              float* __restrict__ amax) {
    const T* x = src + (int64_t)blockIdx.y * src_stride;
    float m = 0.0f;
    if (VEC) {
        int64_t nvec = elems >> 4;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec;
             i += (int64_t)gridDim.x * kThreads) {
            Vec16<T> v;
            v.load(x + (i << 4));
#pragma unroll
            for (int k = 0; k < 16; ++k) m = fmaxf(m, fabsf(v.get(k)));
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < elems;
             i += (int64_t)gridDim.x * kThreads)
            m = fmaxf(m, fabsf(to_f32<T>(x[i])));
    }
    m = warp_max(m);
    __shared__ float wm[kThreads / 32];
    if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        float r = threadIdx.x < kThreads / 32 ? wm[threadIdx.x] : 0.0f;
        r = warp_max(r);
        if (threadIdx.x == 0)
            atomicMax(reinterpret_cast<unsigned int*>(amax + blockIdx.y), __float_as_uint(r));
    }
}

__device__ __forceinline__ float scale_of(float amax) {
    return __fdiv_rn(__fadd_rn(amax, 1e-8f), 127.5f);
}

__device__ __forceinline__ int quant1(float x, float den) {
    float q = __fdiv_rn(x, den);
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    return __float2int_rn(q);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
quantize_kernel(const T* __restrict__ src, int64_t src_stride, int8_t* __restrict__ dst,
                int64_t dst_stride, const float* __restrict__ amax, float* __restrict__ scales,
                int64_t elems) {
    const T* x = src + (int64_t)blockIdx.y * src_stride;
    int8_t* q = dst + (int64_t)blockIdx.y * dst_stride;
    const float scale = scale_of(amax[blockIdx.y]);
    const float den = __fadd_rn(scale, 1e-8f);
    if (blockIdx.x == 0 && threadIdx.x == 0) scales[blockIdx.y] = scale;
    if (VEC) {
        int64_t nvec = elems >> 4;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec;
             i += (int64_t)gridDim.x * kThreads) {
            Vec16<T> v;
            v.load(x + (i << 4));
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t b0 = (uint32_t)quant1(v.get(4 * k + 0), den) & 0xffu;
                uint32_t b1 = (uint32_t)quant1(v.get(4 * k + 1), den) & 0xffu;
                uint32_t b2 = (uint32_t)quant1(v.get(4 * k + 2), den) & 0xffu;
                uint32_t b3 = (uint32_t)quant1(v.get(4 * k + 3), den) & 0xffu;
                w[k] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
            }
            *reinterpret_cast<uint4*>(q + (i << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < elems;
             i += (int64_t)gridDim.x * kThreads)
            q[i] = (int8_t)quant1(to_f32<T>(x[i]), den);
    }
}

// int8 -> 16-bit: the fp32 product q * scale (the reference's nikhilam_dequantize_kernel) rounded once to T
template <typename T>
__global__ void __launch_bounds__(kThreads)
dequantize16_kernel(const int8_t* __restrict__ src, int64_t src_stride, const float* __restrict__ scales,
                    T* __restrict__ dst, int64_t dst_stride, int64_t elems) {
    const int8_t* q = src + (int64_t)blockIdx.y * src_stride;
    T* x = dst + (int64_t)blockIdx.y * dst_stride;
    const float scale = scales[blockIdx.y];
    const int64_t nvec = elems >> 4;          // elems is a multiple of 16, both sides 16-byte aligned
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * kThreads) {
        uint4 w = __ldg(reinterpret_cast<const uint4*>(q + (i << 4)));
        const int8_t* b = reinterpret_cast<const int8_t*>(&w);
        __align__(16) T o[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) o[k] = from_f32<T>((float)b[k] * scale);
        uint4* dst4 = reinterpret_cast<uint4*>(x + (i << 4));
        dst4[0] = reinterpret_cast<const uint4*>(o)[0];
        dst4[1] = reinterpret_cast<const uint4*>(o)[1];
    }
}

template <bool VEC>
__global__ void __launch_bounds__(kThreads)
dequantize_kernel(const int8_t* __restrict__ src, int64_t src_stride,
                  const float* __restrict__ scales, float* __restrict__ dst, int64_t dst_stride,
                  int64_t elems) {
    const int8_t* q = src + (int64_t)blockIdx.y * src_stride;
    float* x = dst + (int64_t)blockIdx.y * dst_stride;
    const float scale = scales[blockIdx.y];
    if (VEC) {
        int64_t nvec = elems >> 4;
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec;
             i += (int64_t)gridDim.x * kThreads) {
            uint4 w = __ldg(reinterpret_cast<const uint4*>(q + (i << 4)));
            const int8_t* b = reinterpret_cast<const int8_t*>(&w);
            float4* o = reinterpret_cast<float4*>(x + (i << 4));
#pragma unroll
            for (int k = 0; k < 4; ++k)
                o[k] = make_float4((float)b[4 * k] * scale, (float)b[4 * k + 1] * scale,
                                   (float)b[4 * k + 2] * scale, (float)b[4 * k + 3] * scale);
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < elems;
             i += (int64_t)gridDim.x * kThreads)
            x[i] = (float)q[i] * scale;
    }
}

// One block per (b,h): DH threads quantize the new K row and the new V row with
// the tensor's stored scale.
template <typename T>
__global__ void append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                              int8_t* __restrict__ k_cache, int8_t* __restrict__ v_cache,
                              const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                              const int32_t* __restrict__ pos, int pos_bias, int H, int S_max, int DH) {
    grid_release_dependents();            // a decode kernel launched to overlap may start: it waits where it reads the row
    int bh = blockIdx.x;
    int b = bh / H;
    int row = pos[b] + pos_bias;
    if (row < 0 || row >= S_max) return;  // out-of-range rows are rejected, not written
    int d = threadIdx.x;
    if (d >= DH) return;
    int64_t off = ((int64_t)bh * S_max + row) * DH + d;
    float kden = __fadd_rn(k_scale[bh], 1e-8f);
    float vden = __fadd_rn(v_scale[bh], 1e-8f);
    k_cache[off] = (int8_t)quant1(to_f32<T>(k_new[(int64_t)bh * DH + d]), kden);
    v_cache[off] = (int8_t)quant1(to_f32<T>(v_new[(int64_t)bh * DH + d]), vden);
}

int blocks_for(const logos_ctx* ctx, int64_t work_items, int n_tensors) {
    // enough blocks per tensor to fill the device about four times over, never
    // more than there is work
    int64_t want = ((int64_t)ctx->sm_count * 8 * 4 + n_tensors - 1) / n_tensors;
    int64_t have = (work_items + kThreads - 1) / kThreads;
    int64_t b = want < have ? want : have;
    return (int)(b < 1 ? 1 : b);
}

template <typename T>
int quantize_typed(logos_ctx* ctx, const T* src, int64_t src_stride, int8_t* dst,
                   int64_t dst_stride, float* scales, int n_tensors, int64_t elems, const float* absmax_known) {
    bool vec = (elems % 16 == 0) && aligned16(src) && aligned16(dst) &&
               ((src_stride * (int64_t)sizeof(T)) % 16 == 0) && (dst_stride % 16 == 0);
    // the per-tensor max|x|: computed here (first pass over the tensor), or handed in by a producer that
    // already had every value in its registers (the projection GEMM's epilogue)
    const float* amax = absmax_known ? absmax_known : ctx->absmax_scratch;
    dim3 grid(blocks_for(ctx, vec ? elems / 16 : elems, n_tensors), n_tensors);
    if (!absmax_known) {
        LOGOS_CUDA_TRY(ctx, cudaMemsetAsync(ctx->absmax_scratch, 0, sizeof(float) * n_tensors, ctx->stream));
        if (vec) absmax_kernel<T, true><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, elems, ctx->absmax_scratch);
        else absmax_kernel<T, false><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, elems, ctx->absmax_scratch);
        LOGOS_LAUNCH_CHECK(ctx, "absmax_kernel");
    }
    if (vec) {
        quantize_kernel<T, true><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, dst,
                                                                      dst_stride, amax, scales, elems);
    } else {
        quantize_kernel<T, false><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, dst,
                                                                       dst_stride, amax, scales, elems);
    }
    LOGOS_LAUNCH_CHECK(ctx, "quantize_kernel");
    return LOGOS_OK;
}

}  // namespace

int kv_quantize(logos_ctx* ctx, int src_dtype, const void* src, int64_t src_stride, int8_t* dst,
                int64_t dst_stride, float* scales, int n_tensors, int64_t elems, const float* absmax_known) {
    if (!src || !dst || !scales || n_tensors <= 0 || elems <= 0 || src_stride < elems ||
        dst_stride < elems)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_quantize: bad pointer, extent or stride");
    if (n_tensors > 65535)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "kv_quantize: more than 65535 tensors per call");
    if (!absmax_known && n_tensors > ctx->absmax_slots)
        return fail(ctx, LOGOS_ERR_WORKSPACE, "kv_quantize: absmax scratch holds %d tensors",
                    ctx->absmax_slots);
    switch (src_dtype) {
        case LOGOS_F32:
            return quantize_typed(ctx, (const float*)src, src_stride, dst, dst_stride, scales,
                                  n_tensors, elems, absmax_known);
        case LOGOS_BF16:
            return quantize_typed(ctx, (const __nv_bfloat16*)src, src_stride, dst, dst_stride,
                                  scales, n_tensors, elems, absmax_known);
        case LOGOS_F16:
            return quantize_typed(ctx, (const __half*)src, src_stride, dst, dst_stride, scales,
                                  n_tensors, elems, absmax_known);
    }
    return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_quantize: unknown dtype %d", src_dtype);
}

int kv_dequantize(logos_ctx* ctx, const int8_t* src, int64_t src_stride, const float* scales,
                  float* dst, int64_t dst_stride, int n_tensors, int64_t elems) {
    if (!src || !dst || !scales || n_tensors <= 0 || elems <= 0 || src_stride < elems ||
        dst_stride < elems)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_dequantize: bad pointer, extent or stride");
    if (n_tensors > 65535)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "kv_dequantize: more than 65535 tensors per call");
    bool vec = (elems % 16 == 0) && aligned16(src) && aligned16(dst) && (src_stride % 16 == 0) &&
               (dst_stride % 4 == 0);
    dim3 grid(blocks_for(ctx, vec ? elems / 16 : elems, n_tensors), n_tensors);
    if (vec)
        dequantize_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, scales, dst,
                                                                    dst_stride, elems);
    else
        dequantize_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, scales, dst,
                                                                     dst_stride, elems);
    LOGOS_LAUNCH_CHECK(ctx, "dequantize_kernel");
    return LOGOS_OK;
}

int kv_dequantize16(logos_ctx* ctx, int dst_dtype, const int8_t* src, int64_t src_stride, const float* scales,
                    void* dst, int64_t dst_stride, int n_tensors, int64_t elems) {
    if (!src || !dst || !scales || n_tensors <= 0 || elems <= 0 || src_stride < elems || dst_stride < elems)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_dequantize16: bad pointer, extent or stride");
    if (dst_dtype != LOGOS_BF16 && dst_dtype != LOGOS_F16)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "kv_dequantize16: the destination is BF16 or FP16");
    if (n_tensors > 65535)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "kv_dequantize16: more than 65535 tensors per call");
    if ((elems % 16) != 0 || !aligned16(src) || !aligned16(dst) || (src_stride % 16) != 0 || (dst_stride % 8) != 0)
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "kv_dequantize16: 16-byte aligned tensors of a multiple of 16 values");
    dim3 grid(blocks_for(ctx, elems / 16, n_tensors), n_tensors);
    if (dst_dtype == LOGOS_BF16)
        dequantize16_kernel<__nv_bfloat16><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, scales, (__nv_bfloat16*)dst, dst_stride, elems);
    else
        dequantize16_kernel<__half><<<grid, kThreads, 0, ctx->stream>>>(src, src_stride, scales, (__half*)dst, dst_stride, elems);
    LOGOS_LAUNCH_CHECK(ctx, "dequantize16_kernel");
    return LOGOS_OK;
}

int kv_append(logos_ctx* ctx, int dtype, const void* k_new, const void* v_new, int8_t* k_cache,
              int8_t* v_cache, const float* k_scale, const float* v_scale, const int32_t* pos,
              int B, int H, int S_max, int DH, int pos_bias) {
    if (!k_new || !v_new || !k_cache || !v_cache || !k_scale || !v_scale || !pos || B <= 0 ||
        H <= 0 || S_max <= 0 || DH <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_append: bad pointer or extent");
    if (DH > 1024) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "kv_append: DH > 1024");
    int threads = (DH + 31) / 32 * 32;
    int grid = B * H;
    switch (dtype) {
        case LOGOS_F32:
            append_kernel<float><<<grid, threads, 0, ctx->stream>>>(
                (const float*)k_new, (const float*)v_new, k_cache, v_cache, k_scale, v_scale, pos, pos_bias,
                H, S_max, DH);
            break;
        case LOGOS_BF16:
            append_kernel<__nv_bfloat16><<<grid, threads, 0, ctx->stream>>>(
                (const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, k_cache, v_cache,
                k_scale, v_scale, pos, pos_bias, H, S_max, DH);
            break;
        case LOGOS_F16:
            append_kernel<__half><<<grid, threads, 0, ctx->stream>>>(
                (const __half*)k_new, (const __half*)v_new, k_cache, v_cache, k_scale, v_scale,
                pos, pos_bias, H, S_max, DH);
            break;
        default:
            return fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_append: unknown dtype %d", dtype);
    }
    LOGOS_LAUNCH_CHECK(ctx, "append_kernel");
    return LOGOS_OK;
}

}  // namespace logos
