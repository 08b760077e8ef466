// decode_generic.cu -- INT8-KV decode attention for head dimensions other than 64.
//
// The reference's attention path takes any head dimension up to 128 (cuda/VedicGEMM.cu:899,
// 1074-1079); the model it ships uses 64, which is what decode_dense_kernel and decode_sparse_kernel
// are built for.  This kernel keeps the entry point whole for the other sizes (DH a multiple of 16,
// at most 128): one CTA per (sequence, head), fp32 SIMT arithmetic, every switch of the parameter
// block (Shunyam window and landmarks, advection, both diffusion stencils, the blend).  The scores of
// the row live in shared memory, so the context length is bounded by it (about 50 000 tokens, half of
// that with a blend).  It is a functional path, not a tuned one: rows of K are read one thread per
// key, V one byte per thread.
#include "common.cuh"

namespace logos {
namespace {

constexpr int kGenThreads = 256;
constexpr int kGenMaxDH = 128;

struct GenArgs {
    const __half* q; const __half* q_prev;
    const int8_t* k_cache; const int8_t* v_cache;
    const float* k_scale; const float* v_scale;
    const int32_t* len;
    float* out;
    int H, S_max, DH;
    float scale, eta, nu, alpha;
    int mode, window, stride;
};

__device__ __forceinline__ float gen_block_reduce(float v, float* red, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kGenThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    __syncthreads();
    return r;
}

template <bool BLEND>
__global__ void __launch_bounds__(kGenThreads)
decode_generic_kernel(const GenArgs a, int p_cap) {
    extern __shared__ float dyn[];
    float* qn = dyn;                        // advected query x scale x k_scale
    float* qs = qn + kGenMaxDH;             // plain query (BLEND)
    float* p_ns = qs + kGenMaxDH;           // [p_cap] scores, then weights
    float* p_std = p_ns + p_cap;            // [p_cap] (BLEND)
    __shared__ float red[kGenThreads / 32];
    __shared__ float part_ns[16][kGenMaxDH], part_std[BLEND ? 16 : 1][kGenMaxDH];

    const int bh = blockIdx.x, b = bh / a.H, DH = a.DH, tid = threadIdx.x;
    int len = a.len[b];
    len = len < 0 ? 0 : (len > a.S_max ? a.S_max : len);
    const int pos = len - 1;
    float* out = a.out + (int64_t)bh * DH;
    if (len == 0) {
        if (tid < DH) out[tid] = 0.0f;
        return;
    }
    const bool advect = a.eta != 0.0f && pos > 0 && a.q_prev != nullptr;
    const float f = a.scale * a.k_scale[bh];
    for (int c = tid; c < DH; c += kGenThreads) {
        const float x = __half2float(a.q[(int64_t)bh * DH + c]);
        const float xp = advect ? __half2float(a.q_prev[(int64_t)bh * DH + c]) : x;
        qn[c] = (x + a.eta * (x - xp)) * f;      // ns_advect_kernel, cuda/ModelGPU.cu:443-451
        qs[c] = x * f;
    }
    __syncthreads();

    const int8_t* K = a.k_cache + (int64_t)bh * a.S_max * DH;
    const int8_t* V = a.v_cache + (int64_t)bh * a.S_max * DH;
    const bool active = shunyam_active(a.window, len);
    float mx = -INFINITY, mx2 = -INFINITY;
    for (int j = tid; j < len; j += kGenThreads) {
        // the query is the last row: j <= pos always; cuda/VedicGEMM.cu:987-996 for the rest
        const bool visible = !active || j >= pos - a.window || (a.stride > 0 && j % a.stride == 0);
        float s = -INFINITY, s2 = -INFINITY;
        if (visible) {
            s = 0.0f; s2 = 0.0f;
            const uint4* row = reinterpret_cast<const uint4*>(K + (int64_t)j * DH);
            for (int c16 = 0; c16 < DH / 16; ++c16) {
                const uint4 w = __ldg(row + c16);
                const int8_t* bts = reinterpret_cast<const int8_t*>(&w);
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    s = fmaf((float)bts[e], qn[16 * c16 + e], s);
                    if (BLEND) s2 = fmaf((float)bts[e], qs[16 * c16 + e], s2);
                }
            }
        }
        p_ns[j] = s;
        mx = fmaxf(mx, s);
        if (BLEND) { p_std[j] = s2; mx2 = fmaxf(mx2, s2); }
    }
    const float m_ns = gen_block_reduce(mx, red, true);
    const float m_std = BLEND ? gen_block_reduce(mx2, red, true) : 0.0f;
    float sum = 0.0f, sum2 = 0.0f;
    for (int j = tid; j < len; j += kGenThreads) {
        const float e = (p_ns[j] == -INFINITY) ? 0.0f : expf(p_ns[j] - m_ns);
        p_ns[j] = e;
        sum += e;
        if (BLEND) {
            const float e2 = (p_std[j] == -INFINITY) ? 0.0f : expf(p_std[j] - m_std);
            p_std[j] = e2;
            sum2 += e2;
        }
    }
    const float l_ns = gen_block_reduce(sum, red, false);      // also orders the weight writes before their reads
    const float l_std = BLEND ? gen_block_reduce(sum2, red, false) : 1.0f;

    // values: thread = (channel c, key group g); group g takes keys g, g + G, ...
    const int G = kGenThreads / DH;                            // 2 .. 16
    const int c = tid % DH, g = tid / DH;
    float acc = 0.0f, acc2 = 0.0f;
    if (g < G) {
        for (int j = g; j < len; j += G) {
            const float p = p_ns[j];
            const float p2 = BLEND ? p_std[j] : 0.0f;
            if (p == 0.0f && p2 == 0.0f) continue;
            const float v = (float)V[(int64_t)j * DH + c];
            float vs = v;
            if (a.mode == LOGOS_DIFFUSE_CAUSAL) {              // ns_diffuse_kernel, cuda/ModelGPU.cu:463-471
                const float vp = j > 0 ? (float)V[(int64_t)(j - 1) * DH + c] : v;
                vs = (1.0f - a.nu) * v + a.nu * vp;
            } else if (a.mode == LOGOS_DIFFUSE_CENTRAL) {      // include/Attention.hpp:173-181, clamped to the context
                const float vl = j > 0 ? (float)V[(int64_t)(j - 1) * DH + c] : v;
                const float vr = j < len - 1 ? (float)V[(int64_t)(j + 1) * DH + c] : v;
                vs = (1.0f - a.nu) * v + (0.5f * a.nu) * (vl + vr);
            }
            acc = fmaf(p, vs, acc);
            if (BLEND) acc2 = fmaf(p2, v, acc2);
        }
        part_ns[g][c] = acc;
        if (BLEND) part_std[g][c] = acc2;
    }
    __syncthreads();
    if (tid < DH) {
        float o = 0.0f, o2 = 0.0f;
        for (int gg = 0; gg < G; ++gg) {
            o += part_ns[gg][tid];
            if (BLEND) o2 += part_std[gg][tid];
        }
        float r = l_ns > 0.0f ? o / l_ns : 0.0f;
        if (BLEND) r = (1.0f - a.alpha) * (l_std > 0.0f ? o2 / l_std : 0.0f) + a.alpha * r;
        out[tid] = r * a.v_scale[bh];
    }
}

}  // namespace

int decode_generic(logos_ctx* ctx, const void* q, const void* q_prev, const int8_t* k_cache, const int8_t* v_cache,
                   const float* k_scale, const float* v_scale, const int32_t* len, int B, int H, int S_max, int DH,
                   const logos_attn_params* p, float* out) {
    if (DH <= 0 || DH > kGenMaxDH || (DH % 16) != 0)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: DH = %d (a multiple of 16, at most 128)", DH);
    if (!out) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: the peer exchange is built for DH = 64");
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    const bool blend = ns_any && p->ns_alpha < 1.0f;
    const size_t smem = sizeof(float) * (2 * (size_t)kGenMaxDH + (size_t)S_max * (blend ? 2 : 1));
    if (smem > 200 * 1024)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: S_max = %d is beyond the DH = %d kernel's shared memory", S_max, DH);
    GenArgs a;
    a.q = (const __half*)q; a.q_prev = (const __half*)q_prev;
    a.k_cache = k_cache; a.v_cache = v_cache; a.k_scale = k_scale; a.v_scale = v_scale;
    a.len = len; a.out = out; a.H = H; a.S_max = S_max; a.DH = DH;
    a.scale = p->scale;
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    a.alpha = p->ns_alpha;
    a.window = p->window; a.stride = p->stride;
    const int BH = B * H;
    if (blend) {
        if (int rc = ensure_smem_limit(ctx, decode_generic_kernel<true>, 200 * 1024)) return rc;
        decode_generic_kernel<true><<<BH, kGenThreads, smem, ctx->stream>>>(a, S_max);
    } else {
        if (int rc = ensure_smem_limit(ctx, decode_generic_kernel<false>, 200 * 1024)) return rc;
        decode_generic_kernel<false><<<BH, kGenThreads, smem, ctx->stream>>>(a, S_max);
    }
    LOGOS_LAUNCH_CHECK(ctx, "decode_generic_kernel");
    return LOGOS_OK;
}

}  // namespace logos
