// attn_simt.cu -- general fp32 attention kernel: every option, every shape.
//
// This is the exact-arithmetic path of the engine.  It accepts fp32, BF16 or FP16
// inputs of any head dimension up to 128 and any sequence length, computes in fp32
// end to end (no rounding of Q_adv, V_s or the softmax weights to 16 bits) and
// implements every switch of the attention parameters: causal mask, Shunyam
// window + landmark rule, Q-advection, both V-diffusion stencils and the alpha
// blend of the standard and the Navier-Stokes outputs.  It serves the fp32
// single-head entry point that stands in for cuda_flash_attention_fwd
// (cuda/VedicGEMM.cu:1065-1104) and all shapes the tensor-core kernel does not take.
//
// Structure: one CTA = 32 query rows x all keys, keys in tiles of 64, online
// softmax (same recurrence as cuda/VedicGEMM.cu:1003-1045).  256 threads = 16 groups
// of 16 lanes; a group owns query rows g and g+16.  Inside a group lane c scores
// keys c, c+16, c+32, c+48 of the tile and owns output channels c, c+16, ...
// The Navier-Stokes prologue is applied while the tiles are written to shared
// memory: Q rows become Q + eta (Q - Q_prev) (cuda/ModelGPU.cu:443-451), V rows
// become the causal (cuda/ModelGPU.cu:463-471) or central
// (include/Attention.hpp:173-181) stencil of their neighbours.
#include "common.cuh"

namespace logos {
namespace {

constexpr int BM = 32;   // query rows per CTA
constexpr int BN = 64;   // keys per tile
constexpr int kThreads = 256;
constexpr int kMaxDH = 128;
constexpr int kMaxCh = kMaxDH / 16;  // output channels per lane

struct SimtArgs {
    const void* Q; const void* K; const void* V; void* O;
    int S, DH, H;
    // elements between two sequences, two heads and two rows of Q / K / V (one layout for the three) and of O
    long long i_batch, i_head, i_row, o_batch, o_head, o_row;
    float scale, eta, nu, alpha;
    int causal, shunyam, window, stride, diffuse_mode;
};

template <typename TIn, typename TOut, bool BLEND>
__global__ void __launch_bounds__(kThreads)
attention_simt_kernel(const SimtArgs a) {
    extern __shared__ float smem[];
    const int S = a.S, DH = a.DH, DHK = DH + 1;
    float* sQa = smem;                               // [BM][DH]   advected queries
    float* sQs = sQa + BM * DH;                      // [BM][DH]   plain queries (BLEND)
    float* sK = sQs + (BLEND ? BM * DH : 0);         // [BN][DH+1]
    float* sVs = sK + BN * DHK;                      // [BN][DH]   diffused values
    float* sVr = sVs + BN * DH;                      // [BN][DH]   raw values (BLEND)
    float* sP = sVr + (BLEND ? BN * DH : 0);         // [BM][BN]
    float* sP2 = sP + BM * BN;                       // [BM][BN]   (BLEND)

    const int b_idx = (int)blockIdx.y / a.H, h_idx = (int)blockIdx.y - b_idx * a.H;
    const int64_t head_off = (int64_t)b_idx * a.i_batch + (int64_t)h_idx * a.i_head;
    const int64_t RS = a.i_row;                       // row pitch of Q, K, V
    const TIn* Q = (const TIn*)a.Q + head_off;
    const TIn* K = (const TIn*)a.K + head_off;
    const TIn* V = (const TIn*)a.V + head_off;
    TOut* O = (TOut*)a.O + (int64_t)b_idx * a.o_batch + (int64_t)h_idx * a.o_head;

    const int tid = threadIdx.x;
    const int grp = tid >> 4, lc = tid & 15;
    const int q0 = blockIdx.x * BM;
    const bool shun = a.shunyam != 0, causal = a.causal != 0;

    // ---- Q tile with advection ----
    for (int e = tid; e < BM * DH; e += kThreads) {
        int r = e / DH, d = e - r * DH, i = q0 + r;
        float q = 0.0f, qa = 0.0f;
        if (i < S) {
            q = to_f32<TIn>(Q[(int64_t)i * RS + d]);
            float qp = (i > 0) ? to_f32<TIn>(Q[(int64_t)(i - 1) * RS + d]) : q;
            qa = q + a.eta * (q - qp);
        }
        sQa[e] = qa;
        if (BLEND) sQs[e] = q;
    }

    float m1[2] = {-INFINITY, -INFINITY}, l1[2] = {0.0f, 0.0f};
    float m2[2] = {-INFINITY, -INFINITY}, l2[2] = {0.0f, 0.0f};
    float o1[2][kMaxCh], o2[BLEND ? 2 : 1][kMaxCh];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int c = 0; c < kMaxCh; ++c) {
            o1[r][c] = 0.0f;
            if (BLEND) o2[r][c] = 0.0f;
        }

    const int i_last = min(S, q0 + BM) - 1;           // last query row of this CTA
    const int k_end = causal ? i_last + 1 : S;        // keys beyond are masked for every row
    for (int k0 = 0; k0 < k_end; k0 += BN) {
        if (shun) {
            // skip tiles with no visible key: outside every row's window and without landmark
            bool in_win = (k0 + BN - 1 >= q0 - a.window) && (k0 <= i_last);
            bool has_land = false;
            if (a.stride > 0) {
                int first = ((k0 + a.stride - 1) / a.stride) * a.stride;
                has_land = first < k0 + BN && first < S;
            }
            if (!in_win && !has_land) continue;
        }
        __syncthreads();  // previous tile fully consumed (also orders the Q tile writes)
        for (int e = tid; e < BN * DH; e += kThreads) {
            int r = e / DH, d = e - r * DH, j = k0 + r;
            float kv = 0.0f, v = 0.0f, vs = 0.0f;
            if (j < S) {
                kv = to_f32<TIn>(K[(int64_t)j * RS + d]);
                v = to_f32<TIn>(V[(int64_t)j * RS + d]);
                if (a.diffuse_mode == LOGOS_DIFFUSE_CAUSAL) {
                    float vp = (j > 0) ? to_f32<TIn>(V[(int64_t)(j - 1) * RS + d]) : v;
                    vs = (1.0f - a.nu) * v + a.nu * vp;
                } else if (a.diffuse_mode == LOGOS_DIFFUSE_CENTRAL) {
                    int jl = (j > 0) ? j - 1 : 0, jr = (j < S - 1) ? j + 1 : S - 1;
                    float vl = to_f32<TIn>(V[(int64_t)jl * RS + d]);
                    float vr = to_f32<TIn>(V[(int64_t)jr * RS + d]);
                    vs = (1.0f - a.nu) * v + (a.nu * 0.5f) * (vl + vr);
                } else {
                    vs = v;
                }
            }
            sK[r * DHK + d] = kv;
            sVs[e] = vs;
            if (BLEND) sVr[e] = v;
        }
        __syncthreads();

#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = grp + rr * 16, i = q0 + row;
            float s1[4], s2[4];
            bool ok[4];
            float tmax1 = -INFINITY, tmax2 = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                int jl = lc + 16 * c, j = k0 + jl;
                ok[c] = (i < S) && (j < S) && key_allowed(i, j, causal, shun, a.window, a.stride);
                s1[c] = -INFINITY; s2[c] = -INFINITY;
                if (ok[c]) {
                    const float* qa = sQa + row * DH;
                    const float* kk = sK + jl * DHK;
                    float d1 = 0.0f, d2 = 0.0f;
                    for (int d = 0; d < DH; ++d) {
                        d1 = fmaf(qa[d], kk[d], d1);
                        if (BLEND) d2 = fmaf(sQs[row * DH + d], kk[d], d2);
                    }
                    s1[c] = d1 * a.scale;
                    tmax1 = fmaxf(tmax1, s1[c]);
                    if (BLEND) { s2[c] = d2 * a.scale; tmax2 = fmaxf(tmax2, s2[c]); }
                }
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, off));
                if (BLEND) tmax2 = fmaxf(tmax2, __shfl_xor_sync(0xffffffffu, tmax2, off));
            }
            // online softmax update; a tile that shows this row nothing leaves it untouched
            float mn1 = fmaxf(m1[rr], tmax1);
            float corr1 = (m1[rr] == -INFINITY) ? 0.0f : expf(m1[rr] - mn1);
            float ps1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float p = ok[c] ? expf(s1[c] - mn1) : 0.0f;
                sP[row * BN + lc + 16 * c] = p;
                ps1 += p;
            }
            float mn2 = -INFINITY, corr2 = 0.0f, ps2 = 0.0f;
            if (BLEND) {
                mn2 = fmaxf(m2[rr], tmax2);
                corr2 = (m2[rr] == -INFINITY) ? 0.0f : expf(m2[rr] - mn2);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    float p = ok[c] ? expf(s2[c] - mn2) : 0.0f;
                    sP2[row * BN + lc + 16 * c] = p;
                    ps2 += p;
                }
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) {
                ps1 += __shfl_xor_sync(0xffffffffu, ps1, off);
                if (BLEND) ps2 += __shfl_xor_sync(0xffffffffu, ps2, off);
            }
            if (mn1 != -INFINITY) { l1[rr] = l1[rr] * corr1 + ps1; m1[rr] = mn1; }
            if (BLEND && mn2 != -INFINITY) { l2[rr] = l2[rr] * corr2 + ps2; m2[rr] = mn2; }
            __syncwarp();  // a row's weights are written and read by the same half-warp
            if (mn1 != -INFINITY) {
#pragma unroll
                for (int c = 0; c < kMaxCh; ++c) {
                    o1[rr][c] *= corr1;
                    if (BLEND) o2[rr][c] *= corr2;
                }
                const int jn = min(BN, S - k0);
                for (int j = 0; j < jn; ++j) {
                    float p = sP[row * BN + j];
                    float p2 = BLEND ? sP2[row * BN + j] : 0.0f;
#pragma unroll
                    for (int c = 0; c < kMaxCh; ++c) {
                        int d = lc + 16 * c;
                        if (d < DH) {
                            o1[rr][c] = fmaf(p, sVs[j * DH + d], o1[rr][c]);
                            if (BLEND) o2[rr][c] = fmaf(p2, sVr[j * DH + d], o2[rr][c]);
                        }
                    }
                }
            }
        }
    }

#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int i = q0 + grp + rr * 16;
        if (i >= S) continue;
        // cuda/VedicGEMM.cu:1049: a row whose weights sum to (almost) nothing outputs zeros
        float inv1 = (l1[rr] > 1e-9f) ? 1.0f / l1[rr] : 0.0f;
        float inv2 = (BLEND && l2[rr] > 1e-9f) ? 1.0f / l2[rr] : 0.0f;
#pragma unroll
        for (int c = 0; c < kMaxCh; ++c) {
            int d = lc + 16 * c;
            if (d < DH) {
                float r = o1[rr][c] * inv1;
                if (BLEND) r = (1.0f - a.alpha) * (o2[rr][c] * inv2) + a.alpha * r;
                O[(int64_t)i * a.o_row + d] = from_f32<TOut>(r);
            }
        }
    }
}

template <typename TIn, typename TOut>
int launch(logos_ctx* ctx, const SimtArgs& a, int BH, bool blend) {
    const int DH = a.DH;
    size_t floats = (size_t)BM * DH * (blend ? 2 : 1) + (size_t)BN * (DH + 1) +
                    (size_t)BN * DH * (blend ? 2 : 1) + (size_t)BM * BN * (blend ? 2 : 1);
    size_t smem = floats * sizeof(float);
    // the limit is raised once, to what the largest head dimension needs
    const int smem_max = (int)(sizeof(float) * ((size_t)BM * kMaxDH * (blend ? 2 : 1) + (size_t)BN * (kMaxDH + 1) +
                                                (size_t)BN * kMaxDH * (blend ? 2 : 1) + (size_t)BM * BN * (blend ? 2 : 1)));
    dim3 grid((a.S + BM - 1) / BM, BH);
    if (blend) {
        int rc = ensure_smem_limit(ctx, attention_simt_kernel<TIn, TOut, true>, smem_max);
        if (rc != LOGOS_OK) return rc;
        attention_simt_kernel<TIn, TOut, true><<<grid, kThreads, smem, ctx->stream>>>(a);
    } else {
        int rc = ensure_smem_limit(ctx, attention_simt_kernel<TIn, TOut, false>, smem_max);
        if (rc != LOGOS_OK) return rc;
        attention_simt_kernel<TIn, TOut, false><<<grid, kThreads, smem, ctx->stream>>>(a);
    }
    LOGOS_LAUNCH_CHECK(ctx, "attention_simt_kernel");
    return LOGOS_OK;
}

}  // namespace

int attention_simt(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                   const void* V, void* O, int B, int H, int S, int DH,
                   const logos_attn_params* p, const logos_strides* in, const logos_strides* out) {
    if (DH > kMaxDH)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention: DH=%d exceeds %d", DH, kMaxDH);
    if ((int64_t)B * H > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention: B*H > 65535");
    SimtArgs a;
    a.Q = Q; a.K = K; a.V = V; a.O = O;
    a.S = S; a.DH = DH; a.H = H;
    a.i_batch = in ? in->batch : (int64_t)H * S * DH; a.i_head = in ? in->head : (int64_t)S * DH; a.i_row = in ? in->row : DH;
    a.o_batch = out ? out->batch : (int64_t)H * S * DH; a.o_head = out ? out->head : (int64_t)S * DH; a.o_row = out ? out->row : DH;
    if (a.i_row < DH || a.o_row < DH)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "attention: a row stride is smaller than DH");
    a.scale = p->scale;
    a.causal = p->causal;
    a.shunyam = shunyam_active(p->window, S) ? 1 : 0;
    a.window = p->window; a.stride = p->stride;
    const bool ns_any = p->ns_alpha > 0.0f &&
                        (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.diffuse_mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    a.alpha = p->ns_alpha;
    const bool blend = ns_any && p->ns_alpha < 1.0f;
    const int BH = B * H;
    if (in_dtype == LOGOS_F32 && out_dtype == LOGOS_F32) return launch<float, float>(ctx, a, BH, blend);
    if (in_dtype == LOGOS_BF16 && out_dtype == LOGOS_F32) return launch<__nv_bfloat16, float>(ctx, a, BH, blend);
    if (in_dtype == LOGOS_BF16 && out_dtype == LOGOS_BF16) return launch<__nv_bfloat16, __nv_bfloat16>(ctx, a, BH, blend);
    if (in_dtype == LOGOS_F16 && out_dtype == LOGOS_F32) return launch<__half, float>(ctx, a, BH, blend);
    if (in_dtype == LOGOS_F16 && out_dtype == LOGOS_F16) return launch<__half, __half>(ctx, a, BH, blend);
    return fail(ctx, LOGOS_ERR_INVALID_ARG, "attention: output dtype must be the input dtype or fp32");
}

}  // namespace logos
