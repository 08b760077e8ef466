// attn_bwd.cu -- gradients of the attention forward with respect to Q, K and V, fp32.
//
// LOGOS runs attention backward per head as a chain of one-output-per-thread kernels over materialised
// seq x seq matrices (cuda/train_gpu.cu:657-748: the probabilities are recomputed from Q_adv and K, then
// attn_dV_kernel :422, attn_dAttnProbs_kernel :434, softmax_bwd_kernel :446, attn_dQ_kernel :461,
// attn_dK_kernel :472, with ns_diffuse_bwd_kernel and ns_advect_bwd_kernel, cuda/ModelGPU.cu:453-482, for the
// prologue).  Here nothing of size seq x seq exists: the probabilities are recomputed tile by tile from the
// row statistics, as in the forward.  Three kernels per path, all heads and sequences at once:
//   bwd_rows_kernel  one CTA per 64 query rows: pass 1 over the visible key tiles gives the row's
//                    log-sum-exp and delta_i = sum_j p_ij dp_ij (= d_out_i . out_i); pass 2 gives
//                    dq_i = scale sum_j p_ij (dp_ij - delta_i) k_j.
//   bwd_keys_kernel  one CTA per 64 keys: over the query tiles that see them,
//                    dv_j = sum_i p_ij d_out_i,  dk_j = scale sum_i p_ij (dp_ij - delta_i) q_i.
//   bwd_adjoint_kernel  the transposes of the advection and diffusion stencils, raw-tensor gradients out.
// The mask is the forward's own (causal, Shunyam window and landmarks): the gradient of what was computed.
// (The reference's recompute applies the causal mask only, whatever the forward used.)
// With 0 < ns_alpha < 1 the forward is a blend of two attentions and the chain runs once per path.
// Every sum has a fixed order (no atomics): results are reproducible bit for bit.
//
// Tiles are 64 x DH fp32 in shared memory, row-major with a pitch of DH + 4 floats; a thread owns rows
// ty + 16 a and columns tx + 16 b of a 64 x 64 product, which makes every shared-memory access of the
// inner loops a conflict-free 16-byte load.
#include <algorithm>

#include "common.cuh"

namespace logos {
namespace {

constexpr int kTS = 64;          // rows per tile (queries or keys)
constexpr int kBwdThreads = 256;
constexpr int kPP = kTS + 4;     // pitch of a 64 x 64 tile

struct BwdArgs {
    const float* Qx; const float* K; const float* Vx; const float* dO;   // [BH][S][DH]
    float* dQx; float* dK; float* dVx;                                    // [BH][S][DH]
    float* lse; float* delta;                                             // [BH][S]
    int S;
    float scale, w;               // w multiplies d_out (the path's share of a blend)
    int causal, shunyam, window, stride;
    int accumulate_dk;            // dK += instead of =
};

// 64 rows x DH of a [S][DH] tensor -> shared, zero beyond S, optionally scaled
template <int DH>
__device__ __forceinline__ void load_tile(float* dst, const float* src, int row0, int S, float mul) {
    constexpr int LD = DH + 4, V4 = DH / 4;
    for (int e = threadIdx.x; e < kTS * V4; e += kBwdThreads) {
        const int r = e / V4, c4 = e - r * V4, i = row0 + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < S) v = *reinterpret_cast<const float4*>(src + (int64_t)i * DH + 4 * c4);
        v.x *= mul; v.y *= mul; v.z *= mul; v.w *= mul;
        *reinterpret_cast<float4*>(dst + r * LD + 4 * c4) = v;
    }
}

// acc[a][b] = sum_k A[ty + 16 a][k] B[tx + 16 b][k]
template <int DH>
__device__ __forceinline__ void gemm_nt(const float* A, const float* B, int ty, int tx, float (&acc)[4][4]) {
    constexpr int LD = DH + 4;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
#pragma unroll 4
    for (int k = 0; k < DH; k += 4) {
        float4 x[4], y[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) x[a] = *reinterpret_cast<const float4*>(A + (ty + 16 * a) * LD + k);
#pragma unroll
        for (int b = 0; b < 4; ++b) y[b] = *reinterpret_cast<const float4*>(B + (tx + 16 * b) * LD + k);
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                acc[a][b] = fmaf(x[a].x, y[b].x, acc[a][b]);
                acc[a][b] = fmaf(x[a].y, y[b].y, acc[a][b]);
                acc[a][b] = fmaf(x[a].z, y[b].z, acc[a][b]);
                acc[a][b] = fmaf(x[a].w, y[b].w, acc[a][b]);
            }
    }
}

// out[a][c] += sum_j W[ty + 16 a][j] X[j][tx CPT + c]   (W: 64 x 64, pitch kPP; X: 64 x DH)
template <int DH>
__device__ __forceinline__ void gemm_nn(const float* W, const float* X, int ty, int tx, float (&out)[4][DH / 16]) {
    constexpr int LD = DH + 4, CPT = DH / 16;
#pragma unroll 2
    for (int j = 0; j < kTS; j += 4) {
        float4 wv[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) wv[a] = *reinterpret_cast<const float4*>(W + (ty + 16 * a) * kPP + j);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            float xv[CPT];
            const float* xrow = X + (j + jj) * LD + tx * CPT;      // 4 CPT bytes aligned: LD and CPT are even
            if constexpr (CPT == 2) {
                const float2 t = *reinterpret_cast<const float2*>(xrow);
                xv[0] = t.x; xv[1] = t.y;
            } else {
#pragma unroll
                for (int c = 0; c < CPT; c += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(xrow + c);
                    xv[c] = t.x; xv[c + 1] = t.y; xv[c + 2] = t.z; xv[c + 3] = t.w;
                }
            }
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float wgt = jj == 0 ? wv[a].x : (jj == 1 ? wv[a].y : (jj == 2 ? wv[a].z : wv[a].w));
#pragma unroll
                for (int c = 0; c < CPT; ++c) out[a][c] = fmaf(wgt, xv[c], out[a][c]);
            }
        }
    }
}

__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// does key tile [k0, k0 + 64) show anything to query rows [q0, q_last]?
__device__ __forceinline__ bool tile_visible(const BwdArgs& a, int q0, int q_last, int k0) {
    if (a.causal && k0 > q_last) return false;
    if (!a.shunyam) return true;
    const bool in_win = (k0 + kTS - 1 >= q0 - a.window) && (k0 <= q_last);
    bool has_land = false;
    if (a.stride > 0) {
        const int first = ((k0 + a.stride - 1) / a.stride) * a.stride;
        has_land = first < k0 + kTS && first < a.S;
    }
    return in_win || has_land;
}

template <int DH>
__global__ void __launch_bounds__(kBwdThreads)
bwd_rows_kernel(const BwdArgs a) {
    constexpr int LD = DH + 4, CPT = DH / 16;
    extern __shared__ __align__(16) float smem[];
    float* sQ = smem;                 // [64][LD]
    float* sG = sQ + kTS * LD;        // d_out
    float* sK = sG + kTS * LD;
    float* sV = sK + kTS * LD;
    float* sW = sV + kTS * LD;        // [64][kPP] weights of the second product

    const int S = a.S;
    const int64_t head = (int64_t)blockIdx.y * S * DH;
    const int q0 = blockIdx.x * kTS, q_last = min(S, q0 + kTS) - 1;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const bool causal = a.causal != 0, shun = a.shunyam != 0;

    load_tile<DH>(sQ, a.Qx + head, q0, S, 1.0f);
    load_tile<DH>(sG, a.dO + head, q0, S, a.w);

    // ---- pass 1: row maximum, sum and out_i (unnormalised), as the forward ----
    float m[4], l[4], o[4][CPT];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = -INFINITY; l[r] = 0.0f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) o[r][c] = 0.0f;
    }
    const int k_end = causal ? q_last + 1 : S;
    for (int k0 = 0; k0 < k_end; k0 += kTS) {
        if (!tile_visible(a, q0, q_last, k0)) continue;
        __syncthreads();
        load_tile<DH>(sK, a.K + head, k0, S, 1.0f);
        load_tile<DH>(sV, a.Vx + head, k0, S, 1.0f);
        __syncthreads();
        float s[4][4];
        gemm_nt<DH>(sQ, sK, ty, tx, s);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = q0 + ty + 16 * r;
            float tmax = -INFINITY;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int j = k0 + tx + 16 * b;
                const bool ok = i < S && j < S && key_allowed(i, j, causal, shun, a.window, a.stride);
                s[r][b] = ok ? s[r][b] * a.scale : -INFINITY;
                tmax = fmaxf(tmax, s[r][b]);
            }
            tmax = group16_max(tmax);
            const float mn = fmaxf(m[r], tmax);
            const float corr = (m[r] == -INFINITY) ? 0.0f : expf(m[r] - mn);
            float ps = 0.0f;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float p = (s[r][b] == -INFINITY) ? 0.0f : expf(s[r][b] - mn);
                sW[(ty + 16 * r) * kPP + tx + 16 * b] = p;
                ps += p;
            }
            ps = group16_sum(ps);
            if (mn != -INFINITY) {
                l[r] = l[r] * corr + ps;
                m[r] = mn;
#pragma unroll
                for (int c = 0; c < CPT; ++c) o[r][c] *= corr;
            }
        }
        __syncthreads();
        gemm_nn<DH>(sW, sV, ty, tx, o);
    }
    // log-sum-exp and delta; a row that saw (almost) nothing was written as zeros by the forward
    // (cuda/VedicGEMM.cu:1049) and gets no gradient
    float lse[4], dlt[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const bool live = l[r] > 1e-9f;
        float dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) dot = fmaf(sG[(ty + 16 * r) * LD + tx * CPT + c], o[r][c], dot);
        dot = group16_sum(dot);
        lse[r] = live ? m[r] + logf(l[r]) : INFINITY;
        dlt[r] = live ? dot / l[r] : 0.0f;
        const int i = q0 + ty + 16 * r;
        if (tx == 0 && i < S) {
            a.lse[(int64_t)blockIdx.y * S + i] = lse[r];
            a.delta[(int64_t)blockIdx.y * S + i] = dlt[r];
        }
    }

    // ---- pass 2: dq ----
    float dq[4][CPT];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < CPT; ++c) dq[r][c] = 0.0f;
    for (int k0 = 0; k0 < k_end; k0 += kTS) {
        if (!tile_visible(a, q0, q_last, k0)) continue;
        __syncthreads();
        load_tile<DH>(sK, a.K + head, k0, S, 1.0f);
        load_tile<DH>(sV, a.Vx + head, k0, S, 1.0f);
        __syncthreads();
        float s[4][4], dp[4][4];
        gemm_nt<DH>(sQ, sK, ty, tx, s);
        gemm_nt<DH>(sG, sV, ty, tx, dp);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = q0 + ty + 16 * r;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int j = k0 + tx + 16 * b;
                const bool ok = i < S && j < S && key_allowed(i, j, causal, shun, a.window, a.stride);
                const float p = ok ? expf(s[r][b] * a.scale - lse[r]) : 0.0f;
                sW[(ty + 16 * r) * kPP + tx + 16 * b] = p * (dp[r][b] - dlt[r]) * a.scale;
            }
        }
        __syncthreads();
        gemm_nn<DH>(sW, sK, ty, tx, dq);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = q0 + ty + 16 * r;
        if (i >= S) continue;
#pragma unroll
        for (int c = 0; c < CPT; ++c) a.dQx[head + (int64_t)i * DH + tx * CPT + c] = dq[r][c];
    }
}

template <int DH>
__global__ void __launch_bounds__(kBwdThreads)
bwd_keys_kernel(const BwdArgs a) {
    constexpr int LD = DH + 4, CPT = DH / 16;
    extern __shared__ __align__(16) float smem[];
    float* sK = smem;
    float* sV = sK + kTS * LD;
    float* sQ = sV + kTS * LD;
    float* sG = sQ + kTS * LD;
    float* sPt = sG + kTS * LD;        // [key][query], pitch kPP
    float* sDt = sPt + kTS * kPP;      // [key][query]
    float* sL = sDt + kTS * kPP;       // [64] log-sum-exp of the query tile
    float* sD = sL + kTS;              // [64] delta

    const int S = a.S;
    const int64_t head = (int64_t)blockIdx.y * S * DH;
    const int k0 = blockIdx.x * kTS, k_last = min(S, k0 + kTS) - 1;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const bool causal = a.causal != 0, shun = a.shunyam != 0;

    load_tile<DH>(sK, a.K + head, k0, S, 1.0f);
    load_tile<DH>(sV, a.Vx + head, k0, S, 1.0f);

    float dv[4][CPT], dk[4][CPT];      // keys ty + 16 b, columns tx CPT + c
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < CPT; ++c) { dv[r][c] = 0.0f; dk[r][c] = 0.0f; }

    // query tiles that can see these keys: from the diagonal on (causal); a pure window ends them early
    const int q_begin = causal ? (k0 / kTS) * kTS : 0;
    int q_stop = S;
    if (shun && a.stride <= 0) q_stop = min(S, k_last + a.window + 1);
    for (int q0 = q_begin; q0 < q_stop; q0 += kTS) {
        const int q_last = min(S, q0 + kTS) - 1;
        if (!tile_visible(a, q0, q_last, k0)) continue;
        __syncthreads();
        load_tile<DH>(sQ, a.Qx + head, q0, S, 1.0f);
        load_tile<DH>(sG, a.dO + head, q0, S, a.w);
        if (tid < kTS) {
            const int i = q0 + tid;
            sL[tid] = i < S ? a.lse[(int64_t)blockIdx.y * S + i] : INFINITY;
            sD[tid] = i < S ? a.delta[(int64_t)blockIdx.y * S + i] : 0.0f;
        }
        __syncthreads();
        float s[4][4], dp[4][4];
        gemm_nt<DH>(sQ, sK, ty, tx, s);      // rows: queries ty + 16 r, columns: keys tx + 16 b
        gemm_nt<DH>(sG, sV, ty, tx, dp);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int il = ty + 16 * r, i = q0 + il;
            const float lse = sL[il], dlt = sD[il];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int jl = tx + 16 * b, j = k0 + jl;
                const bool ok = i < S && j < S && key_allowed(i, j, causal, shun, a.window, a.stride);
                const float p = ok ? expf(s[r][b] * a.scale - lse) : 0.0f;
                sPt[jl * kPP + il] = p;
                sDt[jl * kPP + il] = p * (dp[r][b] - dlt) * a.scale;
            }
        }
        __syncthreads();
        gemm_nn<DH>(sPt, sG, ty, tx, dv);    // dv[key][c] += sum_i p[i][key] d_out[i][c]
        gemm_nn<DH>(sDt, sQ, ty, tx, dk);    // dk[key][c] += sum_i ds[i][key] q[i][c]
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int j = k0 + ty + 16 * r;
        if (j >= S) continue;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int64_t off = head + (int64_t)j * DH + tx * CPT + c;
            a.dVx[off] = dv[r][c];
            a.dK[off] = a.accumulate_dk ? a.dK[off] + dk[r][c] : dk[r][c];
        }
    }
}

// Q_adv and V_s of every head (ns_advect_kernel, ns_diffuse_kernel, cuda/ModelGPU.cu:443-471; the central
// stencil is navier_stokes_attention's, include/Attention.hpp:168-182)
__global__ void bwd_prologue_kernel(const float* __restrict__ Q, const float* __restrict__ V, float* __restrict__ Qa,
                                    float* __restrict__ Vs, int S, int DH, float eta, float nu, int mode, int64_t total) {
    for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)((x / DH) % S);
        const float q = Q[x], v = V[x];
        const float qp = i > 0 ? Q[x - DH] : q;
        Qa[x] = q + eta * (q - qp);
        float vs = v;
        if (mode == LOGOS_DIFFUSE_CAUSAL) {
            const float vp = i > 0 ? V[x - DH] : v;
            vs = (1.0f - nu) * v + nu * vp;
        } else if (mode == LOGOS_DIFFUSE_CENTRAL) {
            const float vl = i > 0 ? V[x - DH] : v, vr = i < S - 1 ? V[x + DH] : v;
            vs = (1.0f - nu) * v + (nu * 0.5f) * (vl + vr);
        }
        Vs[x] = vs;
    }
}

// dQ, dV (+)= the transposed stencils applied to dQ_adv, dV_s (ns_advect_bwd_kernel, ns_diffuse_bwd_kernel,
// cuda/ModelGPU.cu:453-482); `ns` = 0 copies / adds the path's gradients unchanged
__global__ void bwd_adjoint_kernel(const float* __restrict__ dQa, const float* __restrict__ dVs, float* __restrict__ dQ,
                                   float* __restrict__ dV, int S, int DH, float eta, float nu, int mode, int ns,
                                   int accumulate, int64_t total) {
    for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)((x / DH) % S);
        float gq = dQa[x], gv = dVs[x];
        if (ns) {
            gq = dQa[x] * (i == 0 ? 1.0f : 1.0f + eta);
            if (i + 1 < S) gq -= eta * dQa[x + DH];
            if (mode == LOGOS_DIFFUSE_CAUSAL) {
                gv = (1.0f - nu) * dVs[x];
                if (i + 1 < S) gv += nu * dVs[x + DH];
                if (i == 0) gv += nu * dVs[x];
            } else if (mode == LOGOS_DIFFUSE_CENTRAL) {
                gv = (1.0f - nu) * dVs[x];
                if (i + 1 < S) gv += 0.5f * nu * dVs[x + DH];
                if (i == 0) gv += 0.5f * nu * dVs[x];
                if (i > 0) gv += 0.5f * nu * dVs[x - DH];
                if (i == S - 1) gv += 0.5f * nu * dVs[x];
            }
        }
        if (accumulate) { dQ[x] += gq; dV[x] += gv; }
        else { dQ[x] = gq; dV[x] = gv; }
    }
}

template <int DH>
int run_path(logos_ctx* ctx, BwdArgs& a, int BH) {
    constexpr int LD = DH + 4;
    const int smem_rows = (4 * kTS * LD + kTS * kPP) * (int)sizeof(float);
    const int smem_keys = (4 * kTS * LD + 2 * kTS * kPP + 2 * kTS) * (int)sizeof(float);
    if (int rc = ensure_smem_limit(ctx, bwd_rows_kernel<DH>, smem_rows)) return rc;
    if (int rc = ensure_smem_limit(ctx, bwd_keys_kernel<DH>, smem_keys)) return rc;
    dim3 grid((a.S + kTS - 1) / kTS, BH);
    bwd_rows_kernel<DH><<<grid, kBwdThreads, smem_rows, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "bwd_rows_kernel");
    bwd_keys_kernel<DH><<<grid, kBwdThreads, smem_keys, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "bwd_keys_kernel");
    return LOGOS_OK;
}

}  // namespace

// dQ, dV (+)= the transposed stencils applied to a path's dQ_adv, dV_s (shared with the tensor-core backward)
int attention_bwd_adjoint(logos_ctx* ctx, const float* dQa, const float* dVs, float* dQ, float* dV, int S, int DH,
                          float eta, float nu, int mode, int ns, int accumulate, int64_t total) {
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 16);
    bwd_adjoint_kernel<<<blocks, 256, 0, ctx->stream>>>(dQa, dVs, dQ, dV, S, DH, eta, nu, mode, ns, accumulate, total);
    LOGOS_LAUNCH_CHECK(ctx, "bwd_adjoint_kernel");
    return LOGOS_OK;
}

size_t attention_bwd_workspace_bytes(int B, int H, int S, int DH) {
    if (B <= 0 || H <= 0 || S <= 0 || DH <= 0) return 0;
    const size_t t = ((size_t)B * H * S * DH * sizeof(float) + 255) & ~(size_t)255;
    const size_t r = ((size_t)B * H * S * sizeof(float) + 255) & ~(size_t)255;
    return kWorkspaceCounterBytes + 4 * t + 2 * r;     // (decode's counters,) Q_adv, V_s, dQ_adv, dV_s; log-sum-exp, delta
}

int attention_bwd(logos_ctx* ctx, const float* Q, const float* K, const float* V, const float* dO, float* dQ, float* dK,
                  float* dV, int B, int H, int S, int DH, const logos_attn_params* p) {
    if (!Q || !K || !V || !dO || !dQ || !dK || !dV || B <= 0 || H <= 0 || S <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_bwd: bad pointer or extent");
    if (DH != 32 && DH != 64 && DH != 128)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention_bwd: DH = %d (32, 64 or 128)", DH);
    if ((int64_t)B * H > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention_bwd: B*H > 65535");
    const void* ptrs[7] = {Q, K, V, dO, dQ, dK, dV};
    for (const void* q : ptrs)
        if (!aligned16(q)) return fail(ctx, LOGOS_ERR_ALIGNMENT, "attention_bwd: tensors must be 16-byte aligned");
    const size_t need = attention_bwd_workspace_bytes(B, H, S, DH);
    if (!ctx->workspace || ctx->workspace_bytes < need)
        return fail(ctx, LOGOS_ERR_WORKSPACE, "attention_bwd: workspace of %zu bytes needed, %zu reserved "
                    "(logos_attention_bwd_workspace_bytes / logos_ctx_reserve)", need, ctx->workspace_bytes);
    const int BH = B * H;
    const int64_t total = (int64_t)BH * S * DH;
    const size_t t = ((size_t)total * sizeof(float) + 255) & ~(size_t)255;
    const size_t r = ((size_t)BH * S * sizeof(float) + 255) & ~(size_t)255;
    char* ws = static_cast<char*>(ctx->workspace) + kWorkspaceCounterBytes;
    float *Qa = (float*)ws, *Vs = (float*)(ws + t), *dQa = (float*)(ws + 2 * t), *dVs = (float*)(ws + 3 * t);
    float *lse = (float*)(ws + 4 * t), *delta = (float*)(ws + 4 * t + r);

    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    const bool std_on = !ns_any || p->ns_alpha < 1.0f;
    const int mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    const int ew_blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 16);

    BwdArgs a{};
    a.K = K; a.dO = dO; a.dQx = dQa; a.dK = dK; a.dVx = dVs; a.lse = lse; a.delta = delta;
    a.S = S; a.scale = p->scale; a.causal = p->causal;
    a.shunyam = shunyam_active(p->window, S) ? 1 : 0;
    a.window = p->window; a.stride = p->stride;
    auto run = [&](BwdArgs& x) {
        return DH == 32 ? run_path<32>(ctx, x, BH) : (DH == 64 ? run_path<64>(ctx, x, BH) : run_path<128>(ctx, x, BH));
    };
    bool first = true;
    if (ns_any) {
        bwd_prologue_kernel<<<ew_blocks, 256, 0, ctx->stream>>>(Q, V, Qa, Vs, S, DH, p->ns_eta, p->ns_nu, mode, total);
        LOGOS_LAUNCH_CHECK(ctx, "bwd_prologue_kernel");
        a.Qx = Qa; a.Vx = Vs; a.w = p->ns_alpha; a.accumulate_dk = 0;
        if (int rc = run(a)) return rc;
        bwd_adjoint_kernel<<<ew_blocks, 256, 0, ctx->stream>>>(dQa, dVs, dQ, dV, S, DH, p->ns_eta, p->ns_nu, mode, 1, 0, total);
        LOGOS_LAUNCH_CHECK(ctx, "bwd_adjoint_kernel");
        first = false;
    }
    if (std_on) {
        a.Qx = Q; a.Vx = V; a.w = ns_any ? 1.0f - p->ns_alpha : 1.0f; a.accumulate_dk = first ? 0 : 1;
        if (int rc = run(a)) return rc;
        bwd_adjoint_kernel<<<ew_blocks, 256, 0, ctx->stream>>>(dQa, dVs, dQ, dV, S, DH, 0.0f, 0.0f, LOGOS_DIFFUSE_NONE, 0,
                                                               first ? 0 : 1, total);
        LOGOS_LAUNCH_CHECK(ctx, "bwd_adjoint_kernel");
    }
    return LOGOS_OK;
}

}  // namespace logos
