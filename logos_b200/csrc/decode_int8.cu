// decode_int8.cu -- decode attention that reads the Nikhilam INT8 KV cache directly.
//
// For every (sequence, head) the query is the newest token (position len-1); its
// attention row over the cached keys is
//     out = sum_j softmax_j(scale * q_adv . K_j) * Vs_j
// with K_j = k_scale * int8 row, Vs the (optionally diffused) V rows and q_adv the
// advected query.  Numerically this is nikhilam_dequantize_kernel + ns_advect_kernel
// + ns_diffuse_kernel + the last row of flash_attention_kernel of LOGOS
// (cuda/ModelGPU.cu:343-351,443-471, cuda/VedicGEMM.cu:901-1062); the reference
// itself has no incremental decode (cuda/train_gpu.cu:2037-2046).
//
// The path is HBM-bound (one byte of K and one of V per key and channel, ~2 FMA per
// byte), so it runs on the SIMT pipes: every lane issues 16-byte loads, a warp-wide
// load covers 8 consecutive 64-byte rows (512 contiguous bytes), four such loads are
// kept in flight per lane, and int8 -> fp32 happens in registers.
//
// Dense contexts are split over the key axis (split-K): CTA (s, bh) handles keys
// [s*chunk, (s+1)*chunk) of pair bh, writes (max, sum, 64 partial outputs) to the
// workspace and the last CTA to arrive for a pair merges the partials.  Arrival is
// counted with one atomic per CTA; nobody waits on anybody, so the kernel cannot
// hang on a missing peer.
//
// V-diffusion is applied to the softmax weights instead of to V (the stencil is
// linear along the key axis):  sum_j p_j Vs_j = sum_r w_r V_r  with
//   causal : w_r = (1-nu) p_r + nu p_{r+1}             (+ nu   p_0 at r = 0)
//   central: w_r = (1-nu) p_r + nu/2 (p_{r-1}+p_{r+1}) (+ nu/2 p_0 at r = 0,
//                                                       + nu/2 p_{n-1} at r = n-1)
// so V is still read exactly once.
#include "common.cuh"

namespace logos {
namespace {

constexpr int kDH = 64;          // head dimension of the vector path
constexpr int kThreads = 256;    // 8 warps
constexpr int kWarps = kThreads / 32;
constexpr int kRowsPerWarp = 8;  // rows covered by one warp-wide 16-byte load
constexpr int kRowsPerIter = kWarps * kRowsPerWarp;  // 64
constexpr int kUnroll = 4;       // 16-byte loads in flight per lane
constexpr int kMaxChunk = 1024;  // keys per CTA in the dense kernel
constexpr int kPartial = 2 + kDH;  // (max, sum, acc[64]) per split
constexpr size_t kCounterBytes = 64 * 1024;  // head of the workspace: arrival counters
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeArgs {
    const __half* q;
    const __half* q_prev;
    const int8_t* k_cache;
    const int8_t* v_cache;
    const float* k_scale;
    const float* v_scale;
    const int32_t* len;
    float* out;
    float* partials;       // [BH][splits][paths][kPartial]
    unsigned int* counters;  // [BH], zero between launches
    int H, S_max, chunk;
    float scale, eta, nu, alpha;
    int diffuse_mode, window, stride;
};

// Four int8 lanes of a 32-bit word -> four floats.  x ^ 0x80 is the value biased
// by 128 as an unsigned byte; dropping that byte into the mantissa of 2^23 gives
// 8388608 + 128 + x exactly, and one subtraction recovers x.
__device__ __forceinline__ void cvt4(uint32_t w, float* f) {
    uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - 8388736.0f;
}

__device__ __forceinline__ uint4 ld_stream(const int8_t* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ float dot16(const uint4& w, const float* q) {
    float f[16];
    cvt4(w.x, f);
    cvt4(w.y, f + 4);
    cvt4(w.z, f + 8);
    cvt4(w.w, f + 12);
    float a = 0.0f, b = 0.0f;
#pragma unroll
    for (int k = 0; k < 16; k += 2) {
        a = fmaf(f[k], q[k], a);
        b = fmaf(f[k + 1], q[k + 1], b);
    }
    return a + b;
}

__device__ __forceinline__ void axpy16(const uint4& w, float p, float* acc) {
    float f[16];
    cvt4(w.x, f);
    cvt4(w.y, f + 4);
    cvt4(w.z, f + 8);
    cvt4(w.w, f + 12);
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = fmaf(p, f[k], acc[k]);
}

// The query slice of this lane (16 channels), advected and pre-multiplied by
// scale * k_scale * log2(e) so that scores come out in the exp2 domain.
template <bool BLEND>
__device__ __forceinline__ void load_query(const DecodeArgs& a, int bh, int pos, int part,
                                           float* qn, float* qs) {
    const __half* q = a.q + (int64_t)bh * kDH + part * 16;
    const bool advect = (a.eta != 0.0f) && (pos > 0) && (a.q_prev != nullptr);
    const __half* qp = advect ? a.q_prev + (int64_t)bh * kDH + part * 16 : q;
    const float f = a.scale * a.k_scale[bh] * kLog2e;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        float x = __half2float(q[k]);
        float xp = __half2float(qp[k]);
        float xa = x + a.eta * (x - xp);  // ns_advect_kernel; xa == x when not advecting
        qn[k] = xa * f;
        if (BLEND) qs[k] = x * f;
    }
}

__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) r = fmaxf(r, red[w]);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) r += red[w];
    __syncthreads();
    return r;
}

// Sums the per-lane 16-channel accumulators over the 8 rows of a warp and over the
// warps of the block; on return threads 0..63 hold channel threadIdx.x.
__device__ __forceinline__ float block_reduce_acc(float* acc, float (*red)[kDH]) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 4);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 8);
        acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], 16);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane < 4) {
#pragma unroll
        for (int k = 0; k < 16; ++k) red[warp][lane * 16 + k] = acc[k];
    }
    __syncthreads();
    float r = 0.0f;
    if (threadIdx.x < kDH) {
#pragma unroll
        for (int w = 0; w < kWarps; ++w) r += red[w][threadIdx.x];
    }
    __syncthreads();
    return r;
}

// ---------------------------------------------------------------------------
// Dense context: every cached key is visible.
template <bool BLEND>
__global__ void __launch_bounds__(kThreads, 3)
decode_dense_kernel(const DecodeArgs a) {
    constexpr int PATHS = BLEND ? 2 : 1;
    __shared__ float p_ns[kMaxChunk + 2];             // p_ns[1 + t], zero halo at both ends
    __shared__ float p_std[BLEND ? kMaxChunk : 1];
    __shared__ float red[kWarps];
    __shared__ float red_acc[kWarps][kDH];
    __shared__ unsigned int is_last;

    const int bh = blockIdx.y, split = blockIdx.x, n_splits = gridDim.x;
    const int b = bh / a.H;
    int len = a.len[b];
    len = len < 0 ? 0 : (len > a.S_max ? a.S_max : len);
    const int pos = len - 1;
    const int c0 = split * a.chunk;
    const int c1 = min(len, c0 + a.chunk);
    const int n = c1 - c0;  // keys of this CTA (<= 0: nothing to do but report)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_in_warp = lane >> 2, part = lane & 3;

    const int8_t* kbase = a.k_cache + (int64_t)bh * a.S_max * kDH + part * 16;
    const int8_t* vbase = a.v_cache + (int64_t)bh * a.S_max * kDH + part * 16;

    float m_ns = -INFINITY, l_ns = 0.0f, m_std = -INFINITY, l_std = 0.0f;
    float o_ns = 0.0f, o_std = 0.0f;  // channel tid (tid < 64) after the reductions

    if (n > 0) {
        float qn[16], qs[BLEND ? 16 : 1];
        load_query<BLEND>(a, bh, pos, part, qn, qs);

        // ---- scores ----
        for (int r0 = warp * kRowsPerWarp; r0 < n; r0 += kRowsPerIter * kUnroll) {
            uint4 w[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int r = r0 + u * kRowsPerIter + row_in_warp;
                w[u] = (r < n) ? ld_stream(kbase + (int64_t)(c0 + r) * kDH) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int r = r0 + u * kRowsPerIter + row_in_warp;
                float s = dot16(w[u], qn);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                float s2 = 0.0f;
                if (BLEND) {
                    s2 = dot16(w[u], qs);
                    s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
                    s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
                }
                if (part == 0 && r < n) {
                    p_ns[1 + r] = s;
                    if (BLEND) p_std[r] = s2;
                }
            }
        }
        if (tid == 0) { p_ns[0] = 0.0f; p_ns[1 + n] = 0.0f; }
        __syncthreads();

        // ---- softmax over this chunk ----
        float mx = -INFINITY, mx2 = -INFINITY;
        for (int t = tid; t < n; t += kThreads) {
            mx = fmaxf(mx, p_ns[1 + t]);
            if (BLEND) mx2 = fmaxf(mx2, p_std[t]);
        }
        m_ns = block_max(mx, red);
        if (BLEND) m_std = block_max(mx2, red);
        float sum = 0.0f, sum2 = 0.0f;
        for (int t = tid; t < n; t += kThreads) {
            float e = exp2f(p_ns[1 + t] - m_ns);
            p_ns[1 + t] = e;
            sum += e;
            if (BLEND) {
                float e2 = exp2f(p_std[t] - m_std);
                p_std[t] = e2;
                sum2 += e2;
            }
        }
        l_ns = block_sum(sum, red);  // also orders the p_* writes before the reads below
        if (BLEND) l_std = block_sum(sum2, red);

        // ---- weights * V ----
        float cC = 1.0f, cL = 0.0f, cR = 0.0f, b0 = 0.0f, bN = 0.0f;
        if (a.diffuse_mode == LOGOS_DIFFUSE_CAUSAL) {
            cC = 1.0f - a.nu; cR = a.nu; b0 = a.nu;
        } else if (a.diffuse_mode == LOGOS_DIFFUSE_CENTRAL) {
            cC = 1.0f - a.nu; cR = cL = 0.5f * a.nu; b0 = bN = 0.5f * a.nu;
        }
        float acc[16], acc2[BLEND ? 16 : 1];
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[k] = 0.0f;
        if (BLEND) {
#pragma unroll
            for (int k = 0; k < 16; ++k) acc2[k] = 0.0f;
        }
        for (int r0 = warp * kRowsPerWarp; r0 < n; r0 += kRowsPerIter * kUnroll) {
            uint4 w[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int r = r0 + u * kRowsPerIter + row_in_warp;
                w[u] = (r < n) ? ld_stream(vbase + (int64_t)(c0 + r) * kDH) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                int r = r0 + u * kRowsPerIter + row_in_warp;
                if (r < n) {
                    float pc = p_ns[1 + r];
                    float wgt = cC * pc + cR * p_ns[2 + r] + cL * p_ns[r];
                    int j = c0 + r;
                    if (j == 0) wgt += b0 * pc;
                    if (j == len - 1) wgt += bN * pc;
                    axpy16(w[u], wgt, acc);
                    if (BLEND) axpy16(w[u], p_std[r], acc2);
                }
            }
        }
        // halo rows: the row before the chunk takes cR * p(first key), the row after
        // it takes cL * p(last key)
        if (warp == 0 && lane < 4 && c0 > 0 && cR != 0.0f) {
            uint4 w = ld_stream(vbase + (int64_t)(c0 - 1) * kDH);
            axpy16(w, cR * p_ns[1], acc);
        }
        if (warp == 1 && lane < 4 && c1 < len && cL != 0.0f) {
            uint4 w = ld_stream(vbase + (int64_t)c1 * kDH);
            axpy16(w, cL * p_ns[n], acc);
        }
        o_ns = block_reduce_acc(acc, red_acc);
        if (BLEND) o_std = block_reduce_acc(acc2, red_acc);
    }

    const float vs = a.v_scale[bh];
    float* outp = a.out + (int64_t)bh * kDH;

    if (n_splits == 1) {
        if (tid < kDH) {
            float r_ns = (l_ns > 0.0f) ? o_ns / l_ns : 0.0f;
            float r = r_ns;
            if (BLEND) {
                float r_std = (l_std > 0.0f) ? o_std / l_std : 0.0f;
                r = (1.0f - a.alpha) * r_std + a.alpha * r_ns;
            }
            outp[tid] = r * vs;
        }
        return;
    }

    // ---- publish this split's partial, merge if last ----
    float* mine = a.partials + ((int64_t)bh * n_splits + split) * PATHS * kPartial;
    if (tid < kDH) {
        mine[2 + tid] = o_ns;
        if (BLEND) mine[kPartial + 2 + tid] = o_std;
    }
    if (tid == 0) {
        mine[0] = m_ns; mine[1] = l_ns;
        if (BLEND) { mine[kPartial] = m_std; mine[kPartial + 1] = l_std; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned int prev = atomicAdd(a.counters + bh, 1u);
        is_last = (prev == (unsigned int)(n_splits - 1));
        if (is_last) a.counters[bh] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (tid < kDH) {
        const float* all = a.partials + (int64_t)bh * n_splits * PATHS * kPartial;
        float r_path[PATHS];
#pragma unroll
        for (int pth = 0; pth < PATHS; ++pth) {
            float M = -INFINITY;
            for (int s = 0; s < n_splits; ++s)
                M = fmaxf(M, __ldcg(all + (s * PATHS + pth) * kPartial));
            float num = 0.0f, den = 0.0f;
            for (int s = 0; s < n_splits; ++s) {
                const float* ps = all + (s * PATHS + pth) * kPartial;
                float ms = __ldcg(ps);
                float f = (ms == -INFINITY) ? 0.0f : exp2f(ms - M);
                den = fmaf(f, __ldcg(ps + 1), den);
                num = fmaf(f, __ldcg(ps + 2 + tid), num);
            }
            r_path[pth] = (den > 0.0f) ? num / den : 0.0f;
        }
        float r = r_path[0];
        if (BLEND) r = (1.0f - a.alpha) * r_path[1] + a.alpha * r_path[0];
        outp[tid] = r * vs;
    }
}

// ---------------------------------------------------------------------------
// Shunyam context: only the window [pos-window, pos] and the landmarks
// (j % stride == 0) before it are visible; one CTA per pair enumerates them.
// Visible keys are few and scattered, so V diffusion reads the neighbour rows.
template <bool BLEND>
__global__ void __launch_bounds__(kThreads)
decode_sparse_kernel(const DecodeArgs a, int t_max) {
    extern __shared__ float dyn[];
    float* p_ns = dyn;                 // [t_max]
    float* p_std = dyn + t_max;        // [t_max] when BLEND
    __shared__ float red[kWarps];
    __shared__ float red_acc[kWarps][kDH];

    const int bh = blockIdx.x;
    const int b = bh / a.H;
    int len = a.len[b];
    len = len < 0 ? 0 : (len > a.S_max ? a.S_max : len);
    const int pos = len - 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_in_warp = lane >> 2, part = lane & 3;
    float* outp = a.out + (int64_t)bh * kDH;
    if (len == 0) {
        if (tid < kDH) outp[tid] = 0.0f;
        return;
    }
    // enumeration of visible keys: landmarks before the window, then the window
    const bool active = shunyam_active(a.window, len);
    const int win0 = active ? max(0, pos - a.window) : 0;
    const int n_land = (active && a.stride > 0) ? (win0 + a.stride - 1) / a.stride : 0;
    const int T = n_land + (pos - win0 + 1);
    auto key_of = [&](int t) { return t < n_land ? t * a.stride : win0 + (t - n_land); };

    const int8_t* kbase = a.k_cache + (int64_t)bh * a.S_max * kDH + part * 16;
    const int8_t* vbase = a.v_cache + (int64_t)bh * a.S_max * kDH + part * 16;
    float qn[16], qs[BLEND ? 16 : 1];
    load_query<BLEND>(a, bh, pos, part, qn, qs);

    for (int t0 = warp * kRowsPerWarp; t0 < T; t0 += kRowsPerIter * kUnroll) {
        uint4 w[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int t = t0 + u * kRowsPerIter + row_in_warp;
            w[u] = (t < T) ? ld_stream(kbase + (int64_t)key_of(t) * kDH) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int t = t0 + u * kRowsPerIter + row_in_warp;
            float s = dot16(w[u], qn);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            float s2 = 0.0f;
            if (BLEND) {
                s2 = dot16(w[u], qs);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
            }
            if (part == 0 && t < T) {
                p_ns[t] = s;
                if (BLEND) p_std[t] = s2;
            }
        }
    }
    __syncthreads();
    float mx = -INFINITY, mx2 = -INFINITY;
    for (int t = tid; t < T; t += kThreads) {
        mx = fmaxf(mx, p_ns[t]);
        if (BLEND) mx2 = fmaxf(mx2, p_std[t]);
    }
    const float m_ns = block_max(mx, red);
    const float m_std = BLEND ? block_max(mx2, red) : 0.0f;
    float sum = 0.0f, sum2 = 0.0f;
    for (int t = tid; t < T; t += kThreads) {
        float e = exp2f(p_ns[t] - m_ns);
        p_ns[t] = e;
        sum += e;
        if (BLEND) {
            float e2 = exp2f(p_std[t] - m_std);
            p_std[t] = e2;
            sum2 += e2;
        }
    }
    const float l_ns = block_sum(sum, red);
    const float l_std = BLEND ? block_sum(sum2, red) : 1.0f;

    float acc[16], acc2[BLEND ? 16 : 1];
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[k] = 0.0f;
    if (BLEND) {
#pragma unroll
        for (int k = 0; k < 16; ++k) acc2[k] = 0.0f;
    }
    const int mode = a.diffuse_mode;
    for (int t = warp * kRowsPerWarp + row_in_warp; t < T; t += kRowsPerIter) {
        int j = key_of(t);
        uint4 wc = ld_stream(vbase + (int64_t)j * kDH);
        float p = p_ns[t];
        if (mode == LOGOS_DIFFUSE_NONE) {
            axpy16(wc, p, acc);
        } else {
            // Vs_j = (1-nu) V_j + nu V_{j-1}            (cuda/ModelGPU.cu:463-471), or
            // Vs_j = (1-nu) V_j + nu/2 (V_{j-1}+V_{j+1}) (include/Attention.hpp:173-181),
            // neighbours clamped to [0, len-1]
            int jl = j > 0 ? j - 1 : 0;
            uint4 wl = ld_stream(vbase + (int64_t)jl * kDH);
            if (mode == LOGOS_DIFFUSE_CAUSAL) {
                axpy16(wc, p * (1.0f - a.nu), acc);
                axpy16(wl, p * a.nu, acc);
            } else {
                int jr = j < len - 1 ? j + 1 : len - 1;
                uint4 wr = ld_stream(vbase + (int64_t)jr * kDH);
                axpy16(wc, p * (1.0f - a.nu), acc);
                axpy16(wl, p * 0.5f * a.nu, acc);
                axpy16(wr, p * 0.5f * a.nu, acc);
            }
        }
        if (BLEND) axpy16(wc, p_std[t], acc2);
    }
    float o_ns = block_reduce_acc(acc, red_acc);
    float o_std = BLEND ? block_reduce_acc(acc2, red_acc) : 0.0f;
    if (tid < kDH) {
        float r = (l_ns > 0.0f) ? o_ns / l_ns : 0.0f;
        if (BLEND) {
            float r_std = (l_std > 0.0f) ? o_std / l_std : 0.0f;
            r = (1.0f - a.alpha) * r_std + a.alpha * r;
        }
        outp[tid] = r * a.v_scale[bh];
    }
}

int pick_chunk(const logos_ctx* ctx, int BH, int S_max) {
    // largest chunk that still gives every SM about eight CTAs
    int chunk = kMaxChunk;
    while (chunk > 128 && (int64_t)BH * ((S_max + chunk - 1) / chunk) < (int64_t)ctx->sm_count * 8)
        chunk >>= 1;
    return chunk;
}

}  // namespace

size_t decode_workspace_bytes(int B, int H, int S_max, int DH) {
    (void)DH;
    if (B <= 0 || H <= 0 || S_max <= 0) return 0;
    size_t splits = ((size_t)S_max + 127) / 128;  // worst case: smallest chunk
    return kCounterBytes + (size_t)B * H * splits * 2 * kPartial * sizeof(float);
}

int decode_int8(logos_ctx* ctx, const void* q, const void* q_prev, const int8_t* k_cache,
                const int8_t* v_cache, const float* k_scale, const float* v_scale,
                const int32_t* len, int B, int H, int S_max, int DH,
                const logos_attn_params* p, float* out) {
    if (!q || !k_cache || !v_cache || !k_scale || !v_scale || !len || !out || !p || B <= 0 ||
        H <= 0 || S_max <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: bad pointer or extent");
    if (DH != kDH) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: DH must be 64, got %d", DH);
    if (!aligned16(k_cache) || !aligned16(v_cache))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "decode_int8: caches must be 16-byte aligned");
    if (p->diffuse_mode < 0 || p->diffuse_mode > 2)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: bad diffuse_mode");
    if (p->ns_eta != 0.0f && p->ns_alpha > 0.0f && !q_prev)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: q_prev is required when ns_eta != 0");
    const int BH = B * H;
    if ((size_t)BH * sizeof(unsigned int) > kCounterBytes)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: more than 16384 (b,h) pairs");

    DecodeArgs a;
    a.q = (const __half*)q;
    a.q_prev = (const __half*)q_prev;
    a.k_cache = k_cache; a.v_cache = v_cache;
    a.k_scale = k_scale; a.v_scale = v_scale;
    a.len = len; a.out = out;
    a.H = H; a.S_max = S_max;
    a.scale = p->scale;
    a.window = p->window; a.stride = p->stride;
    // alpha <= 0 switches the Navier-Stokes terms off (include/Attention.hpp:236)
    const bool ns_any = p->ns_alpha > 0.0f &&
                        (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.diffuse_mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    a.alpha = p->ns_alpha;
    const bool blend = ns_any && p->ns_alpha < 1.0f;

    if (p->window > 0) {
        int t_max = p->window + 1 + (p->stride > 0 ? (S_max + p->stride - 1) / p->stride : 0);
        if (t_max > S_max) t_max = S_max;
        if (t_max < p->window + 1) t_max = p->window + 1;
        size_t smem = sizeof(float) * (size_t)t_max * (blend ? 2 : 1);
        if (smem > 160 * 1024)
            return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: %d visible keys exceed the sparse kernel", t_max);
        a.partials = nullptr; a.counters = nullptr; a.chunk = 0;
        if (blend) {
            LOGOS_CUDA_TRY(ctx, cudaFuncSetAttribute(decode_sparse_kernel<true>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            decode_sparse_kernel<true><<<BH, kThreads, smem, ctx->stream>>>(a, t_max);
        } else {
            LOGOS_CUDA_TRY(ctx, cudaFuncSetAttribute(decode_sparse_kernel<false>,
                                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            decode_sparse_kernel<false><<<BH, kThreads, smem, ctx->stream>>>(a, t_max);
        }
        LOGOS_LAUNCH_CHECK(ctx, "decode_sparse_kernel");
        return LOGOS_OK;
    }

    a.chunk = pick_chunk(ctx, BH, S_max);
    const int n_splits = (S_max + a.chunk - 1) / a.chunk;
    if (BH > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: B*H > 65535");
    if (n_splits > 1) {
        size_t need = kCounterBytes + (size_t)BH * n_splits * (blend ? 2 : 1) * kPartial * sizeof(float);
        if (!ctx->workspace || ctx->workspace_bytes < need)
            return fail(ctx, LOGOS_ERR_WORKSPACE,
                        "decode_int8: workspace of %zu bytes needed, %zu reserved "
                        "(logos_decode_workspace_bytes / logos_ctx_reserve)",
                        need, ctx->workspace_bytes);
        a.counters = (unsigned int*)ctx->workspace;
        a.partials = (float*)((char*)ctx->workspace + kCounterBytes);
    } else {
        a.counters = nullptr; a.partials = nullptr;
    }
    dim3 grid(n_splits, BH);
    if (blend) decode_dense_kernel<true><<<grid, kThreads, 0, ctx->stream>>>(a);
    else       decode_dense_kernel<false><<<grid, kThreads, 0, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "decode_dense_kernel");
    return LOGOS_OK;
}

}  // namespace logos
