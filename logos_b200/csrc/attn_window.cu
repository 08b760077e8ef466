// attn_window.cu -- Shunyam sparse attention (sliding window + stride landmarks), DH = 64,
// BF16 / FP16 inputs, with the Navier-Stokes prologue fused in.
//
// Rule (include/Attention.hpp:80-98, cuda/VedicGEMM.cu:987-996 of LOGOS): query i sees key j iff
// j <= i and (j >= i - window or j % stride == 0).  The reference kernel still visits every KV
// tile and masks (cuda/VedicGEMM.cu:952); here a CTA touches only what its 64 query rows can see:
//   * the window tiles: keys [q0 - window, q0 + 63], contiguous, anchored at the CTA's last row and
//     walked downwards (window 64 = two 64-key tiles; the one key below feeds the diffusion stencil
//     and is added as a single row);
//   * the landmark tiles: keys m * stride below the window, gathered 64 at a time straight from
//     their strided rows with 16-byte cp.async copies.
// The path is HBM-bound (Q, K, V read once, O written once; neighbouring CTAs share K/V through
// L2), the arithmetic is small, so the kernel is built for occupancy, not for peak math: 128
// threads, 48 KB of shared memory, mma.sync m16n8k16 with fp32 accumulation, several CTAs per SM.
//
// Precision: Q_adv = Q + eta (Q - Q_prev) (ns_advect_kernel, cuda/ModelGPU.cu:443-451) is formed in
// fp32 and fed to the tensor cores as an exact hi + lo pair of 16-bit fragments; so are the
// softmax weights.  V-diffusion (ns_diffuse_kernel, cuda/ModelGPU.cu:463-471) is folded into the
// weights: in the window part w_r = (1-nu) p_r + nu p_{r+1} (neighbours are adjacent keys), in the
// landmark part the gathered rows V[j] and V[j-1] take (1-nu) p_j and nu p_j.
#include "common.cuh"

namespace logos {
namespace {

constexpr int kWM = 64;          // query rows per CTA (16 per warp)
constexpr int kWN = 64;          // keys per tile
constexpr int kWD = 64;          // head dimension
constexpr int kWThreads = 128;
constexpr int kWTile = kWN * kWD * 2;          // 8 KiB
constexpr int kWStage = 3 * kWTile;            // K, V, V[j-1]
constexpr int kWSmem = 2 * kWStage;            // two stages

struct WinArgs {
    const void* Q; const void* K; const void* V; void* O;
    int S, window, stride, out_is_f32, in_is_f16, diffuse;
    float c, eta, nu;            // c = scale * log2(e)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    int bytes = valid ? 16 : 0;  // 0 source bytes = zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool F16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (F16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool F16> __device__ __forceinline__ float lo_f(uint32_t w) {
    return F16 ? __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))) : __uint_as_float(w << 16);
}
template <bool F16> __device__ __forceinline__ float hi_f(uint32_t w) {
    return F16 ? __half2float(__ushort_as_half((unsigned short)(w >> 16))) : __uint_as_float(w & 0xffff0000u);
}
// (x, y) -> packed 16-bit pair (x in the low half) and the packed residual pair
template <bool F16> __device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    if (F16) {
        __half2 h = __floats2half2_rn(x, y);
        float2 b = __half22float2(h);
        __half2 l = __floats2half2_rn(x - b.x, y - b.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
        float2 b = __bfloat1622float2(h);
        __nv_bfloat162 l = __floats2bfloat162_rn(x - b.x, y - b.y);
        hi = *reinterpret_cast<uint32_t*>(&h);
        lo = *reinterpret_cast<uint32_t*>(&l);
    }
}
template <bool F16> __device__ __forceinline__ uint32_t pack2(float x, float y) {
    if (F16) { __half2 h = __floats2half2_rn(x, y); return *reinterpret_cast<uint32_t*>(&h); }
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <bool F16, bool DIFF>
__global__ void __launch_bounds__(kWThreads, 4)
shunyam_window_kernel(const WinArgs a) {
    extern __shared__ __align__(128) unsigned char wsm[];
    const uint32_t sb = (uint32_t)__cvta_generic_to_shared(wsm);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = a.S, W = a.window;
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kWM;
    const size_t head = (size_t)blockIdx.y * S * kWD;
    const unsigned short* Qg = reinterpret_cast<const unsigned short*>(a.Q) + head;
    const unsigned short* Kg = reinterpret_cast<const unsigned short*>(a.K) + head;
    const unsigned short* Vg = reinterpret_cast<const unsigned short*>(a.V) + head;
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;   // this thread's two query rows
    const float nu = DIFF ? a.nu : 0.0f, one_m_nu = 1.0f - nu, c = a.c;

    // ---- tile list: window tiles from the diagonal downwards, then landmark tiles ----
    const int i_last = min(S, q0 + kWM) - 1;
    // window tiles are anchored at the CTA's last row, not at multiples of 64: tile ti covers keys
    // [k_hi - 64 ti - 63, k_hi - 64 ti], so window 64 needs exactly two of them
    const int k_hi = q0 + kWM - 1;
    const int k_lo = max(0, q0 - W);
    const int n_win = (k_hi - k_lo) / kWN + 1;
    // landmarks m * stride strictly below the LAST row's window start (rows mask the rest)
    const int lm_end = i_last - W;                          // landmark keys j < lm_end may matter
    const int n_lm = (a.stride > 0 && lm_end > 0) ? (lm_end + a.stride - 1) / a.stride : 0;
    const int n_lmt = (n_lm + kWN - 1) / kWN;
    const int n_tiles = n_win + n_lmt;

    auto load_tile = [&](int ti, int stage) {
        const uint32_t ks = sb + stage * kWStage, vs = ks + kWTile, ps = vs + kWTile;
        const bool lm = ti >= n_win;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + q * kWThreads, r = idx >> 3, ch = idx & 7;
            int key;
            bool valid;
            if (!lm) {
                key = k_hi - kWN * (ti + 1) + 1 + r;
                valid = key >= 0 && key < S;
            } else {
                const int m = (ti - n_win) * kWN + r;
                key = m * a.stride;
                valid = m < n_lm;
            }
            const int kc = valid ? key : 0;
            const uint32_t off = r * 128 + ((ch ^ (r & 7)) << 4);
            cp_async16(ks + off, Kg + (size_t)kc * kWD + ch * 8, valid);
            cp_async16(vs + off, Vg + (size_t)kc * kWD + ch * 8, valid);
            if (DIFF && lm) cp_async16(ps + off, Vg + (size_t)max(kc - 1, 0) * kWD + ch * 8, valid);
        }
    };

    load_tile(0, 0);
    cp_async_commit();

    // ---- Q_adv fragments (hi, lo) straight from global memory: rows row_a / row_b ----
    uint32_t qh[4][4], ql[4][4];
    {
        auto ldq = [&](int row, int col) -> uint32_t {     // two adjacent channels
            return (row >= 0 && row < S) ? *reinterpret_cast<const uint32_t*>(Qg + (size_t)row * kWD + col) : 0u;
        };
        auto adv = [&](int row, int col, uint32_t& hi, uint32_t& lo) {
            uint32_t cur = ldq(row, col), prv = (row > 0) ? ldq(row - 1, col) : cur;
            float x0 = lo_f<F16>(cur), x1 = hi_f<F16>(cur), p0 = lo_f<F16>(prv), p1 = hi_f<F16>(prv);
            split2<F16>(x0 + a.eta * (x0 - p0), x1 + a.eta * (x1 - p1), hi, lo);
        };
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            adv(row_a, kk * 16 + 2 * t, qh[kk][0], ql[kk][0]);
            adv(row_b, kk * 16 + 2 * t, qh[kk][1], ql[kk][1]);
            adv(row_a, kk * 16 + 2 * t + 8, qh[kk][2], ql[kk][2]);
            adv(row_b, kk * 16 + 2 * t + 8, qh[kk][3], ql[kk][3]);
        }
    }
    const bool has_lo = a.eta != 0.0f;

    float o[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    float carry_a = -INFINITY, carry_b = -INFINITY;   // scaled score of column 0 of the window tile above

    for (int ti = 0; ti < n_tiles; ++ti) {
        const int stage = ti & 1;
        if (ti + 1 < n_tiles) load_tile(ti + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t ks = sb + stage * kWStage, vs = ks + kWTile, ps = vs + kWTile;
        const bool lm = ti >= n_win;

        const int kbase = lm ? (ti - n_win) * kWN : k_hi - kWN * (ti + 1) + 1;   // landmark index or first key

        // ---- S = Q_adv K^T : 16 rows x 64 keys per warp ----
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                const int key = (2 * np + (lane >> 4)) * 8 + (lane & 7), ch = kk * 2 + ((lane >> 3) & 1);
                ldsm_x4(ks + key * 128 + ((ch ^ (key & 7)) << 4), b);
                mma16816<F16>(s[2 * np], qh[kk], b[0], b[1]);
                mma16816<F16>(s[2 * np + 1], qh[kk], b[2], b[3]);
                if (has_lo) {
                    mma16816<F16>(s[2 * np], ql[kk], b[0], b[1]);
                    mma16816<F16>(s[2 * np + 1], ql[kk], b[2], b[3]);
                }
            }

        // ---- mask, scale to the log2 domain, online softmax ----
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int col = kbase + n * 8 + 2 * t + e;
                bool ok_a, ok_b;
                if (!lm) {   // window part: j in [i - W, i]
                    ok_a = col <= row_a && col >= row_a - W && col >= 0 && col < S && row_a < S;
                    ok_b = col <= row_b && col >= row_b - W && col >= 0 && col < S && row_b < S;
                } else {     // landmark part: j = m * stride strictly below the row's window
                    const int j = col * a.stride;
                    ok_a = col < n_lm && j < row_a - W && row_a < S;
                    ok_b = col < n_lm && j < row_b - W && row_b < S;
                }
                s[n][e] = ok_a ? s[n][e] * c : -INFINITY;
                s[n][2 + e] = ok_b ? s[n][2 + e] * c : -INFINITY;
                mx_a = fmaxf(mx_a, s[n][e]);
                mx_b = fmaxf(mx_b, s[n][2 + e]);
            }
        // scaled score of this tile's column 0 (lane t == 0 of the quad holds it): the tile below needs it
        const float col0_a = __shfl_sync(0xffffffffu, s[0][0], lane & ~3);
        const float col0_b = __shfl_sync(0xffffffffu, s[0][2], lane & ~3);
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float f_a = (m_a == -INFINITY) ? 0.0f : ex2f(m_a - mn_a);
        const float f_b = (m_b == -INFINITY) ? 0.0f : ex2f(m_b - mn_b);
        const float sub_a = (mn_a == -INFINITY) ? 0.0f : mn_a, sub_b = (mn_b == -INFINITY) ? 0.0f : mn_b;
        m_a = mn_a; m_b = mn_b;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            o[n][0] *= f_a; o[n][1] *= f_a; o[n][2] *= f_b; o[n][3] *= f_b;
        }
        float ps_a = 0.0f, ps_b = 0.0f;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            s[n][0] = ex2f(s[n][0] - sub_a); s[n][1] = ex2f(s[n][1] - sub_a);
            s[n][2] = ex2f(s[n][2] - sub_b); s[n][3] = ex2f(s[n][3] - sub_b);
            ps_a += s[n][0] + s[n][1];
            ps_b += s[n][2] + s[n][3];
        }
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 1);
        ps_a += __shfl_xor_sync(0xffffffffu, ps_a, 2);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 1);
        ps_b += __shfl_xor_sync(0xffffffffu, ps_b, 2);
        l_a = l_a * f_a + ps_a;
        l_b = l_b * f_b + ps_b;

        // ---- diffusion folded into the weights ----
        if (DIFF && ti == n_win - 1 && kbase > 0) {
            // the key just below the lowest window tile takes nu * p(first key of the tile); only the
            // CTA's first rows can see that first key, but the formula holds for all
            const float h_a = nu * __shfl_sync(0xffffffffu, s[0][0], lane & ~3);
            const float h_b = nu * __shfl_sync(0xffffffffu, s[0][2], lane & ~3);
            const unsigned short* vrow = Vg + (size_t)(kbase - 1) * kWD + 2 * t;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const uint32_t v2 = *reinterpret_cast<const uint32_t*>(vrow + n * 8);
                const float v0 = lo_f<F16>(v2), v1 = hi_f<F16>(v2);
                o[n][0] = fmaf(h_a, v0, o[n][0]); o[n][1] = fmaf(h_a, v1, o[n][1]);
                o[n][2] = fmaf(h_b, v0, o[n][2]); o[n][3] = fmaf(h_b, v1, o[n][3]);
            }
        }
        if (DIFF && !lm) {
            // in place: w_r = (1-nu) p_r + nu p_{r+1}; p_{r+1} of the last column comes from the tile
            // above.  Ascending n: everything read from block n+1 is still the original p.
            const float ab_a = (carry_a == -INFINITY) ? 0.0f : ex2f(carry_a - sub_a);
            const float ab_b = (carry_b == -INFINITY) ? 0.0f : ex2f(carry_b - sub_b);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                // neighbour to the right of this thread's pair: lane t+1's first element, or the next
                // block's first element of lane 0, or the tile above
                const float nx_same_a = __shfl_sync(0xffffffffu, s[n][0], (lane & ~3) | ((t + 1) & 3));
                const float nx_same_b = __shfl_sync(0xffffffffu, s[n][2], (lane & ~3) | ((t + 1) & 3));
                const float nx_blk_a = __shfl_sync(0xffffffffu, s[n < 7 ? n + 1 : 7][0], lane & ~3);
                const float nx_blk_b = __shfl_sync(0xffffffffu, s[n < 7 ? n + 1 : 7][2], lane & ~3);
                const float right_a = (t < 3) ? nx_same_a : ((n < 7) ? nx_blk_a : ab_a);
                const float right_b = (t < 3) ? nx_same_b : ((n < 7) ? nx_blk_b : ab_b);
                const float p0a = s[n][0], p1a = s[n][1], p0b = s[n][2], p1b = s[n][3];
                float w0a = one_m_nu * p0a + nu * p1a, w1a = one_m_nu * p1a + nu * right_a;
                float w0b = one_m_nu * p0b + nu * p1b, w1b = one_m_nu * p1b + nu * right_b;
                if (kbase + n * 8 + 2 * t == 0) { w0a += nu * p0a; w0b += nu * p0b; }   // V_s[0] = V[0]
                s[n][0] = w0a; s[n][1] = w1a; s[n][2] = w0b; s[n][3] = w1b;
            }
            carry_a = col0_a;
            carry_b = col0_b;
        }
        // landmark part: the gathered rows V[j] take (1-nu) p_j, the rows V[j-1] take nu p_j
        const float w_main = (DIFF && lm) ? one_m_nu : 1.0f;

        // ---- O += W V (weights as hi + lo 16-bit fragments) ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t ah[4], al[4];
            split2<F16>(w_main * s[2 * kk][0], w_main * s[2 * kk][1], ah[0], al[0]);
            split2<F16>(w_main * s[2 * kk][2], w_main * s[2 * kk][3], ah[1], al[1]);
            split2<F16>(w_main * s[2 * kk + 1][0], w_main * s[2 * kk + 1][1], ah[2], al[2]);
            split2<F16>(w_main * s[2 * kk + 1][2], w_main * s[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ch = 2 * np + (lane >> 4);
                ldsm_x4_t(vs + key * 128 + ((ch ^ (key & 7)) << 4), b);
                mma16816<F16>(o[2 * np], ah, b[0], b[1]);
                mma16816<F16>(o[2 * np + 1], ah, b[2], b[3]);
                mma16816<F16>(o[2 * np], al, b[0], b[1]);
                mma16816<F16>(o[2 * np + 1], al, b[2], b[3]);
            }
            if (DIFF && lm) {
                split2<F16>(nu * s[2 * kk][0], nu * s[2 * kk][1], ah[0], al[0]);
                split2<F16>(nu * s[2 * kk][2], nu * s[2 * kk][3], ah[1], al[1]);
                split2<F16>(nu * s[2 * kk + 1][0], nu * s[2 * kk + 1][1], ah[2], al[2]);
                split2<F16>(nu * s[2 * kk + 1][2], nu * s[2 * kk + 1][3], ah[3], al[3]);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ch = 2 * np + (lane >> 4);
                    ldsm_x4_t(ps + key * 128 + ((ch ^ (key & 7)) << 4), b);
                    mma16816<F16>(o[2 * np], ah, b[0], b[1]);
                    mma16816<F16>(o[2 * np + 1], ah, b[2], b[3]);
                    mma16816<F16>(o[2 * np], al, b[0], b[1]);
                    mma16816<F16>(o[2 * np + 1], al, b[2], b[3]);
                }
            }
        }
        __syncthreads();   // the stage is free for the load issued at the top of the next iteration
    }

    // ---- O / l ----
    const float inv_a = (l_a > 1e-9f) ? 1.0f / l_a : 0.0f, inv_b = (l_b > 1e-9f) ? 1.0f / l_b : 0.0f;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const int col = n * 8 + 2 * t;
        if (row_a < S) {
            if (a.out_is_f32)
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.O) + head + (size_t)row_a * kWD + col) =
                    make_float2(o[n][0] * inv_a, o[n][1] * inv_a);
            else
                *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned short*>(a.O) + head + (size_t)row_a * kWD + col) =
                    pack2<F16>(o[n][0] * inv_a, o[n][1] * inv_a);
        }
        if (row_b < S) {
            if (a.out_is_f32)
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.O) + head + (size_t)row_b * kWD + col) =
                    make_float2(o[n][2] * inv_b, o[n][3] * inv_b);
            else
                *reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned short*>(a.O) + head + (size_t)row_b * kWD + col) =
                    pack2<F16>(o[n][2] * inv_b, o[n][3] * inv_b);
        }
    }
}

}  // namespace

bool attention_window_eligible(int in_dtype, int out_dtype, int DH, const logos_attn_params* p, int S) {
    if (DH != kWD || !shunyam_active(p->window, S)) return false;
    if (in_dtype != LOGOS_BF16 && in_dtype != LOGOS_F16) return false;
    if (out_dtype != in_dtype && out_dtype != LOGOS_F32) return false;
    if (!p->causal || !(p->scale > 0.0f)) return false;
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    if (ns_any && p->ns_alpha < 1.0f) return false;
    if (ns_any && p->diffuse_mode == LOGOS_DIFFUSE_CENTRAL) return false;
    return true;
}

int attention_window(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K, const void* V,
                     void* O, int B, int H, int S, int DH, const logos_attn_params* p) {
    (void)DH;
    const int BH = B * H;
    if (BH > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention: B*H > 65535");
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "attention: tensors must be 16-byte aligned");
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    WinArgs a;
    a.Q = Q; a.K = K; a.V = V; a.O = O;
    a.S = S; a.window = p->window; a.stride = p->stride > 0 ? p->stride : 0;
    a.out_is_f32 = out_dtype == LOGOS_F32;
    a.in_is_f16 = in_dtype == LOGOS_F16;
    a.c = p->scale * 1.4426950408889634f;
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.diffuse = (ns_any && p->diffuse_mode == LOGOS_DIFFUSE_CAUSAL) ? 1 : 0;
    dim3 grid((S + kWM - 1) / kWM, BH);
    const bool f16 = a.in_is_f16, diff = a.diffuse != 0;
#define LOGOS_LAUNCH_WIN(F, D)                                                                              \
    do {                                                                                                    \
        const int rc__ = ensure_smem_limit(ctx, shunyam_window_kernel<F, D>, kWSmem);                       \
        if (rc__ != LOGOS_OK) return rc__;                                                                  \
        shunyam_window_kernel<F, D><<<grid, kWThreads, kWSmem, ctx->stream>>>(a);                           \
    } while (0)
    if (f16 && diff) LOGOS_LAUNCH_WIN(true, true);
    else if (f16) LOGOS_LAUNCH_WIN(true, false);
    else if (diff) LOGOS_LAUNCH_WIN(false, true);
    else LOGOS_LAUNCH_WIN(false, false);
#undef LOGOS_LAUNCH_WIN
    LOGOS_LAUNCH_CHECK(ctx, "shunyam_window_kernel");
    return LOGOS_OK;
}

}  // namespace logos
