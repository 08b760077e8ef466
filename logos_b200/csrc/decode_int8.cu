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
// The path is HBM-bound: one byte of K and one of V per key and channel, read once
// with 16- and 8-byte vector loads (several in flight per lane) straight into the
// registers that feed the arithmetic; nothing is staged, nothing is re-read.
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
constexpr size_t kCounterBytes = kWorkspaceCounterBytes;  // head of the workspace: arrival counters
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeArgs {
    const __half* q;
    const __half* q_prev;
    const int8_t* k_cache;
    const int8_t* v_cache;
    const float* k_scale;
    const float* v_scale;
    const int32_t* len;
    float* out;            // without peers: [BH][64] in out_dtype
    int out_dtype;
    float* partials;       // [BH][splits][paths][kPartial]
    unsigned int* counters;  // [BH], zero between launches
    int H, S_max, chunk;
    float scale, eta, nu, alpha;
    int diffuse_mode, window, stride;
    PeerEpilogue peer;     // world == 0: rows go to `out`
    // Sparse kernel only: the new token's K and V rows (FP16 [BH][64]), quantised into row len - 1 of the caches by
    // the kernel itself before it reads them (the work of append_kernel, csrc/nikhilam.cu); null: nothing to append.
    const __half* k_new;
    const __half* v_new;
    int8_t* k_cache_w;
    int8_t* v_cache_w;
};

// The finished row of pair bh (thread d < 64 holds channel d); called by every thread of the CTA.
// Without peers the row goes to `out`.  With peers every value goes, as one 8-byte word {bits, step + 1},
// into the current row-area slot of every rank at this rank's head offset -- plain stores over NVLink,
// nothing to wait for: the word carries its own arrival mark.
__device__ __forceinline__ void emit_row(const DecodeArgs& a, int bh, int tid, float value) {
    if (tid >= kDH) return;
    if (a.peer.world == 0) {
        const int64_t at = (int64_t)bh * kDH + tid;
        if (a.out_dtype == LOGOS_F32) a.out[at] = value;
        else if (a.out_dtype == LOGOS_BF16) reinterpret_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(value);
        else reinterpret_cast<__half*>(a.out)[at] = __float2half_rn(value);
        return;
    }
    const unsigned step = *a.peer.step;
    const int b = bh / a.H, h = bh - b * a.H;
    const size_t idx = (size_t)(step & 1u) * a.peer.slot_words +
                       ((size_t)b * a.peer.H_total + a.peer.head0 + h) * kDH + tid;
    const unsigned bits = __float_as_uint(value), mark = step + 1u;
    for (int r = 0; r < a.peer.world; ++r)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(a.peer.rows[r] + idx), "r"(bits), "r"(mark) : "memory");
}

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
//
// Both contractions run as exact integer dot products on the tensor cores
// (mma.sync m16n8k32, int8 x int8 -> int32), because a first SIMT version that
// converted every byte to fp32 was bound by instruction issue at 41 % of DRAM
// bandwidth (about 100 instructions per 16-byte vector).  The float operand of
// each contraction is cut into three int8 "digits" of a 24-bit fixed-point number,
// which the 8-wide N (or 16-high M) dimension of the MMA carries for free:
//   scores : A = 16 keys x 32 channels of K bytes, B = query digits (columns 0-2:
//            advected query, 3-5: plain query for the blend), C = digit dot products;
//   output : A = weight digits (rows 0-2 / 3-5) x 32 keys, B = V bytes transposed in
//            registers to key-major (8 byte-permutes per 4x4 block), C = digit sums.
// int32 accumulation is exact; the digits are recombined in fp32 once per CTA.
// The fixed-point grids (2^-22 of the largest |q| channel, 2^-23 of the largest
// weight) are finer than fp32 rounding of the same sums.

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ld_stream8(const int8_t* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// rows r0..r3 hold 4 consecutive bytes each; out[j] = byte j of (r0, r1, r2, r3)
__device__ __forceinline__ void transpose4x4(uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3,
                                             uint32_t* out) {
    uint32_t t0 = __byte_perm(r0, r1, 0x5140), t1 = __byte_perm(r2, r3, 0x5140);
    uint32_t t2 = __byte_perm(r0, r1, 0x7362), t3 = __byte_perm(r2, r3, 0x7362);
    out[0] = __byte_perm(t0, t1, 0x5410);
    out[1] = __byte_perm(t0, t1, 0x7632);
    out[2] = __byte_perm(t2, t3, 0x5410);
    out[3] = __byte_perm(t2, t3, 0x7632);
}

// byte `idx` of four words packed into one word (word e -> byte e)
__device__ __forceinline__ uint32_t pack_byte(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3,
                                              int idx) {
    uint32_t sel = (uint32_t)idx | ((uint32_t)(4 + idx) << 4);
    uint32_t lo = __byte_perm(w0, w1, sel), hi = __byte_perm(w2, w3, sel);
    return __byte_perm(lo, hi, 0x5410);
}

// Signed base-256 digits of a fixed-point integer: v = d0*65536 + d1*256 + d2, d1,d2 in [-128,127].
__device__ __forceinline__ int signed_digit(int v, int which) {
    int d2 = ((v + 128) & 255) - 128;
    int r = (v - d2) >> 8;
    int d1 = ((r + 128) & 255) - 128;
    int d0 = (r - d1) >> 8;
    return which == 0 ? d0 : (which == 1 ? d1 : d2);
}

constexpr int kDenseWarps = 2;                  // warps per CTA, each with its own key range (512 keys at most)
constexpr int kDenseThreads = kDenseWarps * 32;
constexpr int kSubMax = kMaxChunk / kDenseWarps;  // keys per warp (512)
constexpr int kDigitPitch = kSubMax / 4 + 4;    // words per digit row (+4: no bank aliasing)
constexpr float kQGrid = 4194303.0f;            // 2^22 - 1 levels for the largest |q| channel
constexpr float kWGrid = 8388608.0f;            // 2^23 levels per unit weight

// Every warp streams its own contiguous range of keys (two passes: K then V) and
// only meets the other warps of the CTA once, to merge (max, sum, output).  Inside
// the passes there is no block-wide barrier, and the next 32-key tile is always in
// flight while the current one is consumed.
// NB = tiles of a pass held in registers at once (the one being used and NB - 1 on their way).  Two keep ten
// CTAs on an SM: right when the launch is several waves deep, where the memory system is already full.  Four
// (eight CTAs per SM) are for launches of a single wave, where a warp's chain of load latencies is the whole
// run time and more loads in flight per warp shorten it.
template <bool BLEND, int NB>
__global__ void __launch_bounds__(kDenseThreads, NB == 2 ? 10 : 8)
decode_dense_kernel(const DecodeArgs a) {
    constexpr int PATHS = BLEND ? 2 : 1;
    constexpr int ND = 3 * PATHS;                                   // digit rows / columns in use
    __shared__ float sc[kDenseWarps][PATHS][kSubMax + 2];           // [1 + r], zero halo at both ends
    __shared__ uint32_t wdig[kDenseWarps][ND][kDigitPitch];         // weight digits, 4 keys per word
    __shared__ float part[kDenseWarps][PATHS][kPartial];            // per-warp (max, sum, out[64])
    __shared__ unsigned int is_last;

    const int bh = blockIdx.y, split = blockIdx.x, n_splits = gridDim.x;
    const int b = bh / a.H;
    int len = a.len[b];
    len = len < 0 ? 0 : (len > a.S_max ? a.S_max : len);
    const int pos = len - 1;
    const int c0 = split * a.chunk;
    const int c1 = min(len, c0 + a.chunk);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;   // MMA fragment coordinates: group, thread-in-group
    const int sub = a.chunk / kDenseWarps;   // keys per warp, a multiple of 32
    const int w0 = c0 + warp * sub;
    const int w1 = min(c1, w0 + sub);
    const int nw = w1 - w0;                  // keys of this warp (<= 0: nothing to do but report)

    const int8_t* kbase = a.k_cache + (int64_t)bh * a.S_max * kDH + (int64_t)w0 * kDH;
    const int8_t* vbase = a.v_cache + (int64_t)bh * a.S_max * kDH + (int64_t)w0 * kDH;
    float* p_ns = sc[warp][0];
    float* p_std = sc[warp][PATHS - 1];

    // Launched to overlap the append kernel before it: everything but the newest cache row is older than that
    // kernel and may be read at once; a CTA whose range holds row pos (or ends just before it: the halo) waits
    // for the append to finish first.  The collect kernel after this one may start as soon as every CTA is here.
    grid_release_dependents();
    if (c1 >= pos) grid_wait_for_earlier();

    if (nw > 0) {
        // first K tile goes out before any arithmetic
        uint4 kt[NB][4];
        auto load_k = [&](uint4 (&buf)[4], int r0) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int r = r0 + g + 8 * u;
                buf[u] = (r < nw) ? ld_stream(kbase + (int64_t)r * kDH + 16 * t) : make_uint4(0, 0, 0, 0);
            }
        };
#pragma unroll
        for (int u = 0; u < NB - 1; ++u) load_k(kt[u], 32 * u);

        // ---- query digits: lane (g,t) holds digit g of channels 16t..16t+15 ----
        uint32_t qb[4];
        float qstep_ns, qstep_std = 0.0f;
        {
            float qn[16], qs[BLEND ? 16 : 1];
            load_query<BLEND>(a, bh, pos, t, qn, qs);
            float mx = 0.0f, mx2 = 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                mx = fmaxf(mx, fabsf(qn[k]));
                if (BLEND) mx2 = fmaxf(mx2, fabsf(qs[k]));
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            if (BLEND) {
                mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 1));
                mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, 2));
            }
            const float inv = mx > 0.0f ? kQGrid / mx : 0.0f;
            const float inv2 = (BLEND && mx2 > 0.0f) ? kQGrid / mx2 : 0.0f;
            qstep_ns = mx / kQGrid;
            if (BLEND) qstep_std = mx2 / kQGrid;
            const bool use_std = BLEND && g >= 3;
            const int which = g % 3;
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float x = use_std ? qs[BLEND ? 4 * wd + e : 0] * inv2 : qn[4 * wd + e] * inv;
                    int d = signed_digit(__float2int_rn(x), which);
                    word |= ((uint32_t)d & 0xffu) << (8 * e);
                }
                qb[wd] = (g < ND) ? word : 0u;
            }
        }
        // per-lane recombination weights of the score digits: C column 2t and 2t+1
        const float ns_e = (t == 0) ? 65536.0f : (t == 1 ? 1.0f : 0.0f);
        const float ns_o = (t == 0) ? 256.0f : 0.0f;
        const float st_e = (t == 2) ? 256.0f : 0.0f;
        const float st_o = (t == 1) ? 65536.0f : (t == 2 ? 1.0f : 0.0f);

        // ---- scores: 32 keys per tile = two 16-key MMA pairs ----
        auto score_tile = [&](const uint4 (&buf)[4], int r0) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint4& lo = buf[2 * hf];
                const uint4& hi = buf[2 * hf + 1];
                int ra = r0 + 16 * hf + g, rb = ra + 8;
                int c[4] = {0, 0, 0, 0};
                mma_s8s8(c, lo.x, hi.x, lo.y, hi.y, qb[0], qb[1]);
                mma_s8s8(c, lo.z, hi.z, lo.w, hi.w, qb[2], qb[3]);
                float sa = ns_e * (float)c[0] + ns_o * (float)c[1];
                float sb = ns_e * (float)c[2] + ns_o * (float)c[3];
                sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                sb += __shfl_xor_sync(0xffffffffu, sb, 1);
                sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                sb += __shfl_xor_sync(0xffffffffu, sb, 2);
                float ta = 0.0f, tb = 0.0f;
                if (BLEND) {
                    ta = st_e * (float)c[0] + st_o * (float)c[1];
                    tb = st_e * (float)c[2] + st_o * (float)c[3];
                    ta += __shfl_xor_sync(0xffffffffu, ta, 1);
                    tb += __shfl_xor_sync(0xffffffffu, tb, 1);
                    ta += __shfl_xor_sync(0xffffffffu, ta, 2);
                    tb += __shfl_xor_sync(0xffffffffu, tb, 2);
                }
                if (t == 0) {
                    if (ra < nw) p_ns[1 + ra] = sa * qstep_ns;
                    if (rb < nw) p_ns[1 + rb] = sb * qstep_ns;
                }
                if (BLEND && t == 1) {
                    if (ra < nw) p_std[1 + ra] = ta * qstep_std;
                    if (rb < nw) p_std[1 + rb] = tb * qstep_std;
                }
            }
        };
        for (int r0 = 0; r0 < nw; r0 += 32 * NB) {
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                load_k(kt[(u + NB - 1) % NB], r0 + 32 * (u + NB - 1));
                if (r0 + 32 * u < nw) score_tile(kt[u], r0 + 32 * u);   // warp-uniform
            }
        }

        // first V tile goes out before the softmax
        uint2 vt[NB][8];
        auto load_v = [&](uint2 (&buf)[8], int r0) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                int r = r0 + (u < 4 ? 4 * t + u : 16 + 4 * t + (u - 4));
                buf[u] = (r < nw) ? ld_stream8(vbase + (int64_t)r * kDH + 8 * g) : make_uint2(0, 0);
            }
        };
#pragma unroll
        for (int u = 0; u < NB - 1; ++u) load_v(vt[u], 32 * u);
        if (lane == 0) { p_ns[0] = 0.0f; p_ns[1 + nw] = 0.0f; }
        __syncwarp();

        // ---- softmax over this warp's keys ----
        float mx = -INFINITY, mx2 = -INFINITY;
        for (int i = lane; i < nw; i += 32) {
            mx = fmaxf(mx, p_ns[1 + i]);
            if (BLEND) mx2 = fmaxf(mx2, p_std[1 + i]);
        }
        const float m_ns = warp_max(mx);
        const float m_std = BLEND ? warp_max(mx2) : 0.0f;
        float sum = 0.0f, sum2 = 0.0f;
        for (int i = lane; i < nw; i += 32) {
            float e = exp2f(p_ns[1 + i] - m_ns);
            p_ns[1 + i] = e;
            sum += e;
            if (BLEND) {
                float e2 = exp2f(p_std[1 + i] - m_std);
                p_std[1 + i] = e2;
                sum2 += e2;
            }
        }
        const float l_ns = warp_sum(sum);
        const float l_std = BLEND ? warp_sum(sum2) : 0.0f;
        __syncwarp();

        // ---- value weights (diffusion folded in) as three unsigned digits ----
        float cC = 1.0f, cL = 0.0f, cR = 0.0f, b0 = 0.0f, bN = 0.0f;
        if (a.diffuse_mode == LOGOS_DIFFUSE_CAUSAL) {
            cC = 1.0f - a.nu; cR = a.nu; b0 = a.nu;
        } else if (a.diffuse_mode == LOGOS_DIFFUSE_CENTRAL) {
            cC = 1.0f - a.nu; cR = cL = 0.5f * a.nu; b0 = bN = 0.5f * a.nu;
        }
        const int groups = ((nw + 31) >> 5) << 3;  // 4-key words, padded to whole 32-key tiles
        for (int grp = lane; grp < groups; grp += 32) {
            uint32_t W[4], W2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int r = 4 * grp + e;
                float wgt = 0.0f, wgt2 = 0.0f;
                if (r < nw) {
                    float pc = p_ns[1 + r];
                    wgt = cC * pc + cR * p_ns[2 + r] + cL * p_ns[r];
                    int j = w0 + r;
                    if (j == 0) wgt += b0 * pc;
                    if (j == len - 1) wgt += bN * pc;
                    if (BLEND) wgt2 = p_std[1 + r];
                }
                W[e] = min(__float2uint_rn(wgt * kWGrid), 0xFFFFFFu);
                W2[e] = BLEND ? min(__float2uint_rn(wgt2 * kWGrid), 0xFFFFFFu) : 0u;
            }
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                wdig[warp][d][grp] = pack_byte(W[0], W[1], W[2], W[3], 2 - d);
                if (BLEND) wdig[warp][BLEND ? 3 + d : 0][grp] = pack_byte(W2[0], W2[1], W2[2], W2[3], 2 - d);
            }
        }
        __syncwarp();

        // ---- weights x V: 32 keys per tile, 8 MMAs (one per 8 channels) ----
        int acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0; }
        const uint32_t* my_dig = wdig[warp][g < ND ? g : 0];
        auto value_tile = [&](const uint2 (&buf)[8], int r0) {
            int grp = r0 >> 2;
            uint32_t a0 = (g < ND) ? my_dig[grp + t] : 0u;
            uint32_t a2 = (g < ND) ? my_dig[grp + 4 + t] : 0u;
            uint32_t blo[8], bhi[8];
            transpose4x4(buf[0].x, buf[1].x, buf[2].x, buf[3].x, blo);
            transpose4x4(buf[0].y, buf[1].y, buf[2].y, buf[3].y, blo + 4);
            transpose4x4(buf[4].x, buf[5].x, buf[6].x, buf[7].x, bhi);
            transpose4x4(buf[4].y, buf[5].y, buf[6].y, buf[7].y, bhi + 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) mma_u8s8(acc[j], a0, 0u, a2, 0u, blo[j], bhi[j]);
        };
        for (int r0 = 0; r0 < nw; r0 += 32 * NB) {
#pragma unroll
            for (int u = 0; u < NB; ++u) {
                load_v(vt[(u + NB - 1) % NB], r0 + 32 * (u + NB - 1));
                if (r0 + 32 * u < nw) value_tile(vt[u], r0 + 32 * u);   // warp-uniform
            }
        }
        // halo rows in fp32 (lanes 0-3, 16 channels each): the row before the range takes
        // cR * p(first key), the row after it takes cL * p(last key)
        float hal[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) hal[k] = 0.0f;
        if (lane < 4) {
            if (w0 > 0 && cR != 0.0f) axpy16(ld_stream(vbase - kDH + 16 * lane), cR * p_ns[1], hal);
            if (w1 < len && cL != 0.0f) axpy16(ld_stream(vbase + (int64_t)nw * kDH + 16 * lane), cL * p_ns[nw], hal);
        }
        // digit rows -> fp32: row g carries 65536 / 256 / 1 of path (g / 3)
        const float ns_w = (g == 0) ? 65536.0f : (g == 1 ? 256.0f : (g == 2 ? 1.0f : 0.0f));
        const float st_w = (g == 3) ? 65536.0f : (g == 4 ? 256.0f : (g == 5 ? 1.0f : 0.0f));
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float f = (float)acc[j][h];
                float vn = f * ns_w, vst = BLEND ? f * st_w : 0.0f;
#pragma unroll
                for (int off = 4; off < 32; off <<= 1) {
                    vn += __shfl_xor_sync(0xffffffffu, vn, off);
                    if (BLEND) vst += __shfl_xor_sync(0xffffffffu, vst, off);
                }
                if (g == 0) {   // C column 2t+h of tile j is channel 8*(2t+h) + j
                    part[warp][0][2 + 16 * t + 8 * h + j] = vn * (1.0f / kWGrid) + hal[8 * h + j];
                    if (BLEND) part[warp][PATHS - 1][2 + 16 * t + 8 * h + j] = vst * (1.0f / kWGrid);
                }
            }
        if (lane == 0) {
            part[warp][0][0] = m_ns; part[warp][0][1] = l_ns;
            if (BLEND) { part[warp][PATHS - 1][0] = m_std; part[warp][PATHS - 1][1] = l_std; }
        }
    } else {
        for (int i = lane; i < PATHS * kPartial; i += 32) {
            int pth = i / kPartial, k = i - pth * kPartial;
            part[warp][pth][k] = (k == 0) ? -INFINITY : 0.0f;
        }
    }
    __syncthreads();

    // ---- merge the warps of this CTA: thread d owns channel d ----
    float m_c[PATHS], l_c[PATHS], o_c[PATHS];
    if (tid < kDH) {
#pragma unroll
        for (int pth = 0; pth < PATHS; ++pth) {
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kDenseWarps; ++w) M = fmaxf(M, part[w][pth][0]);
            float num = 0.0f, den = 0.0f;
#pragma unroll
            for (int w = 0; w < kDenseWarps; ++w) {
                float mw = part[w][pth][0];
                float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
                den = fmaf(f, part[w][pth][1], den);
                num = fmaf(f, part[w][pth][2 + tid], num);
            }
            m_c[pth] = M; l_c[pth] = den; o_c[pth] = num;
        }
    }

    const float vs = a.v_scale[bh];

    if (n_splits == 1) {
        float r = 0.0f;
        if (tid < kDH) {
            r = (l_c[0] > 0.0f) ? o_c[0] / l_c[0] : 0.0f;
            if (BLEND) {
                float r_std = (l_c[PATHS - 1] > 0.0f) ? o_c[PATHS - 1] / l_c[PATHS - 1] : 0.0f;
                r = (1.0f - a.alpha) * r_std + a.alpha * r;
            }
        }
        emit_row(a, bh, tid, r * vs);
        return;
    }

    // ---- publish this split's partial, merge if last ----
    float* mine = a.partials + ((int64_t)bh * n_splits + split) * PATHS * kPartial;
    if (tid < kDH) {
#pragma unroll
        for (int pth = 0; pth < PATHS; ++pth) {
            mine[pth * kPartial + 2 + tid] = o_c[pth];
            if (tid == 0) { mine[pth * kPartial] = m_c[pth]; mine[pth * kPartial + 1] = l_c[pth]; }
        }
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
    float r_out = 0.0f;
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
        if (BLEND) r = (1.0f - a.alpha) * r_path[PATHS - 1] + a.alpha * r_path[0];
        r_out = r * vs;
    }
    emit_row(a, bh, tid, r_out);
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
    // the kernel after this one may start at once, if it was launched to overlap (the W_O projection of a decode
    // step then fetches its weights while the rows are still being computed; it waits before it reads them)
    grid_release_dependents();
    grid_wait_for_earlier();           // after an append kernel it is launched to overlap that (only the launch does)
    __shared__ float red[kWarps];
    __shared__ float red_acc[kWarps][kDH];

    const int bh = blockIdx.x;
    const int b = bh / a.H;
    int len = a.len[b];
    len = len < 0 ? 0 : (len > a.S_max ? a.S_max : len);
    const int pos = len - 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row_in_warp = lane >> 2, part = lane & 3;
    // The new token's rows: quantised with the tensors' stored scales exactly as append_kernel does (same division,
    // clamp and rounding; a row index outside the cache is rejected, not written), kept in shared memory for this
    // CTA's own reads -- the streaming loads below may not see a store of the same kernel.
    __shared__ __align__(16) int8_t new_rows[2][kDH];
    int pos_new = -1;
    if (a.k_new) {
        const int row = a.len[b] - 1;
        if (row >= 0 && row < a.S_max) {
            pos_new = row;
            if (tid < 2 * kDH) {
                const int which = tid / kDH, d = tid - which * kDH;
                const float den = __fadd_rn((which ? a.v_scale : a.k_scale)[bh], 1e-8f);
                float x = __half2float((which ? a.v_new : a.k_new)[(int64_t)bh * kDH + d]);
                x = fminf(fmaxf(__fdiv_rn(x, den), -127.0f), 127.0f);
                const int8_t v8 = (int8_t)__float2int_rn(x);
                new_rows[which][d] = v8;
                (which ? a.v_cache_w : a.k_cache_w)[((int64_t)bh * a.S_max + row) * kDH + d] = v8;
            }
        }
        __syncthreads();
    }
    if (len == 0) {
        emit_row(a, bh, tid, 0.0f);
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
    // this lane's 16 bytes of cache row j: the row appended by this kernel comes from shared memory
    auto k_row = [&](int j) {
        return j == pos_new ? *reinterpret_cast<const uint4*>(&new_rows[0][part * 16]) : ld_stream(kbase + (int64_t)j * kDH);
    };
    auto v_row = [&](int j) {
        return j == pos_new ? *reinterpret_cast<const uint4*>(&new_rows[1][part * 16]) : ld_stream(vbase + (int64_t)j * kDH);
    };
    float qn[16], qs[BLEND ? 16 : 1];
    load_query<BLEND>(a, bh, pos, part, qn, qs);

    for (int t0 = warp * kRowsPerWarp; t0 < T; t0 += kRowsPerIter * kUnroll) {
        uint4 w[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            int t = t0 + u * kRowsPerIter + row_in_warp;
            w[u] = (t < T) ? k_row(key_of(t)) : make_uint4(0, 0, 0, 0);
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
        uint4 wc = v_row(j);
        float p = p_ns[t];
        if (mode == LOGOS_DIFFUSE_NONE) {
            axpy16(wc, p, acc);
        } else {
            // Vs_j = (1-nu) V_j + nu V_{j-1}            (cuda/ModelGPU.cu:463-471), or
            // Vs_j = (1-nu) V_j + nu/2 (V_{j-1}+V_{j+1}) (include/Attention.hpp:173-181),
            // neighbours clamped to [0, len-1]
            int jl = j > 0 ? j - 1 : 0;
            uint4 wl = v_row(jl);
            if (mode == LOGOS_DIFFUSE_CAUSAL) {
                axpy16(wc, p * (1.0f - a.nu), acc);
                axpy16(wl, p * a.nu, acc);
            } else {
                int jr = j < len - 1 ? j + 1 : len - 1;
                uint4 wr = v_row(jr);
                axpy16(wc, p * (1.0f - a.nu), acc);
                axpy16(wl, p * 0.5f * a.nu, acc);
                axpy16(wr, p * 0.5f * a.nu, acc);
            }
        }
        if (BLEND) axpy16(wc, p_std[t], acc2);
    }
    float o_ns = block_reduce_acc(acc, red_acc);
    float o_std = BLEND ? block_reduce_acc(acc2, red_acc) : 0.0f;
    float r = 0.0f;
    if (tid < kDH) {
        r = (l_ns > 0.0f) ? o_ns / l_ns : 0.0f;
        if (BLEND) {
            float r_std = (l_std > 0.0f) ? o_std / l_std : 0.0f;
            r = (1.0f - a.alpha) * r_std + a.alpha * r;
        }
        r *= a.v_scale[bh];
    }
    emit_row(a, bh, tid, r);
}

// Keys per split of the dense kernel, the one rule of both entry points.  A warp's fixed cost -- query digits,
// softmax, partial record, merge -- outweighs finer splitting: measured at 8192 keys, the largest chunk
// (1024) is the fastest whenever the launch is more than two waves of CTAs (ten 64-thread CTAs fit an SM) or
// less than one (187 us at 1024 pairs, 99 at 512, 33 at 128; 256-key chunks: 245 / 131 / 42).  Between one
// and two waves the second wave is mostly empty, so the chunk shrinks (in steps of 64 keys) until the CTAs
// just fill two: 58 us instead of 62 at 256 pairs.  For very few pairs the chunk shrinks until every SM has
// about four CTAs.  `forced` != 0 (LOGOS_OPT_DECODE_CHUNK) overrides the rule.
int pick_chunk(int sm_count, int forced, int64_t BH, int S_max) {
    if (forced) return forced;
    int chunk = kMaxChunk;
    while (chunk > 128 && BH * ((S_max + chunk - 1) / chunk) < (int64_t)sm_count * 4) chunk >>= 1;
    const int64_t slots = (int64_t)sm_count * 10;
    const int64_t ctas = BH * ((S_max + chunk - 1) / chunk);
    if (chunk == kMaxChunk && ctas > slots && ctas < 2 * slots) {
        const int64_t per_pair = (2 * slots) / BH;                       // splits per pair that two waves hold
        int c = (int)(((S_max + per_pair - 1) / per_pair + 63) / 64 * 64);
        while (c < kMaxChunk && BH * ((S_max + c - 1) / c) > 2 * slots) c += 64;
        if (c >= 128 && c < kMaxChunk) chunk = c;
    }
    return chunk;
}

// The diffusion-folded weights travel as unsigned fixed-point digits, so every stencil coefficient
// must be non-negative: nu in [0, 1].  (The reference's ns_diffuse_kernel takes any float.)
bool dense_nu_ok(const logos_attn_params* p) {
    const bool diffusing = p->ns_alpha > 0.0f && p->diffuse_mode != LOGOS_DIFFUSE_NONE;
    return !diffusing || (p->ns_nu >= 0.0f && p->ns_nu <= 1.0f);
}

}  // namespace

size_t decode_workspace_bytes(int B, int H, int S_max, int DH) {
    (void)DH;
    if (B <= 0 || H <= 0 || S_max <= 0) return 0;
    size_t splits = ((size_t)S_max + 127) / 128;  // worst case: smallest chunk
    return kCounterBytes + (size_t)B * H * splits * 2 * kPartial * sizeof(float);
}

bool decode_appends_itself(const logos_attn_params* p, int DH) { return p->window > 0 && DH == kDH; }

int decode_int8(logos_ctx* ctx, const void* q, const void* q_prev, const int8_t* k_cache,
                const int8_t* v_cache, const float* k_scale, const float* v_scale,
                const int32_t* len, int B, int H, int S_max, int DH,
                const logos_attn_params* p, float* out, const PeerEpilogue* peer, bool follows_append, int out_dtype,
                const void* append_k, const void* append_v) {
    if ((append_k || append_v) && (!append_k || !append_v || !p || !decode_appends_itself(p, DH)))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: rows to append need both tensors and the window kernel");
    if (!dtype_ok(out_dtype) || (out_dtype != LOGOS_F32 && (peer || DH != kDH)))
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: 16-bit rows are for DH = 64 without peers");
    if (!q || !k_cache || !v_cache || !k_scale || !v_scale || !len || (!out && !peer) || !p || B <= 0 ||
        H <= 0 || S_max <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: bad pointer or extent");
    if (!aligned16(k_cache) || !aligned16(v_cache))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "decode_int8: caches must be 16-byte aligned");
    if (p->diffuse_mode < 0 || p->diffuse_mode > 2)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: bad diffuse_mode");
    if (p->ns_eta != 0.0f && p->ns_alpha > 0.0f && !q_prev)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: q_prev is required when ns_eta != 0");
    if (DH != kDH)       // the head dimensions the model does not use: the general kernel
        return decode_generic(ctx, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, p, out);
    const int BH = B * H;
    if ((size_t)BH * sizeof(unsigned int) > kCounterBytes)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: more than 16384 (b,h) pairs");

    DecodeArgs a;
    a.q = (const __half*)q;
    a.q_prev = (const __half*)q_prev;
    a.k_cache = k_cache; a.v_cache = v_cache;
    a.k_scale = k_scale; a.v_scale = v_scale;
    a.len = len; a.out = out; a.out_dtype = out_dtype;
    a.k_new = static_cast<const __half*>(append_k); a.v_new = static_cast<const __half*>(append_v);
    a.k_cache_w = const_cast<int8_t*>(k_cache); a.v_cache_w = const_cast<int8_t*>(v_cache);
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
    if (peer) a.peer = *peer;
    else a.peer.world = 0;

    if (p->window > 0) {
        int t_max = p->window + 1 + (p->stride > 0 ? (S_max + p->stride - 1) / p->stride : 0);
        if (t_max > S_max) t_max = S_max;
        if (t_max < p->window + 1) t_max = p->window + 1;
        size_t smem = sizeof(float) * (size_t)t_max * (blend ? 2 : 1);
        if (smem > 160 * 1024)
            return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: %d visible keys exceed the sparse kernel", t_max);
        a.partials = nullptr; a.counters = nullptr; a.chunk = 0;
        // more than the default 48 KB of dynamic shared memory needs the attribute (not a hot call: a
        // window with that many visible keys is not a decode shape of the model)
        if (smem > 48 * 1024) {
            if (blend) LOGOS_CUDA_TRY(ctx, cudaFuncSetAttribute(decode_sparse_kernel<true>,
                                                                cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            else LOGOS_CUDA_TRY(ctx, cudaFuncSetAttribute(decode_sparse_kernel<false>,
                                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        }
        auto* sparse = blend ? decode_sparse_kernel<true> : decode_sparse_kernel<false>;
        // Measured and dropped: launching it to overlap the projection before it in a decode step (its 512 waiting
        // CTAs then sit on the SMs under that projection: 0.54 instead of 0.52 ms per 16-layer step).
        if (follows_append) {      // the kernel before this one on the stream is the engine's append of row len - 1
            LOGOS_CUDA_TRY(ctx, launch_overlapped(sparse, dim3(BH), dim3(kThreads), smem, ctx->stream, a, t_max));
        } else {
            sparse<<<BH, kThreads, smem, ctx->stream>>>(a, t_max);
        }
        LOGOS_LAUNCH_CHECK(ctx, "decode_sparse_kernel");
        return LOGOS_OK;
    }

    if (!dense_nu_ok(p))
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_int8: dense contexts need ns_nu in [0, 1], got %g", (double)p->ns_nu);
    a.chunk = pick_chunk(ctx->sm_count, ctx->decode_chunk, BH, S_max);
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
    // a single wave of CTAs (eight per SM): the deep-prefetch form
    const int depth = ctx->decode_depth ? ctx->decode_depth
                                        : ((int64_t)n_splits * BH <= (int64_t)ctx->sm_count * 8 ? 4 : 2);
    void (*kernel)(const DecodeArgs) =
        depth == 4 ? (blend ? decode_dense_kernel<true, 4> : decode_dense_kernel<false, 4>)
                   : (blend ? decode_dense_kernel<true, 2> : decode_dense_kernel<false, 2>);
    if (follows_append) {      // the kernel before this one on the stream is the engine's append of row len - 1
        LOGOS_CUDA_TRY(ctx, launch_overlapped(kernel, grid, dim3(kDenseThreads), 0, ctx->stream, a));
        return LOGOS_OK;
    }
    kernel<<<grid, kDenseThreads, 0, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "decode_dense_kernel");
    return LOGOS_OK;
}

}  // namespace logos

// ---------------------------------------------------------------------------
// Dense decode for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they decode:
// code running inside a memory pool that owns the whole device, a serving loop that
// forbids allocation after start-up, or an embedding that never creates a logos_ctx
// (context creation allocates).  For them the split-K scratch of the dense kernel
// lives in the fixed device array below, which every GPU that loads this library
// holds until the process exits.  The array keeps whatever the previous call left in
// it; only the arrival counters have to start at zero and they are cleared on the
// caller's stream by every call.  Two calls that overlap on one GPU (different
// streams, or different host threads) share the array and race.
namespace logos {
namespace {

constexpr int kNoAllocMaxPairs = 4096;        // (sequence, head) pairs per call
constexpr int kNoAllocMaxPartials = 16384;    // pairs x key splits x paths per call
constexpr size_t kNoAllocCounterBytes = kNoAllocMaxPairs * sizeof(unsigned int);
constexpr size_t kNoAllocBytes = kNoAllocCounterBytes + (size_t)kNoAllocMaxPartials * kPartial * sizeof(float);
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device with that device current.
struct NoAllocDevice {
    void* scratch = nullptr;
    int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];

int noalloc_setup(int* dev_out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
        cudaGetLastError();
        return LOGOS_ERR_NO_DEVICE;
    }
    *dev_out = dev;
    if (g_noalloc_dev[dev].scratch) return LOGOS_OK;
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
        cudaGetLastError();
        return LOGOS_ERR_CUDA;
    }
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        cudaGetLastError();
        return LOGOS_ERR_CUDA;
    }
    if (major != 10) return LOGOS_ERR_NO_DEVICE;
    g_noalloc_dev[dev].sm_count = sms;
    g_noalloc_dev[dev].scratch = p;   // written last: a non-null pointer means set-up is complete
    return LOGOS_OK;
}

}  // namespace
}  // namespace logos

extern "C" int logos_decode_int8_noalloc(void* cuda_stream, const void* q, const void* q_prev,
                                         const int8_t* k_cache, const int8_t* v_cache,
                                         const float* k_scale, const float* v_scale,
                                         const int32_t* len, int B, int H, int S_max, int DH,
                                         const logos_attn_params* p, float* out) {
    using namespace logos;
    if (!q || !k_cache || !v_cache || !k_scale || !v_scale || !len || !out || !p || B <= 0 ||
        H <= 0 || S_max <= 0)
        return LOGOS_ERR_INVALID_ARG;
    if (DH != kDH || p->window > 0) return LOGOS_ERR_UNSUPPORTED;   // dense contexts only
    if (!aligned16(k_cache) || !aligned16(v_cache)) return LOGOS_ERR_ALIGNMENT;
    if (p->diffuse_mode < 0 || p->diffuse_mode > 2 || p->ns_alpha < 0.0f || p->ns_alpha > 1.0f)
        return LOGOS_ERR_INVALID_ARG;
    if (p->ns_eta != 0.0f && p->ns_alpha > 0.0f && !q_prev) return LOGOS_ERR_INVALID_ARG;
    int dev = 0;
    int rc = noalloc_setup(&dev);
    if (rc != LOGOS_OK) return rc;
    const NoAllocDevice& nd = g_noalloc_dev[dev];

    const bool ns_any = p->ns_alpha > 0.0f &&
                        (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    const bool blend = ns_any && p->ns_alpha < 1.0f;
    const int64_t BH = (int64_t)B * H;
    if (BH > kNoAllocMaxPairs) return LOGOS_ERR_SCRATCH_LIMIT;
    if (!dense_nu_ok(p)) return LOGOS_ERR_UNSUPPORTED;
    const int chunk = pick_chunk(nd.sm_count, 0, BH, S_max);   // the rule of the context entry point
    const int n_splits = (S_max + chunk - 1) / chunk;
    if (BH * n_splits * (blend ? 2 : 1) > kNoAllocMaxPartials) return LOGOS_ERR_SCRATCH_LIMIT;

    DecodeArgs a;
    a.q = (const __half*)q; a.q_prev = (const __half*)q_prev;
    a.k_cache = k_cache; a.v_cache = v_cache;
    a.k_scale = k_scale; a.v_scale = v_scale;
    a.len = len; a.out = out; a.out_dtype = LOGOS_F32;
    a.k_new = nullptr; a.v_new = nullptr; a.k_cache_w = nullptr; a.v_cache_w = nullptr;
    a.H = H; a.S_max = S_max; a.chunk = chunk;
    a.scale = p->scale; a.window = 0; a.stride = 0;
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.diffuse_mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    a.alpha = p->ns_alpha;
    a.peer.world = 0;
    a.counters = (unsigned int*)nd.scratch;
    a.partials = (float*)((char*)nd.scratch + kNoAllocCounterBytes);
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (n_splits > 1 &&
        cudaMemsetAsync(a.counters, 0, (size_t)BH * sizeof(unsigned int), st) != cudaSuccess) {
        cudaGetLastError();
        return LOGOS_ERR_CUDA;
    }
    dim3 grid(n_splits, (unsigned)BH);
    if (blend) decode_dense_kernel<true, 2><<<grid, kDenseThreads, 0, st>>>(a);
    else       decode_dense_kernel<false, 2><<<grid, kDenseThreads, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? LOGOS_OK : LOGOS_ERR_CUDA;
}
