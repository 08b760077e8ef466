// attn_bwd_tc.cu -- attention backward on the tensor cores (tcgen05), 16-bit operands, fp32 accumulation.
//
// The same mathematics as attn_bwd.cu (the chain of cuda/train_gpu.cu:657-748 without any seq x seq buffer, the
// forward's own mask), with every product on tcgen05.mma and the operands staged by TMA:
//
//   bwd_tc_rows_kernel   one CTA per 128 query rows, one pass over the visible key tiles with a running maximum:
//       S = Qx K^T, dP = dO Vx^T                         (two M128 N128 products into tensor memory)
//       e = 2^(c S - m), l += sum e, D += sum e dP       (one thread per row; m moves lazily, as in the forward)
//       A += (e dP) K,  B += e K                         (weights written back to tensor memory as 16-bit A operands)
//     and at the end  delta = D / l,  dQx = scale (A - delta B) / l,  lse = m + log2 l.
//   bwd_tc_keys_kernel   one CTA per 128 keys, over the query tiles that see them, transposed so that a thread
//     owns a key:  S^T = K Qx^T, dP^T = Vx dO^T,  P^T = 2^(c S^T - lse_i),  dS^T = P^T (dP^T - delta_i),
//       dVx += P^T dO,  dK += scale dS^T Qx.
//
// Threads: eight weight warps (two threads per row or key) and a warpgroup of four issuing threads, one per kind
// of product (the loads ride with one of them).  What bounds a tile today is the weight threads' pass (tensor-memory
// load, maximum and its exchange, exponentials, packing, store: some 2500 cycles) with the products (some 1900
// cycles of tensor-pipe time) running under it.
//
// Qx, Vx are the advected queries and diffused values (16-bit, made by a prologue kernel when the Navier-Stokes
// terms are on); the transposed stencils and the blend are handled around the kernels as in attn_bwd.cu.
// Tensor memory: 512 columns per CTA (two 128-column products, two 64-column weight operands, two 64-column
// accumulators), so one CTA per SM.  Every mbarrier wait is bounded; a wait that runs out raises the context's
// status word (LOGOS_ERR_KERNEL_TIMEOUT) and the CTA winds down.
#include <algorithm>

#include "tcgen05_ptx.cuh"

namespace logos {
namespace {

using namespace tc;

constexpr int kBT = 128;                     // rows of a tile (queries or keys)
constexpr int kBD = 64;                      // head dimension
constexpr int kBTile = kBT * kBD * 2;        // 16 KiB
// registers per thread after the warpgroups have traded them (the kernels start with 65536 / 384 = 168):
// 256 weight threads x 224 + 128 control-group threads x 56 = 64512
constexpr int kRegsWeight = 224, kRegsCtrl = 56;
constexpr float kLazy = 4.0f;                // the running maximum moves when it would grow by more than 2^4

struct BwdTcArgs {
    float* dQx; float* dK; float* dVx;       // [BH][S][64] fp32
    float* lse; float* delta;                // [BH][S]: log2-domain log-sum-exp (c folded in) and delta
    int S;
    float c, scale, w;                       // c = scale * log2(e); w multiplies the results (share of a blend)
    int causal, shunyam, window, stride, f16, accumulate_dk;
    int* status;
};

// does key tile [k0, k0 + 128) show anything to query rows [q0, q_last]?
__device__ __forceinline__ bool tile_visible(const BwdTcArgs& a, int q0, int q_last, int k0) {
    if (k0 >= a.S) return false;
    if (a.causal && k0 > q_last) return false;
    if (!a.shunyam) return true;
    const bool in_win = (k0 + kBT - 1 >= q0 - a.window) && (k0 <= q_last);
    bool has_land = false;
    if (a.stride > 0) {
        const int first = ((k0 + a.stride - 1) / a.stride) * a.stride;
        has_land = first < k0 + kBT && first < a.S;
    }
    return in_win || has_land;
}

// two values as one word of the operand type; FP16 saturates at +-65504 instead of turning into infinity (a weight
// e dP or dS beyond that is outside what FP16 operands can carry: BF16 has the range)
// The operand type is a template parameter of the kernels: a run-time switch inside the unrolled passes costs
// instructions per pair and doubles their code.
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float x, float y) {
    // one packed conversion per pair: two scalar conversions would go through the XU pipe, which the
    // exponentials already keep busy
    if (F16) {
        uint32_t w;      // x in the lower half; the conversion itself saturates
        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(y), "f"(x));
        return w;
    }
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}

// MN-major B operand: a [128 rows (the k dimension)][64] tile as TMA wrote it, 16 rows (2048 bytes) per k step
__device__ __forceinline__ uint64_t desc_rows(uint32_t tile, int kk) { return smem_desc(tile + (uint32_t)kk * 2048u); }
// K-major operand: 16 of the 64 channels (32 bytes) per k step
__device__ __forceinline__ uint64_t desc_chan(uint32_t tile, int kk) { return smem_desc(tile + (uint32_t)kk * 32u); }

// 32 fp32 values -> 16 packed words written to tensor memory columns [col, col + 16)
template <bool F16>
__device__ __forceinline__ void st_packed32(uint32_t taddr, const float* v) {
    uint32_t pk[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) pk[e] = pack2<F16>(v[16 * h + 2 * e], v[16 * h + 2 * e + 1]);
        tc_st8(taddr + 8u * (uint32_t)h, pk);
    }
}

// The streamed operand pairs (K and V tiles in the rows kernel, Q and dO tiles in the keys kernel) go through a ring
// of kStages stages; a load is issued two tiles before its scores are.
constexpr int kStages = 4;
enum { RB_QG = 0, RB_KVFULL0 = 1, RB_KVEMPTY0 = RB_KVFULL0 + kStages, RB_SFULL = RB_KVEMPTY0 + kStages, RB_SEMPTY, RB_WFULL,
       RB_ACC, RB_XCH, RB_NUM };
constexpr int kRowsOffXch = (2 + 2 * kStages) * kBTile;                       // [2][2][128] floats: the half rows' maxima (and, at the end, sums)
constexpr int kRowsOffBar = kRowsOffXch + 2 * 2 * kBT * 4;
constexpr int kRowsSmem = kRowsOffBar + RB_NUM * 8 + 64 + 1024;
// Eight weight warps: a query row is shared by two threads (warps w and w + 4 own the same tensor-memory lanes), each
// taking 64 of the tile's 128 keys.  They agree on the row's maximum through shared memory once per tile and keep
// partial sums of their own until the end.
constexpr int kRowsThreads = 384;      // three warpgroups: two of weight warps, one of issuing warps
constexpr int kRowsCtrl = 8;

template <bool F16>
__global__ void __launch_bounds__(kRowsThreads, 1)
bwd_tc_rows_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapG, const BwdTcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t sQ = sbase, sG = sbase + kBTile, sK = sbase + 2 * kBTile, sV = sbase + (2 + kStages) * kBTile;
    float* xch = reinterpret_cast<float*>(smem + kRowsOffXch);
    const uint32_t bar0 = sbase + kRowsOffBar;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kRowsOffBar + RB_NUM * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kRowsOffBar + RB_NUM * 8 + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // grid (B H, query blocks), the last query block first: under a causal mask it sees the most key tiles, and CTAs
    // are handed out in this order, so the long ones start first and the short ones fill the end of the grid
    const int S = a.S, bh = blockIdx.x;
    const int q0 = (gridDim.y - 1 - blockIdx.y) * kBT, q_last = min(S, q0 + kBT) - 1;
    const int kt_end = (S + kBT - 1) / kBT;
    constexpr bool f16 = F16;

    if (warp == kRowsCtrl && lane == 0) {
        mbar_init(bar(RB_QG), 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(bar(RB_KVFULL0 + s), 1); mbar_init(bar(RB_KVEMPTY0 + s), 2); }
        mbar_init(bar(RB_SFULL), 2);         // two issuing threads commit each of SFULL, ACC and KVEMPTY
        mbar_init(bar(RB_SEMPTY), 256);
        mbar_init(bar(RB_WFULL), 256);
        mbar_init(bar(RB_ACC), 2);
        mbar_init(bar(RB_XCH), 256);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kRowsCtrl) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S 0, dP 128, W1 = e dP 256, W2 = e 320, A 384, B 448
    constexpr uint32_t cS = 0, cP = 128, cW1 = 256, cW2 = 320, cA = 384, cB = 448;

    auto next_visible = [&](int kt) {        // first visible key tile at or after kt (kt_end: none)
        while (kt < kt_end && !tile_visible(a, q0, q_last, kt * kBT)) ++kt;
        return kt;
    };

    // registers move from the control warpgroup (one thread busy in each warp) to the weight warpgroups, which hold a
    // tile's scores and their gradients in registers
    if (warp >= kRowsCtrl) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsCtrl));
        if (lane == 0) {
            // One thread of each warp of this warpgroup issues one kind of product (an MMA costs its issuing thread some
            // 75 cycles, so one thread issuing a tile's 24 MMAs was the period of the whole CTA):
            //   role 0: A += (e dP) K        role 1: B += e K
            //   role 2: the loads and S = Qx K^T      role 3: dP = dO Vx^T
            const int role = warp - kRowsCtrl;
            const int fmt = f16 ? 0 : 1;
            const uint32_t idesc_s = instr_desc(fmt, fmt, 0, kBT), idesc_acc = instr_desc(fmt, fmt, 1, kBD);
            bool ok = true;
            if (role >= 2) {
                int kt_load = next_visible(0), n_load = 0;
                auto load_next = [&]() {         // the next visible tile into its stage, once the products that read it are done
                    if (kt_load >= kt_end) return;
                    const int st = n_load % kStages;
                    if (n_load >= kStages && !mbar_wait(bar(RB_KVEMPTY0 + st), (n_load / kStages - 1) & 1, abort_flag)) { ok = false; return; }
                    mbar_expect_tx(bar(RB_KVFULL0 + st), 2 * kBTile);
                    tma_load_3d(sK + st * kBTile, &mapK, 0, kt_load * kBT, bh, bar(RB_KVFULL0 + st));
                    tma_load_3d(sV + st * kBTile, &mapV, 0, kt_load * kBT, bh, bar(RB_KVFULL0 + st));
                    ++n_load;
                    kt_load = next_visible(kt_load + 1);
                };
                if (role == 2) {
                    mbar_expect_tx(bar(RB_QG), 2 * kBTile);
                    tma_load_3d(sQ, &mapQ, 0, q0, bh, bar(RB_QG));
                    tma_load_3d(sG, &mapG, 0, q0, bh, bar(RB_QG));
                    for (int u = 0; u < kStages; ++u) load_next();
                }
                int n = 0;
                for (int kt = next_visible(0); ok && kt < kt_end; kt = next_visible(kt + 1), ++n) {
                    // the scores of tile n are issued as soon as the threads hold tile n - 1's in registers, so they run
                    // under the threads' pass over tile n - 1
                    const int st = n % kStages;
                    if (n == 0 && !mbar_wait(bar(RB_QG), 0, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(bar(RB_KVFULL0 + st), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                    if (n > 0 && !mbar_wait(bar(RB_SEMPTY), (n - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBD / 16; ++kk) {
                        if (role == 2) tc_mma_f16(tmem + cS, desc_chan(sQ, kk), desc_chan(sK + st * kBTile, kk), idesc_s, kk > 0 ? 1u : 0u);
                        else           tc_mma_f16(tmem + cP, desc_chan(sG, kk), desc_chan(sV + st * kBTile, kk), idesc_s, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(bar(RB_SFULL));
                    // tile n + 2 goes into the stage of tile n - 2, whose accumulating products end about now; this
                    // thread has the time to wait for them, and the load has two tiles' time to arrive
                    if (role == 2 && n >= kStages - 2) load_next();
                }
            } else {
                int n = 0;
                for (int kt = next_visible(0); ok && kt < kt_end; kt = next_visible(kt + 1), ++n) {
                    const int st = n % kStages;
                    if (!mbar_wait(bar(RB_KVFULL0 + st), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(bar(RB_WFULL), n & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBT / 16; ++kk) {
                        const uint64_t bd = desc_rows(sK + st * kBTile, kk);
                        const uint32_t accu = (n > 0 || kk > 0) ? 1u : 0u;
                        if (role == 0) tc_mma_f16_ta(tmem + cA, tmem + cW1 + 8u * (uint32_t)kk, bd, idesc_acc, accu);
                        else           tc_mma_f16_ta(tmem + cB, tmem + cW2 + 8u * (uint32_t)kk, bd, idesc_acc, accu);
                    }
                    tc_commit(bar(RB_ACC));
                    tc_commit(bar(RB_KVEMPTY0 + st));
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsWeight));
        // ================= two threads per query row: (lane quarter, half of the key columns) =================
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane, i = q0 + r;
        const uint32_t lane_addr = ((uint32_t)(quarter * 32)) << 16;
        const uint32_t col_s = (uint32_t)(64 * half), col_w = (uint32_t)(32 * half);
        const bool causal = a.causal != 0, shun = a.shunyam != 0;
        float m_run = -INFINITY, l_run = 0.0f, d_run = 0.0f;      // l, d: this thread's half of the row's sums
        bool ok = true;
        int n = 0;                // visible tiles done
        int nx = 0;               // exchanges done (one per tile, one more at the end)
        // both halves of a row publish a value and read each other's; two buffers in turn (a thread can only write
        // exchange x + 2 after everyone has arrived for exchange x + 1, i.e. has read exchange x); bounded wait
        auto exchange = [&](float mine, float& other) {
            float* buf = xch + (nx & 1) * 2 * kBT;
            buf[half * kBT + r] = mine;
            mbar_arrive(bar(RB_XCH));
            const bool fine = mbar_wait(bar(RB_XCH), nx & 1, abort_flag);
            other = buf[(half ^ 1) * kBT + r];
            ++nx;
            return fine;
        };
        for (int kt = next_visible(0); ok && kt < kt_end; kt = next_visible(kt + 1), ++n) {
            const int k0 = kt * kBT, kh = k0 + 64 * half;
            if (!mbar_wait(bar(RB_SFULL), n & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            float s[64], dp[64];
            tc_ld32(tmem + lane_addr + cS + col_s, s);
            tc_ld32(tmem + lane_addr + cS + col_s + 32, s + 32);
            tc_ld32(tmem + lane_addr + cP + col_s, dp);
            tc_ld32(tmem + lane_addr + cP + col_s + 32, dp + 32);
            tc_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(RB_SEMPTY));      // S and dP are in registers: the next tile's scores may overwrite them
            // a tile wholly inside the sequence and (if causal) wholly below the diagonal needs no mask
            const bool full = !shun && q0 + kBT <= S && k0 + kBT <= S && (!causal || k0 + kBT - 1 <= q0);
            if (!full) {
                // allowed(i, j) as in key_allowed() (cuda/VedicGEMM.cu:987-996), with the landmark rule's remainder
                // carried along the row instead of divided out per key
                int rem = (shun && a.stride > 0) ? kh % a.stride : 1;
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const int key = kh + j;
                    bool okj = i < S && key < S && (!causal || key <= i);
                    if (shun) okj = okj && ((key >= i - a.window && key <= i) || (a.stride > 0 && rem == 0));
                    rem = (rem + 1 == a.stride) ? 0 : rem + 1;
                    if (!okj) s[j] = -INFINITY;
                }
            }
            // the maximum of the raw products (the factor c is positive and goes into the exponent's multiply-add):
            // three-input maxima on eight independent chains instead of one chain of 64 dependent instructions
            float mx;
            {
                float mc[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) mc[q] = fmaxf(s[2 * q], s[2 * q + 1]);
#pragma unroll
                for (int j = 16; j < 64; j += 16)
#pragma unroll
                    for (int q = 0; q < 8; ++q) mc[q] = fmaxf(fmaxf(mc[q], s[j + 2 * q]), s[j + 2 * q + 1]);
                mx = fmaxf(fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3])), fmaxf(fmaxf(mc[4], mc[5]), fmaxf(mc[6], mc[7]))) * a.c;
                float other;
                if (!exchange(mx, other)) { ok = false; break; }
                mx = fmaxf(mx, other);           // the row's maximum over the whole tile: the same in both threads
            }
            // lazy running maximum: a warp-wide decision, because the correction is a warp-collective access; the two
            // warps of a row see the same maxima and decide alike
            const bool want = (mx > m_run + kLazy) || (m_run == -INFINITY && mx > -INFINITY);
            const bool any = __any_sync(0xffffffffu, want && n > 0 && m_run > -INFINITY);
            float m_new = want ? mx : m_run;
            if (any && m_new < mx) m_new = mx;       // correcting anyway: take the exact maximum
            if (n > 0) {       // the accumulators and the weight columns are in use until the previous products are done
                if (!mbar_wait(bar(RB_ACC), (n - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
            }
            if (any) {
                const float f = (m_run == -INFINITY) ? 0.0f : ex2(m_run - m_new);
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {       // half 0 corrects A, half 1 corrects B (64 columns each)
                    float o[32];
                    const uint32_t col = (half == 0 ? cA : cB) + 32u * (uint32_t)hc;
                    tc_ld32(tmem + lane_addr + col, o);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= f;
                    tc_st32(tmem + lane_addr + col, o);
                }
                l_run *= f;
                d_run *= f;
            }
            // without `any`, a lane only moves its maximum while its sums are still empty (first tile, or nothing seen yet)
            m_run = m_new;
            const float neg_m = (m_run == -INFINITY) ? 0.0f : -m_run;
            // the arithmetic runs on register pairs (two-wide fp32 instructions), the sums on two chains each
            const float2 c2 = make_float2(a.c, a.c), nm2 = make_float2(neg_m, neg_m);
            float2 lsum[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
            float2 dsum[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int x = 32 * cb + j;
                    const float2 t = __ffma2_rn(make_float2(s[x], s[x + 1]), c2, nm2);
                    const float2 e = make_float2(ex2(t.x), ex2(t.y));             // -inf gives 0
                    s[x] = e.x; s[x + 1] = e.y;
                    lsum[(j >> 1) & 1] = __fadd2_rn(lsum[(j >> 1) & 1], e);
                    const float2 w = __fmul2_rn(make_float2(dp[x], dp[x + 1]), e);    // e dP
                    dp[x] = w.x; dp[x + 1] = w.y;
                    dsum[(j >> 1) & 1] = __fadd2_rn(dsum[(j >> 1) & 1], w);
                }
                st_packed32<F16>(tmem + lane_addr + cW1 + col_w + 16 * cb, dp + 32 * cb);
                st_packed32<F16>(tmem + lane_addr + cW2 + col_w + 16 * cb, s + 32 * cb);
            }
            l_run += (lsum[0].x + lsum[0].y) + (lsum[1].x + lsum[1].y);
            d_run += (dsum[0].x + dsum[0].y) + (dsum[1].x + dsum[1].y);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(RB_WFULL));       // the weights are in place
        }
        // the row's sums: this half's plus the other's
        if (ok) {
            float other;
            ok = exchange(l_run, other);
            l_run += other;
            if (ok) {
                ok = exchange(d_run, other);
                d_run += other;
            }
        }
        if (ok && n > 0) ok = mbar_wait(bar(RB_ACC), (n - 1) & 1, abort_flag);
        if (ok) {
            tc_fence_after();
            const bool live = n > 0 && l_run > 1e-9f;     // a row that saw nothing was written as zeros by the forward
            const float inv = live ? 1.0f / l_run : 0.0f;
            const float dlt = d_run * inv;
            if (i < S && half == 0) {
                a.lse[(size_t)bh * S + i] = live ? m_run + log2f(l_run) : INFINITY;
                a.delta[(size_t)bh * S + i] = dlt;
            }
            // each half writes 32 of the row's 64 channels
            float* dst = a.dQx + ((size_t)bh * S + i) * kBD + 32 * half;
            float av[32], bv[32];
            if (n > 0) {
                tc_ld32(tmem + lane_addr + cA + col_w, av);
                tc_ld32(tmem + lane_addr + cB + col_w, bv);
                tc_wait_ld();
            }
            if (i < S) {
                const float k1 = a.scale * inv * a.w;
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (live) o4 = make_float4((av[j] - dlt * bv[j]) * k1, (av[j + 1] - dlt * bv[j + 1]) * k1,
                                               (av[j + 2] - dlt * bv[j + 2]) * k1, (av[j + 3] - dlt * bv[j + 3]) * k1);
                    *reinterpret_cast<float4*>(dst + j) = o4;
                }
            }
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) atomicExch(a.status, (*abort_flag & ~0xffff) | ((*abort_flag - (int)(bar0 & 0xffffu)) & 0xffff));
    if (warp == kRowsCtrl) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

enum { KB_KV = 0, KB_QGFULL0 = 1, KB_QGEMPTY0 = KB_QGFULL0 + kStages, KB_SFULL = KB_QGEMPTY0 + kStages, KB_SEMPTY, KB_WFULL,
       KB_ACC, KB_STAT, KB_NUM };
constexpr int kKeysOffStat = (2 + 2 * kStages) * kBTile;                       // [2][2][128] floats: lse, delta of two query tiles in turn
constexpr int kKeysOffBar = kKeysOffStat + 2 * 2 * kBT * 4;
constexpr int kKeysSmem = kKeysOffBar + KB_NUM * 8 + 64 + 1024;

// Eight weight warps here: a key row is shared by two threads (warps w and w + 4 own the same tensor-memory lanes),
// each taking 64 of the tile's 128 queries -- no exchange is needed, the statistics come from the rows kernel.
constexpr int kKeysThreads = 384;      // as in the rows kernel
constexpr int kKeysCtrl = 8;

template <bool F16>
__global__ void __launch_bounds__(kKeysThreads, 1)
bwd_tc_keys_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapG, const BwdTcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t sK = sbase, sV = sbase + kBTile, sQ = sbase + 2 * kBTile, sG = sbase + (2 + kStages) * kBTile;
    float* stat = reinterpret_cast<float*>(smem + kKeysOffStat);
    const uint32_t bar0 = sbase + kKeysOffBar;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kKeysOffBar + KB_NUM * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kKeysOffBar + KB_NUM * 8 + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // grid (B H, key blocks), the first key block first: under a causal mask it is seen by the most query tiles
    const int S = a.S, bh = blockIdx.x;
    const int k0 = blockIdx.y * kBT, k_last = min(S, k0 + kBT) - 1;
    constexpr bool f16 = F16;
    // query tiles that can see these keys: from the diagonal on (causal); a pure window ends them early
    const int qt_begin = a.causal ? k0 / kBT : 0;
    int qt_end = (S + kBT - 1) / kBT;
    if (a.shunyam && a.stride <= 0) qt_end = min(qt_end, (k_last + a.window) / kBT + 1);

    if (warp == kKeysCtrl && lane == 0) {
        mbar_init(bar(KB_KV), 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(bar(KB_QGFULL0 + s), 1); mbar_init(bar(KB_QGEMPTY0 + s), 2); }
        mbar_init(bar(KB_SFULL), 2);
        mbar_init(bar(KB_SEMPTY), 256);
        mbar_init(bar(KB_WFULL), 256);
        mbar_init(bar(KB_ACC), 2);
        mbar_init(bar(KB_STAT), 256);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kKeysCtrl) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns: S^T 0, dP^T 128, P^T 256, dS^T 320, dV 384, dK 448
    constexpr uint32_t cS = 0, cP = 128, cW1 = 256, cW2 = 320, cV = 384, cK = 448;

    auto next_visible = [&](int qt) {        // first query tile at or after qt that sees this key tile
        while (qt < qt_end && !tile_visible(a, qt * kBT, min(S, qt * kBT + kBT) - 1, k0)) ++qt;
        return qt;
    };

    if (warp >= kKeysCtrl) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsCtrl));
        if (lane == 0) {
            // as in the rows kernel, one issuing thread per kind of product:
            //   role 0: dVx += P^T dO        role 1: dK += dS^T Qx
            //   role 2: the loads and S^T = K Qx^T    role 3: dP^T = Vx dO^T
            const int role = warp - kKeysCtrl;
            const int fmt = f16 ? 0 : 1;
            const uint32_t idesc_s = instr_desc(fmt, fmt, 0, kBT), idesc_acc = instr_desc(fmt, fmt, 1, kBD);
            bool ok = true;
            if (role >= 2) {
                int qt_load = next_visible(qt_begin), n_load = 0;
                auto load_next = [&]() {
                    if (qt_load >= qt_end) return;
                    const int st = n_load % kStages;
                    if (n_load >= kStages && !mbar_wait(bar(KB_QGEMPTY0 + st), (n_load / kStages - 1) & 1, abort_flag)) { ok = false; return; }
                    mbar_expect_tx(bar(KB_QGFULL0 + st), 2 * kBTile);
                    tma_load_3d(sQ + st * kBTile, &mapQ, 0, qt_load * kBT, bh, bar(KB_QGFULL0 + st));
                    tma_load_3d(sG + st * kBTile, &mapG, 0, qt_load * kBT, bh, bar(KB_QGFULL0 + st));
                    ++n_load;
                    qt_load = next_visible(qt_load + 1);
                };
                if (role == 2) {
                    mbar_expect_tx(bar(KB_KV), 2 * kBTile);
                    tma_load_3d(sK, &mapK, 0, k0, bh, bar(KB_KV));
                    tma_load_3d(sV, &mapV, 0, k0, bh, bar(KB_KV));
                    for (int u = 0; u < kStages; ++u) load_next();
                }
                int n = 0;
                for (int qt = next_visible(qt_begin); ok && qt < qt_end; qt = next_visible(qt + 1), ++n) {
                    const int st = n % kStages;
                    if (n == 0 && !mbar_wait(bar(KB_KV), 0, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(bar(KB_QGFULL0 + st), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                    if (n > 0 && !mbar_wait(bar(KB_SEMPTY), (n - 1) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBD / 16; ++kk) {
                        if (role == 2) tc_mma_f16(tmem + cS, desc_chan(sK, kk), desc_chan(sQ + st * kBTile, kk), idesc_s, kk > 0 ? 1u : 0u);
                        else           tc_mma_f16(tmem + cP, desc_chan(sV, kk), desc_chan(sG + st * kBTile, kk), idesc_s, kk > 0 ? 1u : 0u);
                    }
                    tc_commit(bar(KB_SFULL));
                    if (role == 2 && n >= kStages - 2) load_next();
                }
            } else {
                int n = 0;
                for (int qt = next_visible(qt_begin); ok && qt < qt_end; qt = next_visible(qt + 1), ++n) {
                    const int st = n % kStages;
                    if (!mbar_wait(bar(KB_QGFULL0 + st), (n / kStages) & 1, abort_flag)) { ok = false; break; }
                    if (!mbar_wait(bar(KB_WFULL), n & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < kBT / 16; ++kk) {
                        const uint32_t accu = (n > 0 || kk > 0) ? 1u : 0u;
                        if (role == 0) tc_mma_f16_ta(tmem + cV, tmem + cW1 + 8u * (uint32_t)kk, desc_rows(sG + st * kBTile, kk), idesc_acc, accu);
                        else           tc_mma_f16_ta(tmem + cK, tmem + cW2 + 8u * (uint32_t)kk, desc_rows(sQ + st * kBTile, kk), idesc_acc, accu);
                    }
                    tc_commit(bar(KB_ACC));
                    tc_commit(bar(KB_QGEMPTY0 + st));
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsWeight));
        // ================= two threads per key: (lane quarter, half of the query columns) =================
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane, j = k0 + r;
        const uint32_t lane_addr = ((uint32_t)(quarter * 32)) << 16;
        const uint32_t col_s = (uint32_t)(64 * half), col_w = (uint32_t)(32 * half);
        const bool causal = a.causal != 0, shun = a.shunyam != 0;
        bool ok = true;
        int n = 0;
        // a query tile's statistic is fetched one tile ahead, so its way from global memory is hidden behind the
        // previous tile's pass
        auto fetch_stat = [&](int qt) {
            const int q = qt * kBT + r;
            if (qt >= qt_end) return 0.0f;
            // both negated: they enter the pass as addends
            if (half == 0) return q < S ? -a.lse[(size_t)bh * S + q] : -INFINITY;
            return q < S ? -a.delta[(size_t)bh * S + q] : 0.0f;
        };
        int qt_next = next_visible(qt_begin);
        float stat_next = fetch_stat(qt_next);
        for (int qt = qt_next; ok && qt < qt_end; qt = qt_next, ++n) {
            const int q0 = qt * kBT, qh = q0 + 64 * half;
            qt_next = next_visible(qt + 1);
            // the query tile's statistics go through shared memory: the thread pair of row r fetches query r's
            // log-sum-exp and delta, all threads then read all of them (broadcast reads).  Two buffers in turn: a
            // thread can only write tile n + 2's after every thread has arrived for tile n + 1, i.e. has finished
            // reading tile n's.  The hand-over is an mbarrier with a bounded wait, so a CTA that is winding down
            // cannot get stuck in it.
            float* st_lse = stat + (n & 1) * 2 * kBT;
            float* st_dlt = st_lse + kBT;
            if (half == 0) st_lse[r] = stat_next;
            else           st_dlt[r] = stat_next;
            mbar_arrive(bar(KB_STAT));
            stat_next = fetch_stat(qt_next);
            if (!mbar_wait(bar(KB_STAT), n & 1, abort_flag)) { ok = false; break; }
            if (!mbar_wait(bar(KB_SFULL), n & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            float s[64], dp[64];
            tc_ld32(tmem + lane_addr + cS + col_s, s);
            tc_ld32(tmem + lane_addr + cS + col_s + 32, s + 32);
            tc_ld32(tmem + lane_addr + cP + col_s, dp);
            tc_ld32(tmem + lane_addr + cP + col_s + 32, dp + 32);
            tc_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(KB_SEMPTY));      // S^T and dP^T are in registers: the next tile's scores may overwrite them
            // a tile wholly inside the sequence and (if causal) wholly below the diagonal needs no mask
            const bool full = !shun && q0 + kBT <= S && k0 + kBT <= S && (!causal || k0 + kBT - 1 <= q0);
            // the statistics (stored negated) are read four at a time -- every thread reads the same words:
            // broadcasts -- and the arithmetic runs on register pairs (two-wide fp32 instructions)
            const float4* lse4 = reinterpret_cast<const float4*>(st_lse + 64 * half);
            const float4* dlt4 = reinterpret_cast<const float4*>(st_dlt + 64 * half);
            const float2 c2 = make_float2(a.c, a.c);
            if (full) {
#pragma unroll
                for (int q = 0; q < 64; q += 4) {
                    const float4 l = lse4[q >> 2];
                    const float2 t0 = __ffma2_rn(make_float2(s[q], s[q + 1]), c2, make_float2(l.x, l.y));
                    const float2 t1 = __ffma2_rn(make_float2(s[q + 2], s[q + 3]), c2, make_float2(l.z, l.w));
                    s[q] = ex2(t0.x); s[q + 1] = ex2(t0.y);
                    s[q + 2] = ex2(t1.x); s[q + 3] = ex2(t1.y);
                }
            } else {
                // allowed(i, j) as in key_allowed() (cuda/VedicGEMM.cu:987-996); whether this thread's key is a landmark
                // does not depend on the query
                const bool landmark = shun && a.stride > 0 && (j % a.stride) == 0;
#pragma unroll
                for (int q = 0; q < 64; ++q) {
                    const int qi = qh + q;
                    bool okq = j < S && qi < S && (!causal || j <= qi);
                    if (shun) okq = okq && ((j >= qi - a.window && j <= qi) || landmark);
                    s[q] = okq ? ex2(fmaf(s[q], a.c, st_lse[64 * half + q])) : 0.0f;   // p_ij; -lse = -inf for a dead row gives 0
                }
            }
            if (n > 0) {
                if (!mbar_wait(bar(KB_ACC), (n - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
            }
#pragma unroll
            for (int cb = 0; cb < 2; ++cb) {
                // ds_ij without the softmax scale: that factor multiplies the finished dK rows
#pragma unroll
                for (int q = 0; q < 32; q += 4) {
                    const int x = 32 * cb + q;
                    const float4 d = dlt4[x >> 2];
                    const float2 w0 = __fmul2_rn(make_float2(s[x], s[x + 1]), __fadd2_rn(make_float2(dp[x], dp[x + 1]), make_float2(d.x, d.y)));
                    const float2 w1 = __fmul2_rn(make_float2(s[x + 2], s[x + 3]), __fadd2_rn(make_float2(dp[x + 2], dp[x + 3]), make_float2(d.z, d.w)));
                    dp[x] = w0.x; dp[x + 1] = w0.y;
                    dp[x + 2] = w1.x; dp[x + 3] = w1.y;
                }
                st_packed32<F16>(tmem + lane_addr + cW1 + col_w + 16 * cb, s + 32 * cb);
                st_packed32<F16>(tmem + lane_addr + cW2 + col_w + 16 * cb, dp + 32 * cb);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(KB_WFULL));
        }
        if (ok && n > 0) ok = mbar_wait(bar(KB_ACC), (n - 1) & 1, abort_flag);
        if (ok) {
            tc_fence_after();
            // half 0 writes the key's dV row, half 1 its dK row
            float* dst = (half == 0 ? a.dVx : a.dK) + ((size_t)bh * S + j) * kBD;
            const bool acc_out = half == 1 && a.accumulate_dk;
            const float wo = half == 0 ? a.w : a.w * a.scale;
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {
                float v[32];
#pragma unroll
                for (int q = 0; q < 32; ++q) v[q] = 0.0f;
                if (n > 0) {
                    tc_ld32(tmem + lane_addr + (half == 0 ? cV : cK) + 32 * hc, v);
                    tc_wait_ld();
                }
                if (j < S) {
#pragma unroll
                    for (int q = 0; q < 32; q += 4) {
                        float4* p4 = reinterpret_cast<float4*>(dst + 32 * hc + q);
                        float4 o4 = make_float4(v[q] * wo, v[q + 1] * wo, v[q + 2] * wo, v[q + 3] * wo);
                        if (acc_out) { const float4 old = *p4; o4.x += old.x; o4.y += old.y; o4.z += old.z; o4.w += old.w; }
                        *p4 = o4;
                    }
                }
            }
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) atomicExch(a.status, (*abort_flag & ~0xffff) | ((*abort_flag - (int)(bar0 & 0xffffu)) & 0xffff));
    if (warp == kKeysCtrl) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// Qx = advect(Q), Vx = diffuse(V) in the operand type (ns_advect_kernel, ns_diffuse_kernel, cuda/ModelGPU.cu:443-471;
// the central stencil is navier_stokes_attention's, include/Attention.hpp:168-182), fp32 arithmetic, one rounding
template <typename T>
__global__ void bwd16_prologue_kernel(const T* __restrict__ Q, const T* __restrict__ V, T* __restrict__ Qa, T* __restrict__ Vs,
                                      int S, float eta, float nu, int mode, int64_t total) {
    for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (int64_t)gridDim.x * blockDim.x) {
        const int i = (int)((x / kBD) % S);
        const float q = to_f32<T>(Q[x]), v = to_f32<T>(V[x]);
        const float qp = i > 0 ? to_f32<T>(Q[x - kBD]) : q;
        Qa[x] = from_f32<T>(q + eta * (q - qp));
        float vs = v;
        if (mode == LOGOS_DIFFUSE_CAUSAL) {
            const float vp = i > 0 ? to_f32<T>(V[x - kBD]) : v;
            vs = (1.0f - nu) * v + nu * vp;
        } else if (mode == LOGOS_DIFFUSE_CENTRAL) {
            const float vl = i > 0 ? to_f32<T>(V[x - kBD]) : v, vr = i < S - 1 ? to_f32<T>(V[x + kBD]) : v;
            vs = (1.0f - nu) * v + (nu * 0.5f) * (vl + vr);
        }
        Vs[x] = from_f32<T>(vs);
    }
}

// [BH][S][64] 16-bit tensor, box = 128 rows x 64 channels of one head, 128-byte swizzle
bool make_map_bwd(CUtensorMap* m, const void* base, int BH, int S, bool f16) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)kBD, (cuuint64_t)S, (cuuint64_t)BH};
    cuuint64_t strides[2] = {(cuuint64_t)kBD * 2, (cuuint64_t)S * kBD * 2};
    cuuint32_t box[3] = {(cuuint32_t)kBD, (cuuint32_t)kBT, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

size_t attention_bwd16_workspace_bytes(int B, int H, int S, int DH) {
    if (B <= 0 || H <= 0 || S <= 0 || DH <= 0) return 0;
    const size_t n = (size_t)B * H * S * DH;
    const size_t t16 = (n * 2 + 255) & ~(size_t)255, t32 = (n * 4 + 255) & ~(size_t)255;
    const size_t r = ((size_t)B * H * S * 4 + 255) & ~(size_t)255;
    return kWorkspaceCounterBytes + 2 * t16 + 2 * t32 + 2 * r;     // Qx, Vx; dQx, dVx; log-sum-exp, delta
}

int attention_bwd16(logos_ctx* ctx, int dtype, const void* Q, const void* K, const void* V, const void* dO, float* dQ,
                    float* dK, float* dV, int B, int H, int S, int DH, const logos_attn_params* p) {
    if (!Q || !K || !V || !dO || !dQ || !dK || !dV || B <= 0 || H <= 0 || S <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_bwd16: bad pointer or extent");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16)
        return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention_bwd16: operands are BF16 or FP16");
    if (DH != kBD) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention_bwd16: DH must be 64, got %d", DH);
    if ((S + kBT - 1) / kBT > 65535) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "attention_bwd16: more than 65535 blocks of 128 tokens");
    if (!(p->scale > 0.0f)) return fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_bwd16: scale must be positive");
    const void* ptrs[7] = {Q, K, V, dO, dQ, dK, dV};
    for (const void* q : ptrs)
        if (!aligned16(q)) return fail(ctx, LOGOS_ERR_ALIGNMENT, "attention_bwd16: tensors must be 16-byte aligned");
    if (!ctx->tc_status) return fail(ctx, LOGOS_ERR_WORKSPACE, "attention_bwd16: status word missing");
    const size_t need = attention_bwd16_workspace_bytes(B, H, S, DH);
    if (!ctx->workspace || ctx->workspace_bytes < need)
        return fail(ctx, LOGOS_ERR_WORKSPACE, "attention_bwd16: workspace of %zu bytes needed, %zu reserved "
                    "(logos_attention_bwd16_workspace_bytes / logos_ctx_reserve)", need, ctx->workspace_bytes);
    const int BH = B * H;
    const int64_t total = (int64_t)BH * S * DH;
    const size_t t16 = ((size_t)total * 2 + 255) & ~(size_t)255, t32 = ((size_t)total * 4 + 255) & ~(size_t)255;
    const size_t r = ((size_t)BH * S * 4 + 255) & ~(size_t)255;
    char* ws = static_cast<char*>(ctx->workspace) + kWorkspaceCounterBytes;
    void* Qa = ws;
    void* Vs = ws + t16;
    float* dQa = (float*)(ws + 2 * t16);
    float* dVs = (float*)(ws + 2 * t16 + t32);
    float* lse = (float*)(ws + 2 * t16 + 2 * t32);
    float* delta = (float*)(ws + 2 * t16 + 2 * t32 + r);

    const bool f16 = dtype == LOGOS_F16;
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    const bool std_on = !ns_any || p->ns_alpha < 1.0f;
    const int mode = ns_any ? p->diffuse_mode : LOGOS_DIFFUSE_NONE;
    const int ew_blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 16);

    BwdTcArgs a{};
    a.dQx = dQa; a.dK = dK; a.dVx = dVs; a.lse = lse; a.delta = delta;
    a.S = S; a.scale = p->scale; a.c = p->scale * 1.4426950408889634f;
    a.causal = p->causal; a.shunyam = shunyam_active(p->window, S) ? 1 : 0;
    a.window = p->window; a.stride = p->stride; a.f16 = f16; a.status = ctx->tc_status;
    auto* rows_fn = f16 ? bwd_tc_rows_kernel<true> : bwd_tc_rows_kernel<false>;
    auto* keys_fn = f16 ? bwd_tc_keys_kernel<true> : bwd_tc_keys_kernel<false>;
    if (int rc = ensure_smem_limit(ctx, rows_fn, kRowsSmem)) return rc;
    if (int rc = ensure_smem_limit(ctx, keys_fn, kKeysSmem)) return rc;
    CUtensorMap mk, mg;
    if (!make_map_bwd(&mk, K, BH, S, f16) || !make_map_bwd(&mg, dO, BH, S, f16))
        return fail(ctx, LOGOS_ERR_CUDA, "attention_bwd16: cuTensorMapEncodeTiled failed");
    dim3 grid(BH, (S + kBT - 1) / kBT);
    auto run = [&](const void* Qx, const void* Vx) -> int {
        CUtensorMap mq, mv;
        if (!make_map_bwd(&mq, Qx, BH, S, f16) || !make_map_bwd(&mv, Vx, BH, S, f16))
            return fail(ctx, LOGOS_ERR_CUDA, "attention_bwd16: cuTensorMapEncodeTiled failed");
        rows_fn<<<grid, kRowsThreads, kRowsSmem, ctx->stream>>>(mq, mk, mv, mg, a);
        LOGOS_LAUNCH_CHECK(ctx, "bwd_tc_rows_kernel");
        keys_fn<<<grid, kKeysThreads, kKeysSmem, ctx->stream>>>(mq, mk, mv, mg, a);
        LOGOS_LAUNCH_CHECK(ctx, "bwd_tc_keys_kernel");
        return LOGOS_OK;
    };
    bool first = true;
    if (ns_any) {
        if (f16) bwd16_prologue_kernel<__half><<<ew_blocks, 256, 0, ctx->stream>>>((const __half*)Q, (const __half*)V, (__half*)Qa, (__half*)Vs, S, p->ns_eta, p->ns_nu, mode, total);
        else bwd16_prologue_kernel<__nv_bfloat16><<<ew_blocks, 256, 0, ctx->stream>>>((const __nv_bfloat16*)Q, (const __nv_bfloat16*)V, (__nv_bfloat16*)Qa, (__nv_bfloat16*)Vs, S, p->ns_eta, p->ns_nu, mode, total);
        LOGOS_LAUNCH_CHECK(ctx, "bwd16_prologue_kernel");
        a.w = p->ns_alpha; a.accumulate_dk = 0;
        if (int rc = run(Qa, Vs)) return rc;
        if (int rc = attention_bwd_adjoint(ctx, dQa, dVs, dQ, dV, S, DH, p->ns_eta, p->ns_nu, mode, 1, 0, total)) return rc;
        first = false;
    }
    if (std_on) {
        a.w = ns_any ? 1.0f - p->ns_alpha : 1.0f; a.accumulate_dk = first ? 0 : 1;
        if (int rc = run(Q, V)) return rc;
        if (int rc = attention_bwd_adjoint(ctx, dQa, dVs, dQ, dV, S, DH, 0.0f, 0.0f, LOGOS_DIFFUSE_NONE, 0, first ? 0 : 1, total)) return rc;
    }
    return LOGOS_OK;
}

}  // namespace logos
