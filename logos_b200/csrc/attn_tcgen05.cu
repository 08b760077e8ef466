// attn_tcgen05.cu -- causal / sliding-window prefill attention on the 5th-generation
// tensor cores (tcgen05 + TMEM + TMA), BF16 or FP16 inputs, DH = 64.
//
// What it computes, per head: the attention of cuda_flash_attention_fwd
// (cuda/VedicGEMM.cu:901-1062 of LOGOS) on Q_adv and V_s, where Q_adv is the advected
// query (ns_advect_kernel, cuda/ModelGPU.cu:443-451) and V_s the causally diffused value
// (ns_diffuse_kernel, cuda/ModelGPU.cu:463-471) -- both fused here, no extra pass:
//   * Q_adv = Q + eta (Q - Q_prev) is formed once per CTA in fp32 from the TMA-loaded Q
//     tile and the same tile loaded one row higher, and kept as an exact pair of 16-bit
//     tiles (hi + lo), so QK^T costs two MMAs per k-step instead of a re-rounded Q_adv;
//   * V_s is never formed: the stencil is moved onto the softmax weights,
//       sum_j p_j V_s[j] = sum_r ((1-nu) p_r + nu p_{r+1}) V[r]   (+ nu p_0 V[0]),
//     which a softmax thread applies to the row it holds in registers.  KV tiles are
//     visited from the diagonal downwards so that p_{r+1} of the tile above is known.
//
// A work item = 256 query rows of one head as two 128-row tiles that share every K/V tile.  The CTA
// (384 threads, one per SM) is persistent: it walks its share of the item list, and all barriers and
// rings run on across items, so one item's epilogue overlaps the other tile's work and the next
// item's loads.  Roles, one warpgroup each so that registers can be moved between them (setmaxnreg):
//   warps 0-3 / 4-7  softmax of tile 0 / tile 1, one thread per query row (= TMEM lane) with the
//              row's 128 scores in registers: one tcgen05.ld of the row, then the S columns are
//              handed back at once (the next QK^T runs under this tile's exponentials); maximum,
//              weights and the diffusion stencil stay inside the thread; FP16 weights go back to
//              tensor memory with tcgen05.st, and finally O / l to global memory;
//   warp 8     TMA producers: lane 0 loads Q, Q_prev per item (two buffers) and the K tiles, lane 1 the
//              V tiles; K and V have separate two-stage rings (a K stage is free as soon as its scores
//              are done).  This warp also initialises the barriers, so its first loads leave before
//              the CTA's set-up (TMEM allocation, first CTA-wide barrier) has finished;
//   warps 9,10  MMA issuers, one per query tile: S_g = Q_adv,g K^T (M128 N128 K16 x 4 x {hi,lo}) from
//              shared-memory descriptors, O_g += W_g V (M128 N64 K16 x 8) with W read from tensor
//              memory; completion via tcgen05.commit; the scores of the next tile are issued before
//              the current tile's weights are waited for.  The whole warp runs the loop, one elected
//              lane issues;
//   warp 11    V converter: the MMA takes one type for both operands and the weights are FP16, so for
//              BF16 inputs this warp turns every V tile into FP16 in place (exact in FP16's normal range,
//              saturating beyond).  (Measured alternatives, all slower: the softmax threads doing it
//              lengthened their chain by a tenth; four converter warps in a warpgroup of their own left
//              the softmax threads 208 registers, 3 %; this warp with more loads in flight took issue
//              slots and shared-memory bandwidth from the softmax warps of its scheduler in bursts, 5 %.)
// TMEM (512 columns): S of tile 0 / 1 at [0,128) / [128,256), O at [256,320) / [320,384), FP16
// weights (two keys per column) at [384,448) / [448,512).
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA raises an abort
// flag, all roles leave their loops, TMEM is freed and the status word tells the host.
#include "tcgen05_ptx.cuh"

namespace logos {
namespace {

using namespace tc;

template <bool V> struct SkipDead { static constexpr bool value = V; };   // compile-time switch of the weight pass

constexpr int kTiles = 2;             // query tiles per CTA (2: both share every K/V tile, one CTA per SM)
constexpr int kCtasPerSm = kTiles == 1 ? 2 : 1;   // one tile per CTA: two CTAs share an SM and its 512 TMEM columns
constexpr int kBQ = kBM * kTiles;     // query rows per CTA
constexpr int kBN = 128;              // keys per tile
constexpr int kD = 64;                // head dimension
constexpr int kTileBytes = kBM * kD * 2;      // 16 KiB: one 128 x 64 16-bit tile
constexpr int kStages = 2;              // depth of the K ring and of the V ring (3 and 4 measured no faster)
constexpr int kSoftmaxWarps = 4 * kTiles;   // one warpgroup per query tile, one thread per row
constexpr int kSoftmaxThreads = 32 * kSoftmaxWarps;
constexpr int kTmaWarp = kSoftmaxWarps;          // then one MMA warp per query tile (the first also owns TMEM)
constexpr int kMmaWarp = kTmaWarp + 1;
constexpr int kCvtWarp = kMmaWarp + kTiles;      // V converter warp
constexpr int kCvtThreads = 32;
constexpr int kTcThreads = 32 * (kCvtWarp + 1);
static_assert(kTcThreads == 384 && kTmaWarp % 4 == 0, "three warpgroups: two of softmax threads, one of helpers");
// registers per thread after the warpgroups have traded them (the kernel starts with 65536 / 384 = 168):
// 256 softmax threads x 224 + 128 helper threads x 56 = 64512
#ifndef LOGOS_TC_REGS_SOFTMAX
#define LOGOS_TC_REGS_SOFTMAX 224
#define LOGOS_TC_REGS_HELPER 56
#endif
constexpr int kRegsSoftmax = LOGOS_TC_REGS_SOFTMAX, kRegsHelper = LOGOS_TC_REGS_HELPER;
constexpr uint32_t kTmemCols = 256 * kTiles;
constexpr uint32_t kColO = 128 * kTiles, kColP = kColO + 64 * kTiles;   // S first, then O, then the weights
constexpr float kRescaleThreshold = 8.0f;     // log2 units before the running max is moved

// shared memory map (bytes from a 1024-aligned base)
constexpr int kOffQ = 0;                                       // two buffers (work items alternate), each: per query tile hi, lo
constexpr int kQBufBytes = 2 * kTiles * kTileBytes;
constexpr int kOffK = kOffQ + 2 * kQBufBytes;                  // kStages tiles
constexpr int kOffV = kOffK + kStages * kTileBytes;            // kStages tiles
constexpr int kOffVP = kOffV + kStages * kTileBytes;           // two tiles in turn: the V[j-1] rows of a landmark tile (landmark kernels only)
constexpr int kOffBar = kOffVP + 2 * kTileBytes;
constexpr int kNumBars = 8 + 5 * kStages + 8 + 2;
constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 64 + 1024; // + tmem slot/abort + alignment slack

enum Bar { B_QLOAD0 = 0,                                   // two: one per Q buffer
           B_QREADY0 = 2,                                  // four: Q buffer * 2 + query tile
           B_QFREE0 = 6,                                   // two: one per Q buffer
           B_KFULL0 = 8, B_KEMPTY0 = B_KFULL0 + kStages, B_VFULL0 = B_KEMPTY0 + kStages,     // kStages of each
           B_VEMPTY0 = B_VFULL0 + kStages, B_VREADY0 = B_VEMPTY0 + kStages,
           B_SFULL0 = B_VREADY0 + kStages, B_SFULL1, B_SEMPTY0, B_SEMPTY1, B_PFULL0, B_PFULL1, B_PVDONE0, B_PVDONE1,
           B_VPEMPTY0, B_VPEMPTY1,                         // a V[j-1] buffer has been mixed into its V tile
           B_NUM };
static_assert(B_NUM <= kNumBars, "barrier count");

struct TcArgs {
    void* O;
    long long o_row, o_slab;    // elements between the rows of a head's output and between two (sequence, head) outputs
    int S, out_is_f32, in_is_f16;
    int o_al32;                 // O is 32-byte aligned: rows are stored 32 bytes at a time
    float c;            // scale * log2(e)
    float eta, nu;
    int diffuse;        // 0 none, 1 causal
    int window;         // > 0: sliding window active
    int stride;         // > 0: every key j % stride == 0 below the window is visible too (landmark kernels)
    int n_qb, BH, n_items;   // query blocks per head, heads, work items = n_qb * BH
    int* status;        // device word: non-zero = a wait ran out
};

// -------------------------------------------------------------------------------------
// LM: Shunyam landmarks.  After an item's window tiles come its landmark tiles: 128 landmarks m = 128 lt ... at
// keys m * stride, gathered by TMA through strided views of K and V (mapKl, mapVl: row pitch = stride rows).
// They are ordinary key tiles for QK^T, softmax and PV, except that (i) the mask is "key strictly below the
// row's window", (ii) neighbouring landmarks are not neighbouring keys, so the diffusion stencil cannot sit on
// the weights: the converter warp mixes the landmark's V row with the row before it (mapVp: the same view
// one row earlier) into V[j] + rho V[j-1] -- the same "everything divided by 1 - nu" units as the window
// part -- and the row sum takes (1 + rho) p.
// WIN: the launch has a window.  Only then does the weight pass carry its second copy that skips the 16-column chunks
// no row of a warp sees; the causal instantiations are the straight-line code alone.
template <bool DIFF, bool LM, bool WIN>
__global__ void __launch_bounds__(kTcThreads, kCtasPerSm)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapKl,
                  const __grid_constant__ CUtensorMap mapVl, const __grid_constant__ CUtensorMap mapVp, const TcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBar;
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBar + kNumBars * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffBar + kNumBars * 8 + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.S;
    const bool f16 = a.in_is_f16 != 0;
    const bool has_lo = a.eta != 0.0f;
    const int jt_max = (S - 1) / kBN;

    // The CTA is persistent: it works through the items blockIdx.x, blockIdx.x + gridDim.x, ... of the
    // list of (head, block of 256 query rows), long blocks (late rows) first.  Every role walks the
    // same list, barriers and rings run on across items (phases come from running counters), and
    // Q has two buffers, so the loads of the next item and the epilogue of one query tile overlap
    // the other tile's work instead of standing alone at a CTA's start and end.
    // Within an item, iteration i visits KV tile jt_hi - i.  Query tile g (rows q0 + 128 g ...) takes
    // part in iterations [first_iter(g), last_iter(g)]: above its diagonal and below its window it has
    // nothing to do.
    int qb = 0, bh = 0, q0 = 0, jt_hi = 0, jt_top0 = 0, jt_top1 = 0, jt_bot0 = 0, jt_bot1 = 0, n_iter = 0;
    int n_win = 0, n_lt0 = 0, n_lt1 = 0;     // window iterations; landmark tiles each query tile needs
    bool tile1_live = false;
    // landmark tiles whose first landmark lies strictly below the window of row i_last
    auto lm_tiles = [&](int i_last) {
        const int top = i_last - a.window - 1;                 // highest key a landmark of this row may have
        return top < 0 ? 0 : (top / a.stride + 1 + kBN - 1) / kBN;
    };
    auto set_item = [&](int t) {
        qb = a.n_qb - 1 - t / a.BH;
        bh = t % a.BH;
        q0 = qb * kBQ;                        // first row of query tile 0; tile 1 starts 128 later
        jt_hi = min((q0 + kBQ - 1) / kBN, jt_max);
        // diagonal tile of each query tile, and the lowest tile its window reaches (one key below the
        // window still feeds the diffusion stencil)
        jt_top0 = min(q0 / kBN, jt_max);
        jt_top1 = min((q0 + kBM) / kBN, jt_max);
        jt_bot0 = (a.window > 0) ? max(0, q0 - a.window - 1) / kBN : 0;
        jt_bot1 = (a.window > 0) ? max(0, q0 + kBM - a.window - 1) / kBN : 0;
        const int jt_lo = kTiles == 2 ? min(jt_bot0, jt_bot1) : jt_bot0;
        n_win = jt_hi - jt_lo + 1;
        tile1_live = kTiles == 2 && (q0 + kBM) < S;   // query tile 1 may lie wholly beyond the sequence
        if (LM) {
            n_lt0 = lm_tiles(min(q0 + kBM, S) - 1);
            n_lt1 = tile1_live ? lm_tiles(min(q0 + kBQ, S) - 1) : 0;
        }
        n_iter = n_win + (LM ? max(n_lt0, n_lt1) : 0);
    };
    // iteration i of an item: i < n_win visits KV tile jt_hi - i, the others landmark tile i - n_win
    auto active = [&](int g, int i) {
        if (LM && i >= n_win) return (i - n_win) < (g == 0 ? n_lt0 : n_lt1);
        const int jt = jt_hi - i;
        return g == 0 ? (jt <= jt_top0 && jt >= jt_bot0) : (tile1_live && jt <= jt_top1 && jt >= jt_bot1);
    };
    // Items are sorted by length, so the CTAs take them in snake order: round r hands items r G ...
    // r G + G - 1 to CTAs 0 ... G - 1 in even rounds and G - 1 ... 0 in odd ones.  For the causal
    // shapes the longest CTA is then within 2 % of the mean (plain round-robin: 14 %).
    auto item_at = [&](int it) {
        const int G = (int)gridDim.x, cta = (int)blockIdx.x;
        return it * G + ((it & 1) ? G - 1 - cta : cta);
    };
    auto load_q = [&](int qsel) {     // the item's Q tiles (and the same tiles one row up) into buffer qsel
        const int nq = (has_lo ? 2 : 1) * (tile1_live ? 2 : 1);
        mbar_expect_tx(bar(B_QLOAD0 + qsel), nq * kTileBytes);
        for (int g = 0; g < (tile1_live ? 2 : 1); ++g) {
            const uint32_t dst = sbase + kOffQ + qsel * kQBufBytes + (2 * g) * kTileBytes;
            tma_load_3d(dst, &mapQ, 0, q0 + g * kBM, bh, bar(B_QLOAD0 + qsel));
            if (has_lo) tma_load_3d(dst + kTileBytes, &mapQ, 0, q0 + g * kBM - 1, bh, bar(B_QLOAD0 + qsel));
        }
    };

    // K or V tile of iteration i into ring stage st: a window tile, or a landmark tile through the strided views
    auto load_k_tile = [&](int i, int st) {
        mbar_expect_tx(bar(B_KFULL0 + st), kTileBytes);
        if (LM && i >= n_win) tma_load_3d(sbase + kOffK + st * kTileBytes, &mapKl, 0, (i - n_win) * kBN, bh, bar(B_KFULL0 + st));
        else tma_load_3d(sbase + kOffK + st * kTileBytes, &mapK, 0, (jt_hi - i) * kBN, bh, bar(B_KFULL0 + st));
    };
    // V[j-1] tiles requested so far.  Two buffers in turn: with one, the loads of a landmark tile could only start when
    // the tile before it had been mixed, and their latency (strided gathers) was the period of a landmark tile.
    int n_vp = 0;
    auto load_v_tile = [&](int i, int st) -> bool {
        if (LM && i >= n_win) {
            const int m0 = (i - n_win) * kBN;
            if (DIFF) {
                const int vb = n_vp & 1;
                if (n_vp >= 2 && !mbar_wait(bar(B_VPEMPTY0 + vb), ((n_vp >> 1) - 1) & 1, abort_flag)) return false;
                ++n_vp;
                mbar_expect_tx(bar(B_VFULL0 + st), 2 * kTileBytes);
                tma_load_3d(sbase + kOffVP + vb * kTileBytes, &mapVp, 0, m0 - 1, bh, bar(B_VFULL0 + st));   // row -1 of the first tile: zeros
            } else {
                mbar_expect_tx(bar(B_VFULL0 + st), kTileBytes);
            }
            tma_load_3d(sbase + kOffV + st * kTileBytes, &mapVl, 0, m0, bh, bar(B_VFULL0 + st));
        } else {
            mbar_expect_tx(bar(B_VFULL0 + st), kTileBytes);
            tma_load_3d(sbase + kOffV + st * kTileBytes, &mapV, 0, (jt_hi - i) * kBN, bh, bar(B_VFULL0 + st));
        }
        return true;
    };

    if (warp == kTmaWarp && lane == 0) {   // the producer sets the barriers up, so that its first loads can go out at once
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(B_QLOAD0 + b), 1);
            mbar_init(bar(B_QFREE0 + b), kTiles);     // one commit per MMA issuer
            for (int g = 0; g < kTiles; ++g) mbar_init(bar(B_QREADY0 + 2 * b + g), kSoftmaxThreads / kTiles);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(B_KFULL0 + s), 1);
            mbar_init(bar(B_KEMPTY0 + s), kTiles);   // one arrival per MMA issuer
            mbar_init(bar(B_VFULL0 + s), 1);
            mbar_init(bar(B_VEMPTY0 + s), kTiles);
            mbar_init(bar(B_VREADY0 + s), kCvtThreads);    // the converter warpgroup
        }
        for (int g = 0; g < kTiles; ++g) {
            mbar_init(bar(B_SFULL0 + g), 1);
            mbar_init(bar(B_SEMPTY0 + g), kBM);
            mbar_init(bar(B_PFULL0 + g), kBM);
            mbar_init(bar(B_PVDONE0 + g), 1);
        }
        mbar_init(bar(B_VPEMPTY0), kCvtThreads);
        mbar_init(bar(B_VPEMPTY1), kCvtThreads);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kTmaWarp) {
        // Q and the first K / V tiles are requested before the rest of the CTA has finished its own
        // set-up (TMEM allocation, the CTA-wide barrier): their latency is the longest of the prologue
        __syncwarp();
        set_item(item_at(0));
        if (lane == 0) {
            load_q(0);
            for (int i = 0; i < min(kStages, n_iter); ++i) load_k_tile(i, i);
        } else if (lane == 1) {
            for (int i = 0; i < min(kStages, n_iter); ++i) load_v_tile(i, i);
        }
    }
    if (warp == kMmaWarp) {   // TMEM allocation is warp-wide; this warp also frees it
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    // columns per query tile: S 128 (from column 0), O 64 (from kColO), FP16 weights 64 (from kColP, two keys per column)

    // Registers move from the helper warpgroup to the two softmax warpgroups (a row of 128 scores lives
    // in registers there).  Each setmaxnreg stands at the head of the branch it governs, so that the
    // register budget of all code below it is unambiguous.
    if (warp >= kTmaWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsHelper));
    if (warp == kTmaWarp) {
        // ================= TMA producer =================
        if (lane == 0) {
            // Q of the item, then its K tiles: a stage is free again as soon as the scores that read it
            // are done.  The first item's Q and first tiles are already on their way.
            int nk = 0;
            bool ok = true;
            for (int it = 0, t = item_at(0); ok && t < a.n_items; ++it, t = item_at(it)) {
                set_item(t);
                if (it > 0) {
                    const int qsel = it & 1;
                    if (it >= 2 && !mbar_wait(bar(B_QFREE0 + qsel), ((it >> 1) - 1) & 1, abort_flag)) break;
                    load_q(qsel);
                }
                for (int i = 0; i < n_iter; ++i, ++nk) {
                    if (it == 0 && i < kStages) continue;
                    const int st = nk % kStages;
                    if (nk >= kStages && !mbar_wait(bar(B_KEMPTY0 + st), ((nk / kStages) - 1) & 1, abort_flag)) { ok = false; break; }
                    load_k_tile(i, st);
                }
            }
        } else if (lane == 1) {
            // V tiles on their own ring: needed later and freed later than K, so they never hold K back
            int nv = 0;
            bool ok = true;
            for (int it = 0, t = item_at(0); ok && t < a.n_items; ++it, t = item_at(it)) {
                set_item(t);
                for (int i = 0; i < n_iter; ++i, ++nv) {
                    if (it == 0 && i < kStages) continue;
                    const int st = nv % kStages;
                    if (nv >= kStages && !mbar_wait(bar(B_VEMPTY0 + st), ((nv / kStages) - 1) & 1, abort_flag)) { ok = false; break; }
                    if (!load_v_tile(i, st)) { ok = false; break; }
                }
            }
        }
    } else if (warp >= kCvtWarp) {
        // ================= V converter =================
        // BF16 V -> FP16 in place (BF16 inputs), 1024 16-byte chunks per tile over 32 lanes; and for a
        // landmark tile under diffusion the mix V[j] + rho V[j-1] of the gathered rows with the rows
        // before them (FP16 out, whatever the input type).
        if (!LM) {
            // without landmarks every tile is treated alike: one flat loop over all the CTA's tiles
            if (!f16) {
                const int ct = tid - kCvtWarp * 32;
                int n_total = 0;
                for (int it = 0, t = item_at(0); t < a.n_items; ++it, t = item_at(it)) {
                    set_item(t);
                    n_total += n_iter;
                }
                for (int nv = 0; nv < n_total; ++nv) {
                    const int st = nv % kStages;
                    if (!mbar_wait(bar(B_VFULL0 + st), (nv / kStages) & 1, abort_flag)) break;
                    unsigned char* vt = smem + kOffV + st * kTileBytes;
#pragma unroll 4
                    for (int q = 0; q < kTileBytes / 16 / kCvtThreads; ++q) {
                        uint4* pch = reinterpret_cast<uint4*>(vt + (ct + kCvtThreads * q) * 16);
                        uint4 v = *pch;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(hi), "f"(lo));
                        }
                        *pch = v;
                    }
                    fence_async_smem();
                    mbar_arrive(bar(B_VREADY0 + st));
                }
            }
        } else if (!f16 || DIFF) {
            const int ct = tid - kCvtWarp * 32;
            const float rho_c = DIFF ? a.nu / (1.0f - a.nu) : 0.0f;
            int nv = 0, n_vpc = 0;       // V tiles, V[j-1] tiles taken so far
            bool ok = true;
            for (int it = 0, t = item_at(0); ok && t < a.n_items; ++it, t = item_at(it)) {
                set_item(t);
                for (int i = 0; ok && i < n_iter; ++i, ++nv) {
                    const int st = nv % kStages;
                    if (!mbar_wait(bar(B_VFULL0 + st), (nv / kStages) & 1, abort_flag)) { ok = false; break; }
                    unsigned char* vt = smem + kOffV + st * kTileBytes;
                    if (LM && DIFF && i >= n_win) {
                        const int vb = n_vpc & 1;
                        const unsigned char* vp = smem + kOffVP + vb * kTileBytes;
                        const bool first_tile = i == n_win;          // its row 0 is key 0: V_s[0] = V[0]
#pragma unroll 2
                        for (int q = 0; q < kTileBytes / 16 / kCvtThreads; ++q) {
                            const int ch = ct + kCvtThreads * q;      // chunks 0..7 are row 0
                            uint4 v = *reinterpret_cast<uint4*>(vt + ch * 16);
                            uint4 pv = (first_tile && ch < 8) ? v : *reinterpret_cast<const uint4*>(vp + ch * 16);
                            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
                            const uint32_t* pw = reinterpret_cast<const uint32_t*>(&pv);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float2 x, y;
                                if (f16) {
                                    x = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                                    y = __half22float2(*reinterpret_cast<const __half2*>(&pw[e]));
                                } else {
                                    x = make_float2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xffff0000u));
                                    y = make_float2(__uint_as_float(pw[e] << 16), __uint_as_float(pw[e] & 0xffff0000u));
                                }
                                const float lo = fmaf(rho_c, y.x, x.x), hi = fmaf(rho_c, y.y, x.y);
                                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(hi), "f"(lo));
                            }
                            *reinterpret_cast<uint4*>(vt + ch * 16) = v;
                        }
                        mbar_arrive(bar(B_VPEMPTY0 + vb));
                        ++n_vpc;
                    } else if (!f16) {
#pragma unroll 4
                        for (int q = 0; q < kTileBytes / 16 / kCvtThreads; ++q) {
                            uint4* pch = reinterpret_cast<uint4*>(vt + (ct + kCvtThreads * q) * 16);
                            uint4 v = *pch;
                            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float lo = __uint_as_float(w[e] << 16), hi = __uint_as_float(w[e] & 0xffff0000u);
                                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(hi), "f"(lo));
                            }
                            *pch = v;
                        }
                    }
                    fence_async_smem();
                    mbar_arrive(bar(B_VREADY0 + st));
                }
            }
        }
    } else if (warp >= kMmaWarp) {
        // ================= MMA issuers: one warp per query tile =================
        // The whole warp runs the loop and the waits, one elected lane issues the MMAs and commits:
        // with warp-uniform control flow the descriptors stay in uniform registers, which halves the
        // cost of issuing an MMA compared with a single divergent thread.  Everything that can be
        // known in advance is computed before the loop: descriptors are a constant high word plus a
        // 14-bit address field, and the loop only adds to the low word.
        {
            uint32_t elected;
            asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(elected));
            const bool leader = elected != 0;
            auto wait_w = [&](uint32_t b, uint32_t parity) {   // warp-uniform verdict
                return __all_sync(0xffffffffu, mbar_wait(b, parity, abort_flag)) != 0;
            };
            const int g = warp - kMmaWarp;
            const int fmt = f16 ? 0 : 1;
            const uint32_t idesc_qk = instr_desc(fmt, fmt, 0, kBN);
            const uint32_t idesc_pv = instr_desc(0, 0, 1 /* V is MN-major */, kD);   // FP16 weights x FP16 V
            const uint32_t desc_hi = (uint32_t)(smem_desc(0) >> 32);
            auto lo_of = [](uint32_t addr) { return ((addr >> 4) & 0x3FFFu) | (1u << 16); };
            auto desc = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | lo; };
            const uint32_t a_p = tmem + kColP + (uint32_t)g * 64u;
            const uint32_t k_lo0 = lo_of(sbase + kOffK), v_lo0 = lo_of(sbase + kOffV);
            const uint32_t d_s = tmem + (uint32_t)g * 128u, d_o = tmem + kColO + (uint32_t)g * 64u;
            const int v_bar = (f16 && !(LM && DIFF)) ? B_VFULL0 : B_VREADY0;   // tiles the converter has (not) to touch
            // running counters: K / V tiles taken from the rings, score tiles and products issued
            int nt_qk = 0, nt_pv = 0, s_qk = 0, s_pv = 0;
            int k_item = 0;      // products of this tile issued so far in the item (the first one overwrites O)
            int it_first = 0, it_last = -1;   // without landmarks a tile's iterations are one range
            auto mine = [&](int i) { return LM ? active(g, i) : (i >= it_first && i <= it_last); };
            uint32_t qhi_lo = 0, qlo_lo = 0;

            auto issue_qk = [&](int i) {   // S_g = Q_adv,g K(i)^T, then this issuer's release of the K stage
                const int st = nt_qk % kStages;
                if (!wait_w(bar(B_KFULL0 + st), (nt_qk / kStages) & 1)) return false;
                if (mine(i)) {
                    // the previous scores of this tile (of this item or the one before) must have left TMEM
                    if (s_qk > 0 && !wait_w(bar(B_SEMPTY0 + g), (s_qk - 1) & 1)) return false;
                    tc_fence_after();
                    const uint32_t kl = k_lo0 + (uint32_t)st * (kTileBytes >> 4);
                    if (leader) {
#pragma unroll
                        for (int kk = 0; kk < kD / 16; ++kk) {
                            tc_mma_f16(d_s, desc(qhi_lo + 2 * kk), desc(kl + 2 * kk), idesc_qk, kk > 0 ? 1u : 0u);
                            if (has_lo) tc_mma_f16(d_s, desc(qlo_lo + 2 * kk), desc(kl + 2 * kk), idesc_qk, 1u);
                        }
                        tc_commit(bar(B_SFULL0 + g));
                    }
                    ++s_qk;
                }
                if (leader) tc_commit(bar(B_KEMPTY0 + st));   // both issuers arrive, each after its own reads of K(i)
                ++nt_qk;
                __syncwarp();
                return true;
            };
            auto issue_pv = [&](int i) {   // O_g (+)= W_g(i) V(i), then this issuer's release of the V stage
                const int st = nt_pv % kStages, k = k_item;
                if (mine(i)) {
                    ++k_item;
                    if (!wait_w(bar(B_PFULL0 + g), s_pv & 1)) return false;
                    if (!wait_w(bar(v_bar + st), (nt_pv / kStages) & 1)) return false;
                    tc_fence_after();
                    const uint32_t vl = v_lo0 + (uint32_t)st * (kTileBytes >> 4);
                    if (leader) {
#pragma unroll
                        for (int kk = 0; kk < kBN / 16; ++kk) {
                            // weights: from tensor memory, 8 columns per k-step of 16 keys;
                            // V tile: key-major rows of 128 bytes, 16 keys per k-step = 2048 bytes
                            tc_mma_f16_ta(d_o, a_p + 8u * (uint32_t)kk, desc(vl + kk * (2048 >> 4)), idesc_pv,
                                          (k > 0 || kk > 0) ? 1u : 0u);
                        }
                        tc_commit(bar(B_PVDONE0 + g));
                    }
                    ++s_pv;
                } else if (!wait_w(bar(v_bar + st), (nt_pv / kStages) & 1)) {
                    return false;   // an idle issuer still paces itself on the tile it releases
                }
                if (leader) tc_commit(bar(B_VEMPTY0 + st));
                ++nt_pv;
                __syncwarp();
                return true;
            };
            bool ok = true;
            for (int it = 0, t = item_at(0); ok && t < a.n_items; ++it, t = item_at(it)) {
                set_item(t);
                const int qsel = it & 1;
                k_item = 0;
                if (!LM) {
                    it_first = jt_hi - (g == 0 ? jt_top0 : jt_top1);
                    it_last = (g == 0 || tile1_live) ? jt_hi - (g == 0 ? jt_bot0 : jt_bot1) : -1;
                }
                qhi_lo = lo_of(sbase + kOffQ + qsel * kQBufBytes + (2 * g) * kTileBytes);
                qlo_lo = lo_of(sbase + kOffQ + qsel * kQBufBytes + (2 * g + 1) * kTileBytes);
                ok = wait_w(bar(B_QREADY0 + 2 * qsel + g), (it >> 1) & 1);   // this tile's Q_adv is in place
                if (ok) ok = issue_qk(0);
                for (int i = 0; ok && i < n_iter; ++i) {
                    // scores of the next tile first: they only need the previous scores to have left TMEM
                    if (i + 1 < n_iter) ok = issue_qk(i + 1);
                    if (ok) ok = issue_pv(i);
                }
                if (ok && leader) tc_commit(bar(B_QFREE0 + qsel));   // this item's reads of Q are all issued
                __syncwarp();
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ================= softmax warpgroups: one thread per query row =================
        // warp w: query tile g = w / 4, TMEM lane quarter = w % 4 (the lanes a warp may touch).
        const int g = warp >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;         // row in tile = TMEM lane
        const uint32_t lane_addr = ((uint32_t)(quarter * 32)) << 16;
        const uint32_t tmem_S = tmem + (uint32_t)g * 128u + lane_addr;
        const uint32_t tmem_O = tmem + kColO + (uint32_t)g * 64u + lane_addr;
        const uint32_t tmem_P = tmem + kColP + (uint32_t)g * 64u + lane_addr;
        int s_run = 0;               // score tiles of this query tile taken so far, over all items
        bool ok = true;
        const float c = a.c;
        const float rho = DIFF ? a.nu / (1.0f - a.nu) : 0.0f;   // nu <= 1/2 on this path

        // The set-up of an item's Q (wait for its tiles, form Q_adv in place, tell the issuer) is done for
        // the first item here and for every later item before the epilogue of the item before it, so that
        // the next item's first scores are being computed while this item's output is written.
        // Expects set_item() of that item to be in force.
        auto prep_q = [&](int it_of) -> bool {
            const int qsel = it_of & 1;
            const int i_glob = q0 + g * kBM + r;
            const bool fine = mbar_wait(bar(B_QLOAD0 + qsel), (it_of >> 1) & 1, abort_flag);
            // Q_adv = Q + eta (Q - Q_prev) as an exact hi + lo pair, in place (the row's 8 chunks)
            if (fine && has_lo && (g == 0 || tile1_live)) {
                unsigned char* qh = smem + kOffQ + qsel * kQBufBytes + (2 * g) * kTileBytes + r * 128;
                unsigned char* ql = qh + kTileBytes;
#pragma unroll 2
                for (int cidx = 0; cidx < 8; ++cidx) {
                    const int pc = (cidx ^ (r & 7)) * 16;
                    uint4 cur = *reinterpret_cast<uint4*>(qh + pc);
                    uint4 prv = *reinterpret_cast<uint4*>(ql + pc);
                    uint32_t* cw = reinterpret_cast<uint32_t*>(&cur);
                    uint32_t* pw = reinterpret_cast<uint32_t*>(&prv);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t wq = cw[e], wp = (i_glob > 0) ? pw[e] : cw[e];   // row 0 has no predecessor
                        float2 q, pq;
                        if (f16) {
                            q = __half22float2(*reinterpret_cast<const __half2*>(&wq));
                            pq = __half22float2(*reinterpret_cast<const __half2*>(&wp));
                        } else {
                            q = make_float2(__uint_as_float(wq << 16), __uint_as_float(wq & 0xffff0000u));
                            pq = make_float2(__uint_as_float(wp << 16), __uint_as_float(wp & 0xffff0000u));
                        }
                        const float a_a = fmaf(a.eta, q.x - pq.x, q.x), a_b = fmaf(a.eta, q.y - pq.y, q.y);
                        uint32_t hi, lo;
                        if (f16) {
                            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(a_b), "f"(a_a));
                            const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
                            asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(a_b - hf.y), "f"(a_a - hf.x));
                        } else {
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "f"(a_b), "f"(a_a));
                            const float h_a = __uint_as_float(hi << 16), h_b = __uint_as_float(hi & 0xffff0000u);
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "f"(a_b - h_b), "f"(a_a - h_a));
                        }
                        cw[e] = hi;
                        pw[e] = lo;
                    }
                    *reinterpret_cast<uint4*>(qh + pc) = cur;
                    *reinterpret_cast<uint4*>(ql + pc) = prv;
                }
                fence_async_smem();
            }
            mbar_arrive(bar(B_QREADY0 + 2 * qsel + g));
            return fine;
        };
        set_item(item_at(0));
        if (item_at(0) < a.n_items) ok = prep_q(0);

        for (int it = 0, t = item_at(0); ok && t < a.n_items; ++it, t = item_at(it)) {
        set_item(t);
        const int i_glob = q0 + g * kBM + r;

        float m_run = -INFINITY;     // running reference maximum (log2 domain)
        float l_run = 0.0f;          // running sum of the row's weights
        float s_carry = -INFINITY;   // scaled score of the first key of the tile above (for the stencil)
        int k_last = -1, k_cnt = 0;  // index of the last / number of the iterations this tile has taken part in

        for (int i = 0; ok && i < n_iter; ++i) {
            if (!active(g, i)) continue;
            const bool lm = LM && i >= n_win;                 // a landmark tile: keys (i - n_win) * 128 ... times stride
            const int k = k_cnt++, jt = jt_hi - i, k0 = lm ? (i - n_win) * kBN : jt * kBN;   // first key / landmark of the tile
            k_last = k;
            if (!mbar_wait(bar(B_SFULL0 + g), s_run & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            // the whole row of scores into registers, then the S columns go back to the issuer at once:
            // the next tile's QK^T runs while this tile's weights are computed
            float s[kBN];
            tc_ld32(tmem_S, s);
            tc_ld32(tmem_S + 32, s + 32);
            tc_ld32(tmem_S + 64, s + 64);
            tc_ld32(tmem_S + 96, s + 96);
            tc_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(B_SEMPTY0 + g));

            const int r_first = q0 + g * kBM;
            const bool edge = lm || (k0 + kBN - 1 > r_first) || (k0 + kBN > S) ||
                              (a.window > 0 && k0 < r_first + kBM - 1 - a.window);
            // Chunks of 16 columns that no row of this warp sees (bit cb of `dead`) take no part in the maximum and get
            // no exponentials -- under a window a row sees 65 of the 384 columns its item visits -- and only the chunks
            // that some row sees in part are masked element by element.  The visible columns of a row are one range
            // and both of its ends grow with the row, so the warp's first and last lane decide for the warp.
            uint32_t dead = 0;
            if (edge) {
                // visible columns of the row, relative to the tile's first key: [lo_rel, hi_rel]; in a landmark
                // tile column c is key (k0 + c) * stride, visible when it lies strictly below the row's window
                int hi_rel = min(i_glob, S - 1) - k0;
                int lo_rel = (a.window > 0) ? i_glob - a.window - k0 : -(1 << 30);
                if (lm) {
                    const int top = i_glob - a.window - 1;
                    hi_rel = (top < 0 ? -1 : top / a.stride) - k0;
                    lo_rel = -(1 << 30);
                }
                if (WIN) {
                    const int hi_min = __shfl_sync(0xffffffffu, hi_rel, 0), hi_max = __shfl_sync(0xffffffffu, hi_rel, 31);
                    const int lo_min = __shfl_sync(0xffffffffu, lo_rel, 0), lo_max = __shfl_sync(0xffffffffu, lo_rel, 31);
#pragma unroll
                    for (int cb = 0; cb < kBN / 16; ++cb) {
                        const int c_lo = 16 * cb, c_hi = 16 * cb + 15;
                        if (c_lo > hi_max || c_hi < lo_min) {
                            dead |= 1u << cb;
                        } else if (c_hi > hi_min || c_lo < lo_max) {
#pragma unroll
                            for (int j = c_lo; j <= c_hi; ++j) s[j] = (j <= hi_rel && j >= lo_rel) ? s[j] : -INFINITY;
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < kBN; ++j) s[j] = (j <= hi_rel && j >= lo_rel) ? s[j] : -INFINITY;
                }
            }
            float mxr;
            {
                float mc[8];                            // three-input maxima, eight independent chains
                if (WIN) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) mc[q] = -INFINITY;
#pragma unroll
                    for (int j = 0; j < kBN; j += 16) {
                        if (dead & (1u << (j >> 4))) continue;
#pragma unroll
                        for (int q = 0; q < 8; ++q) mc[q] = fmaxf(fmaxf(mc[q], s[j + 2 * q]), s[j + 2 * q + 1]);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q) mc[q] = fmaxf(s[2 * q], s[2 * q + 1]);
#pragma unroll
                    for (int j = 16; j < kBN; j += 16)
#pragma unroll
                        for (int q = 0; q < 8; ++q) mc[q] = fmaxf(fmaxf(mc[q], s[j + 2 * q]), s[j + 2 * q + 1]);
                }
                mxr = fmaxf(fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3])), fmaxf(fmaxf(mc[4], mc[5]), fmaxf(mc[6], mc[7])));
            }
            const float mx = mxr * c;                 // c > 0
            const float s_first = (WIN && (dead & 1u)) ? -INFINITY : s[0] * c;   // the tile below needs it for its last column's stencil
            // move the reference maximum only when it would grow by more than the threshold (weights
            // stay below 2^9, well inside FP16); the decision is warp-wide because the O correction is
            // a warp-collective TMEM access
            const bool want = (mx > m_run + kRescaleThreshold) || (m_run == -INFINITY && mx > -INFINITY);
            const bool any = __any_sync(0xffffffffu, want && k > 0 && m_run > -INFINITY);
            float m_new = want ? mx : m_run;
            if (any && m_new < mx) m_new = mx;       // correcting anyway: take the exact maximum
            bool pv_done = (k == 0);                 // has the previous O += W V of this tile been waited for?
            if (any) {
                if (!mbar_wait(bar(B_PVDONE0 + g), (s_run - 1) & 1, abort_flag)) { ok = false; break; }
                pv_done = true;
                tc_fence_after();
                const float f = (m_run == -INFINITY) ? 0.0f : ex2(m_run - m_new);
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    float o[32];
                    tc_ld32(tmem_O + 32 * hc, o);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] *= f;
                    tc_st32(tmem_O + 32 * hc, o);
                }
                tc_wait_st();
                tc_fence_before();
                l_run *= f;
            }
            m_run = m_new;
            const float neg_m = (m_run == -INFINITY) ? 0.0f : -m_run;   // all scores are -inf in that case

            // FP16 weights with the diffusion stencil folded in, written to tensor memory as the A
            // operand of O += W V.  The weights carry a common factor 1 / (1 - nu), which the
            // normalisation by their own sum removes: w'_r = p_r + rho p_{r+1}, rho = nu / (1 - nu).
            // Arithmetic runs on packed pairs (key k, key k + 8) of a 16-key chunk so that the
            // neighbour pair of the stencil is again a register pair.  The row sum is taken before
            // the FP16 rounding: the two differ by at most 2^-12 relative, far inside the tolerance.
            const bool stencil = DIFF && !lm;                           // landmarks: the mix sits in their V tile instead
            float nxt = stencil ? ex2(s_carry + neg_m) : 0.0f;          // -inf gives 0
            if (!lm) s_carry = s_first;
            const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_m, neg_m), rho2 = make_float2(rho, rho);
            float2 lsum2 = make_float2(0.0f, 0.0f), lsum2b = make_float2(0.0f, 0.0f);
            // chunks of 16 keys, highest first (the stencil walks downwards); the exponentials of the
            // next chunk are issued before the current chunk's stencil, sum, pack and store, so that the
            // exponential unit and the arithmetic pipes of this warp work at the same time
            // (the tiles with dead chunks run a second copy of this code that tests for them: the tests would cost
            // the straight-line copy its overlap of exponentials and arithmetic)
            auto expo16 = [&](auto skip, int cb, float2 (&P)[9]) {     // p = 2^(c s - m) as pairs (key j, key j + 8)
                if (decltype(skip)::value && (dead & (1u << cb))) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) P[e] = make_float2(0.0f, 0.0f);
                    return;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float2 tt = __ffma2_rn(make_float2(s[16 * cb + 2 * e], s[16 * cb + 2 * e + 1]), c2, nm2);
                    const float p0 = ex2(tt.x), p1 = ex2(tt.y);          // keys 2e, 2e+1 of the chunk
                    if (2 * e < 8) { P[2 * e].x = p0; P[2 * e + 1].x = p1; }
                    else { P[2 * e - 8].y = p0; P[2 * e - 7].y = p1; }
                }
            };
            auto store16 = [&](int cb, float2 (&P)[9]) {
                float2 W[8];
                if (DIFF && (!LM || stencil)) {
                    P[8] = make_float2(P[0].y, nxt);                   // keys 8 and 16 (= first key of the chunk above)
                    nxt = P[0].x;
#pragma unroll
                    for (int q = 0; q < 8; ++q) W[q] = __ffma2_rn(rho2, P[q + 1], P[q]);
                    if (cb == 0 && k0 == 0) W[0].x = fmaf(rho, P[0].x, W[0].x);   // V_s[0] = V[0]
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q) W[q] = P[q];
                }
#pragma unroll
                for (int q = 0; q < 8; q += 2) {
                    lsum2 = __fadd2_rn(lsum2, W[q]);
                    lsum2b = __fadd2_rn(lsum2b, W[q + 1]);
                }
                uint32_t pk[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {                          // word e: keys 2e, 2e+1; word 4+e: keys 8+2e, 9+2e
                    __half2 h_lo = __floats2half2_rn(W[2 * e].x, W[2 * e + 1].x);
                    __half2 h_hi = __floats2half2_rn(W[2 * e].y, W[2 * e + 1].y);
                    pk[e] = *reinterpret_cast<uint32_t*>(&h_lo);
                    pk[4 + e] = *reinterpret_cast<uint32_t*>(&h_hi);
                }
                tc_st8(tmem_P + 8 * cb, pk);
            };
            auto all_chunks = [&](auto skip) {
                float2 Pa[9], Pb[9];
                expo16(skip, 7, Pa);
                expo16(skip, 6, Pb);
                if (!pv_done) {
                    // the weight columns are still being read by the previous O += W V until it is done
                    if (!mbar_wait(bar(B_PVDONE0 + g), (s_run - 1) & 1, abort_flag)) ok = false;
                    tc_fence_after();
                }
                store16(7, Pa);
                expo16(skip, 5, Pa);
                store16(6, Pb);
                expo16(skip, 4, Pb);
                store16(5, Pa);
                expo16(skip, 3, Pa);
                store16(4, Pb);
                expo16(skip, 2, Pb);
                store16(3, Pa);
                expo16(skip, 1, Pa);
                store16(2, Pb);
                expo16(skip, 0, Pb);
                store16(1, Pa);
                store16(0, Pb);
            };
            // one copy per instantiation: the loop lives on the instruction cache, and under a window nearly every
            // tile has dead chunks
            all_chunks(SkipDead<WIN>{});
            if (!ok) break;
            lsum2 = __fadd2_rn(lsum2, lsum2b);
            // a landmark's weight stands for V[j] + rho V[j-1]: it counts (1 + rho) times in the row sum
            l_run += (lsum2.x + lsum2.y) * ((LM && DIFF && lm) ? 1.0f + rho : 1.0f);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(B_PFULL0 + g));
            ++s_run;
        }

        // ---- the next item's Q, then this item's epilogue: O / l, the row's 64 channels ----
        {
            const int t_next = item_at(it + 1);
            if (ok && t_next < a.n_items) {
                set_item(t_next);
                ok = prep_q(it + 1);
                set_item(t);
            }
        }
        if (ok && k_last >= 0) {
            if (mbar_wait(bar(B_PVDONE0 + g), (s_run - 1) & 1, abort_flag)) {
                tc_fence_after();
                const float inv = (l_run > 1e-9f) ? 1.0f / l_run : 0.0f;   // cuda/VedicGEMM.cu:1049
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    float o[32];
                    tc_ld32(tmem_O + 32 * hc, o);
                    tc_wait_ld();
                    if (i_glob < S) {
                        const size_t row = (size_t)bh * a.o_slab + (size_t)i_glob * a.o_row + hc * 32;
                        // 32 bytes per store when the output allows it: a full sector per thread and instruction
                        if (a.out_is_f32) {
                            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<float*>(a.O) + row);
                            uint4 w4[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 f = make_float4(o[4 * j] * inv, o[4 * j + 1] * inv, o[4 * j + 2] * inv, o[4 * j + 3] * inv);
                                w4[j] = *reinterpret_cast<const uint4*>(&f);
                            }
#pragma unroll
                            for (int j = 0; j < 8; j += 2) {
                                if (a.o_al32) st_32B(dst + j, w4[j], w4[j + 1]);
                                else { dst[j] = w4[j]; dst[j + 1] = w4[j + 1]; }
                            }
                        } else {
                            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.O) + row);
                            uint4 w4[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint32_t w[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    w[e] = f32x2_to_16(o[8 * j + 2 * e] * inv, o[8 * j + 2 * e + 1] * inv, f16);
                                w4[j] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
#pragma unroll
                            for (int j = 0; j < 4; j += 2) {
                                if (a.o_al32) st_32B(dst + j, w4[j], w4[j + 1]);
                                else { dst[j] = w4[j]; dst[j + 1] = w4[j + 1]; }
                            }
                        }
                    }
                }
                tc_fence_before();
            } else {
                ok = false;
            }
        }
        }   // next work item
    }

    // ---- teardown: every role comes here, aborted or not ----
    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) {   // low half: the barrier's offset from the first one (mod 64 KiB); the rest stays as recorded
        const int f = *abort_flag;
        atomicExch(a.status, (f & ~0xffff) | ((f - (int)(bar0 & 0xffffu)) & 0xffff));
    }
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// -------------------------------------------------------------------------------------
// Bring-up check of the building blocks above on one 128-row tile, one CTA, 128 threads.
//   mode 0: D[128 x 128] = A[128 x 64] B[128 x 64]^T   A, B by TMA, both K-major (the S = Q K^T shape)
//   mode 1: D[128 x 64]  = A[128 x 128] B[128 x 64]    A written by the threads into the swizzled
//           K-major layout, B by TMA and used MN-major (the O = W V shape)
//   mode 2: no load is issued: every thread's bounded wait runs out, the kernel returns and the
//           status word is raised (a check of the time-out path that cannot hang)
//   mode 3: as mode 1, but A is written by the threads into tensor memory (lane = row, two K
//           elements per column) and read from there by the MMA (how the prefill kernel passes W)
//   mode 16 + m (m = 0, 1, 3): the MMAs of mode m issued kSelftestReps times back to back into the same
//           accumulator; D[0] receives the clock cycles from the first issue to the completion of the last (what
//           one MMA of that shape costs a CTA that does nothing else); the rest of D is not meaningful
//   mode 48 + m: the same with the whole first warp running the issue loop and one elected lane issuing (the form the
//           kernels' issuing warps take) instead of a single thread in a divergent branch
constexpr int kSelftestReps = 32;
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     const unsigned short* __restrict__ a_rows, float* __restrict__ D, int mode, int fmt,
                     int* status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    constexpr int offA = 0, offB = 2 * kTileBytes, offBar = 3 * kTileBytes;
    const uint32_t bar_load = sbase + offBar, bar_mma = sbase + offBar + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + offBar + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + offBar + 32);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int reps = mode >= 16 ? kSelftestReps : 1;
    const bool uniform_issue = (mode & 32) != 0;     // the whole first warp runs the issue loop, one elected lane issues
    mode &= 15;

    if (tid == 0) {
        mbar_init(bar_load, 1);
        mbar_init(bar_mma, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(128u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (tid == 0 && mode != 2) {   // mode 2: nothing is loaded, so the wait below must run out
        mbar_expect_tx(bar_load, mode == 0 ? 2 * kTileBytes : kTileBytes);
        if (mode == 0) tma_load_3d(sbase + offA, &mapA, 0, 0, 0, bar_load);
        tma_load_3d(sbase + offB, &mapB, 0, 0, 0, bar_load);
    }
    if (mode == 1) {   // row tid of A: 128 values = 16 chunks of 16 bytes, two 64-column atoms
        const uint4* src = reinterpret_cast<const uint4*>(a_rows + (size_t)tid * 128);
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
            const int atom = ch >> 3, cc = ch & 7;
            *reinterpret_cast<uint4*>(smem + offA + atom * kTileBytes + tid * 128 + ((cc ^ (tid & 7)) * 16)) = src[ch];
        }
        fence_async_smem();
    }
    if (mode == 3) {   // row tid of A -> tensor-memory columns [64,128) of lane tid
        const uint32_t* src = reinterpret_cast<const uint32_t*>(a_rows + (size_t)tid * 128);
        float w[32];
        for (int c0 = 0; c0 < 64; c0 += 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j) w[j] = __uint_as_float(src[c0 + j]);
            tc_st32(tmem + (((uint32_t)(warp * 32)) << 16) + 64u + (uint32_t)c0, w);
        }
        tc_wait_st();
        tc_fence_before();
    }
    bool ok = mbar_wait(bar_load, 0, abort_flag, mode == 2 ? (1u << 14) : kSpinLimit);
    __syncthreads();
    long long t_begin = 0;
    uint32_t elected = 0;
    if (warp == 0) asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(elected));
    const bool issuer = uniform_issue ? elected != 0 : tid == 0;
    if ((uniform_issue ? warp == 0 : tid == 0) && ok) {
        tc_fence_after();
        t_begin = clock64();
        for (int rp = 0; rp < reps; ++rp) {
            if (!issuer) continue;
            if (mode == 3) {
                const uint32_t idesc = instr_desc(fmt, fmt, 1, 64);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc_mma_f16_ta(tmem, tmem + 64u + 8u * (uint32_t)k, smem_desc(sbase + offB + k * 2048), idesc,
                                  (k > 0 || rp > 0) ? 1u : 0u);
            } else if (mode == 0) {
                const uint32_t idesc = instr_desc(fmt, fmt, 0, 128);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma_f16(tmem, smem_desc(sbase + offA + k * 32), smem_desc(sbase + offB + k * 32), idesc,
                               (k > 0 || rp > 0) ? 1u : 0u);
            } else {
                const uint32_t idesc = instr_desc(fmt, fmt, 1, 64);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc_mma_f16(tmem, smem_desc(sbase + offA + (k >> 2) * kTileBytes + (k & 3) * 32),
                               smem_desc(sbase + offB + k * 2048), idesc, (k > 0 || rp > 0) ? 1u : 0u);
            }
        }
        if (issuer) tc_commit(bar_mma);
    }
    ok = ok && mbar_wait(bar_mma, 0, abort_flag);
    const long long t_end = clock64();
    if (ok) {
        tc_fence_after();
        const uint32_t lane_addr = ((uint32_t)(warp * 32)) << 16;
        const int ncol = mode == 0 ? 128 : 64;
        float v[32];
        for (int c0 = 0; c0 < ncol; c0 += 32) {
            tc_ld32(tmem + lane_addr + c0, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) D[(size_t)tid * ncol + c0 + j] = v[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (reps > 1 && ok && issuer) D[0] = (float)(t_end - t_begin);
    if (*abort_flag && tid == 0) atomicExch(status, 1);
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------
// [BH][S][64] 16-bit tensor, box = 128 rows x 64 channels of one head, 128-byte swizzle
// `rows` rows per head taken every `pitch` rows from `base` (pitch 1: the plain tensor; pitch = the landmark
// stride: the strided view whose row m is key m * stride of the head)
// row_elems / slab_elems: elements between two rows of a head and between two (sequence, head) slabs (0: contiguous)
bool make_map(CUtensorMap* m, const void* base, int BH, int S, bool f16, int rows = -1, int pitch = 1,
              int64_t row_elems = 0, int64_t slab_elems = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    if (row_elems == 0) row_elems = kD;
    if (slab_elems == 0) slab_elems = (int64_t)S * kD;
    cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)(rows < 0 ? S : rows), (cuuint64_t)BH};
    cuuint64_t strides[2] = {(cuuint64_t)row_elems * 2 * pitch, (cuuint64_t)slab_elems * 2};
    cuuint32_t box[3] = {(cuuint32_t)kD, (cuuint32_t)kBM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int umma_selftest(logos_ctx* ctx, int mode, int dtype, const void* A, const void* B, float* D) {
    const int base_mode = mode & 15;
    if (!A || !B || !D || mode < 0 || mode > 51 || (mode & 32 && !(mode & 16)) || base_mode > 3 || (mode >= 16 && base_mode == 2) ||
        (dtype != LOGOS_BF16 && dtype != LOGOS_F16))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "selftest: bad argument");
    const bool f16 = dtype == LOGOS_F16;
    CUtensorMap ma, mb;
    // modes 1 and 3 do not load A by TMA; its map then simply aliases B's
    if (!make_map(&ma, base_mode == 0 ? A : B, 1, kBM, f16) || !make_map(&mb, B, 1, kBM, f16))
        return fail(ctx, LOGOS_ERR_CUDA, "selftest: cuTensorMapEncodeTiled failed");
    const int smem = 3 * kTileBytes + 64 + 1024;
    if (int rc = ensure_smem_limit(ctx, umma_selftest_kernel, smem)) return rc;
    umma_selftest_kernel<<<1, 128, smem, ctx->stream>>>(ma, mb, (const unsigned short*)A, D, mode, f16 ? 0 : 1,
                                                        ctx->tc_status);
    LOGOS_LAUNCH_CHECK(ctx, "umma_selftest_kernel");
    return LOGOS_OK;
}

bool attention_tc_eligible(int in_dtype, int out_dtype, int DH, const logos_attn_params* p, int S) {
    if (DH != kD) return false;
    if (in_dtype != LOGOS_BF16 && in_dtype != LOGOS_F16) return false;
    if (out_dtype != in_dtype && out_dtype != LOGOS_F32) return false;
    if (!p->causal || !(p->scale > 0.0f)) return false;
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    if (ns_any && p->ns_alpha < 1.0f) return false;                 // blend: two attention passes
    if (ns_any && p->diffuse_mode == LOGOS_DIFFUSE_CENTRAL) return false;
    // the diffusion weights are carried with a factor 1 / (1 - nu): keep them inside FP16
    if (ns_any && (p->ns_nu < 0.0f || p->ns_nu > 0.5f)) return false;
    return true;
}

// in / out: element strides of Q, K, V and of O (NULL: contiguous [B][H][S][64]).  One launch covers every
// (sequence, head) when the slabs are evenly spaced (batch stride = H x head stride); otherwise one launch per sequence.
int attention_tc(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K, const void* V,
                 void* O, int B, int H, int S, int DH, const logos_attn_params* p, const logos_strides* in,
                 const logos_strides* out) {
    logos_strides si{(int64_t)H * S * kD, (int64_t)S * kD, kD}, so = si;
    if (in) si = *in;
    if (out) so = *out;
    const int esz_o = out_dtype == LOGOS_F32 ? 4 : 2;
    if (si.row < kD || (si.row % 8) || (si.head % 8) || (si.batch % 8) || so.row < kD || (so.row * esz_o) % 16 ||
        (so.head * esz_o) % 16 || (so.batch * esz_o) % 16)
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "attention: strides must keep every row 16-byte aligned");
    if (B > 1 && (si.batch != (int64_t)H * si.head || so.batch != (int64_t)H * so.head)) {
        for (int b = 0; b < B; ++b) {     // slabs not evenly spaced over (sequence, head): one sequence at a time
            logos_strides s1 = si, s2 = so;
            s1.batch = (int64_t)H * si.head; s2.batch = (int64_t)H * so.head;
            const size_t ib = (size_t)b * si.batch * 2, ob = (size_t)b * so.batch * esz_o;
            int rc = attention_tc(ctx, in_dtype, out_dtype, (const char*)Q + ib, (const char*)K + ib, (const char*)V + ib,
                                  (char*)O + ob, 1, H, S, DH, p, &s1, &s2);
            if (rc != LOGOS_OK) return rc;
        }
        return LOGOS_OK;
    }
    (void)DH;
    const int BH = B * H;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "attention: tensors must be 16-byte aligned");
    if (!ctx->tc_status) return fail(ctx, LOGOS_ERR_WORKSPACE, "attention: status word missing");
    const bool f16 = in_dtype == LOGOS_F16;
    CUtensorMap mq, mk, mv, mkl, mvl, mvp;
    if (!make_map(&mq, Q, BH, S, f16, -1, 1, si.row, si.head) || !make_map(&mk, K, BH, S, f16, -1, 1, si.row, si.head) ||
        !make_map(&mv, V, BH, S, f16, -1, 1, si.row, si.head))
        return fail(ctx, LOGOS_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed");
    // Shunyam landmarks: strided views of K and V (row m = key m * stride) and of V one row earlier
    // (row m = key (m + 1) * stride - 1, read at m - 1); each view ends inside its head's rows
    const int lm_stride = (shunyam_active(p->window, S) && p->stride > 0) ? p->stride : 0;
    mkl = mk; mvl = mv; mvp = mv;
    if (lm_stride) {
        const int n_lm = (S + lm_stride - 1) / lm_stride, n_prev = S / lm_stride;
        const unsigned char* v_prev = reinterpret_cast<const unsigned char*>(V) + (size_t)(lm_stride - 1) * si.row * 2;
        if (!make_map(&mkl, K, BH, S, f16, n_lm, lm_stride, si.row, si.head) ||
            !make_map(&mvl, V, BH, S, f16, n_lm, lm_stride, si.row, si.head) ||
            !make_map(&mvp, n_prev > 0 ? v_prev : V, BH, S, f16, n_prev > 0 ? n_prev : 1, lm_stride, si.row, si.head))
            return fail(ctx, LOGOS_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed for the landmark views");
    }
    const bool ns_any = p->ns_alpha > 0.0f && (p->ns_eta != 0.0f || p->diffuse_mode != LOGOS_DIFFUSE_NONE);
    TcArgs a;
    a.O = O; a.S = S;
    a.o_row = so.row; a.o_slab = so.head;
    a.out_is_f32 = out_dtype == LOGOS_F32;
    a.o_al32 = aligned32(O) ? 1 : 0;
    a.in_is_f16 = f16;
    a.c = p->scale * 1.4426950408889634f;
    a.eta = ns_any ? p->ns_eta : 0.0f;
    a.nu = ns_any ? p->ns_nu : 0.0f;
    a.diffuse = (ns_any && p->diffuse_mode == LOGOS_DIFFUSE_CAUSAL) ? 1 : 0;
    a.window = shunyam_active(p->window, S) ? p->window : 0;
    a.stride = lm_stride;
    a.status = ctx->tc_status;
    a.n_qb = (S + kBQ - 1) / kBQ;
    a.BH = BH;
    a.n_items = a.n_qb * BH;
    dim3 grid(a.n_items < ctx->sm_count ? a.n_items : ctx->sm_count);   // persistent: one CTA per SM
#define LOGOS_LAUNCH_TC(DIFF_, LM_, WIN_)                                                                       \
    do {                                                                                                        \
        auto* fn = prefill_tc_kernel<DIFF_, LM_, WIN_>;                                                         \
        if (int rc = ensure_smem_limit(ctx, fn, kSmemBytes)) return rc;                                         \
        fn<<<grid, kTcThreads, kSmemBytes, ctx->stream>>>(mq, mk, mv, mkl, mvl, mvp, a);                        \
    } while (0)
    const bool win = a.window > 0;
    if (a.diffuse && lm_stride) LOGOS_LAUNCH_TC(true, true, true);
    else if (a.diffuse && win) LOGOS_LAUNCH_TC(true, false, true);
    else if (a.diffuse) LOGOS_LAUNCH_TC(true, false, false);
    else if (lm_stride) LOGOS_LAUNCH_TC(false, true, true);
    else if (win) LOGOS_LAUNCH_TC(false, false, true);
    else LOGOS_LAUNCH_TC(false, false, false);
#undef LOGOS_LAUNCH_TC
    LOGOS_LAUNCH_CHECK(ctx, "prefill_tc_kernel");
    return LOGOS_OK;
}

}  // namespace logos
