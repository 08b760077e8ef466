// gemm_tcgen05.cu -- the projections either side of the attention path as tcgen05 GEMMs.
//
// LOGOS projects every head separately: per head and layer three skinny GEMMs [seq x d]·[d x 64]
// for Q, K, V (cuda/ModelGPU.cu:899-906, through amp_gemm -> cuda_gemm_fp16_fp32out,
// cuda/MixedPrecision.cuh:301-330, on an FP16 shadow of the weights), then [seq x 64]·[64 x d] per
// head summed into `concat` (cuda/ModelGPU.cu:974-988) and one [seq x d]·[d x d] for W_proj
// (cuda/ModelGPU.cu:990-1015).  Here a layer's Q, K, V come from ONE GEMM [M x d]·[d x 3 H 64]
// whose epilogue writes them straight into the attention engine's [B][H][S][64] layout and, for K
// and V, reduces max|x| per (sequence, head) tensor -- the first pass of the Nikhilam quantiser
// (absmax_kernel, cuda/ModelGPU.cu:308-326) -- so the cache can be quantised without re-reading them.
// The sum over heads of head_out_h·W_O[h] is one GEMM with the heads concatenated along K.
//
// C[M][N] = A[M][K] · W, fp32 accumulation.  A is row-major 16-bit (BF16 or FP16).  The weight is
// kept K-major, Wt[N][K] (a 16-bit shadow made once at load time, like the reference's FP16 shadow,
// cuda/MixedPrecision.cuh:149-161), so both operands are loaded as 128-byte-swizzled K-major tiles
// and one MMA covers a 128 x 128 block.  One CTA per 128 x 128 output tile, two CTAs per SM (the
// epilogue of one overlaps the main loop of the other), 192 threads:
//   warp 0    TMA producer: A and W tiles of 128 rows x 64 k into a three-stage ring (six stages and one
//             CTA per SM when the grid has fewer CTAs than the device has SMs);
//   warp 1    MMA issuer (one elected lane): four M128 N128 K16 MMAs per stage into 128 TMEM columns;
//   warps 2-5 epilogue: one thread per output row reads its 128 accumulator columns from TMEM.
// Every mbarrier wait is bounded; a wait that runs out raises the context's status word.
#include <algorithm>

#include "tcgen05_ptx.cuh"

namespace logos {
namespace {

using namespace tc;

constexpr int kGN = 128;                 // output columns per CTA
constexpr int kGK = 64;                  // k per stage (one 128-byte swizzle atom of 16-bit values)
constexpr int kGTile = kBM * kGK * 2;    // 16 KiB: one operand tile
constexpr int kGThreads = 192;
constexpr int kSkinnyM = 32, kSkinnyN = 64, kSkinnyStages = 16;   // the decode-time form of the 128-row-tile kernel
// shared memory of the 128-row-tile kernel: the ring, room for the tensor core to read a full 128-row A operand
// from the last stage when the A box is smaller (see the kernel), barriers, alignment slack
__host__ __device__ constexpr int gemm_ring(int stages, int arows, int bn) {
    return stages * (arows + bn) * 128 + ((arows + bn) * 128 < kGTile ? kGTile - (arows + bn) * 128 : 0);
}
constexpr int gemm_smem(int stages, int arows = kBM, int bn = kGN) {
    return gemm_ring(stages, arows, bn) + (2 * stages + 1) * 8 + 64 + 1024;
}

struct GemmArgs {
    int M, N, K;
    int f16;                 // operands are FP16 (else BF16)
    int mode;                // 0: C row-major (+ residual); 1: Q, K, V scatter
    // mode 0
    void* C; const void* R;  // [M][N]; R may be null; same dtype as C
    int c_is_f32;
    // mode 1: N = 3 H 64, rows m = b S + s
    void* q; void* k; void* v;         // [B][H][S][64], 16-bit: the operand dtype, or FP16 with out_f16
    int S, H, out_f16;
    unsigned* k_absmax; unsigned* v_absmax;   // [B][H] float bits (non-negative), atomicMax; may be null
    // A given head-major, [B][a_heads][a_S][64] (the attention's output layout) with K = 64 a_heads: k block kb
    // is head kb, so the tiles are fetched where they lie and nothing is permuted.  0: A is [M][K] row-major.
    int a_heads, a_S;
    int* status;
};

__device__ __forceinline__ uint32_t pack16(float x, float y, bool f16) {
    if (f16) { __half2 h = __floats2half2_rn(x, y); return *reinterpret_cast<uint32_t*>(&h); }
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float round16(float x, bool f16) {
    return f16 ? __half2float(__float2half_rn(x)) : __bfloat162float(__float2bfloat16_rn(x));
}

// ---- epilogue pieces, shared by the two kernels; the calling thread owns output row m ----

// The residual of 32 output columns of row m (64 or 128 bytes), fetched ahead of the accumulator so that its
// latency is not part of the epilogue's chain.  Zeros when there is no residual or the chunk is not live.
struct ResChunk { uint4 v[8]; };
__device__ __forceinline__ void load_residual_chunk(const GemmArgs& a, int m, int n, bool live, ResChunk& r) {
#pragma unroll
    for (int j = 0; j < 8; ++j) r.v[j] = make_uint4(0, 0, 0, 0);
    if (!a.R || !live || n >= a.N) return;
    const size_t off = (size_t)m * a.N + n;
    if (a.c_is_f32) {
        const uint4* res = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.R) + off);
#pragma unroll
        for (int j = 0; j < 8; j += 2) ld_nc_32B(res + j, r.v[j], r.v[j + 1]);
    } else {
        const uint4* res = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(a.R) + off);
#pragma unroll
        for (int j = 0; j < 4; j += 2) ld_nc_32B(res + j, r.v[j], r.v[j + 1]);
    }
}

// 32 accumulator columns (already in registers) plus their residual -> C[m][n .. n+31]
__device__ __forceinline__ void write_c_chunk(const GemmArgs& a, const float (&v)[32], int m, int n, bool live,
                                              const ResChunk& r) {
    const bool f16 = a.f16 != 0;
    if (!live || n >= a.N) return;                 // N is a multiple of 32
    const size_t off = (size_t)m * a.N + n;
    if (a.c_is_f32) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<float*>(a.C) + off);
        uint4 o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 r4 = *reinterpret_cast<const float4*>(&r.v[j]);
            const float4 f = make_float4(v[4 * j] + r4.x, v[4 * j + 1] + r4.y, v[4 * j + 2] + r4.z, v[4 * j + 3] + r4.w);
            o[j] = *reinterpret_cast<const uint4*>(&f);
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2) st_32B(dst + j, o[j], o[j + 1]);
    } else {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(a.C) + off);
        uint4 o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
            const uint32_t* rw = reinterpret_cast<const uint32_t*>(&r.v[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = v[8 * j + 2 * e], y = v[8 * j + 2 * e + 1];
                if (f16) {
                    float2 rr = __half22float2(*reinterpret_cast<const __half2*>(&rw[e]));
                    x += rr.x; y += rr.y;
                } else {
                    x += __uint_as_float(rw[e] << 16); y += __uint_as_float(rw[e] & 0xffff0000u);
                }
                w[e] = pack16(x, y, f16);
            }
            o[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        st_32B(dst, o[0], o[1]);
        st_32B(dst + 2, o[2], o[3]);
    }
}

// One output row's columns [n0, n0 + cols) from the accumulator at t_row, the residual of chunk c + 1 on its way
// while chunk c is written.  `first` was fetched by the caller (before it waited for the accumulator); cols is a
// multiple of 64.  (Having the next chunk's accumulator columns in flight as well measured no faster.)
__device__ __forceinline__ void store_c_row(const GemmArgs& a, uint32_t t_row, int m, int n0, int cols, bool live,
                                            ResChunk& first) {
    ResChunk next;
    float v[32];
#pragma unroll 1
    for (int c0 = 0; c0 < cols; c0 += 64) {
        load_residual_chunk(a, m, n0 + c0 + 32, live, next);
        tc_ld32(t_row + c0, v);
        tc_wait_ld();
        write_c_chunk(a, v, m, n0 + c0, live, first);
        load_residual_chunk(a, m, n0 + c0 + 64, live && c0 + 64 < cols, first);
        tc_ld32(t_row + c0 + 32, v);
        tc_wait_ld();
        write_c_chunk(a, v, m, n0 + c0 + 32, live, next);
    }
}

// 64 accumulator columns = one (projection, head) slice: scatter into Q, K or V [B][H][S][64] and reduce
// max|x| of the stored (rounded) K or V values per (sequence, head) tensor
__device__ __forceinline__ void scatter_head_slice(const GemmArgs& a, uint32_t t_addr, int m, int n, bool row_live,
                                                   int lane) {
    const bool f16 = a.f16 != 0 || a.out_f16 != 0;    // the type Q, K, V are stored in
    const int b = m / a.S, s = m - b * a.S;
    const int hg = n / 64;                           // head slot among 3 H
    const int which = hg / a.H, h = hg - which * a.H;
    float amax = 0.0f;
    unsigned short* base = reinterpret_cast<unsigned short*>(which == 0 ? a.q : (which == 1 ? a.k : a.v));
    const bool live = row_live && which < 3;
    uint4* dst = reinterpret_cast<uint4*>(base + (((size_t)b * a.H + h) * a.S + s) * 64);
#pragma unroll 1
    for (int hc = 0; hc < 2; ++hc) {
        float v[32];
        tc_ld32(t_addr + 32 * hc, v);
        tc_wait_ld();
        if (live) {
            uint4 o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float x = v[8 * j + 2 * e], y = v[8 * j + 2 * e + 1];
                    w[e] = pack16(x, y, f16);
                    amax = fmaxf(amax, fmaxf(fabsf(round16(x, f16)), fabsf(round16(y, f16))));
                }
                o[j] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            st_32B(dst + 4 * hc, o[0], o[1]);
            st_32B(dst + 4 * hc + 2, o[2], o[3]);
        }
    }
    // one atomic per warp when its 32 rows lie in one sequence, else one per row; non-negative floats order
    // like integers
    unsigned* tgt = which == 1 ? a.k_absmax : (which == 2 ? a.v_absmax : nullptr);
    if (tgt) {
        const int b_first = __shfl_sync(0xffffffffu, b, 0), b_last = __shfl_sync(0xffffffffu, b, 31);
        const bool all_live = __all_sync(0xffffffffu, live);
        if (b_first == b_last && all_live) {
            amax = warp_max(amax);
            if (lane == 0) atomicMax(tgt + (size_t)b * a.H + h, __float_as_uint(amax));
        } else if (live) {
            atomicMax(tgt + (size_t)b * a.H + h, __float_as_uint(amax));
        }
    }
}

// STAGES = depth of the operand ring: 3 (96 KiB, two CTAs per SM) when the grid fills the device, 6 (192 KiB) for
// small problems -- a decode-time GEMM has fewer CTAs than SMs and is a chain of TMA round trips, which a deeper
// ring shortens.
// AROWS, BN = rows of the A box and output columns per CTA.  The decode-time form <16, 32, 64> is for M <= 32: a
// stage is 4 KiB of A and 8 KiB of W, so with K = 1024 every k block of the CTA is in flight at once and the chain
// of round trips is one long.  The MMA still reads a 128-row A operand: rows AROWS.. are whatever lies behind the A
// box in shared memory (the W tile, the next stage), they only reach accumulator rows that no one stores.
template <int STAGES, int AROWS = kBM, int BN = kGN>
__global__ void __launch_bounds__(kGThreads, STAGES == 3 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW, const GemmArgs a) {
    constexpr int kABytes = AROWS * 128, kStage = (AROWS + BN) * 128;
    constexpr int kOffBarT = gemm_ring(STAGES, AROWS, BN);
    static_assert(kABytes % 1024 == 0 && kStage % 1024 == 0, "tiles start on swizzle-atom boundaries");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBarT;
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(STAGES + s); };
    const uint32_t acc_full = bar0 + 8u * (uint32_t)(2 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffBarT + (2 * STAGES + 1) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffBarT + (2 * STAGES + 1) * 8 + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN;
    const int n_kb = (a.K + kGK - 1) / kGK;
    // rows of this tile: m0 .. m0 + 127, below m_lim.  Head-major A: tiles never straddle two sequences.
    int m0 = blockIdx.y * kBM, m_lim = a.M, a_row = m0, a_slab = 0;
    if (a.a_heads) {
        const int tiles = (a.a_S + kBM - 1) / kBM;
        const int b = blockIdx.y / tiles;
        a_row = (blockIdx.y - b * tiles) * kBM;
        a_slab = b * a.a_heads;
        m0 = b * a.a_S + a_row;
        m_lim = (b + 1) * a.a_S;
    }

    if (warp == 0 && lane == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Programmatic dependent launch (a no-op for an ordinary launch): the kernel after this one may start at once,
    // and this one, when launched to overlap the kernel before it, fetches its weight tiles -- which no kernel
    // writes -- straight away and waits for that kernel only where it first touches activations.
    grid_release_dependents();
    if (warp == 0) {
        if (lane == 0) {
            auto load_a = [&](int kb, int s) {
                if (a.a_heads) tma_load_3d(sbase + s * kStage, &mapA, 0, a_row, a_slab + kb, full(s));
                else           tma_load_3d(sbase + s * kStage, &mapA, kb * kGK, m0, 0, full(s));
            };
            const int first = n_kb < STAGES ? n_kb : STAGES;
            for (int kb = 0; kb < first; ++kb) {
                mbar_expect_tx(full(kb), kStage);
                tma_load_3d(sbase + kb * kStage + kABytes, &mapW, kb * kGK, n0, 0, full(kb));
            }
            grid_wait_for_earlier();
            for (int kb = 0; kb < first; ++kb) load_a(kb, kb);
            for (int kb = first; kb < n_kb; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(empty(s), ((kb / STAGES) - 1) & 1, abort_flag)) break;
                mbar_expect_tx(full(s), kStage);
                load_a(kb, s);
                tma_load_3d(sbase + s * kStage + kABytes, &mapW, kb * kGK, n0, 0, full(s));
            }
        }
    } else if (warp == 1) {
        uint32_t elected;
        asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(elected));
        const bool leader = elected != 0;
        const int fmt = a.f16 ? 0 : 1;
        const uint32_t idesc = instr_desc(fmt, fmt, 0, BN);
        bool ok = true;
        for (int kb = 0; ok && kb < n_kb; ++kb) {
            const int s = kb % STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(full(s), (kb / STAGES) & 1, abort_flag)) != 0;
            if (!ok) break;
            tc_fence_after();
            if (leader) {
                const uint32_t sa = sbase + s * kStage, sw = sa + kABytes;
#pragma unroll
                for (int kk = 0; kk < kGK / 16; ++kk)
                    tc_mma_f16(tmem, smem_desc(sa + 32 * kk), smem_desc(sw + 32 * kk), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                tc_commit(empty(s));                    // the stage is free once these MMAs have read it
                if (kb == n_kb - 1) tc_commit(acc_full);
            }
            __syncwarp();
        }
    } else {
        // ---- epilogue: thread = output row, TMEM lane quarter = warp % 4 ----
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane, m = m0 + row;
        const uint32_t t_row = tmem + (((uint32_t)(quarter * 32)) << 16);
        ResChunk res0;
        grid_wait_for_earlier();          // the residual, the outputs and the max|x| tables belong to the stream's order
        if (a.mode == 0) load_residual_chunk(a, m, n0, m < m_lim, res0);
        if (mbar_wait(acc_full, 0, abort_flag)) {
            tc_fence_after();
            if (a.mode == 0) {
                store_c_row(a, t_row, m, n0, BN, m < m_lim, res0);
            } else {
#pragma unroll 1
                for (int gi = 0; gi < BN / 64; ++gi) scatter_head_slice(a, t_row + 64 * gi, m, n0 + 64 * gi, m < m_lim, lane);
            }
            tc_fence_before();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) atomicExch(a.status, (*abort_flag & ~0xffff) | ((*abort_flag - (int)(bar0 & 0xffffu)) & 0xffff));
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128u) : "memory");
    }
}

// ---- the wide kernel: persistent CTAs, 128 x 256 tiles, two accumulators ----
//
// A 128 x 128 MMA reads 8 KiB of operands from shared memory for 64 cycles of tensor-pipe work: that is the
// whole shared-memory bandwidth of an SM, and it is what holds the kernel above near half of the pipe's
// peak.  With N = 256 the same A tile feeds twice the columns (12 KiB per 128 cycles).  One CTA per SM walks
// the tiles (n fastest, so the CTAs running together share A rows and the whole weight stays in L2); the
// accumulator is double-buffered in tensor memory (2 x 256 columns), so the epilogue warps drain tile t while
// the MMA warp fills tile t + 1; four stages of 48 KiB keep TMA ahead of the MMAs.
constexpr int kWN = 256;
constexpr int kWStages = 4;
constexpr int kWTileB = kWN * kGK * 2;            // 32 KiB
constexpr int kWStage = kGTile + kWTileB;         // 48 KiB
constexpr int kWOffBar = kWStages * kWStage;
constexpr int kWSmem = kWOffBar + (2 * kWStages + 4) * 8 + 64 + 1024;

__global__ void __launch_bounds__(kGThreads, 1)
gemm_tc_wide_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapW, const GemmArgs a,
                    int m_tiles, int n_tiles) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kWOffBar;
    auto full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(kWStages + s); };
    auto acc_full = [&](int t) { return bar0 + 8u * (uint32_t)(2 * kWStages + t); };
    auto acc_empty = [&](int t) { return bar0 + 8u * (uint32_t)(2 * kWStages + 2 + t); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kWOffBar + (2 * kWStages + 4) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kWOffBar + (2 * kWStages + 4) * 8 + 16);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_kb = (a.K + kGK - 1) / kGK;
    const int total = m_tiles * n_tiles;

    if (warp == 0 && lane == 0) {
        for (int s = 0; s < kWStages; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int t = 0; t < 2; ++t) { mbar_init(acc_full(t), 1); mbar_init(acc_empty(t), 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // rows of m tile mt: m0 .. m0 + 127 below m_lim; head-major A: (row in the sequence, first slab)
    auto tile_rows = [&](int mt, int& m0, int& m_lim, int& a_row, int& a_slab) {
        m0 = mt * kBM; m_lim = a.M; a_row = m0; a_slab = 0;
        if (a.a_heads) {
            const int tiles = (a.a_S + kBM - 1) / kBM;
            const int b = mt / tiles;
            a_row = (mt - b * tiles) * kBM;
            a_slab = b * a.a_heads;
            m0 = b * a.a_S + a_row;
            m_lim = (b + 1) * a.a_S;
        }
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                                   // k blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
                const int mt = tile / n_tiles, n0 = (tile - mt * n_tiles) * kWN;
                int m0, m_lim, a_row, a_slab;
                tile_rows(mt, m0, m_lim, a_row, a_slab);
                bool ok = true;
                for (int kb = 0; kb < n_kb; ++kb, ++it) {
                    const int s = it % kWStages;
                    if (!mbar_wait(empty(s), ((it / kWStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(full(s), kWStage);
                    const uint32_t dst = sbase + s * kWStage;
                    if (a.a_heads) tma_load_3d(dst, &mapA, 0, a_row, a_slab + kb, full(s));
                    else           tma_load_3d(dst, &mapA, kb * kGK, m0, 0, full(s));
                    tma_load_3d(dst + kGTile, &mapW, kb * kGK, n0, 0, full(s));
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        uint32_t elected;
        asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(elected));
        const bool leader = elected != 0;
        const int fmt = a.f16 ? 0 : 1;
        const uint32_t idesc = instr_desc(fmt, fmt, 0, kWN);
        uint32_t it = 0, lt = 0;                               // k blocks and tiles done by this CTA
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x, ++lt) {
            const int acc = lt & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(acc_empty(acc), ((lt >> 1) & 1) ^ 1, abort_flag)) != 0;
            if (!ok) break;
            tc_fence_after();
            const uint32_t d = tmem + (uint32_t)(acc * kWN);
            for (int kb = 0; kb < n_kb; ++kb, ++it) {
                const int s = it % kWStages;
                ok = __all_sync(0xffffffffu, mbar_wait(full(s), (it / kWStages) & 1, abort_flag)) != 0;
                if (!ok) break;
                tc_fence_after();
                if (leader) {
                    const uint32_t sa = sbase + s * kWStage, sw = sa + kGTile;
#pragma unroll
                    for (int kk = 0; kk < kGK / 16; ++kk)
                        tc_mma_f16(d, smem_desc(sa + 32 * kk), smem_desc(sw + 32 * kk), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(empty(s));
                    if (kb == n_kb - 1) tc_commit(acc_full(acc));
                }
                __syncwarp();
            }
        }
    } else {
        // ---- epilogue: thread = output row, TMEM lane quarter = warp % 4 ----
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        uint32_t lt = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++lt) {
            const int mt = tile / n_tiles, n0 = (tile - mt * n_tiles) * kWN;
            int m0, m_lim, a_row, a_slab;
            tile_rows(mt, m0, m_lim, a_row, a_slab);
            const int m = m0 + row, acc = lt & 1;
            ResChunk res0;
            if (a.mode == 0) load_residual_chunk(a, m, n0, m < m_lim, res0);
            if (!mbar_wait(acc_full(acc), (lt >> 1) & 1, abort_flag)) break;
            tc_fence_after();
            const uint32_t t_row = tmem + (((uint32_t)(quarter * 32)) << 16) + (uint32_t)(acc * kWN);
            if (a.mode == 0) {
                store_c_row(a, t_row, m, n0, kWN, m < m_lim, res0);
            } else {
#pragma unroll 1
                for (int gi = 0; gi < kWN / 64; ++gi)
                    scatter_head_slice(a, t_row + 64 * gi, m, n0 + 64 * gi, m < m_lim && n0 + 64 * gi < a.N, lane);
            }
            tc_fence_before();
            mbar_arrive(acc_empty(acc));               // this accumulator may be overwritten
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && tid == 0) atomicExch(a.status, (*abort_flag & ~0xffff) | ((*abort_flag - (int)(bar0 & 0xffffu)) & 0xffff));
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// [rows][K] 16-bit row-major matrix, box = 128 rows x 64 k, 128-byte swizzle
bool make_map_2d(CUtensorMap* m, const void* base, int rows, int K, bool f16, int box_rows = kBM) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, 1};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)rows * K * 2};
    cuuint32_t box[3] = {(cuuint32_t)kGK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [slabs][S][64] 16-bit (one slab per (sequence, head)), box = 128 rows x 64, 128-byte swizzle
bool make_map_slabs(CUtensorMap* m, const void* base, int S, int slabs, bool f16) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {64, (cuuint64_t)S, (cuuint64_t)slabs};
    cuuint64_t strides[2] = {128, (cuuint64_t)S * 128};
    cuuint32_t box[3] = {(cuuint32_t)kGK, (cuuint32_t)kBM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_gemm(logos_ctx* ctx, const void* A, const void* Wt, GemmArgs& a) {
    if (a.M <= 0 || a.N <= 0 || a.K <= 0 || (a.K % 8) != 0 || (a.N % 64) != 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "projection: M, N, K = %d, %d, %d (K a multiple of 8, N of 64)", a.M, a.N, a.K);
    if (!aligned16(A) || !aligned16(Wt))
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "projection: operands must be 16-byte aligned");
    if (!ctx->tc_status) return fail(ctx, LOGOS_ERR_WORKSPACE, "projection: status word missing");
    CUtensorMap ma, mw;
    const int m_tiles = a.a_heads ? (a.M / a.a_S) * ((a.a_S + kBM - 1) / kBM) : (a.M + kBM - 1) / kBM;
    const int n_wide = (a.N + kWN - 1) / kWN;
    // enough 128 x 256 tiles to give every SM one: the persistent wide kernel; otherwise the 128 x 128 kernel,
    // which has twice the CTAs for a small problem
    const bool wide = (int64_t)m_tiles * n_wide >= ctx->sm_count && !ctx->gemm_narrow;
    // a decode step's projections: at most 32 rows
    const bool skinny = a.M <= kSkinnyM && !a.a_heads && !wide;
    const bool a_ok = a.a_heads ? make_map_slabs(&ma, A, a.a_S, (a.M / a.a_S) * a.a_heads, a.f16 != 0)
                                : make_map_2d(&ma, A, a.M, a.K, a.f16 != 0, skinny ? kSkinnyM : kBM);
    if (!a_ok || !make_map_2d(&mw, Wt, a.N, a.K, a.f16 != 0, wide ? kWN : (skinny ? kSkinnyN : kBM)))
        return fail(ctx, LOGOS_ERR_CUDA, "projection: cuTensorMapEncodeTiled failed");
    a.status = ctx->tc_status;
    if (wide) {
        if (int rc = ensure_smem_limit(ctx, gemm_tc_wide_kernel, kWSmem)) return rc;
        const int ctas = (int)std::min<int64_t>((int64_t)m_tiles * n_wide, ctx->sm_count);
        gemm_tc_wide_kernel<<<ctas, kGThreads, kWSmem, ctx->stream>>>(ma, mw, a, m_tiles, n_wide);
        LOGOS_LAUNCH_CHECK(ctx, "gemm_tc_wide_kernel");
        return LOGOS_OK;
    }
    if (skinny) {
        auto* fn = gemm_tc_kernel<kSkinnyStages, kSkinnyM, kSkinnyN>;
        constexpr int smem = gemm_smem(kSkinnyStages, kSkinnyM, kSkinnyN);
        if (int rc = ensure_smem_limit(ctx, fn, smem)) return rc;
        const dim3 sgrid((a.N + kSkinnyN - 1) / kSkinnyN, 1);
        if (ctx->project_overlap) {      // launched to overlap the kernel before it on the stream: see the kernel
            LOGOS_CUDA_TRY(ctx, launch_overlapped(fn, sgrid, dim3(kGThreads), (size_t)smem, ctx->stream, ma, mw, a));
        } else {
            fn<<<sgrid, kGThreads, smem, ctx->stream>>>(ma, mw, a);
        }
        LOGOS_LAUNCH_CHECK(ctx, "gemm_tc_kernel (decode form)");
        return LOGOS_OK;
    }
    dim3 grid((a.N + kGN - 1) / kGN, m_tiles);
    if ((int64_t)grid.x * grid.y <= ctx->sm_count) {       // fewer CTAs than SMs: the deep ring
        if (int rc = ensure_smem_limit(ctx, gemm_tc_kernel<6>, gemm_smem(6))) return rc;
        gemm_tc_kernel<6><<<grid, kGThreads, gemm_smem(6), ctx->stream>>>(ma, mw, a);
    } else {
        if (int rc = ensure_smem_limit(ctx, gemm_tc_kernel<3>, gemm_smem(3))) return rc;
        gemm_tc_kernel<3><<<grid, kGThreads, gemm_smem(3), ctx->stream>>>(ma, mw, a);
    }
    LOGOS_LAUNCH_CHECK(ctx, "gemm_tc_kernel");
    return LOGOS_OK;
}

}  // namespace

int project(logos_ctx* ctx, int dtype, int out_dtype, const void* A, const void* Wt, const void* residual, void* C,
            int M, int N, int K) {
    if (!A || !Wt || !C) return fail(ctx, LOGOS_ERR_INVALID_ARG, "project: null pointer");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "project: operands must be BF16 or FP16");
    if (out_dtype != dtype && out_dtype != LOGOS_F32) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "project: output is the operand type or fp32");
    if (!aligned32(C) || (residual && !aligned32(residual)) || (N % 64) != 0)
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "project: C and the residual must be 32-byte aligned, N a multiple of 64");
    GemmArgs a{};
    a.M = M; a.N = N; a.K = K; a.f16 = dtype == LOGOS_F16; a.mode = 0;
    a.C = C; a.R = residual; a.c_is_f32 = out_dtype == LOGOS_F32;
    return launch_gemm(ctx, A, Wt, a);
}

int project_heads(logos_ctx* ctx, int dtype, int out_dtype, const void* head_out, const void* Wt, const void* residual,
                  void* C, int B, int S, int H, int N) {
    if (!head_out || !Wt || !C || B <= 0 || S <= 0 || H <= 0 || N <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "project_heads: bad pointer or extent");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "project_heads: operands must be BF16 or FP16");
    if (out_dtype != dtype && out_dtype != LOGOS_F32) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "project_heads: output is the operand type or fp32");
    if (!aligned32(C) || (residual && !aligned32(residual)) || (N % 64) != 0)
        return fail(ctx, LOGOS_ERR_ALIGNMENT, "project_heads: C and the residual must be 32-byte aligned, N a multiple of 64");
    GemmArgs a{};
    a.M = B * S; a.N = N; a.K = H * 64; a.f16 = dtype == LOGOS_F16; a.mode = 0;
    a.C = C; a.R = residual; a.c_is_f32 = out_dtype == LOGOS_F32;
    a.a_heads = H; a.a_S = S;
    return launch_gemm(ctx, head_out, Wt, a);
}

int qkv_project(logos_ctx* ctx, int dtype, const void* X, const void* Wt, void* Q, void* K, void* V, int B, int S,
                int H, int D, float* k_absmax, float* v_absmax) {
    if (!X || !Wt || !Q || !K || !V || B <= 0 || S <= 0 || H <= 0 || D <= 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "qkv_project: bad pointer or extent");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16) return fail(ctx, LOGOS_ERR_UNSUPPORTED, "qkv_project: operands must be BF16 or FP16");
    if (!aligned32(Q) || !aligned32(K) || !aligned32(V)) return fail(ctx, LOGOS_ERR_ALIGNMENT, "qkv_project: outputs must be 32-byte aligned");
    if ((k_absmax == nullptr) != (v_absmax == nullptr))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "qkv_project: the two absmax tables are given together or not at all");
    if (k_absmax) {
        LOGOS_CUDA_TRY(ctx, cudaMemsetAsync(k_absmax, 0, sizeof(float) * (size_t)B * H, ctx->stream));
        LOGOS_CUDA_TRY(ctx, cudaMemsetAsync(v_absmax, 0, sizeof(float) * (size_t)B * H, ctx->stream));
    }
    GemmArgs a{};
    a.M = B * S; a.N = 3 * H * 64; a.K = D; a.f16 = dtype == LOGOS_F16; a.mode = 1;
    a.q = Q; a.k = K; a.v = V; a.S = S; a.H = H; a.out_f16 = ctx->qkv_out_f16 ? 1 : 0;
    a.k_absmax = reinterpret_cast<unsigned*>(k_absmax); a.v_absmax = reinterpret_cast<unsigned*>(v_absmax);
    return launch_gemm(ctx, X, Wt, a);
}

}  // namespace logos
