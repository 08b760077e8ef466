// comm.cu -- exchange of attention outputs between the GPUs that share a model's heads.
//
// The path shards by (sequence, head): each GPU owns a contiguous block of heads with their INT8
// cache, and the one exchange is the all-gather of the per-head outputs along the head axis (the
// reference has no multi-GPU path; its head loop is serial, cuda/ModelGPU.cu:892-988).  At decode
// sizes that gather is 32 KB per GPU and a library collective costs more than the attention, so the
// exchange is done by the kernels themselves over peer-mapped memory:
//   * every rank owns one block of device memory (logos_comm) that all peers map -- in the same
//     process directly, across processes through a CUDA IPC handle;
//   * decode rows (small, latency-bound): the decode kernel's epilogue stores every value into the
//     row area of EVERY rank as an 8-byte word {value, step + 1} with plain st.global over NVLink.  An
//     aligned 8-byte store arrives whole, so each word is its own arrival flag: the sender needs no
//     fence, no completion counter and no separate flag message.  collect_rows_kernel on each rank
//     polls the words themselves, writes the packed fp32 rows to the caller's tensor and advances
//     the rank's step counter.  Its launch overlaps the flight of the last stores.
//   * any other per-head tensor (large, bandwidth-bound): push_kernel stores the local tensor into
//     the staging slot of every rank, then one fence per CTA, a completion counter and a flag per
//     rank; gather_wait_kernel waits for all ranks' flags, copies the slot out and advances the step.
// Staging has two slots used in alternation (step parity): a rank that is already one step ahead
// writes the other slot, and it cannot get two steps ahead because its own wait needs this rank's
// next flag.  The step counter lives in device memory, so a CUDA graph of the step replays unchanged.
// No TMA, no multicast, no multimem: loads are local, stores are ordinary peer stores.
// The only waits are in the two receiving kernels and they are bounded by wall time
// (LOGOS_OPT_PEER_WAIT_MS); when a wait runs out the kernel raises the context's status word and returns.
#include <cuda.h>

#include <cstring>
#include <new>

#include "common.cuh"

namespace logos {
namespace {

struct WaitArgs {
    const unsigned* flags;     // this rank's block: one word per source rank, kCommFlagStride apart
    unsigned* step;
    unsigned* copy_done;
    const float4* stage;       // two slots of slot_f4 float4 each
    float4* dst;
    size_t slot_f4, n_f4;
    int world;
    unsigned long long limit_ns;
    int* status;
};

__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(256)
gather_wait_kernel(const WaitArgs w) {
    __shared__ unsigned step_s;
    if (threadIdx.x == 0) step_s = *reinterpret_cast<volatile unsigned*>(w.step);
    __syncthreads();
    const unsigned step = step_s;
    if ((int)threadIdx.x < w.world) {
        const unsigned* f = w.flags + threadIdx.x * (kCommFlagStride / sizeof(unsigned));
        const unsigned long long t0 = global_ns();
        unsigned spins = 0;
        // relaxed polls and one acquire fence at the end: an acquire on every poll would pay for a
        // system-scope fence each time round
        while ((int)(ld_relaxed_sys(f) - (step + 1u)) < 0) {
            if ((++spins & 31u) == 0u && global_ns() - t0 > w.limit_ns) {
                // bits [16,24): the rank that did not arrive; 0x20000000 marks a peer wait
                atomicCAS(w.status, 0, 0x20000000 | ((int)threadIdx.x << 16) | 1);
                break;
            }
            __nanosleep(32);
        }
        asm volatile("fence.acq_rel.sys;" ::: "memory");
    }
    __syncthreads();
    // staging -> the caller's tensor; the rows came from other GPUs, so they are read past L1
    const float4* src = w.stage + (size_t)(step & 1u) * w.slot_f4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < w.n_f4; i += (size_t)gridDim.x * blockDim.x)
        w.dst[i] = __ldcg(src + i);
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(w.copy_done, 1u);
        if (prev == gridDim.x - 1) {       // every CTA has read the step: it may move on
            *w.copy_done = 0;
            *reinterpret_cast<volatile unsigned*>(w.step) = step + 1u;
        }
    }
}

struct CollectArgs {
    const uint4* rows;         // this rank's row area: two slots of slot_words 8-byte words, read two at a time
    float2* dst;               // packed rows
    unsigned* step;
    unsigned* copy_done;
    size_t slot_pairs, n_pairs;   // 16-byte units (two values) per slot / to collect
    int H_total, DH, world;       // rows are [B][H_total][DH]; used to name a missing rank
    unsigned long long limit_ns;
    int* status;
};

// Polls the 8-byte words {value, mark} that the peers' decode kernels store into this rank's row area
// until every mark shows the current step, and writes the values out packed.
__global__ void __launch_bounds__(256)
collect_rows_kernel(const CollectArgs c) {
    __shared__ unsigned step_s;
    if (threadIdx.x == 0) step_s = *reinterpret_cast<volatile unsigned*>(c.step);
    __syncthreads();
    const unsigned step = step_s, mark = step + 1u;
    const uint4* src = c.rows + (size_t)(step & 1u) * c.slot_pairs;
    const unsigned long long t0 = global_ns();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < c.n_pairs; i += (size_t)gridDim.x * blockDim.x) {
        uint4 w;
        unsigned spins = 0;
        for (;;) {
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(src + i) : "memory");
            if (w.y == mark && w.w == mark) break;
            if ((++spins & 63u) == 0u && global_ns() - t0 > c.limit_ns) {
                // which rank's rows are missing: value 2 i lies in head (2 i / DH) % H_total
                const int rank = (int)(((2 * i) / (size_t)c.DH) % (size_t)c.H_total) / (c.H_total / c.world);
                atomicCAS(c.status, 0, 0x20000000 | (rank << 16) | 1);
                break;
            }
            __nanosleep(20);
        }
        c.dst[i] = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
    }
    // launched to overlap the decode kernel before it (the words above carry their own marks, so nothing
    // of that kernel had to be complete to read them): this kernel still may not end before it has
    grid_wait_for_earlier();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(c.copy_done, 1u);
        if (prev == gridDim.x - 1) {       // every CTA has read the step: it may move on
            *c.copy_done = 0;
            *reinterpret_cast<volatile unsigned*>(c.step) = step + 1u;
        }
    }
}

// Where the flag protocol sends a tensor: every rank's staging slot and flag word.
struct PushTargets {
    float* stage[kMaxPeers];      // staging area of each rank: two slots of slot_floats floats (step parity)
    unsigned* flag[kMaxPeers];    // in rank r's block: the word THIS rank sets to step + 1
    const unsigned* step;
    unsigned* done;               // CTAs of this launch that have stored their part; zero between launches
    size_t slot_floats;
    int world, H_total, head0;
};

struct PushArgs {
    const uint4* local;        // [B][H_local][row16] 16-byte vectors
    PushTargets peer;
    int B, H_local;
    size_t row16;              // 16-byte vectors per (b, h) row
};

// Any [B][H_local][row] tensor of this rank into every rank's staging slot at its head offset.
__global__ void __launch_bounds__(256)
push_kernel(const PushArgs a) {
    const unsigned step = *a.peer.step;
    const size_t n = (size_t)a.B * a.H_local * a.row16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t bh = i / a.row16, e = i - bh * a.row16;
        const size_t b = bh / a.H_local, h = bh - b * a.H_local;
        const size_t o = (size_t)(step & 1u) * (a.peer.slot_floats / 4) + ((b * a.peer.H_total + a.peer.head0 + h) * a.row16 + e);
        const uint4 v = a.local[i];
        for (int r = 0; r < a.peer.world; ++r) reinterpret_cast<uint4*>(a.peer.stage[r])[o] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {      // one fence per CTA: the barrier orders all threads' stores before it
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        const unsigned prev = atomicAdd(a.peer.done, 1u);
        if (prev == gridDim.x - 1) {
            *a.peer.done = 0;
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            for (int r = 0; r < a.peer.world; ++r)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.peer.flag[r]), "r"(step + 1u) : "memory");
        }
    }
}

int comm_ready(logos_ctx* ctx, const logos_comm* c) {
    if (!ctx || !c) return LOGOS_ERR_INVALID_ARG;
    if (c->ctx != ctx) return fail(ctx, LOGOS_ERR_INVALID_ARG, "comm belongs to another context");
    if (!c->connected) return fail(ctx, LOGOS_ERR_INVALID_ARG, "comm is not connected to its peers yet");
    return LOGOS_OK;
}

}  // namespace

void comm_peer_epilogue(const logos_comm* c, int H_local, PeerEpilogue* out) {
    for (int r = 0; r < c->world; ++r)
        out->rows[r] = reinterpret_cast<uint2*>(c->peer[r] + kCommStageOff + 2 * c->slot_bytes);
    out->step = reinterpret_cast<const unsigned*>(c->block + kCommStepOff);
    out->slot_words = c->row_slot_bytes / sizeof(uint2);
    out->world = c->world;
    out->H_total = H_local * c->world;
    out->head0 = H_local * c->rank;
}

namespace {
void push_targets(const logos_comm* c, int H_local, PushTargets* out) {
    for (int r = 0; r < c->world; ++r) {
        out->stage[r] = reinterpret_cast<float*>(c->peer[r] + kCommStageOff);
        out->flag[r] = reinterpret_cast<unsigned*>(c->peer[r] + (size_t)c->rank * kCommFlagStride);
    }
    out->step = reinterpret_cast<const unsigned*>(c->block + kCommStepOff);
    out->done = reinterpret_cast<unsigned*>(c->block + kCommDoneOff);
    out->slot_floats = c->slot_bytes / sizeof(float);
    out->world = c->world;
    out->H_total = H_local * c->world;
    out->head0 = H_local * c->rank;
}
}  // namespace

int comm_collect_rows(logos_ctx* ctx, logos_comm* c, float* gathered, int B, int H_total, int DH,
                      bool follows_decode) {
    int rc = comm_ready(ctx, c);
    if (rc != LOGOS_OK) return rc;
    if (B <= 0 || H_total <= 0 || DH <= 0 || H_total % c->world != 0)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "collect_rows: bad extents");
    const size_t values = (size_t)B * H_total * DH;
    if (!gathered || values == 0 || (values & 1u) || values * sizeof(uint2) > c->row_slot_bytes ||
        (reinterpret_cast<uintptr_t>(gathered) & 7u))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "collect_rows: %zu values do not fit the row area (%zu bytes per slot)",
                    values, c->row_slot_bytes);
    CollectArgs a;
    a.rows = reinterpret_cast<const uint4*>(c->block + kCommStageOff + 2 * c->slot_bytes);
    a.dst = reinterpret_cast<float2*>(gathered);
    a.step = reinterpret_cast<unsigned*>(c->block + kCommStepOff);
    a.copy_done = reinterpret_cast<unsigned*>(c->block + kCommCopyDoneOff);
    a.slot_pairs = c->row_slot_bytes / sizeof(uint4);
    a.n_pairs = values / 2;
    a.H_total = H_total; a.DH = DH; a.world = c->world;
    a.limit_ns = (unsigned long long)ctx->peer_wait_ms * 1000000ull;
    a.status = ctx->tc_status;
    size_t ctas = (a.n_pairs + 255) / 256;
    if (ctas > (size_t)ctx->sm_count * 4) ctas = (size_t)ctx->sm_count * 4;
    if (follows_decode) {      // the kernel before this one on the stream is the decode that feeds it
        LOGOS_CUDA_TRY(ctx, launch_overlapped(collect_rows_kernel, dim3((unsigned)ctas), dim3(256), 0, ctx->stream, a));
        return LOGOS_OK;
    }
    collect_rows_kernel<<<(unsigned)ctas, 256, 0, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "collect_rows_kernel");
    return LOGOS_OK;
}

int comm_wait(logos_ctx* ctx, logos_comm* c, void* gathered, size_t bytes) {
    int rc = comm_ready(ctx, c);
    if (rc != LOGOS_OK) return rc;
    if (!gathered || bytes == 0 || bytes > c->slot_bytes || (bytes & 15u) || !aligned16(gathered))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "comm_wait: %zu bytes do not fit a slot of %zu (16-byte units)", bytes,
                    c->slot_bytes);
    WaitArgs w;
    w.flags = reinterpret_cast<const unsigned*>(c->block);
    w.step = reinterpret_cast<unsigned*>(c->block + kCommStepOff);
    w.copy_done = reinterpret_cast<unsigned*>(c->block + kCommCopyDoneOff);
    w.stage = reinterpret_cast<const float4*>(c->block + kCommStageOff);
    w.dst = reinterpret_cast<float4*>(gathered);
    w.slot_f4 = c->slot_bytes / 16;
    w.n_f4 = bytes / 16;
    w.world = c->world;
    w.limit_ns = (unsigned long long)ctx->peer_wait_ms * 1000000ull;
    w.status = ctx->tc_status;
    size_t ctas = (w.n_f4 + 255) / 256;
    if (ctas > (size_t)ctx->sm_count * 4) ctas = (size_t)ctx->sm_count * 4;
    gather_wait_kernel<<<(unsigned)ctas, 256, 0, ctx->stream>>>(w);
    LOGOS_LAUNCH_CHECK(ctx, "gather_wait_kernel");
    return LOGOS_OK;
}

int comm_push(logos_ctx* ctx, logos_comm* c, const void* local, int B, int H_local, size_t row_bytes) {
    int rc = comm_ready(ctx, c);
    if (rc != LOGOS_OK) return rc;
    if (!local || B <= 0 || H_local <= 0 || row_bytes == 0 || (row_bytes & 15u) || !aligned16(local))
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "comm_push: bad tensor (rows are whole 16-byte vectors)");
    if ((size_t)B * H_local * c->world * row_bytes > c->slot_bytes)
        return fail(ctx, LOGOS_ERR_INVALID_ARG, "comm_push: gathered tensor exceeds the slot of %zu bytes", c->slot_bytes);
    PushArgs a;
    a.local = reinterpret_cast<const uint4*>(local);
    push_targets(c, H_local, &a.peer);
    a.B = B; a.H_local = H_local; a.row16 = row_bytes / 16;
    size_t n = (size_t)B * H_local * a.row16, ctas = (n + 255) / 256;
    if (ctas > (size_t)ctx->sm_count * 8) ctas = (size_t)ctx->sm_count * 8;
    push_kernel<<<(unsigned)ctas, 256, 0, ctx->stream>>>(a);
    LOGOS_LAUNCH_CHECK(ctx, "push_kernel");
    return LOGOS_OK;
}

}  // namespace logos

extern "C" {

int logos_comm_create(logos_ctx* ctx, int rank, int world, size_t gathered_bytes, logos_comm** out) {
    if (!ctx || !out) return LOGOS_ERR_INVALID_ARG;
    *out = nullptr;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world || gathered_bytes == 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "comm_create: rank %d of %d (at most %d ranks)", rank, world, kMaxPeers);
    logos_comm* c = new (std::nothrow) logos_comm();
    if (!c) return LOGOS_ERR_CUDA;
    c->ctx = ctx; c->rank = rank; c->world = world;
    c->slot_bytes = (gathered_bytes + 255) & ~(size_t)255;
    // the row area takes 8 bytes per fp32 value of a gathered decode output, up to a cap: decode
    // outputs are small, the staging slots may be sized for a prefill tensor
    c->row_slot_bytes = 2 * c->slot_bytes < logos::kCommRowSlotMax ? 2 * c->slot_bytes : logos::kCommRowSlotMax;
    const size_t total = logos::kCommStageOff + 2 * c->slot_bytes + 2 * c->row_slot_bytes;
    if (cudaSetDevice(ctx->device) != cudaSuccess || cudaMalloc(&c->block, total) != cudaSuccess ||
        cudaMemset(c->block, 0, total) != cudaSuccess) {
        const cudaError_t e = cudaGetLastError();
        if (c->block) cudaFree(c->block);
        delete c;
        return logos::fail(ctx, LOGOS_ERR_CUDA, "comm_create: %s", cudaGetErrorString(e));
    }
    c->peer[rank] = c->block;
    c->connected = world == 1;
    *out = c;
    return LOGOS_OK;
}

// What a rank sends to its peers: the CUDA IPC handle of the allocation that holds its block, the
// block's offset inside that allocation (an IPC mapping always starts at the allocation's base, and
// the driver may place a small cudaMalloc inside a larger one), and a word that the block carries at
// a known place, so that the peer can check it mapped the right memory.
struct CommHandle {
    cudaIpcMemHandle_t ipc;
    unsigned long long offset;
    unsigned long long magic;
};
static_assert(sizeof(CommHandle) == LOGOS_COMM_HANDLE_BYTES, "handle size");

int logos_comm_handle(logos_comm* c, void* handle_out) {
    if (!c || !handle_out) return LOGOS_ERR_INVALID_ARG;
    CommHandle h;
    memset(&h, 0, sizeof(h));
    LOGOS_CUDA_TRY(c->ctx, cudaSetDevice(c->ctx->device));
    LOGOS_CUDA_TRY(c->ctx, cudaIpcGetMemHandle(&h.ipc, c->block));
    // the driver entry point is looked up at run time: the library must load where there is no driver
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess || !fn)
        return logos::fail(c->ctx, LOGOS_ERR_CUDA, "comm_handle: cuMemGetAddressRange is not available");
    CUdeviceptr base = 0;
    size_t size = 0;
    if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(c->block)) != CUDA_SUCCESS)
        return logos::fail(c->ctx, LOGOS_ERR_CUDA, "comm_handle: cuMemGetAddressRange failed");
    h.offset = reinterpret_cast<CUdeviceptr>(c->block) - base;
    h.magic = 0x4c4f474f53000000ull ^ (reinterpret_cast<unsigned long long>(c->block) * 0x9e3779b97f4a7c15ull) ^ (unsigned)c->rank;
    LOGOS_CUDA_TRY(c->ctx, cudaMemcpy(c->block + logos::kCommMagicOff, &h.magic, sizeof(h.magic), cudaMemcpyHostToDevice));
    memcpy(handle_out, &h, sizeof(h));
    return LOGOS_OK;
}

int logos_comm_connect(logos_comm* c, const void* handles) {
    if (!c || !handles) return LOGOS_ERR_INVALID_ARG;
    if (c->connected) return logos::fail(c->ctx, LOGOS_ERR_INVALID_ARG, "comm_connect: already connected");
    LOGOS_CUDA_TRY(c->ctx, cudaSetDevice(c->ctx->device));
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        CommHandle h;
        memcpy(&h, static_cast<const unsigned char*>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        LOGOS_CUDA_TRY(c->ctx, cudaIpcOpenMemHandle(&p, h.ipc, cudaIpcMemLazyEnablePeerAccess));
        c->ipc_base[r] = p;
        c->peer[r] = static_cast<unsigned char*>(p) + h.offset;
        unsigned long long seen = 0;
        LOGOS_CUDA_TRY(c->ctx, cudaMemcpy(&seen, c->peer[r] + logos::kCommMagicOff, sizeof(seen), cudaMemcpyDeviceToHost));
        if (seen != h.magic)
            return logos::fail(c->ctx, LOGOS_ERR_CUDA, "comm_connect: the mapping of rank %d's block does not show its mark", r);
    }
    c->connected = true;
    return LOGOS_OK;
}

int logos_comm_connect_local(logos_comm* const* comms, int world) {
    if (!comms || world < 1 || world > kMaxPeers) return LOGOS_ERR_INVALID_ARG;
    for (int r = 0; r < world; ++r)
        if (!comms[r] || comms[r]->world != world || comms[r]->rank != r || comms[r]->connected != (world == 1))
            return LOGOS_ERR_INVALID_ARG;
    for (int r = 0; r < world; ++r) {
        logos_comm* c = comms[r];
        for (int s = 0; s < world; ++s) {
            if (s == r) continue;
            const int dev_r = c->ctx->device, dev_s = comms[s]->ctx->device;
            if (dev_r != dev_s) {      // another GPU of this process: its memory must be reachable from here
                int can = 0;
                LOGOS_CUDA_TRY(c->ctx, cudaDeviceCanAccessPeer(&can, dev_r, dev_s));
                if (!can) return logos::fail(c->ctx, LOGOS_ERR_UNSUPPORTED, "comm: device %d cannot reach device %d", dev_r, dev_s);
                LOGOS_CUDA_TRY(c->ctx, cudaSetDevice(dev_r));
                const cudaError_t e = cudaDeviceEnablePeerAccess(dev_s, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    return logos::fail(c->ctx, LOGOS_ERR_CUDA, "comm: cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
                cudaGetLastError();
            }
            c->peer[s] = comms[s]->block;
        }
        c->connected = true;
    }
    return LOGOS_OK;
}

int logos_comm_destroy(logos_comm* c) {
    if (!c) return LOGOS_OK;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    for (int r = 0; r < c->world; ++r)
        if (c->ipc_base[r]) cudaIpcCloseMemHandle(c->ipc_base[r]);
    if (c->block) cudaFree(c->block);
    delete c;
    return LOGOS_OK;
}

int logos_comm_push(logos_ctx* ctx, logos_comm* comm, const void* local, int B, int H_local, size_t row_bytes) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::comm_push(ctx, comm, local, B, H_local, row_bytes);
}

int logos_comm_wait(logos_ctx* ctx, logos_comm* comm, void* gathered, size_t bytes) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::comm_wait(ctx, comm, gathered, bytes);
}

int logos_comm_all_gather_heads(logos_ctx* ctx, logos_comm* comm, const void* local, void* gathered, int B,
                                int H_local, size_t row_bytes) {
    if (!ctx || !comm) return LOGOS_ERR_INVALID_ARG;
    int rc = logos::comm_push(ctx, comm, local, B, H_local, row_bytes);
    if (rc != LOGOS_OK) return rc;
    return logos::comm_wait(ctx, comm, gathered, (size_t)B * H_local * comm->world * row_bytes);
}

}  // extern "C"
