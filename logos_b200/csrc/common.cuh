// common.cuh -- context object, error plumbing and small device helpers shared by
// the kernels of the attention engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/logos_attn.h"

struct logos_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    void* workspace = nullptr;        // scratch used by hot calls
    size_t workspace_bytes = 0;
    bool owns_workspace = false;
    float* absmax_scratch = nullptr;  // per-tensor absmax words for kv_quantize
    int absmax_slots = 0;
    int* tc_status = nullptr;         // device word raised by a kernel whose bounded wait ran out
    bool force_general = false;       // LOGOS_OPT_FORCE_GENERAL: never use the tensor-core kernels
    int decode_chunk = 0;             // LOGOS_OPT_DECODE_CHUNK: 0 = chosen from the problem size
    int peer_wait_ms = 2000;          // LOGOS_OPT_PEER_WAIT_MS
    bool workspace_locked = false;    // LOGOS_OPT_WORKSPACE_LOCK
    bool gemm_narrow = false;         // LOGOS_OPT_GEMM_NARROW
    int decode_depth = 0;             // LOGOS_OPT_DECODE_DEPTH
    bool qkv_out_f16 = false;         // LOGOS_OPT_QKV_OUT_F16
    bool project_overlap = false;     // LOGOS_OPT_PROJECT_OVERLAP
    logos_alloc_fn alloc_fn = nullptr;   // caller's allocator for the workspace (null: cudaMalloc / cudaFree)
    logos_free_fn free_fn = nullptr;
    void* alloc_user = nullptr;
    logos_free_fn ws_free_fn = nullptr;  // how the current workspace block is given back (null: cudaFree)
    void* ws_free_user = nullptr;
    const void* smem_set[48] = {};    // kernels whose dynamic shared-memory limit this context has raised
    int smem_set_n = 0;
    char err[512] = {0};
};

// Heads spread over several GPUs: where a finished decode row goes.  Every rank owns one block of
// device memory that its peers can write (logos_comm).  A row is stored into the row area of EVERY
// rank, each value as one 8-byte word {value bits, step + 1}: an aligned 8-byte store arrives whole,
// so the word is its own arrival flag and the sender needs no fence, no counter and no second
// message; the receiving kernel polls the words themselves (collect_rows_kernel in comm.cu).
constexpr int kMaxPeers = 8;
struct PeerEpilogue {
    uint2* rows[kMaxPeers];       // row area of each rank: two slots of slot_words words (step parity)
    const unsigned* step;         // this rank's step counter (advanced by the collecting kernel)
    size_t slot_words;
    int world;                    // 0: no peers, rows go to DecodeArgs::out
    int H_total, head0;           // heads of the whole model, first head of this rank
};

struct logos_comm {
    logos_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    size_t slot_bytes = 0;                 // bytes of one gathered tensor, rounded up to 256
    size_t row_slot_bytes = 0;             // bytes of one slot of the row area: 8 per fp32 value
    unsigned char* block = nullptr;        // this rank's block (cudaMalloc)
    unsigned char* peer[kMaxPeers] = {};   // every rank's block as seen from this device (peer[rank] == block)
    void* ipc_base[kMaxPeers] = {};        // what cudaIpcOpenMemHandle returned for a peer (to be closed)
    bool connected = false;
};

namespace logos {

// layout of a logos_comm block
constexpr size_t kCommFlagStride = 128;    // one flag word per source rank, a cache line apart
constexpr size_t kCommStepOff = 1024;      // step counter, then the two completion counters
constexpr size_t kCommDoneOff = 1028;
constexpr size_t kCommCopyDoneOff = 1032;
constexpr size_t kCommMagicOff = 1040;     // 8-byte mark written at hand-out, checked by peers after mapping
constexpr size_t kCommStageOff = 4096;
constexpr size_t kCommRowSlotMax = 2u << 20;   // bytes of one row-area slot at most (2 x 1 MiB of fp32 rows)

inline int fail(logos_ctx* ctx, int status, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return status;
}

#define LOGOS_CUDA_TRY(ctx, expr)                                                         \
    do {                                                                                  \
        cudaError_t e__ = (expr);                                                         \
        if (e__ != cudaSuccess)                                                           \
            return ::logos::fail((ctx), LOGOS_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,   \
                                 cudaGetErrorString(e__), __FILE__, __LINE__);            \
    } while (0)

#define LOGOS_LAUNCH_CHECK(ctx, what)                                                     \
    do {                                                                                  \
        cudaError_t e__ = cudaGetLastError();                                             \
        if (e__ != cudaSuccess)                                                           \
            return ::logos::fail((ctx), LOGOS_ERR_CUDA, "launch of %s failed: %s", what,  \
                                 cudaGetErrorString(e__));                                \
    } while (0)

// Raises a kernel's dynamic shared-memory limit once per context (not before every launch: the
// attribute call costs more than a short kernel).  `bytes` must be the most the kernel is ever given.
template <typename Fn>
inline int ensure_smem_limit(logos_ctx* ctx, Fn* kernel, int bytes) {
    const void* key = reinterpret_cast<const void*>(kernel);
    for (int i = 0; i < ctx->smem_set_n; ++i)
        if (ctx->smem_set[i] == key) return LOGOS_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess)
        return fail(ctx, LOGOS_ERR_CUDA, "cudaFuncSetAttribute(%d bytes) failed: %s", bytes, cudaGetErrorString(e));
    if (ctx->smem_set_n < 48) ctx->smem_set[ctx->smem_set_n++] = key;
    return LOGOS_OK;
}

// Programmatic dependent launch.  A kernel launched with launch_overlapped() may begin as soon as every
// CTA of the kernel before it on the stream has passed grid_release_dependents() (or exited); what that
// earlier kernel wrote is only safe to read after grid_wait_for_earlier().  Both calls do nothing in a
// kernel that was launched the ordinary way, and everything older than the previous kernel is complete
// and visible as usual.
__device__ __forceinline__ void grid_release_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_wait_for_earlier() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The first 64 KiB of a context's workspace are the split-K arrival counters of the decode kernel.  They are
// zero whenever no decode kernel is running (cleared when the block is attached, put back to zero by the
// kernel itself); every other user of the workspace starts beyond them.
constexpr size_t kWorkspaceCounterBytes = 64 * 1024;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

inline size_t dtype_size(int dt) { return dt == LOGOS_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == LOGOS_F32 || dt == LOGOS_BF16 || dt == LOGOS_F16; }

// Rule switch shared by every kernel: Shunyam sparsity applies only to sequences
// longer than the window (include/Attention.hpp:228, cuda/ModelGPU.cu:966).
__host__ __device__ inline bool shunyam_active(int window, int seq) {
    return window > 0 && seq > window;
}

// allowed(i,j) = j <= i (if causal) and (j >= i - window or j % stride == 0)
// (cuda/VedicGEMM.cu:987-996, include/Attention.hpp:88-96).
__device__ __forceinline__ bool key_allowed(int i, int j, bool causal, bool shunyam, int window,
                                            int stride) {
    if (causal && j > i) return false;
    if (shunyam) {
        bool in_window = (j >= i - window) && (j <= i);
        bool landmark = (stride > 0) && (j % stride == 0);
        if (!in_window && !landmark) return false;
    }
    return true;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace logos

// Kernel-side entry points implemented in the other translation units.
namespace logos {
int kv_quantize(logos_ctx*, int, const void*, int64_t, int8_t*, int64_t, float*, int, int64_t,
                const float* absmax_known = nullptr);
int project(logos_ctx*, int dtype, int out_dtype, const void* A, const void* Wt, const void* residual, void* C,
            int M, int N, int K);
int decode_generic(logos_ctx*, const void* q, const void* q_prev, const int8_t*, const int8_t*, const float*,
                   const float*, const int32_t* len, int B, int H, int S_max, int DH, const logos_attn_params*, float* out);
int attention_bwd_adjoint(logos_ctx*, const float* dQa, const float* dVs, float* dQ, float* dV, int S, int DH, float eta,
                          float nu, int mode, int ns, int accumulate, int64_t total);
size_t attention_bwd16_workspace_bytes(int B, int H, int S, int DH);
int attention_bwd16(logos_ctx*, int dtype, const void* Q, const void* K, const void* V, const void* dO, float* dQ, float* dK,
                    float* dV, int B, int H, int S, int DH, const logos_attn_params*);
size_t attention_bwd_workspace_bytes(int B, int H, int S, int DH);
int attention_bwd(logos_ctx*, const float* Q, const float* K, const float* V, const float* dO, float* dQ, float* dK,
                  float* dV, int B, int H, int S, int DH, const logos_attn_params*);
int gemm_f32(logos_ctx*, const float* A, int lda, int64_t strideA, const float* B, int ldb, int64_t strideB, float* C,
             int ldc, int64_t strideC, int M, int N, int K, int batch);
int project_heads(logos_ctx*, int dtype, int out_dtype, const void* head_out, const void* Wt, const void* residual,
                  void* C, int B, int S, int H, int N);
int kv_dequantize16(logos_ctx*, int dst_dtype, const int8_t*, int64_t, const float*, void*, int64_t, int, int64_t);
int qkv_project(logos_ctx*, int dtype, const void* X, const void* Wt, void* Q, void* K, void* V, int B, int S,
                int H, int D, float* k_absmax, float* v_absmax);
int kv_dequantize(logos_ctx*, const int8_t*, int64_t, const float*, float*, int64_t, int, int64_t);
// pos_bias is added to every pos[b]: -1 appends at len - 1 when `pos` is the length after the append
int kv_append(logos_ctx*, int, const void*, const void*, int8_t*, int8_t*, const float*,
              const float*, const int32_t* pos, int, int, int, int, int pos_bias = 0);
// out_dtype: the type of the rows written to `out` without peers (LOGOS_F32, or 16 bits for the projection after it)
int decode_int8(logos_ctx*, const void*, const void*, const int8_t*, const int8_t*, const float*,
                const float*, const int32_t*, int, int, int, int, const logos_attn_params*,
                float*, const PeerEpilogue* peer = nullptr, bool follows_append = false, int out_dtype = LOGOS_F32,
                const void* append_k = nullptr, const void* append_v = nullptr);
// true when decode_int8 takes the new token's rows itself (append_k / append_v): the window kernel at DH = 64
bool decode_appends_itself(const logos_attn_params* p, int DH);
size_t decode_workspace_bytes(int B, int H, int S_max, int DH);
int layer_norm(logos_ctx*, int dtype, const void* X, const float* gamma, const float* beta, void* Y, int rows, int D,
               float eps);
int attention_simt(logos_ctx*, int in_dtype, int out_dtype, const void* Q, const void* K,
                   const void* V, void* O, int B, int H, int S, int DH,
                   const logos_attn_params*, const logos_strides* in = nullptr, const logos_strides* out = nullptr);
bool attention_window_eligible(int in_dtype, int out_dtype, int DH, const logos_attn_params* p, int S);
int attention_window(logos_ctx*, int in_dtype, int out_dtype, const void* Q, const void* K, const void* V,
                     void* O, int B, int H, int S, int DH, const logos_attn_params*);
int umma_selftest(logos_ctx*, int mode, int dtype, const void* A, const void* B, float* D);
bool attention_tc_eligible(int in_dtype, int out_dtype, int DH, const logos_attn_params* p, int S);
int attention_tc(logos_ctx*, int in_dtype, int out_dtype, const void* Q, const void* K, const void* V,
                 void* O, int B, int H, int S, int DH, const logos_attn_params*, const logos_strides* in = nullptr,
                 const logos_strides* out = nullptr);
void comm_peer_epilogue(const logos_comm* c, int H_local, PeerEpilogue* out);
int comm_wait(logos_ctx*, logos_comm*, void* gathered, size_t bytes);
int comm_collect_rows(logos_ctx*, logos_comm*, float* gathered, int B, int H_total, int DH,
                      bool follows_decode = false);
int comm_push(logos_ctx*, logos_comm*, const void* local, int B, int H_local, size_t row_bytes);
}  // namespace logos
