/*
 * logos_attn.h -- C ABI of the B200 (sm_100a) attention engine for LOGOS.
 *
 * Scope: the multi-head-attention hot path of the LOGOS model -- causal
 * prefill attention, Shunyam window(+landmark) attention, the Nikhilam INT8
 * KV cache (quantize, append, decode) and the Navier-Stokes Q-advection /
 * V-diffusion prologue.  Each entry point names the reference interface it
 * stands in for (paths relative to the LOGOS source tree).
 *
 * Conventions (they follow the reference call site, cuda/ModelGPU.cu:892-988):
 *  - all tensor pointers are DEVICE pointers unless the name ends in _host;
 *  - the caller owns every buffer; the engine never frees or keeps them;
 *  - work is issued on the context's stream (default: the legacy default
 *    stream, as in the reference) and is NOT synchronised before return,
 *    except for the *_host entry points which return finished results;
 *  - every function returns a logos_status; no C++ exception crosses the ABI;
 *  - hot calls never allocate: scratch comes from the context's workspace
 *    (logos_ctx_reserve / logos_ctx_set_workspace).
 * There is no CPU fallback: without a CUDA device the context cannot be
 * created and every call fails with LOGOS_ERR_NO_DEVICE.
 */
#ifndef LOGOS_ATTN_H
#define LOGOS_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LOGOS_ATTN_ABI_VERSION 1

typedef struct logos_ctx logos_ctx;

typedef enum {
    LOGOS_OK = 0,
    LOGOS_ERR_INVALID_ARG = 1,   /* null pointer, non-positive extent, bad enum      */
    LOGOS_ERR_UNSUPPORTED = 2,   /* valid request the engine does not implement      */
    LOGOS_ERR_WORKSPACE = 3,     /* context workspace too small for this call        */
    LOGOS_ERR_CUDA = 4,          /* a CUDA runtime call or launch failed             */
    LOGOS_ERR_NO_DEVICE = 5,     /* no usable sm_100 device                          */
    LOGOS_ERR_ALIGNMENT = 6,     /* pointer or extent breaks a 16-byte requirement   */
    LOGOS_ERR_SCRATCH_LIMIT = 7, /* request exceeds the fixed scratch of
                                    logos_decode_int8_noalloc                        */
    LOGOS_ERR_KERNEL_TIMEOUT = 8 /* a bounded wait inside a kernel ran out           */
} logos_status;

typedef enum { LOGOS_F32 = 0, LOGOS_BF16 = 1, LOGOS_F16 = 2 } logos_dtype;

/* V-diffusion variant.  CAUSAL is the GPU model's one-sided stencil
 * (cuda/ModelGPU.cu:463-471); CENTRAL is the CPU model's two-sided stencil with
 * mirror boundaries (include/Attention.hpp:173-181). */
typedef enum { LOGOS_DIFFUSE_NONE = 0, LOGOS_DIFFUSE_CAUSAL = 1, LOGOS_DIFFUSE_CENTRAL = 2 } logos_diffuse;

/* The attention-related fields of GPUPhysicsConfig (cuda/ModelGPU.cuh:67-82)
 * and of AttentionHead (include/Attention.hpp:205-214). */
typedef struct {
    float scale;        /* score multiplier, 1/sqrt(DH) at the reference call site        */
    int   causal;       /* 1: key j > query i is masked                                    */
    int   window;       /* Shunyam window; the rule is active iff window > 0 && seq > window
                           (include/Attention.hpp:228, cuda/ModelGPU.cu:966)               */
    int   stride;       /* Shunyam landmark stride (every j % stride == 0 is visible);
                           <= 0 means no landmarks, a pure sliding window                  */
    float ns_eta;       /* Q-advection strength, Q_adv[i] = Q[i] + eta (Q[i] - Q[i-1])     */
    float ns_nu;        /* V-diffusion viscosity (used when diffuse_mode != NONE)          */
    float ns_alpha;     /* out = (1-alpha) standard + alpha NS; 1 = the GPU model, 0 = off */
    int   diffuse_mode; /* logos_diffuse                                                   */
} logos_attn_params;

/* ---- context ------------------------------------------------------------ */

int logos_abi_version(void);
const char* logos_status_string(int status);

/* Binds to CUDA device `device` (must be compute capability 10.x). */
int logos_ctx_create(int device, logos_ctx** out);
int logos_ctx_destroy(logos_ctx* ctx);
/* cudaStream_t as void*; NULL selects the legacy default stream (reference behaviour:
 * every launch in cuda/ModelGPU.cu and cuda/VedicGEMM.cu is on stream 0). */
int logos_ctx_set_stream(logos_ctx* ctx, void* cuda_stream);
/* Grows the context-owned workspace to at least `bytes` (cudaMalloc; not a hot call).  Growing frees
 * the old block: see LOGOS_OPT_WORKSPACE_LOCK when captured graphs use it. */
int logos_ctx_reserve(logos_ctx* ctx, size_t bytes);
/* The allocator logos_ctx_reserve takes the workspace from, for hosts whose memory pool owns the device
 * (null functions restore cudaMalloc / cudaFree).  alloc returns 0 and a 256-byte aligned device pointer,
 * or non-zero; then logos_ctx_reserve fails with LOGOS_ERR_WORKSPACE and the context keeps the
 * workspace it had.  A block is always released through the free function that was current when it
 * was allocated. */
typedef int (*logos_alloc_fn)(void** device_ptr, size_t bytes, void* user);
typedef void (*logos_free_fn)(void* device_ptr, void* user);
int logos_ctx_set_allocator(logos_ctx* ctx, logos_alloc_fn alloc, logos_free_fn free_fn, void* user);
/* Uses caller memory as workspace instead (256-byte aligned device memory). */
int logos_ctx_set_workspace(logos_ctx* ctx, void* device_ptr, size_t bytes);
/* Waits for the context's stream and reports LOGOS_ERR_KERNEL_TIMEOUT if a kernel gave up
 * on one of its bounded internal waits since the last check (its output is then invalid).
 * The reference has no such channel: its kernels have no internal waits. */
int logos_ctx_synchronize(logos_ctx* ctx);
/* Text of the last failure on this context (owned by the context). */
const char* logos_last_error(const logos_ctx* ctx);

/* Switches of a context; they replace what the reference reads from GPUPhysicsConfig at build time
 * (cuda/ModelGPU.cuh:67-82) and are never read from the environment.
 *   LOGOS_OPT_FORCE_GENERAL  1: every attention call takes the exact fp32 kernel (tests compare the
 *                            tensor-core kernels with it); 0 (default): normal dispatch.
 *   LOGOS_OPT_DECODE_CHUNK   keys per split of the dense decode kernel: a multiple of 64 from 128 to 1024;
 *                            0 (default) = chosen from the problem size.  Results of two calls are
 *                            bit-identical only when they use the same chunk.
 *   LOGOS_OPT_PEER_WAIT_MS   longest time a kernel waits for the other GPUs of a logos_comm before it
 *                            gives up and raises LOGOS_ERR_KERNEL_TIMEOUT (default 2000).
 *   LOGOS_OPT_WORKSPACE_LOCK 1: logos_ctx_reserve / logos_ctx_set_workspace calls that would replace
 *                            the workspace fail with LOGOS_ERR_WORKSPACE.  A CUDA graph captured from
 *                            decode calls holds the workspace's address: lock it for as long as such
 *                            a graph can still be launched.
 *   LOGOS_OPT_GEMM_NARROW    1: the projections always take the 128 x 128-tile kernel; 0 (default): the
 *                            persistent 128 x 256-tile kernel whenever the problem fills the device.
 *                            The two give bit-identical results (same products, same order of k).
 *   LOGOS_OPT_DECODE_DEPTH   tiles of 32 keys a warp of the dense decode kernel holds at once: 2 or 4;
 *                            0 (default) = 4 when the launch is a single wave of CTAs, else 2.  The
 *                            arithmetic and its order do not depend on it.
 *   LOGOS_OPT_QKV_OUT_F16    1: logos_qkv_project stores Q, K and V as FP16 whatever the operand type
 *                            (the decode entry points take FP16: a BF16 model's decode step then needs no
 *                            conversion pass); the max|x| tables are those of the stored FP16 values.
 *   LOGOS_OPT_PROJECT_OVERLAP 1: a projection of at most 32 rows (a decode step's) is launched to overlap the
 *                            kernel before it on the stream: it fetches its weight tiles while that kernel
 *                            still runs and waits for it before it touches A, the residual or any output.
 *                            The caller promises that the kernel before such a call does not write the
 *                            weights.  0 (default): ordinary launches. */
typedef enum { LOGOS_OPT_FORCE_GENERAL = 0, LOGOS_OPT_DECODE_CHUNK = 1, LOGOS_OPT_PEER_WAIT_MS = 2,
               LOGOS_OPT_WORKSPACE_LOCK = 3, LOGOS_OPT_GEMM_NARROW = 4, LOGOS_OPT_DECODE_DEPTH = 5,
               LOGOS_OPT_QKV_OUT_F16 = 6, LOGOS_OPT_PROJECT_OVERLAP = 7 } logos_option;
int logos_ctx_set_option(logos_ctx* ctx, int option, int value);

/* ---- attention ---------------------------------------------------------- */

/* Stand-in for cuda_flash_attention_fwd (cuda/VedicGEMM.cuh:236-243,
 * cuda/VedicGEMM.cu:1065-1104): one head, fp32 row-major [seq x DH] device
 * tensors, DH <= 128.  attn_ptr must be NULL (the reference forward never passes
 * anything else, cuda/ModelGPU.cu:935,962); non-NULL returns LOGOS_ERR_UNSUPPORTED.
 * `shunyam` is the caller's already-evaluated "rule active" flag, as in the reference. */
int logos_flash_attention_fwd_f32(logos_ctx* ctx, const float* Q, const float* K, const float* V,
                                  float* out, float* attn_ptr, int seq, int DH, float scale,
                                  int causal, int shunyam, int window, int stride);

/* Batched attention over B*H independent heads with the Navier-Stokes prologue
 * fused in.  Replaces, per head, ns_advect_kernel + ns_diffuse_kernel
 * (cuda/ModelGPU.cu:443-471) + cuda_flash_attention_fwd, and on the CPU side the
 * attention part of AttentionHead::forward (include/Attention.hpp:225-265).
 * Q,K,V: [B][H][S][DH] contiguous, dtype `in_dtype`; O: same shape, dtype `out_dtype`
 * (the input dtype or LOGOS_F32). */
int logos_attention_fwd(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                        const void* V, void* O, int B, int H, int S, int DH,
                        const logos_attn_params* params);
size_t logos_attention_workspace_bytes(int B, int H, int S, int DH);

/* logos_attention_fwd on tensors that are not packed [B][H][S][DH]: element strides between two sequences,
 * two heads and two rows; the DH values of a row are contiguous.  `qkv` describes Q, K and V (one layout for
 * the three, as one projection writes them), `out` describes O; NULL = packed.  Examples: token-major
 * [B][S][H][DH] is {S*H*DH, DH, H*DH}; one head of a packed tensor is the packed strides with a shifted base.
 * Same kernels, same results bit for bit as the packed call on the same values.  For 16-bit tensors every row
 * must start on a 16-byte boundary (strides multiples of 8 elements); when the sequences' slabs are not evenly
 * spaced (batch != H * head, B > 1) the tensor-core kernel is launched once per sequence. */
typedef struct { int64_t batch, head, row; } logos_strides;
int logos_attention_fwd_strided(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                                const void* V, void* O, int B, int H, int S, int DH,
                                const logos_strides* qkv, const logos_strides* out,
                                const logos_attn_params* params);

/* Attention backward: dQ, dK, dV of logos_attention_fwd's output with respect to its raw Q, K, V, for the
 * gradient dO of that output; all tensors fp32 [B][H][S][DH], DH 32, 64 or 128, 16-byte aligned.
 * Replaces, for all heads at once and without any seq x seq buffer, the per-head chain of
 * run_backward (cuda/train_gpu.cu:657-748: recompute of the probabilities, attn_dV_kernel,
 * attn_dAttnProbs_kernel, softmax_bwd_kernel, attn_dQ_kernel, attn_dK_kernel, :422-481) together with
 * ns_diffuse_bwd_kernel and ns_advect_bwd_kernel (cuda/ModelGPU.cu:453-482).  `params` is the forward's:
 * the mask that was applied in the forward is applied here (the reference's recompute uses the causal
 * mask whatever the forward did), every diffuse_mode and 0 < ns_alpha < 1 included.  Sums have a fixed
 * order: the result is reproducible bit for bit.  Workspace from the context
 * (logos_attention_bwd_workspace_bytes / logos_ctx_reserve). */
size_t logos_attention_bwd_workspace_bytes(int B, int H, int S, int DH);
int logos_attention_bwd(logos_ctx* ctx, const float* Q, const float* K, const float* V, const float* dO,
                        float* dQ, float* dK, float* dV, int B, int H, int S, int DH,
                        const logos_attn_params* params);

/* The same gradients on the tensor cores: Q, K, V, dO in `dtype` (BF16 or FP16) [B][H][S][64], dQ, dK, dV
 * fp32; every product a tcgen05 MMA with fp32 accumulation, the probabilities recomputed per 128 x 128 tile
 * and handed to the next product as 16-bit operands (so results carry the 16-bit rounding of the weights:
 * about 1e-2 of the largest gradient in BF16, 2e-3 in FP16).  Same `params` rules as logos_attention_bwd.
 * Workspace from the context (logos_attention_bwd16_workspace_bytes / logos_ctx_reserve). */
size_t logos_attention_bwd16_workspace_bytes(int B, int H, int S, int DH);
int logos_attention_bwd16(logos_ctx* ctx, int dtype, const void* Q, const void* K, const void* V, const void* dO,
                          float* dQ, float* dK, float* dV, int B, int H, int S, int DH,
                          const logos_attn_params* params);

/* Prefill of one layer in one call: logos_attention_fwd, and before it -- when k_cache is non-NULL --
 * the layer's INT8 cache filled from the raw K and V.  This is the order of ModelGPU::forward, which
 * quantises a head's K and V (cuda/ModelGPU.cu:908) before the Navier-Stokes prologue and the attention
 * (cuda/ModelGPU.cu:915-968), done here for all heads at once.
 * k_cache, v_cache: int8 [B][H][S_max][DH], rows [0, S) of every (b, h) tensor are written;
 * k_scale, v_scale: float [B][H].  The four are given together or all NULL; S <= S_max.
 * Bytes and scales are those of logos_kv_quantize, the output that of logos_attention_fwd. */
int logos_prefill_fwd(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                      const void* V, void* O, int B, int H, int S, int DH,
                      const logos_attn_params* params, int8_t* k_cache, int8_t* v_cache,
                      float* k_scale, float* v_scale, int S_max);

/* Hardware bring-up check of the tensor-core building blocks (TMA tile load with 128-byte
 * swizzle, tcgen05.mma from shared-memory descriptors, TMEM read-back) on one 128-row tile;
 * no counterpart in the reference.  dtype: LOGOS_BF16 or LOGOS_F16.
 *   mode 0: D[128][128] = A[128][64] * B[128][64]^T        (the S = Q K^T operand layouts)
 *   mode 1: D[128][64]  = A[128][128] * B[128][64]         (the O = W V operand layouts)
 *   mode 2: issues no load, so the kernel's bounded wait runs out and it returns: the following
 *           logos_ctx_synchronize must report LOGOS_ERR_KERNEL_TIMEOUT (D is not written)
 *   mode 3: as mode 1 with A held in tensor memory (the way the prefill kernel passes W)
 *   mode 16 + m (m = 0, 1, 3): a timing run -- the MMAs of mode m (4, 8, 8 of them) issued 32 times back to back;
 *           D[0] receives the clock cycles they took, the rest of D is not meaningful
 *   mode 48 + m: the same timing run with a whole warp running the issue loop and one elected lane issuing
 * D is fp32, row-major.  Check the result with logos_ctx_synchronize. */
int logos_selftest_umma(logos_ctx* ctx, int mode, int dtype, const void* A, const void* B, float* D);

/* ---- Nikhilam INT8 KV cache --------------------------------------------- */

/* Stand-in for nikhilam_compress (cuda/ModelGPU.cu:357-386: absmax_kernel,
 * scale = (absmax + 1e-8) / 127.5, nikhilam_quantize_kernel), batched over
 * n_tensors tensors of `elems` values each with ONE scale per tensor and no host
 * round-trip.  Tensor t is read at src + t*src_stride elements and written at
 * dst + t*dst_stride bytes; scales[t] receives the fp32 scale.  Bytes and scales
 * are bit-identical to the reference arithmetic (IEEE division, round-half-even). */
int logos_kv_quantize(logos_ctx* ctx, int src_dtype, const void* src, int64_t src_stride,
                      int8_t* dst, int64_t dst_stride, float* scales, int n_tensors,
                      int64_t elems);

/* logos_kv_quantize without its first pass: absmax[t] = max|x| of tensor t is already known (the
 * projection GEMM below reduces it in its epilogue, over exactly the values it stored).  Same bytes
 * and scales as logos_kv_quantize on the same tensors. */
int logos_kv_quantize_absmax(logos_ctx* ctx, int src_dtype, const void* src, int64_t src_stride,
                             int8_t* dst, int64_t dst_stride, const float* absmax, float* scales,
                             int n_tensors, int64_t elems);

/* Stand-in for nikhilam_decompress / nikhilam_dequantize_kernel
 * (cuda/ModelGPU.cu:343-351,388-395): dst = (float)q * scale. */
int logos_kv_dequantize(logos_ctx* ctx, const int8_t* src, int64_t src_stride, const float* scales,
                        float* dst, int64_t dst_stride, int n_tensors, int64_t elems);

/* Quantize-on-append: writes the new token's K and V rows ([B][H][DH], dtype
 * `dtype`) into the caches ([B][H][S_max][DH] int8) at row pos[b], using the
 * scales already stored for each (b,h) tensor and saturating at +-127 -- the
 * contract of nikhilam_quantize_kernel (cuda/ModelGPU.cu:329-340) applied to one
 * row.  The reference has no incremental path (cuda/train_gpu.cu:2037-2046). */
int logos_kv_append(logos_ctx* ctx, int dtype, const void* k_new, const void* v_new,
                    int8_t* k_cache, int8_t* v_cache, const float* k_scale, const float* v_scale,
                    const int32_t* pos, int B, int H, int S_max, int DH);

/* Decode attention straight from the INT8 cache: for every (b,h) the query is the
 * token at position len[b]-1 (already appended), K/V rows [0,len[b]) are streamed
 * as int8, dequantized in registers with their per-tensor scales, and the last
 * row of the attention defined by `params` is produced.  q, q_prev: FP16
 * [B][H][DH] (q_prev = the previous token's query, needed by the advection term;
 * may be NULL when ns_eta == 0).  out: FP32 [B][H][DH].  Replaces the full
 * re-forward per generated token of cuda/train_gpu.cu:2037-2046; numerically it
 * is nikhilam_decompress + ns kernels + the last row of cuda_flash_attention_fwd.
 * DH = 64 (the model's) runs the split-K kernels; any other multiple of 16 up to 128 (the reference's
 * attention takes DH <= 128, cuda/VedicGEMM.cu:899) runs a general fp32 kernel, one CTA per (b,h), with
 * the context bounded by shared memory (S_max <= about 50 000, half of that when 0 < ns_alpha < 1). */
int logos_decode_int8(logos_ctx* ctx, const void* q, const void* q_prev, const int8_t* k_cache,
                      const int8_t* v_cache, const float* k_scale, const float* v_scale,
                      const int32_t* len, int B, int H, int S_max, int DH,
                      const logos_attn_params* params, float* out);
size_t logos_decode_workspace_bytes(int B, int H, int S_max, int DH);

/* One whole decode step on device buffers: the new token's K and V rows (FP16 [B][H][DH]) are
 * quantised into row len[b]-1 of the caches (logos_kv_append with pos = len - 1), then
 * logos_decode_int8 runs over rows [0, len[b]).  len is the length AFTER the append.  Two
 * launches, nothing else (one with a window at DH = 64: that kernel quantises the new rows itself, with the
 * same arithmetic); this is the per-layer body of an incremental generate loop, which the
 * reference does not have (cuda/train_gpu.cu:2037-2046 re-runs the whole forward per token). */
int logos_decode_step_int8(logos_ctx* ctx, const void* q, const void* q_prev, const void* k_new,
                           const void* v_new, int8_t* k_cache, int8_t* v_cache, const float* k_scale,
                           const float* v_scale, const int32_t* len, int B, int H, int S_max, int DH,
                           const logos_attn_params* params, float* out);
/* The same with the rows stored in out_dtype (LOGOS_F32, LOGOS_BF16, LOGOS_F16): a 16-bit `out` is the A operand
 * of the W_O projection after it (logos_project), with no conversion pass between them.  DH = 64. */
int logos_decode_step_int8_to(logos_ctx* ctx, const void* q, const void* q_prev, const void* k_new,
                              const void* v_new, int8_t* k_cache, int8_t* v_cache, const float* k_scale,
                              const float* v_scale, const int32_t* len, int B, int H, int S_max, int DH,
                              const logos_attn_params* params, int out_dtype, void* out);

/* One whole decode step with HOST buffers for the per-step data: copies q, q_prev,
 * k_new, v_new (FP16 [B][H][DH]) and len (int32 [B], the length AFTER the append)
 * to the device, appends at row len[b]-1, runs logos_decode_int8 and copies the
 * FP32 result back to out_host; returns when out_host is complete.  The caches
 * and scales stay resident on the device (they are engine state, like HeadCache in
 * cuda/ModelGPU.cuh:42-49).  Staging memory comes from the workspace.  Host tensors that lie
 * one after the other in memory in the order q, q_prev, k_new, v_new, len are sent as one copy. */
int logos_decode_step_int8_host(logos_ctx* ctx, const void* q_host, const void* q_prev_host,
                                const void* k_new_host, const void* v_new_host,
                                int8_t* k_cache, int8_t* v_cache, const float* k_scale,
                                const float* v_scale, const int32_t* len_host, int B, int H,
                                int S_max, int DH, const logos_attn_params* params,
                                float* out_host);

/* Dense INT8-KV decode for callers that cannot allocate device memory when they
 * decode -- a host that gave the whole device to its own memory pool, a serving loop
 * that forbids allocation after start-up, or an embedding that never creates a
 * logos_ctx (creating one allocates).  It has no counterpart in the reference.
 * Same arguments and result as logos_decode_int8 with params->window == 0, but no
 * context: work goes to `cuda_stream` (cudaStream_t as void*, NULL = default stream)
 * on the CURRENT device, and the split-K scratch is a fixed 4.3 MB array inside the
 * library (held by every GPU that loads it until the process exits) instead of a
 * workspace.  Limits: B*H <= 4096 pairs and B*H * key-splits * (2 if 0 < ns_alpha < 1
 * else 1) <= 16384 partial records, where key-splits = ceil(S_max / chunk) and chunk is
 * between 128 and 1024 keys (64 x 16 x 8192 needs 8192 records); larger requests return
 * LOGOS_ERR_SCRATCH_LIMIT, window > 0 returns LOGOS_ERR_UNSUPPORTED.  The call makes no
 * cudaMalloc / cudaFree and uses no allocating library routine.  The first call on a
 * device looks up the array's device address; make that first call before any stream
 * capture.  That first call is also where the CUDA runtime may load this library's
 * device code into the device (kernel images and the array itself, if nothing of the
 * library ran there before): the runtime takes device memory for it at that moment,
 * and fails if none is left.  A caller whose pool will own the whole device therefore
 * makes one warm-up call at start-up, before the pool takes the device; from the
 * second call on no device memory moves.  All calls share the one array and it keeps the previous call's contents
 * (the call clears the counters it needs on its stream), so calls that overlap on a
 * GPU -- two streams, two threads -- race: issue them on one stream, one at a time. */
int logos_decode_int8_noalloc(void* cuda_stream, const void* q, const void* q_prev,
                              const int8_t* k_cache, const int8_t* v_cache, const float* k_scale,
                              const float* v_scale, const int32_t* len, int B, int H, int S_max,
                              int DH, const logos_attn_params* params, float* out);

/* ---- projections either side of the attention ---------------------------- */

/* The reference projects head by head: three [seq x d]·[d x 64] GEMMs per head for Q, K, V
 * (cuda/ModelGPU.cu:899-906, amp_gemm -> cuda_gemm_fp16_fp32out, cuda/MixedPrecision.cuh:301-330, on
 * the FP16 shadow of the weights, cuda/MixedPrecision.cuh:149-161), one [seq x 64]·[64 x d] per head
 * summed into `concat` (cuda/ModelGPU.cu:974-988), one [seq x d]·[d x d] for W_proj (:990-1015).  Here:
 *
 * logos_qkv_project -- all heads' Q, K and V of a layer in ONE tensor-core GEMM, X [B*S][D_model] times
 *   the stacked weights, written straight into the attention layout [B][H][S][64] (same 16-bit dtype as
 *   X).  Wt_qkv is the K-major 16-bit shadow of the stacked weight: row n = (which * H + h) * 64 + c holds
 *   column c of W_Q[h] (which 0), W_K[h] (1) or W_V[h] (2), i.e. Wt_qkv[n][k] = W[k][c].  With k_absmax /
 *   v_absmax (float [B][H], both or neither) the epilogue also leaves max|x| of every stored K and V
 *   tensor there, ready for logos_kv_quantize_absmax.  DH is 64; D_model a multiple of 8.
 *   Operands 16-byte aligned; outputs (Q, K, V, C) and the residual 32-byte aligned (they are written and read 32
 *   bytes per thread and instruction).
 *
 * logos_project -- C [M][N] = A [M][K] · W (+ residual [M][N]), A and the K-major shadow Wt [N][K] in
 *   one 16-bit dtype, C and the residual in out_dtype (that dtype or LOGOS_F32).  With the heads'
 *   outputs laid side by side ([M][H*64]) and W_O[h] stacked along K it is the reference's sum over
 *   heads; with W_proj it is the output projection plus the residual add that follows it. */
int logos_qkv_project(logos_ctx* ctx, int dtype, const void* X, const void* Wt_qkv, void* Q, void* K, void* V,
                      int B, int S, int H, int D_model, float* k_absmax, float* v_absmax);
int logos_project(logos_ctx* ctx, int dtype, int out_dtype, const void* A, const void* Wt, const void* residual,
                  void* C, int M, int N, int K);

/* logos_project_heads -- logos_project whose A operand is the attention's own output, still head-major
 *   ([B][H][S][64], what logos_attention_fwd writes): C [B*S][N] = sum over heads of head_out[b][h] ·
 *   W_O[h] (+ residual), Wt_o [N][H*64] K-major.  The kernel fetches head h's rows as k block h, so the
 *   per-token concatenation of the head outputs (include/Attention.hpp:292-299, cuda/ModelGPU.cu:974-988)
 *   never exists in memory. */
int logos_project_heads(logos_ctx* ctx, int dtype, int out_dtype, const void* head_out, const void* Wt_o,
                        const void* residual, void* C, int B, int S, int H, int N);

/* The LayerNorm in front of a layer's projections (layernorm_kernel, cuda/VedicGEMM.cu:157-199; per layer at
 * cuda/ModelGPU.cu:772): Y = gamma (X - mean) / sqrt(var + eps) + beta per row, biased variance, fp32 arithmetic,
 * X and Y [rows][D] in one 16-bit dtype, gamma and beta fp32 [D].  D a multiple of 8, at most 2048; 16-byte
 * aligned.  It belongs to the layer stack around the attention, not to the attention path: it is here because
 * a decode step is a chain of small kernels, and this one lets the projection after it start at once (with
 * LOGOS_OPT_PROJECT_OVERLAP it also starts under the kernel before it; gamma and beta count as weights). */
int logos_layer_norm(logos_ctx* ctx, int dtype, const void* X, const float* gamma, const float* beta, void* Y,
                     int rows, int D, float eps);

/* INT8 -> BF16 / FP16: logos_kv_dequantize's fp32 product rounded once to the 16-bit type; tensors of a
 * multiple of 16 values, 16-byte aligned.  (A 16-bit attention over K and V that went through the cache.) */
int logos_kv_dequantize16(logos_ctx* ctx, int dst_dtype, const int8_t* src, int64_t src_stride,
                          const float* scales, void* dst, int64_t dst_stride, int n_tensors, int64_t elems);

/* ---- multi-head attention forward in one call ---------------------------- */

/* Replaces MultiHeadAttention::forward (include/Attention.hpp:290-300; per head AttentionHead::forward,
 * :218-267) and the attention half of ModelGPU::forward's layer loop (cuda/ModelGPU.cu:892-1015) for all
 * heads and sequences at once:
 *   Q, K, V = X · W_{Q,K,V}            one GEMM, written in the engine's [B][H][S][64] layout
 *   [cache]  K, V -> INT8 + scale      when k_cache is given (the order of cuda/ModelGPU.cu:908); with
 *                                      LOGOS_MHA_ATTEND_DEQUANTIZED the attention then reads them back
 *                                      from the cache (K and V "passed through" the quantiser)
 *   head_out = attention(Q, K, V)      Navier-Stokes prologue, masks, softmax as `params` says
 *   concat   = sum_h head_out_h · W_O[h]
 *   out      = concat · W_proj (+ residual)
 * X: [B*S][D_model] in `dtype` (BF16 or FP16); Wt_qkv [3*H*64][D_model], Wt_o [D_model][H*64], Wt_proj
 * [D_model][D_model]: K-major 16-bit shadows of the weights in the same dtype,
 *   Wt_qkv[(which*H + h)*64 + c][k] = W_which[h][k][c]   (which = 0, 1, 2 for Q, K, V),
 *   Wt_o[n][h*64 + c] = W_O[h][c][n],   Wt_proj[n][k] = W_proj[k][n];
 * for the CPU classes, which keep columns [h*64, h*64+64) of head_out_h · W_O[h], Wt_o is block diagonal
 * (Wt_o[h*64 + j][h*64 + c] = W_O[h][c][j], zero elsewhere).  out, residual: [B*S][D_model] in out_dtype (`dtype` or LOGOS_F32); residual may be NULL.
 * k_cache, v_cache: int8 [B][H][S_max][64], k_scale, v_scale: float [B][H]; the four together or all NULL.
 * scratch: device memory of logos_mha_workspace_bytes(B, S, H, D_model) bytes, 256-byte aligned, owned by
 * the caller and free again when the call's work on the stream has finished.  H * 64 need not equal D_model. */
#define LOGOS_MHA_ATTEND_DEQUANTIZED 1
size_t logos_mha_workspace_bytes(int B, int S, int H, int D_model);
int logos_mha_forward(logos_ctx* ctx, int dtype, int out_dtype, const void* X, const void* Wt_qkv,
                      const void* Wt_o, const void* Wt_proj, const void* residual, void* out, int B, int S,
                      int H, int D_model, const logos_attn_params* params, int8_t* k_cache, int8_t* v_cache,
                      float* k_scale, float* v_scale, int S_max, int flags, void* scratch, size_t scratch_bytes);

/* The same forward in fp32 with the CPU classes' own weight layout -- the drop-in for
 * `Tensor MultiHeadAttention::forward(const Tensor& X)` (include/Attention.hpp:290-300) on one sequence:
 * X [seq][d_model]; W_Q, W_K, W_V [H][d_model][d_k]; W_O [H][d_k][d_model]; W_proj [d_model][d_model], all
 * row-major fp32 as Tensor stores them, d_k = d_model / H <= 128.  Per head Q, K, V = X · W, the attention
 * `params` describes (blend included), head_out · W_O[h] of which columns [0, d_k) go to columns
 * [h d_k, (h+1) d_k) of concat, then concat · W_proj.  kv_int8 != 0 passes K and V through the Nikhilam
 * quantiser and back before the attention (cuda/ModelGPU.cu:908, nikhilam_decompress).  The GEMMs are
 * fp32 FMA loops in k order (logos_gemm_f32), the attention is logos_attention_fwd in fp32.
 * scratch: logos_mha_f32_workspace_bytes(seq, d_model, H) bytes of device memory, 256-byte aligned. */
size_t logos_mha_f32_workspace_bytes(int seq, int d_model, int H);
int logos_mha_forward_f32(logos_ctx* ctx, const float* X, const float* W_Q, const float* W_K, const float* W_V,
                          const float* W_O, const float* W_proj, float* out, int seq, int d_model, int H,
                          const logos_attn_params* params, int kv_int8, void* scratch, size_t scratch_bytes);

/* C_b [M][N] = A_b [M][K] · B_b [K][N] for b < batch, row-major fp32 with leading dimensions and batch
 * strides in elements (stride 0: one operand for the whole batch); fp32 FMA accumulation in k order --
 * the arithmetic of the reference's vedic_gemm (include/VedicGEMM.hpp) up to the order of the additions. */
int logos_gemm_f32(logos_ctx* ctx, const float* A, int lda, int64_t strideA, const float* B, int ldb,
                   int64_t strideB, float* C, int ldc, int64_t strideC, int M, int N, int K, int batch);

/* ---- heads over several GPUs -------------------------------------------- */

/* The path shards by (sequence, head): GPU r of N owns heads [r H/N, (r+1) H/N) and their cache, and
 * the only exchange is the all-gather of the per-head outputs along the head axis.  The reference has
 * no counterpart (its head loop is serial on one GPU, cuda/ModelGPU.cu:892-988).  A logos_comm is one
 * rank's end of that exchange: a block of device memory that the other ranks map and write with
 * ordinary peer stores (no TMA, no multicast): two staging slots of `gathered_bytes` each, a row area for
 * decode outputs (8 bytes per value, at most 2 MiB per slot, i.e. B * H * DH <= 262144 values) and flags.
 *   set-up, once:  logos_comm_create on every rank; then either
 *                    logos_comm_handle -> exchange the 80-byte handles by any means -> logos_comm_connect
 *                    (one process per GPU: the blocks are shared through CUDA IPC), or
 *                    logos_comm_connect_local (all ranks are contexts of one process).
 *   per step:      a producing call stores this rank's rows into every rank's block, then a collecting
 *                  call queues a kernel that waits until all ranks' rows of the step have arrived -- at
 *                  most LOGOS_OPT_PEER_WAIT_MS, then logos_ctx_synchronize reports
 *                  LOGOS_ERR_KERNEL_TIMEOUT -- and writes them to `gathered`.  Two pairs exist:
 *                    logos_decode_int8_push / logos_decode_int8_collect   decode rows (small): every value
 *                        travels as an 8-byte word that carries its own arrival mark, no fence or flag;
 *                    logos_comm_push / logos_comm_wait                    any per-head tensor (large): plain
 *                        copies, then one flag per rank.
 *                  Exactly one producing call per collecting call, in the same order on every rank.
 * The step counter is device memory, so a CUDA graph that holds a step replays unchanged.  Nothing here
 * allocates after logos_comm_create; destroy the comm after its last kernel has finished. */
typedef struct logos_comm logos_comm;
#define LOGOS_COMM_HANDLE_BYTES 80
int logos_comm_create(logos_ctx* ctx, int rank, int world, size_t gathered_bytes, logos_comm** out);
int logos_comm_handle(logos_comm* comm, void* handle_out /* LOGOS_COMM_HANDLE_BYTES */);
int logos_comm_connect(logos_comm* comm, const void* handles /* world x LOGOS_COMM_HANDLE_BYTES, rank order */);
int logos_comm_connect_local(logos_comm* const* comms /* [world], rank order */, int world);
int logos_comm_destroy(logos_comm* comm);

/* logos_decode_int8 over this rank's H_local heads whose merged rows go straight from the kernel's
 * epilogue into every rank's staging slot at head offset rank * H_local (the gathered tensor is
 * float [B][H_local * world][DH]); no separate gather pass and no library collective. */
int logos_decode_int8_push(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                           const int8_t* k_cache, const int8_t* v_cache, const float* k_scale,
                           const float* v_scale, const int32_t* len, int B, int H_local, int S_max, int DH,
                           const logos_attn_params* params);
/* The collecting half: waits for every rank's rows of the step and writes float [B][H_total][DH]. */
int logos_decode_int8_collect(logos_ctx* ctx, logos_comm* comm, float* gathered, int B, int H_total, int DH);
/* logos_decode_int8_push followed by logos_decode_int8_collect into `gathered` (float [B][H_local * world][DH]). */
int logos_decode_int8_gather(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                             const int8_t* k_cache, const int8_t* v_cache, const float* k_scale,
                             const float* v_scale, const int32_t* len, int B, int H_local, int S_max, int DH,
                             const logos_attn_params* params, float* gathered);
/* logos_decode_step_int8 over this rank's heads with the gathered result on every rank: append,
 * decode with the peer epilogue, wait-and-copy (three launches). */
int logos_decode_step_int8_gather(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                                  const void* k_new, const void* v_new, int8_t* k_cache, int8_t* v_cache,
                                  const float* k_scale, const float* v_scale, const int32_t* len, int B,
                                  int H_local, int S_max, int DH, const logos_attn_params* params,
                                  float* gathered);
/* The same exchange for any per-head tensor this rank has already computed (the prefill output):
 * local is [B][H_local][row_bytes], gathered [B][H_local * world][row_bytes]; row_bytes a multiple of 16. */
int logos_comm_push(logos_ctx* ctx, logos_comm* comm, const void* local, int B, int H_local, size_t row_bytes);
int logos_comm_wait(logos_ctx* ctx, logos_comm* comm, void* gathered, size_t bytes);
int logos_comm_all_gather_heads(logos_ctx* ctx, logos_comm* comm, const void* local, void* gathered, int B,
                                int H_local, size_t row_bytes);

#ifdef __cplusplus
}
#endif
#endif /* LOGOS_ATTN_H */
