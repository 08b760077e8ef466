// abi.cu -- the extern "C" surface declared in include/logos_attn.h: context
// management, argument checks and dispatch to the kernels.
#include <cstring>
#include <new>

#include "common.cuh"

namespace {

constexpr int kAbsmaxSlots = 65536;

bool params_ok(const logos_attn_params* p) {
    return p && p->diffuse_mode >= LOGOS_DIFFUSE_NONE && p->diffuse_mode <= LOGOS_DIFFUSE_CENTRAL &&
           p->ns_alpha >= 0.0f && p->ns_alpha <= 1.0f && p->window >= 0;
}

// the workspace block and how to give it back
void release_workspace(logos_ctx* ctx) {
    if (ctx->owns_workspace && ctx->workspace) {
        if (ctx->ws_free_fn) ctx->ws_free_fn(ctx->workspace, ctx->ws_free_user);
        else cudaFree(ctx->workspace);
    }
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    ctx->owns_workspace = false;
    ctx->ws_free_fn = nullptr;
    ctx->ws_free_user = nullptr;
}


// scratch of logos_mha_forward: Q, K, V, head outputs ([B][H][S][64], 16-bit), concat ([B*S][D], 16-bit),
// two tables of max|x| per (sequence, head); every part 256-byte aligned
struct mha_layout { size_t q, k, v, o, concat, kmax, vmax, total; };
mha_layout mha_scratch(int B, int S, int H, int D) {
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t heads = up((size_t)B * H * S * 64 * 2), cc = up((size_t)B * S * D * 2), tab = up((size_t)B * H * 4);
    mha_layout l;
    l.q = 0; l.k = heads; l.v = 2 * heads; l.o = 3 * heads; l.concat = 4 * heads;
    l.kmax = l.concat + cc; l.vmax = l.kmax + tab; l.total = l.vmax + tab;
    return l;
}

// scratch of logos_mha_forward_f32: Q, K, V, head outputs ([H][seq][d_k] fp32), concat ([seq][d_model]), the INT8
// copies of K and V and their scales
struct mha_f32_layout { size_t q, k, v, o, concat, k8, v8, scales, total; };
mha_f32_layout mha_f32_scratch(int seq, int D, int H) {
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t heads = up((size_t)seq * D * 4), bytes8 = up((size_t)seq * D);
    mha_f32_layout l;
    l.q = 0; l.k = heads; l.v = 2 * heads; l.o = 3 * heads; l.concat = 4 * heads;
    l.k8 = 5 * heads; l.v8 = l.k8 + bytes8; l.scales = l.v8 + bytes8; l.total = l.scales + up((size_t)2 * H * 4);
    return l;
}

// decode whose rows go to every rank of the comm; `follows_append`: the launch before it is the engine's append
int decode_push(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev, const int8_t* k_cache,
                const int8_t* v_cache, const float* k_scale, const float* v_scale, const int32_t* len, int B,
                int H_local, int S_max, int DH, const logos_attn_params* params, bool follows_append) {
    if (!ctx || !comm) return LOGOS_ERR_INVALID_ARG;
    if (comm->ctx != ctx || !comm->connected)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8_push: comm is not connected or belongs to another context");
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8_push: bad parameter block");
    if (B <= 0 || H_local <= 0 || DH <= 0 || (size_t)B * H_local * comm->world * DH * 8 > comm->row_slot_bytes)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8_push: gathered output exceeds the comm's row area (%zu bytes per slot, 8 per value)",
                           comm->row_slot_bytes);
    PeerEpilogue pe;
    logos::comm_peer_epilogue(comm, H_local, &pe);
    return logos::decode_int8(ctx, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H_local, S_max, DH, params,
                              nullptr, &pe, follows_append);
}
}  // namespace

extern "C" {

int logos_abi_version(void) { return LOGOS_ATTN_ABI_VERSION; }

const char* logos_status_string(int status) {
    switch (status) {
        case LOGOS_OK: return "ok";
        case LOGOS_ERR_INVALID_ARG: return "invalid argument";
        case LOGOS_ERR_UNSUPPORTED: return "unsupported request";
        case LOGOS_ERR_WORKSPACE: return "workspace too small";
        case LOGOS_ERR_CUDA: return "CUDA error";
        case LOGOS_ERR_NO_DEVICE: return "no sm_100 CUDA device";
        case LOGOS_ERR_ALIGNMENT: return "misaligned pointer or extent";
        case LOGOS_ERR_KERNEL_TIMEOUT: return "a bounded wait inside a kernel ran out";
        case LOGOS_ERR_SCRATCH_LIMIT: return "request exceeds the fixed scratch of the no-allocation entry point";
    }
    return "unknown status";
}

int logos_ctx_create(int device, logos_ctx** out) {
    if (!out) return LOGOS_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        cudaGetLastError();
        return LOGOS_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) return LOGOS_ERR_INVALID_ARG;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return LOGOS_ERR_CUDA;
    if (prop.major != 10) return LOGOS_ERR_NO_DEVICE;  // kernels are built for sm_100a only
    if (cudaSetDevice(device) != cudaSuccess) return LOGOS_ERR_CUDA;
    logos_ctx* ctx = new (std::nothrow) logos_ctx();
    if (!ctx) return LOGOS_ERR_CUDA;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(&ctx->absmax_scratch, sizeof(float) * kAbsmaxSlots) != cudaSuccess) {
        delete ctx;
        return LOGOS_ERR_CUDA;
    }
    ctx->absmax_slots = kAbsmaxSlots;
    if (cudaMalloc(&ctx->tc_status, sizeof(int)) != cudaSuccess ||
        cudaMemset(ctx->tc_status, 0, sizeof(int)) != cudaSuccess) {
        cudaFree(ctx->absmax_scratch);
        delete ctx;
        return LOGOS_ERR_CUDA;
    }
    *out = ctx;
    return LOGOS_OK;
}

int logos_ctx_destroy(logos_ctx* ctx) {
    if (!ctx) return LOGOS_OK;
    cudaSetDevice(ctx->device);
    release_workspace(ctx);
    if (ctx->absmax_scratch) cudaFree(ctx->absmax_scratch);
    if (ctx->tc_status) cudaFree(ctx->tc_status);
    delete ctx;
    return LOGOS_OK;
}

int logos_ctx_set_stream(logos_ctx* ctx, void* cuda_stream) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    return LOGOS_OK;
}

int logos_ctx_set_allocator(logos_ctx* ctx, logos_alloc_fn alloc, logos_free_fn free_fn, void* user) {
    if (!ctx || ((alloc == nullptr) != (free_fn == nullptr))) return LOGOS_ERR_INVALID_ARG;
    ctx->alloc_fn = alloc;
    ctx->free_fn = free_fn;
    ctx->alloc_user = user;
    return LOGOS_OK;
}

int logos_ctx_reserve(logos_ctx* ctx, size_t bytes) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (ctx->workspace && ctx->workspace_bytes >= bytes) return LOGOS_OK;
    if (ctx->workspace_locked)
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "reserve: the workspace is locked (a captured graph uses it) and holds "
                           "%zu bytes, %zu wanted; reserve the largest size before capturing", ctx->workspace_bytes, bytes);
    LOGOS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    // the new block first: if it cannot be had, the context keeps what it has
    void* p = nullptr;
    if (ctx->alloc_fn) {
        if (ctx->alloc_fn(&p, bytes, ctx->alloc_user) != 0 || !p)
            return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "reserve: the caller's allocator could not supply %zu bytes", bytes);
        if (reinterpret_cast<uintptr_t>(p) & 255u) {
            ctx->free_fn(p, ctx->alloc_user);
            return logos::fail(ctx, LOGOS_ERR_ALIGNMENT, "reserve: the caller's allocator returned a block that is not 256-byte aligned");
        }
    } else if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "reserve: cudaMalloc of %zu bytes failed", bytes);
    }
    // Work queued on the stream may still use the old block.
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    // arrival counters at the head of the workspace must start at zero
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e != cudaSuccess) {
        if (ctx->alloc_fn) ctx->free_fn(p, ctx->alloc_user); else cudaFree(p);
        return logos::fail(ctx, LOGOS_ERR_CUDA, "reserve: %s", cudaGetErrorString(e));
    }
    release_workspace(ctx);
    ctx->workspace = p;
    ctx->workspace_bytes = bytes;
    ctx->owns_workspace = true;
    ctx->ws_free_fn = ctx->alloc_fn ? ctx->free_fn : nullptr;
    ctx->ws_free_user = ctx->alloc_user;
    return LOGOS_OK;
}

int logos_ctx_set_workspace(logos_ctx* ctx, void* device_ptr, size_t bytes) {
    if (!ctx || (!device_ptr && bytes)) return LOGOS_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(device_ptr) & 255u)
        return logos::fail(ctx, LOGOS_ERR_ALIGNMENT, "workspace must be 256-byte aligned");
    if (ctx->workspace_locked)
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "set_workspace: the workspace is locked (a captured graph uses it)");
    LOGOS_CUDA_TRY(ctx, cudaSetDevice(ctx->device));
    LOGOS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    release_workspace(ctx);
    ctx->workspace = device_ptr;
    ctx->workspace_bytes = bytes;
    ctx->owns_workspace = false;
    if (device_ptr) LOGOS_CUDA_TRY(ctx, cudaMemset(device_ptr, 0, bytes));
    return LOGOS_OK;
}

int logos_ctx_synchronize(logos_ctx* ctx) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    LOGOS_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    int flag = 0;
    LOGOS_CUDA_TRY(ctx, cudaMemcpy(&flag, ctx->tc_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(ctx->tc_status, 0, sizeof(int));
        if (flag & 0x20000000)
            return logos::fail(ctx, LOGOS_ERR_KERNEL_TIMEOUT,
                               "rank %d of the comm did not deliver its rows within %d ms; the gathered output is invalid",
                               (flag >> 16) & 0xff, ctx->peer_wait_ms);
        return logos::fail(ctx, LOGOS_ERR_KERNEL_TIMEOUT,
                           "a bounded wait inside a kernel ran out (barrier %d, thread %d); results of that call are invalid",
                           (flag & 0xffff) / 8, (flag >> 16) & 0x3fff);
    }
    return LOGOS_OK;
}

const char* logos_last_error(const logos_ctx* ctx) { return ctx ? ctx->err : "null context"; }

int logos_ctx_set_option(logos_ctx* ctx, int option, int value) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    switch (option) {
        case LOGOS_OPT_FORCE_GENERAL:
            ctx->force_general = value != 0;
            return LOGOS_OK;
        case LOGOS_OPT_DECODE_CHUNK:
            if (value != 0 && (value < 128 || value > 1024 || (value % 64) != 0))
                return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "set_option: decode chunk must be 0 or a multiple of 64 in [128, 1024]");
            ctx->decode_chunk = value;
            return LOGOS_OK;
        case LOGOS_OPT_PEER_WAIT_MS:
            if (value < 1 || value > 60000)
                return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "set_option: peer wait must be 1..60000 ms");
            ctx->peer_wait_ms = value;
            return LOGOS_OK;
        case LOGOS_OPT_WORKSPACE_LOCK:
            ctx->workspace_locked = value != 0;
            return LOGOS_OK;
        case LOGOS_OPT_GEMM_NARROW:
            ctx->gemm_narrow = value != 0;
            return LOGOS_OK;
        case LOGOS_OPT_DECODE_DEPTH:
            if (value != 0 && value != 2 && value != 4)
                return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "set_option: decode depth must be 0, 2 or 4");
            ctx->decode_depth = value;
            return LOGOS_OK;
        case LOGOS_OPT_QKV_OUT_F16:
            ctx->qkv_out_f16 = value != 0;
            return LOGOS_OK;
        case LOGOS_OPT_PROJECT_OVERLAP:
            ctx->project_overlap = value != 0;
            return LOGOS_OK;
    }
    return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "set_option: unknown option %d", option);
}

int logos_flash_attention_fwd_f32(logos_ctx* ctx, const float* Q, const float* K, const float* V,
                                  float* out, float* attn_ptr, int seq, int DH, float scale,
                                  int causal, int shunyam, int window, int stride) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!Q || !K || !V || !out || seq <= 0 || DH <= 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "flash_attention_fwd: bad pointer or extent");
    if (attn_ptr)
        return logos::fail(ctx, LOGOS_ERR_UNSUPPORTED,
                           "flash_attention_fwd: saving the seq x seq weights is not supported");
    if (shunyam && (window <= 0 || stride <= 0))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG,
                           "flash_attention_fwd: shunyam needs window > 0 and stride > 0");
    logos_attn_params p;
    p.scale = scale;
    p.causal = causal;
    // The reference caller passes "shunyam && seq > window" (cuda/ModelGPU.cu:966) and the
    // kernel re-checks seq > window (cuda/VedicGEMM.cu:990); window 0 switches the rule off.
    p.window = shunyam ? window : 0;
    p.stride = stride;
    p.ns_eta = 0.0f; p.ns_nu = 0.0f; p.ns_alpha = 0.0f;
    p.diffuse_mode = LOGOS_DIFFUSE_NONE;
    return logos::attention_simt(ctx, LOGOS_F32, LOGOS_F32, Q, K, V, out, 1, 1, seq, DH, &p);
}

int logos_selftest_umma(logos_ctx* ctx, int mode, int dtype, const void* A, const void* B, float* D) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::umma_selftest(ctx, mode, dtype, A, B, D);
}

size_t logos_attention_workspace_bytes(int B, int H, int S, int DH) {
    (void)B; (void)H; (void)S; (void)DH;
    return 0;
}

int logos_attention_fwd(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                        const void* V, void* O, int B, int H, int S, int DH,
                        const logos_attn_params* params) {
    return logos_attention_fwd_strided(ctx, in_dtype, out_dtype, Q, K, V, O, B, H, S, DH, nullptr, nullptr, params);
}

int logos_attention_fwd_strided(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                                const void* V, void* O, int B, int H, int S, int DH,
                                const logos_strides* qkv, const logos_strides* out,
                                const logos_attn_params* params) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    for (const logos_strides* st : {qkv, out})
        if (st && (st->row < DH || st->head < 0 || st->batch < 0))
            return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_fwd: a row stride below DH or a negative stride");
    const bool strided = qkv != nullptr || out != nullptr;
    if (!Q || !K || !V || !O || B <= 0 || H <= 0 || S <= 0 || DH <= 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_fwd: bad pointer or extent");
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_fwd: bad parameter block");
    if (!logos::dtype_ok(in_dtype) || !logos::dtype_ok(out_dtype))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_fwd: unknown dtype");
    // What the tensor-core kernel takes (causal, Shunyam window with or without landmarks) goes there; the
    // gather kernel keeps the Shunyam shapes it declines (viscosity above 1/2); everything else is fp32 SIMT.
    if (!ctx->force_general && logos::attention_tc_eligible(in_dtype, out_dtype, DH, params, S))
        return logos::attention_tc(ctx, in_dtype, out_dtype, Q, K, V, O, B, H, S, DH, params, qkv, out);
    if (!strided && !ctx->force_general && logos::attention_window_eligible(in_dtype, out_dtype, DH, params, S))
        return logos::attention_window(ctx, in_dtype, out_dtype, Q, K, V, O, B, H, S, DH, params);
    return logos::attention_simt(ctx, in_dtype, out_dtype, Q, K, V, O, B, H, S, DH, params, qkv, out);
}

size_t logos_attention_bwd_workspace_bytes(int B, int H, int S, int DH) {
    return logos::attention_bwd_workspace_bytes(B, H, S, DH);
}

int logos_attention_bwd(logos_ctx* ctx, const float* Q, const float* K, const float* V, const float* dO,
                        float* dQ, float* dK, float* dV, int B, int H, int S, int DH,
                        const logos_attn_params* params) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!params_ok(params)) return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_bwd: bad parameter block");
    return logos::attention_bwd(ctx, Q, K, V, dO, dQ, dK, dV, B, H, S, DH, params);
}

size_t logos_attention_bwd16_workspace_bytes(int B, int H, int S, int DH) {
    return logos::attention_bwd16_workspace_bytes(B, H, S, DH);
}

int logos_attention_bwd16(logos_ctx* ctx, int dtype, const void* Q, const void* K, const void* V, const void* dO,
                          float* dQ, float* dK, float* dV, int B, int H, int S, int DH,
                          const logos_attn_params* params) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!params_ok(params)) return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "attention_bwd16: bad parameter block");
    return logos::attention_bwd16(ctx, dtype, Q, K, V, dO, dQ, dK, dV, B, H, S, DH, params);
}

int logos_prefill_fwd(logos_ctx* ctx, int in_dtype, int out_dtype, const void* Q, const void* K,
                      const void* V, void* O, int B, int H, int S, int DH,
                      const logos_attn_params* params, int8_t* k_cache, int8_t* v_cache,
                      float* k_scale, float* v_scale, int S_max) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    const int given = (k_cache != nullptr) + (v_cache != nullptr) + (k_scale != nullptr) + (v_scale != nullptr);
    if (given != 0 && given != 4)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "prefill_fwd: caches and scales are given together or not at all");
    if (given == 4) {
        if (!K || !V || B <= 0 || H <= 0 || S <= 0 || DH <= 0 || S > S_max)
            return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "prefill_fwd: bad pointer or extent (S=%d, S_max=%d)", S, S_max);
        // the raw K and V, before diffusion; at most 65535 tensors per quantise call
        const int64_t elems = (int64_t)S * DH, dst_stride = (int64_t)S_max * DH;
        const size_t esz = in_dtype == LOGOS_F32 ? 4 : 2;
        const int n = B * H;
        for (int t0 = 0; t0 < n; t0 += 32768) {
            const int nt = n - t0 < 32768 ? n - t0 : 32768;
            int rc = logos::kv_quantize(ctx, in_dtype, (const char*)K + (size_t)t0 * elems * esz, elems,
                                        k_cache + (size_t)t0 * dst_stride, dst_stride, k_scale + t0, nt, elems);
            if (rc != LOGOS_OK) return rc;
            rc = logos::kv_quantize(ctx, in_dtype, (const char*)V + (size_t)t0 * elems * esz, elems,
                                    v_cache + (size_t)t0 * dst_stride, dst_stride, v_scale + t0, nt, elems);
            if (rc != LOGOS_OK) return rc;
        }
    }
    return logos_attention_fwd(ctx, in_dtype, out_dtype, Q, K, V, O, B, H, S, DH, params);
}

int logos_project_heads(logos_ctx* ctx, int dtype, int out_dtype, const void* head_out, const void* Wt_o,
                        const void* residual, void* C, int B, int S, int H, int N) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::project_heads(ctx, dtype, out_dtype, head_out, Wt_o, residual, C, B, S, H, N);
}

int logos_kv_dequantize16(logos_ctx* ctx, int dst_dtype, const int8_t* src, int64_t src_stride,
                          const float* scales, void* dst, int64_t dst_stride, int n_tensors, int64_t elems) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::kv_dequantize16(ctx, dst_dtype, src, src_stride, scales, dst, dst_stride, n_tensors, elems);
}

size_t logos_mha_workspace_bytes(int B, int S, int H, int D_model) {
    if (B <= 0 || S <= 0 || H <= 0 || D_model <= 0) return 0;
    const mha_layout l = mha_scratch(B, S, H, D_model);
    return l.total;
}

int logos_mha_forward(logos_ctx* ctx, int dtype, int out_dtype, const void* X, const void* Wt_qkv,
                      const void* Wt_o, const void* Wt_proj, const void* residual, void* out, int B, int S,
                      int H, int D_model, const logos_attn_params* params, int8_t* k_cache, int8_t* v_cache,
                      float* k_scale, float* v_scale, int S_max, int flags, void* scratch, size_t scratch_bytes) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!X || !Wt_qkv || !Wt_o || !Wt_proj || !out || !scratch || B <= 0 || S <= 0 || H <= 0 || D_model <= 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward: bad pointer or extent");
    if (!params_ok(params)) return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward: bad parameter block");
    if (dtype != LOGOS_BF16 && dtype != LOGOS_F16)
        return logos::fail(ctx, LOGOS_ERR_UNSUPPORTED, "mha_forward: X and the weight shadows are BF16 or FP16");
    const int given = (k_cache != nullptr) + (v_cache != nullptr) + (k_scale != nullptr) + (v_scale != nullptr);
    if (given != 0 && given != 4)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward: caches and scales are given together or not at all");
    if (given == 4 && S > S_max)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward: S = %d exceeds S_max = %d", S, S_max);
    if ((flags & LOGOS_MHA_ATTEND_DEQUANTIZED) && given != 4)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward: attending the dequantised K and V needs the caches");
    if ((int64_t)B * H > 65535)
        return logos::fail(ctx, LOGOS_ERR_UNSUPPORTED, "mha_forward: more than 65535 (sequence, head) tensors");
    const mha_layout l = mha_scratch(B, S, H, D_model);
    if (scratch_bytes < l.total || (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "mha_forward: scratch of %zu bytes, 256-byte aligned, needed (%zu given)",
                           l.total, scratch_bytes);
    char* base = static_cast<char*>(scratch);
    void *Q = base + l.q, *K = base + l.k, *V = base + l.v, *O = base + l.o, *concat = base + l.concat;
    float* kmax = reinterpret_cast<float*>(base + l.kmax);
    float* vmax = reinterpret_cast<float*>(base + l.vmax);

    int rc = logos::qkv_project(ctx, dtype, X, Wt_qkv, Q, K, V, B, S, H, D_model, given ? kmax : nullptr,
                                given ? vmax : nullptr);
    if (rc != LOGOS_OK) return rc;
    if (given) {
        const int64_t elems = (int64_t)S * 64, dst_stride = (int64_t)S_max * 64;
        rc = logos::kv_quantize(ctx, dtype, K, elems, k_cache, dst_stride, k_scale, B * H, elems, kmax);
        if (rc != LOGOS_OK) return rc;
        rc = logos::kv_quantize(ctx, dtype, V, elems, v_cache, dst_stride, v_scale, B * H, elems, vmax);
        if (rc != LOGOS_OK) return rc;
        if (flags & LOGOS_MHA_ATTEND_DEQUANTIZED) {
            rc = logos::kv_dequantize16(ctx, dtype, k_cache, dst_stride, k_scale, K, elems, B * H, elems);
            if (rc != LOGOS_OK) return rc;
            rc = logos::kv_dequantize16(ctx, dtype, v_cache, dst_stride, v_scale, V, elems, B * H, elems);
            if (rc != LOGOS_OK) return rc;
        }
    }
    rc = logos_attention_fwd(ctx, dtype, dtype, Q, K, V, O, B, H, S, 64, params);
    if (rc != LOGOS_OK) return rc;
    rc = logos::project_heads(ctx, dtype, dtype, O, Wt_o, nullptr, concat, B, S, H, D_model);
    if (rc != LOGOS_OK) return rc;
    return logos::project(ctx, dtype, out_dtype, concat, Wt_proj, residual, out, B * S, D_model, D_model);
}

size_t logos_mha_f32_workspace_bytes(int seq, int d_model, int H) {
    if (seq <= 0 || d_model <= 0 || H <= 0 || d_model % H != 0) return 0;
    return mha_f32_scratch(seq, d_model, H).total;
}

int logos_gemm_f32(logos_ctx* ctx, const float* A, int lda, int64_t strideA, const float* B, int ldb,
                   int64_t strideB, float* C, int ldc, int64_t strideC, int M, int N, int K, int batch) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::gemm_f32(ctx, A, lda, strideA, B, ldb, strideB, C, ldc, strideC, M, N, K, batch);
}

int logos_mha_forward_f32(logos_ctx* ctx, const float* X, const float* W_Q, const float* W_K, const float* W_V,
                          const float* W_O, const float* W_proj, float* out, int seq, int d_model, int H,
                          const logos_attn_params* params, int kv_int8, void* scratch, size_t scratch_bytes) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!X || !W_Q || !W_K || !W_V || !W_O || !W_proj || !out || !scratch || seq <= 0 || d_model <= 0 || H <= 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward_f32: bad pointer or extent");
    if (d_model % H != 0)     // the reference throws std::invalid_argument here (include/Attention.hpp:281-282)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward_f32: d_model must be divisible by num_heads");
    if (!params_ok(params)) return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "mha_forward_f32: bad parameter block");
    const int dk = d_model / H;
    const mha_f32_layout l = mha_f32_scratch(seq, d_model, H);
    if (scratch_bytes < l.total || (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "mha_forward_f32: scratch of %zu bytes, 256-byte aligned, needed (%zu given)",
                           l.total, scratch_bytes);
    char* base = static_cast<char*>(scratch);
    float *Q = (float*)(base + l.q), *K = (float*)(base + l.k), *V = (float*)(base + l.v), *O = (float*)(base + l.o);
    float* concat = (float*)(base + l.concat);
    const int64_t head = (int64_t)seq * dk, wqkv = (int64_t)d_model * dk;
    const float* W[3] = {W_Q, W_K, W_V};
    float* D3[3] = {Q, K, V};
    for (int i = 0; i < 3; ++i) {      // [H] x ([seq][d_model] · [d_model][d_k]), X shared by the heads
        int rc = logos::gemm_f32(ctx, X, d_model, 0, W[i], dk, wqkv, D3[i], dk, head, seq, dk, d_model, H);
        if (rc != LOGOS_OK) return rc;
    }
    if (kv_int8) {
        int8_t* k8 = (int8_t*)(base + l.k8);
        int8_t* v8 = (int8_t*)(base + l.v8);
        float* ks = (float*)(base + l.scales);
        float* vs = ks + H;
        int rc = logos::kv_quantize(ctx, LOGOS_F32, K, head, k8, head, ks, H, head);
        if (rc == LOGOS_OK) rc = logos::kv_quantize(ctx, LOGOS_F32, V, head, v8, head, vs, H, head);
        if (rc == LOGOS_OK) rc = logos::kv_dequantize(ctx, k8, head, ks, K, head, H, head);
        if (rc == LOGOS_OK) rc = logos::kv_dequantize(ctx, v8, head, vs, V, head, H, head);
        if (rc != LOGOS_OK) return rc;
    }
    int rc = logos_attention_fwd(ctx, LOGOS_F32, LOGOS_F32, Q, K, V, O, 1, H, seq, dk, params);
    if (rc != LOGOS_OK) return rc;
    // columns [0, d_k) of head_out_h · W_O[h] -> columns [h d_k, (h+1) d_k) of concat
    rc = logos::gemm_f32(ctx, O, dk, head, W_O, d_model, (int64_t)dk * d_model, concat, d_model, dk, seq, dk, dk, H);
    if (rc != LOGOS_OK) return rc;
    return logos::gemm_f32(ctx, concat, d_model, 0, W_proj, d_model, 0, out, d_model, 0, seq, d_model, d_model, 1);
}

int logos_kv_quantize(logos_ctx* ctx, int src_dtype, const void* src, int64_t src_stride,
                      int8_t* dst, int64_t dst_stride, float* scales, int n_tensors,
                      int64_t elems) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::kv_quantize(ctx, src_dtype, src, src_stride, dst, dst_stride, scales, n_tensors, elems);
}

int logos_kv_quantize_absmax(logos_ctx* ctx, int src_dtype, const void* src, int64_t src_stride,
                             int8_t* dst, int64_t dst_stride, const float* absmax, float* scales, int n_tensors,
                             int64_t elems) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!absmax) return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "kv_quantize_absmax: absmax table missing");
    return logos::kv_quantize(ctx, src_dtype, src, src_stride, dst, dst_stride, scales, n_tensors, elems, absmax);
}

int logos_project(logos_ctx* ctx, int dtype, int out_dtype, const void* A, const void* Wt, const void* residual,
                  void* C, int M, int N, int K) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::project(ctx, dtype, out_dtype, A, Wt, residual, C, M, N, K);
}

int logos_qkv_project(logos_ctx* ctx, int dtype, const void* X, const void* Wt_qkv, void* Q, void* K, void* V,
                      int B, int S, int H, int D_model, float* k_absmax, float* v_absmax) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::qkv_project(ctx, dtype, X, Wt_qkv, Q, K, V, B, S, H, D_model, k_absmax, v_absmax);
}

int logos_kv_dequantize(logos_ctx* ctx, const int8_t* src, int64_t src_stride, const float* scales,
                        float* dst, int64_t dst_stride, int n_tensors, int64_t elems) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::kv_dequantize(ctx, src, src_stride, scales, dst, dst_stride, n_tensors, elems);
}

int logos_kv_append(logos_ctx* ctx, int dtype, const void* k_new, const void* v_new,
                    int8_t* k_cache, int8_t* v_cache, const float* k_scale, const float* v_scale,
                    const int32_t* pos, int B, int H, int S_max, int DH) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::kv_append(ctx, dtype, k_new, v_new, k_cache, v_cache, k_scale, v_scale, pos, B, H, S_max, DH);
}

size_t logos_decode_workspace_bytes(int B, int H, int S_max, int DH) {
    // split-K partials + arrival counters, plus staging for the *_host entry point
    size_t stage = (size_t)(B > 0 ? B : 0) * (H > 0 ? H : 0) * (DH > 0 ? DH : 0) * (4 * 2 + 4) +
                   (size_t)(B > 0 ? B : 0) * 8 + 1024;
    return logos::decode_workspace_bytes(B, H, S_max, DH) + stage;
}

int logos_decode_int8(logos_ctx* ctx, const void* q, const void* q_prev, const int8_t* k_cache,
                      const int8_t* v_cache, const float* k_scale, const float* v_scale,
                      const int32_t* len, int B, int H, int S_max, int DH,
                      const logos_attn_params* params, float* out) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_int8: bad parameter block");
    return logos::decode_int8(ctx, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, params, out);
}

// append + decode on device buffers.  The window kernel quantises the new rows itself (one launch); the dense kernel
// follows an append kernel and is launched to overlap it.
static int decode_step(logos_ctx* ctx, const void* q, const void* q_prev, const void* k_new, const void* v_new,
                       int8_t* k_cache, int8_t* v_cache, const float* k_scale, const float* v_scale, const int32_t* len,
                       int B, int H, int S_max, int DH, const logos_attn_params* params, int out_dtype, void* out) {
    if (k_new && v_new && logos::decode_appends_itself(params, DH))
        return logos::decode_int8(ctx, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, params,
                                  static_cast<float*>(out), nullptr, /*follows_append*/ false, out_dtype, k_new, v_new);
    int rc = logos::kv_append(ctx, LOGOS_F16, k_new, v_new, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, -1);
    if (rc != LOGOS_OK) return rc;
    return logos::decode_int8(ctx, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, params,
                              static_cast<float*>(out), nullptr, /*follows_append*/ true, out_dtype);
}

int logos_decode_step_int8(logos_ctx* ctx, const void* q, const void* q_prev, const void* k_new, const void* v_new,
                           int8_t* k_cache, int8_t* v_cache, const float* k_scale, const float* v_scale,
                           const int32_t* len, int B, int H, int S_max, int DH, const logos_attn_params* params,
                           float* out) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_step: bad parameter block");
    return decode_step(ctx, q, q_prev, k_new, v_new, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, params,
                       LOGOS_F32, out);
}

int logos_layer_norm(logos_ctx* ctx, int dtype, const void* X, const float* gamma, const float* beta, void* Y,
                     int rows, int D, float eps) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    return logos::layer_norm(ctx, dtype, X, gamma, beta, Y, rows, D, eps);
}

int logos_decode_step_int8_to(logos_ctx* ctx, const void* q, const void* q_prev, const void* k_new, const void* v_new,
                              int8_t* k_cache, int8_t* v_cache, const float* k_scale, const float* v_scale,
                              const int32_t* len, int B, int H, int S_max, int DH, const logos_attn_params* params,
                              int out_dtype, void* out) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_step: bad parameter block");
    return decode_step(ctx, q, q_prev, k_new, v_new, k_cache, v_cache, k_scale, v_scale, len, B, H, S_max, DH, params,
                       out_dtype, out);
}

int logos_decode_step_int8_gather(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                                  const void* k_new, const void* v_new, int8_t* k_cache, int8_t* v_cache,
                                  const float* k_scale, const float* v_scale, const int32_t* len, int B,
                                  int H_local, int S_max, int DH, const logos_attn_params* params, float* gathered) {
    if (!ctx || !comm) return LOGOS_ERR_INVALID_ARG;
    int rc = logos::kv_append(ctx, LOGOS_F16, k_new, v_new, k_cache, v_cache, k_scale, v_scale, len, B, H_local, S_max,
                              DH, -1);
    if (rc != LOGOS_OK) return rc;
    rc = decode_push(ctx, comm, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H_local, S_max, DH, params,
                     /*follows_append*/ true);
    if (rc != LOGOS_OK) return rc;
    return logos::comm_collect_rows(ctx, comm, gathered, B, H_local * comm->world, DH, /*follows_decode*/ true);
}

int logos_decode_int8_push(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                           const int8_t* k_cache, const int8_t* v_cache, const float* k_scale,
                           const float* v_scale, const int32_t* len, int B, int H_local, int S_max, int DH,
                           const logos_attn_params* params) {
    return decode_push(ctx, comm, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H_local, S_max, DH, params,
                       false);
}

int logos_decode_int8_gather(logos_ctx* ctx, logos_comm* comm, const void* q, const void* q_prev,
                             const int8_t* k_cache, const int8_t* v_cache, const float* k_scale,
                             const float* v_scale, const int32_t* len, int B, int H_local, int S_max, int DH,
                             const logos_attn_params* params, float* gathered) {
    const int rc = decode_push(ctx, comm, q, q_prev, k_cache, v_cache, k_scale, v_scale, len, B, H_local, S_max, DH,
                               params, false);
    if (rc != LOGOS_OK) return rc;
    return logos::comm_collect_rows(ctx, comm, gathered, B, H_local * comm->world, DH, /*follows_decode*/ true);
}

int logos_decode_int8_collect(logos_ctx* ctx, logos_comm* comm, float* gathered, int B, int H_total, int DH) {
    if (!ctx || !comm) return LOGOS_ERR_INVALID_ARG;
    return logos::comm_collect_rows(ctx, comm, gathered, B, H_total, DH);
}

int logos_decode_step_int8_host(logos_ctx* ctx, const void* q_host, const void* q_prev_host,
                                const void* k_new_host, const void* v_new_host,
                                int8_t* k_cache, int8_t* v_cache, const float* k_scale,
                                const float* v_scale, const int32_t* len_host, int B, int H,
                                int S_max, int DH, const logos_attn_params* params,
                                float* out_host) {
    if (!ctx) return LOGOS_ERR_INVALID_ARG;
    if (!q_host || !k_new_host || !v_new_host || !len_host || !out_host || B <= 0 || H <= 0 || DH <= 0)
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_step_host: bad pointer or extent");
    if (!params_ok(params))
        return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_step_host: bad parameter block");
    const size_t vec = (size_t)B * H * DH;           // elements per [B][H][DH] tensor
    const size_t kernel_ws = logos::decode_workspace_bytes(B, H, S_max, DH);
    const size_t need = logos_decode_workspace_bytes(B, H, S_max, DH);
    if (!ctx->workspace || ctx->workspace_bytes < need)
        return logos::fail(ctx, LOGOS_ERR_WORKSPACE, "decode_step_host: workspace of %zu bytes needed, %zu reserved",
                           need, ctx->workspace_bytes);
    if (B > 4096) return logos::fail(ctx, LOGOS_ERR_UNSUPPORTED, "decode_step_host: B > 4096");
    for (int b = 0; b < B; ++b)
        if (len_host[b] < 1 || len_host[b] > S_max)
            return logos::fail(ctx, LOGOS_ERR_INVALID_ARG, "decode_step_host: len[%d]=%d outside [1,%d]", b,
                               len_host[b], S_max);
    // staging layout behind the kernel workspace: q | q_prev | k_new | v_new (fp16), len (int32), out (fp32)
    char* base = (char*)ctx->workspace + ((kernel_ws + 255) & ~(size_t)255);
    __half* d_q = (__half*)base;
    __half* d_qp = d_q + vec;
    __half* d_k = d_qp + vec;
    __half* d_v = d_k + vec;
    int32_t* d_len = (int32_t*)(d_v + vec);
    float* d_out = (float*)((char*)d_len + (((size_t)B * sizeof(int32_t) + 15) & ~(size_t)15));
    cudaStream_t st = ctx->stream;
    const size_t hb = vec * sizeof(__half);
    // Host tensors that lie one after the other (q | q_prev | k_new | v_new | len, the order of the staging area)
    // travel as one copy: each copy costs a few microseconds of issue and engine turnaround on top of its bytes.
    {
        const char* src[5] = {(const char*)q_host, (const char*)q_prev_host, (const char*)k_new_host, (const char*)v_new_host,
                              (const char*)len_host};
        char* dst[5] = {(char*)d_q, (char*)d_qp, (char*)d_k, (char*)d_v, (char*)d_len};
        const size_t bytes[5] = {hb, hb, hb, hb, sizeof(int32_t) * (size_t)B};
        for (int i = 0; i < 5;) {
            if (!src[i]) { ++i; continue; }
            int j = i + 1;
            size_t run = bytes[i];
            while (j < 5 && src[j] == src[j - 1] + bytes[j - 1]) run += bytes[j++];
            if (j - i > 1 && cudaMemcpyAsync(dst[i], src[i], run, cudaMemcpyHostToDevice, st) != cudaSuccess) {
                // neighbours in address space but separate page-locked allocations: the runtime refuses a copy
                // that spans them -- send them one by one
                cudaGetLastError();
                j = i;
            }
            if (j - i <= 1) {
                LOGOS_CUDA_TRY(ctx, cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyHostToDevice, st));
                j = i + 1;
            }
            i = j;
        }
    }
    int rc = logos::kv_append(ctx, LOGOS_F16, d_k, d_v, k_cache, v_cache, k_scale, v_scale, d_len, B, H, S_max, DH, -1);
    if (rc != LOGOS_OK) return rc;
    rc = logos::decode_int8(ctx, d_q, q_prev_host ? d_qp : nullptr, k_cache, v_cache, k_scale, v_scale, d_len, B,
                            H, S_max, DH, params, d_out, nullptr, /*follows_append*/ true);
    if (rc != LOGOS_OK) return rc;
    LOGOS_CUDA_TRY(ctx, cudaMemcpyAsync(out_host, d_out, vec * sizeof(float), cudaMemcpyDeviceToHost, st));
    LOGOS_CUDA_TRY(ctx, cudaStreamSynchronize(st));
    return LOGOS_OK;
}

}  // extern "C"
