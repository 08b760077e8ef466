// logos_attn_shim.cu -- the reference's own attention entry point, served by the engine.
//
// LOGOS declares (cuda/VedicGEMM.cuh:236-243) and defines (cuda/VedicGEMM.cu:1065-1104)
//     void cuda_flash_attention_fwd(const float* Q, const float* K, const float* V, float* out,
//                                   float* attn_ptr, int seq, int DH, float scale, bool causal,
//                                   bool shunyam, int window, int stride);
// and calls it once per head from ModelGPU::forward (cuda/ModelGPU.cu:959-968).  This file defines
// the same C++ symbol on top of the C ABI, so a LOGOS build that leaves the original definition out
// and links liblogos_attn_shim.so + liblogos_attn.so needs no other change.  Conventions kept:
// the caller owns every buffer, work goes to the default stream of the current device without a
// synchronisation, and every failure surfaces as std::runtime_error: the reference throws that type
// both for the argument it rejects (DH > 128, cuda/VedicGEMM.cu:1074-1079) and for a failed launch
// (cuda/VedicGEMM.cu:1094-1102, CUDA_CHECK at cuda/VedicGEMM.cuh:111-133), so a caller's
// catch (const std::runtime_error&) keeps working.
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include "../../include/logos_attn.h"

namespace {

// one engine context per device, made on first use from the calling thread's current device
logos_ctx* context_of_current_device() {
    static std::mutex mu;
    static std::map<int, logos_ctx*> ctxs;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw std::runtime_error("logos_attn: cudaGetDevice failed");
    std::lock_guard<std::mutex> lock(mu);
    auto it = ctxs.find(dev);
    if (it != ctxs.end()) return it->second;
    logos_ctx* c = nullptr;
    const int rc = logos_ctx_create(dev, &c);
    if (rc != LOGOS_OK) throw std::runtime_error(std::string("logos_attn: ") + logos_status_string(rc));
    ctxs[dev] = c;
    return c;
}

}  // namespace

void cuda_flash_attention_fwd(const float* Q, const float* K, const float* V, float* out, float* attn_ptr,
                              int seq, int DH, float scale, bool causal, bool shunyam, int window, int stride) {
    logos_ctx* ctx = context_of_current_device();
    const int rc = logos_flash_attention_fwd_f32(ctx, Q, K, V, out, attn_ptr, seq, DH, scale, causal ? 1 : 0,
                                                 shunyam ? 1 : 0, window, stride);
    if (rc == LOGOS_OK) return;
    throw std::runtime_error(std::string("cuda_flash_attention_fwd: ") + logos_last_error(ctx));
}
