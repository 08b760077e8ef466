// ref_gpu_harness.cu -- C entry points around the reference's own CUDA kernels.
//
// TEST INFRASTRUCTURE ONLY.  Declares nothing of its own: the kernels and the
// host wrapper come from the reference's cuda/ModelGPU.cuh and
// cuda/VedicGEMM.cuh, compiled unmodified for sm_100a from the reference tree
// (see the Makefile in this folder).  It serves as a second witness for the
// Nikhilam INT8 arithmetic and as the "reference kernel on the same GPU"
// baseline.  All pointers are device pointers; work runs on the default stream
// as in the reference; every call returns a cudaError_t as int.
#include "ModelGPU.cuh"

#include <cstdio>

extern "C" {

int refgpu_absmax(const float* x, float* out_scalar, int n) {
    cudaMemset(out_scalar, 0, sizeof(float));
    absmax_kernel<<<(n + 255) / 256, 256>>>(x, out_scalar, n);
    return (int)cudaGetLastError();
}

int refgpu_quantize(const float* x, int8_t* q, float scale, int n) {
    nikhilam_quantize_kernel<<<(n + 255) / 256, 256>>>(x, q, scale, n);
    return (int)cudaGetLastError();
}

int refgpu_dequantize(const int8_t* q, float* x, float scale, int n) {
    nikhilam_dequantize_kernel<<<(n + 255) / 256, 256>>>(q, x, scale, n);
    return (int)cudaGetLastError();
}

int refgpu_ns_advect(const float* Q, float* Qa, int seq, int d, float eta) {
    ns_advect_kernel<<<(seq * d + 255) / 256, 256>>>(Q, Qa, seq, d, eta);
    return (int)cudaGetLastError();
}

int refgpu_ns_diffuse(const float* V, float* Vs, int seq, int d, float nu) {
    ns_diffuse_kernel<<<(seq * d + 255) / 256, 256>>>(V, Vs, seq, d, nu);
    return (int)cudaGetLastError();
}

int refgpu_flash_attention_fwd(const float* Q, const float* K, const float* V, float* out,
                               int seq, int DH, float scale, int causal, int shunyam,
                               int window, int stride) {
    try {
        cuda_flash_attention_fwd(Q, K, V, out, nullptr, seq, DH, scale, causal != 0,
                                 shunyam != 0, window, stride);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "refgpu_flash_attention_fwd: %s\n", e.what());
        return -1;
    }
    return (int)cudaGetLastError();
}

}  // extern "C"
