// ref_bwd_harness.cu -- C entry point around the reference's own attention-backward kernels.
//
// TEST INFRASTRUCTURE ONLY.  The kernels come from the reference tree, compiled unmodified for
// sm_100a where they lie (cuda/train_gpu.cu with its main() renamed on the command line,
// cuda/ModelGPU.cu, cuda/VedicGEMM.cu; see the Makefile in this folder).  This file declares their
// signatures and launches them in the order run_backward() does for one head
// (cuda/train_gpu.cu:657-748): recompute the probabilities from Q_adv and K under the causal mask,
// then dV_s -> dV through ns_diffuse_bwd, dP, the softmax backward, dQ_adv -> dQ through
// ns_advect_bwd, and dK.  It is the second witness for the backward oracle.  All pointers are
// device pointers, work runs on the default stream, the return value is a cudaError_t as int.
#include "ModelGPU.cuh"

#include <cmath>

// cuda/train_gpu.cu:422-481
__global__ void attn_dV_kernel(const float*, const float*, float*, int, int);
__global__ void attn_dAttnProbs_kernel(const float*, const float*, float*, int, int);
__global__ void softmax_bwd_kernel(const float*, const float*, float*, int, float);
__global__ void attn_dQ_kernel(const float*, const float*, float*, int, int);
__global__ void attn_dK_kernel(const float*, const float*, float*, int, int);
// cuda/train_gpu.cu:61-65 (defined in cuda/ModelGPU.cu and cuda/VedicGEMM.cu)
extern __global__ void gpu_transpose_kernel(const float*, float*, int, int);
extern __global__ void grad_scale_kernel(float*, float, int);
extern __global__ void vedic_gemm_kernel(const float*, const float*, float*, int, int, int);
extern __global__ void boltzmann_softmax_kernel(const float*, float*, int, int, float);
extern __global__ void causal_mask_kernel(float*, int);

extern "C" {

// Q_adv, K, V_s, d_head_out: [seq][DH] as the forward cached them; dQ, dK, dV: [seq][DH] gradients with respect
// to the raw Q, K, V.  scratch: 3 seq^2 + 3 seq DH floats.
// run_backward launches gpu_transpose_kernel on a grid of (seq/16, DH/16) blocks (cuda/train_gpu.cu:683-684) while
// the kernel takes its row from blockIdx.y and its column from blockIdx.x (cuda/ModelGPU.cu:89-98): the launch covers
// min(seq, DH) rows and columns of K, all of it only when seq = DH, and what is not covered scores zero.
// transpose_all_rows = 0 keeps that launch; 1 launches the same kernel on (DH/16, seq/16) blocks so that every key
// and channel takes part, which is what the chain means to compute.
int refbwd_attention_head(const float* Q_adv, const float* K, const float* V_s, const float* d_head_out,
                          float* dQ, float* dK, float* dV, int seq, int DH, float eta, float nu, float* scratch,
                          int transpose_all_rows) {
    float* probs = scratch;
    float* d_probs = probs + (size_t)seq * seq;
    float* d_scores = d_probs + (size_t)seq * seq;
    float* K_T = d_scores + (size_t)seq * seq;
    float* dV_s = K_T + (size_t)seq * DH;
    float* dQ_adv = dV_s + (size_t)seq * DH;
    const float inv_sqrt_DH = 1.0f / sqrtf((float)DH);
    const int sz = seq * seq;
    cudaMemset(K_T, 0, sizeof(float) * (size_t)seq * DH);
    if (transpose_all_rows) gpu_transpose_kernel<<<dim3((DH + 15) / 16, (seq + 15) / 16), dim3(16, 16)>>>(K, K_T, seq, DH);
    else                    gpu_transpose_kernel<<<dim3((seq + 15) / 16, (DH + 15) / 16), dim3(16, 16)>>>(K, K_T, seq, DH);
    vedic_gemm_kernel<<<dim3((seq + 15) / 16, (seq + 15) / 16), dim3(16, 16)>>>(Q_adv, K_T, probs, seq, DH, seq);
    grad_scale_kernel<<<(sz + 255) / 256, 256>>>(probs, inv_sqrt_DH, sz);
    causal_mask_kernel<<<dim3(seq, (seq + 255) / 256), 256>>>(probs, seq);
    boltzmann_softmax_kernel<<<seq, 256>>>(probs, probs, seq, seq, 1.0f);
    cudaMemset(dV_s, 0, sizeof(float) * (size_t)seq * DH);
    attn_dV_kernel<<<dim3(DH, (seq + 31) / 32), 32>>>(probs, d_head_out, dV_s, seq, DH);
    ns_diffuse_bwd_kernel<<<(seq * DH + 255) / 256, 256>>>(dV_s, dV, seq, DH, nu);
    attn_dAttnProbs_kernel<<<dim3(seq, (seq + 31) / 32), 32>>>(d_head_out, V_s, d_probs, seq, DH);
    softmax_bwd_kernel<<<seq, 256>>>(probs, d_probs, d_scores, seq, inv_sqrt_DH);
    attn_dQ_kernel<<<dim3(seq, (DH + 31) / 32), 32>>>(d_scores, K, dQ_adv, seq, DH);
    ns_advect_bwd_kernel<<<(seq * DH + 255) / 256, 256>>>(dQ_adv, dQ, seq, DH, eta);
    attn_dK_kernel<<<dim3(seq, (DH + 31) / 32), 32>>>(d_scores, Q_adv, dK, seq, DH);
    return (int)cudaGetLastError();
}

}  // extern "C"
