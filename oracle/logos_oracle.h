/*
 * logos_oracle.h -- CPU restatement of the LOGOS attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this code; it exists so that tests (and the CPU-baseline leg of the
 * benchmark) have an independent statement of what the reference computes.
 *
 * Every function names the reference file:line it restates (paths are
 * relative to the LOGOS source tree).
 *
 * Parity status: the fp32 CPU-path functions (gemm, softmax, masks,
 * ns_attention, head/MHA forward) are pinned against the reference's own
 * include/Attention.hpp compiled unmodified (oracle/_ref) and against the
 * fixtures of the reference's tests M12/M20/M27.  The Nikhilam INT8
 * functions restate CUDA kernels that have no CPU twin in the reference;
 * they are pinned against the property fixtures of the reference's tests
 * (S13, M5, M6, MEM3) on CPU and against the reference's own kernels
 * compiled for sm_100a on a GPU box.
 */
#ifndef LOGOS_ORACLE_H
#define LOGOS_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- fp32 CPU path: include/Attention.hpp, include/VedicGEMM.hpp ---- */

/* C[MxN] = A[MxK] * B[KxN]; 64-blocked i/k/j order of vedic_gemm
 * (include/VedicGEMM.hpp:26-55), so the fp32 rounding sequence is the same. */
void lo_gemm(const float* A, const float* B, float* C, int M, int K, int N);

/* boltzmann_softmax, include/Attention.hpp:19-36. */
void lo_boltzmann_softmax(const float* scores, float* probs, int rows, int cols,
                          float temperature);

/* causal_mask_cached, include/Attention.hpp:47-60: 0 on/below the diagonal, -1e9 above. */
void lo_causal_mask(float* mask, int seq);

/* shunyam_sparse_mask, include/Attention.hpp:80-98. */
void lo_shunyam_mask(float* mask, int seq, int window, int stride);

/* navier_stokes_attention, include/Attention.hpp:139-187 (central diffusion, mirror BC). */
void lo_ns_attention(const float* Q, const float* K, const float* V, const float* mask,
                     float temperature, float eta, float nu, float* out,
                     int seq, int dk, int dv);

/* Standard path of AttentionHead::forward, include/Attention.hpp:258-265, without W_O. */
void lo_std_attention(const float* Q, const float* K, const float* V, const float* mask,
                      float temperature, float* out, int seq, int dk, int dv);

typedef struct {
    int   use_sparse;        /* AttentionHead::use_sparse      */
    int   sparse_window;     /* AttentionHead::sparse_window   */
    int   sparse_stride;     /* AttentionHead::sparse_stride   */
    int   use_navier_stokes; /* AttentionHead::use_navier_stokes */
    float ns_alpha, ns_eta, ns_nu;
    int   kv_int8_roundtrip; /* 1: K and V pass through Nikhilam quantize->dequantize
                                (one scale per [seq x dk] tensor) before attention.  The
                                reference has no single function for this; it composes
                                ModelGPU.cu:908 with the CPU attention. */
    int   threads;           /* heads farmed over this many OpenMP threads (>=1) */
} lo_head_cfg;

/* AttentionHead::forward, include/Attention.hpp:217-266.  out is [seq x d_model].
 * If head_out (nullable) is given it receives the blended pre-W_O output [seq x dk]. */
void lo_head_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                     const float* WO, int seq, int d_model, int dk, const lo_head_cfg* cfg,
                     float* out, float* head_out);

/* MultiHeadAttention::forward, include/Attention.hpp:290-300.  Per-head weights are
 * packed head-major: WQ/WK/WV [H][d_model][dk], WO [H][dk][d_model]; Wproj [d_model][d_model]. */
void lo_mha_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                    const float* WO, const float* Wproj, int seq, int d_model, int H,
                    const lo_head_cfg* cfg, float* out);

/* ---- Navier-Stokes prologue kernels ---- */

/* ns_advect_kernel, cuda/ModelGPU.cu:443-451 (same formula as Attention.hpp:151-158). */
void lo_ns_advect(const float* Q, float* Qa, int seq, int d, float eta);
/* ns_diffuse_kernel, cuda/ModelGPU.cu:463-471 (one-sided, causal). */
void lo_ns_diffuse_causal(const float* V, float* Vs, int seq, int d, float nu);
/* central two-sided diffusion with mirror boundary, include/Attention.hpp:173-181. */
void lo_ns_diffuse_central(const float* V, float* Vs, int seq, int d, float nu);

/* ---- general attention, fp64 accumulation, O(seq*d) memory ---- */

enum { LO_DIFFUSE_NONE = 0, LO_DIFFUSE_CAUSAL = 1, LO_DIFFUSE_CENTRAL = 2 };

typedef struct {
    float scale;        /* score multiplier (1/sqrt(dk)) */
    int   causal;       /* mask j > i */
    int   window;       /* Shunyam window; rule active iff window > 0 && seq > window */
    int   stride;       /* landmark stride; <= 0 disables landmarks (pure window) */
    float ns_eta;       /* advection strength; 0 = off */
    float ns_nu;        /* viscosity; used when diffuse_mode != NONE */
    float ns_alpha;     /* out = (1-alpha)*standard + alpha*NS */
    int   diffuse_mode; /* LO_DIFFUSE_* */
} lo_attn_params;

/* Allowed(i,j) under causal + Shunyam (include/Attention.hpp:80-98,
 * cuda/VedicGEMM.cu:987-996, cuda/ModelGPU.cu:435-441). */
int lo_allowed(int i, int j, int seq, const lo_attn_params* p);

/* Rows [row0,row1) of one head's attention with every option; masked keys are
 * skipped (cuda/VedicGEMM.cu:984-1049), which equals the additive -1e9 mask of
 * the CPU path to within fp32 underflow.  Q,K,V are [seq x d] fp32. */
void lo_attention_rows_f64(const float* Q, const float* K, const float* V, float* out,
                           int seq, int d, int row0, int row1, const lo_attn_params* p);

/* Gradients of one head's attention (the function above, all rows) with respect to the raw Q, K, V for a
 * given d_out [seq x d]: the chain of cuda/train_gpu.cu:657-748 (dV, dP, softmax backward, dQ, dK) and the
 * adjoints of the prologue, cuda/ModelGPU.cu:453-482, in fp64; the mask is the forward's own. */
void lo_attention_bwd_f64(const float* Q, const float* K, const float* V, const float* dO, int seq, int d,
                          const lo_attn_params* p, float* dQ, float* dK, float* dV);

/* ---- Nikhilam INT8 KV: cuda/ModelGPU.cu:293-395 ---- */

float lo_absmax(const float* x, long n);                 /* absmax_kernel :308-326 */
float lo_nikhilam_scale(float absmax);                   /* nikhilam_compress :379 */
void  lo_nikhilam_quantize(const float* x, int8_t* q, float scale, long n);   /* :329-340 */
void  lo_nikhilam_dequantize(const int8_t* q, float* x, float scale, long n); /* :343-351 */
/* nikhilam_compress :357-386: absmax -> scale -> quantize; returns the scale. */
float lo_nikhilam_compress(const float* x, int8_t* q, long n);

/* ---- decode composition (no single counterpart in the reference) ---- */

/* One decode step for one (sequence, head): the query is the token at position
 * len-1 (its K/V rows are already in the cache), K/V are dequantized with their
 * per-tensor scales and the last row of the attention above is returned.
 * q_prev may be NULL (no advection, or len == 1). */
void lo_decode_int8(const float* q, const float* q_prev, const int8_t* Kq, const int8_t* Vq,
                    float k_scale, float v_scale, int len, int d, const lo_attn_params* p,
                    float* out);

/* Batched form over n independent (sequence, head) pairs, OpenMP over pairs.
 * q,q_prev: [n][d] fp32; Kq,Vq: [n][s_max][d]; scales [n]; lens [n]; out [n][d]. */
void lo_decode_int8_batch(const float* q, const float* q_prev, const int8_t* Kq,
                          const int8_t* Vq, const float* k_scale, const float* v_scale,
                          const int* lens, int n, int s_max, int d, const lo_attn_params* p,
                          float* out, int threads);

int lo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
