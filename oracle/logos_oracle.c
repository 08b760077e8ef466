/*
 * logos_oracle.c -- CPU restatement of the LOGOS attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY: used by tests, by the smoke check and by the
 * CPU-baseline leg of the benchmark as the checker.  The product never calls it.
 *
 * Build: gcc -O2 -std=c11 -ffp-contract=off -fopenmp -fPIC -shared
 * (no -ffast-math, no FMA contraction: fp32 results follow the source order).
 */
#include "logos_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LO_BLOCK 64
#define LO_NEG   (-1e9f)

static inline int imin(int a, int b) { return a < b ? a : b; }
static inline int imax(int a, int b) { return a > b ? a : b; }

int lo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* include/VedicGEMM.hpp:26-55 -- blocks of 64 over i, then k, then j; inside a
 * block the order is i, k, j with a scalar a[i][k] broadcast over a row of B. */
void lo_gemm(const float* A, const float* B, float* C, int M, int K, int N) {
    memset(C, 0, sizeof(float) * (size_t)M * N);
    for (int ib = 0; ib < M; ib += LO_BLOCK) {
        int ie = imin(ib + LO_BLOCK, M);
        for (int kb = 0; kb < K; kb += LO_BLOCK) {
            int ke = imin(kb + LO_BLOCK, K);
            for (int jb = 0; jb < N; jb += LO_BLOCK) {
                int je = imin(jb + LO_BLOCK, N);
                for (int i = ib; i < ie; ++i)
                    for (int k = kb; k < ke; ++k) {
                        float a = A[(size_t)i * K + k];
                        float* c = C + (size_t)i * N;
                        const float* b = B + (size_t)k * N;
                        for (int j = jb; j < je; ++j) c[j] += a * b[j];
                    }
            }
        }
    }
}

/* include/Attention.hpp:19-36 -- max over the whole row, exp((s-max)/T),
 * then divide by (sum + 1e-9). */
void lo_boltzmann_softmax(const float* scores, float* probs, int rows, int cols,
                          float temperature) {
    for (int i = 0; i < rows; ++i) {
        const float* s = scores + (size_t)i * cols;
        float* p = probs + (size_t)i * cols;
        float mx = s[0];
        for (int j = 1; j < cols; ++j) mx = s[j] > mx ? s[j] : mx;
        float sum = 0.0f;
        for (int j = 0; j < cols; ++j) {
            float e = expf((s[j] - mx) / temperature);
            p[j] = e;
            sum += e;
        }
        for (int j = 0; j < cols; ++j) p[j] /= (sum + 1e-9f);
    }
}

/* include/Attention.hpp:47-60 */
void lo_causal_mask(float* mask, int seq) {
    for (int i = 0; i < seq; ++i)
        for (int j = 0; j < seq; ++j) mask[(size_t)i * seq + j] = (j > i) ? LO_NEG : 0.0f;
}

/* include/Attention.hpp:80-98 -- everything void, then the local window
 * [max(0,i-window), i] and every stride-th position strictly before i are opened. */
void lo_shunyam_mask(float* mask, int seq, int window, int stride) {
    for (size_t t = 0; t < (size_t)seq * seq; ++t) mask[t] = LO_NEG;
    for (int i = 0; i < seq; ++i) {
        float* row = mask + (size_t)i * seq;
        for (int j = imax(0, i - window); j <= i; ++j) row[j] = 0.0f;
        for (int j = 0; j < i; j += stride) row[j] = 0.0f;
    }
}

/* cuda/ModelGPU.cu:443-451 and include/Attention.hpp:151-158 */
void lo_ns_advect(const float* Q, float* Qa, int seq, int d, float eta) {
    for (int i = 0; i < seq; ++i)
        for (int c = 0; c < d; ++c) {
            float q = Q[(size_t)i * d + c];
            float qp = (i > 0) ? Q[(size_t)(i - 1) * d + c] : q;
            Qa[(size_t)i * d + c] = q + eta * (q - qp);
        }
}

/* cuda/ModelGPU.cu:463-471 */
void lo_ns_diffuse_causal(const float* V, float* Vs, int seq, int d, float nu) {
    for (int i = 0; i < seq; ++i)
        for (int c = 0; c < d; ++c) {
            float v = V[(size_t)i * d + c];
            float vp = (i > 0) ? V[(size_t)(i - 1) * d + c] : v;
            Vs[(size_t)i * d + c] = (1.0f - nu) * v + nu * vp;
        }
}

/* include/Attention.hpp:173-181 */
void lo_ns_diffuse_central(const float* V, float* Vs, int seq, int d, float nu) {
    for (int i = 0; i < seq; ++i) {
        int il = (i > 0) ? i - 1 : 0;
        int ir = (i < seq - 1) ? i + 1 : seq - 1;
        for (int c = 0; c < d; ++c)
            Vs[(size_t)i * d + c] = (1.0f - nu) * V[(size_t)i * d + c] +
                                    (nu * 0.5f) * (V[(size_t)il * d + c] + V[(size_t)ir * d + c]);
    }
}

static void transpose(const float* A, float* At, int rows, int cols) {
    for (int i = 0; i < rows; ++i)
        for (int j = 0; j < cols; ++j) At[(size_t)j * rows + i] = A[(size_t)i * cols + j];
}

/* scores = Q K^T + mask ; probs = softmax ; out = probs * V  (Attention.hpp:258-264) */
void lo_std_attention(const float* Q, const float* K, const float* V, const float* mask,
                      float temperature, float* out, int seq, int dk, int dv) {
    float* Kt = (float*)malloc(sizeof(float) * (size_t)seq * dk);
    float* sc = (float*)malloc(sizeof(float) * (size_t)seq * seq);
    float* pr = (float*)malloc(sizeof(float) * (size_t)seq * seq);
    transpose(K, Kt, seq, dk);
    lo_gemm(Q, Kt, sc, seq, dk, seq);
    for (size_t t = 0; t < (size_t)seq * seq; ++t) sc[t] += mask[t];
    lo_boltzmann_softmax(sc, pr, seq, seq, temperature);
    lo_gemm(pr, V, out, seq, seq, dv);
    free(Kt); free(sc); free(pr);
}

/* include/Attention.hpp:139-187 */
void lo_ns_attention(const float* Q, const float* K, const float* V, const float* mask,
                     float temperature, float eta, float nu, float* out,
                     int seq, int dk, int dv) {
    float* Qa = (float*)malloc(sizeof(float) * (size_t)seq * dk);
    float* Vs = (float*)malloc(sizeof(float) * (size_t)seq * dv);
    lo_ns_advect(Q, Qa, seq, dk, eta);
    lo_ns_diffuse_central(V, Vs, seq, dv, nu);
    lo_std_attention(Qa, K, Vs, mask, temperature, out, seq, dk, dv);
    free(Qa); free(Vs);
}

static void int8_roundtrip(float* x, long n) {
    int8_t* q = (int8_t*)malloc((size_t)n);
    float s = lo_nikhilam_compress(x, q, n);
    lo_nikhilam_dequantize(q, x, s, n);
    free(q);
}

/* include/Attention.hpp:217-266 */
void lo_head_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                     const float* WO, int seq, int d_model, int dk, const lo_head_cfg* cfg,
                     float* out, float* head_out) {
    float temperature = sqrtf((float)dk);
    size_t nqk = (size_t)seq * dk;
    float* Q = (float*)malloc(sizeof(float) * nqk);
    float* K = (float*)malloc(sizeof(float) * nqk);
    float* V = (float*)malloc(sizeof(float) * nqk);
    lo_gemm(X, WQ, Q, seq, d_model, dk);
    lo_gemm(X, WK, K, seq, d_model, dk);
    lo_gemm(X, WV, V, seq, d_model, dk);
    if (cfg->kv_int8_roundtrip) {
        int8_roundtrip(K, (long)nqk);
        int8_roundtrip(V, (long)nqk);
    }
    float* mask = (float*)malloc(sizeof(float) * (size_t)seq * seq);
    if (cfg->use_sparse && seq > cfg->sparse_window)
        lo_shunyam_mask(mask, seq, cfg->sparse_window, cfg->sparse_stride);
    else
        lo_causal_mask(mask, seq);

    float* o_std = (float*)malloc(sizeof(float) * nqk);
    lo_std_attention(Q, K, V, mask, temperature, o_std, seq, dk, dk);
    if (cfg->use_navier_stokes && cfg->ns_alpha > 0.0f) {
        float* o_ns = (float*)malloc(sizeof(float) * nqk);
        float* p_std = (float*)malloc(sizeof(float) * (size_t)seq * d_model);
        float* p_ns = (float*)malloc(sizeof(float) * (size_t)seq * d_model);
        lo_ns_attention(Q, K, V, mask, temperature, cfg->ns_eta, cfg->ns_nu, o_ns, seq, dk, dk);
        lo_gemm(o_std, WO, p_std, seq, dk, d_model);
        lo_gemm(o_ns, WO, p_ns, seq, dk, d_model);
        float w1 = 1.0f - cfg->ns_alpha, w2 = cfg->ns_alpha;
        for (size_t t = 0; t < (size_t)seq * d_model; ++t) out[t] = w1 * p_std[t] + w2 * p_ns[t];
        if (head_out)
            for (size_t t = 0; t < nqk; ++t) head_out[t] = w1 * o_std[t] + w2 * o_ns[t];
        free(o_ns); free(p_std); free(p_ns);
    } else {
        lo_gemm(o_std, WO, out, seq, dk, d_model);
        if (head_out) memcpy(head_out, o_std, sizeof(float) * nqk);
    }
    free(Q); free(K); free(V); free(mask); free(o_std);
}

/* include/Attention.hpp:290-300 -- only the first dk columns of each head's
 * [seq x d_model] output are kept, placed at column h*dk of concat. */
void lo_mha_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                    const float* WO, const float* Wproj, int seq, int d_model, int H,
                    const lo_head_cfg* cfg, float* out) {
    int dk = d_model / H;
    float* concat = (float*)calloc((size_t)seq * d_model, sizeof(float));
    int nthreads = cfg->threads > 0 ? cfg->threads : 1;
    (void)nthreads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
    for (int h = 0; h < H; ++h) {
        float* ho = (float*)malloc(sizeof(float) * (size_t)seq * d_model);
        size_t wsz = (size_t)d_model * dk;
        lo_head_forward(X, WQ + h * wsz, WK + h * wsz, WV + h * wsz, WO + h * wsz, seq, d_model,
                        dk, cfg, ho, NULL);
        for (int i = 0; i < seq; ++i)
            for (int j = 0; j < dk; ++j)
                concat[(size_t)i * d_model + h * dk + j] = ho[(size_t)i * d_model + j];
        free(ho);
    }
    lo_gemm(concat, Wproj, out, seq, d_model, d_model);
    free(concat);
}

/* ------------------------------------------------------------------ */

int lo_allowed(int i, int j, int seq, const lo_attn_params* p) {
    if (j < 0 || j >= seq) return 0;
    if (p->causal && j > i) return 0;
    if (p->window > 0 && seq > p->window) {
        /* cuda/VedicGEMM.cu:991-996: in window = [i-window, i]; landmark = j % stride == 0.
         * The CPU mask (Attention.hpp:88-96) opens the same set below the diagonal. */
        int in_window = (j >= i - p->window) && (j <= i);
        int landmark = (p->stride > 0) && (j % p->stride == 0);
        if (!in_window && !landmark) return 0;
    }
    return 1;
}

/* One softmax(QK^T)V row in fp64 over the allowed keys.  qrow is the (possibly
 * advected) query; vmode selects which V variant is mixed. */
static void attend_row(const float* qrow, const float* K, const float* V, int seq, int d, int i,
                       const lo_attn_params* p, int vmode, float nu, double* acc, double* sc) {
    double mx = -INFINITY;
    for (int j = 0; j < seq; ++j) {
        if (!lo_allowed(i, j, seq, p)) { sc[j] = -INFINITY; continue; }
        double s = 0.0;
        const float* k = K + (size_t)j * d;
        for (int c = 0; c < d; ++c) s += (double)qrow[c] * (double)k[c];
        s *= (double)p->scale;
        sc[j] = s;
        if (s > mx) mx = s;
    }
    double l = 0.0;
    for (int c = 0; c < d; ++c) acc[c] = 0.0;
    for (int j = 0; j < seq; ++j) {
        if (sc[j] == -INFINITY) continue;
        double e = exp(sc[j] - mx);
        l += e;
        const float* v = V + (size_t)j * d;
        if (vmode == LO_DIFFUSE_NONE) {
            for (int c = 0; c < d; ++c) acc[c] += e * (double)v[c];
        } else if (vmode == LO_DIFFUSE_CAUSAL) {
            const float* vp = (j > 0) ? v - d : v;
            for (int c = 0; c < d; ++c) {
                float vs = (1.0f - nu) * v[c] + nu * vp[c];
                acc[c] += e * (double)vs;
            }
        } else {
            const float* vl = (j > 0) ? v - d : v;
            const float* vr = (j < seq - 1) ? v + d : v;
            for (int c = 0; c < d; ++c) {
                float vs = (1.0f - nu) * v[c] + (nu * 0.5f) * (vl[c] + vr[c]);
                acc[c] += e * (double)vs;
            }
        }
    }
    /* Attention.hpp:34 divides by sum+1e-9; VedicGEMM.cu:1049 uses 1/l when l > 1e-9. */
    double inv = (l > 1e-9) ? 1.0 / l : 0.0;
    for (int c = 0; c < d; ++c) acc[c] *= inv;
}

void lo_attention_rows_f64(const float* Q, const float* K, const float* V, float* out,
                           int seq, int d, int row0, int row1, const lo_attn_params* p) {
    int ns_on = (p->ns_alpha > 0.0f) && (p->ns_eta != 0.0f || p->diffuse_mode != LO_DIFFUSE_NONE);
    int std_on = !ns_on || p->ns_alpha < 1.0f;
#pragma omp parallel
    {
        double* sc = (double*)malloc(sizeof(double) * (size_t)seq);
        double* a_ns = (double*)malloc(sizeof(double) * (size_t)d);
        double* a_std = (double*)malloc(sizeof(double) * (size_t)d);
        float* qa = (float*)malloc(sizeof(float) * (size_t)d);
#pragma omp for schedule(dynamic, 8)
        for (int i = row0; i < row1; ++i) {
            const float* q = Q + (size_t)i * d;
            if (ns_on) {
                for (int c = 0; c < d; ++c) {
                    float qp = (i > 0) ? q[c - d] : q[c];
                    qa[c] = q[c] + p->ns_eta * (q[c] - qp);
                }
                attend_row(qa, K, V, seq, d, i, p, p->diffuse_mode, p->ns_nu, a_ns, sc);
            }
            if (std_on) attend_row(q, K, V, seq, d, i, p, LO_DIFFUSE_NONE, 0.0f, a_std, sc);
            float* o = out + (size_t)(i - row0) * d;
            for (int c = 0; c < d; ++c) {
                double r;
                if (!ns_on) r = a_std[c];
                else if (!std_on) r = a_ns[c];
                else r = (1.0 - (double)p->ns_alpha) * a_std[c] + (double)p->ns_alpha * a_ns[c];
                o[c] = (float)r;
            }
        }
        free(sc); free(a_ns); free(a_std); free(qa);
    }
}

/* ------------------------------------------------------------------ */
/* Attention backward: cuda/train_gpu.cu:657-748 (one head), with the    */
/* adjoints of the prologue from cuda/ModelGPU.cu:453-482.               */

/* One path (queries qx, values vx already advected / diffused), weight w on d_out:
 *   p      = softmax over the allowed keys of scale * qx_i . k_j        (recompute, train_gpu.cu:671-701)
 *   dvx_j += p_ij d_out_i                                                (attn_dV_kernel :422-432)
 *   dp_ij  = d_out_i . vx_j                                              (attn_dAttnProbs_kernel :434-444)
 *   ds_ij  = p_ij (dp_ij - sum_j p_ij dp_ij) scale                       (softmax_bwd_kernel :446-459)
 *   dqx_i += ds_ij k_j ;  dk_j += ds_ij qx_i                             (attn_dQ_kernel, attn_dK_kernel :461-481)
 * Unlike the reference's recompute, which applies the causal mask only, the mask is the one the
 * forward used (Shunyam window and landmarks included): the gradient of the forward that was run. */
static void bwd_path(const float* qx, const float* K, const float* vx, const float* dO, int seq, int d,
                     const lo_attn_params* p, double w, double* dqx, double* dk, double* dvx) {
    double* sc = (double*)malloc(sizeof(double) * (size_t)seq);
    double* dp = (double*)malloc(sizeof(double) * (size_t)seq);
    for (int i = 0; i < seq; ++i) {
        const float* q = qx + (size_t)i * d;
        const float* g = dO + (size_t)i * d;
        double mx = -INFINITY;
        for (int j = 0; j < seq; ++j) {
            if (!lo_allowed(i, j, seq, p)) { sc[j] = -INFINITY; continue; }
            double s = 0.0;
            for (int c = 0; c < d; ++c) s += (double)q[c] * (double)K[(size_t)j * d + c];
            sc[j] = s * (double)p->scale;
            if (sc[j] > mx) mx = sc[j];
        }
        double l = 0.0;
        for (int j = 0; j < seq; ++j) if (sc[j] != -INFINITY) { sc[j] = exp(sc[j] - mx); l += sc[j]; } else sc[j] = 0.0;
        if (!(l > 1e-9)) continue;            /* the forward wrote zeros for this row */
        double delta = 0.0;
        for (int j = 0; j < seq; ++j) {
            if (sc[j] == 0.0) { dp[j] = 0.0; continue; }
            sc[j] /= l;
            double t = 0.0;
            for (int c = 0; c < d; ++c) t += w * (double)g[c] * (double)vx[(size_t)j * d + c];
            dp[j] = t;
            delta += sc[j] * t;
        }
        for (int j = 0; j < seq; ++j) {
            if (sc[j] == 0.0) continue;
            double ds = sc[j] * (dp[j] - delta) * (double)p->scale;
            for (int c = 0; c < d; ++c) {
                dvx[(size_t)j * d + c] += sc[j] * w * (double)g[c];
                dqx[(size_t)i * d + c] += ds * (double)K[(size_t)j * d + c];
                dk[(size_t)j * d + c] += ds * (double)q[c];
            }
        }
    }
    free(sc); free(dp);
}

void lo_attention_bwd_f64(const float* Q, const float* K, const float* V, const float* dO, int seq, int d,
                          const lo_attn_params* p, float* dQ, float* dK, float* dV) {
    size_t n = (size_t)seq * d;
    int ns_on = (p->ns_alpha > 0.0f) && (p->ns_eta != 0.0f || p->diffuse_mode != LO_DIFFUSE_NONE);
    int std_on = !ns_on || p->ns_alpha < 1.0f;
    double* aq = (double*)calloc(n, sizeof(double));   /* gradients with respect to the raw Q, K, V */
    double* ak = (double*)calloc(n, sizeof(double));
    double* av = (double*)calloc(n, sizeof(double));
    if (ns_on) {
        float* qa = (float*)malloc(sizeof(float) * n);
        float* vs = (float*)malloc(sizeof(float) * n);
        double* dqa = (double*)calloc(n, sizeof(double));
        double* dvs = (double*)calloc(n, sizeof(double));
        lo_ns_advect(Q, qa, seq, d, p->ns_eta);
        if (p->diffuse_mode == LO_DIFFUSE_CAUSAL) lo_ns_diffuse_causal(V, vs, seq, d, p->ns_nu);
        else if (p->diffuse_mode == LO_DIFFUSE_CENTRAL) lo_ns_diffuse_central(V, vs, seq, d, p->ns_nu);
        else memcpy(vs, V, sizeof(float) * n);
        bwd_path(qa, K, vs, dO, seq, d, p, (double)p->ns_alpha, dqa, ak, dvs);
        double eta = (double)p->ns_eta, nu = (double)p->ns_nu;
        for (int i = 0; i < seq; ++i)
            for (int c = 0; c < d; ++c) {
                size_t x = (size_t)i * d + c;
                /* ns_advect_bwd_kernel, cuda/ModelGPU.cu:453-461 */
                double g = dqa[x] * ((i == 0) ? 1.0 : (1.0 + eta));
                if (i + 1 < seq) g -= eta * dqa[x + d];
                aq[x] += g;
                if (p->diffuse_mode == LO_DIFFUSE_CAUSAL) {
                    /* ns_diffuse_bwd_kernel, cuda/ModelGPU.cu:473-482 */
                    double h = (1.0 - nu) * dvs[x];
                    if (i + 1 < seq) h += nu * dvs[x + d];
                    if (i == 0) h += nu * dvs[x];
                    av[x] += h;
                } else if (p->diffuse_mode == LO_DIFFUSE_CENTRAL) {
                    /* transpose of the stencil of navier_stokes_attention (include/Attention.hpp:166-182):
                     * row j reads max(j-1, 0) and min(j+1, seq-1) */
                    double h = (1.0 - nu) * dvs[x];
                    if (i + 1 < seq) h += 0.5 * nu * dvs[x + d];      /* row i+1 reads i as its left */
                    if (i == 0) h += 0.5 * nu * dvs[x];               /* row 0 reads itself as its left */
                    if (i > 0) h += 0.5 * nu * dvs[x - d];            /* row i-1 reads i as its right */
                    if (i == seq - 1) h += 0.5 * nu * dvs[x];         /* the last row reads itself as its right */
                    av[x] += h;
                } else {
                    av[x] += dvs[x];
                }
            }
        free(qa); free(vs); free(dqa); free(dvs);
    }
    if (std_on) bwd_path(Q, K, V, dO, seq, d, p, ns_on ? 1.0 - (double)p->ns_alpha : 1.0, aq, ak, av);
    for (size_t x = 0; x < n; ++x) { dQ[x] = (float)aq[x]; dK[x] = (float)ak[x]; dV[x] = (float)av[x]; }
    free(aq); free(ak); free(av);
}

/* ------------------------------------------------------------------ */
/* Nikhilam INT8: cuda/ModelGPU.cu:293-395                             */

float lo_absmax(const float* x, long n) {
    float m = 0.0f; /* the device accumulator starts at zero (CudaPtr zero-init, :363) */
    for (long i = 0; i < n; ++i) {
        float a = fabsf(x[i]);
        m = fmaxf(m, a);
    }
    return m;
}

float lo_nikhilam_scale(float absmax) { return (absmax + 1e-8f) / 127.5f; }

void lo_nikhilam_quantize(const float* x, int8_t* q, float scale, long n) {
    float den = scale + 1e-8f;
    for (long i = 0; i < n; ++i) {
        float v = x[i] / den;
        v = fminf(fmaxf(v, -127.0f), 127.0f);
        q[i] = (int8_t)lrintf(v); /* round-half-even, as __float2int_rn */
    }
}

void lo_nikhilam_dequantize(const int8_t* q, float* x, float scale, long n) {
    for (long i = 0; i < n; ++i) x[i] = (float)q[i] * scale;
}

float lo_nikhilam_compress(const float* x, int8_t* q, long n) {
    float s = lo_nikhilam_scale(lo_absmax(x, n));
    lo_nikhilam_quantize(x, q, s, n);
    return s;
}

/* ------------------------------------------------------------------ */

void lo_decode_int8(const float* q, const float* q_prev, const int8_t* Kq, const int8_t* Vq,
                    float k_scale, float v_scale, int len, int d, const lo_attn_params* p,
                    float* out) {
    size_t n = (size_t)len * d;
    float* K = (float*)malloc(sizeof(float) * n);
    float* V = (float*)malloc(sizeof(float) * n);
    float* Q2 = (float*)calloc(2 * (size_t)d, sizeof(float));
    lo_nikhilam_dequantize(Kq, K, k_scale, (long)n);
    lo_nikhilam_dequantize(Vq, V, v_scale, (long)n);
    int i = len - 1;
    /* rows i-1 and i of a virtual Q matrix: only those two are read for row i */
    const float* qp = (q_prev && i > 0) ? q_prev : q;
    memcpy(Q2, qp, sizeof(float) * d);
    memcpy(Q2 + d, q, sizeof(float) * d);
    int ns_on = (p->ns_alpha > 0.0f) && (p->ns_eta != 0.0f || p->diffuse_mode != LO_DIFFUSE_NONE);
    int std_on = !ns_on || p->ns_alpha < 1.0f;
    double* sc = (double*)malloc(sizeof(double) * (size_t)len);
    double* a_ns = (double*)malloc(sizeof(double) * (size_t)d);
    double* a_std = (double*)malloc(sizeof(double) * (size_t)d);
    float* qa = (float*)malloc(sizeof(float) * (size_t)d);
    if (ns_on) {
        for (int c = 0; c < d; ++c) qa[c] = q[c] + p->ns_eta * (q[c] - qp[c]);
        attend_row(qa, K, V, len, d, i, p, p->diffuse_mode, p->ns_nu, a_ns, sc);
    }
    if (std_on) attend_row(q, K, V, len, d, i, p, LO_DIFFUSE_NONE, 0.0f, a_std, sc);
    for (int c = 0; c < d; ++c) {
        double r;
        if (!ns_on) r = a_std[c];
        else if (!std_on) r = a_ns[c];
        else r = (1.0 - (double)p->ns_alpha) * a_std[c] + (double)p->ns_alpha * a_ns[c];
        out[c] = (float)r;
    }
    free(K); free(V); free(Q2); free(sc); free(a_ns); free(a_std); free(qa);
}

void lo_decode_int8_batch(const float* q, const float* q_prev, const int8_t* Kq,
                          const int8_t* Vq, const float* k_scale, const float* v_scale,
                          const int* lens, int n, int s_max, int d, const lo_attn_params* p,
                          float* out, int threads) {
    int nthreads = threads > 0 ? threads : 1;
    (void)nthreads;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
    for (int t = 0; t < n; ++t) {
        size_t off = (size_t)t * s_max * d;
        lo_decode_int8(q + (size_t)t * d, q_prev ? q_prev + (size_t)t * d : NULL, Kq + off,
                       Vq + off, k_scale[t], v_scale[t], lens[t], d, p, out + (size_t)t * d);
    }
}
