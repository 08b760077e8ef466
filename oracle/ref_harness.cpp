// ref_harness.cpp -- C entry points around the reference's own CPU attention.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no attention arithmetic of its
// own: it includes the LOGOS headers (include/Attention.hpp, Tensor.hpp,
// VedicGEMM.hpp) unmodified from the reference tree given with -I at build time
// and forwards plain-pointer calls to them.  The result (oracle/_ref/) is used
// to pin the C restatement in logos_oracle.c, to generate the golden fixtures
// under tests/golden/, and as the timed CPU baseline.  No reference source is
// copied into this repository.
#include "Attention.hpp"

#include <cstring>
#include <thread>
#include <vector>

namespace {

Tensor make(const float* src, int r, int c) {
    Tensor t({r, c}, 0.0f);
    std::memcpy(t.data.data(), src, sizeof(float) * (size_t)r * c);
    return t;
}

void put(const Tensor& t, float* dst) {
    std::memcpy(dst, t.data.data(), sizeof(float) * (size_t)t.total_size);
}

// The mask selection of AttentionHead::forward (Attention.hpp:225-234).
Tensor pick_mask(int seq, int use_sparse, int window, int stride) {
    if (use_sparse && seq > window) return shunyam_sparse_mask_cached(seq, window, stride);
    return causal_mask_cached(seq);
}

}  // namespace

extern "C" {

void ref_gemm(const float* A, const float* B, float* C, int M, int K, int N) {
    put(vedic_gemm(make(A, M, K), make(B, K, N)), C);
}

void ref_boltzmann_softmax(const float* s, float* p, int rows, int cols, float T) {
    put(boltzmann_softmax(make(s, rows, cols), T), p);
}

void ref_causal_mask(float* mask, int seq) { put(causal_mask(seq), mask); }

void ref_shunyam_mask(float* mask, int seq, int window, int stride) {
    put(shunyam_sparse_mask(seq, window, stride), mask);
}

void ref_ns_attention(const float* Q, const float* K, const float* V, const float* mask,
                      float T, float eta, float nu, float* out, int seq, int dk, int dv) {
    put(navier_stokes_attention(make(Q, seq, dk), make(K, seq, dk), make(V, seq, dv),
                                make(mask, seq, seq), T, eta, nu),
        out);
}

// The body of AttentionHead::forward after the projections and before W_O
// (Attention.hpp:225-265), composed only of the reference's own functions.
void ref_attention_full(const float* Qp, const float* Kp, const float* Vp, int seq, int dk,
                        int use_sparse, int window, int stride, int use_ns, float alpha,
                        float eta, float nu, float* out) {
    Tensor Q = make(Qp, seq, dk), K = make(Kp, seq, dk), V = make(Vp, seq, dk);
    float T = std::sqrt(static_cast<float>(dk));
    Tensor mask = pick_mask(seq, use_sparse, window, stride);
    Tensor K_T = K.transpose();
    Tensor sc = vedic_gemm(Q, K_T);
    sc += mask;
    Tensor o_std = vedic_gemm(boltzmann_softmax(sc, T), V);
    if (use_ns && alpha > 0.0f) {
        Tensor o_ns = navier_stokes_attention(Q, K, V, mask, T, eta, nu);
        float w1 = 1.0f - alpha, w2 = alpha;
        for (int i = 0; i < o_std.total_size; ++i)
            out[i] = w1 * o_std.data[i] + w2 * o_ns.data[i];
    } else {
        put(o_std, out);
    }
}

struct ref_head_cfg {
    int use_sparse, sparse_window, sparse_stride, use_navier_stokes;
    float ns_alpha, ns_eta, ns_nu;
    int kv_int8_roundtrip;  // not available in the reference: must be 0 here
    int threads;
};

static void configure(AttentionHead& h, const ref_head_cfg* c) {
    h.use_sparse = c->use_sparse != 0;
    h.sparse_window = c->sparse_window;
    h.sparse_stride = c->sparse_stride;
    h.use_navier_stokes = c->use_navier_stokes != 0;
    h.ns_alpha = c->ns_alpha;
    h.ns_eta = c->ns_eta;
    h.ns_nu = c->ns_nu;
}

void ref_head_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                      const float* WO, int seq, int d_model, int dk, const ref_head_cfg* cfg,
                      float* out) {
    AttentionHead h(d_model, dk);
    h.W_Q = make(WQ, d_model, dk);
    h.W_K = make(WK, d_model, dk);
    h.W_V = make(WV, d_model, dk);
    h.W_O = make(WO, dk, d_model);
    configure(h, cfg);
    put(h.forward(make(X, seq, d_model)), out);
}

// MultiHeadAttention::forward (Attention.hpp:290-300).  threads <= 1 runs the
// reference method as it is; threads > 1 runs the same per-head forward calls on
// worker threads (mask caches are warmed first because they are not thread-safe)
// and then the reference's own concat + W_proj step.
void ref_mha_forward(const float* X, const float* WQ, const float* WK, const float* WV,
                     const float* WO, const float* Wproj, int seq, int d_model, int H,
                     const ref_head_cfg* cfg, float* out) {
    MultiHeadAttention mha(d_model, H);
    int dk = mha.d_k;
    size_t wsz = (size_t)d_model * dk;
    for (int h = 0; h < H; ++h) {
        mha.heads[h].W_Q = make(WQ + h * wsz, d_model, dk);
        mha.heads[h].W_K = make(WK + h * wsz, d_model, dk);
        mha.heads[h].W_V = make(WV + h * wsz, d_model, dk);
        mha.heads[h].W_O = make(WO + h * wsz, dk, d_model);
        configure(mha.heads[h], cfg);
    }
    mha.W_proj = make(Wproj, d_model, d_model);
    Tensor Xt = make(X, seq, d_model);
    if (cfg->threads <= 1) {
        put(mha.forward(Xt), out);
        return;
    }
    (void)pick_mask(seq, cfg->use_sparse, cfg->sparse_window, cfg->sparse_stride);
    std::vector<Tensor> outs(H);
    std::vector<std::thread> pool;
    int nt = cfg->threads < H ? cfg->threads : H;
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&, t] {
            for (int h = t; h < H; h += nt) outs[h] = mha.heads[h].forward(Xt);
        });
    for (auto& th : pool) th.join();
    Tensor concat({seq, d_model}, 0.0f);
    for (int h = 0; h < H; ++h)
        for (int i = 0; i < seq; ++i)
            for (int j = 0; j < dk; ++j) concat.at(i, h * dk + j) = outs[h].at(i, j);
    put(vedic_gemm(concat, mha.W_proj), out);
}

// n independent (sequence, head) attention problems, each re-run over its whole
// context as the reference's generate loop does (cuda/train_gpu.cu:2037-2046),
// farmed over `threads` workers.  Q,K,V: [n][seq][dk]; out: [n][seq][dk].
void ref_attention_full_batch(const float* Q, const float* K, const float* V, int n, int seq,
                              int dk, int use_sparse, int window, int stride, int use_ns,
                              float alpha, float eta, float nu, float* out, int threads) {
    (void)pick_mask(seq, use_sparse, window, stride);
    int nt = threads < 1 ? 1 : (threads < n ? threads : n);
    std::vector<std::thread> pool;
    size_t sz = (size_t)seq * dk;
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([=] {
            for (int i = t; i < n; i += nt)
                ref_attention_full(Q + i * sz, K + i * sz, V + i * sz, seq, dk, use_sparse,
                                   window, stride, use_ns, alpha, eta, nu, out + i * sz);
        });
    for (auto& th : pool) th.join();
}

// n independent heads through navier_stokes_attention alone (alpha == 1, the GPU model's
// setting: no standard path is computed), full causal mask taken from the reference's
// own cache.  Q,K,V,out: [n][seq][dk].
void ref_ns_attention_batch(const float* Q, const float* K, const float* V, int n, int seq,
                            int dk, float eta, float nu, float* out, int threads) {
    const Tensor& mask = causal_mask_cached(seq);
    float T = std::sqrt(static_cast<float>(dk));
    int nt = threads < 1 ? 1 : (threads < n ? threads : n);
    std::vector<std::thread> pool;
    size_t sz = (size_t)seq * dk;
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([=, &mask] {
            for (int i = t; i < n; i += nt)
                put(navier_stokes_attention(make(Q + i * sz, seq, dk), make(K + i * sz, seq, dk),
                                            make(V + i * sz, seq, dk), mask, T, eta, nu),
                    out + i * sz);
        });
    for (auto& th : pool) th.join();
}

// Tensor::fill_random after logos_rng::set_global_seed (Tensor.hpp:14-45,97-104): the
// generator behind the seeded fixtures of the reference's unit tests.
void ref_seed(unsigned seed) { logos_rng::set_global_seed(seed); }
void ref_fill_random(float* out, int rows, int cols, float lo, float hi) {
    Tensor t({rows, cols});
    t.fill_random(lo, hi);
    put(t, out);
}

int ref_hardware_threads() { return (int)std::thread::hardware_concurrency(); }

}  // extern "C"
