// ref_model_harness.cu -- the reference's own GPU model run on a small seeded configuration.
//
// TEST INFRASTRUCTURE ONLY.  Nothing of the model is written here: ModelGPU comes from the reference's
// cuda/ModelGPU.cu and cuda/VedicGEMM.cu, compiled unmodified from the reference tree (Makefile in
// this folder).  The program is built twice from this one source:
//   refmodel_stock   everything from the reference, its own cuda_flash_attention_fwd included;
//   refmodel_dropin  cuda/VedicGEMM.cu compiled with its definition of cuda_flash_attention_fwd renamed
//                    away, so that the call in ModelGPU::forward (cuda/ModelGPU.cu:959-968) binds to
//                    the symbol of the same name in liblogos_attn_shim.so -- the link-time drop-in.
// Both fill every parameter from the same generator, run ModelGPU::forward on the same token ids and
// write the logits; a test compares the two files.
//   refmodel_* <out.bin> vocab d_model heads layers seq window stride
#include "ModelGPU.cuh"

#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

int main(int argc, char** argv) {
    if (argc != 9) return 2;
    ModelConfig cfg;
    cfg.vocab_size = atoi(argv[2]);
    cfg.d_model = atoi(argv[3]);
    cfg.num_heads = atoi(argv[4]);
    cfg.num_layers = atoi(argv[5]);
    const int seq = atoi(argv[6]);
    cfg.max_seq_len = seq;
    HyperConfig hyper;
    hyper.enabled = false;
    try {
        ModelGPU model(cfg, hyper);
        model.phys.window = atoi(argv[7]);
        model.phys.stride = atoi(argv[8]);
        model.phys.shunyam = model.phys.window > 0;
        model.phys.feynman_dropout = false;
        model.phys.training = false;
        std::mt19937 gen(20240u);
        std::normal_distribution<float> nd(0.0f, 0.05f);
        for (GPUTensor* p : model.all_parameters()) {
            std::vector<float> h((size_t)p->size);
            for (float& x : h) x = nd(gen);
            // LayerNorm scales stay near one so that the activations keep a usable range
            if (p->rows == 1 && p->cols == cfg.d_model) for (float& x : h) x += 1.0f;
            h2d(*p, h.data(), p->size);
        }
        std::vector<int> ids((size_t)seq);
        for (int i = 0; i < seq; ++i) ids[i] = (int)(gen() % (unsigned)cfg.vocab_size);
        GPUTensor logits = model.forward(ids);
        if (cudaDeviceSynchronize() != cudaSuccess) return 5;
        std::vector<float> out((size_t)seq * cfg.vocab_size);
        d2h(out.data(), logits, (int)out.size());
        FILE* f = fopen(argv[1], "wb");
        if (!f || fwrite(out.data(), sizeof(float), out.size(), f) != out.size()) return 6;
        fclose(f);
    } catch (const std::exception& e) {
        fprintf(stderr, "refmodel: %s\n", e.what());
        return 7;
    }
    return 0;
}
