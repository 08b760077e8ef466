// Test driver for the drop-in symbol: what ModelGPU::forward does per head (cuda/ModelGPU.cu:959-968),
// written against nothing but the reference's declaration of cuda_flash_attention_fwd.
//   shim_driver <in.bin> <out.bin> seq DH window stride
// in.bin = Q, K, V as fp32 [seq][DH] each; out.bin = the attention output.  Afterwards the call is
// repeated with DH = 256, which the reference rejects with an exception (cuda/VedicGEMM.cu:1074-1079).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <vector>

void cuda_flash_attention_fwd(const float* Q, const float* K, const float* V, float* out, float* attn_ptr,
                              int seq, int DH, float scale, bool causal, bool shunyam, int window, int stride);

int main(int argc, char** argv) {
    if (argc != 7) return 2;
    const int seq = atoi(argv[3]), DH = atoi(argv[4]), window = atoi(argv[5]), stride = atoi(argv[6]);
    const size_t n = (size_t)seq * DH;
    std::vector<float> h(3 * n), o(n);
    FILE* f = fopen(argv[1], "rb");
    if (!f || fread(h.data(), sizeof(float), 3 * n, f) != 3 * n) return 3;
    fclose(f);
    float *dQ, *dK, *dV, *dO;
    if (cudaMalloc(&dQ, n * 4) || cudaMalloc(&dK, n * 4) || cudaMalloc(&dV, n * 4) || cudaMalloc(&dO, n * 4)) return 4;
    cudaMemcpy(dQ, h.data(), n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dK, h.data() + n, n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dV, h.data() + 2 * n, n * 4, cudaMemcpyHostToDevice);
    cuda_flash_attention_fwd(dQ, dK, dV, dO, nullptr, seq, DH, 1.0f / sqrtf((float)DH), true, window > 0, window, stride);
    if (cudaDeviceSynchronize() != cudaSuccess) return 5;
    cudaMemcpy(o.data(), dO, n * 4, cudaMemcpyDeviceToHost);
    f = fopen(argv[2], "wb");
    if (!f || fwrite(o.data(), sizeof(float), n, f) != n) return 6;
    fclose(f);
    try {
        cuda_flash_attention_fwd(dQ, dK, dV, dO, nullptr, seq, 256, 0.0625f, true, false, 0, 0);
        printf("accepted\n");
    } catch (const std::runtime_error& e) {      // the type the reference throws (cuda/VedicGEMM.cu:1074-1079)
        printf("rejected: %s\n", e.what());
    } catch (const std::exception& e) {
        printf("wrong exception type: %s\n", e.what());
    }
    return 0;
}
