/*
 * Runs HipGPT's own TransformerLayer and GPTModel (their sources compiled where they lie, see
 * oracle/Makefile) on a CUDA device, with every launch_* call on the forward path resolved by this
 * repository's library.  TEST INFRASTRUCTURE ONLY: it shows that the unchanged reference classes run
 * against the library, and gives the GPU tests something to compare with the CPU oracle.
 *
 *   ref_model_run layer <layer.bin> <x.bin> <out.bin> B S E H F
 *       layer.bin: what TransformerLayer::load reads (src/transformer_layer.cpp:347-405);
 *       x.bin: [B*S][E] floats; out.bin receives TransformerLayer::forward's output.
 *   ref_model_run generate <ckpt.bin> V S E H F L n_new id0 id1 ...
 *       ckpt.bin: what GPTModel::load_checkpoint reads (src/gpt_model.cpp:390-420); prints the ids that
 *       GPTModel::generate returns with top_k = 1, temperature 1, no repetition penalty, top_p = 1
 *       (the first maximum of the last row's logits at every step).
 *
 * The training-only launchers that the two sources also name (backward passes, Adam, gradient
 * clipping) are outside the library's path; they are defined here to stop the program loudly.
 */
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "gpt_model.h"
#include "hip_kernels.h"
#include "transformer_layer.h"

#define OUTSIDE(sig) sig { std::fprintf(stderr, "%s: training is outside this library's path\n", __func__); std::abort(); }
OUTSIDE(void launch_matmul_backward_bias(const float*, const float*, float*, float*, int, int, int))
OUTSIDE(void launch_matmul_transpose_A(const float*, const float*, float*, int, int, int))
OUTSIDE(void launch_matmul_transpose_B(const float*, const float*, float*, int, int, int))
OUTSIDE(void launch_backprop_activation(const float*, const float*, float*, int))
OUTSIDE(void launch_embedding_backward(const float*, const int*, float*, float*, int, int, int, int))
OUTSIDE(void launch_adam_update(float*, const float*, float*, float*, float, float, float, float, int, int))
OUTSIDE(void launch_layer_norm_backward(const float*, const float*, float*, const float*, float*, float*, int, int))
OUTSIDE(void launch_dropout_backward(const float*, const float*, float, float*, int, int))
OUTSIDE(void launch_l2_accumulate(const float*, int, float*))
OUTSIDE(void launch_scale_inplace(float*, int, float))
#ifndef HIPGPT_HAVE_ATTENTION_BACKWARD
OUTSIDE(void launch_multihead_attention_backward(const float*, const float*, const float*, float*, int, int, int, int))
#endif

static std::vector<float> read_floats(const char *path, size_t n)
{
    std::vector<float> v(n);
    std::ifstream is(path, std::ios::binary);
    if (!is || !is.read(reinterpret_cast<char *>(v.data()), (std::streamsize)(n * sizeof(float)))) {
        std::fprintf(stderr, "cannot read %zu floats from %s\n", n, path);
        std::exit(2);
    }
    return v;
}

int main(int argc, char **argv)
{
    const std::string mode = argc > 1 ? argv[1] : "";
    if (mode == "layer" && argc == 10) {
        const int B = std::atoi(argv[5]), S = std::atoi(argv[6]), E = std::atoi(argv[7]), H = std::atoi(argv[8]), F = std::atoi(argv[9]);
        const size_t n = (size_t)B * S * E;
        TransformerLayer layer(E, H, F);
        {
            std::ifstream is(argv[2], std::ios::binary);
            if (!is) { std::fprintf(stderr, "cannot open %s\n", argv[2]); return 2; }
            layer.load(is);
        }
        const std::vector<float> x = read_floats(argv[3], n);
        float *d_x = nullptr, *d_y = nullptr;
        if (cudaMalloc(&d_x, n * sizeof(float)) != cudaSuccess || cudaMalloc(&d_y, n * sizeof(float)) != cudaSuccess) return 3;
        cudaMemcpy(d_x, x.data(), n * sizeof(float), cudaMemcpyHostToDevice);
        layer.forward(d_x, d_y, B, S);
        std::vector<float> y(n);
        const cudaError_t e = cudaMemcpy(y.data(), d_y, n * sizeof(float), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { std::fprintf(stderr, "forward failed: %s\n", cudaGetErrorString(e)); return 4; }
        std::ofstream os(argv[4], std::ios::binary);
        os.write(reinterpret_cast<const char *>(y.data()), (std::streamsize)(n * sizeof(float)));
        cudaFree(d_x);
        cudaFree(d_y);
        return os ? 0 : 5;
    }
    if (mode == "generate" && argc >= 11) {
        const int V = std::atoi(argv[3]), S = std::atoi(argv[4]), E = std::atoi(argv[5]), H = std::atoi(argv[6]), F = std::atoi(argv[7]),
                  L = std::atoi(argv[8]), n_new = std::atoi(argv[9]);
        std::vector<int> prompt;
        for (int i = 10; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
        GPTModel model(V, S, E, H, F, L);
        model.load_checkpoint(argv[2]);
        const std::vector<int> out = model.generate(prompt, n_new, /*top_k=*/1, /*temperature=*/1.0f, /*rep_penalty=*/1.0f, /*top_p=*/1.0f);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { std::fprintf(stderr, "generate failed: %s\n", cudaGetErrorString(e)); return 4; }
        for (size_t i = prompt.size(); i < out.size(); ++i) std::printf("%d%c", out[i], i + 1 == out.size() ? '\n' : ' ');
        return 0;
    }
    std::fprintf(stderr, "usage: %s layer <layer.bin> <x.bin> <out.bin> B S E H F | generate <ckpt.bin> V S E H F L n_new ids...\n", argv[0]);
    return 1;
}
