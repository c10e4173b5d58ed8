// Reference-named entry points over the C ABI (declared in include/hipgpt_launchers.hpp).
// Each one stands where HipGPT's own definition stood: launch_multihead_attention
// (src/hip_kernels.cpp:404-451), launch_scaled_dot_product (:468-473), launch_softmax
// (:506-511), launch_attention_weighted_sum (:527-532).
#include "hipgpt_launchers.hpp"

#include <cstdio>
#include <cstdlib>

#include "hipgpt_attn.h"

namespace {
void die_on(int rc, const char* what)
{
    if (rc == HIPGPT_OK) return;
    std::fprintf(stderr, "%s failed (%d): %s\n", what, rc, hipgpt_last_error());
    std::abort();
}
}  // namespace

void launch_multihead_attention(const float* d_qkv, float* d_output, float* d_attn_probs,
                                int B, int S, int E, int H)
{
    if (H <= 0 || (E % H) != 0) {
        std::fprintf(stderr, "Bad MHA config: E=%d H=%d\n", E, H);
        std::abort();
    }
    die_on(hipgpt_mha_forward_planes(d_qkv, d_output, d_attn_probs, B, S, E, H, /*causal=*/0, /*stream=*/nullptr),
           "launch_multihead_attention");
}

void launch_scaled_dot_product(const float* Q, const float* K, float* scores, int B, int S, int D)
{
    die_on(hipgpt_scaled_dot_product(Q, K, scores, B, S, D, nullptr), "launch_scaled_dot_product");
}

void launch_softmax(const float* scores, float* softmax_out, int B, int S)
{
    die_on(hipgpt_softmax(scores, softmax_out, B, S, nullptr), "launch_softmax");
}

void launch_attention_weighted_sum(const float* softmax, const float* V, float* output, int B, int S, int D)
{
    die_on(hipgpt_attention_weighted_sum(softmax, V, output, B, S, D, nullptr), "launch_attention_weighted_sum");
}
