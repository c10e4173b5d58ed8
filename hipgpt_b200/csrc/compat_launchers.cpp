// Reference-named entry points over the C ABI (declared in include/hipgpt_launchers.hpp).
// Each one stands where HipGPT's own definition stood: launch_multihead_attention
// (src/hip_kernels.cpp:404-451), launch_scaled_dot_product (:468-473), launch_softmax
// (:506-511), launch_attention_weighted_sum (:527-532); and the launchers either side of attention in
// TransformerLayer::forward / GPTModel::forward: launch_matmul (:102-109), launch_matmul_add_bias (:147-154),
// launch_layer_norm_forward (:838-848), launch_dropout_forward (:966-970), launch_add_inplace (:726-730),
// launch_relu (:254-258), launch_embedding_lookup (:583-599); and launch_multihead_attention_backward (:1242-1272).
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

// HIPGPT_FAST_MATMUL=1 in the environment sends the products that are not in place to the tensor-core kernel (fp32-grade
// instead of the reference's summation order bit for bit); the in-place output projection
// (src/transformer_layer.cpp:220) and everything else keep the exact kernel.
static bool fast_matmul()
{
    static const bool on = [] { const char *e = getenv("HIPGPT_FAST_MATMUL"); return e && *e && *e != '0'; }();
    return on;
}

void launch_matmul(const float* A, const float* B, float* C, int M, int N, int K)
{
    if (fast_matmul() && C != A && C != B && N > 0) die_on(hipgpt_matmul_tc(A, B, nullptr, C, M, N, K, nullptr), "launch_matmul");
    else die_on(hipgpt_matmul(A, B, nullptr, C, M, N, K, nullptr), "launch_matmul");
}

void launch_matmul_add_bias(const float* A, const float* B, const float* bias, float* C, int M, int N, int K)
{
    if (fast_matmul() && C != A && C != B && N > 0) die_on(hipgpt_matmul_tc(A, B, bias, C, M, N, K, nullptr), "launch_matmul_add_bias");
    else die_on(hipgpt_matmul(A, B, bias, C, M, N, K, nullptr), "launch_matmul_add_bias");
}

void launch_layer_norm_forward(const float* input, float* output, const float* gamma, const float* beta, int N, int E)
{
    die_on(hipgpt_layer_norm(input, output, gamma, beta, N, E, nullptr), "launch_layer_norm_forward");
}

void launch_dropout_forward(const float* input, float* output, float* mask, float p, int N, int E)
{
    die_on(hipgpt_dropout(input, output, mask, p, N, E, nullptr), "launch_dropout_forward");
}

void launch_add_inplace(float* a, const float* b, int n)
{
    die_on(hipgpt_add_inplace(a, b, n, nullptr), "launch_add_inplace");
}

void launch_relu(float* A, int size)
{
    die_on(hipgpt_relu(A, size, nullptr), "launch_relu");
}

void launch_embedding_lookup(const int* d_token_ids, const float* d_token_embed, const float* d_pos_embed,
                             float* d_output, int batch_size, int seq_len, int vocab_size, int embed_dim)
{
    die_on(hipgpt_embedding_lookup(d_token_ids, d_token_embed, d_pos_embed, d_output, batch_size, seq_len, vocab_size, embed_dim, nullptr),
           "launch_embedding_lookup");
}

void launch_multihead_attention_backward(const float* d_grad_attn_output, const float* d_qkv, const float* d_softmax,
                                         float* d_grad_qkv, int B, int S, int E, int H)
{
    die_on(hipgpt_mha_backward_planes(d_grad_attn_output, d_qkv, d_softmax, d_grad_qkv, B, S, E, H, /*causal=*/0, nullptr),
           "launch_multihead_attention_backward");
}
