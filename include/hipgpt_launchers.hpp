// hipgpt_launchers.hpp — the attention group of HipGPT's kernel API, with the reference's
// exact names and signatures (include/hip_kernels.h:39-46 in the HipGPT tree), defined by this
// library.  C++ linkage on purpose: HipGPT's TransformerLayer and GPTModel objects refer to
// the mangled names, so linking them against libhipgpt_attn.so in place of the reference's
// hip_kernels.o needs no source change.
//
// Behaviour kept from the reference: all pointers are device pointers owned by the caller;
// the call is asynchronous on the legacy default stream (the reference launches with stream
// 0); nothing is returned; a head configuration with H <= 0 or E % H != 0 prints
// "Bad MHA config: E=.. H=.." to stderr and aborts (src/hip_kernels.cpp:410-413).
// Narrower than the reference: head_dim (E / H) up to 512 (the reference's fallback kernel takes any), and at most
// 65535 (batch, head) rows per call of the decode and backward entry points.
// Behaviour added: d_attn_probs may be nullptr on every path (the probabilities are then not
// written); any other failure prints the library's error text to stderr and aborts, where the
// reference would have continued silently.
#pragma once

#if defined(__GNUC__)
#define HIPGPT_LAUNCHER_API __attribute__((visibility("default")))
#else
#define HIPGPT_LAUNCHER_API
#endif

// softmax(Q K^T / sqrt(E/H)) V for every (batch, head); NOT causal, like the reference.
// d_qkv: three stacked [B*S][E] planes; d_output [B*S][E]; d_attn_probs [B][H][S][S] or nullptr.
HIPGPT_LAUNCHER_API void launch_multihead_attention(const float* d_qkv, float* d_output, float* d_attn_probs,
                                int B, int S, int E, int H);
// scores[t][j] = (Q[t] . K[batch(t)][j]) / sqrt(D) on [B][S][D] tensors (B counts batch*heads).
HIPGPT_LAUNCHER_API void launch_scaled_dot_product(const float* Q, const float* K, float* scores, int B, int S, int D);
// Row softmax over the last dimension of [B*S][S].
HIPGPT_LAUNCHER_API void launch_softmax(const float* scores, float* softmax_out, int B, int S);
// output[t][d] = sum_j softmax[t][j] * V[batch(t)][j][d].
HIPGPT_LAUNCHER_API void launch_attention_weighted_sum(const float* softmax, const float* V, float* output, int B, int S, int D);

// ---- the launchers either side of attention in TransformerLayer::forward and GPTModel::forward ----------
// (include/hip_kernels.h:6-7, 16, 29-30, 37, 49, 53 in the HipGPT tree).  Same conventions: device pointers,
// legacy default stream, nothing returned, abort with the library's error text on failure.
// C[M][K] = A[M][N] B[N][K]: N is the inner dimension, as in the reference.
HIPGPT_LAUNCHER_API void launch_matmul(const float* A, const float* B, float* C, int M, int N, int K);
HIPGPT_LAUNCHER_API void launch_matmul_add_bias(const float* A, const float* B, const float* bias, float* C, int M, int N, int K);
HIPGPT_LAUNCHER_API void launch_layer_norm_forward(const float* input, float* output, const float* gamma, const float* beta, int N, int E);
// mask (1 kept, 0 dropped) depends on the element index only; output = input / (1 - p) where kept.
HIPGPT_LAUNCHER_API void launch_dropout_forward(const float* input, float* output, float* mask, float p, int N, int E);
HIPGPT_LAUNCHER_API void launch_add_inplace(float* a, const float* b, int n);
HIPGPT_LAUNCHER_API void launch_relu(float* A, int size);
HIPGPT_LAUNCHER_API void launch_embedding_lookup(const int* d_token_ids, const float* d_token_embed, const float* d_pos_embed,
                             float* d_output, int batch_size, int seq_len, int vocab_size, int embed_dim);

// dQ, dK, dV (three stacked planes in d_grad_qkv) from dO, the stacked Q, K, V planes and the stored
// probabilities (include/hip_kernels.h:59-62).  d_softmax may be nullptr here: the probabilities are then recomputed.
HIPGPT_LAUNCHER_API void launch_multihead_attention_backward(const float* d_grad_attn_output, const float* d_qkv, const float* d_softmax,
                                         float* d_grad_qkv, int B, int S, int E, int H);
