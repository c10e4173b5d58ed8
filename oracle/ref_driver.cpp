/*
 * C entry points over the reference's own launchers, built on host cores.  TEST
 * INFRASTRUCTURE ONLY.  This translation unit supplies the storage that the host stand-in
 * for <hip/hip_runtime.h> declares and forwards plain-C calls to the functions that
 * HipGPT's src/hip_kernels.cpp defines (include/hip_kernels.h:39-46).  All pointers are
 * host pointers.  Built by oracle/Makefile into oracle/_ref/libhipgpt_ref.so.
 */
#include <hip/hip_runtime.h>
#include "hip_kernels.h"
#ifdef _OPENMP
#include <omp.h>
#endif

thread_local dim3 threadIdx, blockIdx, blockDim, gridDim;
int hipgpt_ref_unique_rows_only = 0;

/* `extern __shared__` arrays named by kernels that this library never runs
 * (layer norm, layer-norm backward, sampler, l2 norm); they only need to link. */
float smem[1];
float shm[1];
unsigned char smem_u8_logits[1];
float shmem[1];

extern "C" {

__attribute__((visibility("default")))
void ref_mha(const float *qkv, float *out, float *probs, int B, int S, int E, int H, int unique_rows_only)
{
    hipgpt_ref_unique_rows_only = unique_rows_only;
    launch_multihead_attention(qkv, out, probs, B, S, E, H);
    hipgpt_ref_unique_rows_only = 0;
}

__attribute__((visibility("default")))
void ref_sdp(const float *Q, const float *K, float *scores, int B, int S, int D)
{
    launch_scaled_dot_product(Q, K, scores, B, S, D);
}

__attribute__((visibility("default")))
void ref_softmax(const float *scores, float *out, int B, int S)
{
    launch_softmax(scores, out, B, S);
}

__attribute__((visibility("default")))
void ref_weighted_sum(const float *P, const float *V, float *out, int B, int S, int D)
{
    launch_attention_weighted_sum(P, V, out, B, S, D);
}

/* The elementwise launchers around the attention call in the reference's layer and model forward
 * (src/transformer_layer.cpp:242,250; src/gpt_model.cpp:107): none of their kernels synchronises
 * threads, so the loop form of a launch is valid for them. */
__attribute__((visibility("default")))
void ref_dropout_forward(const float *in, float *out, float *mask, float p, int N, int E)
{
    launch_dropout_forward(in, out, mask, p, N, E);
}

__attribute__((visibility("default")))
void ref_embedding_lookup(const int *ids, const float *tok, const float *pos, float *out, int B, int S, int V, int E)
{
    launch_embedding_lookup(ids, tok, pos, out, B, S, V, E);
}

/* The attention backward launcher (src/hip_kernels.cpp:1242-1272).  Its kernel adds into dK and dV with
 * atomicAdd, which the host stand-in runs as a plain add: call it with ONE host thread (ref_set_num_threads(1)),
 * where the order of those additions is ascending in the query index. */
__attribute__((visibility("default")))
void ref_mha_backward(const float *gout, const float *qkv, const float *probs, float *gqkv, int B, int S, int E, int H)
{
    launch_multihead_attention_backward(gout, qkv, probs, gqkv, B, S, E, H);
}

__attribute__((visibility("default")))
int ref_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

__attribute__((visibility("default")))
void ref_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

} /* extern "C" */
