/*
 * hipgpt_attn.h — C ABI of the B200 (sm_100a) attention-forward library.
 *
 * The library replaces the attention group of HipGPT's kernel API
 * (include/hip_kernels.h:38-46 there) with hand-written CUDA kernels.  Two layers:
 *
 *   1. the C entry points below: plain pointers and sizes, an explicit stream, an int status;
 *   2. include/hipgpt_launchers.hpp: C++ functions with the reference's exact names and
 *      signatures (launch_multihead_attention, ...) that forward here, so that HipGPT's
 *      TransformerLayer / GPTModel objects link against this library unchanged.
 *
 * Conventions shared by every entry point
 *   - pointers named d_* are DEVICE pointers, h_* are HOST pointers; the caller owns them all;
 *   - nothing is allocated, kept or freed by the device-pointer entry points;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is
 *     what the reference's hipLaunchKernelGGL(..., 0, 0, ...) calls use); calls are
 *     asynchronous with respect to the host;
 *   - the return value is HIPGPT_OK or a negative HIPGPT_ERR_* code; hipgpt_last_error()
 *     then describes the failure for the calling thread.  Nothing aborts here; the
 *     reference-named wrappers reproduce the reference's abort on a bad head configuration;
 *   - all arithmetic is fp32; offsets are 64-bit, so planes and probability tensors beyond
 *     2^31 elements are addressed correctly.
 */
#ifndef HIPGPT_ATTN_H
#define HIPGPT_ATTN_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility; these are its exports. */
#if defined(__GNUC__)
#define HIPGPT_API __attribute__((visibility("default")))
#else
#define HIPGPT_API
#endif

#define HIPGPT_OK               0
#define HIPGPT_ERR_BAD_ARG     (-1)   /* a size is negative, H <= 0, E % H != 0, ctx > cap ...   */
#define HIPGPT_ERR_NULL        (-2)   /* a required pointer is NULL                              */
#define HIPGPT_ERR_UNSUPPORTED (-3)   /* head_dim beyond what the kernels hold in registers      */
#define HIPGPT_ERR_CUDA        (-4)   /* the CUDA runtime reported an error (text in last_error) */
#define HIPGPT_ERR_SCRATCH     (-5)   /* scratch buffer missing or smaller than required         */

/* Kernel selector of hipgpt_mha_forward_ex (profiling and tests; 0 is what every other
 * entry point uses). */
#define HIPGPT_ALGO_AUTO     0   /* tensor-core kernels for head_dim 32/64 (with or without the
                                    probabilities), FFMA rows kernel for head_dim 128, generic kernel
                                    for every other head_dim                                        */
#define HIPGPT_ALGO_GENERIC  1   /* one warp per query row, any head_dim <= 512                    */
#define HIPGPT_ALGO_ROWS     2   /* exact fp32 FFMA: register-resident query rows, shared-memory K/V */
#define HIPGPT_ALGO_TENSOR   3   /* tcgen05 kernels, head_dim 32/64; `warps` picks one of HIPGPT_TENSOR_* */

/* Tensor-core kernels (the `warps` argument of hipgpt_mha_forward_ex with HIPGPT_ALGO_TENSOR). */
#define HIPGPT_TENSOR_DEFAULT     0   /* what HIPGPT_ALGO_AUTO runs: WHOLE_HEAD where it applies, else TILED */
#define HIPGPT_TENSOR_SPLIT_TF32  1   /* three TF32 products per product: 1e-5 accuracy over the whole fp32 range;
                                         stores no probabilities                                                */
#define HIPGPT_TENSOR_TILED       5   /* TF32 main products + FP16 correction products, 64-key tiles, any S;
                                         stores the probabilities by a second sweep when asked                  */
#define HIPGPT_TENSOR_WHOLE_HEAD  6   /* head_dim 32, S <= 256: one block per (batch, head), TMA loads, 128-key
                                         products, every score tile of the head in tensor memory                */

/*
 * Fused multi-head attention forward:  out = softmax(Q K^T / sqrt(D)) V  per (batch, head).
 * Replaces launch_multihead_attention's two kernels (src/hip_kernels.cpp:263-325 and
 * :329-402, dispatch :404-451).
 *   d_q, d_k, d_v  [B*S][E] fp32; head h of token t at t*E + h*D, D = E/H
 *   d_out          [B*S][E], same indexing, fully overwritten
 *   d_probs        [B][H][S][S] normalised probabilities, fully overwritten, or NULL to skip
 *   causal         0 = the reference's semantics (every query sees all S keys);
 *                  1 = extension: query i sees keys j <= i; stored probabilities above the
 *                      diagonal are 0
 */
HIPGPT_API int hipgpt_mha_forward(const float *d_q, const float *d_k, const float *d_v,
                       float *d_out, float *d_probs,
                       int B, int S, int E, int H, int causal, void *stream);

/* The same with an explicit kernel selector (HIPGPT_ALGO_*).  `warps`: for HIPGPT_ALGO_ROWS the
 * number of warps per thread block (0 = default); for HIPGPT_ALGO_TENSOR one of HIPGPT_TENSOR_*.
 * Every kernel holds 1e-5 on unit-scale data.  TILED scales its operands into fp16's range by exact powers of two
 * (per query row, per 64-key tile of K and of V) and keeps that accuracy for any fp32 magnitude; it keeps the fp16
 * images of K and V in a buffer of the library (per device and stream; hipgpt_release_workspace() frees it).
 * WHOLE_HEAD keeps the accuracy while Q and K stay within fp16's range (about 1e-4 .. 6e4; it rescales V by a
 * power of two per head, so V may have any magnitude); outside it its correction terms saturate or are flushed,
 * the result falls to plain TF32 grade (~3e-4 relative), and the launch raises the flag that
 * hipgpt_accuracy_notice() reports.  SPLIT_TF32 and the FFMA kernels have the full fp32 range. */
HIPGPT_API int hipgpt_mha_forward_ex(const float *d_q, const float *d_k, const float *d_v,
                          float *d_out, float *d_probs,
                          int B, int S, int E, int H, int causal,
                          int algo, int warps, void *stream);

/* The launcher's own view of its input: d_qkv holds three stacked [B*S][E] planes, Q then K
 * then V (src/hip_kernels.cpp:415-417). */
HIPGPT_API int hipgpt_mha_forward_planes(const float *d_qkv, float *d_out, float *d_probs,
                              int B, int S, int E, int H, int causal, void *stream);

/*
 * The same attention with 16-bit storage: d_q, d_k, d_v are [B*S][E] planes of bf16 (IEEE
 * bfloat16, the upper half of an fp32), d_out is [B*S][E] bf16; products run on the tensor
 * cores with fp32 accumulation, the softmax in fp32.  head_dim (E/H) must be 64, the four
 * pointers 16-byte aligned.  Results agree with the fp32 arithmetic on the same
 * (bf16-rounded) inputs to about 1e-2 absolute for unit-variance data: the probabilities and
 * the output are rounded to bf16.  No probabilities are written.
 */
HIPGPT_API int hipgpt_mha_forward_bf16(const void *d_q, const void *d_k, const void *d_v, void *d_out,
                            int B, int S, int E, int H, int causal, void *stream);
/* The same call with a `variant` argument that earlier versions used to choose between schedules of the
 * kernel.  There is one schedule now: 0, 1 and 2 are accepted and run it, anything else is refused. */
HIPGPT_API int hipgpt_mha_forward_bf16_ex(const void *d_q, const void *d_k, const void *d_v, void *d_out,
                               int B, int S, int E, int H, int causal, int variant, void *stream);

/* The same call for HOST buffers: copies the planes to the device, runs the kernel, copies
 * the output (and the probabilities when h_probs is not NULL) back and waits.  The device
 * workspace is owned by the library, grows to the largest call and is released by
 * hipgpt_release_workspace().  Pinned host memory makes the copies asynchronous. */
HIPGPT_API int hipgpt_mha_forward_host(const float *h_qkv, float *h_out, float *h_probs,
                            int B, int S, int E, int H, int causal);
/* The host-buffer call for bf16 planes (hipgpt_mha_forward_bf16's contract: h_qkv = three stacked
 * [B*S][E] bf16 planes, h_out [B*S][E] bf16, head_dim 64, no probabilities); same workspace. */
HIPGPT_API int hipgpt_mha_forward_bf16_host(const void *h_qkv, void *h_out, int B, int S, int E, int H, int causal);
HIPGPT_API void hipgpt_release_workspace(void);

/*
 * The unfused chain, head-contiguous layout: Q, K, V, out are [B'][S][D] (the caller folds
 * heads into B'), scores / probabilities are [B'][S][S].
 *   hipgpt_scaled_dot_product       replaces launch_scaled_dot_product      (src/hip_kernels.cpp:455-473)
 *   hipgpt_softmax                  replaces launch_softmax                 (src/hip_kernels.cpp:478-511)
 *   hipgpt_attention_weighted_sum   replaces launch_attention_weighted_sum  (src/hip_kernels.cpp:514-532)
 * The two contractions keep the reference's summation order (one accumulator, ascending
 * index, fused multiply-add), so they are equal bit for bit to that arithmetic.
 */
HIPGPT_API int hipgpt_scaled_dot_product(const float *d_Q, const float *d_K, float *d_scores,
                              int B, int S, int D, void *stream);
HIPGPT_API int hipgpt_softmax(const float *d_scores, float *d_softmax_out, int B, int S, void *stream);
HIPGPT_API int hipgpt_attention_weighted_sum(const float *d_softmax, const float *d_V, float *d_output,
                                  int B, int S, int D, void *stream);

/*
 * Attention backward: gradients of Q, K, V from the gradient of the attention output.  Replaces
 * launch_multihead_attention_backward (src/hip_kernels.cpp:1162-1272, declared include/hip_kernels.h:59-62,
 * called at src/transformer_layer.cpp:285-286).
 *   d_grad_out     [B*S][E]   dL/d(output); d_q, d_k, d_v as in hipgpt_mha_forward
 *   d_probs        [B][H][S][S] as hipgpt_mha_forward stored them, or NULL: the probabilities are then formed
 *                  again from Q and K (row maxima and sums recomputed first), so the forward need not have
 *                  written them at all
 *   d_grad_q/k/v   [B*S][E], fully overwritten
 *   d_scratch      hipgpt_mha_backward_scratch_bytes(B, H, S) bytes (2 B H S floats)
 * No atomics: a key row's gradients add its queries in ascending order, so results are reproducible run to
 * run (the reference's atomicAdd order is not); they agree with the reference's arithmetic to rounding.
 * hipgpt_mha_backward_planes is the launcher's own view (three stacked planes in d_qkv and d_grad_qkv) with
 * the scratch kept in a buffer of the library, which grows with cudaMalloc to the largest call per device.
 */
HIPGPT_API size_t hipgpt_mha_backward_scratch_bytes(int B, int H, int S);
HIPGPT_API int hipgpt_mha_backward(const float *d_grad_out, const float *d_q, const float *d_k, const float *d_v, const float *d_probs,
                        float *d_grad_q, float *d_grad_k, float *d_grad_v, float *d_scratch, size_t scratch_bytes,
                        int B, int S, int E, int H, int causal, void *stream);
HIPGPT_API int hipgpt_mha_backward_planes(const float *d_grad_out, const float *d_qkv, const float *d_probs, float *d_grad_qkv,
                               int B, int S, int E, int H, int causal, void *stream);

/*
 * The launchers either side of attention in the reference's layer and model forward, restated with the
 * reference's arithmetic (device pointers, explicit stream):
 *   hipgpt_matmul            C[M][K] = A[M][N] B[N][K] (+ bias[K] when d_bias is not NULL); the reference's
 *                            argument order, N being the inner dimension.  Replaces launch_matmul and
 *                            launch_matmul_add_bias (src/hip_kernels.cpp:69-154): one accumulator per output,
 *                            k ascending, fused multiply-add, bias added once at the end, so bit-identical to
 *                            that arithmetic.  d_A == d_C (the reference's in-place output projection,
 *                            src/transformer_layer.cpp:220) is allowed when K <= 256 and K % 4 == 0.
 *   hipgpt_matmul_tc         the same product on the tensor pipe (tcgen05): every operand cut into fp16 pieces after a
 *                            power-of-two scaling (per row of A, one for B), three products per product, fp32
 *                            accumulation: 1e-5 on unit-scale data instead of identical bits, several times the
 *                            rate.  Not in place.  The packed operands live in a buffer of the library (per device
 *                            and stream; hipgpt_release_workspace() frees it).
 *   hipgpt_matmul_tc_prepare / _prepared / _release
 *                            the same with the right-hand side (a layer's weights) packed once: prepare() allocates
 *                            device memory for B's packed form and fills it (asynchronously on `stream`; B may be
 *                            freed once that stream has passed the call), prepared() multiplies any number of A's
 *                            with it (on streams ordered after it), release() frees it.  Saves two of the four
 *                            launches of every product.
 *   hipgpt_ln_matmul_tc, hipgpt_ln_matmul_tc_prepared
 *                            C = LayerNorm(A) B (+ bias): the layer norm before each projection of the reference's
 *                            block (src/transformer_layer.cpp:240-241 and 246-247) done by the kernel that packs
 *                            A, so it costs no pass over memory and no launch of its own; fp32-grade like the product.
 *   hipgpt_layer_norm        replaces launch_layer_norm_forward (src/hip_kernels.cpp:757-848), eps 1e-5;
 *                            agrees with the reference's 64-lane reduction order to rounding (~1e-7).
 *   hipgpt_dropout           replaces launch_dropout_forward (src/hip_kernels.cpp:944-970): the mask depends
 *                            on the element index only (generator at :24-42); bit-identical; d_mask may be
 *                            NULL; in place (d_in == d_out) allowed.
 *   hipgpt_dropout_residual  out = residual + dropout(in): the tail of each sub-layer of the reference's block
 *                            (src/transformer_layer.cpp:242-244, 250-252: dropout in place, device copy, add) in one
 *                            pass over memory; bit-identical to hipgpt_dropout followed by hipgpt_add_inplace; d_out
 *                            may be d_in or d_residual; d_mask may be NULL.
 *   hipgpt_add_inplace       a += b           (launch_add_inplace, src/hip_kernels.cpp:721-730)
 *   hipgpt_relu              a = max(0, a)    (launch_relu, src/hip_kernels.cpp:248-258)
 *   hipgpt_embedding_lookup  out[t] = tok[id_t] + pos[t mod S], zeros for an id outside [0, V)
 *                            (launch_embedding_lookup, src/hip_kernels.cpp:537-599)
 */
HIPGPT_API int hipgpt_matmul(const float *d_A, const float *d_B, const float *d_bias, float *d_C, int M, int N, int K, void *stream);
HIPGPT_API int hipgpt_matmul_tc(const float *d_A, const float *d_B, const float *d_bias, float *d_C, int M, int N, int K, void *stream);
typedef struct hipgpt_packed_matrix hipgpt_packed_matrix;
HIPGPT_API int hipgpt_matmul_tc_prepare(const float *d_B, int N, int K, hipgpt_packed_matrix **out, void *stream);
HIPGPT_API int hipgpt_matmul_tc_prepared(const float *d_A, const hipgpt_packed_matrix *b, const float *d_bias, float *d_C, int M, void *stream);
HIPGPT_API void hipgpt_matmul_tc_release(hipgpt_packed_matrix *b);
HIPGPT_API int hipgpt_ln_matmul_tc(const float *d_A, const float *d_gamma, const float *d_beta, const float *d_B, const float *d_bias, float *d_C,
                        int M, int N, int K, void *stream);
HIPGPT_API int hipgpt_ln_matmul_tc_prepared(const float *d_A, const float *d_gamma, const float *d_beta, const hipgpt_packed_matrix *b,
                                 const float *d_bias, float *d_C, int M, void *stream);
HIPGPT_API int hipgpt_layer_norm(const float *d_in, float *d_out, const float *d_gamma, const float *d_beta, int rows, int E, void *stream);
HIPGPT_API int hipgpt_dropout(const float *d_in, float *d_out, float *d_mask, float p, int rows, int E, void *stream);
HIPGPT_API int hipgpt_dropout_residual(const float *d_in, const float *d_residual, float *d_out, float *d_mask, float p, int rows, int E, void *stream);
HIPGPT_API int hipgpt_add_inplace(float *d_a, const float *d_b, long long n, void *stream);
HIPGPT_API int hipgpt_relu(float *d_a, long long n, void *stream);
HIPGPT_API int hipgpt_embedding_lookup(const int *d_ids, const float *d_tok, const float *d_pos, float *d_out,
                            int B, int S, int V, int E, void *stream);

/*
 * Single-query-row attention over a key/value cache, split over the context (extension; the
 * reference's generation loop, src/gpt_model.cpp:261-280, re-runs the whole window instead).
 *   d_q, d_out       [B][E]          the new token's query / the attention output
 *   d_kcache/vcache  [B][cap][E]     head h of position j at (b*cap + j)*E + h*D
 *   ctx              positions 0..ctx-1 are attended (ctx <= cap)
 *   d_scratch        hipgpt_mha_decode_scratch_bytes(B, H, D, ctx) bytes of device memory for
 *                    the per-split partial results (may be NULL when that size is 0)
 */
HIPGPT_API size_t hipgpt_mha_decode_scratch_bytes(int B, int H, int D, int ctx);
HIPGPT_API int hipgpt_mha_decode(const float *d_q, const float *d_kcache, const float *d_vcache, float *d_out,
                      float *d_scratch, size_t scratch_bytes,
                      int B, int H, int D, int ctx, int cap, void *stream);

/*
 * The same decode for callers that have no scratch to give and may not allocate (no counterpart
 * in the reference).  HipGPT-style call sites are stateless `void launch_x(pointers, ints)`
 * functions under objects that allocate a fixed set of buffers per shape; a per-token
 * generation loop built on them has nowhere to keep a scratch pointer, and a cudaMalloc in
 * that loop would synchronise the device (or be refused by a process whose pool already owns
 * the memory).  Here the partial results live in a fixed array inside the library image
 * (HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES on every GPU that loads the library, until exit).
 *   - a call whose partial results do not fit returns HIPGPT_ERR_SCRATCH;
 *   - all calls on a GPU share that array: calls that may overlap on the GPU race, order them;
 *   - nothing is allocated or freed; every call looks up the array's device address (nothing is
 *     cached, so the entry point stays valid across a cudaDeviceReset); the first lookup on a
 *     device loads the library's module there, so make that call before any stream capture
 *     starts on the device.
 */
#define HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES (1u << 20)
HIPGPT_API int hipgpt_mha_decode_noalloc(const float *d_q, const float *d_kcache, const float *d_vcache, float *d_out,
                              int B, int H, int D, int ctx, int cap, void *stream);

/*
 * Greedy generation with a HipGPT-shaped model on one GPU, KV-cache form: the host driver that
 * stands where GPTModel::generate's loop stands (src/gpt_model.cpp:248-353) for the benchmark's
 * whole-model shape.  Every token runs once, at its own position, against cached keys and
 * values (hipgpt_mha_decode's kernels); no dropout; the next id is the first maximum of the
 * logits and stays on the device.  The reference instead re-runs a left-padded, unmasked window
 * of max_seq_len tokens per token and samples on the host; results of the two are not comparable.
 *   h_weights  fp32 blob in the reference's checkpoint order without its integer headers
 *              (src/gpt_model.cpp:355-420, src/transformer_layer.cpp:312-405): tok_emb[V][E],
 *              pos_emb[S][E], per layer {Wqkv[E][3E], Wo[E][E], W1[E][F], W2[F][E], bqkv, bo, b1, b2,
 *              attn gamma, beta, ffn gamma, beta}, out_proj[E][V]; hipgpt_gpt_weight_count floats
 *   h_prompts  [B][n_prompt] token ids; h_out_ids [B][n_new]; h_logits_last [B][V] or NULL
 *   ms_prompt / ms_decode  (optional) device time of the n_prompt prompt steps / the n_new-1 later steps
 */
typedef struct hipgpt_gpt hipgpt_gpt;
HIPGPT_API long long hipgpt_gpt_weight_count(int V, int S, int E, int L, int H, int F);
HIPGPT_API int hipgpt_gpt_create(hipgpt_gpt **out, const float *h_weights, int V, int S, int E, int L, int H, int F,
                      int max_batch);
HIPGPT_API int hipgpt_gpt_generate(hipgpt_gpt *g, const int *h_prompts, int B, int n_prompt, int n_new, int *h_out_ids,
                        float *h_logits_last, float *ms_prompt, float *ms_decode);
HIPGPT_API void hipgpt_gpt_destroy(hipgpt_gpt *g);
/*
 * HipGPT's own files (host code): the checkpoint written by GPTModel::save_checkpoint (src/gpt_model.cpp:355-388;
 * per layer src/transformer_layer.cpp:312-344; read back at src/gpt_model.cpp:390-420) and the run configuration
 * written by save_config (src/train_gpt.cpp:60-102; read at src/generate.cpp:90-103).
 *   hipgpt_checkpoint_header   V, S, E, L from the file's header, H and F from the first layer's
 *   hipgpt_checkpoint_weights  the tensors in file order without the integer headers (what hipgpt_gpt_create takes):
 *                              `count` must be hipgpt_gpt_weight_count(V, S, E, L, H, F); every layer's header is checked
 *   hipgpt_run_config          the six "model" numbers and, when asked, "checkpoint"."latest" and "tokenizer"."path"
 *                              (file names relative to the configuration's own directory)
 *   hipgpt_gpt_create_from_checkpoint / _from_run   the generation driver for such a file
 */
HIPGPT_API int hipgpt_checkpoint_header(const char *path, int *V, int *S, int *E, int *L, int *H, int *F);
HIPGPT_API int hipgpt_checkpoint_weights(const char *path, float *h_weights, long long count);
HIPGPT_API int hipgpt_run_config(const char *json_path, int *V, int *S, int *E, int *H, int *F, int *L,
                      char *ckpt_name, size_t ckpt_cap, char *tok_name, size_t tok_cap);
HIPGPT_API int hipgpt_gpt_create_from_checkpoint(hipgpt_gpt **out, const char *path, int max_batch);
HIPGPT_API int hipgpt_gpt_create_from_run(hipgpt_gpt **out, const char *json_path, int max_batch);

/*
 * Two forms of the same token step, same arithmetic and the same ids (extension, like the driver itself):
 *   HIPGPT_GPT_MODE_GRAPH (default): one step = 52 kernel launches captured once as a CUDA graph and replayed
 *     per token.
 *   HIPGPT_GPT_MODE_PERSISTENT (head_dim % 4 == 0 and head_dim <= 128): one cooperative launch runs all
 *     prompt positions, a second one the remaining tokens; the phases of a step follow one another inside the
 *     kernel, separated by a bounded barrier over the grid (one block per SM).  If a wait at that barrier runs
 *     out, hipgpt_gpt_generate returns HIPGPT_ERR_CUDA and the handle stays usable.  Measured no faster than the
 *     graph on B200 (335 against 327 us per step of 8 tokens).
 */
#define HIPGPT_GPT_MODE_GRAPH 0
#define HIPGPT_GPT_MODE_PERSISTENT 1
HIPGPT_API int hipgpt_gpt_set_mode(hipgpt_gpt *g, int mode);

/*
 * Sharding of the (batch x head) space over the GPUs of one box (no counterpart in the reference, which runs on one
 * GPU).  Every (batch, head) pair is independent (src/hip_kernels.cpp:269-277), so the kernels exchange nothing: a rank
 * computes its own batches from its own memory, and the only collective is the all-gather of the outputs.
 *
 *   hipgpt_shard_range        contiguous split: rank r of `world` owns batches [*b_begin, *b_end) (sizes differ by <= 1).
 *   hipgpt_shard_chunk_range  the split the driver below uses, for B a multiple of world * chunks: chunk c covers
 *                             batches [c*world*k, (c+1)*world*k), k = B / (world*chunks), and rank r owns the r-th run
 *                             of k batches inside it.  In the output every chunk is then one contiguous block with the
 *                             ranks' parts in rank order, the in-place form of ncclAllGather.
 *   hipgpt_shard_unique_id    128 bytes made by rank 0 and handed to every rank (by the job's own means);
 *   hipgpt_shard_create       collective over the ranks, each with its own GPU current: an NCCL communicator (NCCL is
 *                             loaded at run time, libnccl.so.2), a communication stream of the highest priority, events;
 *   hipgpt_mha_forward_sharded  d_q, d_k, d_v hold THIS rank's batches, chunk after chunk; d_out is the whole
 *                             [B*S][E] output.  Per chunk the attention kernels run on `stream`, then that chunk is
 *                             all-gathered in place on the communication stream while the next chunk computes; `stream`
 *                             finally waits for the last gather.  gather = 0 leaves only this rank's batches valid.
 *                             elem_bytes 4 = fp32 planes, 2 = bf16 planes (head_dim 64).  Results are the bits of the
 *                             unsharded call.
 *                             gather = HIPGPT_GATHER_PEER_STORES (2): the same result without the collective's kernels:
 *                             d_out must lie in the buffer of hipgpt_shard_output_buffer, which every rank has mapped
 *                             from every other; after a chunk's kernels a small copy kernel of this library stores
 *                             the chunk into the peers' buffers over NVLink, beside the next chunk's arithmetic (its
 *                             blocks fit on SMs that attention blocks occupy; NCCL's do not).  A collective of four
 *                             bytes per rank before the first and after the last copy orders the ranks: none writes
 *                             into a peer that has not reached the call on its `stream`, and `stream` continues once
 *                             every rank's copies have landed.  World size at most 8.
 *                             gather = HIPGPT_GATHER_PEER_COPIES (3): the same with one cudaMemcpyAsync per peer and chunk,
 *                             each on a stream of its peer: copy engines move the data and no SM is taken from the
 *                             attention kernels (measured the best of the three beside them).
 *   hipgpt_shard_output_buffer  collective: allocates `bytes` of device memory on every rank (the same size on all),
 *                             exchanges inter-process memory handles and maps the peers' buffers; *d_out is this
 *                             rank's.  One per context; a second call, and hipgpt_shard_destroy, release the first
 *                             (collectively).
 */
#define HIPGPT_GATHER_NONE        0
#define HIPGPT_GATHER_NCCL        1
#define HIPGPT_GATHER_PEER_STORES 2
#define HIPGPT_GATHER_PEER_COPIES 3   /* as 2, but one cudaMemcpyAsync per peer and chunk on a stream per peer: copy engines, no SM */
#define HIPGPT_GATHER_PEER_BOTH   4   /* 3 for the first three sevenths of the peers, 2 for the others, side by side */
typedef struct hipgpt_shard_ctx hipgpt_shard_ctx;
HIPGPT_API int hipgpt_shard_range(int B, int world, int rank, int *b_begin, int *b_end);
HIPGPT_API int hipgpt_shard_chunk_range(int B, int world, int rank, int chunks, int chunk, int *b_begin, int *b_end);
HIPGPT_API int hipgpt_shard_unique_id(void *id128);
HIPGPT_API int hipgpt_shard_create(hipgpt_shard_ctx **out, const void *id128, int rank, int world);
HIPGPT_API void hipgpt_shard_destroy(hipgpt_shard_ctx *ctx);
HIPGPT_API int hipgpt_mha_forward_sharded(hipgpt_shard_ctx *ctx, const void *d_q, const void *d_k, const void *d_v, void *d_out,
                               int B, int S, int E, int H, int causal, int elem_bytes, int chunks, int gather, void *stream);
HIPGPT_API int hipgpt_shard_output_buffer(hipgpt_shard_ctx *ctx, size_t bytes, void **d_out);
HIPGPT_API int hipgpt_shard_nccl_version(void);

/*
 * Measurement helper (no counterpart in the reference): enqueues a register-resident fp32
 * FMA loop on `blocks` thread blocks of 256 threads and stores in *flops the floating-point
 * operations it performs.  Timed with CUDA events by the caller it gives the FMA-pipe ceiling
 * that the exact-fp32 kernels are measured against.  d_sink: one float of device memory.
 */
HIPGPT_API int hipgpt_probe_fma(float *d_sink, int blocks, int iters, double *flops, void *stream);

/*
 * Device-side status of the tensor-core kernels (no counterpart in the reference).  Their
 * waits on hardware barriers are bounded; a block whose wait runs out stores nothing and records
 * which wait it was: 1..8 for the split-TF32 kernel, 100 + site for the bf16 kernel, 300 + site
 * for the tiled fp32 kernel, 400 + site for the whole-head kernel, 900 + site for the test hook
 * hipgpt_debug_wait_expiry.  This call waits for the whole
 * device (cudaDeviceSynchronize), stores the status word in *status and clears it.  0 means every
 * launch since the last call completed normally.  Callers of the device-pointer entry points
 * that need to know must poll this; hipgpt_mha_forward_host does it itself and returns
 * HIPGPT_ERR_CUDA when the word is set.
 */
HIPGPT_API int hipgpt_kernel_status(int *status);

/*
 * Accuracy notice of the default fp32 tensor-core kernels (no counterpart in the reference: its kernels
 * are plain fp32).  Bit 0 of *notice is set when, since the last call, some launch met Q, K or V values
 * outside the range in which its fp16 correction terms are exact (beyond +-65504, or so small beside the
 * other operand that the flushed bits matter): that launch's result is TF32-grade (~3e-4 relative), not
 * 1e-5-grade.  Waits for the device, then reads and clears the flag.
 * hipgpt_set_full_range(1) (or the environment variable HIPGPT_FULL_RANGE=1, read at the first call)
 * makes every entry point, the reference-named launchers included, use the kernels whose accuracy does
 * not depend on magnitude (split-TF32; exact FFMA when the probabilities are stored).
 */
HIPGPT_API int hipgpt_accuracy_notice(int *notice);
HIPGPT_API int hipgpt_set_full_range(int on);

/*
 * Test hooks for the give-up paths (no counterpart in the reference).  Nothing here traps, faults or
 * spins without a limit.
 *   hipgpt_debug_wait_expiry  launches two small blocks that run the tensor-core kernels' wait protocol
 *       (bounded mbarrier wait, abort flag, status word, stores skipped) on a barrier at which nothing
 *       arrives, with a limit of `limit_cycles` SM cycles (at most 2^24, a few milliseconds).  Afterwards
 *       hipgpt_kernel_status() reports 907 and d_canary[0..n) is untouched.
 *   hipgpt_gpt_debug_stall_barrier  makes the NEXT persistent-mode hipgpt_gpt_generate call start with a
 *       grid-barrier counter that cannot complete and a wait limit of `limit_cycles`: every block gives up
 *       at its first barrier, the call returns HIPGPT_ERR_CUDA, and the handle stays usable.
 */
HIPGPT_API int hipgpt_debug_wait_expiry(float *d_canary, int n, long long limit_cycles, void *stream);
HIPGPT_API int hipgpt_gpt_debug_stall_barrier(hipgpt_gpt *g, long long limit_cycles);

/* Text of the calling thread's most recent failure ("" if none). */
HIPGPT_API const char *hipgpt_last_error(void);

/* 10000*major + 100*minor + patch of this library. */
HIPGPT_API int hipgpt_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HIPGPT_ATTN_H */
