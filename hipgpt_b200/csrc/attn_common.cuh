// Shared device helpers and the error channel of the attention library (sm_100a).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#include "hipgpt_attn.h"

namespace hipgpt {

// Records the calling thread's failure text and returns `code` (host side, capi.cu).
int fail(int code, const char *fmt, ...);
// Checks the launch that was just enqueued; HIPGPT_OK or HIPGPT_ERR_CUDA.
int check_launch(const char *what);

// Launch with programmatic stream serialization: the kernel's blocks may become resident, and run their prologue
// (barriers, TMEM, roles), while the last blocks of the kernel before it on the stream are still running, once those
// have let their dependents go.  Such a kernel must execute dependency_wait() before its first access to global
// memory; the wait returns when the kernel before it has completed and its writes are visible.
// HIPGPT_NO_OVERLAPPED_LAUNCH=1 launches the plain way.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    static const bool plain = [] { const char *e = getenv("HIPGPT_NO_OVERLAPPED_LAUNCH"); return e && *e && *e != '0'; }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = plain ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
// The kernel before this one on the stream has completed and its writes are visible (returns at once for a plain launch).
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The kernel after this one on the stream may start its blocks as soon as every block of this grid has said so or exited.
__device__ __forceinline__ void dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 16-byte asynchronous global -> shared copy; `valid == false` writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, bool valid)
{
    const unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// Kernel launch wrappers (one per .cu file), all returning an HIPGPT_* status.
int launch_mha_rows(const float *q, const float *k, const float *v, float *out, float *probs,
                    int B, int S, int E, int H, int causal, int warps, cudaStream_t st);
bool mha_rows_supports(int D);
int launch_mha_tc(const float *q, const float *k, const float *v, float *out,
                  int B, int S, int E, int H, int causal, cudaStream_t st);
bool mha_tc_supports(int D);
int tc_status_fetch(int *status);
int launch_mha_tc16(const float *q, const float *k, const float *v, float *out, float *probs,
                    int B, int S, int E, int H, int causal, cudaStream_t st);
bool mha_tc16_supports(int head_dim);
int tc16_status_fetch(int *status);
void tc16_release_scratch();
// Copies `bytes` from src to each of up to seven peer addresses with plain stores (shard_push.cu).
int launch_shard_push(const void *src, void *const *dst, int ndst, size_t bytes, cudaStream_t st);
int tc16_notice_fetch(int *notice);
// whole-head kernel (head_dim 32, S <= 256): TMA loads, 128-key products, all score tiles of a head in TMEM
int launch_mha_head(const float *q, const float *k, const float *v, float *out, float *probs, int B, int S, int E, int H, int causal, cudaStream_t st);
bool mha_head_supports(int head_dim, int S, int E, const void *q, const void *k, const void *v, const void *out);
int head_status_fetch(int *status);
int head_notice_fetch(int *notice);
int probe_status_fetch(int *status);
int launch_mha_bf16(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, int causal, cudaStream_t st,
                    int variant = 0);
bool mha_bf16_supports(int D);
int bf16_status_fetch(int *status);
// attention backward (attn_bwd.cu): scratch = 2 B H S floats (row sums w_i, then log-sum-exp of the rows)
size_t mha_backward_scratch_bytes(int B, int H, int S);
int launch_mha_backward(const float *g, const float *q, const float *k, const float *v, const float *probs,
                        float *dq, float *dk, float *dv, float *scratch, int B, int S, int E, int H, int causal, cudaStream_t st);
// the launchers either side of attention (layer_ops.cu)
int launch_matmul_exact(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, cudaStream_t st);
// The same product on the tensor pipe with fp32-grade (not bit-identical) results (gemm_tc.cu); its status word and scratch.
int launch_matmul_tc(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, cudaStream_t st, const float *ln_g = nullptr, const float *ln_b = nullptr);
struct PackedB;                                  // a right-hand side packed once for many products
int matmul_tc_prepare(const float *B, int N, int K, PackedB **out, cudaStream_t st);
int launch_matmul_tc_prepared(const float *A, const PackedB *b, const float *bias, float *C, int M, cudaStream_t st, const float *ln_g = nullptr, const float *ln_b = nullptr);
void matmul_tc_release(PackedB *p);
int gemm_tc_status_fetch(int *status);
void gemm_tc_release_scratch();
int launch_mha_generic(const float *q, const float *k, const float *v, float *out, float *probs,
                       int B, int S, int E, int H, int causal, cudaStream_t st);
int launch_sdp(const float *Q, const float *K, float *scores, int B, int S, int D, cudaStream_t st);
int launch_softmax_rows(const float *scores, float *out, int B, int S, cudaStream_t st);
int launch_weighted_sum(const float *P, const float *V, float *out, int B, int S, int D, cudaStream_t st);
// pos_ptr (optional): device int holding ctx - 1; when given it overrides ctx inside the kernels,
// so that one captured launch serves every step of a generation loop.
int launch_decode(const float *q, const float *kc, const float *vc, float *out, float *scratch,
                  int B, int H, int D, int ctx, int cap, int nsplit, cudaStream_t st, const int *pos_ptr = nullptr);
int decode_splits(int B, int H, int D, int ctx);

}  // namespace hipgpt
