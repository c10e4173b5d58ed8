// C ABI of the attention library: argument checks, dispatch, the host-buffer call and the
// per-thread error text.  Declarations and the reference interfaces they replace are in
// include/hipgpt_attn.h.
#include "attn_common.cuh"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <stdlib.h>

#include <atomic>
#include <mutex>

namespace hipgpt {

namespace {
thread_local char g_err[512] = "";
}

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char *what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return HIPGPT_OK;
}

namespace {

// 0: fp32-grade kernels with fp16 correction terms (exact for operands within fp16's range);
// 1: kernels whose accuracy holds over the whole fp32 range.  -1 until first read.
std::atomic<int> g_full_range{-1};

bool full_range()
{
    int v = g_full_range.load(std::memory_order_relaxed);
    if (v < 0) {
        const char *e = getenv("HIPGPT_FULL_RANGE");
        v = (e && e[0] && e[0] != '0') ? 1 : 0;
        g_full_range.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

int check_mha_args(const void *q, const void *k, const void *v, const void *out, int B, int S, int E, int H)
{
    if (H <= 0 || E <= 0 || (E % H) != 0) return fail(HIPGPT_ERR_BAD_ARG, "Bad MHA config: E=%d H=%d", E, H);
    if (B < 0 || S < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: B=%d S=%d", B, S);
    if (B == 0 || S == 0) return 1;   // nothing to do
    if (!q || !k || !v || !out) return fail(HIPGPT_ERR_NULL, "q, k, v and out must not be NULL");
    return HIPGPT_OK;
}

int mha_dispatch(const float *q, const float *k, const float *v, float *out, float *probs,
                 int B, int S, int E, int H, int causal, int algo, int warps, cudaStream_t st)
{
    const int rc = check_mha_args(q, k, v, out, B, S, E, H);
    if (rc != HIPGPT_OK) return rc > 0 ? HIPGPT_OK : rc;
    const int D = E / H;
    // The rows kernel moves 16 bytes at a time: every row start must be 16-byte aligned.
    const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                           reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                         (probs == nullptr || (reinterpret_cast<uintptr_t>(probs) & 15) == 0);
    const bool tensor_ok = aligned && (D == 32 || D == 64);
    switch (algo) {
    case HIPGPT_ALGO_AUTO:
        if (tensor_ok && full_range()) {
            // operands of any fp32 magnitude: split-TF32 products; with the probabilities the exact FFMA kernel
            if (!probs) return launch_mha_tc(q, k, v, out, B, S, E, H, causal, st);
            return launch_mha_rows(q, k, v, out, probs, B, S, E, H, causal, warps, st);
        }
        // tensor pipe when it applies (fp32-grade TF32 + FP16 products): the whole-head kernel for the default
        // model's shape, the tiled kernel otherwise (it also stores the probabilities, by a second sweep);
        // FFMA rows kernel for head_dim 128; generic kernel for everything else
        if (mha_head_supports(D, S, E, q, k, v, out)) return launch_mha_head(q, k, v, out, probs, B, S, E, H, causal, st);
        if (tensor_ok) return launch_mha_tc16(q, k, v, out, probs, B, S, E, H, causal, st);
        if (mha_rows_supports(D) && aligned) return launch_mha_rows(q, k, v, out, probs, B, S, E, H, causal, warps, st);
        return launch_mha_generic(q, k, v, out, probs, B, S, E, H, causal, st);
    case HIPGPT_ALGO_GENERIC:
        return launch_mha_generic(q, k, v, out, probs, B, S, E, H, causal, st);
    case HIPGPT_ALGO_ROWS:
        if (!aligned) return fail(HIPGPT_ERR_BAD_ARG, "rows kernel needs 16-byte aligned pointers");
        return launch_mha_rows(q, k, v, out, probs, B, S, E, H, causal, warps, st);
    case HIPGPT_ALGO_TENSOR:
        if (!aligned) return fail(HIPGPT_ERR_BAD_ARG, "tensor-core kernel needs 16-byte aligned pointers");
        if (!tensor_ok) return fail(HIPGPT_ERR_UNSUPPORTED, "tensor-core kernel: head_dim %d is not 32 or 64", D);
        switch (warps) {                             // `warps` selects the kernel here
        case HIPGPT_TENSOR_DEFAULT:
            if (mha_head_supports(D, S, E, q, k, v, out)) return launch_mha_head(q, k, v, out, probs, B, S, E, H, causal, st);
            return launch_mha_tc16(q, k, v, out, probs, B, S, E, H, causal, st);
        case HIPGPT_TENSOR_SPLIT_TF32:
            if (probs) return fail(HIPGPT_ERR_UNSUPPORTED, "split-TF32 kernel stores no probabilities");
            return launch_mha_tc(q, k, v, out, B, S, E, H, causal, st);
        case HIPGPT_TENSOR_TILED:
            return launch_mha_tc16(q, k, v, out, probs, B, S, E, H, causal, st);
        case HIPGPT_TENSOR_WHOLE_HEAD:
            if (!mha_head_supports(D, S, E, q, k, v, out))
                return fail(HIPGPT_ERR_UNSUPPORTED, "whole-head kernel: needs head_dim 32 and S <= 256 (head_dim %d, S %d)", D, S);
            return launch_mha_head(q, k, v, out, probs, B, S, E, H, causal, st);
        default:
            return fail(HIPGPT_ERR_BAD_ARG, "unknown tensor-core kernel %d", warps);
        }
    default:
        return fail(HIPGPT_ERR_BAD_ARG, "unknown algo %d", algo);
    }
}

// Device workspace of the host-buffer call: grows to the largest request, one per process.
struct Workspace {
    static constexpr int kStreams = 3;     // copies in, kernels, copies out
#ifndef HIPGPT_HOST_CHUNKS
#define HIPGPT_HOST_CHUNKS 8
#endif
#ifndef HIPGPT_HOST_CHUNK_BYTES
#define HIPGPT_HOST_CHUNK_BYTES (6u << 20)
#endif
    static constexpr int kChunks = HIPGPT_HOST_CHUNKS;   // most pieces a call is cut into
    // input bytes a piece should hold at least: every copy costs several microseconds on top of its
    // bytes, so a small call is cut into fewer pieces
    static constexpr size_t kChunkBytes = HIPGPT_HOST_CHUNK_BYTES;
    std::mutex mu;
    float *dev = nullptr;
    size_t bytes = 0;
    cudaStream_t streams[kStreams] = {nullptr, nullptr, nullptr};
    cudaEvent_t in_ready[kChunks] = {}, out_ready[kChunks] = {};
    int device = -1;
};
Workspace g_ws;

}  // namespace
}  // namespace hipgpt

using namespace hipgpt;

// First non-zero status word of the tensor-core kernels, as hipgpt_kernel_status reports it.
static int fetch_status_words(int *status)
{
    int a = 0, b = 0, d = 0, h = 0;
    int rc = tc_status_fetch(&a);
    if (rc == HIPGPT_OK) rc = bf16_status_fetch(&b);
    if (rc == HIPGPT_OK) rc = tc16_status_fetch(&d);
    if (rc == HIPGPT_OK) rc = head_status_fetch(&h);
    int pr = 0, gm = 0;
    if (rc == HIPGPT_OK) rc = probe_status_fetch(&pr);
    if (rc == HIPGPT_OK) rc = gemm_tc_status_fetch(&gm);
    if (rc != HIPGPT_OK) return rc;
    *status = a ? a : (b ? 100 + b : (d ? 300 + d : (h ? 400 + h : (gm ? 500 + gm : (pr ? 900 + pr : 0)))));
    return HIPGPT_OK;
}


extern "C" {

int hipgpt_mha_forward(const float *d_q, const float *d_k, const float *d_v, float *d_out, float *d_probs,
                       int B, int S, int E, int H, int causal, void *stream)
{
    return mha_dispatch(d_q, d_k, d_v, d_out, d_probs, B, S, E, H, causal, HIPGPT_ALGO_AUTO, 0,
                        static_cast<cudaStream_t>(stream));
}

int hipgpt_mha_forward_ex(const float *d_q, const float *d_k, const float *d_v, float *d_out, float *d_probs,
                          int B, int S, int E, int H, int causal, int algo, int warps, void *stream)
{
    return mha_dispatch(d_q, d_k, d_v, d_out, d_probs, B, S, E, H, causal, algo, warps,
                        static_cast<cudaStream_t>(stream));
}

int hipgpt_mha_forward_planes(const float *d_qkv, float *d_out, float *d_probs,
                              int B, int S, int E, int H, int causal, void *stream)
{
    if (B < 0 || S < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: B=%d S=%d E=%d", B, S, E);
    const size_t plane = (size_t)B * S * E;
    const float *k = d_qkv ? d_qkv + plane : nullptr;
    const float *v = d_qkv ? d_qkv + 2 * plane : nullptr;
    return mha_dispatch(d_qkv, k, v, d_out, d_probs, B, S, E, H, causal, HIPGPT_ALGO_AUTO, 0,
                        static_cast<cudaStream_t>(stream));
}

int hipgpt_mha_forward_bf16(const void *d_q, const void *d_k, const void *d_v, void *d_out,
                            int B, int S, int E, int H, int causal, void *stream)
{
    return hipgpt_mha_forward_bf16_ex(d_q, d_k, d_v, d_out, B, S, E, H, causal, 0, stream);
}

int hipgpt_mha_forward_bf16_ex(const void *d_q, const void *d_k, const void *d_v, void *d_out,
                               int B, int S, int E, int H, int causal, int variant, void *stream)
{
    if (B < 0 || S < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: B=%d S=%d E=%d", B, S, E);
    if (H <= 0 || E % H != 0) return fail(HIPGPT_ERR_BAD_ARG, "Bad MHA config: E=%d H=%d", E, H);
    if (B == 0 || S == 0 || E == 0) return HIPGPT_OK;
    if (!d_q || !d_k || !d_v || !d_out) return fail(HIPGPT_ERR_NULL, "q, k, v and out must not be NULL");
    if ((reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v) |
         reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(HIPGPT_ERR_BAD_ARG, "bf16 planes must be 16-byte aligned");
    return launch_mha_bf16(d_q, d_k, d_v, d_out, B, S, E, H, causal, static_cast<cudaStream_t>(stream), variant);
}

// Host buffers in, host buffers out, for planes of `esz`-byte elements (4: fp32, 2: bf16; the
// probabilities exist in the fp32 form only).
static int mha_forward_host_impl(const void *h_qkv_v, void *h_out_v, float *h_probs,
                                 int B, int S, int E, int H, int causal, size_t esz)
{
    const uint8_t *h_qkv = static_cast<const uint8_t *>(h_qkv_v);
    uint8_t *h_out = static_cast<uint8_t *>(h_out_v);
    const int rc = check_mha_args(h_qkv, h_qkv, h_qkv, h_out, B, S, E, H);
    if (rc != HIPGPT_OK) return rc > 0 ? HIPGPT_OK : rc;
    if (esz == 2 && E / H != 64) return fail(HIPGPT_ERR_UNSUPPORTED, "bf16 tensor-core kernel: head_dim %d is not 64", E / H);
    const size_t plane = (size_t)B * S * E * esz;    // bytes of one plane
    const size_t nprobs = h_probs ? (size_t)B * H * S * S : 0;
    const size_t need = 4 * plane + nprobs * sizeof(float);
    std::lock_guard<std::mutex> lock(g_ws.mu);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (g_ws.device != dev || g_ws.bytes < need) {
        if (g_ws.dev) cudaFree(g_ws.dev);
        g_ws.dev = nullptr;
        g_ws.bytes = 0;
        if (g_ws.device != dev) {
            for (int i = 0; i < Workspace::kStreams; ++i) if (g_ws.streams[i]) { cudaStreamDestroy(g_ws.streams[i]); g_ws.streams[i] = nullptr; }
            for (int i = 0; i < Workspace::kChunks; ++i) {
                if (g_ws.in_ready[i]) { cudaEventDestroy(g_ws.in_ready[i]); g_ws.in_ready[i] = nullptr; }
                if (g_ws.out_ready[i]) { cudaEventDestroy(g_ws.out_ready[i]); g_ws.out_ready[i] = nullptr; }
            }
        }
        e = cudaMalloc(&g_ws.dev, need);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMalloc(%zu): %s", need, cudaGetErrorString(e));
        g_ws.bytes = need;
        g_ws.device = dev;
    }
    for (int i = 0; i < Workspace::kStreams; ++i)
        if (!g_ws.streams[i]) {
            e = cudaStreamCreateWithFlags(&g_ws.streams[i], cudaStreamNonBlocking);
            if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
        }
    for (int i = 0; i < Workspace::kChunks; ++i) {
        if (!g_ws.in_ready[i]) e = cudaEventCreateWithFlags(&g_ws.in_ready[i], cudaEventDisableTiming);
        if (e == cudaSuccess && !g_ws.out_ready[i]) e = cudaEventCreateWithFlags(&g_ws.out_ready[i], cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
    }
    // Batches are independent, so the call is cut into chunks of batches that flow through three
    // streams: host-to-device copies, kernels, device-to-host copies.  PCIe moves both directions
    // at once, so the call takes about as long as its larger direction alone.
    cudaStream_t s_in = g_ws.streams[0], s_k = g_ws.streams[1], s_out = g_ws.streams[2];
    uint8_t *d_qkv = reinterpret_cast<uint8_t *>(g_ws.dev), *d_out = d_qkv + 3 * plane;
    float *d_probs = h_probs ? reinterpret_cast<float *>(d_qkv + 4 * plane) : nullptr;
    int nchunks = (int)((3 * plane) / Workspace::kChunkBytes);
    nchunks = nchunks < 1 ? 1 : nchunks > Workspace::kChunks ? Workspace::kChunks : nchunks;
    if (nchunks > B) nchunks = B;
    // the three planes' slabs of a chunk go up as one strided copy (three rows one plane apart) where the
    // pitch limit of such copies allows it
    const bool strided = plane <= (size_t)0x7fffffff;
    for (int c = 0; c < nchunks; ++c) {
        int b0, b1;
        hipgpt_shard_range(B, nchunks, c, &b0, &b1);
        const size_t off = (size_t)b0 * S * E * esz, cnt = (size_t)(b1 - b0) * S * E * esz;   // bytes
        if (strided)
            e = cudaMemcpy2DAsync(d_qkv + off, plane, h_qkv + off, plane, cnt, 3, cudaMemcpyHostToDevice, s_in);
        else
            for (int pl = 0; pl < 3 && e == cudaSuccess; ++pl)
                e = cudaMemcpyAsync(d_qkv + pl * plane + off, h_qkv + pl * plane + off, cnt, cudaMemcpyHostToDevice, s_in);
        if (e == cudaSuccess) e = cudaEventRecord(g_ws.in_ready[c], s_in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s_k, g_ws.in_ready[c], 0);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "copy to device: %s", cudaGetErrorString(e));
        float *pr = d_probs ? d_probs + (size_t)b0 * H * S * S : nullptr;
        const int krc = esz == 2
            ? launch_mha_bf16(d_qkv + off, d_qkv + plane + off, d_qkv + 2 * plane + off, d_out + off, b1 - b0, S, E, H, causal, s_k)
            : mha_dispatch(reinterpret_cast<const float *>(d_qkv + off), reinterpret_cast<const float *>(d_qkv + plane + off),
                           reinterpret_cast<const float *>(d_qkv + 2 * plane + off), reinterpret_cast<float *>(d_out + off), pr,
                           b1 - b0, S, E, H, causal, HIPGPT_ALGO_AUTO, 0, s_k);
        if (krc != HIPGPT_OK) { cudaDeviceSynchronize(); return krc; }
        e = cudaEventRecord(g_ws.out_ready[c], s_k);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s_out, g_ws.out_ready[c], 0);
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_out + off, d_out + off, cnt, cudaMemcpyDeviceToHost, s_out);
        if (e == cudaSuccess && h_probs)
            e = cudaMemcpyAsync(h_probs + (size_t)b0 * H * S * S, pr, (size_t)(b1 - b0) * H * S * S * sizeof(float), cudaMemcpyDeviceToHost, s_out);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "copy to host: %s", cudaGetErrorString(e));
    }
    e = cudaStreamSynchronize(s_out);                // its last copy waits for the last kernel, which waits for the last copy in
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "host-buffer call: %s", cudaGetErrorString(e));
    // a block whose bounded wait ran out stored nothing: the output would be stale.  Only the status word of the
    // kernel this call ran is read (one small copy; the words of the other kernels stay for hipgpt_kernel_status).
    int status = 0, src = HIPGPT_OK;
    const int D = E / H;
    if (esz == 2) src = bf16_status_fetch(&status);
    else if ((D == 32 || D == 64) && full_range()) src = h_probs ? HIPGPT_OK : tc_status_fetch(&status);
    else if (D == 32 && S <= 256) src = head_status_fetch(&status), status = status ? 400 + status : 0;
    else if (D == 32 || D == 64) src = tc16_status_fetch(&status), status = status ? 300 + status : 0;
    if (src != HIPGPT_OK) return src;
    if (status != 0) return fail(HIPGPT_ERR_CUDA, "a bounded wait inside a kernel ran out (status %d); the output is incomplete", status);
    return HIPGPT_OK;
}

int hipgpt_mha_forward_host(const float *h_qkv, float *h_out, float *h_probs,
                            int B, int S, int E, int H, int causal)
{
    return mha_forward_host_impl(h_qkv, h_out, h_probs, B, S, E, H, causal, sizeof(float));
}

int hipgpt_mha_forward_bf16_host(const void *h_qkv, void *h_out, int B, int S, int E, int H, int causal)
{
    return mha_forward_host_impl(h_qkv, h_out, nullptr, B, S, E, H, causal, 2);
}

void hipgpt_release_workspace(void)
{
    tc16_release_scratch();
    gemm_tc_release_scratch();
    std::lock_guard<std::mutex> lock(g_ws.mu);
    if (g_ws.dev) cudaFree(g_ws.dev);
    for (int i = 0; i < Workspace::kStreams; ++i) if (g_ws.streams[i]) { cudaStreamDestroy(g_ws.streams[i]); g_ws.streams[i] = nullptr; }
    for (int i = 0; i < Workspace::kChunks; ++i) {
        if (g_ws.in_ready[i]) { cudaEventDestroy(g_ws.in_ready[i]); g_ws.in_ready[i] = nullptr; }
        if (g_ws.out_ready[i]) { cudaEventDestroy(g_ws.out_ready[i]); g_ws.out_ready[i] = nullptr; }
    }
    g_ws.dev = nullptr;
    g_ws.bytes = 0;
    g_ws.device = -1;
}

int hipgpt_scaled_dot_product(const float *d_Q, const float *d_K, float *d_scores, int B, int S, int D, void *stream)
{
    if (B < 0 || S < 0 || D <= 0) return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d S=%d D=%d", B, S, D);
    if (B == 0 || S == 0) return HIPGPT_OK;
    if (!d_Q || !d_K || !d_scores) return fail(HIPGPT_ERR_NULL, "Q, K and scores must not be NULL");
    return launch_sdp(d_Q, d_K, d_scores, B, S, D, static_cast<cudaStream_t>(stream));
}

int hipgpt_softmax(const float *d_scores, float *d_softmax_out, int B, int S, void *stream)
{
    if (B < 0 || S < 0) return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d S=%d", B, S);
    if (B == 0 || S == 0) return HIPGPT_OK;
    if (!d_scores || !d_softmax_out) return fail(HIPGPT_ERR_NULL, "scores and softmax_out must not be NULL");
    return launch_softmax_rows(d_scores, d_softmax_out, B, S, static_cast<cudaStream_t>(stream));
}

int hipgpt_attention_weighted_sum(const float *d_softmax, const float *d_V, float *d_output,
                                  int B, int S, int D, void *stream)
{
    if (B < 0 || S < 0 || D <= 0) return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d S=%d D=%d", B, S, D);
    if (B == 0 || S == 0) return HIPGPT_OK;
    if (!d_softmax || !d_V || !d_output) return fail(HIPGPT_ERR_NULL, "softmax, V and output must not be NULL");
    return launch_weighted_sum(d_softmax, d_V, d_output, B, S, D, static_cast<cudaStream_t>(stream));
}

size_t hipgpt_mha_decode_scratch_bytes(int B, int H, int D, int ctx)
{
    if (B <= 0 || H <= 0 || D <= 0 || ctx <= 0) return 0;
    const int ns = decode_splits(B, H, D, ctx);
    if (ns <= 1) return 0;
    const size_t stride = (size_t)((D + 3) / 4) * 4 + 4;
    return (size_t)B * H * ns * stride * sizeof(float);
}

int hipgpt_mha_decode(const float *d_q, const float *d_kcache, const float *d_vcache, float *d_out,
                      float *d_scratch, size_t scratch_bytes,
                      int B, int H, int D, int ctx, int cap, void *stream)
{
    if (B < 0 || H <= 0 || D <= 0 || ctx < 0 || cap < ctx)
        return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d H=%d D=%d ctx=%d cap=%d", B, H, D, ctx, cap);
    if (B == 0) return HIPGPT_OK;
    if (!d_q || !d_out || (ctx > 0 && (!d_kcache || !d_vcache)))
        return fail(HIPGPT_ERR_NULL, "q, out and the caches must not be NULL");
    const size_t need = hipgpt_mha_decode_scratch_bytes(B, H, D, ctx);
    if (need > 0 && (!d_scratch || scratch_bytes < need))
        return fail(HIPGPT_ERR_SCRATCH, "scratch of %zu bytes needed, %zu given", need, d_scratch ? scratch_bytes : (size_t)0);
    // only the vector kernels (head_dim % 4 == 0, up to 128) move 16 bytes at a time
    if (D % 4 == 0 && D <= 128 && ((reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_kcache) |
                                    reinterpret_cast<uintptr_t>(d_vcache) | reinterpret_cast<uintptr_t>(d_out) |
                                    reinterpret_cast<uintptr_t>(d_scratch)) & 15) != 0)
        return fail(HIPGPT_ERR_BAD_ARG, "decode needs 16-byte aligned pointers");
    const int ns = need > 0 ? decode_splits(B, H, D, ctx) : 1;
    return launch_decode(d_q, d_kcache, d_vcache, d_out, d_scratch, B, H, D, ctx, cap, ns, static_cast<cudaStream_t>(stream));
}

size_t hipgpt_mha_backward_scratch_bytes(int B, int H, int S)
{
    if (B <= 0 || H <= 0 || S <= 0) return 0;
    return mha_backward_scratch_bytes(B, H, S);
}

int hipgpt_mha_backward(const float *d_grad_out, const float *d_q, const float *d_k, const float *d_v, const float *d_probs,
                        float *d_grad_q, float *d_grad_k, float *d_grad_v, float *d_scratch, size_t scratch_bytes,
                        int B, int S, int E, int H, int causal, void *stream)
{
    const int rc = check_mha_args(d_q, d_k, d_v, d_grad_out, B, S, E, H);
    if (rc != HIPGPT_OK) return rc > 0 ? HIPGPT_OK : rc;
    if (!d_grad_q || !d_grad_k || !d_grad_v) return fail(HIPGPT_ERR_NULL, "the three gradient outputs must not be NULL");
    const size_t need = mha_backward_scratch_bytes(B, H, S);
    if (!d_scratch || scratch_bytes < need)
        return fail(HIPGPT_ERR_SCRATCH, "scratch of %zu bytes needed, %zu given", need, d_scratch ? scratch_bytes : (size_t)0);
    return launch_mha_backward(d_grad_out, d_q, d_k, d_v, d_probs, d_grad_q, d_grad_k, d_grad_v, d_scratch, B, S, E, H, causal,
                               static_cast<cudaStream_t>(stream));
}

// The reference's launcher has no scratch argument (include/hip_kernels.h:59-62): its drop-in form keeps the row
// sums in a buffer of the library that grows to the largest call on the current device.
int hipgpt_mha_backward_planes(const float *d_grad_out, const float *d_qkv, const float *d_probs, float *d_grad_qkv,
                               int B, int S, int E, int H, int causal, void *stream)
{
    if (B < 0 || S < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: B=%d S=%d E=%d", B, S, E);
    if (H <= 0 || E % H != 0) return fail(HIPGPT_ERR_BAD_ARG, "Bad MHA config: E=%d H=%d", E, H);
    if (B == 0 || S == 0 || E == 0) return HIPGPT_OK;
    if (!d_grad_out || !d_qkv || !d_grad_qkv) return fail(HIPGPT_ERR_NULL, "grad_out, qkv and grad_qkv must not be NULL");
    static std::mutex mu;
    static float *buf[64] = {};
    static size_t cap[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(HIPGPT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    const size_t need = mha_backward_scratch_bytes(B, H, S);
    float *scratch;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (cap[dev] < need) {
            if (buf[dev]) cudaFree(buf[dev]);
            buf[dev] = nullptr;
            cap[dev] = 0;
            e = cudaMalloc(&buf[dev], need);
            if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMalloc(%zu): %s", need, cudaGetErrorString(e));
            cap[dev] = need;
        }
        scratch = buf[dev];
    }
    const size_t plane = (size_t)B * S * E;
    return launch_mha_backward(d_grad_out, d_qkv, d_qkv + plane, d_qkv + 2 * plane, d_probs, d_grad_qkv, d_grad_qkv + plane,
                               d_grad_qkv + 2 * plane, scratch, B, S, E, H, causal, static_cast<cudaStream_t>(stream));
}

int hipgpt_shard_range(int B, int world, int rank, int *b_begin, int *b_end)
{
    if (B < 0 || world <= 0 || rank < 0 || rank >= world)
        return fail(HIPGPT_ERR_BAD_ARG, "bad shard request: B=%d world=%d rank=%d", B, world, rank);
    if (!b_begin || !b_end) return fail(HIPGPT_ERR_NULL, "b_begin and b_end must not be NULL");
    // the first B % world ranks take one batch more
    const int base = B / world, extra = B % world;
    *b_begin = rank * base + (rank < extra ? rank : extra);
    *b_end = *b_begin + base + (rank < extra ? 1 : 0);
    return HIPGPT_OK;
}

int hipgpt_kernel_status(int *status)
{
    if (!status) return fail(HIPGPT_ERR_NULL, "status must not be NULL");
    const cudaError_t e = cudaDeviceSynchronize();   // the kernels may run on non-blocking streams
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    return fetch_status_words(status);
}

int hipgpt_accuracy_notice(int *notice)
{
    if (!notice) return fail(HIPGPT_ERR_NULL, "notice must not be NULL");
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int n16 = 0, nh = 0;
    int rc = tc16_notice_fetch(&n16);
    if (rc == HIPGPT_OK) rc = head_notice_fetch(&nh);
    if (rc != HIPGPT_OK) return rc;
    *notice = n16 | nh;
    return HIPGPT_OK;
}

int hipgpt_set_full_range(int on)
{
    g_full_range.store(on ? 1 : 0, std::memory_order_relaxed);
    return HIPGPT_OK;
}

const char *hipgpt_last_error(void) { return g_err; }

int hipgpt_version(void) { return 100; }

}  // extern "C"
