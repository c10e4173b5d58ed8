// Copies a block of this GPU's memory to the same place in up to seven peers' buffers with plain stores over
// NVLink: the transport of the sharded driver's all-gather (sharded.cpp).  No counterpart in the reference.
//
// The kernel is small on purpose: 128 threads, no shared memory, at most 32 registers, so that its blocks fit on
// SMs that already hold two blocks of an attention kernel and the transfer of one chunk runs beside the arithmetic
// of the next.  A warp moves 512 contiguous bytes per instruction (16 per lane); four loads are in flight per
// thread.  Nothing here waits for another GPU: ordering between the ranks is the driver's (stream order and a
// collective of the communication library before and after the copies).
#include "attn_common.cuh"

namespace hipgpt {
namespace {

constexpr int kPushThreads = 128;
constexpr int kPushUnroll = 4;

struct PushTargets {
    uint4 *dst[7];
    int n;
};

__global__ void __launch_bounds__(kPushThreads, 16)
shard_push_kernel(const uint4 *__restrict__ src, PushTargets t, size_t n16)
{
    const size_t stride = (size_t)gridDim.x * kPushThreads;
    size_t i = (size_t)blockIdx.x * kPushThreads + threadIdx.x;
    for (; i + (kPushUnroll - 1) * stride < n16; i += kPushUnroll * stride) {
        uint4 v[kPushUnroll];
#pragma unroll
        for (int u = 0; u < kPushUnroll; ++u) v[u] = src[i + u * stride];
        for (int p = 0; p < t.n; ++p) {
#pragma unroll
            for (int u = 0; u < kPushUnroll; ++u) t.dst[p][i + u * stride] = v[u];
        }
    }
    for (; i < n16; i += stride) {
        const uint4 v = src[i];
        for (int p = 0; p < t.n; ++p) t.dst[p][i] = v;
    }
}

}  // namespace

// src and every dst[p] 16-byte aligned, bytes a multiple of 16, 1 <= ndst <= 7.
int launch_shard_push(const void *src, void *const *dst, int ndst, size_t bytes, cudaStream_t st)
{
    if (ndst < 1 || ndst > 7) return fail(HIPGPT_ERR_BAD_ARG, "%d peers: the copy kernel takes 1 to 7", ndst);
    if ((bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return fail(HIPGPT_ERR_BAD_ARG, "the block to copy must be 16-byte aligned and sized");
    PushTargets t = {};
    t.n = ndst;
    for (int p = 0; p < ndst; ++p) {
        if (reinterpret_cast<uintptr_t>(dst[p]) & 15) return fail(HIPGPT_ERR_BAD_ARG, "peer %d: address not 16-byte aligned", p);
        t.dst[p] = static_cast<uint4 *>(dst[p]);
    }
    if (bytes == 0) return HIPGPT_OK;
    const size_t n16 = bytes / 16;
    size_t blocks = (n16 + (size_t)kPushThreads * kPushUnroll - 1) / ((size_t)kPushThreads * kPushUnroll);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    size_t per_sm = 4;
    if (const char *env = getenv("HIPGPT_PUSH_BLOCKS_PER_SM")) { const long v = atol(env); if (v > 0 && v <= 16) per_sm = (size_t)v; }
    if (blocks > (size_t)sms * per_sm) blocks = (size_t)sms * per_sm;
    shard_push_kernel<<<(unsigned)blocks, kPushThreads, 0, st>>>(static_cast<const uint4 *>(src), t, n16);
    return check_launch("shard_push_kernel");
}

}  // namespace hipgpt
