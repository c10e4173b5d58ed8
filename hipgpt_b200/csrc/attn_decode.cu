// Single-query-row attention over a key/value cache, split over the context (sm_100a).
//
// Extension with no kernel of its own in the reference: HipGPT's generation loop
// (src/gpt_model.cpp:261-280) re-runs the whole window through launch_multihead_attention for
// every new token.  With a cache, one token needs one query row per (batch, head) against
// ctx cached keys: B*H rows are far too few to fill 148 SMs, so the context is cut into
// `nsplit` ranges, each thread block reduces one range to a partial (max, sum, weighted V)
// and a second small kernel merges the partials.  Cache rows are read once, with 128-bit
// loads when head_dim allows; the work is bound by those reads and by launch latency.
//
// Scratch layout: [B*H][nsplit][stride] floats, stride = roundup4(D) + 4:
//   [0, D) un-normalised weighted V, [roundup4(D)] running max (log2 domain), [+1] sum.
#include "attn_common.cuh"

#include <math.h>


namespace hipgpt {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxD = 512;

__host__ __device__ inline int rec_stride(int D) { return ((D + 3) / 4) * 4 + 4; }

struct Partial4 {
    float m, l;
    float4 o;
};

__device__ __forceinline__ void merge(Partial4 &a, float m2, float l2, const float4 &o2)
{
    const float mn = fmaxf(a.m, m2);
    const float a1 = ex2_approx(a.m - mn), a2 = ex2_approx(m2 - mn);
    a.l = a.l * a1 + l2 * a2;
    a.o.x = a.o.x * a1 + o2.x * a2;
    a.o.y = a.o.y * a1 + o2.y * a2;
    a.o.z = a.o.z * a1 + o2.z * a2;
    a.o.w = a.o.w * a1 + o2.w * a2;
    a.m = mn;
}

// head_dim % 4 == 0 and head_dim <= 4*LPK: LPK lanes share one key, one float4 each.
template <int LPK>
__global__ void __launch_bounds__(kThreads)
decode_split_vec_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                        float *__restrict__ out, float *__restrict__ scratch,
                        int H, int D, int ctx, int cap, int nsplit, float qscale, const int *__restrict__ pos_ptr)
{
    dependency_wait();                             // overlapped launch: nothing is read before the kernel before this one has completed
    dependents_may_start();
    if (pos_ptr) ctx = *pos_ptr + 1;               // context length kept on the device (replayed CUDA graphs)
    constexpr int KPW = 32 / LPK;                  // keys per warp and step
    __shared__ float sm[kWarps][LPK][6];
    const int bh = blockIdx.y, split = blockIdx.x;
    const int b = bh / H, h = bh % H;
    const int E = H * D;
    const int per = (ctx + nsplit - 1) / nsplit;
    const int k0 = split * per, k1 = min(ctx, k0 + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lik = lane % LPK, kg = lane / LPK;
    const bool act = lik * 4 < D;
    const size_t col = (size_t)h * D + lik * 4;

    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (act) {
        q4 = __ldg(reinterpret_cast<const float4 *>(q + (size_t)b * E + col));
        q4.x *= qscale; q4.y *= qscale; q4.z *= qscale; q4.w *= qscale;
    }
    Partial4 acc{-1e30f, 0.0f, make_float4(0.f, 0.f, 0.f, 0.f)};
    const int steps = (max(k1 - k0, 0) + kWarps * KPW - 1) / (kWarps * KPW);
    for (int it = 0; it < steps; ++it) {
        const int j = k0 + (it * kWarps + warp) * KPW + kg;
        const bool valid = j < k1;
        float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
        if (valid && act) {
            const size_t off = ((size_t)b * cap + j) * (size_t)E + col;
            k4 = __ldg(reinterpret_cast<const float4 *>(kc + off));
            v4 = __ldg(reinterpret_cast<const float4 *>(vc + off));
        }
        float s = q4.x * k4.x;
        s = fmaf(q4.y, k4.y, s);
        s = fmaf(q4.z, k4.z, s);
        s = fmaf(q4.w, k4.w, s);
#pragma unroll
        for (int off = 1; off < LPK; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (!valid) s = -INFINITY;
        const float mn = fmaxf(acc.m, s);
        const float alpha = ex2_approx(acc.m - mn), p = ex2_approx(s - mn);
        acc.l = fmaf(acc.l, alpha, p);
        acc.o.x = fmaf(p, v4.x, acc.o.x * alpha);
        acc.o.y = fmaf(p, v4.y, acc.o.y * alpha);
        acc.o.z = fmaf(p, v4.z, acc.o.z * alpha);
        acc.o.w = fmaf(p, v4.w, acc.o.w * alpha);
        acc.m = mn;
    }
    // key groups of one warp
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, acc.m, off);
        const float l2 = __shfl_xor_sync(0xffffffffu, acc.l, off);
        float4 o2;
        o2.x = __shfl_xor_sync(0xffffffffu, acc.o.x, off);
        o2.y = __shfl_xor_sync(0xffffffffu, acc.o.y, off);
        o2.z = __shfl_xor_sync(0xffffffffu, acc.o.z, off);
        o2.w = __shfl_xor_sync(0xffffffffu, acc.o.w, off);
        merge(acc, m2, l2, o2);
    }
    if (kg == 0) {
        float *r = sm[warp][lik];
        r[0] = acc.m; r[1] = acc.l; r[2] = acc.o.x; r[3] = acc.o.y; r[4] = acc.o.z; r[5] = acc.o.w;
    }
    __syncthreads();
    if (warp == 0 && lane < LPK) {
        Partial4 t{sm[0][lane][0], sm[0][lane][1], make_float4(sm[0][lane][2], sm[0][lane][3], sm[0][lane][4], sm[0][lane][5])};
#pragma unroll
        for (int w = 1; w < kWarps; ++w)
            merge(t, sm[w][lane][0], sm[w][lane][1], make_float4(sm[w][lane][2], sm[w][lane][3], sm[w][lane][4], sm[w][lane][5]));
        if (lane * 4 < D) {
            if (nsplit == 1) {
                const float inv = 1.0f / fmaxf(t.l, 1e-20f);
                *reinterpret_cast<float4 *>(out + (size_t)b * E + (size_t)h * D + lane * 4) =
                    make_float4(t.o.x * inv, t.o.y * inv, t.o.z * inv, t.o.w * inv);
            } else {
                float *rec = scratch + ((size_t)bh * nsplit + split) * rec_stride(D);
                *reinterpret_cast<float4 *>(rec + lane * 4) = t.o;
                if (lane == 0) { rec[rec_stride(D) - 4] = t.m; rec[rec_stride(D) - 3] = t.l; }
            }
        }
    }
}

// any head_dim <= 512: one warp per key, lane d handles elements d, d+32, ...
__global__ void __launch_bounds__(kThreads)
decode_split_scalar_kernel(const float *__restrict__ q, const float *__restrict__ kc, const float *__restrict__ vc,
                           float *__restrict__ out, float *__restrict__ scratch,
                           int H, int D, int ctx, int cap, int nsplit, float qscale, const int *__restrict__ pos_ptr)
{
    dependency_wait();
    dependents_may_start();
    if (pos_ptr) ctx = *pos_ptr + 1;
    constexpr int EPL = kMaxD / 32;
    __shared__ float sm_o[kWarps][kMaxD];
    __shared__ float sm_ml[kWarps][2];
    const int bh = blockIdx.y, split = blockIdx.x;
    const int b = bh / H, h = bh % H;
    const int E = H * D;
    const int per = (ctx + nsplit - 1) / nsplit;
    const int k0 = split * per, k1 = min(ctx, k0 + per);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t col = (size_t)h * D;
    float qv[EPL], o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? __ldg(q + (size_t)b * E + col + d) * qscale : 0.0f;
        o[i] = 0.0f;
    }
    float m = -1e30f, l = 0.0f;
    for (int j = k0 + warp; j < k1; j += kWarps) {
        const size_t off = ((size_t)b * cap + j) * (size_t)E + col;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int d = lane + 32 * i;
            if (d < D) s = fmaf(qv[i], __ldg(kc + off + d), s);
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) s += __shfl_xor_sync(0xffffffffu, s, sh);
        const float mn = fmaxf(m, s);
        const float alpha = ex2_approx(m - mn), p = ex2_approx(s - mn);
        l = fmaf(l, alpha, p);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int d = lane + 32 * i;
            if (d < D) o[i] = fmaf(p, __ldg(vc + off + d), o[i] * alpha);
        }
        m = mn;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) sm_o[warp][d] = o[i];
    }
    if (lane == 0) { sm_ml[warp][0] = m; sm_ml[warp][1] = l; }
    __syncthreads();
    float M = sm_ml[0][0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) M = fmaxf(M, sm_ml[w][0]);
    float L = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) L += sm_ml[w][1] * ex2_approx(sm_ml[w][0] - M);
    for (int d = threadIdx.x; d < D; d += kThreads) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) acc += sm_o[w][d] * ex2_approx(sm_ml[w][0] - M);
        if (nsplit == 1) out[(size_t)b * E + col + d] = acc * (1.0f / fmaxf(L, 1e-20f));
        else scratch[((size_t)bh * nsplit + split) * rec_stride(D) + d] = acc;
    }
    if (nsplit > 1 && threadIdx.x == 0) {
        float *rec = scratch + ((size_t)bh * nsplit + split) * rec_stride(D);
        rec[rec_stride(D) - 4] = M;
        rec[rec_stride(D) - 3] = L;
    }
}

__global__ void __launch_bounds__(kThreads)
decode_combine_kernel(const float *__restrict__ scratch, float *__restrict__ out, int H, int D, int nsplit)
{
    dependency_wait();
    dependents_may_start();
    const int bh = blockIdx.x;
    const int b = bh / H, h = bh % H;
    const int stride = rec_stride(D);
    const float *rec = scratch + (size_t)bh * nsplit * stride;
    float M = -1e30f;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, rec[(size_t)s * stride + stride - 4]);
    float L = 0.0f;
    for (int s = 0; s < nsplit; ++s)
        L += rec[(size_t)s * stride + stride - 3] * ex2_approx(rec[(size_t)s * stride + stride - 4] - M);
    const float inv = 1.0f / fmaxf(L, 1e-20f);
    for (int d = threadIdx.x; d < D; d += kThreads) {
        float acc = 0.0f;
        for (int s = 0; s < nsplit; ++s)
            acc += rec[(size_t)s * stride + d] * ex2_approx(rec[(size_t)s * stride + stride - 4] - M);
        out[(size_t)b * H * D + (size_t)h * D + d] = acc * inv;
    }
}

}  // namespace

// Splits of the context: enough thread blocks for two waves over 148 SMs, at least 32 keys each.
int decode_splits(int B, int H, int D, int ctx)
{
    (void)D;
    const long long bh = (long long)B * H;
    if (bh <= 0 || ctx <= 0) return 1;
    long long want = (2 * 148 + bh - 1) / bh;
    long long cap = ctx / 32;
    if (cap < 1) cap = 1;
    if (want > cap) want = cap;
    if (want > 64) want = 64;
    if (want < 1) want = 1;
    return (int)want;
}

int launch_decode(const float *q, const float *kc, const float *vc, float *out, float *scratch,
                  int B, int H, int D, int ctx, int cap, int nsplit, cudaStream_t st, const int *pos_ptr)
{
    if (D > kMaxD) return fail(HIPGPT_ERR_UNSUPPORTED, "head_dim %d exceeds %d", D, kMaxD);
    if ((long long)B * H > 65535) return fail(HIPGPT_ERR_BAD_ARG, "B*H = %lld exceeds 65535 rows per launch", (long long)B * H);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    const dim3 grid(nsplit, B * H);
    // Overlapped launches: a kernel's blocks are placed while the kernel before it on the stream drains, and wait for it
    // before they read anything (the first statement of every kernel here).
    cudaError_t le = cudaSuccess;
    if (D % 4 == 0 && D <= 128) {
        if (D <= 32)
            le = launch_overlapped(decode_split_vec_kernel<8>, grid, dim3(kThreads), 0, st, q, kc, vc, out, scratch, H, D, ctx, cap, nsplit, qscale, pos_ptr);
        else if (D <= 64)
            le = launch_overlapped(decode_split_vec_kernel<16>, grid, dim3(kThreads), 0, st, q, kc, vc, out, scratch, H, D, ctx, cap, nsplit, qscale, pos_ptr);
        else
            le = launch_overlapped(decode_split_vec_kernel<32>, grid, dim3(kThreads), 0, st, q, kc, vc, out, scratch, H, D, ctx, cap, nsplit, qscale, pos_ptr);
    } else {
        le = launch_overlapped(decode_split_scalar_kernel, grid, dim3(kThreads), 0, st, q, kc, vc, out, scratch, H, D, ctx, cap, nsplit, qscale, pos_ptr);
    }
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "decode_split_kernel launch: %s", cudaGetErrorString(le));
    int rc = check_launch("decode_split_kernel");
    if (rc != HIPGPT_OK || nsplit == 1) return rc;
    le = launch_overlapped(decode_combine_kernel, dim3(B * H), dim3(kThreads), 0, st, (const float *)scratch, out, H, D, nsplit);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "decode_combine_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("decode_combine_kernel");
}

}  // namespace hipgpt

// ---------------------------------------------------------------------------------------------
// hipgpt_mha_decode_noalloc: the split-context decode for callers that cannot bring scratch.
//
// Who that is.  The reference-shaped call sites of this library keep no state and own no spare
// buffers: a launcher in HipGPT's style is `void launch_x(const float*, float*, ints...)`, and
// the objects that call it (TransformerLayer) allocate a fixed set of activations once per
// (batch, sequence) shape.  A generation loop built on them reaches this kernel once per token
// and layer, from code that has nowhere to keep a scratch pointer and must not call cudaMalloc
// there: an allocation in the token loop synchronises the whole device, and a serving process
// that has handed all free memory to its own pool may simply be refused.  For those callers
// the partial results live in the array below, which is part of the library image: every GPU
// that loads the library sets these bytes aside until the process exits, so the size is modest.
//
// Rules of use
//   * B*H*splits*(roundup4(D)+4)*4 bytes must fit in HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES; a
//     larger request is refused with HIPGPT_ERR_SCRATCH (use hipgpt_mha_decode instead).
//   * All calls on one GPU share the one array.  Two calls whose kernels may overlap on the
//     GPU (different streams, no dependency between them) race on it; serialise them.
//   * The array keeps what the last call left.  Nothing needs clearing: the first kernel
//     writes every partial record the second one reads.
//   * Every call looks the array's device address up with the device current (a lookup, not an
//     allocation; nothing is cached, so the entry point stays valid after a cudaDeviceReset).
//     The first lookup on a device loads the library's module there: make that first call
//     before any stream capture begins on that device.
// ---------------------------------------------------------------------------------------------
namespace hipgpt {
namespace {

constexpr size_t kNoAllocFloats = HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_decode_scratch[kNoAllocFloats];

// Device address of g_decode_scratch on the current device.  In host code the array's name is
// only a handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress,
// asked while the device that will run the kernel is current.  It is asked on every call and
// never kept: after the first call on a device it is a table lookup, and an address kept across a
// cudaDeviceReset (or the loss of the primary context) would point into memory that is gone.
int decode_scratch_address(float **addr)
{
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr)
        return fail(HIPGPT_ERR_CUDA, "cudaGetSymbolAddress(decode scratch): %s", cudaGetErrorString(e));
    *addr = static_cast<float *>(p);
    return HIPGPT_OK;
}

}  // namespace
}  // namespace hipgpt

extern "C" int hipgpt_mha_decode_noalloc(const float *d_q, const float *d_kcache, const float *d_vcache, float *d_out,
                                         int B, int H, int D, int ctx, int cap, void *stream)
{
    using namespace hipgpt;
    if (B < 0 || H <= 0 || D <= 0 || ctx < 0 || cap < ctx)
        return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d H=%d D=%d ctx=%d cap=%d", B, H, D, ctx, cap);
    if (B == 0) return HIPGPT_OK;
    if (!d_q || !d_out || (ctx > 0 && (!d_kcache || !d_vcache)))
        return fail(HIPGPT_ERR_NULL, "q, out and the caches must not be NULL");
    const int ns = ctx > 0 ? decode_splits(B, H, D, ctx) : 1;
    const size_t need = ns > 1 ? (size_t)B * H * ns * rec_stride(D) * sizeof(float) : 0;
    if (need > (size_t)HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES)
        return fail(HIPGPT_ERR_SCRATCH,
                    "decode without allocation holds %zu bytes of partial results, this call needs %zu "
                    "(B=%d H=%d D=%d ctx=%d); use hipgpt_mha_decode with caller scratch",
                    (size_t)HIPGPT_DECODE_NOALLOC_SCRATCH_BYTES, need, B, H, D, ctx);
    float *scratch = nullptr;
    const int rc = decode_scratch_address(&scratch);
    if (rc != HIPGPT_OK) return rc;
    // only the vector kernels (head_dim % 4 == 0, up to 128) move 16 bytes at a time
    if (D % 4 == 0 && D <= 128 && ((reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_kcache) |
                                    reinterpret_cast<uintptr_t>(d_vcache) | reinterpret_cast<uintptr_t>(d_out)) & 15) != 0)
        return fail(HIPGPT_ERR_BAD_ARG, "decode needs 16-byte aligned pointers");
    return launch_decode(d_q, d_kcache, d_vcache, d_out, scratch, B, H, D, ctx, cap, ns, static_cast<cudaStream_t>(stream));
}
