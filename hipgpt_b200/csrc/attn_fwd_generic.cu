// Generic fused attention forward: any head_dim up to 512, any S (sm_100a).
//
// Takes the shapes the rows kernel does not (head_dim other than 32 / 64 / 128), the way the
// reference's fallback kernel takes what its flash kernel does not
// (src/hip_kernels.cpp:329-402, chosen at :422).  One warp owns one query row: the lanes split
// the keys for the scores (online softmax per lane, merged by shuffles) and split the head
// dimension for the P.V accumulation, so K and V rows are read with consecutive lanes on
// consecutive addresses.  Probabilities are written by a second sweep over the keys.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kMaxD = 512;
constexpr int kDPerLane = kMaxD / 32;
constexpr int kWarpsPerBlock = 4;

template <bool CAUSAL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
mha_generic_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                   float *__restrict__ O, float *__restrict__ P, int S, int E, int H, long long rows, float qscale)
{
    extern __shared__ float qs_all[];                     // [warps][D] scaled query rows
    const int D = E / H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarpsPerBlock + warp;
    if (row >= rows) return;                              // whole warp leaves together
    const int qi = (int)(row % S);
    const int h = (int)((row / S) % H);
    const int b = (int)(row / ((long long)S * H));
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    float *qs = qs_all + warp * D;
    for (int d = lane; d < D; d += 32) qs[d] = Q[(tok0 + qi) * (size_t)E + hcol + d] * qscale;
    __syncwarp();

    const int jend = CAUSAL ? qi + 1 : S;
    float acc[kDPerLane];
#pragma unroll
    for (int i = 0; i < kDPerLane; ++i) acc[i] = 0.0f;
    float m = -1e30f, l = 0.0f;

    for (int j0 = 0; j0 < jend; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j < jend) {
            const float *kr = K + (tok0 + j) * (size_t)E + hcol;
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], __ldg(kr + d), dot);
            s = dot;
        }
        float mx = s;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float mn = fmaxf(m, mx);
        const float alpha = ex2_approx(m - mn);
        const float p = ex2_approx(s - mn);               // 0 for the lanes past jend
        float ps = p;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        l = fmaf(l, alpha, ps);
        m = mn;
#pragma unroll
        for (int i = 0; i < kDPerLane; ++i) acc[i] *= alpha;
        const int nk = min(32, jend - j0);
        for (int jj = 0; jj < nk; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float *vr = V + (tok0 + j0 + jj) * (size_t)E + hcol;
#pragma unroll
            for (int i = 0; i < kDPerLane; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pj, __ldg(vr + d), acc[i]);
            }
        }
    }
    const float inv = 1.0f / fmaxf(l, 1e-20f);
#pragma unroll
    for (int i = 0; i < kDPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < D) O[(tok0 + qi) * (size_t)E + hcol + d] = acc[i] * inv;
    }

    if (P != nullptr) {
        float *prow = P + ((size_t)(b * (long long)H + h) * S + qi) * (size_t)S;
        for (int j0 = 0; j0 < S; j0 += 32) {
            const int j = j0 + lane;
            if (j >= S) break;
            float p = 0.0f;
            if (j < jend) {
                const float *kr = K + (tok0 + j) * (size_t)E + hcol;
                float dot = 0.0f;
                for (int d = 0; d < D; ++d) dot = fmaf(qs[d], __ldg(kr + d), dot);
                p = ex2_approx(dot - m) * inv;
            }
            prow[j] = p;
        }
    }
}

}  // namespace

int launch_mha_generic(const float *q, const float *k, const float *v, float *out, float *probs,
                       int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (D > kMaxD) return fail(HIPGPT_ERR_UNSUPPORTED, "head_dim %d exceeds %d", D, kMaxD);
    const long long rows = (long long)B * H * S;
    const long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    const size_t smem = (size_t)kWarpsPerBlock * D * sizeof(float);
    if (causal)
        mha_generic_kernel<true><<<(unsigned)blocks, kWarpsPerBlock * 32, smem, st>>>(q, k, v, out, probs, S, E, H, rows, qscale);
    else
        mha_generic_kernel<false><<<(unsigned)blocks, kWarpsPerBlock * 32, smem, st>>>(q, k, v, out, probs, S, E, H, rows, qscale);
    return check_launch("mha_generic_kernel");
}

}  // namespace hipgpt
