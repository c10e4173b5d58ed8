// The unfused attention chain on head-contiguous [B'][S][D] tensors (sm_100a):
//   scaled dot product   replaces scaled_dot_product_kernel      src/hip_kernels.cpp:455-473
//   row softmax          replaces softmax_kernel                 src/hip_kernels.cpp:478-511
//   weighted sum         replaces attention_weighted_sum_kernel  src/hip_kernels.cpp:514-532
//
// The reference gives each query row to one thread, which walks its operands alone.  Here
// the two contractions are tiled through shared memory so that global loads are coalesced,
// while every output keeps the reference's arithmetic: a single accumulator that starts at
// 0.0f, the reduction index ascending, one fused multiply-add per term.  Their results are
// therefore the same bits as that arithmetic evaluated anywhere else.  The softmax gives a
// row to a warp; its sum is a tree, so it agrees with the reference to rounding only.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kTile = 32;

// scores[b][i][j] = (sum_d Q[b][i][d] * K[b][j][d]) * (1 / sqrt(D))
__global__ void __launch_bounds__(kTile * 8)
sdp_kernel(const float *__restrict__ Q, const float *__restrict__ K, float *__restrict__ scores, int S, int D, float inv)
{
    __shared__ float qs[kTile][kTile + 1];
    __shared__ float ks[kTile][kTile + 1];
    const int b = blockIdx.z;
    const int i0 = blockIdx.y * kTile, j0 = blockIdx.x * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;          // 32 x 8
    const float *Qb = Q + (size_t)b * S * D;
    const float *Kb = K + (size_t)b * S * D;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int d0 = 0; d0 < D; d0 += kTile) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = ty + 8 * r;
            const int d = d0 + tx;
            qs[row][tx] = (i0 + row < S && d < D) ? Qb[(size_t)(i0 + row) * D + d] : 0.0f;
            ks[row][tx] = (j0 + row < S && d < D) ? Kb[(size_t)(j0 + row) * D + d] : 0.0f;
        }
        __syncthreads();
        const int dn = min(kTile, D - d0);                  // never add padding terms: -0.0f + 0.0f would change a sign bit
        for (int d = 0; d < dn; ++d) {
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[r] = fmaf(qs[ty + 8 * r][d], ks[tx][d], acc[r]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = i0 + ty + 8 * r, j = j0 + tx;
        if (i < S && j < S) scores[((size_t)b * S + i) * S + j] = acc[r] * inv;
    }
}

// one warp per row of S scores
__global__ void __launch_bounds__(128)
softmax_rows_kernel(const float *scores, float *out, long long rows, int S)   // may alias: in-place is allowed
{
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float *src = scores + (size_t)row * S;
    float *dst = out + (size_t)row * S;
    float mx = -1e30f;
    for (int j = lane; j < S; j += 32) mx = fmaxf(mx, src[j]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.0f;
    for (int j = lane; j < S; j += 32) {
        const float e = expf(src[j] - mx);
        dst[j] = e;
        sum += e;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = 1.0f / fmaxf(sum, 1e-20f);
    for (int j = lane; j < S; j += 32) dst[j] *= inv;     // each lane re-reads only what it wrote
}

// out[b][i][d] = sum_j P[b][i][j] * V[b][j][d], j ascending
__global__ void __launch_bounds__(kTile * 8)
weighted_sum_kernel(const float *__restrict__ P, const float *__restrict__ V, float *__restrict__ out, int S, int D)
{
    __shared__ float ps[kTile][kTile + 1];
    __shared__ float vs[kTile][kTile + 1];
    const int b = blockIdx.z;
    const int i0 = blockIdx.y * kTile, d0 = blockIdx.x * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const float *Pb = P + (size_t)b * S * S;
    const float *Vb = V + (size_t)b * S * D;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int j0 = 0; j0 < S; j0 += kTile) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = ty + 8 * r;
            ps[row][tx] = (i0 + row < S && j0 + tx < S) ? Pb[(size_t)(i0 + row) * S + j0 + tx] : 0.0f;
            vs[row][tx] = (j0 + row < S && d0 + tx < D) ? Vb[(size_t)(j0 + row) * D + d0 + tx] : 0.0f;
        }
        __syncthreads();
        const int jn = min(kTile, S - j0);
        for (int j = 0; j < jn; ++j) {
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[r] = fmaf(ps[ty + 8 * r][j], vs[j][tx], acc[r]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = i0 + ty + 8 * r, d = d0 + tx;
        if (i < S && d < D) out[((size_t)b * S + i) * D + d] = acc[r];
    }
}

}  // namespace

int launch_sdp(const float *Q, const float *K, float *scores, int B, int S, int D, cudaStream_t st)
{
    const float inv = 1.0f / sqrtf((float)D);              // IEEE divide and sqrt: the host's value
    // the batch index rides on grid.z, which holds 65535 at most: more batch items take several launches
    for (int b0 = 0; b0 < B; b0 += 65535) {
        const int nb = B - b0 < 65535 ? B - b0 : 65535;
        const dim3 grid((S + kTile - 1) / kTile, (S + kTile - 1) / kTile, nb), block(kTile, 8);
        sdp_kernel<<<grid, block, 0, st>>>(Q + (size_t)b0 * S * D, K + (size_t)b0 * S * D, scores + (size_t)b0 * S * S, S, D, inv);
        const int rc = check_launch("sdp_kernel");
        if (rc != HIPGPT_OK) return rc;
    }
    return HIPGPT_OK;
}

int launch_softmax_rows(const float *scores, float *out, int B, int S, cudaStream_t st)
{
    const long long rows = (long long)B * S;
    const long long blocks = (rows + 3) / 4;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "too many rows");
    softmax_rows_kernel<<<(unsigned)blocks, 128, 0, st>>>(scores, out, rows, S);
    return check_launch("softmax_rows_kernel");
}

int launch_weighted_sum(const float *P, const float *V, float *out, int B, int S, int D, cudaStream_t st)
{
    for (int b0 = 0; b0 < B; b0 += 65535) {
        const int nb = B - b0 < 65535 ? B - b0 : 65535;
        const dim3 grid((D + kTile - 1) / kTile, (S + kTile - 1) / kTile, nb), block(kTile, 8);
        weighted_sum_kernel<<<grid, block, 0, st>>>(P + (size_t)b0 * S * S, V + (size_t)b0 * S * D, out + (size_t)b0 * S * D, S, D);
        const int rc = check_launch("weighted_sum_kernel");
        if (rc != HIPGPT_OK) return rc;
    }
    return HIPGPT_OK;
}

}  // namespace hipgpt
