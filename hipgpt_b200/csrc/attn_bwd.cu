// Attention backward: dQ, dK, dV from dO, Q, K, V and either the stored probabilities or nothing
// more (the probabilities are then recomputed from row maxima and sums that this file forms itself).
//
// Replaces multihead_attention_backward_kernel behind launch_multihead_attention_backward
// (HipGPT src/hip_kernels.cpp:1162-1272; consumer src/transformer_layer.cpp:285-286).  Per (batch, head),
// with g_i = dO_i, c = 1/sqrt(D):
//     vd_ij = g_i . V_j            w_i  = sum_j P_ij vd_ij        ds_ij = P_ij (vd_ij - w_i)
//     dQ_i  = c sum_j ds_ij K_j    dK_j = c sum_i ds_ij Q_i       dV_j  = sum_i P_ij g_i
// The reference gives one thread a query row and adds its dK, dV terms with atomicAdd, so the order
// of those additions changes from run to run there.  Here nothing is atomic: one kernel owns query
// rows (w_i, dQ_i), a second one owns key rows (dK_j, dV_j) and adds over the queries in ascending
// order, so results are reproducible, and equal to the reference's to rounding.
//
// The stored probabilities [B][H][S][S] are the only reason the forward has to write 4 B H S^2
// bytes.  When they are not given, P_ij = 2^(c log2e q_i.k_j - lse_i) is formed again from Q and K;
// lse_i (log2 of the row's sum of exponentials, plus its maximum) comes from a first sweep of the
// row kernel.  Scratch: w_i and lse_i, 2 B H S floats, from the caller.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kBwdThreads = 256;
constexpr int kBwdWarps = kBwdThreads / 32;
constexpr int kBwdTile = 32;           // rows of the other side staged in shared memory at a time
constexpr int kBwdMaxD = 128;

// dot product of a register-held vector with a row of a [32][D + 1] shared-memory tile
template <int DP>
__device__ __forceinline__ float dot_row(const float (&a)[DP], const float *row, int D)
{
    float s = 0.0f;
#pragma unroll
    for (int d = 0; d < DP; ++d)
        if (d < D) s = fmaf(a[d], row[d], s);
    return s;
}

// ---- kernel 1: one warp per query row: lse_i (when P is recomputed), w_i, dQ_i -----------------------
template <int DP, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads)
attn_bwd_rows_kernel(const float *__restrict__ G, const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                     const float *__restrict__ P, float *__restrict__ dQ, float *__restrict__ wsum, float *__restrict__ lse,
                     int S, int E, int H, int D, float c)
{
    extern __shared__ float smem[];
    float *ks = smem, *vs = ks + kBwdTile * (DP + 1);          // [32][DP + 1] each
    float *dsb = vs + kBwdTile * (DP + 1);                     // [warps][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int i = blockIdx.x * kBwdWarps + warp;               // query row of this warp
    const bool live = i < S;
    const size_t tok0 = (size_t)b * S, hcol = (size_t)h * D;
    const int ntiles = (S + kBwdTile - 1) / kBwdTile;
    const float cl2 = c * kLog2e;

    float q[DP], g[DP];
#pragma unroll
    for (int d = 0; d < DP; ++d) {
        q[d] = (live && d < D) ? Q[(tok0 + i) * E + hcol + d] : 0.0f;
        g[d] = (live && d < D) ? G[(tok0 + i) * E + hcol + d] : 0.0f;
    }
    auto stage = [&](int t, bool want_k, bool want_v) {
        __syncthreads();
        for (int f = threadIdx.x; f < kBwdTile * D; f += kBwdThreads) {
            const int r = f / D, d = f % D, j = t * kBwdTile + r;
            if (want_k) ks[r * (DP + 1) + d] = j < S ? K[(tok0 + j) * E + hcol + d] : 0.0f;
            if (want_v) vs[r * (DP + 1) + d] = j < S ? V[(tok0 + j) * E + hcol + d] : 0.0f;
        }
        __syncthreads();
    };
    const int jend = CAUSAL ? i + 1 : S;                        // keys this row sees

    // sweep 0 (only without stored probabilities): the row's maximum and sum of exponentials
    float my_lse = 0.0f;
    if (!P) {
        float m = -INFINITY, l = 0.0f;
        for (int t = 0; t < ntiles; ++t) {
            stage(t, true, false);
            const int j = t * kBwdTile + lane;
            const float s = (live && j < jend) ? dot_row<DP>(q, ks + lane * (DP + 1), D) * cl2 : -INFINITY;
            float tm = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float mn = fmaxf(m, tm);
            float e = (s == -INFINITY) ? 0.0f : exp2f(s - mn);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
            l = (mn == -INFINITY) ? 0.0f : l * exp2f(m - mn) + e;
            m = mn;
        }
        my_lse = m + log2f(fmaxf(l, 1e-30f));
        if (live && lane == 0) lse[(size_t)bh * S + i] = my_lse;
    }
    auto prob = [&](int j, float s_scaled) -> float {       // P_ij for a visible key
        return P ? P[((size_t)bh * S + i) * S + j] : exp2f(s_scaled - my_lse);
    };

    // sweep 1: w_i = sum_j P_ij (g_i . V_j)
    float w = 0.0f;
    for (int t = 0; t < ntiles; ++t) {
        stage(t, !P, true);
        const int j = t * kBwdTile + lane;
        if (live && j < jend) {
            const float s = P ? 0.0f : dot_row<DP>(q, ks + lane * (DP + 1), D) * cl2;
            w = fmaf(prob(j, s), dot_row<DP>(g, vs + lane * (DP + 1), D), w);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if (live && lane == 0) wsum[(size_t)bh * S + i] = w;

    // sweep 2: dQ_i = c sum_j ds_ij K_j, the lanes now standing for head-dim columns
    float acc[(DP + 31) / 32];
#pragma unroll
    for (int u = 0; u < (DP + 31) / 32; ++u) acc[u] = 0.0f;
    for (int t = 0; t < ntiles; ++t) {
        stage(t, true, true);
        const int j = t * kBwdTile + lane;
        float ds = 0.0f;
        if (live && j < jend) {
            const float s = dot_row<DP>(q, ks + lane * (DP + 1), D) * cl2;
            ds = prob(j, s) * (dot_row<DP>(g, vs + lane * (DP + 1), D) - w);
        }
        dsb[warp * 32 + lane] = ds;
        __syncwarp();
#pragma unroll
        for (int u = 0; u < (DP + 31) / 32; ++u) {
            const int d = lane + 32 * u;
            if (d < D)
                for (int r = 0; r < kBwdTile; ++r) acc[u] = fmaf(dsb[warp * 32 + r], ks[r * (DP + 1) + d], acc[u]);
        }
        __syncwarp();
    }
    if (live)
#pragma unroll
        for (int u = 0; u < (DP + 31) / 32; ++u) {
            const int d = lane + 32 * u;
            if (d < D) dQ[(tok0 + i) * E + hcol + d] = acc[u] * c;
        }
}

// ---- kernel 2: one warp per key row: dK_j, dV_j, queries added in ascending order ----------------------
template <int DP, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads)
attn_bwd_cols_kernel(const float *__restrict__ G, const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                     const float *__restrict__ P, const float *__restrict__ wsum, const float *__restrict__ lse,
                     float *__restrict__ dK, float *__restrict__ dV, int S, int E, int H, int D, float c)
{
    extern __shared__ float smem[];
    float *qs = smem, *gs = qs + kBwdTile * (DP + 1);          // [32][DP + 1] each: Q and dO rows of a query tile
    float *dsb = gs + kBwdTile * (DP + 1), *pb = dsb + kBwdWarps * 32;   // [warps][32] each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int j = blockIdx.x * kBwdWarps + warp;               // key row of this warp
    const bool live = j < S;
    const size_t tok0 = (size_t)b * S, hcol = (size_t)h * D;
    const int ntiles = (S + kBwdTile - 1) / kBwdTile;
    const float cl2 = c * kLog2e;

    float k[DP], v[DP];
#pragma unroll
    for (int d = 0; d < DP; ++d) {
        k[d] = (live && d < D) ? K[(tok0 + j) * E + hcol + d] : 0.0f;
        v[d] = (live && d < D) ? V[(tok0 + j) * E + hcol + d] : 0.0f;
    }
    float ak[(DP + 31) / 32], av[(DP + 31) / 32];
#pragma unroll
    for (int u = 0; u < (DP + 31) / 32; ++u) ak[u] = av[u] = 0.0f;
    // with the causal mask the first query that sees key j is query j: the tiles before it contribute nothing
    const int t0 = CAUSAL ? (blockIdx.x * kBwdWarps) / kBwdTile : 0;
    for (int t = t0; t < ntiles; ++t) {
        __syncthreads();
        for (int f = threadIdx.x; f < kBwdTile * D; f += kBwdThreads) {
            const int r = f / D, d = f % D, i = t * kBwdTile + r;
            qs[r * (DP + 1) + d] = i < S ? Q[(tok0 + i) * E + hcol + d] : 0.0f;
            gs[r * (DP + 1) + d] = i < S ? G[(tok0 + i) * E + hcol + d] : 0.0f;
        }
        __syncthreads();
        const int i = t * kBwdTile + lane;
        float p = 0.0f, ds = 0.0f;
        if (live && i < S && (!CAUSAL || j <= i)) {
            p = P ? P[((size_t)bh * S + i) * S + j]
                  : exp2f(dot_row<DP>(k, qs + lane * (DP + 1), D) * cl2 - lse[(size_t)bh * S + i]);
            ds = p * (dot_row<DP>(v, gs + lane * (DP + 1), D) - wsum[(size_t)bh * S + i]);
        }
        dsb[warp * 32 + lane] = ds;
        pb[warp * 32 + lane] = p;
        __syncwarp();
#pragma unroll
        for (int u = 0; u < (DP + 31) / 32; ++u) {
            const int d = lane + 32 * u;
            if (d < D)
                for (int r = 0; r < kBwdTile; ++r) {
                    ak[u] = fmaf(dsb[warp * 32 + r], qs[r * (DP + 1) + d], ak[u]);
                    av[u] = fmaf(pb[warp * 32 + r], gs[r * (DP + 1) + d], av[u]);
                }
        }
        __syncwarp();
    }
    if (live)
#pragma unroll
        for (int u = 0; u < (DP + 31) / 32; ++u) {
            const int d = lane + 32 * u;
            if (d < D) {
                dK[(tok0 + j) * E + hcol + d] = ak[u] * c;
                dV[(tok0 + j) * E + hcol + d] = av[u];
            }
        }
}

template <int DP, bool CAUSAL>
int launch_bwd_cfg(const float *g, const float *q, const float *k, const float *v, const float *probs, float *dq, float *dk, float *dv,
                   float *scratch, int B, int S, int E, int H, cudaStream_t st)
{
    const int D = E / H;
    const float c = 1.0f / sqrtf((float)D);
    float *wsum = scratch, *lse = scratch + (size_t)B * H * S;
    const dim3 grid((S + kBwdWarps - 1) / kBwdWarps, B * H);
    if ((long long)B * H > 65535) return fail(HIPGPT_ERR_BAD_ARG, "B*H = %lld exceeds 65535 rows per launch", (long long)B * H);
    const size_t sm1 = (size_t)(2 * kBwdTile * (DP + 1) + kBwdWarps * 32) * sizeof(float);
    const size_t sm2 = (size_t)(2 * kBwdTile * (DP + 1) + 2 * kBwdWarps * 32) * sizeof(float);
    attn_bwd_rows_kernel<DP, CAUSAL><<<grid, kBwdThreads, sm1, st>>>(g, q, k, v, probs, dq, wsum, lse, S, E, H, D, c);
    int rc = check_launch("attn_bwd_rows_kernel");
    if (rc != HIPGPT_OK) return rc;
    attn_bwd_cols_kernel<DP, CAUSAL><<<grid, kBwdThreads, sm2, st>>>(g, q, k, v, probs, wsum, lse, dk, dv, S, E, H, D, c);
    return check_launch("attn_bwd_cols_kernel");
}

}  // namespace

size_t mha_backward_scratch_bytes(int B, int H, int S) { return (size_t)2 * B * H * S * sizeof(float); }

int launch_mha_backward(const float *g, const float *q, const float *k, const float *v, const float *probs,
                        float *dq, float *dk, float *dv, float *scratch, int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (D > kBwdMaxD) return fail(HIPGPT_ERR_UNSUPPORTED, "attention backward: head_dim %d exceeds %d", D, kBwdMaxD);
    if (B == 0 || S == 0) return HIPGPT_OK;
#define HIPGPT_BWD(DP) (causal ? launch_bwd_cfg<DP, true>(g, q, k, v, probs, dq, dk, dv, scratch, B, S, E, H, st) \
                               : launch_bwd_cfg<DP, false>(g, q, k, v, probs, dq, dk, dv, scratch, B, S, E, H, st))
    if (D <= 32) return HIPGPT_BWD(32);
    if (D <= 64) return HIPGPT_BWD(64);
    return HIPGPT_BWD(128);
#undef HIPGPT_BWD
}

}  // namespace hipgpt
