// Fused exact-fp32 attention forward for head_dim 32 / 64 / 128 on sm_100a.
//
// Replaces the two kernels behind HipGPT's launch_multihead_attention
// (src/hip_kernels.cpp:263-325 flash_attention_kernel, :329-402 fallback kernel).
//
// Design ("rows" kernel)
//   * A thread owns R = 2 query rows: their 32-wide slice of q and of the output accumulator
//     live in registers for the whole kernel (head_dim 64 / 128 split a row over 2 / 4
//     neighbouring lanes, joined by one shuffle-add per score).
//   * K and V stream through shared memory in tiles of KT keys, double buffered with
//     16-byte cp.async copies, so every K/V element is fetched once per thread block.
//     All lanes of a warp read the same K (or V) address at the same time: a broadcast,
//     free of bank conflicts, and each 128-bit shared load feeds 4*R FMAs.
//   * Online softmax over chunks of C keys: scores are kept in the log2 domain
//     (q is pre-multiplied by log2(e)/sqrt(D)), one ex2 per score, the accumulator is
//     rescaled once per chunk.  The contraction itself is plain fp32 FFMA.
//   * Causal mode walks only the key tiles at or below the block's last query, orders the
//     grid heaviest block first, skips whole chunks per warp, drops a warp's lower row group
//     once the keys have passed it, and masks only the chunks that cross the diagonal.
//   * Probabilities, when asked for, are produced by a second sweep that recomputes the
//     scores against the final row maximum and sum (nothing is stored in between).
//   * Q and O are moved with 128-bit accesses, a full 128-byte line per thread and row.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

template <int NT>
__device__ __forceinline__ float group_sum(float x)
{
#pragma unroll
    for (int o = 1; o < NT; o <<= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Scores of RA rows (the last RA of the thread's R rows) against C keys of the staged tile.
template <int D, int R, int RA, int C>
__device__ __forceinline__ void qk_chunk(const float (&q)[R][32], const float *__restrict__ kb, float (&s)[R][C])
{
    constexpr int R0 = R - RA;
#pragma unroll
    for (int r = R0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < C; ++c) s[r][c] = 0.0f;
#pragma unroll
    for (int d4 = 0; d4 < 8; ++d4) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const float4 kv = *reinterpret_cast<const float4 *>(kb + c * D + d4 * 4);
#pragma unroll
            for (int r = R0; r < R; ++r) {
                s[r][c] = fmaf(q[r][d4 * 4 + 0], kv.x, s[r][c]);
                s[r][c] = fmaf(q[r][d4 * 4 + 1], kv.y, s[r][c]);
                s[r][c] = fmaf(q[r][d4 * 4 + 2], kv.z, s[r][c]);
                s[r][c] = fmaf(q[r][d4 * 4 + 3], kv.w, s[r][c]);
            }
        }
    }
    if (D > 32) {
#pragma unroll
        for (int r = R0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < C; ++c) s[r][c] = group_sum<D / 32>(s[r][c]);
    }
}

// One chunk of C keys: scores, online-softmax update, accumulate P.V.
template <int D, int R, int RA, int C, bool CAUSAL>
__device__ __forceinline__ void attend_chunk(const float (&q)[R][32], float (&o)[R][32], float (&m)[R], float (&l)[R],
                                             const int (&qi)[R], const float *__restrict__ kb,
                                             const float *__restrict__ vb, int jc, int S, bool need_mask)
{
    constexpr int R0 = R - RA;
    float s[R][C];
    qk_chunk<D, R, RA, C>(q, kb, s);
    if (need_mask) {
#pragma unroll
        for (int r = R0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const int j = jc + c;
                if (j >= S || (CAUSAL && j > qi[r])) s[r][c] = -INFINITY;
            }
    }
#pragma unroll
    for (int r = R0; r < R; ++r) {
        float mx = s[r][0];
#pragma unroll
        for (int c = 1; c < C; ++c) mx = fmaxf(mx, s[r][c]);
        const float mn = fmaxf(m[r], mx);
        const float alpha = ex2_approx(m[r] - mn);
        m[r] = mn;
        float psum = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const float p = ex2_approx(s[r][c] - mn);
            s[r][c] = p;
            psum += p;
        }
        l[r] = fmaf(l[r], alpha, psum);
#pragma unroll
        for (int d = 0; d < 32; ++d) o[r][d] *= alpha;
    }
#pragma unroll
    for (int c = 0; c < C; ++c) {
#pragma unroll
        for (int d4 = 0; d4 < 8; ++d4) {
            const float4 vv = *reinterpret_cast<const float4 *>(vb + c * D + d4 * 4);
#pragma unroll
            for (int r = R0; r < R; ++r) {
                o[r][d4 * 4 + 0] = fmaf(s[r][c], vv.x, o[r][d4 * 4 + 0]);
                o[r][d4 * 4 + 1] = fmaf(s[r][c], vv.y, o[r][d4 * 4 + 1]);
                o[r][d4 * 4 + 2] = fmaf(s[r][c], vv.z, o[r][d4 * 4 + 2]);
                o[r][d4 * 4 + 3] = fmaf(s[r][c], vv.w, o[r][d4 * 4 + 3]);
            }
        }
    }
}

template <int D, int R, int WARPS, int KT, int C, bool CAUSAL, bool PROBS>
__global__ void __launch_bounds__(WARPS * 32)
mha_rows_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                float *__restrict__ O, float *__restrict__ P, int S, int E, int H, int BH, int nqblk, float qscale)
{
    constexpr int NT = D / 32;         // lanes that share one query row
    constexpr int G = 32 / NT;         // query rows per warp and row group
    constexpr int QW = G * R;          // query rows per warp
    constexpr int QB = QW * WARPS;     // query rows per thread block
    constexpr int THREADS = WARPS * 32;
    static_assert(KT % C == 0 && C % 4 == 0, "tile/chunk shape");

    extern __shared__ __align__(16) float smem[];
    float *ks = smem;                  // [2][KT][D]
    float *vs = smem + 2 * KT * D;     // [2][KT][D]

    const int tid = threadIdx.x, lane = tid & 31;
    // read from one lane, so that the compiler knows the warp's number (and every role that follows from it) to be warp-uniform
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int grp = lane / NT, part = lane % NT;
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);   // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * QB;
    const int wq0 = q0 + warp * QW;

    int qi[R];
    float q[R][32], o[R][32], m[R], l[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        qi[r] = wq0 + r * G + grp;
        m[r] = -1e30f;
        l[r] = 0.0f;
        if (qi[r] < S) {
            const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + qi[r]) * (size_t)E + hcol + part * 32);
#pragma unroll
            for (int d4 = 0; d4 < 8; ++d4) {
                const float4 t = __ldg(src + d4);
                q[r][d4 * 4 + 0] = t.x * qscale;
                q[r][d4 * 4 + 1] = t.y * qscale;
                q[r][d4 * 4 + 2] = t.z * qscale;
                q[r][d4 * 4 + 3] = t.w * qscale;
            }
        } else {
#pragma unroll
            for (int d = 0; d < 32; ++d) q[r][d] = 0.0f;
        }
#pragma unroll
        for (int d = 0; d < 32; ++d) o[r][d] = 0.0f;
    }

    const int kend_cta = CAUSAL ? min(S, q0 + QB) : S;      // keys [0, kend) are walked
    const int ntiles = (kend_cta + KT - 1) / KT;
    const int kend_warp = CAUSAL ? min(S, wq0 + QW) : S;

    auto load_tile = [&](int t, int buf) {
        constexpr int V4 = D / 4;
        for (int i = tid; i < KT * V4; i += THREADS) {
            const int row = i / V4, c4 = i % V4;
            const int j = t * KT + row;
            const bool ok = j < S;
            const size_t g = (tok0 + (ok ? j : 0)) * (size_t)E + hcol + c4 * 4;
            cp_async16(ks + (buf * KT + row) * D + c4 * 4, K + g, ok);
            cp_async16(vs + (buf * KT + row) * D + c4 * 4, V + g, ok);
        }
        cp_async_commit();
    };

    if (ntiles > 0) load_tile(0, 0);
    for (int t = 0; t < ntiles; ++t) {
        cp_async_wait_all();
        __syncthreads();
        if (t + 1 < ntiles) load_tile(t + 1, (t + 1) & 1);
        const int j0 = t * KT;
        if (j0 < kend_warp) {
            const float *kb = ks + (t & 1) * KT * D + part * 32;
            const float *vb = vs + (t & 1) * KT * D + part * 32;
#pragma unroll 1
            for (int c0 = 0; c0 < KT; c0 += C) {
                const int jc = j0 + c0;
                if (jc >= kend_warp) break;
                // the lower row group (queries wq0 .. wq0+G-1) is finished once jc is past it
                const bool low_active = !CAUSAL || R == 1 || (jc <= wq0 + G - 1);
                const int first_q = low_active ? wq0 : wq0 + (R - 1) * G;
                const bool need_mask = (jc + C > S) || (CAUSAL && (jc + C - 1 > first_q));
                if (R > 1 && !low_active)
                    attend_chunk<D, R, 1, C, CAUSAL>(q, o, m, l, qi, kb + c0 * D, vb + c0 * D, jc, S, need_mask);
                else
                    attend_chunk<D, R, R, C, CAUSAL>(q, o, m, l, qi, kb + c0 * D, vb + c0 * D, jc, S, need_mask);
            }
        }
    }

    float inv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        inv[r] = 1.0f / fmaxf(l[r], 1e-20f);
        if (qi[r] < S) {
            float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + qi[r]) * (size_t)E + hcol + part * 32);
#pragma unroll
            for (int d4 = 0; d4 < 8; ++d4)
                dst[d4] = make_float4(o[r][d4 * 4 + 0] * inv[r], o[r][d4 * 4 + 1] * inv[r],
                                      o[r][d4 * 4 + 2] * inv[r], o[r][d4 * 4 + 3] * inv[r]);
        }
    }

    if (PROBS) {
        // Second sweep: p = 2^(s - m) / l against the final m and l, written row by row.
        const bool vec_ok = (S % 4) == 0;
        float *prow[R];
#pragma unroll
        for (int r = 0; r < R; ++r) prow[r] = P + ((size_t)bh * S + (size_t)min(qi[r], S - 1)) * (size_t)S;
        __syncthreads();   // every warp is done with the last tile of the first sweep
        if (ntiles > 0) load_tile(0, 0);
        for (int t = 0; t < ntiles; ++t) {
            cp_async_wait_all();
            __syncthreads();
            if (t + 1 < ntiles) load_tile(t + 1, (t + 1) & 1);
            const int j0 = t * KT;
            const float *kb = ks + (t & 1) * KT * D + part * 32;
#pragma unroll 1
            for (int c0 = 0; c0 < KT; c0 += C) {
                const int jc = j0 + c0;
                if (jc >= S) break;
                float s[R][C];
                if (CAUSAL && jc >= kend_warp) {
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int c = 0; c < C; ++c) s[r][c] = 0.0f;
                } else {
                    qk_chunk<D, R, R, C>(q, kb + c0 * D, s);
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int c = 0; c < C; ++c) {
                            const int j = jc + c;
                            const bool dead = CAUSAL && j > qi[r];
                            s[r][c] = dead ? 0.0f : ex2_approx(s[r][c] - m[r]) * inv[r];
                        }
                }
                if (part == 0) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (qi[r] >= S) continue;
                        if (vec_ok && jc + C <= S) {
#pragma unroll
                            for (int c = 0; c < C; c += 4)
                                *reinterpret_cast<float4 *>(prow[r] + jc + c) =
                                    make_float4(s[r][c], s[r][c + 1], s[r][c + 2], s[r][c + 3]);
                        } else {
#pragma unroll
                            for (int c = 0; c < C; ++c)
                                if (jc + c < S) prow[r][jc + c] = s[r][c];
                        }
                    }
                }
            }
        }
        if (CAUSAL && part == 0) {
            // keys beyond the tiles this block walked: zeros
            const int jz = ntiles * KT;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (qi[r] >= S) continue;
                for (int j = jz; j < S; ++j) prow[r][j] = 0.0f;
            }
        }
    }
}

template <int D, int WARPS, bool CAUSAL, bool PROBS>
int launch_cfg(const float *q, const float *k, const float *v, float *out, float *probs,
               int B, int S, int E, int H, cudaStream_t st)
{
    constexpr int R = 2, KT = 32, C = 8;
    constexpr int QB = (32 / (D / 32)) * R * WARPS;
    auto kern = mha_rows_kernel<D, R, WARPS, KT, C, CAUSAL, PROBS>;
    const size_t smem = (size_t)4 * KT * D * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    const int nqblk = (S + QB - 1) / QB;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, WARPS * 32, smem, st>>>(q, k, v, out, probs, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_rows_kernel");
}

template <int D, int WARPS>
int launch_flags(const float *q, const float *k, const float *v, float *out, float *probs,
                 int B, int S, int E, int H, int causal, cudaStream_t st)
{
    if (causal) {
        return probs ? launch_cfg<D, WARPS, true, true>(q, k, v, out, probs, B, S, E, H, st)
                     : launch_cfg<D, WARPS, true, false>(q, k, v, out, probs, B, S, E, H, st);
    }
    return probs ? launch_cfg<D, WARPS, false, true>(q, k, v, out, probs, B, S, E, H, st)
                 : launch_cfg<D, WARPS, false, false>(q, k, v, out, probs, B, S, E, H, st);
}

template <int D>
int launch_warps(const float *q, const float *k, const float *v, float *out, float *probs,
                 int B, int S, int E, int H, int causal, int warps, cudaStream_t st)
{
    switch (warps) {
    case 1: return launch_flags<D, 1>(q, k, v, out, probs, B, S, E, H, causal, st);
    case 2: return launch_flags<D, 2>(q, k, v, out, probs, B, S, E, H, causal, st);
    case 4: return launch_flags<D, 4>(q, k, v, out, probs, B, S, E, H, causal, st);
    default: return fail(HIPGPT_ERR_BAD_ARG, "warps per block must be 1, 2 or 4 (got %d)", warps);
    }
}

}  // namespace

bool mha_rows_supports(int D) { return D == 32 || D == 64 || D == 128; }

int launch_mha_rows(const float *q, const float *k, const float *v, float *out, float *probs,
                    int B, int S, int E, int H, int causal, int warps, cudaStream_t st)
{
    const int D = E / H;
    if (warps == 0) {
        // Measured on B200: short causal problems (head_dim 32) run best with one warp per block
        // (finest load balance across the diagonal), everything else with two.
        warps = (causal && D == 32) ? 1 : 2;
    }
    switch (D) {
    case 32: return launch_warps<32>(q, k, v, out, probs, B, S, E, H, causal, warps, st);
    case 64: return launch_warps<64>(q, k, v, out, probs, B, S, E, H, causal, warps, st);
    case 128: return launch_warps<128>(q, k, v, out, probs, B, S, E, H, causal, warps, st);
    default: return fail(HIPGPT_ERR_UNSUPPORTED, "rows kernel: head_dim %d is not 32, 64 or 128", D);
    }
}

}  // namespace hipgpt
