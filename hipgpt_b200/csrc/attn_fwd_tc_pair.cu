// Fused attention forward on the Blackwell tensor pipe, fp32-grade results (split-TF32), head_dim 32:
// the variant in which a thread block works on TWO query tiles of 128 rows that take turns on the
// tensor core, and the output accumulates in tensor memory across all key tiles.
//
// Replaces the same reference kernels as attn_fwd_tc.cu (HipGPT src/hip_kernels.cpp:263-325 and
// :329-402) and uses the same arithmetic: every fp32 operand x is cut into hi (TF32-exact) and
// lo = x - hi, and a product is accumulated as a_lo*b_hi + a_hi*b_lo + a_hi*b_hi in the tensor
// core's fp32 accumulator.  What differs is the schedule:
//   * 256 query rows of one (batch, head) per block = tiles A and B, each owned by 128 worker threads
//     (worker = query row = TMEM lane); both use every staged K/V tile, so staging work per query row
//     is halved;
//   * the issuing lane alternates  P V_x(t), Q K_x(t+1)^T  between x = A and x = B, so one tile's
//     products run while the other tile is in its softmax;
//   * O_ext_x = [P_hi V_hi | P_hi V_lo + P_lo V_hi] accumulates in TMEM over all tiles; a worker
//     does not read it back per tile.  The running maximum is only moved (and the accumulator
//     rescaled, by the whole warp) when a row's maximum grew by more than 2^8 since the last
//     rescale; until then exponentials may reach 2^8, which the hi / lo split carries without loss;
//   * producers (128 threads) fetch K(t+1), V(t+1) with cp.async into raw buffers, split them and
//     write the swizzled operand layouts into a two-stage ring (full / free mbarriers).
// TMEM columns per query tile: S (64, P_hi in place) | P_lo (64) | O_ext (64); 384 of 512 in use.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per tile (two tiles per block)
constexpr int kKeys = 64;         // keys per K/V tile
constexpr int kWorkers = 2 * kRows;
constexpr int kProducers = 128;
constexpr int kThreads = kWorkers + 32 + kProducers;
constexpr float kRescaleStep = 8.0f;     // log2 of the growth of a row maximum that forces a rescale
constexpr int D = 32;             // head_dim: one 128-byte row per operand row
constexpr int QBLK = kRows * 32;  // floats per [128][32] block
constexpr int KBLK = kKeys * 32;  // floats per [64][32] block
constexpr uint32_t kColsPerTile = 192, kColPlo = 64, kColO = 128;
constexpr uint32_t kTmemCols = 512;
// Q hi/lo of two tiles, two stages of K hi/lo, two stages of V [hi | lo], raw K and V
constexpr size_t kSmemFloats = (size_t)4 * QBLK + 4 * KBLK + 4 * KBLK + 2 * kKeys * D;

__device__ int g_pair_status = 0;

template <bool CAUSAL>
__global__ void __launch_bounds__(kThreads, 1)
mha_tc_pair_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                   float *__restrict__ O, int S, int E, int H, int BH, int nqblk, float qscale)
{
    constexpr int CPR = D / 4;                       // 16-byte chunks per row
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *q_hi = base, *q_lo = q_hi + 2 * QBLK;     // [tile][128][32] each
    float *k_hi = q_lo + 2 * QBLK;                   // [stage][hi, lo][64][32]
    float *v_s = k_hi + 4 * KBLK;                    // [stage][hi, lo][64][32]: hi and lo blocks form one 2D-column operand
    float *k_raw = v_s + 4 * KBLK, *v_raw = k_raw + kKeys * D;   // as the tiles lie in global memory
    __shared__ uint64_t k_full[2], k_free[2], v_full[2], v_free[2], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);     // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * 2 * kRows;

    // key tiles each query tile needs (0 when the tile lies past the end of the sequence)
    int nt[2];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int first = q0 + g * kRows;
        const int kend = CAUSAL ? min(S, first + kRows) : S;
        nt[g] = first < S ? (kend + kKeys - 1) / kKeys : 0;
    }
    const int NT = max(nt[0], nt[1]);

    if (tid == 0) {
        abort_flag = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], kProducers / 32);     // one arrival per producer warp
            mbar_init(&v_full[i], kProducers / 32);
            mbar_init(&k_free[i], 1);                // tcgen05.commit
            mbar_init(&v_free[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&o_done[i], 1);
            mbar_init(&p_full[i], kRows / 32);       // one arrival per worker warp of the tile
        }
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K staged,
    // 5 P written, 6 V staged, 7 K stage free, 8 V stage free
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) { abort_flag = 1; atomicCAS(&g_pair_status, 0, site); }
    };
    // one arrival for the whole warp: every lane's writes are ordered before it by the warp barrier
    auto arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };

    if (warp == kWorkers / 32) {
        // ================= the issuing warp =====================================================
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();                             // Q staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kRows, kKeys, 0);
            constexpr uint32_t idesc_pv1 = make_idesc(kRows, 2 * D, 1);      // P_hi x [V_hi | V_lo]
            constexpr uint32_t idesc_pv2 = make_idesc(kRows, D, 1);          // P_lo x V_hi
            auto issue_qk = [&](int g, int stage) {
                uint32_t acc = 0;
#pragma unroll
                for (int pass = 0; pass < 3; ++pass) {
                    // the two correction terms first: the accumulator is still tiny while they are added
                    const float *qa = (pass == 0 ? q_lo : q_hi) + g * QBLK;
                    const float *kb = k_hi + stage * 2 * KBLK + (pass == 1 ? KBLK : 0);
                    const uint64_t da = make_desc(smem_u32(qa), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(kb), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {            // 8 floats = 32 bytes per instruction
                        mma_ss(tmem + g * kColsPerTile, da + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, acc);
                        acc = 1;
                    }
                }
                tc_commit(&s_full[g]);
            };
            auto issue_pv = [&](int g, int stage, bool first) {
                // N-major B: 8 keys of 128 bytes per instruction = 1024 bytes
                const uint64_t dv = make_desc(smem_u32(v_s + stage * 2 * KBLK), KBLK * 4, 512, 1);
                const uint32_t t0 = tmem + g * kColsPerTile;
#pragma unroll
                for (int k = 0; k < kKeys / 8; ++k)
                    mma_ts(t0 + kColO, t0 + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv1, (first && k == 0) ? 0u : 1u);
                // the second correction term joins the first one in columns [D, 2D): both are small
#pragma unroll
                for (int k = 0; k < kKeys / 8; ++k)
                    mma_ts(t0 + kColO + D, t0 + kColPlo + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv2, 1);
                tc_commit(&o_done[g]);
            };
            if (NT > 0) {
                wait(&k_full[0], 0, 4);
                tc_fence_after();
#pragma unroll
                for (int g = 0; g < 2; ++g)
                    if (nt[g] > 0) issue_qk(g, 0);
                tc_commit(&k_free[0]);
            }
            for (int t = 0; t < NT; ++t) {
                const int st = t & 1;
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (t < nt[g]) {
                        wait(&p_full[g], (uint32_t)(t & 1), 5);                  // P_g(t) is in TMEM
                        wait(&v_full[st], (uint32_t)((t >> 1) & 1), 6);          // V(t) is in shared memory
                        tc_fence_after();
                        issue_pv(g, st, t == 0);
                    }
                    if (g == 1) tc_commit(&v_free[st]);                          // both tiles' P V(t) issued
                    if (t + 1 < nt[g]) {
                        wait(&k_full[st ^ 1], (uint32_t)(((t + 1) >> 1) & 1), 4);   // K(t+1) is in shared memory
                        tc_fence_after();
                        issue_qk(g, st ^ 1);                                     // executes after P V_g(t): S_g is free then
                    }
                    if (g == 1 && t + 1 < NT) tc_commit(&k_free[st ^ 1]);
                }
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read the outputs
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        return;
    }

    if (warp > kWorkers / 32) {
        // ================= the producers: global -> raw -> split -> operand layout ==============
        // The producer that fetched a 16-byte chunk is also the one that later splits it, so it
        // only waits for its own cp.async groups.
        constexpr int RPP = kProducers / CPR;        // rows per pass
        constexpr int NP = kKeys / RPP;              // passes per tile
        const int ptid = tid - kWorkers - 32;
        const int sc = ptid % CPR, sr0 = ptid / CPR;
        auto fetch_tile = [&](const float *__restrict__ plane, float *raw, int t) {
            if (t < NT) {
#pragma unroll
                for (int p = 0; p < NP; ++p) {
                    const int r = sr0 + p * RPP;
                    const int j = t * kKeys + r;
                    const bool ok = j < S;
                    cp_async16(raw + r * D + sc * 4, plane + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + sc * 4, ok);
                }
            }
            cp_async_commit();                       // an empty group keeps the count of the waits
        };
        auto store_k = [&](int stage) {
            float *blk = k_hi + stage * 2 * KBLK;
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const int r = sr0 + p * RPP;
                store_split(blk, blk + KBLK, r, sc, *reinterpret_cast<const float4 *>(k_raw + r * D + sc * 4));
            }
        };
        auto store_v = [&](int stage) {
            float *blk = v_s + stage * 2 * KBLK;
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const int r = sr0 + p * RPP;
                store_split_nmajor(blk, blk + KBLK, r, sc, *reinterpret_cast<const float4 *>(v_raw + r * D + sc * 4));
            }
        };
        fetch_tile(K, k_raw, 0);
        fetch_tile(V, v_raw, 0);
        __syncthreads();                             // matches the block-wide barrier after Q staging
        // iteration u stages K(u) and V(u) and starts the fetch of K(u+1), V(u+1)
        for (int u = 0; u < NT; ++u) {
            const int st = u & 1;
            if (u >= 2) wait(&k_free[st], (uint32_t)(((u >> 1) - 1) & 1), 7);    // both Q K(u-2)^T have completed
            cp_async_wait_1();                       // K(u) has landed (V(u) may still be in flight)
            store_k(st);
            proxy_fence();                           // generic-proxy writes -> visible to the tensor core
            arrive(&k_full[st]);
            fetch_tile(K, k_raw, u + 1);
            if (u >= 2) wait(&v_free[st], (uint32_t)(((u >> 1) - 1) & 1), 8);    // both P V(u-2) have completed
            cp_async_wait_1();                       // V(u) has landed
            store_v(st);
            proxy_fence();
            arrive(&v_full[st]);
            fetch_tile(V, v_raw, u + 1);
        }
        cp_async_wait_all();
        __syncthreads();
        return;
    }

    // ===================== the workers ===========================================================
    const int g = warp >> 2;                         // query tile A / B
    const int wq = warp & 3;                         // TMEM lane quadrant of this warp
    const int rloc = wq * 32 + lane;                 // row inside the tile = TMEM lane
    const int row = q0 + g * kRows + rloc;
    const int ntg = nt[g];
    {
        const bool ok = row < S;
        const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int c = 0; c < CPR; ++c) {
            float4 x = ok ? __ldg(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            x.x *= qscale; x.y *= qscale; x.z *= qscale; x.w *= qscale;     // scores come out in the log2 domain
            store_split(q_hi + g * QBLK, q_lo + g * QBLK, rloc, c, x);
        }
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16) + g * kColsPerTile;
    const uint32_t s_addr = lane_base, plo_addr = lane_base + kColPlo, o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (log2 domain) and row sum
    for (int t = 0; t < ntg; ++t) {
        const int j0 = t * kKeys;
        wait(&s_full[g], (uint32_t)(t & 1), 1);      // S_g(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + g * kRows + wq * 32;  // first row of this warp
        const bool warp_dead = CAUSAL && j0 > wrow0 + 31;          // these columns are above the diagonal for the whole warp
        const bool need_mask = (CAUSAL && j0 + kKeys - 1 > wrow0) || j0 + kKeys > S;
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : kKeys);     // visible columns of this row

        // ---- first sweep: the row maximum ----------------------------------------------------
        float mx = -INFINITY;
        if (!warp_dead) {
            float v0[32], v1[32];
            tmem_ld32(s_addr, v0);
            tmem_ld32(s_addr + 32, v1);
            tmem_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v0[c] = (c < nvalid) ? v0[c] : -INFINITY;
                    v1[c] = (32 + c < nvalid) ? v1[c] : -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                m4[(c >> 1) & 1] = fmaxf(m4[(c >> 1) & 1], fmaxf(v0[c], v0[c + 1]));
                m4[2 + ((c >> 1) & 1)] = fmaxf(m4[2 + ((c >> 1) & 1)], fmaxf(v1[c], v1[c + 1]));
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        if (t == 0) {
            m_ref = fmaxf(mx, -1e30f);
        } else {
            const bool grow = mx > m_ref + kRescaleStep;
            if (__any_sync(0xffffffffu, grow)) {
                // the accumulator is rescaled by the whole warp (TMEM accesses are warp-wide);
                // rows that did not grow use factor 1
                const float alpha = grow ? ex2_approx(m_ref - mx) : 1.0f;
                if (grow) m_ref = mx;
                l *= alpha;
                wait(&o_done[g], (uint32_t)((t - 1) & 1), 2);       // P V_g(t-1) has completed
                tc_fence_after();
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    float a[32];
                    tmem_ld32(o_addr + hh * 32, a);
                    tmem_wait_ld();
                    float lo[16], hi[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) { lo[c] = a[c] * alpha; hi[c] = a[16 + c] * alpha; }
                    tmem_st16(o_addr + hh * 32, lo);
                    tmem_st16(o_addr + hh * 32 + 16, hi);
                }
            }
        }

        // ---- second sweep: exponentials, split into hi (over S in place) and lo ------------------
        float psum = 0.0f;
        if (warp_dead) {
            float z[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) z[c] = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                tmem_st16(s_addr + k * 16, z);
                tmem_st16(plo_addr + k * 16, z);
            }
        } else if (need_mask) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float v[16], lo[16];
                tmem_ld16(s_addr + k * 16, v);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p = (k * 16 + c < nvalid) ? ex2_approx(v[c] - m_ref) : 0.0f;
                    psum += p;
                    v[c] = tf32_hi(p);
                    lo[c] = p - v[c];
                }
                tmem_st16(s_addr + k * 16, v);
                tmem_st16(plo_addr + k * 16, lo);
            }
        } else {
            // the next chunk's load is in flight while this one is computed; four summation chains
            float cur[16], nxt[16];
            float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            tmem_ld16(s_addr, cur);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                tmem_wait_ld();
                if (k + 1 < 4) tmem_ld16(s_addr + (k + 1) * 16, nxt);
                float lo[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p = ex2_approx(cur[c] - m_ref);
                    ps4[c & 3] += p;
                    cur[c] = tf32_hi(p);
                    lo[c] = p - cur[c];
                }
                tmem_st16(s_addr + k * 16, cur);
                tmem_st16(plo_addr + k * 16, lo);
                if (k + 1 < 4) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) cur[c] = nxt[c];
                }
            }
            psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        }
        l += psum;
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[g]);
    }

    if (ntg > 0) {
        wait(&o_done[g], (uint32_t)((ntg - 1) & 1), 3);
        tc_fence_after();
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        float a[32], c2[32];
        tmem_ld32(o_addr, a);                        // P_hi V_hi
        tmem_ld32(o_addr + D, c2);                   // the correction terms
        tmem_wait_ld();
        if (!abort_flag && row < S) {
            float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + row) * (size_t)E + hcol);
#pragma unroll
            for (int c = 0; c < D / 4; ++c)
                dst[c] = make_float4((a[c * 4 + 0] + c2[c * 4 + 0]) * inv, (a[c * 4 + 1] + c2[c * 4 + 1]) * inv,
                                     (a[c * 4 + 2] + c2[c * 4 + 2]) * inv, (a[c * 4 + 3] + c2[c * 4 + 3]) * inv);
        }
    }
    tc_fence_before();
    __syncthreads();
}

template <bool CAUSAL>
int launch_pair_cfg(const float *q, const float *k, const float *v, float *out, int B, int S, int E, int H, cudaStream_t st)
{
    auto kern = mha_tc_pair_kernel<CAUSAL>;
    const size_t smem = kSmemFloats * sizeof(float) + 1024;       // more than half an SM: one block per SM, its 512 TMEM columns always fit
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + 2 * kRows - 1) / (2 * kRows);
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(q, k, v, out, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_tc_pair_kernel");
}

}  // namespace

bool mha_tc_pair_supports(int head_dim) { return head_dim == D; }

int launch_mha_tc_pair(const float *q, const float *k, const float *v, float *out, int B, int S, int E, int H, int causal, cudaStream_t st)
{
    if (!mha_tc_pair_supports(E / H)) return fail(HIPGPT_ERR_UNSUPPORTED, "paired tensor-core kernel: head_dim %d is not 32", E / H);
    if (B == 0 || S == 0) return HIPGPT_OK;
    return causal ? launch_pair_cfg<true>(q, k, v, out, B, S, E, H, st) : launch_pair_cfg<false>(q, k, v, out, B, S, E, H, st);
}

int tc_pair_status_fetch(int *status)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, g_pair_status, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_pair_status, &zero, sizeof(int));
    }
    *status = s;
    return HIPGPT_OK;
}

}  // namespace hipgpt
