// Fused attention forward with bf16 operands on the Blackwell tensor pipe (tcgen05 + TMEM),
// fp32 accumulation, bf16 output.  Same contract as HipGPT's launch_multihead_attention
// (src/hip_kernels.cpp:404-451: three [B*S][E] planes in, one out, head h of token t at
// t*E + h*D), with 16-bit storage; head_dim 64.
//
// One thread block works on 256 query rows of one (batch, head) as two tiles of 128 rows, A and
// B, each owned by one group of 128 worker threads (worker = query row = TMEM lane).  The two
// tiles share every K/V tile and take turns on the tensor core, so one tile's softmax runs
// while the other's products are computed:
//   producers (128 threads)   cp.async K(t), V(t) straight into the 128-byte-swizzled operand
//                             layout (no conversion), two stages each, ring of full/free mbarriers;
//   issuing warp (one lane)   S_x(t) = Q_x K(t)^T (M=128, N=128, 4 x K=16) into TMEM, then, once
//                             the workers have written P_x(t), O_x += P_x(t) V(t) (A operand from
//                             TMEM, 8 x K=16, N=64) directly followed by S_x(t+1);
//   workers                   row maximum and exponentials straight from TMEM (two sweeps, 32
//                             scores in registers at a time), P rounded to bf16 and written over
//                             S in place; the output accumulates in TMEM across all tiles and is
//                             only rescaled when a row's maximum grew by more than 2^8 since the
//                             last rescale (then the whole warp rescales; until then exponentials
//                             may reach 2^8, harmless in bf16 / fp32).
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per tile (two tiles per block)
constexpr int kKeys = 128;        // keys per K/V tile
constexpr int kWorkers = 2 * kRows;
constexpr int kProducers = 128;
constexpr int kThreads = kWorkers + 32 + kProducers;
constexpr float kRescaleStep = 8.0f;     // log2 of the growth of a row maximum that forces a rescale

__device__ int g_bf16_status = 0;

__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, int b_n_major)
{
    // fp32 accumulator, bf16 A and B, A K-major, B K- or N-major
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_n_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// two floats -> one word of two bf16 (round to nearest even), `lo` in the low half
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// TMEM columns: S_A | S_B (128 each, P over the first 64 in place) | O_A | O_B (D each)
template <int D>
struct Bf16Cfg {
    static constexpr uint32_t kColS = 0, kColO = 2 * kKeys;
    static constexpr uint32_t kTmemCols = 512;
    static constexpr int kTileBytes = kKeys * D * 2;            // one Q, K or V tile
    static constexpr size_t kSmemBytes = (size_t)6 * kTileBytes;   // Q_A, Q_B, 2 x K, 2 x V
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kThreads, 1)
mha_bf16_kernel(const __nv_bfloat16 *__restrict__ Q, const __nv_bfloat16 *__restrict__ K, const __nv_bfloat16 *__restrict__ V,
                __nv_bfloat16 *__restrict__ O, int S, int E, int H, int BH, int nqblk, float cscale)
{
    static_assert(D == 64, "rows of the operand tiles are 128 bytes");
    using C = Bf16Cfg<D>;
    constexpr int CPR = D / 8;                       // 16-byte chunks per row
    constexpr int TILE = C::kTileBytes;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = base;                             // [2 tiles][128][D] bf16, row r chunk c at r*128 + ((c ^ (r & 7)) * 16)
    uint8_t *k_s = q_s + 2 * TILE;                   // [2 stages][128 keys][D], the same layout (K-major operand)
    uint8_t *v_s = k_s + 2 * TILE;                   // [2 stages][128 keys][D], the same bytes read as an N-major operand
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
            mbar_init(&k_full[i], kProducers);
            mbar_init(&v_full[i], kProducers);
            mbar_init(&k_free[i], 1);                // tcgen05.commit
            mbar_init(&v_free[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&o_done[i], 1);
            mbar_init(&p_full[i], kRows);            // the workers of one tile
        }
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K staged,
    // 5 P written, 6 V staged, 7 K stage free, 8 V stage free
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) { abort_flag = 1; atomicCAS(&g_bf16_status, 0, site); }
    };
    auto arrive = [&](uint64_t *bar) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };

    if (warp == kWorkers / 32) {
        // ================= the issuing warp =====================================================
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();                             // Q staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (lane == 0) {
            constexpr uint32_t idesc_qk = idesc_bf16(kRows, kKeys, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(kRows, D, 1);
            auto issue_qk = [&](int g, int stage) {
                const uint64_t dq = make_desc(smem_u32(q_s + g * TILE), 16, 1024, 2);
                const uint64_t dk = make_desc(smem_u32(k_s + stage * TILE), 16, 1024, 2);
#pragma unroll
                for (int k = 0; k < D / 16; ++k)         // 16 bf16 = 32 bytes per instruction
                    mma_f16_ss(tmem + C::kColS + g * kKeys, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, k ? 1u : 0u);
                tc_commit(&s_full[g]);
            };
            auto issue_pv = [&](int g, int stage, bool first) {
                // N-major B: 16 keys (two groups of 8 rows of 128 bytes) per instruction = 2048 bytes
                const uint64_t dv = make_desc(smem_u32(v_s + stage * TILE), 1024, 1024, 2);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    mma_f16_ts(tmem + C::kColO + g * D, tmem + C::kColS + g * kKeys + (uint32_t)(k * 8), dv + (uint64_t)(k * 128), idesc_pv,
                               (first && k == 0) ? 0u : 1u);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
        return;
    }

    if (warp > kWorkers / 32) {
        // ================= the producers ========================================================
        const int ptid = tid - kWorkers - 32;
        const int sc = ptid % CPR, sr0 = ptid / CPR;     // chunk of a row, first row
        constexpr int RPP = kProducers / CPR;            // rows per pass
        auto fetch = [&](const __nv_bfloat16 *__restrict__ plane, uint8_t *stage, int t) {
#pragma unroll
            for (int p = 0; p < kKeys / RPP; ++p) {
                const int r = sr0 + p * RPP;
                const int j = t * kKeys + r;
                const bool ok = j < S;
                cp_async16(stage + r * 128 + ((sc ^ (r & 7)) << 4), plane + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + sc * 8, ok);
            }
            cp_async_commit();
        };
        fetch(K, k_s, 0);
        fetch(V, v_s, 0);
        __syncthreads();                             // matches the block-wide barrier after Q staging
        for (int t = 0; t < NT; ++t) {
            const int st = t & 1;
            cp_async_wait<1>();                      // K(t) has landed (V(t) may still be in flight)
            proxy_fence();                           // generic-proxy writes -> visible to the tensor core
            arrive(&k_full[st]);
            if (t + 1 < NT) {
                if (t >= 1) wait(&k_free[st ^ 1], (uint32_t)(((t - 1) >> 1) & 1), 7);   // Q K(t-1)^T has completed
                fetch(K, k_s + (st ^ 1) * TILE, t + 1);
            } else {
                cp_async_commit();                   // keeps the group count of the waits below
            }
            cp_async_wait<1>();                      // V(t) has landed
            proxy_fence();
            arrive(&v_full[st]);
            if (t + 1 < NT) {
                if (t >= 1) wait(&v_free[st ^ 1], (uint32_t)(((t - 1) >> 1) & 1), 8);   // P V(t-1) has completed
                fetch(V, v_s + (st ^ 1) * TILE, t + 1);
            } else {
                cp_async_commit();
            }
        }
        cp_async_wait<0>();
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
        const __nv_bfloat16 *src = Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol;
        uint8_t *dst = q_s + g * TILE + rloc * 128;
#pragma unroll
        for (int c = 0; c < CPR; ++c) cp_async16(dst + ((c ^ (rloc & 7)) << 4), src + c * 8, ok);
        cp_async_commit();
        cp_async_wait<0>();
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t s_addr = lane_base + C::kColS + g * kKeys;
    const uint32_t o_addr = lane_base + C::kColO + g * D;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (scaled, log2 domain) and row sum
    for (int t = 0; t < ntg; ++t) {
        const int j0 = t * kKeys;
        wait(&s_full[g], (uint32_t)(t & 1), 1);      // S_g(t) is in TMEM
        tc_fence_after();
        const bool need_mask = (CAUSAL && j0 + kKeys - 1 > q0 + g * kRows + wq * 32) || j0 + kKeys > S;
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : kKeys);     // visible columns of this row

        // ---- first sweep: the row maximum ----------------------------------------------------
        float mx = -INFINITY;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float v0[32], v1[32];
            tmem_ld32(s_addr + hh * 64, v0);
            tmem_ld32(s_addr + hh * 64 + 32, v1);
            tmem_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v0[c] = (hh * 64 + c < nvalid) ? v0[c] : -INFINITY;
                    v1[c] = (hh * 64 + 32 + c < nvalid) ? v1[c] : -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                m4[(c >> 1) & 1] = fmaxf(m4[(c >> 1) & 1], fmaxf(v0[c], v0[c + 1]));
                m4[2 + ((c >> 1) & 1)] = fmaxf(m4[2 + ((c >> 1) & 1)], fmaxf(v1[c], v1[c + 1]));
            }
            mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        }
        const float mxs = mx * cscale;               // cscale > 0; -inf stays -inf (a row that sees nothing of this tile)
        if (t == 0) {
            m_ref = fmaxf(mxs, -1e30f);
        } else {
            const bool grow = mxs > m_ref + kRescaleStep;
            if (__any_sync(0xffffffffu, grow)) {
                // the accumulator is rescaled by the whole warp (TMEM accesses are warp-wide);
                // rows that did not grow use factor 1
                const float alpha = grow ? ex2_approx(m_ref - mxs) : 1.0f;
                if (grow) m_ref = mxs;
                l *= alpha;
                wait(&o_done[g], (uint32_t)((t - 1) & 1), 2);       // P V_g(t-1) has completed
                tc_fence_after();
#pragma unroll
                for (int hh = 0; hh < D / 32; ++hh) {
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

        // ---- second sweep: exponentials, rounded to bf16, over S in place ------------------------
        float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {
            float cur[32], nxt[32];
            tmem_ld32(s_addr, cur);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                tmem_wait_ld();
                if (k + 1 < 4) tmem_ld32(s_addr + (k + 1) * 32, nxt);
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    float p0 = ex2_approx(fmaf(cur[c], cscale, -m_ref));
                    float p1 = ex2_approx(fmaf(cur[c + 1], cscale, -m_ref));
                    if (need_mask) {
                        p0 = (k * 32 + c < nvalid) ? p0 : 0.0f;
                        p1 = (k * 32 + c + 1 < nvalid) ? p1 : 0.0f;
                    }
                    ps4[(c >> 1) & 3] += p0 + p1;
                    pk[c >> 1] = pack_bf16(p0, p1);
                }
                tmem_st16_u32(s_addr + k * 16, pk);        // columns [16k, 16k+16): all of them read already
                if (k + 1 < 4) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) cur[c] = nxt[c];
                }
            }
        }
        l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[g]);
    }

    if (ntg > 0) {
        wait(&o_done[g], (uint32_t)((ntg - 1) & 1), 3);
        tc_fence_after();
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        const bool store = !abort_flag && row < S;
        uint4 *dst = reinterpret_cast<uint4 *>(O + (tok0 + (row < S ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int hh = 0; hh < D / 32; ++hh) {
            float a[32];
            tmem_ld32(o_addr + hh * 32, a);
            tmem_wait_ld();
            if (store) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    dst[hh * 4 + c] = make_uint4(pack_bf16(a[c * 8 + 0] * inv, a[c * 8 + 1] * inv), pack_bf16(a[c * 8 + 2] * inv, a[c * 8 + 3] * inv),
                                                 pack_bf16(a[c * 8 + 4] * inv, a[c * 8 + 5] * inv), pack_bf16(a[c * 8 + 6] * inv, a[c * 8 + 7] * inv));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
}

template <int D, bool CAUSAL>
int launch_bf16_cfg(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, cudaStream_t st)
{
    using C = Bf16Cfg<D>;
    auto kern = mha_bf16_kernel<D, CAUSAL>;
    // more than half of an SM's shared memory: one block per SM, so its 512 TMEM columns always fit
    size_t smem = C::kSmemBytes + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + 2 * kRows - 1) / (2 * kRows);
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float cscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
                                                    static_cast<const __nv_bfloat16 *>(v), static_cast<__nv_bfloat16 *>(out), S, E, H, B * H,
                                                    nqblk, cscale);
    return check_launch("mha_bf16_kernel");
}

}  // namespace

bool mha_bf16_supports(int D) { return D == 64; }

int launch_mha_bf16(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (!mha_bf16_supports(D)) return fail(HIPGPT_ERR_UNSUPPORTED, "bf16 attention supports head_dim 64, got %d", D);
    if (B == 0 || S == 0) return HIPGPT_OK;
    return causal ? launch_bf16_cfg<64, true>(q, k, v, out, B, S, E, H, st) : launch_bf16_cfg<64, false>(q, k, v, out, B, S, E, H, st);
}

int bf16_status_fetch(int *status)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, g_bf16_status, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_bf16_status, &zero, sizeof(int));
    }
    *status = s;
    return HIPGPT_OK;
}

}  // namespace hipgpt
