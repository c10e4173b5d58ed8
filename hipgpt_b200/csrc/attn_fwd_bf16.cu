// Fused attention forward with bf16 operands on the Blackwell tensor pipe (tcgen05 + TMEM),
// fp32 accumulation, bf16 output.  Same contract as HipGPT's launch_multihead_attention
// (src/hip_kernels.cpp:404-451: three [B*S][E] planes in, one out, head h of token t at
// t*E + h*D), with 16-bit storage; head_dim 64.
//
// One thread block = 128 query rows of one (batch, head): 128 worker threads (worker = query row
// = TMEM lane) and two issuing warps.  Two blocks per SM.  Per tile of 64 keys:
//   copy     one lane asks the TMA unit for the bf16 K / V tile ([64 keys][64 values] = rows of 128 bytes, rank-3
//            maps {E, S, B} over this GPU's own memory, 128-byte swizzle, keys past S arrive as zeros) straight into
//            its operand layout, four stages each; a stage is refilled once the product that read it has completed
//            (the query tile comes the same way, once, as two such boxes);
//   S        = Q K^T (M=128, N=64, 4 instructions of K=16) into one of three TMEM buffers, up to two tiles
//            ahead of the softmax;
//   softmax  the worker reads its 64 scores from TMEM once; maximum, exponentials (scale folded into
//            the exponent, so Q is not rescaled in bf16) and the row sum work on those registers; P is
//            rounded to bf16 and written over S in place (32 columns of packed pairs);
//   O        += P V (A operand from TMEM, 4 instructions of K=16, N=64), accumulated in TMEM over ALL
//            tiles.  The reference maximum is only moved (and O rescaled, by the whole warp) when a
//            row's maximum grew by more than 2^8 since the last rescale; until then exponentials may
//            reach 2^8, harmless in bf16 / fp32.  The worker therefore goes from tile t straight to
//            tile t+1 while P V(t) runs.
// One issuing warp fetches K and issues every Q K^T, the other fetches V and issues every P V (an instruction costs
// its issuer more than it costs the tensor pipe, and two warps issue side by side); both stay converged and elect
// the issuing lane per instruction.  Each accumulator is written by one warp, in tile order.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"
#include "tma_host.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per block
constexpr int kKeys = 64;         // keys per tile
constexpr int kWorkers = kRows;
constexpr int kThreads = kWorkers + 64;  // workers and the two issuing warps
constexpr int kStages = 4;        // K and V tiles in flight
constexpr int kBufs = 3;          // S / P buffers in TMEM
constexpr float kRescaleStep = 8.0f;     // log2 of the growth of a row maximum that forces a rescale
constexpr uint32_t kColX = 0, kColO = kBufs * kKeys, kTmemCols = 256;

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

// (A cubic on the FMA pipe for a share of the exponentials, to relieve the special-function unit, was measured:
// +3 % at S = 1024, -2 % at S = 2048, not kept.)

// The polling part of a bounded wait; on expiry the block's abort flag is raised and the site recorded.
__device__ __noinline__ void bf16_wait_slow(uint64_t *bar, uint32_t parity, int site, volatile int *abort_flag)
{
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicCAS(&g_bf16_status, 0, site);
    }
}

template <int D>
struct Bf16Cfg {
    static constexpr int kQBytes = kRows * D * 2;               // the Q tile
    static constexpr int kTileBytes = kKeys * D * 2;            // one K or V tile
    static constexpr size_t kSmemBytes = (size_t)kQBytes + 2 * kStages * kTileBytes;
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kThreads, 2)
mha_bf16_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                __nv_bfloat16 *__restrict__ O, int S, int E, int H, int BH, int nqblk, float cscale)
{
    static_assert(D == 64, "rows of the operand tiles are 128 bytes");
    using C = Bf16Cfg<D>;
    constexpr int TILE = C::kTileBytes;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = base;                             // [128][D] bf16, row r chunk c at r*128 + ((c ^ (r & 7)) * 16)
    uint8_t *k_s = q_s + C::kQBytes;                 // [stage][64 keys][D], the same layout (K-major operand)
    uint8_t *v_s = k_s + kStages * TILE;             // [stage][64 keys][D], the same bytes read as an N-major operand
    __shared__ uint64_t k_full[kStages], v_full[kStages], s_full[kStages], o_done[kStages], p_full[kBufs], q_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31;
    // read from one lane, so that the compiler knows the warp's number (and every role that follows from it) to be warp-uniform
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);     // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * kRows;
    const int kend = CAUSAL ? min(S, q0 + kRows) : S;
    const int nt = (kend + kKeys - 1) / kKeys;       // >= 1: q0 < S

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&k_full[i], 1);                // the copy of a tile: one announcement, then its bytes
            mbar_init(&v_full[i], 1);
            mbar_init(&s_full[i], 1);                // tcgen05.commit after Q K(t)^T, t mod 4 = i: S is ready, and the K stage is free
            mbar_init(&o_done[i], 1);                // tcgen05.commit after P V(t): O is up to date, and the V stage is free
        }
        for (int i = 0; i < kBufs; ++i) mbar_init(&p_full[i], kWorkers / 32);    // one arrival per worker warp
        mbar_init(&q_full, 1);
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K tile landed,
    // 5 P written, 6 V tile landed, 7 K stage free, 8 V stage free, 9 Q tile landed
    // (the polling loop exists once, out of line: an already completed phase costs one test)
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag || mbar_test(bar, parity)) return;
        bf16_wait_slow(bar, parity, site, &abort_flag);
    };
    // one arrival for the whole warp: every lane's writes are ordered before it by the warp barrier
    auto arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };
    // phase parity of tile t on a barrier that is indexed by tile mod n
    auto phn = [](int t, int n) { return (uint32_t)((t / n) & 1); };

    if (warp >= kWorkers / 32) {
        // ================= the two issuing warps =================================================
        const bool qk_role = warp == kWorkers / 32;
        if (qk_role) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        auto copy_tile = [&](const CUtensorMap *map, uint8_t *ring, uint64_t *full, int u) {
            if (lane == 0 && u < nt) {
                mbar_arrive_expect_tx(&full[u % kStages], (uint32_t)TILE);
                tma_load_3d(ring + (u % kStages) * TILE, map, (int)hcol, u * kKeys, b, &full[u % kStages]);
            }
            __syncwarp();
        };
        // Up to here the block ran beside the tail of the kernel before it on the stream (overlapped launch); its first
        // read of global memory waits for that kernel, and the kernel after this one may bring its blocks in.
        dependents_may_start();
        dependency_wait();
        // the query tile: two boxes of 64 rows (rows past S come as zeros); no thread touches it
        if (qk_role && lane == 0) {
            mbar_arrive_expect_tx(&q_full, (uint32_t)C::kQBytes);
            tma_load_3d(q_s, &qmap, (int)hcol, q0, b, &q_full);
            tma_load_3d(q_s + TILE, &qmap, (int)hcol, q0 + kKeys, b, &q_full);
        }
        __syncwarp();
        for (int u = 0; u < kStages; ++u) {
            if (qk_role) copy_tile(&kmap, k_s, k_full, u);
            else copy_tile(&vmap, v_s, v_full, u);
        }
        tc_fence_before();
        __syncthreads();                             // TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (qk_role) {
            constexpr uint32_t idesc_qk = idesc_bf16(kRows, kKeys, 0);
            const uint64_t dq = make_desc(smem_u32(q_s), 16, 1024, 2);
            auto issue_qk = [&](int t) {
                const uint64_t dk = make_desc(smem_u32(k_s + (t % kStages) * TILE), 16, 1024, 2);
#pragma unroll
                for (int k = 0; k < D / 16; ++k)         // 16 bf16 = 32 bytes per instruction
                    if (elect_one()) mma_f16_ss(tmem + kColX + (t % kBufs) * kKeys, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, k ? 1u : 0u);
                if (elect_one()) tc_commit(&s_full[t % kStages]);    // S is ready, and this K stage may be refilled
            };
            wait(&q_full, 0, 9);
            wait(&k_full[0], 0, 4);
            tc_fence_after();
            issue_qk(0);
            for (int t = 0; t + 1 < nt; ++t) {
                wait(&k_full[(t + 1) % kStages], phn(t + 1, kStages), 4);        // K(t+1) is in its stage
                // the buffer of S(t+1) held P(t-2): with three buffers the product runs up to two tiles ahead of the
                // exponentials and never waits for the P V product before it
                if (t >= 2) wait(&o_done[(t - 2) % kStages], phn(t - 2, kStages), 2);
                tc_fence_after();
                issue_qk(t + 1);
                // Q K(t)^T was issued a whole step ago: it has completed, or does so before the product above
                wait(&s_full[t % kStages], phn(t, kStages), 7);
                copy_tile(&kmap, k_s, k_full, t + kStages);
            }
        } else {
            constexpr uint32_t idesc_pv = idesc_bf16(kRows, D, 1);
            for (int t = 0; t < nt; ++t) {
                wait(&p_full[t % kBufs], phn(t, kBufs), 5);                      // P(t) is in TMEM
                wait(&v_full[t % kStages], phn(t, kStages), 6);                  // V(t) is in its stage
                tc_fence_after();
                // N-major B: 16 keys (two groups of 8 rows of 128 bytes) per instruction = 2048 bytes
                const uint64_t dv = make_desc(smem_u32(v_s + (t % kStages) * TILE), 1024, 1024, 2);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    if (elect_one()) mma_f16_ts(tmem + kColO, tmem + kColX + (t % kBufs) * kKeys + (uint32_t)(k * 8), dv + (uint64_t)(k * 128), idesc_pv,
                                                (t == 0 && k == 0) ? 0u : 1u);
                if (elect_one()) tc_commit(&o_done[t % kStages]);    // O is up to date; this V stage may be refilled, Q K^T may take the buffer
                // P V(t-1) was issued a whole step ago: its stage takes V(t-1+4)
                if (t >= 1) {
                    wait(&o_done[(t - 1) % kStages], phn(t - 1, kStages), 8);
                    copy_tile(&vmap, v_s, v_full, t - 1 + kStages);
                }
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read the output
        if (qk_role) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        return;
    }

    // ===================== the workers ===========================================================
    const int wq = warp;                             // TMEM lane quadrant of this warp
    const int rloc = wq * 32 + lane;                 // row inside the block = TMEM lane
    const int row = q0 + rloc;
    tc_fence_before();
    __syncthreads();                                 // TMEM allocated
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (scaled, log2 domain) and row sum
    for (int t = 0; t < nt; ++t) {
        const int buf = t % kBufs;
        const int j0 = t * kKeys;
        const uint32_t s_addr = lane_base + kColX + buf * kKeys;
        wait(&s_full[t % kStages], phn(t, kStages), 1);    // S(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + wq * 32;              // first row of this warp
        const bool warp_dead = CAUSAL && j0 > wrow0 + 31;          // these columns are above the diagonal for the whole warp
        const bool need_mask = (CAUSAL && j0 + kKeys - 1 > wrow0) || j0 + kKeys > S;
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : kKeys);     // visible columns of this row

        // ---- the worker's scores are read from TMEM once and stay in registers --------------------
        float v0[32], v1[32];
        float mx = -INFINITY;
        if (!warp_dead) {
            tmem_ld32(s_addr, v0);
            tmem_ld32(s_addr + 32, v1);
            tmem_wait_ld();
            if (need_mask) {
                // a masked score becomes -inf: its exponential below is exactly 0
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v0[c] = (c < nvalid) ? v0[c] : -INFINITY;
                    v1[c] = (32 + c < nvalid) ? v1[c] : -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                m4[(c >> 1) & 1] = max3(m4[(c >> 1) & 1], v0[c], v0[c + 1]);
                m4[2 + ((c >> 1) & 1)] = max3(m4[2 + ((c >> 1) & 1)], v1[c], v1[c + 1]);
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
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
                wait(&o_done[(t - 1) % kStages], phn(t - 1, kStages), 2);        // P V(t-1) has completed
                tc_fence_after();
#pragma unroll
                for (int hh = 0; hh < D / 16; ++hh) {
                    float a[16];
                    tmem_ld16(o_addr + hh * 16, a);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) a[c] *= alpha;
                    tmem_st16(o_addr + hh * 16, a);
                }
            }
        }

        // ---- exponentials, rounded to bf16, over S in place --------------------------------------------
        float2 ps2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};      // four summation chains, two per instruction
        const float2 cs2 = make_float2(cscale, cscale), nm2 = make_float2(-m_ref, -m_ref);
        if (warp_dead) {
            uint32_t zz[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) zz[c] = 0u;
            tmem_st16_u32(s_addr, zz);
            tmem_st16_u32(s_addr + 16, zz);
        } else {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float2 x = ffma2(make_float2(k ? v1[c] : v0[c], k ? v1[c + 1] : v0[c + 1]), cs2, nm2);
                    const float2 pp = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                    ps2[(c >> 1) & 1] = fadd2(ps2[(c >> 1) & 1], pp);
                    pk[c >> 1] = pack_bf16(pp.x, pp.y);
                }
                tmem_st16_u32(s_addr + k * 16, pk);   // packed pairs: 16 columns per 32 keys; every score they overwrite is in registers
            }
        }
        l += (ps2[0].x + ps2[0].y) + (ps2[1].x + ps2[1].y);
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[buf]);
    }

    {
        wait(&o_done[(nt - 1) % kStages], phn(nt - 1, kStages), 3);
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

// Rank-3 map {E, S, B} over one [B*S][E] bf16 plane; a box is [1][64 keys][64 values] = rows of 128 bytes, 128-byte swizzled.
int bf16_plane_map(CUtensorMap *m, const void *plane, int B, int S, int E)
{
    EncodeTiledFn enc = tma_encode_fn();
    if (!enc) return fail(HIPGPT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[3] = {(cuuint64_t)E, (cuuint64_t)S, (cuuint64_t)B};
    const cuuint64_t strides[2] = {(cuuint64_t)E * 2, (cuuint64_t)S * E * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)kKeys, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(plane), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HIPGPT_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return HIPGPT_OK;
}

template <int D, bool CAUSAL>
int launch_bf16_cfg(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, cudaStream_t st)
{
    using C = Bf16Cfg<D>;
    auto kern = mha_bf16_kernel<D, CAUSAL>;
    // at least 100 KB: at most two blocks share an SM, so their 256-column TMEM allocations always fit in the 512 columns
    size_t smem = C::kSmemBytes + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kRows - 1) / kRows;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return fail(HIPGPT_ERR_BAD_ARG, "bf16 attention needs 16-byte aligned planes");
    CUtensorMap qmap, kmap, vmap;
    int rc = bf16_plane_map(&qmap, q, B, S, E);
    if (rc == HIPGPT_OK) rc = bf16_plane_map(&kmap, k, B, S, E);
    if (rc == HIPGPT_OK) rc = bf16_plane_map(&vmap, v, B, S, E);
    if (rc != HIPGPT_OK) return rc;
    const float cscale = (1.0f / sqrtf((float)D)) * kLog2e;
    const cudaError_t le = launch_overlapped(kern, dim3((unsigned)blocks), dim3(kThreads), smem, st, qmap, kmap, vmap, static_cast<__nv_bfloat16 *>(out), S, E, H, B * H,
                                             nqblk, cscale);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "mha_bf16_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("mha_bf16_kernel");
}

}  // namespace

bool mha_bf16_supports(int D) { return D == 64; }

// `variant` selected between schedules of earlier versions; there is one schedule now and the argument is only range-checked.
int launch_mha_bf16(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, int causal, cudaStream_t st, int variant)
{
    const int D = E / H;
    if (!mha_bf16_supports(D)) return fail(HIPGPT_ERR_UNSUPPORTED, "bf16 attention supports head_dim 64, got %d", D);
    if (variant < 0 || variant > 2) return fail(HIPGPT_ERR_BAD_ARG, "bf16 attention: unknown variant %d", variant);
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
