// Fused attention forward with bf16 operands on the Blackwell tensor pipe (tcgen05 + TMEM),
// fp32 accumulation, bf16 output.  Same contract as HipGPT's launch_multihead_attention
// (src/hip_kernels.cpp:404-451: three [B*S][E] planes in, one out, head h of token t at
// t*E + h*D), with 16-bit storage; head_dim 64.
//
// One thread block = 128 query rows of one (batch, head): 128 worker threads (worker = query row
// = TMEM lane), one warp whose elected lane issues the tensor-core instructions, one warp that
// copies K tiles and one that copies V tiles.  Two blocks per SM.  Per tile of 64 keys:
//   copy     cp.async brings the bf16 K / V tile straight into its 128-byte-swizzled operand
//            layout (no conversion), four stages each; a stage is free again when the product that read
//            it has completed (the S-ready barrier for K, the O-done barrier for V);
//   S        = Q K^T (M=128, N=64, 4 instructions of K=16) into one of two TMEM buffers, issued one
//            tile ahead of the softmax;
//   softmax  the worker reads its 64 scores from TMEM once; maximum, exponentials (scale folded into
//            the exponent, so Q is not rescaled in bf16) and the row sum work on those registers; P is
//            rounded to bf16 and written over S in place (32 columns of packed pairs);
//   O        += P V (A operand from TMEM, 4 instructions of K=16, N=64), accumulated in TMEM over ALL
//            tiles.  The reference maximum is only moved (and O rescaled, by the whole warp) when a
//            row's maximum grew by more than 2^8 since the last rescale; until then exponentials may
//            reach 2^8, harmless in bf16 / fp32.  The worker therefore goes from tile t straight to
//            tile t+1 while P V(t) runs.
// The template also holds two schedules that were measured slower and are kept selectable: two workers
// per row (WPR = 2), and tiles of 128 keys with one S / P buffer (KEYS = 128).
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per block
// WPR = workers per query row: 1 (a worker owns the 64 scores of its row) or 2 (two workers, in warps w and
// w + 4 that share a TMEM lane quadrant, own 32 scores each and exchange the row maximum through shared
// memory once per tile): twice the warps to hide the latencies of the softmax behind.
template <int WPR> __host__ __device__ constexpr int workers_of() { return kRows * WPR; }
template <int WPR> __host__ __device__ constexpr int threads_of() { return workers_of<WPR>() + 32 + 64; }     // workers, the issuing warp, the K warp, the V warp
constexpr int kDefaultWorkersPerRow = 1;
constexpr float kRescaleStep = 8.0f;     // log2 of the growth of a row maximum that forces a rescale
constexpr uint32_t kColX = 0, kColO = 128, kTmemCols = 256;

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

// KEYS = keys per tile: 64 (two S / P buffers in TMEM, Q K^T one tile ahead of the softmax, four stages of K and
// V) or 128 (one S / P buffer of 128 columns, two stages; Q K^T with N = 128 costs the tensor pipe what N = 64
// costs, so a tile of twice the keys takes 14 instead of 20 tensor-core operations)
template <int D, int KEYS>
struct Bf16Cfg {
    static constexpr int kStages = KEYS == 64 ? 4 : 2;          // K and V tiles in flight
    static constexpr int kQBytes = kRows * D * 2;               // the Q tile
    static constexpr int kTileBytes = KEYS * D * 2;             // one K or V tile
    static constexpr size_t kSmemBytes = (size_t)kQBytes + 2 * kStages * kTileBytes;
};

template <int D, bool CAUSAL, int WPR, int KEYS>
__global__ void __launch_bounds__(threads_of<WPR>(), 2)
mha_bf16_kernel(const __nv_bfloat16 *__restrict__ Q, const __nv_bfloat16 *__restrict__ K, const __nv_bfloat16 *__restrict__ V,
                __nv_bfloat16 *__restrict__ O, int S, int E, int H, int BH, int nqblk, float cscale)
{
    static_assert(D == 64, "rows of the operand tiles are 128 bytes");
    static_assert(WPR == 1 || WPR == 2, "one or two workers per row");
    constexpr int kWorkers = workers_of<WPR>();
    static_assert(KEYS == 64 || (KEYS == 128 && WPR == 2), "128-key tiles need two workers per row");
    constexpr int kKeys = KEYS, kStages = Bf16Cfg<D, KEYS>::kStages;
    constexpr int CW = kKeys / WPR;                  // score columns per worker and tile: 64 or 32
    constexpr bool TWO = CW == 64;                   // a worker holds two arrays of 32 scores
    constexpr int XB = KEYS == 64 ? 2 : 1;           // S / P buffers in TMEM
    using C = Bf16Cfg<D, KEYS>;
    constexpr int CPR = D / 8;                       // 16-byte chunks per row
    constexpr int TILE = C::kTileBytes;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = base;                             // [128][D] bf16, row r chunk c at r*128 + ((c ^ (r & 7)) * 16)
    uint8_t *k_s = q_s + C::kQBytes;                 // [stage][64 keys][D], the same layout (K-major operand)
    uint8_t *v_s = k_s + kStages * TILE;             // [stage][64 keys][D], the same bytes read as an N-major operand
    __shared__ uint64_t k_full[kStages], v_full[kStages], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float xch[2][2][kRows];               // WPR == 2: row maxima of the two halves, by tile parity
    __shared__ float lx[2][kRows];                   // WPR == 2: row sums of the two halves

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
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&k_full[i], 1);                // the K warp
            mbar_init(&v_full[i], 1);                // the V warp
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], kWorkers / 32);    // one arrival per worker warp
            mbar_init(&o_done[i], 1);                // by tile parity: a worker may be two tiles ahead of the P V products
        }
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K staged,
    // 5 P written, 6 V staged, 7 K stage free, 8 V stage free
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) { abort_flag = 1; atomicCAS(&g_bf16_status, 0, site); }
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
        // The warp stays converged and elects the issuing lane per instruction: descriptors are then computed
        // warp-uniformly (uniform registers), which roughly halves what an instruction costs its issuer.
        {
            constexpr uint32_t idesc_qk = idesc_bf16(kRows, kKeys, 0);
            constexpr uint32_t idesc_pv = idesc_bf16(kRows, D, 1);
            const uint64_t dq = make_desc(smem_u32(q_s), 16, 1024, 2);
            auto issue_qk = [&](int buf, int stage) {
                const uint64_t dk = make_desc(smem_u32(k_s + stage * TILE), 16, 1024, 2);
#pragma unroll
                for (int k = 0; k < D / 16; ++k)         // 16 bf16 = 32 bytes per instruction
                    if (elect_one()) mma_f16_ss(tmem + kColX + (XB == 2 ? buf * kKeys : 0), dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, k ? 1u : 0u);
                if (elect_one()) tc_commit(&s_full[buf]);             // S is ready; it also tells the K warp that this product no longer reads its stage
            };
            auto issue_pv = [&](int buf, int stage, bool first) {
                // N-major B: 16 keys (two groups of 8 rows of 128 bytes) per instruction = 2048 bytes
                const uint64_t dv = make_desc(smem_u32(v_s + stage * TILE), 1024, 1024, 2);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    if (elect_one()) mma_f16_ts(tmem + kColO, tmem + kColX + (XB == 2 ? buf * kKeys : 0) + (uint32_t)(k * 8), dv + (uint64_t)(k * 128), idesc_pv,
                               (first && k == 0) ? 0u : 1u);
                if (elect_one()) tc_commit(&o_done[buf]);             // O is up to date; it also tells the V warp that this product no longer reads its stage
            };
            wait(&k_full[0], 0, 4);
            tc_fence_after();
            issue_qk(0, 0);
            for (int t = 0; t < nt; ++t) {
                const int buf = t & 1;               // barrier slot of tile t (and its S / P buffer when there are two)
                if (XB == 2 && t + 1 < nt) {
                    wait(&k_full[(t + 1) % kStages], (uint32_t)(((t + 1) / kStages) & 1), 4);    // K(t+1) is in shared memory
                    tc_fence_after();
                    issue_qk(buf ^ 1, (t + 1) % kStages);    // its buffer held P(t-1): P V(t-1) was issued before, instructions run in order
                }
                wait(&p_full[buf], (uint32_t)((t >> 1) & 1), 5);                         // P(t) is in TMEM
                wait(&v_full[t % kStages], (uint32_t)((t / kStages) & 1), 6);            // V(t) is in shared memory
                tc_fence_after();
                issue_pv(buf, t % kStages, t == 0);
                if (XB == 1 && t + 1 < nt) {
                    // one buffer: S(t+1) overwrites P(t), which the product just issued reads first (instructions run in order)
                    wait(&k_full[(t + 1) % kStages], (uint32_t)(((t + 1) / kStages) & 1), 4);
                    tc_fence_after();
                    issue_qk(buf ^ 1, (t + 1) % kStages);
                }
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read the output
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
        return;
    }

    if (warp > kWorkers / 32) {
        // ================= the K warp and the V warp ==============================================
        // Tile u goes to stage u mod 4; its copy is issued three tiles ahead, as soon as the product
        // that read the stage's previous tile has completed.
        const bool is_v = warp == kWorkers / 32 + 2;
        const __nv_bfloat16 *__restrict__ plane = is_v ? V : K;
        uint8_t *ring = is_v ? v_s : k_s;
        uint64_t *full = is_v ? v_full : k_full;
        uint64_t *done = is_v ? o_done : s_full;     // completion of the product that read a stage, by tile parity
        const int sc = lane % CPR, sr0 = lane / CPR;     // chunk of a row, first row
        constexpr int RPP = 32 / CPR;                    // rows per pass
        auto copy = [&](int u) {
            if (u < nt) {
                uint8_t *stage = ring + (u % kStages) * TILE;
#pragma unroll
                for (int p = 0; p < kKeys / RPP; ++p) {
                    const int r = sr0 + p * RPP;
                    const int j = u * kKeys + r;
                    const bool ok = j < S;
                    cp_async16(stage + r * 128 + ((sc ^ (r & 7)) << 4), plane + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + sc * 8, ok);
                }
            }
            cp_async_commit();                       // an empty group keeps the count of the waits
        };
#pragma unroll
        for (int u = 0; u < kStages - 1; ++u) copy(u);
        __syncthreads();                             // matches the block-wide barrier after Q staging
        for (int u = 0; u < nt; ++u) {
            // tile u is published first: the wait for a free stage below ends only when a product two tiles
            // back has completed, and the consumer of tile u must not stand behind that
            cp_async_wait<kStages - 2>();            // the copies of tiles u+1, u+2 may be in flight: tile u has landed
            proxy_fence();                           // generic-proxy writes -> visible to the tensor core
            arrive(&full[u % kStages]);
            const int w = u + kStages - 1;           // the tile whose copy is issued now
            // stage w mod 4 held tile w - 4 = u - 1: free once Q K(u-1)^T (for V: P V(u-1)) has completed.  A commit
            // costs the issuing lane about as much as a tensor-core instruction, so the stages have no barriers of
            // their own; the later product on the same barrier, u + 1, cannot complete before tile u + 1 is published
            if (w < nt && w >= kStages) wait(&done[(u - 1) & 1], (uint32_t)(((u - 1) >> 1) & 1), is_v ? 8 : 7);
            copy(w);
        }
        cp_async_wait<0>();
        __syncthreads();
        return;
    }

    // ===================== the workers ===========================================================
    const int wq = warp & 3;                         // TMEM lane quadrant of this warp
    const int half = warp >> 2;                      // which CW columns of a tile this worker owns (0 when WPR == 1)
    const int rloc = wq * 32 + lane;                 // row inside the block = TMEM lane
    const int row = q0 + rloc;
    // the two workers of a row meet at a named barrier of their two warps
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory"); };
    {
        const bool ok = row < S;
        const __nv_bfloat16 *src = Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol;
        uint8_t *dst = q_s + rloc * 128;
#pragma unroll
        for (int c = half * (CPR / WPR); c < (half + 1) * (CPR / WPR); ++c) cp_async16(dst + ((c ^ (rloc & 7)) << 4), src + c * 8, ok);
        cp_async_commit();
        cp_async_wait<0>();
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (scaled, log2 domain) and row sum
    for (int t = 0; t < nt; ++t) {
        const int buf = t & 1;
        const int j0 = t * kKeys;
        const uint32_t s_addr = lane_base + kColX + (XB == 2 ? buf * kKeys : 0);
        wait(&s_full[buf], (uint32_t)((t >> 1) & 1), 1);   // S(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + wq * 32;              // first row of this warp
        const bool warp_dead = CAUSAL && j0 > wrow0 + 31;          // these columns are above the diagonal for the whole warp (both halves)
        const bool need_mask = (CAUSAL && j0 + kKeys - 1 > wrow0) || j0 + kKeys > S;
        // visible columns of this row among this worker's CW columns
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : kKeys) - half * CW;

        // ---- the worker's scores are read from TMEM once and stay in registers --------------------
        float v0[32], v1[32];                    // v1: the worker's columns 32..63, used when it owns 64
        float mx = -INFINITY;
        if (!warp_dead) {
            tmem_ld32(s_addr + half * CW, v0);
            if (TWO) tmem_ld32(s_addr + half * CW + 32, v1);
            tmem_wait_ld();
            if (need_mask) {
                // a masked score becomes -inf: its exponential below is exactly 0
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v0[c] = (c < nvalid) ? v0[c] : -INFINITY;
                    if (TWO) v1[c] = (32 + c < nvalid) ? v1[c] : -INFINITY;
                }
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                m4[(c >> 1) & 1] = fmaxf(m4[(c >> 1) & 1], fmaxf(v0[c], v0[c + 1]));
                if (TWO) m4[2 + ((c >> 1) & 1)] = fmaxf(m4[2 + ((c >> 1) & 1)], fmaxf(v1[c], v1[c + 1]));
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            if (WPR == 2) {
                // the row maximum over both halves; the partner has read its scores when it arrives,
                // so P may be written over S afterwards
                xch[t & 1][half][rloc] = mx;
                pair_sync();
                mx = fmaxf(mx, xch[t & 1][half ^ 1][rloc]);
            }
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
                wait(&o_done[(t - 1) & 1], (uint32_t)(((t - 1) >> 1) & 1), 2);   // P V(t-1) has completed
                tc_fence_after();
#pragma unroll
                for (int hh = half * (D / 16 / WPR); hh < (half + 1) * (D / 16 / WPR); ++hh) {
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
        float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};    // four summation chains
        if (warp_dead) {
            uint32_t zz[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) zz[c] = 0u;
            tmem_st16_u32(s_addr + half * (CW / 2), zz);
            if (TWO) tmem_st16_u32(s_addr + half * (CW / 2) + 16, zz);
        } else {
#pragma unroll
            for (int k = 0; k < CW / 32; ++k) {
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float s0 = (TWO && k) ? v1[c] : v0[c], s1 = (TWO && k) ? v1[c + 1] : v0[c + 1];
                    const float p0 = ex2_approx(fmaf(s0, cscale, -m_ref));
                    const float p1 = ex2_approx(fmaf(s1, cscale, -m_ref));
                    ps4[(c >> 1) & 3] += p0 + p1;
                    pk[c >> 1] = pack_bf16(p0, p1);
                }
                tmem_st16_u32(s_addr + half * (CW / 2) + k * 16, pk);   // packed pairs: 16 columns per 32 keys; every score they overwrite is in registers
            }
        }
        l += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[buf]);
    }

    {
        wait(&o_done[(nt - 1) & 1], (uint32_t)(((nt - 1) >> 1) & 1), 3);
        tc_fence_after();
        if (WPR == 2) {
            lx[half][rloc] = l;
            pair_sync();
            l += lx[half ^ 1][rloc];
        }
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        const bool store = !abort_flag && row < S;
        uint4 *dst = reinterpret_cast<uint4 *>(O + (tok0 + (row < S ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int hh = half * (D / 32 / WPR); hh < (half + 1) * (D / 32 / WPR); ++hh) {
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

template <int D, bool CAUSAL, int WPR, int KEYS>
int launch_bf16_cfg(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, cudaStream_t st)
{
    using C = Bf16Cfg<D, KEYS>;
    auto kern = mha_bf16_kernel<D, CAUSAL, WPR, KEYS>;
    // at least 100 KB: at most two blocks share an SM, so their 256-column TMEM allocations always fit in the 512 columns
    size_t smem = C::kSmemBytes + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kRows - 1) / kRows;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float cscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, threads_of<WPR>(), smem, st>>>(static_cast<const __nv_bfloat16 *>(q), static_cast<const __nv_bfloat16 *>(k),
                                                    static_cast<const __nv_bfloat16 *>(v), static_cast<__nv_bfloat16 *>(out), S, E, H, B * H,
                                                    nqblk, cscale);
    return check_launch("mha_bf16_kernel");
}

}  // namespace

bool mha_bf16_supports(int D) { return D == 64; }

// variant: 0 = default, 1 = one worker per query row, 2 = two workers per query row
int launch_mha_bf16(const void *q, const void *k, const void *v, void *out, int B, int S, int E, int H, int causal, cudaStream_t st, int variant)
{
    const int D = E / H;
    if (!mha_bf16_supports(D)) return fail(HIPGPT_ERR_UNSUPPORTED, "bf16 attention supports head_dim 64, got %d", D);
    if (variant < 0 || variant > 2) return fail(HIPGPT_ERR_BAD_ARG, "bf16 attention: unknown variant %d", variant);
    if (B == 0 || S == 0) return HIPGPT_OK;
    if (variant == 0) variant = kDefaultWorkersPerRow;
    if (variant == 2)
        return causal ? launch_bf16_cfg<64, true, 2, 64>(q, k, v, out, B, S, E, H, st) : launch_bf16_cfg<64, false, 2, 64>(q, k, v, out, B, S, E, H, st);
    return causal ? launch_bf16_cfg<64, true, 1, 64>(q, k, v, out, B, S, E, H, st) : launch_bf16_cfg<64, false, 1, 64>(q, k, v, out, B, S, E, H, st);
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
