// Fused attention forward for the shape HipGPT's default model runs (head_dim 32, up to 256 tokens):
// one thread block owns a whole (batch, head), so K and V are fetched and converted once for both
// query tiles, every score tile of the head sits in tensor memory at the same time (no online
// rescaling: a row's true maximum is known before its exponentials are taken), and a block that
// has more than one head to do fetches the next head's operands while it finishes the current one.
//
// Replaces flash_attention_kernel<32> behind launch_multihead_attention for S <= 256
// (HipGPT src/hip_kernels.cpp:263-325, dispatch :404-451); same arithmetic contract as the other
// fp32-grade kernels here: results within 1e-5 of the scalar fp32 arithmetic on unit-scale data.
//
// Data movement: Q, K and V tiles of [128 rows][32 floats] arrive by TMA (cp.async.bulk.tensor, rank-3
// maps {E, S, B} over this GPU's own memory, 128-byte swizzle, rows past S filled with zeros, no
// multicast), six copies per head issued by one lane, completion counted on mbarriers.
//
// Products (tcgen05.mma, M = 128, accumulators in TMEM, issued by one lane):
//   S = Q K^T, N = 128 keys:  the landed fp32 tiles ARE the TF32 operands (the tensor core ignores the
//       13 low mantissa bits): 4 kind::tf32 instructions; the correction terms Q_lo K_hi + Q K_lo
//       run as 4 kind::f16 instructions on fp16 copies [Q_lo | Q] x [K_hi | K_lo] concatenated along
//       the reduction dimension.  8 instructions per 128 x 128 score tile.
//   O = P V:  P = 2^(s c - m c + 8) is cut into fp16 P_hi (11 bits, exact) and P_lo, V (scaled by a
//       power of two per head so that its largest magnitude sits near 2^14) into fp16 V_hi and V_lo:
//       P_hi [V_hi | V_lo] (N = 64) and P_lo V_hi (N = 32, added to the second half), A operand from
//       TMEM, 16 instructions per 128 keys.  The dropped P_lo V_lo is below 2^-22 relative.
// TMEM (512 columns): three score/probability buffers of 128 columns (P_hi and P_lo overwrite S in
// place as packed fp16), two output accumulators of 64 columns (one per query tile).
// Tiles of a head: causal (q0,k0) (q1,k0) (q1,k1); unmasked (q0,k0) (q0,k1) (q1,k0) (q1,k1), the fourth
// reusing the first buffer once its P V product has been issued.
// Threads: three groups of 128 workers (thread = query row = TMEM lane) and three issuing warps.  A group
// first converts one operand (K, Q or V) for the whole head, then owns one score tile (two for group 0
// of an unmasked head): row maximum, exchange of the maximum with the group that holds the other key
// tile of the same rows (shared memory + mbarrier), exponentials, P to TMEM; at the end the groups of a
// query tile share its output columns.  One issuing warp issues the copies and every Q K^T, the other two the
// P V products of one query tile each, in a fixed order, so results do not depend on timing.
// Probabilities (when asked for): a row's sum is known once all its tiles have been through the exponentials;
// the workers then read P_hi + P_lo back from TMEM, divide by the sum and store [B][H][S][S]: no second Q K^T.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short, records a
// site code for hipgpt_kernel_status, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"
#include "tma_host.cuh"

#include <cuda_fp16.h>
#include <math.h>

namespace hipgpt {
namespace {

constexpr int kTile = 128;                       // rows of a query tile = keys of a key tile
constexpr int kHeadWorkers = 3 * kTile;
constexpr int kHeadIssuers = 3;                  // warps that issue copies and tensor-core instructions
constexpr int kHeadThreads = kHeadWorkers + 32 * kHeadIssuers;
constexpr uint32_t kTileBytes = kTile * 128;     // one [128][128 byte] operand block
constexpr uint32_t kOffQraw = 0, kOffKraw = 2 * kTileBytes, kOffVraw = 4 * kTileBytes;
constexpr uint32_t kOffQ16 = 6 * kTileBytes, kOffK16 = 8 * kTileBytes, kOffV16 = 10 * kTileBytes;
constexpr uint32_t kHeadSmemBytes = 12 * kTileBytes;
constexpr uint32_t kColO = 384;                  // after three buffers of 128 columns
constexpr float kPShift = 8.0f;                  // P carries a factor 2^8: small probabilities stay normal fp16 numbers
constexpr long long kHeadCycleLimit = 1LL << 28; // per wait, about 0.14 s
constexpr long long kHeadPollLimit = 1LL << 22;

__device__ int g_head_status = 0;                // first wait site that ran out (0 = none)
__device__ int g_head_notice = 0;                // bit 0: Q or K left the range in which the fp16 correction terms are exact

// The polling part of a bounded wait; on expiry the block's abort flag is raised and the site recorded.
__device__ __noinline__ void head_wait_slow(uint64_t *bar, uint32_t parity, int site, volatile int *abort_flag)
{
    if (!mbar_wait_for(bar, parity, kHeadCycleLimit, kHeadPollLimit)) {
        *abort_flag = 1;
        atomicCAS(&g_head_status, 0, site);
    }
}

// Largest score of one 32-column chunk; columns from `nvalid` on (counted from the tile's first column) are hidden.
__device__ __forceinline__ float chunk_max(float (&v)[32], int col0, int nvalid, bool need_mask)
{
    if (need_mask) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (col0 + j < nvalid) ? v[j] : -INFINITY;
    }
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
        m4[0] = max3(m4[0], v[j], v[j + 1]); m4[1] = max3(m4[1], v[j + 2], v[j + 3]);
        m4[2] = max3(m4[2], v[j + 4], v[j + 5]); m4[3] = max3(m4[3], v[j + 6], v[j + 7]);
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// One chunk of scores -> P = 2^(s c + nmc), cut into fp16 hi and lo, written over the chunk's own 32 TMEM
// columns (16 of packed P_hi, then 16 of packed P_lo).  Returns the sum of P.
__device__ __forceinline__ float chunk_exp(float (&v)[32], uint32_t addr, int col0, int nvalid, bool need_mask, float cscale, float nmc)
{
    if (need_mask) {
        // a hidden score becomes -inf: its exponential is exactly 0
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (col0 + j < nvalid) ? v[j] : -INFINITY;
    }
    // pairs of values per instruction where the hardware has one (multiply-add, add)
    float2 ps[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
    const float2 cs2 = make_float2(cscale, cscale), nm2 = make_float2(nmc, nmc);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float2 x = ffma2(make_float2(v[16 * half + j], v[16 * half + j + 1]), cs2, nm2);
            const float2 p = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            ps[(j >> 1) & 1] = fadd2(ps[(j >> 1) & 1], p);
            const float2 h = make_float2(tf32_hi(p.x), tf32_hi(p.y));            // 11 leading bits: exact in fp16
            const float2 l = fadd2(p, make_float2(-h.x, -h.y));
            hi[j >> 1] = pack_f16(h.x, h.y);
            lo[j >> 1] = pack_f16(l.x, l.y);
        }
        tmem_st8_u32(addr + 8 * half, hi);
        tmem_st8_u32(addr + 16 + 8 * half, lo);
    }
    return (ps[0].x + ps[0].y) + (ps[1].x + ps[1].y);
}

__device__ __forceinline__ void chunk_zero(uint32_t addr)
{
    uint32_t z[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) z[j] = 0u;
    tmem_st16_u32(addr, z);
    tmem_st16_u32(addr + 16, z);
}

struct HeadMaps {
    CUtensorMap q, k, v;
    CUtensorMap q32;                             // Q in boxes of 32 rows (a causal head's first query tile, below)
};

template <bool CAUSAL, bool PROBS>
__global__ void __launch_bounds__(kHeadThreads, 1)
mha_head_kernel(const __grid_constant__ HeadMaps maps, float *__restrict__ O, float *__restrict__ P, int S, int E, int H, int BH, float cscale)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_raw = base + kOffQraw, *k_raw = base + kOffKraw, *v_raw = base + kOffVraw;
    uint8_t *q_16 = base + kOffQ16;              // per query tile: rows of [Q_lo (32) | Q (32)] fp16, K-major, 128-byte swizzle
    uint8_t *k_16 = base + kOffK16;              // per key tile:   rows of [K_hi (32) | K_lo (32)]
    uint8_t *v_16 = base + kOffV16;              // [V_hi | V_lo] (64 columns) fp16, N-major without swizzle: 8 keys x 8 columns
                                                 // form one 128-byte core matrix, column blocks 128 bytes apart, key groups 1024
    __shared__ uint64_t ld_q[2], ld_k[2], ld_v[2], cv_q[2], cv_k[2], cv_v[2];
    __shared__ uint64_t s_full[3], p_full[4], o_done[2], xm[2], xs[2], epi_done, vx, pr_done, b0_free;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float xmax[2][2][2][kTile];       // [head parity][query tile][slot][row]
    __shared__ float xsum[2][2][2][kTile];
    __shared__ float vmaxw[2][4];                // [head parity][warp of the V group]
    __shared__ float s_vinv[2];                  // 1 / (V's power-of-two scale), by head parity
    __shared__ unsigned s_amax[2];               // bit patterns of max |Q| and max |K| of the current head

    const int tid = threadIdx.x, lane = tid & 31;
    // the warp's number, read from one lane so that the compiler knows it (and the role, tile and buffer numbers
    // that follow from it) to be the same for the whole warp: descriptors then live in uniform registers
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int nq = S > kTile ? 2 : 1;            // query tiles = key tiles of a head
    // A causal head of two tiles has two diagonal score tiles, (q0, k0) and (q1, k1), where a warp's work grows with its
    // rows: the warp of TMEM lanes 96-127 sweeps four 32-column chunks, that of lanes 0-31 one.  A warp's number fixes
    // both its lanes and its scheduler (warp mod 4), so one scheduler would get 4 + 4 + 4 chunks of exponentials per
    // head and another 1 + 4 + 1.  The first query tile's rows are therefore kept in TMEM lanes with the four groups of
    // 32 in reverse order (tile row r in lanes of group 3 - r / 32): the copies place them so, and every place that
    // turns a lane of that tile into a row (mask, output row, probabilities) turns it back.  9 chunks per scheduler.
    const bool flip0 = CAUSAL && nq == 2;

    // site codes: 1 Q/K/V landed, 2 operand converted, 3 S ready, 4 P written, 5 output complete,
    // 6 row maxima exchanged, 7 row sums exchanged, 8 previous head's output read, 9 V maximum exchanged,
    // 10 probabilities of the first tile read back, 11 first product of an unmasked head complete
    // (the kernel's instructions are fetched cold by every SM, so the code is kept small: the polling loop of a
    // wait exists once, out of line, behind a one-instruction test that is all an already completed phase costs)
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag || mbar_test(bar, parity)) return;
        head_wait_slow(bar, parity, site, &abort_flag);
    };
    auto arrive = [&](uint64_t *bar) {           // one arrival per warp, after every lane's writes
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };

    if (warp >= kHeadWorkers / 32) {
        // ================= the three issuing warps =====================================================
        // role 0: the copies and every Q K^T; role 1: the P V products of query tile 0; role 2: those of query
        // tile 1.  A tcgen05.mma costs the thread that issues it far more than it costs the tensor pipe (measured:
        // about 100 cycles per instruction from one lane of a diverged warp, 55 - 85 from a converged warp that
        // elects the lane per instruction, and two warps issue side by side at that rate each), so the warps stay
        // converged, compute the descriptors warp-uniformly and share the head's 72 - 96 instructions between them.
        // Instructions of one thread run in order; between the warps the order is made by mbarriers, and each
        // accumulator is written by one warp only, in a fixed order: results do not depend on timing.
        const int role = warp - kHeadWorkers / 32;
        auto load_qk = [&](int hd) {
            if (lane == 0) {
                const int b = hd / H, c0 = (hd % H) * 32;
                for (int t = 0; t < nq; ++t) {
                    mbar_arrive_expect_tx(&ld_k[t], kTileBytes);
                    tma_load_3d(k_raw + t * kTileBytes, &maps.k, c0, t * kTile, b, &ld_k[t]);
                    mbar_arrive_expect_tx(&ld_q[t], kTileBytes);
                    if (t == 0 && flip0) {
                        for (int g = 0; g < 4; ++g)
                            tma_load_3d(q_raw + (3 - g) * (32 * 128), &maps.q32, c0, g * 32, b, &ld_q[0]);
                    } else {
                        tma_load_3d(q_raw + t * kTileBytes, &maps.q, c0, t * kTile, b, &ld_q[t]);
                    }
                }
            }
            __syncwarp();
        };
        auto load_v = [&](int hd) {
            if (lane == 0) {
                const int b = hd / H, c0 = (hd % H) * 32;
                for (int t = 0; t < nq; ++t) {
                    mbar_arrive_expect_tx(&ld_v[t], kTileBytes);
                    tma_load_3d(v_raw + t * kTileBytes, &maps.v, c0, t * kTile, b, &ld_v[t]);
                }
            }
            __syncwarp();
        };
        if (role == 0) {
            if (lane == 0) {
                abort_flag = 0;
                s_amax[0] = s_amax[1] = 0u;
                for (int i = 0; i < 2; ++i) {
                    mbar_init(&ld_q[i], 1); mbar_init(&ld_k[i], 1); mbar_init(&ld_v[i], 1);
                    mbar_init(&cv_q[i], 4); mbar_init(&cv_k[i], 4); mbar_init(&cv_v[i], 4);
                    mbar_init(&o_done[i], 1);
                    mbar_init(&xm[i], 8); mbar_init(&xs[i], 8);
                }
                for (int i = 0; i < 3; ++i) mbar_init(&s_full[i], 1);
                for (int i = 0; i < 4; ++i) mbar_init(&p_full[i], 4);
                mbar_init(&epi_done, kHeadWorkers / 32);
                mbar_init(&vx, 4);
                mbar_init(&pr_done, 4);
                mbar_init(&b0_free, 1);
            }
            __syncwarp();
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
            // Everything above ran beside the tail of the kernel before this one on the stream; the first read of global
            // memory waits for it.  The kernel after this one may bring its blocks in as soon as this grid's SMs free up.
            // The first head's tiles are asked into L2 before the wait (a prefetch reads nothing into the SM; L2 is
            // where the other kernel's writes land too, so it cannot go stale): all SMs ask for their operands in the
            // same microsecond after the wait, and that burst then hits L2 instead of HBM.
            if (lane == 0 && (int)blockIdx.x < BH) {
                const int b = (int)blockIdx.x / H, c0 = ((int)blockIdx.x % H) * 32;
                for (int t = 0; t < nq; ++t) {
                    tma_prefetch_3d(&maps.k, c0, t * kTile, b);
                    tma_prefetch_3d(&maps.q, c0, t * kTile, b);
                }
                for (int t = 0; t < nq; ++t) tma_prefetch_3d(&maps.v, c0, t * kTile, b);
            }
            __syncwarp();
            dependents_may_start();
            dependency_wait();
            if ((int)blockIdx.x < BH) { load_qk(blockIdx.x); load_v(blockIdx.x); }
        }
        tc_fence_before();
        __syncthreads();                             // barriers initialised, TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (role == 0) {
            constexpr uint32_t id_qk_h = idesc_f16(kTile, kTile);             // [Q_lo | Q] x [K_hi | K_lo], fp16
            constexpr uint32_t id_qk_t = make_idesc(kTile, kTile, 0);         // Q x K, tf32
            auto issue_qk = [&](int q, int k, int buf) {
                const uint32_t d = tmem + (uint32_t)(buf * kTile);
                const uint64_t dq16 = make_desc(smem_u32(q_16 + q * kTileBytes), 16, 1024, 2);
                const uint64_t dk16 = make_desc(smem_u32(k_16 + k * kTileBytes), 16, 1024, 2);
                // the correction terms first: the accumulator is still tiny while they are added
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)       // 16 fp16 = 32 bytes per instruction
                    if (elect_one()) mma_h_ss(d, dq16 + (uint64_t)(ks * 2), dk16 + (uint64_t)(ks * 2), id_qk_h, ks ? 1u : 0u);
                const uint64_t dq = make_desc(smem_u32(q_raw + q * kTileBytes), 16, 1024, 2);
                const uint64_t dk = make_desc(smem_u32(k_raw + k * kTileBytes), 16, 1024, 2);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)       // 8 floats = 32 bytes per instruction
                    if (elect_one()) mma_ss(d, dq + (uint64_t)(ks * 2), dk + (uint64_t)(ks * 2), id_qk_t, 1u);
                if (elect_one()) tc_commit(&s_full[buf]);
            };
            const int nfirst = nq == 1 ? 1 : 3;      // tiles whose buffers are free at the start of a head
            int it = 0;
#pragma unroll 1
            for (int hd = blockIdx.x; hd < BH; hd += gridDim.x, ++it) {
                const uint32_t par = (uint32_t)(it & 1), ppar = (uint32_t)((it - 1) & 1);
                const int next = hd + (int)gridDim.x;
                const bool has_next = next < BH;
                // ---- Q K^T of every tile whose buffer is free ---------------------------------------
                // (with the probabilities stored, the workers read P back from these buffers until their output is out,
                // and stage them in the Q and K areas of shared memory, so this head's Q and K are fetched only now)
                if (PROBS && it > 0) {
                    wait(&epi_done, ppar, 8);
                    load_qk(hd);
                }
                // tile t: causal (q0,k0) (q1,k0) (q1,k1), unmasked (q0,k0) (q0,k1) (q1,k0), into buffer t.  A buffer still
                // holds the previous head's P until the P V products that read it have completed: the first buffer is
                // read by query tile 0 only in a causal head, every other case waits for both accumulators.
#pragma unroll 1
                for (int t = 0; t < nfirst; ++t) {
                    const int q = CAUSAL ? (t > 0) : (t >> 1), k = CAUSAL ? (t > 1) : (t & 1);
                    if (it > 0) {
                        if (t == 0) wait(&o_done[0], ppar, 5);
                        if (nq == 2 && t == (CAUSAL ? 1 : 0)) wait(&o_done[1], ppar, 5);
                    }
                    wait(&cv_k[k], par, 2);
                    wait(&cv_q[q], par, 2);
                    tc_fence_after();
                    issue_qk(q, k, t);
                    // The next head's tiles are asked into L2 now: this head's operands have landed, so the memory system is
                    // idle, and the copies that fetch them once this head's Q K^T products have completed (all SMs within the
                    // same microsecond again) then hit L2.
                    if (CAUSAL && t == 0 && has_next && !PROBS && lane == 0) {
                        const int nb = next / H, nc0 = (next % H) * 32;
                        for (int u = 0; u < nq; ++u) {
                            tma_prefetch_3d(&maps.k, nc0, u * kTile, nb);
                            tma_prefetch_3d(&maps.q, nc0, u * kTile, nb);
                        }
                        for (int u = 0; u < nq; ++u) tma_prefetch_3d(&maps.v, nc0, u * kTile, nb);
                    }
                    __syncwarp();
                }
                // ---- the operands' range (see g_head_notice) ------------------------------------------
                if (lane == 0) {
                    const float aq = __uint_as_float(s_amax[0]), ak = __uint_as_float(s_amax[1]);
                    s_amax[0] = 0u;
                    s_amax[1] = 0u;
                    // beyond fp16's largest number the correction terms saturate; below its smallest normal
                    // numbers they are flushed, an absolute error of up to 2^-25 per fp16 value, which matters
                    // when it is neither small in itself nor small beside the scores it is added to
                    const bool over = !(aq <= 65504.0f) || !(ak <= 65504.0f);
                    const float flush = 32.0f * cscale * 2.98e-8f * (aq + ak);
                    if (over || (flush > 3.8e-6f && (aq + ak) > 8.0f * aq * ak)) atomicOr(&g_head_notice, 1);
                }
                __syncwarp();
                const bool tail_qk = !CAUSAL && nq == 2;    // the fourth tile's Q K^T comes after the first P V product
                if (has_next && !tail_qk && !PROBS) {
                    // the raw Q and K tiles and their fp16 copies are free once every Q K^T has completed
                    wait(&s_full[0], par, 3);
                    if (nq == 2) { wait(&s_full[1], par, 3); wait(&s_full[2], par, 3); }
                    load_qk(next);
                }
                wait(&cv_v[0], par, 2);
                if (nq == 2) wait(&cv_v[1], par, 2);
                if (has_next) load_v(next);              // the raw V tiles have been read
                if (tail_qk) {
                    // (q1, k1) into the first buffer, once the product that reads (q0, k0)'s P from it has completed;
                    // with the probabilities stored its workers must also have read that P back
                    wait(&b0_free, par, 11);
                    if (PROBS) wait(&pr_done, par, 10);
                    tc_fence_after();
                    issue_qk(1, 1, 0);
                    if (has_next && !PROBS) {
                        wait(&s_full[0], 1u, 3);         // second completion of this barrier in this head
                        wait(&s_full[1], par, 3);
                        wait(&s_full[2], par, 3);
                        load_qk(next);
                    }
                }
            }
        } else if (role - 1 < nq) {
            // ---- P V of one query tile, in a fixed order ----------------------------------------------
            const int q = role - 1;
            constexpr uint32_t id_pv_a = idesc_f16(kTile, 64) | (1u << 16);   // P_hi x [V_hi | V_lo], B N-major
            constexpr uint32_t id_pv_b = idesc_f16(kTile, 32) | (1u << 16);   // P_lo x V_hi
            // the tiles of this query tile in the order of their products, packed: bit 0 key tile, 1-2 buffer, 3-4 p_full barrier
            auto pk = [](int k, int buf, int ptile) { return (uint32_t)(k | (buf << 1) | (ptile << 3)); };
            const uint32_t pj0 = (nq == 1 || q == 0) ? pk(0, 0, 0) : CAUSAL ? pk(1, 2, 2) : pk(0, 2, 2);
            const uint32_t pj1 = q == 0 ? pk(1, 1, 1) : CAUSAL ? pk(0, 1, 1) : pk(1, 0, 3);
            const int npv = (nq == 1 || (CAUSAL && q == 0)) ? 1 : 2;
            const uint32_t d = tmem + kColO + (uint32_t)(q * 64);
            int it = 0;
#pragma unroll 1
            for (int hd = blockIdx.x; hd < BH; hd += gridDim.x, ++it) {
                const uint32_t par = (uint32_t)(it & 1);
                if (it > 0) wait(&epi_done, (uint32_t)((it - 1) & 1), 8);     // the previous head's output has left TMEM
#pragma unroll 1
                for (int j = 0; j < npv; ++j) {
                    const uint32_t pj = j ? pj1 : pj0;
                    const int k = pj & 1, buf = (pj >> 1) & 3, ptile = (pj >> 3) & 3;
                    wait(&cv_v[k], par, 2);
                    wait(&p_full[ptile], par, 4);
                    tc_fence_after();
                    // keys 32c .. 32c+31 of the tile: P_hi in columns [32c, 32c+16) of the buffer, P_lo in [32c+16, 32c+32)
                    const uint32_t a0 = tmem + (uint32_t)(buf * kTile);
                    const uint64_t dv = make_desc(smem_u32(v_16 + k * kTileBytes), 1024, 128, 0);
                    const int nks = (min(kTile, S - k * kTile) + 15) >> 4;        // 16 keys per instruction; keys past S hold zeros
                    // (unrolled: a rolled loop's address arithmetic between the instructions was measured to double their cost)
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)       // 16 keys = 8 TMEM columns of packed fp16 = two key groups of V
                        if (ks < nks && elect_one()) mma_h_ts(d, a0 + (uint32_t)(32 * (ks >> 1) + 8 * (ks & 1)), dv + (uint64_t)(ks * 128), id_pv_a, (j == 0 && ks == 0) ? 0u : 1u);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        if (ks < nks && elect_one()) mma_h_ts(d + 32, a0 + (uint32_t)(32 * (ks >> 1) + 8 * (ks & 1) + 16), dv + (uint64_t)(ks * 128), id_pv_b, 1u);
                    // an unmasked head's fourth score tile goes into the first buffer once this product has read it
                    if (!CAUSAL && nq == 2 && q == 0 && j == 0 && elect_one()) tc_commit(&b0_free);
                }
                if (elect_one()) tc_commit(&o_done[q]);
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read their last output
        if (role == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
        return;
    }

    // ===================== the workers ===============================================================
    const int grp = warp >> 2;                       // 0: converts K, 1: converts Q, 2: converts V
    const int wq = warp & 3;                         // TMEM lane quadrant of this warp
    const int rloc = wq * 32 + lane;                 // row inside a tile = TMEM lane
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);

    // The score tiles this group owns, packed: bit 0 query tile, 1 key tile, 2-3 S/P buffer, 4-5 index of the
    // p_full barrier, 6 slot in the exchange with the group that holds the other key tile of the same rows,
    // 7 whether there is such a group, 8-9 parity of s_full[buffer] (0: the head's parity, 1: always 0, 2: always 1).
    auto mk = [](int q, int k, int buf, int ptile, int slot, int paired, int sp) {
        return (uint32_t)(q | (k << 1) | (buf << 2) | (ptile << 4) | (slot << 6) | (paired << 7) | (sp << 8));
    };
    uint32_t job0 = 0, job1 = 0;
    int njobs = 0;
    if (nq == 1) {
        if (grp == 0) { job0 = mk(0, 0, 0, 0, 0, 0, 0); njobs = 1; }
    } else if (CAUSAL) {
        njobs = 1;
        job0 = grp == 0 ? mk(0, 0, 0, 0, 0, 0, 0) : grp == 1 ? mk(1, 0, 1, 1, 0, 1, 0) : mk(1, 1, 2, 2, 1, 1, 0);
    } else {
        // s_full[0] completes twice per head here: first for (q0, k0), then for (q1, k1)
        njobs = grp == 0 ? 2 : 1;
        job0 = grp == 0 ? mk(0, 0, 0, 0, 0, 1, 1) : grp == 1 ? mk(0, 1, 1, 1, 1, 1, 0) : mk(1, 0, 2, 2, 0, 1, 0);
        job1 = mk(1, 1, 0, 3, 1, 1, 2);
    }

    // ---- conversion of K (group 0) or Q (group 1) for the head this block takes `itn`-th: thread = one row of each tile ----
    auto convert_kq = [&](int itn) {
        const uint32_t parn = (uint32_t)(itn & 1);
        // K: [K_hi | K_lo];  Q: [Q_lo | Q].  hi = the 11 leading bits (exact in fp16), lo = x - hi.
        uint8_t *raw = grp == 0 ? k_raw : q_raw, *dst16 = grp == 0 ? k_16 : q_16;
        uint64_t *ld = grp == 0 ? ld_k : ld_q, *cv = grp == 0 ? cv_k : cv_q;
        float amax = 0.0f;
        for (int t = 0; t < nq; ++t) {
            wait(&ld[t], parn, 1);
            const uint8_t *src = raw + t * kTileBytes;
            uint8_t *dst = dst16 + t * kTileBytes;
            float4 x[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) x[c] = *reinterpret_cast<const float4 *>(src + sw128(rloc, c));
#pragma unroll
            for (int pc = 0; pc < 4; ++pc) {
                const float4 a = x[2 * pc], c4 = x[2 * pc + 1];
                const float4 ah = hi4(a), ch = hi4(c4);
                amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                                         fmaxf(fmaxf(fabsf(c4.x), fabsf(c4.y)), fmaxf(fabsf(c4.z), fabsf(c4.w)))));
                const uint4 lo = make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                                            pack_f16(c4.x - ch.x, c4.y - ch.y), pack_f16(c4.z - ch.z, c4.w - ch.w));
                if (grp == 0) {
                    *reinterpret_cast<uint4 *>(dst + sw128(rloc, pc)) =
                        make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
                    *reinterpret_cast<uint4 *>(dst + sw128(rloc, 4 + pc)) = lo;
                } else {
                    *reinterpret_cast<uint4 *>(dst + sw128(rloc, pc)) = lo;
                    *reinterpret_cast<uint4 *>(dst + sw128(rloc, 4 + pc)) =
                        make_uint4(pack_f16(a.x, a.y), pack_f16(a.z, a.w), pack_f16(c4.x, c4.y), pack_f16(c4.z, c4.w));
                }
            }
            if (t == nq - 1) {
                // a NaN compares false everywhere: its bit pattern is what reaches the range test
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (lane == 0) atomicMax(&s_amax[grp == 0 ? 1 : 0], __float_as_uint(amax));
            }
            proxy_fence();                       // generic-proxy writes -> visible to the tensor core
            arrive(&cv[t]);
        }
    };
    if (grp < 2 && (int)blockIdx.x < BH) convert_kq(0);

    int it = 0;
    float v_sc = 1.0f;                               // group 2: V's scale for the head about to be converted,
    bool v_scale_known = false;                      // ... when it was found during the head before
    for (int hd = blockIdx.x; hd < BH; hd += gridDim.x, ++it) {
        const uint32_t par = (uint32_t)(it & 1);
        const int b = hd / H, h = hd % H;

        // ---- conversion of V (group 2): scaled by a power of two so that the head's largest magnitude lies in
        // [2^14, 2^15), then [V_hi | V_lo], before the group turns to its score tile.  (Placed between the
        // group's two sweeps it ran beside the other groups' exponentials and took longer: measured slower.)
        // K and Q of this head were converted before the loop (first head) or behind the previous head's
        // exponentials.
        // The power of two for the head this block takes `itn`-th, from the largest magnitude of its raw V tiles (a
        // sweep over them and an exchange between the group's four warps).  It needs the raw tiles only, so for every
        // head but the first it runs early: behind the group's exponentials of the head before, while that head's P V
        // products still read the fp16 copy.  What then stands between two heads is the conversion alone.
        auto v_scale = [&](int itn) {
            const uint32_t parn = (uint32_t)(itn & 1);
            float amax = 0.0f;
            for (int t = 0; t < nq; ++t) {
                wait(&ld_v[t], parn, 1);
                const uint8_t *src = v_raw + t * kTileBytes;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 x = *reinterpret_cast<const float4 *>(src + sw128(rloc, c));
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w))));
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) vmaxw[parn][wq] = amax;
            arrive(&vx);
            wait(&vx, parn, 9);
            const float vm = fmaxf(fmaxf(vmaxw[parn][0], vmaxw[parn][1]), fmaxf(vmaxw[parn][2], vmaxw[parn][3]));
            float sc = 1.0f, inv = 1.0f;
            if (vm > 0.0f && vm <= 3.0e38f) {
                const int e = (int)((__float_as_uint(vm) >> 23) & 0xffu) - 127;
                const int sh = min(14 - e, 126);
                sc = __uint_as_float((uint32_t)(127 + sh) << 23);
                inv = __uint_as_float((uint32_t)(127 - sh) << 23);
            }
            if (tid == 2 * kTile) s_vinv[parn] = inv;
            return sc;
        };
        auto convert_v = [&](float sc) {
            // V: scaled, then [V_hi | V_lo].  The previous head's P V products must have completed before V16 is overwritten.
            if (it > 0) {
                wait(&o_done[0], (uint32_t)((it - 1) & 1), 5);
                if (nq == 2) wait(&o_done[1], (uint32_t)((it - 1) & 1), 5);
            }
            for (int t = 0; t < nq; ++t) {
                const int key = t * kTile + rloc;
                const uint8_t *src = v_raw + t * kTileBytes;
                uint8_t *dst = v_16 + (key >> 3) * 1024 + (key & 7) * 16;
#pragma unroll
                for (int pc = 0; pc < 4; ++pc) {
                    float4 a = *reinterpret_cast<const float4 *>(src + sw128(rloc, 2 * pc));
                    float4 c4 = *reinterpret_cast<const float4 *>(src + sw128(rloc, 2 * pc + 1));
                    a.x *= sc; a.y *= sc; a.z *= sc; a.w *= sc;
                    c4.x *= sc; c4.y *= sc; c4.z *= sc; c4.w *= sc;
                    const float4 ah = hi4(a), ch = hi4(c4);
                    *reinterpret_cast<uint4 *>(dst + pc * 128) =
                        make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
                    *reinterpret_cast<uint4 *>(dst + (4 + pc) * 128) =
                        make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                                   pack_f16(c4.x - ch.x, c4.y - ch.y), pack_f16(c4.z - ch.z, c4.w - ch.w));
                }
                proxy_fence();
                arrive(&cv_v[t]);
            }
        
        };
        // (Letting the conversion wait until the group has swept its score tile for the row maxima, so that the group at
        // the other end of the exchange is not held up by it, measured slower: 15.42 against 15.30 us.)
        if (grp == 2) {
            if (!v_scale_known) v_sc = v_scale(it);
            v_scale_known = false;
            convert_v(v_sc);
        }

        // ---- score tiles of this group --------------------------------------------------------------------
        // Per tile: row maximum (first sweep over the tile's columns in TMEM), exchange of the maximum with
        // the group that holds the other key tile of the same rows, exponentials (second sweep), P_hi and
        // P_lo over S in place.  Chunk c = score columns [32c, 32c+32): its P_hi (packed fp16) goes to
        // columns [32c, 32c+16), its P_lo to [32c+16, 32c+32), so a chunk is rewritten where it was read.
        // The probabilities of one tile, normalised: P_hi + P_lo read back from TMEM, divided by the row's sum over all
        // of its tiles (P carries a factor 2^8, and so does the sum).  A worker holds a row, so its own stores would be
        // 16-byte pieces S floats apart; the warp turns each 32 x 32 chunk through shared memory instead and stores four
        // rows of 128 contiguous bytes per instruction.  The scratch is the first tile of the raw Q (group 0), of the fp16
        // Q (group 1) or of the raw K (group 2): free once the products that read them have completed, which the caller
        // has made sure of.  Chunks that no row of the warp sees are zeros.
        auto store_probs = [&](uint32_t job, float l_total) {
            const int q = job & 1, k = (job >> 1) & 1, buf = (job >> 2) & 3;
            const uint32_t s_addr = lane_base + (uint32_t)(buf * kTile);
            const int ncols = min(kTile, S - k * kTile);
            const bool diag = CAUSAL && q == k;
            const int eq = (flip0 && q == 0) ? 3 - wq : wq;     // the group of 32 rows of the tile that this warp's lanes hold
            const int nwarp = diag ? min(ncols, eq * 32 + 32) : ncols;
            const int nch = (nwarp + 31) >> 5;
            const int wrow0 = q * kTile + eq * 32;              // first row of this warp
            const float inv = 1.0f / fmaxf(l_total, 1e-20f);
            uint8_t *tb = (grp == 0 ? q_raw : grp == 1 ? q_16 : k_raw) + wq * 4096;   // [32 rows][128 bytes], 16-byte chunks swizzled by the row
            float *pw = P + ((size_t)hd * S + wrow0) * (size_t)S + (size_t)k * kTile;
            const bool vec = (S & 3) == 0;                      // then every group of four columns is 16-byte aligned
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int nleft = ncols - c * 32;               // columns of this chunk that exist
                if (nleft <= 0) break;
                if (c < nch) {
                    float w[32];
                    tmem_ld32(s_addr + c * 32, w);              // 16 words of packed P_hi, then 16 of packed P_lo
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float o[4];
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const __half2 hh = *reinterpret_cast<const __half2 *>(&w[2 * j + i]), ll = *reinterpret_cast<const __half2 *>(&w[16 + 2 * j + i]);
                            o[2 * i] = (__low2float(hh) + __low2float(ll)) * inv;
                            o[2 * i + 1] = (__high2float(hh) + __high2float(ll)) * inv;
                        }
                        *reinterpret_cast<float4 *>(tb + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4 *>(tb + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                __syncwarp();
                if (!abort_flag) {
                    if (vec) {
                        const int ch = lane & 7;                // 16-byte piece of a row
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = 4 * i + (lane >> 3);
                            const float4 val = *reinterpret_cast<const float4 *>(tb + rr * 128 + ((ch ^ (rr & 7)) << 4));
                            if (wrow0 + rr < S && 4 * ch < nleft) *reinterpret_cast<float4 *>(pw + (size_t)rr * S + c * 32 + 4 * ch) = val;
                        }
                    } else {
                        for (int rr = 0; rr < 32 && wrow0 + rr < S; ++rr)
                            if (lane < nleft)
                                pw[(size_t)rr * S + c * 32 + lane] = *reinterpret_cast<const float *>(tb + rr * 128 + (((lane >> 2) ^ (rr & 7)) << 4) + (lane & 3) * 4);
                    }
                }
                __syncwarp();                                   // the chunk is out before the next one is staged
            }
            // a causal head's first query tile has no second key tile: those columns are zeros
            if (CAUSAL && q == 0 && k == 0 && !abort_flag)
                for (int rr = 0; rr < 32 && wrow0 + rr < S; ++rr) {
                    float *pr = P + ((size_t)hd * S + wrow0 + rr) * (size_t)S;
                    if (vec) for (int col = kTile + 4 * lane; col < S; col += 128) *reinterpret_cast<float4 *>(pr + col) = make_float4(0.f, 0.f, 0.f, 0.f);
                    else for (int col = kTile + lane; col < S; col += 32) pr[col] = 0.0f;
                }
        };
        float lsum[2] = {0.0f, 0.0f};
#pragma unroll 1
        for (int ji = 0; ji < njobs; ++ji) {
            const uint32_t job = ji ? job1 : job0;
            const int q = job & 1, k = (job >> 1) & 1, buf = (job >> 2) & 3, ptile = (job >> 4) & 3, slot = (job >> 6) & 1;
            const bool paired = (job >> 7) & 1;
            const uint32_t spar = ((job >> 8) & 3) == 0 ? par : ((job >> 8) & 3) - 1;   // parity of s_full[buf] for this tile
            const uint32_t s_addr = lane_base + (uint32_t)(buf * kTile);
            const int ncols = min(kTile, S - k * kTile);                      // keys of this tile that exist
            const bool diag = CAUSAL && q == k;
            const int eq = (flip0 && q == 0) ? 3 - wq : wq;                   // the group of 32 rows of the tile that this warp's lanes hold
            const int nvalid = diag ? min(ncols, eq * 32 + lane + 1) : ncols; // keys this row sees
            const int nwarp = diag ? min(ncols, eq * 32 + 32) : ncols;        // ... the warp's last row sees
            const int nmin = diag ? min(ncols, eq * 32 + 1) : ncols;          // ... its first row sees
            const int nch = (nwarp + 31) >> 5;                                // 32-column chunks with any visible key
            wait(&s_full[buf], spar, 3);
            tc_fence_after();
            // One chunk of 32 columns at a time, one copy of the code per sweep: the loads' latency is covered by
            // the SM's other warps, and the instruction footprint matters more than the overlap inside a warp.
            float mx = -INFINITY;
            float v[32];
#pragma unroll 1
            for (int c = 0; c < nch; ++c) {
                tmem_ld32(s_addr + c * 32, v);
                tmem_wait_ld();
                mx = fmaxf(mx, chunk_max(v, c * 32, nvalid, c * 32 + 32 > nmin));
            }
            if (paired) {
                xmax[par][q][slot][rloc] = mx;
                arrive(&xm[q]);
                wait(&xm[q], par, 6);
                mx = fmaxf(mx, xmax[par][q][slot ^ 1][rloc]);
            }
            mx = fmaxf(mx, -1e30f);
            const float nmc = kPShift - mx * cscale;     // p = 2^(s c - m c + 8)
            float ps = 0.0f;
#pragma unroll 1
            for (int c = 0; c < nch; ++c) {
                tmem_ld32(s_addr + c * 32, v);
                tmem_wait_ld();
                ps += chunk_exp(v, s_addr + c * 32, c * 32, nvalid, c * 32 + 32 > nmin, cscale, nmc);
            }
#pragma unroll 1
            for (int c = nch; c < 4; ++c) chunk_zero(s_addr + c * 32);       // chunks that no row of this warp sees
            tmem_wait_st();
            tc_fence_before();
            arrive(&p_full[ptile]);
            if (paired) {
                xsum[par][q][slot][rloc] = ps;
                arrive(&xs[q]);
            }
            if (ji) lsum[1] = ps; else lsum[0] = ps;
            if (PROBS && !CAUSAL && njobs == 2 && ji == 0) {
                // this tile's buffer is taken by the group's second tile: its probabilities leave now
                wait(&xs[q], par, 7);
                store_probs(job, ps + xsum[par][q][slot ^ 1][rloc]);
                tc_fence_before();
                arrive(&pr_done);
            }
        }
        // the next head's K and Q have landed by now (their copies were issued when this head's Q K^T had
        // completed): converting them here lets its Q K^T run while this head's output is stored
        if (!PROBS && grp < 2 && hd + (int)gridDim.x < BH) convert_kq(it + 1);
        if (!PROBS && grp == 2 && hd + (int)gridDim.x < BH) {
            v_sc = v_scale(it + 1);                  // the next head's raw V has landed (its copies were issued when this head's V had been converted)
            v_scale_known = true;
        }
        // ---- output: (P_hi V_hi + corrections) / (l * V's scale); the groups of a query tile share its columns ----
#pragma unroll 1
        for (int ji = 0; ji < njobs; ++ji) {
            const uint32_t job = ji ? job1 : job0;
            const int q = job & 1, slot = (job >> 6) & 1;
            const bool paired = (job >> 7) & 1;
            const int c0 = paired ? 16 * slot : 0, nc = paired ? 16 : 32;
            float l = ji ? lsum[1] : lsum[0];
            if (paired) {
                wait(&xs[q], par, 7);
                l += xsum[par][q][slot ^ 1][rloc];
            }
            wait(&o_done[q], par, 5);                    // every product of this head issued so far has completed
            tc_fence_after();
            if (PROBS && !(!CAUSAL && njobs == 2 && ji == 0)) store_probs(job, l);
            const float inv = (1.0f / fmaxf(l, 1e-20f)) * s_vinv[par];
            const int row = q * kTile + ((flip0 && q == 0) ? 3 - wq : wq) * 32 + lane;
            const bool store = !abort_flag && row < S;
            float4 *dst = reinterpret_cast<float4 *>(O + ((size_t)b * S + (row < S ? row : 0)) * (size_t)E + (size_t)h * 32);
            const uint32_t o_addr = lane_base + kColO + (uint32_t)(q * 64);
#pragma unroll 1
            for (int cc = c0; cc < c0 + nc; cc += 16) {
                float a[16], c2[16];
                tmem_ld16(o_addr + cc, a);
                tmem_ld16(o_addr + 32 + cc, c2);
                tmem_wait_ld();
                if (store) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        dst[(cc >> 2) + j] = make_float4((a[4 * j] + c2[4 * j]) * inv, (a[4 * j + 1] + c2[4 * j + 1]) * inv,
                                                         (a[4 * j + 2] + c2[4 * j + 2]) * inv, (a[4 * j + 3] + c2[4 * j + 3]) * inv);
                }
            }
        }
        tc_fence_before();
        arrive(&epi_done);
        // with the probabilities stored, shared memory of this head served as their staging area until now
        if (PROBS && grp < 2 && hd + (int)gridDim.x < BH) convert_kq(it + 1);
    }
    tc_fence_before();
    __syncthreads();
}

// ---- host side: tensor maps and the launch ---------------------------------------------------------

template <bool CAUSAL, bool PROBS>
int launch_head_cfg(const HeadMaps &maps, float *out, float *probs, int B, int S, int E, int H, cudaStream_t st)
{
    auto kern = mha_head_kernel<CAUSAL, PROBS>;
    const size_t smem = kHeadSmemBytes + 1024;
    static bool attr_set = false;                    // per instantiation; setting it twice is harmless
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    const long long bh = (long long)B * H;
    if (bh > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "%lld (batch, head) pairs are too many", bh);
    const unsigned grid = (unsigned)(bh < sms ? bh : sms);
    const float cscale = (1.0f / sqrtf(32.0f)) * kLog2e;
    const cudaError_t le = launch_overlapped(kern, dim3(grid), dim3(kHeadThreads), smem, st, maps, out, probs, S, E, H, (int)bh, cscale);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "mha_head_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("mha_head_kernel");
}

}  // namespace

// head_dim 32, at most 256 tokens, planes whose rows TMA can address (16-byte aligned base and row pitch)
bool mha_head_supports(int head_dim, int S, int E, const void *q, const void *k, const void *v, const void *out)
{
    return head_dim == 32 && S >= 1 && S <= 2 * kTile && (E % 4) == 0 &&
           ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
             reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
           tma_encode_fn() != nullptr;
}

int launch_mha_head(const float *q, const float *k, const float *v, float *out, float *probs, int B, int S, int E, int H, int causal, cudaStream_t st)
{
    if (E / H != 32 || S > 2 * kTile) return fail(HIPGPT_ERR_UNSUPPORTED, "whole-head kernel: head_dim %d, S %d", E / H, S);
    if (B == 0 || S == 0) return HIPGPT_OK;
    HeadMaps maps;
    int rc = tma_plane_map(&maps.q, q, B, S, E, kTile, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == HIPGPT_OK) rc = tma_plane_map(&maps.q32, q, B, S, E, 32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == HIPGPT_OK) rc = tma_plane_map(&maps.k, k, B, S, E, kTile, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == HIPGPT_OK) rc = tma_plane_map(&maps.v, v, B, S, E, kTile, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HIPGPT_OK) return rc;
    if (probs) return causal ? launch_head_cfg<true, true>(maps, out, probs, B, S, E, H, st) : launch_head_cfg<false, true>(maps, out, probs, B, S, E, H, st);
    return causal ? launch_head_cfg<true, false>(maps, out, nullptr, B, S, E, H, st) : launch_head_cfg<false, false>(maps, out, nullptr, B, S, E, H, st);
}

// Reads and clears a status word of this file.
static int fetch_word(int &sym, int *value)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, sym, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(sym, &zero, sizeof(int));
    }
    *value = s;
    return HIPGPT_OK;
}
int head_status_fetch(int *status) { return fetch_word(g_head_status, status); }
int head_notice_fetch(int *notice) { return fetch_word(g_head_notice, notice); }

}  // namespace hipgpt
