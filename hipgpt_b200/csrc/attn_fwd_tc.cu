// Fused attention forward on the Blackwell tensor pipe (tcgen05 + TMEM), fp32-grade results.
//
// Replaces, like the FFMA rows kernel, the two kernels behind HipGPT's
// launch_multihead_attention (src/hip_kernels.cpp:263-325 and :329-402).
//
// The contraction runs as split-TF32 ("3xTF32"): every fp32 operand x is cut into
//   hi = x with the 13 low mantissa bits cleared (exactly a TF32 number), lo = x - hi (exact),
// and a product a*b is accumulated as a_lo*b_hi + a_hi*b_lo + a_hi*b_hi in the tensor core's
// fp32 accumulator (correction terms first, while the accumulator is small).  The dropped
// a_lo*b_lo term and the truncation of lo are below 2^-21 relative; measured against the
// fp32 oracle the outputs differ by at most 2.4e-6.
//
// One thread block = 128 query rows of one (batch, head): 128 worker threads (worker t owns
// query row q0+t = TMEM lane t) plus one warp whose single elected lane issues the MMAs.
// A tcgen05.mma with M=128, K=8 costs 64 cycles for any N up to 128 (measured), so the P V
// product concatenates its operands along N.  Per tile of 64 keys:
//   stage   K and V are read from global with coalesced 128-bit loads one tile ahead (they wait
//           in registers), split into hi / lo and written to shared memory in the tensor
//           core's canonical 128-byte-swizzled layouts (K: K-major SWIZZLE_128B; V: N-major,
//           which for 32-bit operands must be SWIZZLE_128B with a 32-byte base, hi blocks then
//           lo blocks so that [V_hi | V_lo] is one operand of 2D columns);
//   S       = Q K^T in three passes (Q_lo K_hi, Q_hi K_lo, Q_hi K_hi) of D/8 instructions,
//           M=128 N=64, accumulator in TMEM; two S buffers, so tile t+1 is computed while
//           tile t is in the softmax;
//   softmax the worker reads its row with tcgen05.ld, applies the causal / tail mask, keeps the
//           running maximum and sum in the log2 domain (one ex2 per score), splits P into
//           hi / lo and writes both back to TMEM (P_hi over S in place, P_lo beside it);
//   O_ext   = P_hi [V_hi | V_lo] (N = 2D) and P_lo V_hi added to its second half, A = P from
//           TMEM, fresh accumulator per tile; it is collected one iteration later, so its
//           latency hides behind the next tile's softmax;
//   update  o = o * alpha + (both halves of O_ext) in registers.
// Hand-offs use mbarriers: tcgen05.commit signals the MMAs' completion, 128 arrivals signal
// "next K staged" and "P written, V staged".  Two blocks per SM (head_dim 32) overlap one
// block's softmax with the other's MMAs.  Every wait is bounded: on expiry the block raises a
// flag that cuts all its later waits short, records a status code, skips its stores, frees
// its TMEM and returns.  No probabilities are written by this kernel; callers that want them
// get the FFMA rows kernel.
#include "tc_primitives.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kM = 128;          // query rows per block

__device__ int g_tc_status = 0;   // 0 ok; otherwise the site code of the first wait that ran out


// Shape of one kernel variant.
//   D        head_dim (32 or 64)
//   KN       keys per tile (64 or 128)
//   HALVES   workers per query row (1 or 2): each worker handles 64 consecutive keys of a tile and
//            D/HALVES output columns, so KN = 64 * HALVES
//   PRODUCERS threads that stage K and V
template <int D, int KN, int PRODUCERS>
struct TcCfg {
    static constexpr int HALVES = KN / 64;
    static constexpr int WORKERS = kM * HALVES;
    static constexpr int THREADS = WORKERS + 32 + PRODUCERS;   // workers, the issuing warp, producers
    static constexpr int DB = D / 32;                     // 32-float column blocks per row
    static constexpr int QBLK = kM * 32;                  // floats per [128][32] block
    static constexpr int KBLK = KN * 32;                  // floats per [KN][32] block
    // TMEM columns: S (two buffers of KN) | P_lo (KN) | O_ext (2D)
    static constexpr uint32_t kColS = 0;                  // scores, later P_hi in place
    static constexpr uint32_t kColPlo = 2 * KN;
    static constexpr uint32_t kColO = 3 * KN;             // [0,D): P_hi V_hi, [D,2D): P_hi V_lo + P_lo V_hi
    static constexpr uint32_t kTmemCols = (3 * KN + 2 * D) <= 256 ? 256 : 512;
    static constexpr int BLOCKS_PER_SM = kTmemCols == 256 ? 2 : 1;
    // Q hi/lo, K hi/lo, two V buffers of hi/lo, raw K and V tiles
    static constexpr size_t kSmemFloats = (size_t)2 * DB * QBLK + 2 * DB * KBLK + 4 * DB * KBLK + 2 * KN * D;
};

template <int D, int KN, int PRODUCERS, bool CAUSAL>
__global__ void __launch_bounds__(TcCfg<D, KN, PRODUCERS>::THREADS, TcCfg<D, KN, PRODUCERS>::BLOCKS_PER_SM)
mha_tc_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
              float *__restrict__ O, int S, int E, int H, int BH, int nqblk, float qscale)
{
    using C = TcCfg<D, KN, PRODUCERS>;
    constexpr int DB = C::DB, QBLK = C::QBLK, KBLK = C::KBLK, HALVES = C::HALVES, WORKERS = C::WORKERS;
    constexpr int CPR = D / 4;                   // 16-byte chunks per row
    constexpr int DW = D / HALVES;               // output columns per worker
    constexpr uint32_t kColS = C::kColS, kColPlo = C::kColPlo, kColO = C::kColO;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment is what the swizzled layouts assume
    float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *q_hi = base, *q_lo = q_hi + DB * QBLK;        // [DB][128][32] each
    float *k_hi = q_lo + DB * QBLK, *k_lo = k_hi + DB * KBLK;   // [DB][KN][32] each
    float *v_s = k_lo + DB * KBLK;               // [2 buffers][hi, lo][DB][KN][32]: hi and lo blocks form one 2D-column operand
    float *k_raw = v_s + 4 * DB * KBLK;          // [KN][D] as it lies in global memory, filled by cp.async
    float *v_raw = k_raw + KN * D;
    __shared__ uint64_t mbar_s[2], mbar_k, mbar_v[2], mbar_p, mbar_o;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float xchg[2][2][kM];             // [tile parity][half][row]: row maxima, at the end row sums

    const int tid = threadIdx.x, lane = tid & 31;
    // read from one lane, so that the compiler knows the warp's number (and every role that follows from it) to be warp-uniform
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);   // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * kM;

    const int kend = CAUSAL ? min(S, q0 + kM) : S;
    const int ntiles = (kend + KN - 1) / KN;

    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&mbar_s[0], 1);                // tcgen05.commit after Q K^T into S buffer 0 / 1
        mbar_init(&mbar_s[1], 1);
        mbar_init(&mbar_k, PRODUCERS);           // every producer: next K tile staged
        mbar_init(&mbar_v[0], PRODUCERS);        // every producer: V tile staged in buffer 0 / 1
        mbar_init(&mbar_v[1], PRODUCERS);
        mbar_init(&mbar_p, WORKERS);             // every worker: P written
        mbar_init(&mbar_o, 1);                   // tcgen05.commit after P V
    }
    __syncthreads();                             // barriers are initialised before anyone arrives on them

    // Bounded wait that gives up at once when another thread already gave up.
    // `site` names the wait in the status word: 1 S ready (worker), 2 O ready (worker), 3 K staged,
    // 5 P written, 6 V staged, 7 K buffer free (producer), 8 V buffer free (producer)
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) { abort_flag = 1; atomicCAS(&g_tc_status, 0, site); }
    };
    auto arrive = [&](uint64_t *bar) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };

    if (warp == WORKERS / 32) {
        // ================= the issuing warp: one lane feeds the tensor core ====================
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();                         // Q, K(0), V(0) staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kM, KN, 0);
            constexpr uint32_t idesc_pv1 = make_idesc(kM, 2 * D, 1);     // P_hi  x [V_hi | V_lo]
            constexpr uint32_t idesc_pv2 = make_idesc(kM, D, 1);         // P_lo  x V_hi
            auto issue_qk = [&](int buf) {
                uint32_t acc = 0;
#pragma unroll
                for (int pass = 0; pass < 3; ++pass) {
                    // the two correction terms first: the accumulator is still tiny while they
                    // are added, so the tensor core's truncating adds cost no accuracy there
                    const float *qa = pass == 0 ? q_lo : q_hi;
                    const float *kb = pass == 1 ? k_lo : k_hi;
#pragma unroll
                    for (int db = 0; db < DB; ++db) {
                        const uint64_t da = make_desc(smem_u32(qa + db * QBLK), 16, 1024, 2);
                        const uint64_t dk = make_desc(smem_u32(kb + db * KBLK), 16, 1024, 2);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {        // 8 floats = 32 bytes per instruction
                            mma_ss(tmem + kColS + buf * KN, da + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, acc);
                            acc = 1;
                        }
                    }
                }
                tc_commit(&mbar_s[buf]);
            };
            auto issue_pv = [&](int buf) {
                // N-major B: 8 reduction rows (keys) of 128 bytes per instruction = 1024 bytes
                const uint64_t dv = make_desc(smem_u32(v_s + buf * 2 * DB * KBLK), KBLK * 4, 512, 1);
#pragma unroll
                for (int k = 0; k < KN / 8; ++k)
                    mma_ts(tmem + kColO, tmem + kColS + buf * KN + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv1, k ? 1u : 0u);
                // the second correction term joins the first one in columns [D,2D): both are small
#pragma unroll
                for (int k = 0; k < KN / 8; ++k)
                    mma_ts(tmem + kColO + D, tmem + kColPlo + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv2, 1);
                tc_commit(&mbar_o);
            };
            if (ntiles > 0) issue_qk(0);
            for (int t = 0; t < ntiles; ++t) {
                wait(&mbar_k, (uint32_t)(t & 1), 3);     // K(t+1) is in shared memory
                tc_fence_after();
                // MMAs of one thread execute in issue order: P V(t-1), which still reads P_hi from
                // this S buffer, was issued before
                if (t + 1 < ntiles) issue_qk((t + 1) & 1);
                wait(&mbar_p, (uint32_t)(t & 1), 5);                    // P(t) is in TMEM
                wait(&mbar_v[t & 1], (uint32_t)((t >> 1) & 1), 6);      // V(t) is in shared memory
                tc_fence_after();
                issue_pv(t & 1);
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                         // the workers have collected the last O_ext
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
        return;
    }

    if (warp > WORKERS / 32) {
        // ================= the producers: global -> split -> shared memory =====================
        // A tile first lands, as it lies in global memory, in a raw buffer (cp.async, no
        // registers held while it is in flight).  The producer that fetched a 16-byte chunk is
        // also the one that later splits it, so it only waits for its own cp.async groups.
        constexpr int RPP = PRODUCERS / CPR;     // rows per pass
        constexpr int NP = KN / RPP;             // passes per tile
        const int ptid = tid - WORKERS - 32;
        const int sc = ptid % CPR, sr0 = ptid / CPR;
        auto fetch_tile = [&](const float *__restrict__ plane, float *raw, int t) {
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const int r = sr0 + p * RPP;
                const int j = t * KN + r;
                const bool ok = t < ntiles && j < S;
                cp_async16(raw + r * D + sc * 4, plane + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + sc * 4, ok);
            }
            cp_async_commit();
        };
        auto store_k = [&]() {
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const int r = sr0 + p * RPP;
                store_split(k_hi + (sc >> 3) * KBLK, k_lo + (sc >> 3) * KBLK, r, sc & 7,
                            *reinterpret_cast<const float4 *>(k_raw + r * D + sc * 4));
            }
        };
        auto store_v = [&](int buf) {
            float *blk = v_s + buf * 2 * DB * KBLK + (sc >> 3) * KBLK;
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                const int r = sr0 + p * RPP;
                store_split_nmajor(blk, blk + DB * KBLK, r, sc & 7, *reinterpret_cast<const float4 *>(v_raw + r * D + sc * 4));
            }
        };
        fetch_tile(K, k_raw, 0);
        fetch_tile(V, v_raw, 0);
        cp_async_wait_1();
        store_k();
        fetch_tile(K, k_raw, 1);
        cp_async_wait_1();
        store_v(0);
        fetch_tile(V, v_raw, 1);                 // from here on: K(t+1), then V(t+1) in flight at the top of iteration t
        proxy_fence();                           // generic-proxy writes -> visible to the tensor core's reads
        arrive(&mbar_v[0]);
        __syncthreads();
        for (int t = 0; t < ntiles; ++t) {
            wait(&mbar_s[t & 1], (uint32_t)((t >> 1) & 1), 7);     // Q K(t)^T has completed: the K buffer is free
            cp_async_wait_1();                                  // K(t+1) has landed
            if (t + 1 < ntiles) store_k();
            proxy_fence();
            arrive(&mbar_k);
            fetch_tile(K, k_raw, t + 2);
            if (t > 0) wait(&mbar_o, (uint32_t)((t - 1) & 1), 8); // P V(t-1) has completed: its V buffer is free
            cp_async_wait_1();                                  // V(t+1) has landed
            if (t + 1 < ntiles) store_v((t + 1) & 1);
            proxy_fence();
            arrive(&mbar_v[(t + 1) & 1]);
            fetch_tile(V, v_raw, t + 2);
        }
        cp_async_wait_all();
        __syncthreads();
        return;
    }

    // ===================== the workers: softmax and output ====================================
    const int half = warp >> 2;                  // which 64 keys of a tile / which output columns (0 when HALVES == 1)
    const int wq = warp & 3;                     // TMEM lane quadrant of this warp
    const int rloc = wq * 32 + lane;             // row inside the block = TMEM lane
    const int row = q0 + rloc;                   // this worker's query row
    {
        // Q: the workers of a row share its chunks
        constexpr int QC = CPR / HALVES;
        const bool ok = row < S;
        const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol) + half * QC;
#pragma unroll
        for (int c = 0; c < QC; ++c) {
            float4 x = ok ? __ldg(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            x.x *= qscale; x.y *= qscale; x.z *= qscale; x.w *= qscale;
            const int cc = half * QC + c;
            store_split(q_hi + (cc >> 3) * QBLK, q_lo + (cc >> 3) * QBLK, rloc, cc & 7, x);
        }
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;
    const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);   // this warp's 32 TMEM lanes

    float o[DW];
#pragma unroll
    for (int d = 0; d < DW; ++d) o[d] = 0.0f;
    float m = -1e30f, l = 0.0f, alpha_prev = 1.0f;

    // o = o * alpha_prev + (both parts of) O_ext of the previous tile, this worker's DW columns
    auto collect_o = [&]() {
        if (DW % 32 == 0) {
#pragma unroll
            for (int g = 0; g < DW / 32; ++g) {
                float a[32], c[32];
                tmem_ld32(lane_base + kColO + half * DW + g * 32, a);        // both loads in flight, one wait
                tmem_ld32(lane_base + kColO + D + half * DW + g * 32, c);
                tmem_wait_ld();
#pragma unroll
                for (int d = 0; d < 32; ++d) o[(g * 32 + d) % DW] = fmaf(o[(g * 32 + d) % DW], alpha_prev, a[d] + c[d]);
            }
        } else {
            float a[16], c[16];
            tmem_ld16(lane_base + kColO + half * DW, a);
            tmem_ld16(lane_base + kColO + D + half * DW, c);
            tmem_wait_ld();
#pragma unroll
            for (int d = 0; d < 16; ++d) o[d % DW] = fmaf(o[d % DW], alpha_prev, a[d] + c[d]);
        }
    };

    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        const int j0 = t * KN + half * 64;            // first key of this worker's 64 columns
        wait(&mbar_s[buf], (uint32_t)((t >> 1) & 1), 1);     // S(t) is in TMEM
        tc_fence_after();

        // ---- softmax of this worker's 64 scores (tcgen05 ops are warp-wide: uniform control flow) ----
        // Two sweeps over the scores in TMEM, so that only a few of them are in registers at
        // once: the first finds the row maximum, the second exponentiates.
        const bool warp_dead = CAUSAL && j0 > q0 + wq * 32 + 31;       // these columns are above the diagonal
        const bool need_mask = (CAUSAL && j0 + 63 > q0 + wq * 32) || j0 + 64 > S;
        // columns [0, nvalid) of this worker's 64 are visible to its row
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : 64);
        const uint32_t s_addr = lane_base + kColS + buf * KN + half * 64;
        const uint32_t plo_addr = lane_base + kColPlo + half * 64;
        float mx = -INFINITY;
        if (!warp_dead) {
            float v0[32], v1[32];
            tmem_ld32(s_addr, v0);                // both loads in flight, one wait
            tmem_ld32(s_addr + 32, v1);
            tmem_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    v0[c] = (c < nvalid) ? v0[c] : -INFINITY;
                    v1[c] = (32 + c < nvalid) ? v1[c] : -INFINITY;
                }
            }
            // four independent chains instead of one of depth 64
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
                m4[(c >> 1) & 1] = fmaxf(m4[(c >> 1) & 1], fmaxf(v0[c], v0[c + 1]));
                m4[2 + ((c >> 1) & 1)] = fmaxf(m4[2 + ((c >> 1) & 1)], fmaxf(v1[c], v1[c + 1]));
            }
            mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        }
        if (HALVES == 2) {
            // the two workers of a row agree on the tile's maximum through shared memory; the slot
            // alternates with the tile parity, so it is not overwritten before the partner read it
            xchg[buf][half][rloc] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory");
            mx = fmaxf(mx, xchg[buf][half ^ 1][rloc]);
        }
        const float mn = fmaxf(m, mx);            // m is finite (-1e30f at worst), so is mn
        const float alpha = ex2_approx(m - mn);
        m = mn;

        // ---- the previous tile's P V: collect it; P_lo is free afterwards ----------------------
        if (t > 0) {
            wait(&mbar_o, (uint32_t)((t - 1) & 1), 2);
            tc_fence_after();
            collect_o();
        }
        alpha_prev = alpha;

        float psum = 0.0f;
        if (warp_dead) {
            // nothing of these columns is visible to this warp's rows: P = 0
            float z[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) z[c] = 0.0f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                tmem_st16(s_addr + g * 16, z);
                tmem_st16(plo_addr + g * 16, z);
            }
        } else if (need_mask) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float v[16], lo[16];
                tmem_ld16(s_addr + g * 16, v);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p = (g * 16 + c < nvalid) ? ex2_approx(v[c] - mn) : 0.0f;
                    psum += p;
                    v[c] = tf32_hi(p);
                    lo[c] = p - v[c];
                }
                tmem_st16(s_addr + g * 16, v);                  // P_hi over S, in place
                tmem_st16(plo_addr + g * 16, lo);
            }
        } else {
            // chunks of 16 scores; the next chunk's load is in flight while this one is computed,
            // and the row sum runs in four independent chains
            float cur[16], nxt[16];
            float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            tmem_ld16(s_addr, cur);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                tmem_wait_ld();
                if (g + 1 < 4) tmem_ld16(s_addr + (g + 1) * 16, nxt);
                float lo[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p = ex2_approx(cur[c] - mn);
                    ps4[c & 3] += p;
                    cur[c] = tf32_hi(p);
                    lo[c] = p - cur[c];
                }
                tmem_st16(s_addr + g * 16, cur);                // P_hi over S, in place
                tmem_st16(plo_addr + g * 16, lo);
                if (g + 1 < 4) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) cur[c] = nxt[c];
                }
            }
            psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        }
        l = fmaf(l, alpha, psum);
        tmem_wait_st();
        tc_fence_before();
        arrive(&mbar_p);
    }
    if (ntiles > 0) {
        wait(&mbar_o, (uint32_t)((ntiles - 1) & 1), 2);
        tc_fence_after();
        collect_o();
    }
    if (HALVES == 2) {
        // row sums of the two halves (the maxima slots are idle now: every worker is past its last tile
        // once its partner has arrived at this barrier)
        asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory");
        xchg[0][half][rloc] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + wq) : "memory");
        l += xchg[0][half ^ 1][rloc];
    }
    if (!abort_flag && row < S) {
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + row) * (size_t)E + hcol + half * DW);
#pragma unroll
        for (int c = 0; c < DW / 4; ++c)
            dst[c] = make_float4(o[c * 4 + 0] * inv, o[c * 4 + 1] * inv, o[c * 4 + 2] * inv, o[c * 4 + 3] * inv);
    }
    tc_fence_before();
    __syncthreads();
}

template <int D, int KN, int PRODUCERS, bool CAUSAL>
int launch_tc_cfg(const float *q, const float *k, const float *v, float *out, int B, int S, int E, int H, cudaStream_t st)
{
    using C = TcCfg<D, KN, PRODUCERS>;
    auto kern = mha_tc_kernel<D, KN, PRODUCERS, CAUSAL>;
    // operands + alignment slack; a variant that allocates 256 TMEM columns asks for at least 100 KB,
    // so that at most two blocks share an SM and their allocations always fit in the 512 columns
    size_t smem = C::kSmemFloats * sizeof(float) + 1024;
    if (C::BLOCKS_PER_SM == 2 && smem < 100 * 1024) smem = 100 * 1024;
    if (C::BLOCKS_PER_SM == 1 && smem < 120 * 1024) smem = 120 * 1024;     // 512 columns: one block per SM
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kM - 1) / kM;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, C::THREADS, smem, st>>>(q, k, v, out, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_tc_kernel");
}

}  // namespace

bool mha_tc_supports(int D) { return D == 32 || D == 64; }

// The full-range split-TF32 kernel: 64-key tiles, one worker per query row.
int launch_mha_tc(const float *q, const float *k, const float *v, float *out,
                  int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (D == 32) return causal ? launch_tc_cfg<32, 64, 64, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<32, 64, 64, false>(q, k, v, out, B, S, E, H, st);
    if (D == 64) return causal ? launch_tc_cfg<64, 64, 64, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<64, 64, 64, false>(q, k, v, out, B, S, E, H, st);
    return fail(HIPGPT_ERR_UNSUPPORTED, "tensor-core kernel: head_dim %d is not 32 or 64", D);
}

// Reads and clears the status word of the tensor-core kernels (synchronises the device).
int tc_status_fetch(int *status)
{
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "status fetch: %s", cudaGetErrorString(e));
    return HIPGPT_OK;
}

}  // namespace hipgpt
