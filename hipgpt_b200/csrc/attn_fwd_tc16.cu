// Fused attention forward on the Blackwell tensor pipe (tcgen05 + TMEM), fp32-grade results, head_dim 32 or 64,
// any sequence length: the tiled kernel.
//
// Replaces the same reference kernels as attn_fwd_tc.cu (HipGPT src/hip_kernels.cpp:263-325 and :329-402).
// Arithmetic: every fp32 operand x is cut into hi (its 11 leading bits, exact in fp16) and lo = x - hi (rounded to
// fp16's 11 bits).  A product a*b = a_hi*b_hi + a_lo*b_hi + a_hi*b_lo runs as three kind::f16 instruction groups
// with fp32 accumulation in the tensor core; the dropped a_lo*b_lo and the rounding of the lo parts are 2^-22
// relative to the product.  Nothing but fp16 copies of the operands is kept in shared memory, which is what makes
// room for three stages of K and V beside Q at head_dim 64.
//   S = Q K^T:  [Q_hi | Q_lo] and [K_hi | K_lo] rows, K-major, 128-byte swizzle: Q_lo K_hi, Q_hi K_lo, Q_hi K_hi
//               (corrections first), 3 D/16 instructions per 64-key tile with N = 64.
//   O = P V:    P = 2^(s - m + 6) cut into fp16 P_hi, P_lo, written over S in place (per 32-column chunk: 16 columns
//               of packed P_hi, 16 of packed P_lo); V as [V_hi | V_lo], N-major:  P_hi [V_hi | V_lo] (N = 2 D) and
//               P_lo V_hi (N = D, added to the second half), A operand from TMEM, 8 instructions per 64 keys.
// Range: magnitudes up to fp16's largest number; beyond it the conversions saturate and the kernel raises the
// accuracy notice.  Small magnitudes cost absolute, not relative, accuracy: a lo part below 6e-5 is a subnormal fp16
// (steps of 6e-8), which the notice's test weighs against the scores it is added to.  The split-TF32 kernel
// (attn_fwd_tc.cu) has the whole fp32 range.
//
// One block = 128 query rows of one (batch, head); two blocks per SM at head_dim 32, one at head_dim 64.
//   Copies: one lane asks the TMA unit for whole raw tiles ([64 keys][32 floats] boxes, keys past S arrive as zeros)
//   into a ring of landing slots, as many tiles ahead as there are slots; the K and V warps turn a landed tile into
//   its fp16 operand stage (three stages) and publish it.  A stage is rewritten once the product that read it three
//   tiles ago has completed (barriers indexed by tile mod 3, completed by tcgen05.commit).
//   TMEM (256 columns): X0, X1 (64 each): S(t), overwritten in place by P(t);  O (2 D): [P_hi V_hi | P_hi V_lo + P_lo V_hi],
//   accumulated over ALL tiles.  Workers (thread = query row = TMEM lane) never read O back per tile: the reference
//   maximum only moves (and O is rescaled, by the whole warp) when a row's maximum grew by more than 2^8.
//   With P double-buffered, the worker goes from tile t straight to tile t+1 while P V(t) runs.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"
#include "tma_host.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per block
constexpr int kKeys = 64;         // keys per tile
constexpr int kWorkers = kRows;
constexpr int kStages = 3;        // fp16 operand stages of K and of V
constexpr float kRescaleStep = 8.0f;
constexpr float kPShift = 6.0f;   // P carries a factor 2^6: with the lazy reference maximum it stays below 2^15
constexpr int kBufs = 3;          // S / P buffers in TMEM
constexpr uint32_t kColX = 0, kColO = kBufs * kKeys;
static_assert(kBufs == kStages, "the barriers of buffers and stages share the tile-mod-3 phase arithmetic");

// Sizes that depend on head_dim.  An operand row is cut into blocks of 128 bytes (32 floats or 64
// fp16 values); a block of a tile is [rows][128 bytes], 128-byte swizzled.
template <int D>
struct Tc16Cfg {
    static constexpr int DB = D / 32;                         // fp32 blocks per row
    static constexpr int HB = (2 * D) / 64;                   // fp16 blocks per row of [x_hi | x_lo]
    static constexpr int PPR = D / 8;                         // 32-byte pieces per row
    static constexpr int PWK = D == 64 ? 4 : 1;               // warps that convert K
    static constexpr int PWV = D == 64 ? 4 : 2;               // warps that convert V
    static constexpr int NRAW = D == 64 ? 3 : 2;              // landing slots per operand
    static constexpr int THREADS = kWorkers + 64 + (PWK + PWV) * 32;   // workers, the two issuing warps, the K warps, the V warps
    static constexpr int BLOCKS_PER_SM = D == 64 ? 1 : 2;
    static constexpr uint32_t kTmemCols = (kColO + 2 * D) <= 256 ? 256 : 512;
    static constexpr int kQBlk = kRows * 128, kKBlk = kKeys * 128;      // bytes of one block of a Q / K tile
    static constexpr int kQ16Bytes = HB * kQBlk;
    static constexpr int kK16Stage = HB * kKBlk;              // [K_hi | K_lo] rows
    static constexpr int kV16Stage = kKeys * 2 * D * 2;       // [V_hi | V_lo], N-major without swizzle
    static constexpr int kRawSlot = DB * kKBlk;               // one raw fp32 tile
    static constexpr size_t kSmemBytes = (size_t)kQ16Bytes + kStages * (kK16Stage + kV16Stage) + 2 * NRAW * kRawSlot;
};

__device__ int g_tc16_status = 0;
__device__ int g_tc16_notice = 0;                // bit 0: an operand left the range in which the fp16 pieces are exact

__device__ __forceinline__ float amax8(float m, float4 a, float4 c)
{
    return fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                          fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(c.z), fabsf(c.w)))));
}
// The warp's largest magnitude into a shared word (as a bit pattern: non-negative floats order like integers).
__device__ __forceinline__ void publish_amax(unsigned *slot, float m)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(slot, __float_as_uint(m));
}

// The polling part of a bounded wait; on expiry the block's abort flag is raised and the site recorded.
__device__ __noinline__ void tc16_wait_slow(uint64_t *bar, uint32_t parity, int site, volatile int *abort_flag)
{
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicCAS(&g_tc16_status, 0, site);
    }
}

// Largest of 32 scores; columns from `nvalid` on (counted from the chunk's first column `col0`) are hidden.
__device__ __forceinline__ float chunk_max(float (&v)[32], int col0, int nvalid, bool need_mask)
{
    if (need_mask) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (col0 + j < nvalid) ? v[j] : -INFINITY;
    }
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        m4[0] = fmaxf(m4[0], v[j]); m4[1] = fmaxf(m4[1], v[j + 1]);
        m4[2] = fmaxf(m4[2], v[j + 2]); m4[3] = fmaxf(m4[3], v[j + 3]);
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// One chunk of scores (log2 domain) -> P = 2^(s + nm), cut into fp16 hi and lo, written over the chunk's own 32 TMEM
// columns (16 of packed P_hi, then 16 of packed P_lo).  Returns the sum of P.
__device__ __forceinline__ float chunk_exp(float (&v)[32], uint32_t addr, int col0, int nvalid, bool need_mask, float nm)
{
    if (need_mask) {
        // a hidden score becomes -inf: its exponential is exactly 0
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (col0 + j < nvalid) ? v[j] : -INFINITY;
    }
    float ps[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float p0 = ex2_approx(v[16 * half + j] + nm), p1 = ex2_approx(v[16 * half + j + 1] + nm);
            ps[j & 3] += p0;
            ps[(j + 1) & 3] += p1;
            const float h0 = tf32_hi(p0), h1 = tf32_hi(p1);      // 11 leading bits: exact in fp16
            hi[j >> 1] = pack_f16(h0, h1);
            lo[j >> 1] = pack_f16(p0 - h0, p1 - h1);
        }
        tmem_st8_u32(addr + 8 * half, hi);
        tmem_st8_u32(addr + 16 + 8 * half, lo);
    }
    return (ps[0] + ps[1]) + (ps[2] + ps[3]);
}

// Which pieces of a 64-row tile a converting thread owns.  A piece is 32 bytes (8 floats) of a row; a
// thread owns pieces of pairs of adjacent rows.  PT = threads that convert this operand, PPR = pieces per row.
template <int PT, int PPR>
struct PieceMap {
    static constexpr int NPC = (kKeys * PPR) / PT;            // pieces per thread and tile
    static constexpr int RPP = 2 * (PT / PPR);                // rows covered by a pair of passes
    static constexpr int BATCH = NPC < 8 ? NPC : 8;           // pieces converted at a time
    int pc, pq, pblk, pch;                                    // piece of a row, row pair, fp32 block and first 16-byte chunk of the piece
    __device__ explicit PieceMap(int pid) : pc(pid % PPR), pq(pid / PPR), pblk((pid % PPR) >> 2), pch(2 * ((pid % PPR) & 3)) {}
    __device__ int row(int p) const { return RPP * (p >> 1) + 2 * pq + (p & 1); }
};

template <int D, bool CAUSAL, bool PROBS>
__global__ void __launch_bounds__(Tc16Cfg<D>::THREADS, Tc16Cfg<D>::BLOCKS_PER_SM)
mha_tc16_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, const float *__restrict__ Q,
                float *__restrict__ O, float *__restrict__ P, int S, int E, int H, int BH, int nqblk, float qscale)
{
    using C = Tc16Cfg<D>;
    constexpr int DB = C::DB, PPR = C::PPR, PWK = C::PWK, PWV = C::PWV, NRAW = C::NRAW;
    constexpr int kQBlk = C::kQBlk, kKBlk = C::kKBlk;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_16 = base;                                    // fp16 [HB][128][64]: a row is [Q_hi (D) | Q_lo (D)], K-major
    uint8_t *k_16 = q_16 + C::kQ16Bytes;                     // per stage: fp16 [HB][64][64]: [K_hi (D) | K_lo (D)]
    uint8_t *k_raw = k_16 + kStages * C::kK16Stage;          // landing slots: fp32 [DB][64][32], 128-byte swizzled
    uint8_t *v_16 = k_raw + NRAW * C::kRawSlot;              // per stage: [V_hi | V_lo] fp16, N-major: 8 keys x 8 columns form one
                                                             // 128-byte core matrix, column blocks 128 bytes apart, key groups 32 D
    uint8_t *v_raw = v_16 + kStages * C::kV16Stage;          // landing slots (the second sweep's staging area starts at v_16)
    __shared__ uint64_t k_land[NRAW], v_land[NRAW], k_full[kStages], v_full[kStages], s_full[kStages], o_done[kStages], p_full[kBufs];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ unsigned s_amax[3];                   // largest |Q| (scaled), |K|, |V| this block has seen

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
    // With PROBS the key tiles are swept a second time once a row's maximum and sum are final:
    // Q K^T is formed again and the normalised probabilities go to global memory.  Sweep-2 tile
    // u (nt <= u < 2 nt) is key tile u - nt; stages, buffers and barrier phases continue by u.
    const int nk = PROBS ? 2 * nt : nt;              // K tiles staged, Q K^T products issued

    if (tid == 0) {
        abort_flag = 0;
        s_amax[0] = s_amax[1] = s_amax[2] = 0u;
        for (int i = 0; i < NRAW; ++i) {
            mbar_init(&k_land[i], 1);                // the copy of a tile: one announcement, then its bytes
            mbar_init(&v_land[i], 1);
        }
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&k_full[i], PWK);              // one arrival per K warp
            mbar_init(&v_full[i], PWV);              // one arrival per V warp
            mbar_init(&s_full[i], 1);                // tcgen05.commit after Q K(t)^T, t mod 3 = i: S is ready, and the K stage is free
            mbar_init(&o_done[i], 1);                // tcgen05.commit after P V(t): O is up to date, and the V stage is free
        }
        for (int i = 0; i < kBufs; ++i) mbar_init(&p_full[i], kWorkers / 32);    // one arrival per worker warp
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K staged,
    // 5 P written, 6 V staged, 7 K stage free, 8 V stage free, 9 K tile landed, 10 V tile landed
    // (the polling loop exists once, out of line: an already completed phase costs one test)
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag || mbar_test(bar, parity)) return;
        tc16_wait_slow(bar, parity, site, &abort_flag);
    };
    // one arrival for the whole warp: every lane's writes are ordered before it by the warp barrier
    auto arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };
    // byte offset, inside an fp16 operand of rows [hi (D) | lo (D)], of the 16-byte chunk holding values
    // 8 e8 .. 8 e8 + 7 of row r; blk = bytes of one 128-byte-row block of that operand
    auto off16 = [](int r, int e8, int blk) { return (e8 >> 3) * blk + sw128(r, e8 & 7); };
    // barrier slot and phase parity of tile t for the barriers that are indexed by tile mod 3
    auto ph3 = [](int t) { return (uint32_t)((t / kStages) & 1); };

    if (warp == kWorkers / 32 || warp == kWorkers / 32 + 1) {
        // ================= the two issuing warps =================================================
        // One issues the K copies and every Q K^T, the other the V copies and every P V: an instruction costs the warp
        // that issues it 60 - 100 cycles, more than it costs the tensor pipe, and two warps issue side by side.  Each
        // accumulator is written by one warp, in tile order; what one warp's products need from the other's is
        // ordered by the tcgen05.commit barriers.  The warps stay converged and elect the issuing lane per instruction
        // (descriptors are then computed warp-uniformly, in uniform registers).
        const bool qk_role = warp == kWorkers / 32;
        if (qk_role) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        // one lane asks the TMA unit for a whole raw tile; the first tiles are asked for before anything else happens
        auto copy_k = [&](int u) {                   // u counts staged K tiles: the second sweep reads the tiles again
            if (lane == 0 && u < nk) {
                const int slot = u % NRAW, j0 = (u < nt ? u : u - nt) * kKeys;
                mbar_arrive_expect_tx(&k_land[slot], (uint32_t)C::kRawSlot);
#pragma unroll
                for (int db = 0; db < DB; ++db)
                    tma_load_3d(k_raw + slot * C::kRawSlot + db * kKBlk, &kmap, (int)hcol + 32 * db, j0, b, &k_land[slot]);
            }
            __syncwarp();
        };
        auto copy_v = [&](int u) {
            if (lane == 0 && u < nt) {
                const int slot = u % NRAW;
                mbar_arrive_expect_tx(&v_land[slot], (uint32_t)C::kRawSlot);
#pragma unroll
                for (int db = 0; db < DB; ++db)
                    tma_load_3d(v_raw + slot * C::kRawSlot + db * kKBlk, &vmap, (int)hcol + 32 * db, u * kKeys, b, &v_land[slot]);
            }
            __syncwarp();
        };
        if (qk_role) {
            for (int u = 0; u < NRAW; ++u) copy_k(u);
        } else {
            for (int u = 0; u < NRAW; ++u) copy_v(u);
        }
        tc_fence_before();
        __syncthreads();                             // Q staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (qk_role) {
            constexpr uint32_t id_qk = idesc_f16(kRows, kKeys);                    // fp16 x fp16, both K-major
            auto issue_qk = [&](int buf, int t) {
                const uint32_t d = tmem + kColX + buf * kKeys;
                const uint8_t *kst = k_16 + (t % kStages) * C::kK16Stage;
                // the correction terms first: the accumulator is still tiny while they are added
#pragma unroll
                for (int prod = 0; prod < 3; ++prod) {
                    const int qc = prod == 0 ? D : 0, kc = prod == 1 ? D : 0;      // Q_lo K_hi, Q_hi K_lo, Q_hi K_hi
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const int qa = qc + 16 * k, ka = kc + 16 * k;              // first of 16 columns of a row of [hi | lo]
                        const uint64_t dq = make_desc(smem_u32(q_16 + (qa >> 6) * kQBlk), 16, 1024, 2) + (uint64_t)(((qa & 63) >> 4) * 2);
                        const uint64_t dk = make_desc(smem_u32(kst + (ka >> 6) * kKBlk), 16, 1024, 2) + (uint64_t)(((ka & 63) >> 4) * 2);
                        if (elect_one()) mma_h_ss(d, dq, dk, id_qk, (prod | k) ? 1u : 0u);
                    }
                }
                if (elect_one()) tc_commit(&s_full[t % kStages]);    // S is ready; it also tells the K warps that this stage is free
            };
            wait(&k_full[0], 0, 4);
            tc_fence_after();
            issue_qk(0, 0);
            for (int t = 0; t + 1 < nk; ++t) {
                // the landing slot of K(t) was read when K(t) was converted, before Q K(t)^T was issued
                copy_k(t + NRAW);
                wait(&k_full[(t + 1) % kStages], ph3(t + 1), 4);                 // K(t+1) is in its stage
                // the buffer of S(t+1) held P(t-2) (first sweep) or S(t-2) (second sweep): with three buffers the product
                // runs up to two tiles ahead of the exponentials and never waits for the P V product before it
                if (t >= 2) {
                    if (t - 2 < nt) wait(&o_done[(t - 2) % kStages], ph3(t - 2), 2);          // P V(t-2) has read it
                    else wait(&p_full[(t - 2) % kBufs], ph3(t - 2), 5);                       // the workers have read it
                }
                tc_fence_after();
                issue_qk((t + 1) % kBufs, t + 1);
            }
        } else {
            constexpr uint32_t id_pv_a = idesc_f16(kRows, 2 * D) | (1u << 16);     // P_hi x [V_hi | V_lo], B N-major
            constexpr uint32_t id_pv_b = idesc_f16(kRows, D) | (1u << 16);         // P_lo x V_hi
            for (int t = 0; t < nt; ++t) {
                const int buf = t % kBufs;
                wait(&p_full[buf], ph3(t), 5);                                   // P(t) is in TMEM
                wait(&v_full[t % kStages], ph3(t), 6);                           // V(t) is in its stage: its landing slot has been read
                copy_v(t + NRAW);
                tc_fence_after();
                const uint32_t a0 = tmem + kColX + buf * kKeys;
                // N-major B without swizzle: lbo = bytes between groups of 8 keys, sbo = bytes between blocks of 8 columns
                const uint64_t dv = make_desc(smem_u32(v_16 + (t % kStages) * C::kV16Stage), 32 * D, 128, 0);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)  // 16 keys = 8 TMEM columns of packed fp16 = two key groups of V
                    if (elect_one()) mma_h_ts(tmem + kColO, a0 + (uint32_t)(32 * (k >> 1) + 8 * (k & 1)), dv + (uint64_t)(k * 4 * D), id_pv_a, (t == 0 && k == 0) ? 0u : 1u);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    if (elect_one()) mma_h_ts(tmem + kColO + D, a0 + (uint32_t)(32 * (k >> 1) + 8 * (k & 1) + 16), dv + (uint64_t)(k * 4 * D), id_pv_b, 1u);
                if (elect_one()) tc_commit(&o_done[t % kStages]);    // O is up to date; the V warps may rewrite this stage, Q K^T this buffer
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read the output
        if (qk_role) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
        return;
    }

    // ================= the converting warps ===========================================================
    // A raw fp32 tile lands in a slot by TMA; a thread reads its own 32-byte pieces (8 floats of pairs of adjacent
    // rows), cuts them into hi and lo and writes the fp16 operand stage.  The stage of tile u was read by the product
    // of tile u - 3.
    if (warp > kWorkers / 32 + 1 && warp <= kWorkers / 32 + 1 + PWK) {
        const PieceMap<32 * PWK, PPR> pm(tid - kWorkers - 64);
        constexpr int NPC = pm.NPC, BATCH = pm.BATCH;
        const int pc = pm.pc, pblk = pm.pblk, pch = pm.pch;
        float amax = 0.0f;
        __syncthreads();                             // matches the block-wide barrier after Q staging
        for (int u = 0; u < nk; ++u) {
            const uint8_t *raw = k_raw + (u % NRAW) * C::kRawSlot + pblk * kKBlk;
            uint8_t *k16 = k_16 + (u % kStages) * C::kK16Stage;
            wait(&k_land[u % NRAW], (uint32_t)((u / NRAW) & 1), 9);              // the raw tile has landed
            if (u >= kStages) wait(&s_full[u % kStages], ph3(u - kStages), 7);   // Q K(u-3)^T has completed
#pragma unroll
            for (int half = 0; half < NPC / BATCH; ++half) {
                float4 a[BATCH], c[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = pm.row(half * BATCH + i);
                    a[i] = *reinterpret_cast<const float4 *>(raw + sw128(r, pch));
                    c[i] = *reinterpret_cast<const float4 *>(raw + sw128(r, pch + 1));
                }
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = pm.row(half * BATCH + i);
                    const float4 ah = hi4(a[i]), ch = hi4(c[i]);
                    amax = amax8(amax, a[i], c[i]);
                    *reinterpret_cast<uint4 *>(k16 + off16(r, pc, kKBlk)) =
                        make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
                    *reinterpret_cast<uint4 *>(k16 + off16(r, PPR + pc, kKBlk)) =
                        make_uint4(pack_f16(a[i].x - ah.x, a[i].y - ah.y), pack_f16(a[i].z - ah.z, a[i].w - ah.w),
                                   pack_f16(c[i].x - ch.x, c[i].y - ch.y), pack_f16(c[i].z - ch.z, c[i].w - ch.w));
                }
            }
            proxy_fence();                           // generic-proxy writes -> visible to the tensor core
            arrive(&k_full[u % kStages]);
        }
        publish_amax(&s_amax[1], amax);
        __syncthreads();
        return;
    }
    if (warp > kWorkers / 32 + 1 + PWK) {
        const PieceMap<32 * PWV, PPR> pm(tid - kWorkers - 64 - 32 * PWK);
        constexpr int NPC = pm.NPC, BATCH = pm.BATCH;
        const int pc = pm.pc, pblk = pm.pblk, pch = pm.pch;
        float amax = 0.0f;
        __syncthreads();
        for (int u = 0; u < nt; ++u) {
            const uint8_t *raw = v_raw + (u % NRAW) * C::kRawSlot + pblk * kKBlk;
            uint8_t *v16 = v_16 + (u % kStages) * C::kV16Stage;
            wait(&v_land[u % NRAW], (uint32_t)((u / NRAW) & 1), 10);             // the raw tile has landed
            if (u >= kStages) wait(&o_done[u % kStages], ph3(u - kStages), 8);   // P V(u-3) has completed
#pragma unroll
            for (int half = 0; half < NPC / BATCH; ++half) {
                float4 a[BATCH], c[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = pm.row(half * BATCH + i);
                    a[i] = *reinterpret_cast<const float4 *>(raw + sw128(r, pch));
                    c[i] = *reinterpret_cast<const float4 *>(raw + sw128(r, pch + 1));
                }
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = pm.row(half * BATCH + i);
                    const float4 ah = hi4(a[i]), ch = hi4(c[i]);
                    amax = amax8(amax, a[i], c[i]);
                    // key r, columns 8 pc ..: V_hi in column block pc, V_lo in column block D / 8 + pc
                    uint8_t *dst = v16 + (r >> 3) * (32 * D) + (r & 7) * 16;
                    *reinterpret_cast<uint4 *>(dst + pc * 128) =
                        make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
                    *reinterpret_cast<uint4 *>(dst + (PPR + pc) * 128) =
                        make_uint4(pack_f16(a[i].x - ah.x, a[i].y - ah.y), pack_f16(a[i].z - ah.z, a[i].w - ah.w),
                                   pack_f16(c[i].x - ch.x, c[i].y - ch.y), pack_f16(c[i].z - ch.z, c[i].w - ch.w));
                }
            }
            proxy_fence();
            arrive(&v_full[u % kStages]);
        }
        publish_amax(&s_amax[2], amax);
        __syncthreads();
        return;
    }

    // ===================== the workers ===========================================================
    const int wq = warp;                             // TMEM lane quadrant of this warp
    const int rloc = wq * 32 + lane;                 // row inside the block = TMEM lane
    const int row = q0 + rloc;
    {
        float amax = 0.0f;
        const bool ok = row < S;
        const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int j = 0; j < PPR; ++j) {              // 8 floats at a time
            float4 a = ok ? __ldg(src + 2 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 c = ok ? __ldg(src + 2 * j + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            a.x *= qscale; a.y *= qscale; a.z *= qscale; a.w *= qscale;     // scores come out in the log2 domain
            c.x *= qscale; c.y *= qscale; c.z *= qscale; c.w *= qscale;
            const float4 ah = hi4(a), ch = hi4(c);
            amax = amax8(amax, a, c);
            *reinterpret_cast<uint4 *>(q_16 + off16(rloc, j, kQBlk)) =
                make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
            *reinterpret_cast<uint4 *>(q_16 + off16(rloc, PPR + j, kQBlk)) =
                make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                           pack_f16(c.x - ch.x, c.y - ch.y), pack_f16(c.z - ch.z, c.w - ch.w));
        }
        publish_amax(&s_amax[0], amax);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (log2 domain) and row sum (of P, which carries 2^6)
    for (int t = 0; t < nt; ++t) {
        const int buf = t % kBufs;
        const int j0 = t * kKeys;
        const uint32_t s_addr = lane_base + kColX + buf * kKeys;
        wait(&s_full[t % kStages], ph3(t), 1);       // S(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + wq * 32;              // first row of this warp
        // columns of this tile that the row sees; the warp's last row sees the most, its first row the fewest
        const int ncols = min(kKeys, S - j0);
        const int nvalid = CAUSAL ? max(0, min(ncols, row - j0 + 1)) : ncols;
        const int nwarp = CAUSAL ? max(0, min(ncols, wrow0 + 31 - j0 + 1)) : ncols;
        const int nmin = CAUSAL ? max(0, min(ncols, wrow0 - j0 + 1)) : ncols;
        const int nch = (nwarp + 31) >> 5;           // 32-column chunks with any visible key (0: the tile is above the diagonal for the warp)

        // ---- first sweep: the row's largest score of this tile ------------------------------------
        float mx = -INFINITY;
        float v[32];
#pragma unroll 1
        for (int c = 0; c < nch; ++c) {
            tmem_ld32(s_addr + c * 32, v);
            tmem_wait_ld();
            mx = fmaxf(mx, chunk_max(v, c * 32, nvalid, c * 32 + 32 > nmin));
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
                wait(&o_done[(t - 1) % kStages], ph3(t - 1), 2);     // P V(t-1) has completed
                tc_fence_after();
#pragma unroll 1
                for (int hh = 0; hh < (2 * D) / 16; ++hh) {
                    float a[16];
                    tmem_ld16(o_addr + hh * 16, a);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) a[c] *= alpha;
                    tmem_st16(o_addr + hh * 16, a);
                }
            }
        }

        // ---- second sweep: exponentials; P_hi and P_lo over S in place ---------------------------------
        const float nm = kPShift - m_ref;
        float psum = 0.0f;
#pragma unroll 1
        for (int c = 0; c < nch; ++c) {
            tmem_ld32(s_addr + c * 32, v);
            tmem_wait_ld();
            psum += chunk_exp(v, s_addr + c * 32, c * 32, nvalid, c * 32 + 32 > nmin, nm);
        }
#pragma unroll 1
        for (int c = nch; c < kKeys / 32; ++c) {     // chunks that no row of this warp sees
            uint32_t z[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) z[j] = 0u;
            tmem_st16_u32(s_addr + c * 32, z);
            tmem_st16_u32(s_addr + c * 32 + 16, z);
        }
        l += psum;
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[buf]);
    }

    {
        wait(&o_done[(nt - 1) % kStages], ph3(nt - 1), 3);
        tc_fence_after();
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        const bool store = !abort_flag && row < S;
        float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + (row < S ? row : 0)) * (size_t)E + hcol);
#pragma unroll 1
        for (int hh = 0; hh < D / 16; ++hh) {
            float a[16], c2[16];
            tmem_ld16(o_addr + hh * 16, a);              // P_hi V_hi
            tmem_ld16(o_addr + D + hh * 16, c2);         // the correction terms
            tmem_wait_ld();
            if (store) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    dst[hh * 4 + c] = make_float4((a[c * 4 + 0] + c2[c * 4 + 0]) * inv, (a[c * 4 + 1] + c2[c * 4 + 1]) * inv,
                                                  (a[c * 4 + 2] + c2[c * 4 + 2]) * inv, (a[c * 4 + 3] + c2[c * 4 + 3]) * inv);
            }
        }
        if (PROBS) {
            // ---- second sweep: p = 2^(s - m_ref) / l for every key of the row, zeros where masked -----
            // A worker holds one row, so its own stores would be 16-byte pieces S floats apart.  The warp
            // turns its 32 x 64 tile through shared memory instead (the V stages are free: the last P V
            // product has completed) and stores two rows of 256 contiguous bytes per instruction.
            uint8_t *tb = v_16 + wq * (32 * kKeys * 4);  // 16-byte chunk c of row r at r * 256 + ((c ^ (r & 7)) << 4)
            const int wrow0 = q0 + wq * 32;              // first row of this warp
            float *pwarp = P + ((size_t)bh * S + wrow0) * (size_t)S;
            const bool vec = (S & 3) == 0;               // then every 4-column group of a row is 16-byte aligned
            for (int u = nt; u < nk; ++u) {
                const int buf = u % kBufs, j0 = (u - nt) * kKeys;
                const uint32_t s_addr = lane_base + kColX + buf * kKeys;
                wait(&s_full[u % kStages], ph3(u), 1);
                tc_fence_after();
                const bool warp_dead = CAUSAL && j0 > wrow0 + 31;
                const int ncols = min(kKeys, S - j0);                                   // columns of this tile that exist
                const int nvalid = min(ncols, CAUSAL ? row - j0 + 1 : kKeys);           // ... that this row sees
                float v0[32], v1[32];
                if (!warp_dead) {
                    tmem_ld32(s_addr, v0);
                    tmem_ld32(s_addr + 32, v1);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v0[c] = v1[c] = 0.0f;
                }
                tc_fence_before();
                arrive(&p_full[buf]);                    // the issuing lane may overwrite this buffer with S(u+2)
#pragma unroll
                for (int c4 = 0; c4 < 16; ++c4) {
                    float o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = 4 * c4 + i;
                        const float sc = c < 32 ? v0[c & 31] : v1[c & 31];
                        o[i] = c < nvalid ? ex2_approx(sc - m_ref + kPShift) * inv : 0.0f;
                    }
                    *reinterpret_cast<float4 *>(tb + lane * 256 + ((c4 ^ (lane & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
                }
                __syncwarp();
                if (!abort_flag) {
                    if (vec) {
                        const int ch = lane & 15;
#pragma unroll 4
                        for (int i = 0; i < 16; ++i) {
                            const int rr = 2 * i + (lane >> 4);
                            const float4 val = *reinterpret_cast<const float4 *>(tb + rr * 256 + ((ch ^ (rr & 7)) << 4));
                            if (wrow0 + rr < S && 4 * ch < ncols)
                                *reinterpret_cast<float4 *>(pwarp + (size_t)rr * S + j0 + 4 * ch) = val;
                        }
                    } else {
                        for (int rr = 0; rr < 32 && wrow0 + rr < S; ++rr)
                            for (int c = lane; c < ncols; c += 32)
                                pwarp[(size_t)rr * S + j0 + c] =
                                    *reinterpret_cast<const float *>(tb + rr * 256 + (((c >> 2) ^ (rr & 7)) << 4) + (c & 3) * 4);
                    }
                }
                __syncwarp();                            // the tile is out before the next one is staged
            }
            // keys past the last tile of a causal block are all masked
            if (CAUSAL && !abort_flag) {
                const int z0 = nt * kKeys;
                for (int rr = 0; rr < 32 && wrow0 + rr < S; ++rr) {
                    float *pr = pwarp + (size_t)rr * S;
                    if (vec) {
                        for (int c = z0 + 4 * lane; c < S; c += 128) *reinterpret_cast<float4 *>(pr + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                    } else {
                        for (int c = z0 + lane; c < S; c += 32) pr[c] = 0.0f;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        // Range of the fp16 pieces: beyond fp16's largest number they saturate; below its smallest normal numbers a
        // lo part is flushed, an absolute error of up to 2^-25 per fp16 value, which matters when it is neither small
        // in itself nor small beside the scores it is added to.  (Q carries the softmax scale here.)
        const float aq = __uint_as_float(s_amax[0]), ak = __uint_as_float(s_amax[1]), av = __uint_as_float(s_amax[2]);
        const bool over = !(aq <= 65504.0f) || !(ak <= 65504.0f) || !(av <= 65504.0f);
        const float flush = (float)D * 2.98e-8f * (aq + ak);
        if (over || (flush > 3.8e-6f && (aq + ak) > 8.0f * aq * ak)) atomicOr(&g_tc16_notice, 1);
    }
}

template <int D, bool CAUSAL, bool PROBS>
int launch_tc16_cfg(const float *q, const float *k, const float *v, float *out, float *probs, int B, int S, int E, int H, cudaStream_t st)
{
    using C = Tc16Cfg<D>;
    auto kern = mha_tc16_kernel<D, CAUSAL, PROBS>;
    // two blocks per SM (256 TMEM columns each): at least 100 KB, so that a third block never shares the SM;
    // one block per SM (512 columns): more than half of the SM's shared memory
    size_t smem = C::kSmemBytes + 1024;
    if (C::BLOCKS_PER_SM == 2 && smem < 100 * 1024) smem = 100 * 1024;
    if (C::BLOCKS_PER_SM == 1 && smem < 120 * 1024) smem = 120 * 1024;
    static_assert(C::kSmemBytes + 1024 + 2048 <= 232448 / C::BLOCKS_PER_SM, "shared memory of a block");
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kRows - 1) / kRows;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    // raw tiles land as rows of 128 bytes with the 128-byte swizzle; the converting threads read them back the same way
    CUtensorMap kmap, vmap;
    int rc = tma_plane_map(&kmap, k, B, S, E, kKeys, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == HIPGPT_OK) rc = tma_plane_map(&vmap, v, B, S, E, kKeys, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != HIPGPT_OK) return rc;
    kern<<<(unsigned)blocks, C::THREADS, smem, st>>>(kmap, vmap, q, out, probs, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_tc16_kernel");
}

}  // namespace

bool mha_tc16_supports(int head_dim) { return head_dim == 32 || head_dim == 64; }

// `probs` (optional): [B][H][S][S], written by a second sweep over the key tiles
int launch_mha_tc16(const float *q, const float *k, const float *v, float *out, float *probs,
                    int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (!mha_tc16_supports(D)) return fail(HIPGPT_ERR_UNSUPPORTED, "tf32+fp16 tensor-core kernel: head_dim %d is not 32 or 64", D);
    if (B == 0 || S == 0) return HIPGPT_OK;
    const int sel = (D == 64 ? 4 : 0) | (causal ? 2 : 0) | (probs ? 1 : 0);
    switch (sel) {
    case 0: return launch_tc16_cfg<32, false, false>(q, k, v, out, probs, B, S, E, H, st);
    case 1: return launch_tc16_cfg<32, false, true>(q, k, v, out, probs, B, S, E, H, st);
    case 2: return launch_tc16_cfg<32, true, false>(q, k, v, out, probs, B, S, E, H, st);
    case 3: return launch_tc16_cfg<32, true, true>(q, k, v, out, probs, B, S, E, H, st);
    case 4: return launch_tc16_cfg<64, false, false>(q, k, v, out, probs, B, S, E, H, st);
    case 5: return launch_tc16_cfg<64, false, true>(q, k, v, out, probs, B, S, E, H, st);
    case 6: return launch_tc16_cfg<64, true, false>(q, k, v, out, probs, B, S, E, H, st);
    default: return launch_tc16_cfg<64, true, true>(q, k, v, out, probs, B, S, E, H, st);
    }
}

int tc16_status_fetch(int *status)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, g_tc16_status, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc16_status, &zero, sizeof(int));
    }
    *status = s;
    return HIPGPT_OK;
}

int tc16_notice_fetch(int *notice)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, g_tc16_notice, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc16_notice, &zero, sizeof(int));
    }
    *notice = s;
    return HIPGPT_OK;
}

}  // namespace hipgpt
