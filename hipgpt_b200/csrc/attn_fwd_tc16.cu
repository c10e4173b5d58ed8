// Fused attention forward on the Blackwell tensor pipe (tcgen05 + TMEM), fp32-grade results,
// head_dim 32 or 64: TF32 main products with FP16 correction products, and a pipeline in which the
// softmax of tile t+1 does not wait for the P V product of tile t.
//
// Replaces the same reference kernels as attn_fwd_tc.cu (HipGPT src/hip_kernels.cpp:263-325 and
// :329-402).  Arithmetic: every fp32 operand x is cut into hi (TF32-exact, 11 significant bits)
// and lo = x - hi (exact).  A product a*b = a_hi*b_hi + a_lo*b_hi + a*b_lo is accumulated in the
// tensor core's fp32 accumulator as
//     a_hi*b_hi             one kind::tf32 instruction group,
//     a_lo*b_hi + a*b_lo    one kind::f16 group on fp16 copies, concatenated along the reduction
//                           dimension: [a_lo | a] x [b_hi | b_lo].  b_hi is exact in fp16 (11 bits),
//                           a_lo, b_lo and a are rounded to 11 bits, an error of 2^-22 relative to
//                           the product, the same order as the dropped a_lo*b_lo of plain split-TF32.
// fp16 has K=16 per instruction against 8 for TF32, so a 64-key tile takes 20 instructions
// instead of 28 at head_dim 32 and 28 instead of 40 at head_dim 64 (an instruction with M=128
// costs about 64 cycles for any N <= 128).
// Range: the fp16 copies are good to 11 bits for magnitudes within fp16's normal range.  Conversions
// saturate: an operand beyond +-65504 keeps its TF32 main product but loses its correction term,
// and lo parts below 6e-5 become subnormal.  Measured against the fp32 arithmetic: V of magnitude
// 1e5, or Q and K of magnitudes 1e5 and 1e-5, give 2e-4 .. 5e-4 relative (plain TF32 grade)
// instead of 5e-7; magnitudes from 1e-4 to 1e2 stay at 5e-7.  The split-TF32 kernel
// (attn_fwd_tc.cu) has the full fp32 range and is what callers with such operands select.
//
// One block = 128 query rows of one (batch, head): 128 workers (worker = row = TMEM lane), one
// issuing warp, one warp that stages K and one that stages V.  Two blocks per SM at head_dim 32,
// one at head_dim 64 (the sizes below are those of head_dim 32).
//   TMEM (256 columns): X0, X1 (64 each): S(t), overwritten in place by P_hi(t);  L0, L1 (32
//   each): P_lo(t) as packed fp16;  O_ext (64): [P_hi V_hi | P_hi V_lo + P_lo V], accumulated over
//   ALL tiles.  Workers never read O_ext back per tile: the running maximum is only moved (and O_ext
//   rescaled, by the whole warp) when a row's maximum grew by more than 2^8 since the last rescale.
//   With P double-buffered, the worker goes from tile t straight to tile t+1 while P V(t) runs.
//   A worker reads its 64 scores from TMEM once; maximum, exponentials and the hi / lo cut all
//   work on those registers.
//   Shared memory: Q_hi (fp32) and [Q_lo | Q] (fp16); two stages of K (raw fp32 = the TF32
//   operand, since the tensor core ignores the 13 low mantissa bits) and [K_hi | K_lo] (fp16); two
//   stages of V (raw fp32, N-major), V_lo (fp32, N-major) and an fp16 copy of V (N-major, no swizzle).
//   The K and V warps copy a tile with cp.async straight into its operand place, then read their
//   own pieces back to derive the fp16 copies and V_lo.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per block
constexpr int kKeys = 64;         // keys per tile
constexpr int kWorkers = kRows;
constexpr float kRescaleStep = 8.0f;
constexpr uint32_t kColX = 0, kColL = 128, kColO = 192;

// Sizes that depend on head_dim.  An operand row is cut into blocks of 128 bytes (32 floats or 64
// fp16 values); a block of a tile is [rows][128 bytes], 128-byte swizzled.
template <int D>
struct Tc16Cfg {
    static constexpr int DB = D / 32;                         // fp32 blocks per row
    static constexpr int HB = (2 * D) / 64;                   // fp16 blocks per row of [x_lo | x] or [x_hi | x_lo]
    static constexpr int PPR = D / 8;                         // 32-byte pieces per row
    static constexpr int PWK = D / 32;                        // warps that stage K
    static constexpr int PWV = D / 16;                        // warps that stage V (its conversion is the longer one)
    static constexpr int THREADS = kWorkers + 32 + (PWK + PWV) * 32;   // workers, the issuing warp, the K warps, the V warps
    static constexpr uint32_t kTmemCols = (kColO + 2 * D) <= 256 ? 256 : 512;
    static constexpr int BLOCKS_PER_SM = kTmemCols == 256 ? 2 : 1;
    static constexpr int kQBlk = kRows * 128, kKBlk = kKeys * 128;      // bytes of one block of a Q / K / V tile
    static constexpr int kQhiBytes = DB * kQBlk, kQ16Bytes = HB * kQBlk;
    static constexpr int kKhiBytes = DB * kKBlk, kK16Bytes = HB * kKBlk, kKStage = kKhiBytes + kK16Bytes;
    static constexpr int kVhlBytes = 2 * DB * kKBlk, kV16Bytes = kKeys * D * 2, kVStage = kVhlBytes + kV16Bytes;
    static constexpr size_t kSmemBytes = (size_t)kQhiBytes + kQ16Bytes + 2 * kKStage + 2 * kVStage;
};

__device__ int g_tc16_status = 0;
__device__ int g_tc16_notice = 0;                // bit 0: an operand left the range in which the fp16 correction terms are exact

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

// Which pieces of a 64-row tile a staging thread owns.  A piece is 32 bytes (8 floats) of a row; a
// thread owns pieces of pairs of adjacent rows.  PT = threads that stage this operand, PPR = pieces per row.
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
mha_tc16_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
                float *__restrict__ O, float *__restrict__ P, int S, int E, int H, int BH, int nqblk, float qscale)
{
    using C = Tc16Cfg<D>;
    constexpr int DB = C::DB, HB = C::HB, PPR = C::PPR, PWK = C::PWK, PWV = C::PWV;
    constexpr int kQBlk = C::kQBlk, kKBlk = C::kKBlk, kKStage = C::kKStage, kVStage = C::kVStage;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_hi = base;                            // fp32 [DB][128][32], K-major
    uint8_t *q_16 = q_hi + C::kQhiBytes;             // fp16 [HB][128][64]: a row is [Q_lo (D) | Q (D)], K-major
    uint8_t *k_st = q_16 + C::kQ16Bytes;             // per stage: K fp32 [DB][64][32], then fp16 [HB][64][64]: [K_hi (D) | K_lo (D)]
    uint8_t *v_st = k_st + 2 * kKStage;              // per stage: fp32 N-major [V blocks | V_lo blocks], then the fp16 copy of V
    __shared__ uint64_t k_full[2], v_full[2], s_full[2], p_full[2], o_done[2];
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
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], PWK);              // one arrival per K warp
            mbar_init(&v_full[i], PWV);              // one arrival per V warp
            mbar_init(&s_full[i], 1);                // tcgen05.commit after Q K^T: S is ready, and the K stage is free
            mbar_init(&p_full[i], kWorkers / 32);    // one arrival per worker warp
            mbar_init(&o_done[i], 1);                // tcgen05.commit after P V: O is up to date, and the V stage is free;
                                                     // by tile parity: a worker may be two tiles ahead of the P V products
        }
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K staged,
    // 5 P written, 6 V staged, 7 K stage free, 8 V stage free
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) { abort_flag = 1; atomicCAS(&g_tc16_status, 0, site); }
    };
    // one arrival for the whole warp: every lane's writes are ordered before it by the warp barrier
    auto arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
    };
    // byte offset, inside an fp16 operand of rows [lo (D) | hi (D)], of the 16-byte chunk holding values
    // 8 e8 .. 8 e8 + 7 of row r; blk = bytes of one 128-byte-row block of that operand
    auto off16 = [](int r, int e8, int blk) { return (e8 >> 3) * blk + sw128(r, e8 & 7); };

    if (warp == kWorkers / 32) {
        // ================= the issuing warp =====================================================
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncthreads();                             // Q staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        // The warp stays converged and elects the issuing lane per instruction: descriptors are then computed
        // warp-uniformly (uniform registers), which roughly halves what an instruction costs its issuer.
        {
            constexpr uint32_t id_qk_h = idesc_f16(kRows, kKeys);            // [Q_lo | Q] x [K_hi | K_lo], fp16
            constexpr uint32_t id_qk_t = make_idesc(kRows, kKeys, 0);        // Q_hi x K_hi, tf32
            constexpr uint32_t id_pv_t = make_idesc(kRows, 2 * D, 1);        // P_hi x [V_hi | V_lo], tf32, B N-major
            constexpr uint32_t id_pv_h = idesc_f16(kRows, D) | (1u << 16);   // P_lo x V (fp16 copy), B N-major
            auto issue_qk = [&](int buf, int stage) {
                const uint32_t d = tmem + kColX + buf * kKeys;
                // the correction terms first: the accumulator is still tiny while they are added
#pragma unroll
                for (int hb = 0; hb < HB; ++hb) {
                    const uint64_t dq = make_desc(smem_u32(q_16 + hb * kQBlk), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(k_st + stage * kKStage + C::kKhiBytes + hb * kKBlk), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k)      // 16 fp16 = 32 bytes per instruction
                        if (elect_one()) mma_h_ss(d, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), id_qk_h, (hb | k) ? 1u : 0u);
                }
#pragma unroll
                for (int db = 0; db < DB; ++db) {
                    const uint64_t dq = make_desc(smem_u32(q_hi + db * kQBlk), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(k_st + stage * kKStage + db * kKBlk), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k)      // 8 floats = 32 bytes per instruction
                        if (elect_one()) mma_ss(d, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), id_qk_t, 1);
                }
                if (elect_one()) tc_commit(&s_full[buf]);             // also tells the K warp that this stage (same parity as buf) is free
            };
            auto issue_pv = [&](int buf, int stage, bool first) {
                // fp32 N-major B: 8 keys of 128 bytes per instruction; lbo = bytes between 32-column blocks
                // (V blocks, then V_lo blocks: one operand of 2D columns)
                const uint64_t dv = make_desc(smem_u32(v_st + stage * kVStage), kKBlk, 512, 1);
                // fp16 copy, no swizzle, N-major: lbo = bytes between groups of 8 keys, sbo = bytes between blocks of 8 columns
                const uint64_t dvt = make_desc(smem_u32(v_st + stage * kVStage + C::kVhlBytes), D * 16, 128, 0);
#pragma unroll
                for (int k = 0; k < kKeys / 8; ++k)
                    if (elect_one()) mma_ts(tmem + kColO, tmem + kColX + buf * kKeys + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), id_pv_t, (first && k == 0) ? 0u : 1u);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)  // 16 keys = 8 TMEM columns of packed fp16 = two key groups of the fp16 V
                    if (elect_one()) mma_h_ts(tmem + kColO + D, tmem + kColL + buf * 32 + (uint32_t)(k * 8), dvt + (uint64_t)(k * 2 * D), id_pv_h, 1);
                if (elect_one()) tc_commit(&o_done[buf]);             // also tells the V warp that this stage is free
            };
            wait(&k_full[0], 0, 4);
            tc_fence_after();
            issue_qk(0, 0);
            for (int t = 0; t < nt; ++t) {
                const int st = t & 1;
                if (t + 1 < nt) {
                    wait(&k_full[st ^ 1], (uint32_t)(((t + 1) >> 1) & 1), 4);    // K(t+1) is in shared memory
                    tc_fence_after();
                    issue_qk(st ^ 1, st ^ 1);        // its buffer held P(t-1): P V(t-1) was issued before, instructions run in order
                }
                wait(&p_full[st], (uint32_t)((t >> 1) & 1), 5);                  // P(t) is in TMEM
                wait(&v_full[st], (uint32_t)((t >> 1) & 1), 6);                  // V(t) is in shared memory
                tc_fence_after();
                issue_pv(st, st, t == 0);
            }
            if (PROBS) {
                // X[u & 1] held P(u-2) (consumed by P V(u-2), issued before) or, from the third tile of
                // this sweep on, S(u-2), which the workers must have read
                for (int u = nt; u < nk; ++u) {
                    const int bf = u & 1;
                    wait(&k_full[bf], (uint32_t)((u >> 1) & 1), 4);
                    if (u - 2 >= nt) wait(&p_full[bf], (uint32_t)(((u - 2) >> 1) & 1), 5);
                    tc_fence_after();
                    issue_qk(bf, bf);
                }
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                             // the workers have read the output
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
        return;
    }

    // ================= the producers: D/32 warps for K, D/16 for V ===================================
    // A tile goes from global memory straight to its place in the TF32 operand (cp.async, no
    // registers held): the tensor core ignores the 13 low mantissa bits of a TF32 operand, so the
    // raw fp32 tile IS the hi operand.  When it has landed the same thread reads its pieces back,
    // derives the fp16 copies (and V_lo) and publishes the stage.  The copy of tile u+1 is issued
    // before tile u is converted, as soon as its stage is free.
    // A thread owns 32-byte pieces (8 floats) of pairs of adjacent rows, eight per tile: an fp16 chunk
    // is 16 bytes = 8 values.
    // byte offset of 16-byte chunk c of row r in a block of the N-major fp32 operand (32-byte pieces permuted by r mod 4)
    auto nmaj = [](int r, int c) { return r * 128 + (((((c >> 1) ^ (r & 3)) << 1) | (c & 1)) << 4); };
    if (warp > kWorkers / 32 && warp <= kWorkers / 32 + PWK) {
        const PieceMap<32 * PWK, PPR> pm(tid - kWorkers - 32);
        constexpr int NPC = pm.NPC, BATCH = pm.BATCH;
        const int pc = pm.pc, pblk = pm.pblk, pch = pm.pch;
        auto piece_row = [&](int p) { return pm.row(p); };
        auto copy_k = [&](int t, int stage) {
            uint8_t *khi = k_st + stage * kKStage + pblk * kKBlk;
#pragma unroll
            for (int p = 0; p < NPC; ++p) {
                const int r = piece_row(p), j = t * kKeys + r;
                const bool ok = j < S;
                const float *src = K + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + 8 * pc;
                cp_async16(khi + sw128(r, pch), src, ok);
                cp_async16(khi + sw128(r, pch + 1), src + 4, ok);
            }
            cp_async_commit();
        };
        float amax = 0.0f;
        auto convert_k = [&](int stage) {
            uint8_t *khi = k_st + stage * kKStage + pblk * kKBlk, *k16 = k_st + stage * kKStage + C::kKhiBytes;
#pragma unroll
            for (int half = 0; half < NPC / BATCH; ++half) {
                float4 a[BATCH], c[BATCH];           // all loads first: the stores below may alias them for the compiler
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = piece_row(half * BATCH + i);
                    a[i] = *reinterpret_cast<const float4 *>(khi + sw128(r, pch));
                    c[i] = *reinterpret_cast<const float4 *>(khi + sw128(r, pch + 1));
                }
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = piece_row(half * BATCH + i);
                    const float4 ah = hi4(a[i]), ch = hi4(c[i]);
                    amax = amax8(amax, a[i], c[i]);
                    *reinterpret_cast<uint4 *>(k16 + off16(r, pc, kKBlk)) =
                        make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
                    *reinterpret_cast<uint4 *>(k16 + off16(r, PPR + pc, kKBlk)) =
                        make_uint4(pack_f16(a[i].x - ah.x, a[i].y - ah.y), pack_f16(a[i].z - ah.z, a[i].w - ah.w),
                                   pack_f16(c[i].x - ch.x, c[i].y - ch.y), pack_f16(c[i].z - ch.z, c[i].w - ch.w));
                }
            }
        };
        copy_k(0, 0);
        __syncthreads();                             // matches the block-wide barrier after Q staging
        for (int u = 0; u < nk; ++u) {
            const int st = u & 1;
            if (u + 1 < nk) {
                if (u >= 1) wait(&s_full[st ^ 1], (uint32_t)(((u - 1) >> 1) & 1), 7);   // Q K(u-1)^T has completed
                copy_k(u + 1 < nt ? u + 1 : u + 1 - nt, st ^ 1);
            } else {
                cp_async_commit();                   // keeps the group count of the wait below
            }
            cp_async_wait_1();                       // K(u) has landed
            convert_k(st);
            proxy_fence();                           // generic-proxy writes -> visible to the tensor core
            arrive(&k_full[st]);
        }
        publish_amax(&s_amax[1], amax);
        cp_async_wait_all();
        __syncthreads();
        return;
    }
    if (warp > kWorkers / 32 + PWK) {
        const PieceMap<32 * PWV, PPR> pm(tid - kWorkers - 32 - 32 * PWK);
        constexpr int NPC = pm.NPC, BATCH = pm.BATCH;
        const int pc = pm.pc, pblk = pm.pblk, pch = pm.pch;
        auto piece_row = [&](int p) { return pm.row(p); };
        auto copy_v = [&](int t, int stage) {
            uint8_t *vhi = v_st + stage * kVStage + pblk * kKBlk;
#pragma unroll
            for (int p = 0; p < NPC; ++p) {
                const int r = piece_row(p), j = t * kKeys + r;
                const bool ok = j < S;
                const float *src = V + (tok0 + (ok ? j : 0)) * (size_t)E + hcol + 8 * pc;
                cp_async16(vhi + nmaj(r, pch), src, ok);
                cp_async16(vhi + nmaj(r, pch + 1), src + 4, ok);
            }
            cp_async_commit();
        };
        float amax = 0.0f;
        auto convert_v = [&](int stage) {
            uint8_t *vhi = v_st + stage * kVStage + pblk * kKBlk, *vlo = vhi + DB * kKBlk, *v16 = v_st + stage * kVStage + C::kVhlBytes;
#pragma unroll
            for (int half = 0; half < NPC / BATCH; ++half) {
                float4 a[BATCH], c[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = piece_row(half * BATCH + i);
                    a[i] = *reinterpret_cast<const float4 *>(vhi + nmaj(r, pch));
                    c[i] = *reinterpret_cast<const float4 *>(vhi + nmaj(r, pch + 1));
                }
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int r = piece_row(half * BATCH + i);
                    const float4 ah = hi4(a[i]), ch = hi4(c[i]);
                    amax = amax8(amax, a[i], c[i]);
                    *reinterpret_cast<float4 *>(vlo + nmaj(r, pch)) = make_float4(a[i].x - ah.x, a[i].y - ah.y, a[i].z - ah.z, a[i].w - ah.w);
                    *reinterpret_cast<float4 *>(vlo + nmaj(r, pch + 1)) = make_float4(c[i].x - ch.x, c[i].y - ch.y, c[i].z - ch.z, c[i].w - ch.w);
                    // fp16 copy, N-major without swizzle: 8 keys x 8 columns form one 128-byte core matrix (key i of
                    // the group at 16 i); column blocks 128 bytes apart, key groups D/8 such blocks apart
                    *reinterpret_cast<uint4 *>(v16 + (r >> 3) * (D * 16) + pc * 128 + (r & 7) * 16) =
                        make_uint4(pack_f16(a[i].x, a[i].y), pack_f16(a[i].z, a[i].w), pack_f16(c[i].x, c[i].y), pack_f16(c[i].z, c[i].w));
                }
            }
        };
        copy_v(0, 0);
        __syncthreads();
        for (int u = 0; u < nt; ++u) {
            const int st = u & 1;
            cp_async_wait_all();                     // V(u) has landed
            convert_v(st);
            proxy_fence();
            arrive(&v_full[st]);
            if (u + 1 < nt) {
                // the stage of V(u+1) held V(u-1); V(u) is published before this warp waits for that product
                if (u >= 1) wait(&o_done[st ^ 1], (uint32_t)(((u - 1) >> 1) & 1), 8);   // P V(u-1) has completed
                copy_v(u + 1, st ^ 1);
            }
        }
        publish_amax(&s_amax[2], amax);
        cp_async_wait_all();
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
            uint8_t *qb = q_hi + (j >> 2) * kQBlk;
            *reinterpret_cast<float4 *>(qb + sw128(rloc, 2 * (j & 3))) = ah;
            *reinterpret_cast<float4 *>(qb + sw128(rloc, 2 * (j & 3) + 1)) = ch;
            *reinterpret_cast<uint4 *>(q_16 + off16(rloc, j, kQBlk)) =
                make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                           pack_f16(c.x - ch.x, c.y - ch.y), pack_f16(c.z - ch.z, c.w - ch.w));
            *reinterpret_cast<uint4 *>(q_16 + off16(rloc, PPR + j, kQBlk)) =
                make_uint4(pack_f16(a.x, a.y), pack_f16(a.z, a.w), pack_f16(c.x, c.y), pack_f16(c.z, c.w));
        }
        publish_amax(&s_amax[0], amax);
    }
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (log2 domain) and row sum
    for (int t = 0; t < nt; ++t) {
        const int buf = t & 1;
        const int j0 = t * kKeys;
        const uint32_t s_addr = lane_base + kColX + buf * kKeys, l_addr = lane_base + kColL + buf * 32;
        wait(&s_full[buf], (uint32_t)((t >> 1) & 1), 1);   // S(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + wq * 32;              // first row of this warp
        const bool warp_dead = CAUSAL && j0 > wrow0 + 31;          // these columns are above the diagonal for the whole warp
        const bool need_mask = (CAUSAL && j0 + kKeys - 1 > wrow0) || j0 + kKeys > S;
        const int nvalid = min(S - j0, CAUSAL ? row - j0 + 1 : kKeys);     // visible columns of this row

        // ---- the row's 64 scores are read from TMEM once and stay in registers --------------------
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
                wait(&o_done[(t - 1) & 1], (uint32_t)(((t - 1) >> 1) & 1), 2);   // P V(t-1) has completed
                tc_fence_after();
#pragma unroll
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

        // ---- exponentials; P_hi over S in place, P_lo as packed fp16 ---------------------------------
        float psum = 0.0f;
        if (warp_dead) {
            float z[16];
            uint32_t zz[8];
#pragma unroll
            for (int c = 0; c < 16; ++c) z[c] = 0.0f;
#pragma unroll
            for (int c = 0; c < 8; ++c) zz[c] = 0u;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                tmem_st16(s_addr + k * 16, z);
                tmem_st8_u32(l_addr + k * 8, zz);
            }
        } else {
            float ps4[4] = {0.0f, 0.0f, 0.0f, 0.0f};    // four summation chains
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float hi[16];
                uint32_t pk[8];
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                    const float s0 = (k < 2) ? v0[(k & 1) * 16 + c] : v1[(k & 1) * 16 + c];
                    const float s1 = (k < 2) ? v0[(k & 1) * 16 + c + 1] : v1[(k & 1) * 16 + c + 1];
                    const float p0 = ex2_approx(s0 - m_ref), p1 = ex2_approx(s1 - m_ref);
                    ps4[c & 3] += p0;
                    ps4[(c + 1) & 3] += p1;
                    hi[c] = tf32_hi(p0);
                    hi[c + 1] = tf32_hi(p1);
                    pk[c >> 1] = pack_f16(p0 - hi[c], p1 - hi[c + 1]);
                }
                tmem_st16(s_addr + k * 16, hi);
                tmem_st8_u32(l_addr + k * 8, pk);
            }
            psum = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        }
        l += psum;
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[buf]);
    }

    {
        wait(&o_done[(nt - 1) & 1], (uint32_t)(((nt - 1) >> 1) & 1), 3);
        tc_fence_after();
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        const bool store = !abort_flag && row < S;
        float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + (row < S ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int hh = 0; hh < D / 32; ++hh) {
            float a[32], c2[32];
            tmem_ld32(o_addr + hh * 32, a);              // P_hi V_hi
            tmem_ld32(o_addr + D + hh * 32, c2);         // the correction terms
            tmem_wait_ld();
            if (store) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    dst[hh * 8 + c] = make_float4((a[c * 4 + 0] + c2[c * 4 + 0]) * inv, (a[c * 4 + 1] + c2[c * 4 + 1]) * inv,
                                                  (a[c * 4 + 2] + c2[c * 4 + 2]) * inv, (a[c * 4 + 3] + c2[c * 4 + 3]) * inv);
            }
        }
        if (PROBS) {
            // ---- second sweep: p = 2^(s - m_ref) / l for every key of the row, zeros where masked -----
            // A worker holds one row, so its own stores would be 16-byte pieces S floats apart.  The warp
            // turns its 32 x 64 tile through shared memory instead (the V stages are free: the last P V
            // product has completed) and stores two rows of 256 contiguous bytes per instruction.
            uint8_t *tb = v_st + wq * (32 * kKeys * 4);  // 16-byte chunk c of row r at r * 256 + ((c ^ (r & 7)) << 4)
            const int wrow0 = q0 + wq * 32;              // first row of this warp
            float *pwarp = P + ((size_t)bh * S + wrow0) * (size_t)S;
            const bool vec = (S & 3) == 0;               // then every 4-column group of a row is 16-byte aligned
            for (int u = nt; u < nk; ++u) {
                const int buf = u & 1, j0 = (u - nt) * kKeys;
                const uint32_t s_addr = lane_base + kColX + buf * kKeys;
                wait(&s_full[buf], (uint32_t)((u >> 1) & 1), 1);
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
                        o[i] = c < nvalid ? ex2_approx(sc - m_ref) * inv : 0.0f;
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
        // Range of the fp16 copies: beyond fp16's largest number a correction term saturates; below its smallest
        // normal numbers it is flushed, an absolute error of up to 2^-25 per fp16 value, which matters when it is
        // neither small in itself nor small beside the scores it is added to.  (Q carries the softmax scale here.)
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
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kRows - 1) / kRows;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, C::THREADS, smem, st>>>(q, k, v, out, probs, S, E, H, B * H, nqblk, qscale);
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
