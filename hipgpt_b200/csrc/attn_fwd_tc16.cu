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
// Range: the whole fp32 range.  Every fp16 piece is formed from a copy of the operand scaled by a power of two (exact)
// that brings the largest magnitude of its unit into [2^14, 2^15): per query row for Q, per 64-key tile for K and for V.
// The factors leave again where they cost nothing: Q's and K's inside the multiply-add that forms the exponent, V's
// tile factor (relative to the head's) as a power of two folded into P, the head's with the final division.  The
// accuracy notice is therefore never raised by this kernel.
//
// Two kernels.  kv_pack_kernel cuts K and V into their fp16 pieces once per call and writes them, tile by tile, as
// the exact shared-memory images of the operand stages (K: rows of [K_hi | K_lo], K-major, 128-byte swizzle; V:
// [V_hi | V_lo], N-major) into a scratch buffer of the library: a 64-key tile is needed by every block of query rows
// of its head (8 at S = 1024, 16 at S = 2048), and converting it in each of them was measured to be what paced the
// attention kernel (no conversion: 1.4 x faster).  mha_tc16_kernel then fetches a stage with one bulk copy.
// One block = 128 query rows of one (batch, head); two blocks per SM.
//   Copies: one lane of an issuing warp asks for a whole operand stage (cp.async.bulk, completion counted on an
//   mbarrier); a stage is refilled once the product that read it has completed (tcgen05.commit barriers).
//   TMEM (256 columns): X0, X1 (64 each): S(t), overwritten in place by P(t);  O (2 D): [P_hi V_hi | P_hi V_lo + P_lo V_hi],
//   accumulated over ALL tiles.  Workers (thread = query row = TMEM lane) never read O back per tile: the reference
//   maximum only moves (and O is rescaled, by the whole warp) when a row's maximum grew by more than 2^8.
//   With P double-buffered, the worker goes from tile t straight to tile t+1 while P V(t) runs.  It reads a tile's
//   scores from TMEM once and keeps them in registers for the maximum and for the exponentials; additions and
//   multiply-adds work on pairs of values per instruction (the sweeps are bound by the instructions they issue).
//   A warp stages its 32 query rows with whole-line reads (D / 4 lanes per row), all in flight at once.
// Every wait is bounded: on expiry the block raises a flag that cuts all later waits short,
// records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <math.h>
#include <stdlib.h>

#include <mutex>
#include <vector>

namespace hipgpt {
namespace {

constexpr int kRows = 128;        // query rows per block
constexpr int kKeys = 64;         // keys per tile
constexpr int kWorkers = kRows;
constexpr float kRescaleStep = 8.0f;
constexpr float kPShift = 6.0f;   // P carries a factor 2^6: with the lazy reference maximum it stays below 2^15
constexpr int kBufs = 2;          // S / P buffers in TMEM
constexpr uint32_t kColX = 0, kColO = kBufs * kKeys, kTmemCols = 256;
constexpr int kPackThreads = 128;

// Sizes that depend on head_dim.  An operand row is cut into blocks of 128 bytes (32 floats or 64
// fp16 values); a block of a tile is [rows][128 bytes], 128-byte swizzled.
template <int D>
struct Tc16Cfg {
    static constexpr int HB = (2 * D) / 64;                   // fp16 blocks per row of [x_hi | x_lo]
    static constexpr int PPR = D / 8;                         // 32-byte pieces (8 floats) per row
    static constexpr int KST = D == 64 ? 2 : 3;               // operand stages of K
    static constexpr int VST = D == 64 ? 2 : 4;               // ... of V (the second sweep stages 32 KB of probabilities there)
    static constexpr int THREADS = kWorkers + 64;             // workers and the two issuing warps
    static constexpr int BLOCKS_PER_SM = 2;
    static constexpr int kQBlk = kRows * 128, kKBlk = kKeys * 128;      // bytes of one block of a Q / K tile
    static constexpr int kQ16Bytes = HB * kQBlk;
    static constexpr int kK16Stage = HB * kKBlk;              // [K_hi | K_lo] rows
    static constexpr int kV16Stage = kKeys * 2 * D * 2;       // [V_hi | V_lo], N-major without swizzle
    static constexpr size_t kSmemBytes = (size_t)kQ16Bytes + KST * kK16Stage + VST * kV16Stage;
    static_assert(VST * kV16Stage >= 4 * 32 * kKeys * 4, "the second sweep's staging area");
};

__device__ int g_tc16_status = 0;
__device__ int g_tc16_notice = 0;                // never raised by this kernel: its operands are scaled into fp16's range

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
    for (int j = 0; j < 32; j += 8) {
        m4[0] = max3(m4[0], v[j], v[j + 1]); m4[1] = max3(m4[1], v[j + 2], v[j + 3]);
        m4[2] = max3(m4[2], v[j + 4], v[j + 5]); m4[3] = max3(m4[3], v[j + 6], v[j + 7]);
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// One chunk of scores (log2 domain, times 1 / sfac; hidden ones are -inf: their exponential is exactly 0) -> P = 2^(s sfac + nm),
// cut into fp16 hi and lo, written over the chunk's own 32 TMEM columns (16 of packed P_hi, then 16 of packed P_lo).
// Returns the sum of P.
__device__ __forceinline__ float chunk_exp(const float (&v)[32], uint32_t addr, float sfac, float nm)
{
    float2 ps[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
    const float2 sf2 = make_float2(sfac, sfac), nm2 = make_float2(nm, nm);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const float2 x = ffma2(make_float2(v[16 * half + j], v[16 * half + j + 1]), sf2, nm2);
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

__device__ __forceinline__ void tmem_zero32(uint32_t addr)
{
    uint32_t z[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) z[j] = 0u;
    tmem_st16_u32(addr, z);
    tmem_st16_u32(addr + 16, z);
}

// The power of two that brings a largest magnitude `amax` into [2^14, 2^15): fp16 then holds the 11 leading bits of
// every value that matters beside the largest one.  1 for zero, infinite or NaN input.
__device__ __forceinline__ float range_scale(float amax)
{
    if (!(amax > 0.0f && amax <= 3.0e38f)) return 1.0f;
    const int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
    int sh = 14 - e;
    sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
    return __uint_as_float((uint32_t)(127 + sh) << 23);
}

// log2 of a positive power of two (its exponent field)
__device__ __forceinline__ float log2_of_pow2(float p) { return (float)((int)((__float_as_uint(p) >> 23) & 0xffu) - 127); }

// ---- the pack kernel: K and V of one (batch, head, 64-key tile) -> the fp16 images of their operand stages ----
// Thread pid owns 32-byte pieces (8 floats): piece pid % PPR of rows pid / PPR, + 128 / PPR, ...  A warp reads whole
// rows (coalesced) and writes 16-byte chunks that fill whole 128-byte lines of the image.
// Every tile is scaled by a power of two of its own (range_scale of the tile's largest magnitude), so that no operand
// magnitude costs accuracy: the block holds its pieces in registers, finds the two maxima, converts.  The maxima go to
// tmax[0][tile] (K) and tmax[1][tile] (V): the attention kernel takes the factors out again.
// K image: [HB blocks][64 rows][128 bytes], a row of block j holds values 64 j .. 64 j + 63 of [K_hi (D) | K_lo (D)],
// 16-byte chunks swizzled by the row (the layout a K-major, 128-byte-swizzled operand has in shared memory).
// V image: key r, column block cb (8 columns of [V_hi (D) | V_lo (D)]) at (r / 8) * 32 D + cb * 128 + (r % 8) * 16:
// 8 keys x 8 columns form one 128-byte core matrix of an N-major operand without swizzle.  Keys past S are zeros.
template <int D>
__global__ void __launch_bounds__(kPackThreads)
kv_pack_kernel(const float *__restrict__ K, const float *__restrict__ V, float *__restrict__ tmax,
               uint8_t *__restrict__ kimg, uint8_t *__restrict__ vimg, int S, int E, int H, int ntk, int ntiles)
{
    using C = Tc16Cfg<D>;
    constexpr int PPR = C::PPR, RPT = kPackThreads / PPR, NP = kKeys / RPT;      // rows covered per pass, pieces per thread
    __shared__ float red[2][kPackThreads / 32];
    dependents_may_start();                          // the attention kernel's blocks may come in as this grid's blocks leave
    const int kt = blockIdx.x, bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int pid = threadIdx.x, pc = pid % PPR, r0 = pid / PPR;
    const size_t tile = (size_t)bh * ntk + kt;
    uint8_t *kout = kimg + tile * C::kK16Stage, *vout = vimg + tile * C::kV16Stage;
    float4 ka[NP], kc[NP], va[NP], vc[NP];
    float mk = 0.0f, mv = 0.0f;
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int j = kt * kKeys + r0 + i * RPT;
        const bool ok = j < S;
        const size_t off = ((size_t)b * S + (ok ? j : 0)) * (size_t)E + (size_t)h * D + 8 * pc;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        ka[i] = ok ? __ldg(reinterpret_cast<const float4 *>(K + off)) : z;
        kc[i] = ok ? __ldg(reinterpret_cast<const float4 *>(K + off) + 1) : z;
        va[i] = ok ? __ldg(reinterpret_cast<const float4 *>(V + off)) : z;
        vc[i] = ok ? __ldg(reinterpret_cast<const float4 *>(V + off) + 1) : z;
        mk = fmaxf(mk, fmaxf(fmaxf(fmaxf(fabsf(ka[i].x), fabsf(ka[i].y)), fmaxf(fabsf(ka[i].z), fabsf(ka[i].w))),
                             fmaxf(fmaxf(fabsf(kc[i].x), fabsf(kc[i].y)), fmaxf(fabsf(kc[i].z), fabsf(kc[i].w)))));
        mv = fmaxf(mv, fmaxf(fmaxf(fmaxf(fabsf(va[i].x), fabsf(va[i].y)), fmaxf(fabsf(va[i].z), fabsf(va[i].w))),
                             fmaxf(fmaxf(fabsf(vc[i].x), fabsf(vc[i].y)), fmaxf(fabsf(vc[i].z), fabsf(vc[i].w)))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
    if ((pid & 31) == 0) { red[0][pid >> 5] = mk; red[1][pid >> 5] = mv; }
    __syncthreads();
    mk = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    mv = fmaxf(fmaxf(red[1][0], red[1][1]), fmaxf(red[1][2], red[1][3]));
    if (pid == 0) {
        tmax[tile] = mk;
        tmax[ntiles + tile] = mv;
    }
    const float sk = range_scale(mk), sv = range_scale(mv);
#pragma unroll
    for (int i = 0; i < NP; ++i) {
        const int r = r0 + i * RPT;
        float4 a = ka[i], c = kc[i];
        a.x *= sk; a.y *= sk; a.z *= sk; a.w *= sk; c.x *= sk; c.y *= sk; c.z *= sk; c.w *= sk;
        {
            const float4 ah = hi4(a), ch = hi4(c);
            // values 8 pc .. of the hi half, 8 (PPR + pc) .. of the lo half of the row
            *reinterpret_cast<uint4 *>(kout + (pc >> 3) * C::kKBlk + sw128(r, pc & 7)) =
                make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
            *reinterpret_cast<uint4 *>(kout + ((PPR + pc) >> 3) * C::kKBlk + sw128(r, (PPR + pc) & 7)) =
                make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                           pack_f16(c.x - ch.x, c.y - ch.y), pack_f16(c.z - ch.z, c.w - ch.w));
        }
        a = va[i]; c = vc[i];
        a.x *= sv; a.y *= sv; a.z *= sv; a.w *= sv; c.x *= sv; c.y *= sv; c.z *= sv; c.w *= sv;
        {
            const float4 ah = hi4(a), ch = hi4(c);
            uint8_t *dst = vout + (r >> 3) * (32 * D) + (r & 7) * 16;
            *reinterpret_cast<uint4 *>(dst + pc * 128) =
                make_uint4(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w), pack_f16(ch.x, ch.y), pack_f16(ch.z, ch.w));
            *reinterpret_cast<uint4 *>(dst + (PPR + pc) * 128) =
                make_uint4(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w),
                           pack_f16(c.x - ch.x, c.y - ch.y), pack_f16(c.z - ch.z, c.w - ch.w));
        }
    }
}

template <int D, bool CAUSAL, bool PROBS>
__global__ void __launch_bounds__(Tc16Cfg<D>::THREADS, Tc16Cfg<D>::BLOCKS_PER_SM)
mha_tc16_kernel(const uint8_t *__restrict__ kimg, const uint8_t *__restrict__ vimg, const float *__restrict__ tmax, int ntiles, const float *__restrict__ Q,
                float *__restrict__ O, float *__restrict__ P, int S, int E, int H, int BH, int nqblk, int ntk, float qscale)
{
    using C = Tc16Cfg<D>;
    constexpr int PPR = C::PPR, KST = C::KST, VST = C::VST;
    constexpr int kQBlk = C::kQBlk, kKBlk = C::kKBlk;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *q_16 = base;                                    // fp16 [HB][128][64]: a row is [Q_hi (D) | Q_lo (D)], K-major
    uint8_t *k_16 = q_16 + C::kQ16Bytes;                     // per stage: fp16 [HB][64][64]: [K_hi (D) | K_lo (D)]
    uint8_t *v_16 = k_16 + KST * C::kK16Stage;               // per stage: [V_hi | V_lo] fp16, N-major
    __shared__ uint64_t k_full[KST], v_full[VST], s_full[KST], o_done[VST], p_full[kBufs];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float q_sfac[kRows];                  // per query row: one over the power of two that its staged copy carries

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
        for (int i = 0; i < KST; ++i) {
            mbar_init(&k_full[i], 1);                // the copy of a stage: one announcement, then its bytes
            mbar_init(&s_full[i], 1);                // tcgen05.commit after Q K(t)^T, t mod KST = i: S is ready, and the K stage is free
        }
        for (int i = 0; i < VST; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&o_done[i], 1);                // tcgen05.commit after P V(t): O is up to date, and the V stage is free
        }
        for (int i = 0; i < kBufs; ++i) mbar_init(&p_full[i], kWorkers / 32);    // one arrival per worker warp
    }
    __syncthreads();

    // site codes in the status word: 1 S ready, 2 O complete (rescale), 3 O complete (end), 4 K stage landed,
    // 5 P written, 6 V stage landed, 7 K stage free, 8 V stage free
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
    // phase parity of tile t on a barrier that is indexed by tile mod n
    auto phn = [](int t, int n) { return (uint32_t)((t / n) & 1); };

    if (warp == kWorkers / 32 || warp == kWorkers / 32 + 1) {
        // ================= the two issuing warps =================================================
        // One fetches the K stages and issues every Q K^T, the other fetches the V stages and issues every P V: an
        // instruction costs the warp that issues it 60 - 100 cycles, more than it costs the tensor pipe, and two warps
        // issue side by side.  Each accumulator is written by one warp, in tile order; what one warp's products need
        // from the other's is ordered by the tcgen05.commit barriers.  The warps stay converged and elect the issuing
        // lane per instruction (descriptors are then computed warp-uniformly, in uniform registers).
        const bool qk_role = warp == kWorkers / 32;
        if (qk_role) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        // one lane asks for a whole packed stage (u counts staged K tiles: the second sweep reads the tiles again)
        auto copy_k = [&](int u) {
            if (lane == 0 && u < nk) {
                const int kt = u < nt ? u : u - nt;
                mbar_arrive_expect_tx(&k_full[u % KST], (uint32_t)C::kK16Stage);
                bulk_load(k_16 + (u % KST) * C::kK16Stage, kimg + ((size_t)bh * ntk + kt) * C::kK16Stage, (uint32_t)C::kK16Stage, &k_full[u % KST]);
            }
            __syncwarp();
        };
        auto copy_v = [&](int u) {
            if (lane == 0 && u < nt) {
                mbar_arrive_expect_tx(&v_full[u % VST], (uint32_t)C::kV16Stage);
                bulk_load(v_16 + (u % VST) * C::kV16Stage, vimg + ((size_t)bh * ntk + u) * C::kV16Stage, (uint32_t)C::kV16Stage, &v_full[u % VST]);
            }
            __syncwarp();
        };
        dependency_wait();                           // the pack kernel has completed: its images may be fetched
        if (qk_role) {
            for (int u = 0; u < KST; ++u) copy_k(u);
        } else {
            for (int u = 0; u < VST; ++u) copy_v(u);
        }
        tc_fence_before();
        __syncthreads();                             // Q staged; TMEM allocated
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        if (qk_role) {
            constexpr uint32_t id_qk = idesc_f16(kRows, kKeys);                    // fp16 x fp16, both K-major
            auto issue_qk = [&](int buf, int t) {
                const uint32_t d = tmem + kColX + buf * kKeys;
                const uint8_t *kst = k_16 + (t % KST) * C::kK16Stage;
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
                if (elect_one()) tc_commit(&s_full[t % KST]);        // S is ready, and this K stage may be refilled
            };
            wait(&k_full[0], 0, 4);
            tc_fence_after();
            issue_qk(0, 0);
            for (int t = 0; t + 1 < nk; ++t) {
                wait(&k_full[(t + 1) % KST], phn(t + 1, KST), 4);                // K(t+1) is in its stage
                // the buffer of S(t+1) held P(t-1) (first sweep) or S(t-1) (second sweep)
                if (t >= 1) {
                    if (t - 1 < nt) wait(&o_done[(t - 1) % VST], phn(t - 1, VST), 2);        // P V(t-1) has read it
                    else wait(&p_full[(t - 1) % kBufs], phn(t - 1, kBufs), 5);               // the workers have read it
                }
                tc_fence_after();
                issue_qk((t + 1) % kBufs, t + 1);
                // Q K(t)^T was issued a whole step ago: it has completed, or does so before the product above
                wait(&s_full[t % KST], phn(t, KST), 7);
                copy_k(t + KST);
            }
        } else {
            constexpr uint32_t id_pv_a = idesc_f16(kRows, 2 * D) | (1u << 16);     // P_hi x [V_hi | V_lo], B N-major
            constexpr uint32_t id_pv_b = idesc_f16(kRows, D) | (1u << 16);         // P_lo x V_hi
            for (int t = 0; t < nt; ++t) {
                const int buf = t % kBufs;
                wait(&p_full[buf], phn(t, kBufs), 5);                            // P(t) is in TMEM
                wait(&v_full[t % VST], phn(t, VST), 6);                          // V(t) is in its stage
                tc_fence_after();
                const uint32_t a0 = tmem + kColX + buf * kKeys;
                // N-major B without swizzle: lbo = bytes between groups of 8 keys, sbo = bytes between blocks of 8 columns
                const uint64_t dv = make_desc(smem_u32(v_16 + (t % VST) * C::kV16Stage), 32 * D, 128, 0);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)  // 16 keys = 8 TMEM columns of packed fp16 = two key groups of V
                    if (elect_one()) mma_h_ts(tmem + kColO, a0 + (uint32_t)(32 * (k >> 1) + 8 * (k & 1)), dv + (uint64_t)(k * 4 * D), id_pv_a, (t == 0 && k == 0) ? 0u : 1u);
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    if (elect_one()) mma_h_ts(tmem + kColO + D, a0 + (uint32_t)(32 * (k >> 1) + 8 * (k & 1) + 16), dv + (uint64_t)(k * 4 * D), id_pv_b, 1u);
                if (elect_one()) tc_commit(&o_done[t % VST]);        // O is up to date; this V stage may be refilled, Q K^T may take the buffer
                // P V(t-1) was issued a whole step ago: its stage takes V(t-1+VST)
                if (t >= 1) {
                    wait(&o_done[(t - 1) % VST], phn(t - 1, VST), 8);
                    copy_v(t - 1 + VST);
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
    // The warp stages its 32 query rows: times the softmax scale (scores come out in the log2 domain) and times a power of
    // two per row that brings the row's largest magnitude near 2^14; what the scores then carry too much (the row's factor
    // and K's per-tile factor) is taken out again by `sfac` below, inside the exponent's multiply-add.  D / 4 lanes read
    // one row (whole 128-byte lines per request; a thread reading its own row would touch 32 lines per instruction, twice,
    // and cost the block ~9000 cycles before its first product), all loads in flight at once.
    float sfac;
    {
        constexpr int LPR = D / 4, RPI = 32 / LPR, NI = 32 / RPI;      // lanes per row, rows per instruction, instructions
        const int c4 = lane % LPR, rsub = lane / LPR;
        float4 qv[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int rg = q0 + wq * 32 + i * RPI + rsub;
            qv[i] = rg < S ? __ldg(reinterpret_cast<const float4 *>(Q + (tok0 + rg) * (size_t)E + hcol) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // the rows' largest magnitudes first, all exchanges side by side (an exchange between two stores would keep the
        // compiler from overlapping the rows' dependent chains)
        float amax[NI];
#pragma unroll
        for (int i = 0; i < NI; ++i) amax[i] = fmaxf(fmaxf(fabsf(qv[i].x), fabsf(qv[i].y)), fmaxf(fabsf(qv[i].z), fabsf(qv[i].w)));
#pragma unroll
        for (int o = 1; o < LPR; o <<= 1) {
#pragma unroll
            for (int i = 0; i < NI; ++i) amax[i] = fmaxf(amax[i], __shfl_xor_sync(0xffffffffu, amax[i], o));
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int r = wq * 32 + i * RPI + rsub;
            float4 a = qv[i];
            const float sq = range_scale(amax[i] * qscale);
            const float qs = qscale * sq;
            a.x *= qs; a.y *= qs; a.z *= qs; a.w *= qs;
            const float4 ah = hi4(a);
            // values 4 c4 .. 4 c4 + 3 of the row: one half of a 16-byte chunk of the hi part, and of the lo part
            *reinterpret_cast<uint2 *>(q_16 + off16(r, c4 >> 1, kQBlk) + (c4 & 1) * 8) = make_uint2(pack_f16(ah.x, ah.y), pack_f16(ah.z, ah.w));
            *reinterpret_cast<uint2 *>(q_16 + off16(r, PPR + (c4 >> 1), kQBlk) + (c4 & 1) * 8) =
                make_uint2(pack_f16(a.x - ah.x, a.y - ah.y), pack_f16(a.z - ah.z, a.w - ah.w));
            if (c4 == 0) q_sfac[r] = __uint_as_float(0x7F000000u - __float_as_uint(sq));      // 1 / sq, a power of two within 2^+-126
        }
        __syncwarp();
        sfac = q_sfac[rloc];
    }
    // The rows above were read beside the tail of the pack kernel; what it wrote is read from here on.
    dependency_wait();
    // V's tiles carry factors of their own; P(t) is made smaller by tile t's factor over the smallest one among the
    // block's tiles (that of their largest |V|), which leaves with the output
    const float *tmax_k = tmax + (size_t)bh * ntk, *tmax_v = tmax + ntiles + (size_t)bh * ntk;
    float vmax_all = 0.0f;
    for (int t = lane; t < nt; t += 32) vmax_all = fmaxf(vmax_all, __ldg(tmax_v + t));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) vmax_all = fmaxf(vmax_all, __shfl_xor_sync(0xffffffffu, vmax_all, o));
    const float vhs = range_scale(vmax_all), vinv = 1.0f / vhs;
    proxy_fence();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t lane_base = tmem_base_slot + ((uint32_t)(wq * 32) << 16);
    const uint32_t o_addr = lane_base + kColO;

    float m_ref = 0.0f, l = 0.0f;                    // reference maximum (log2 domain) and row sum (of P, which carries 2^6)
    // the tiles' largest magnitudes are fetched one tile ahead: their latency (L2) must not stand between the sweeps
    float kmx_next = __ldg(tmax_k), vmx_next = __ldg(tmax_v);
    for (int t = 0; t < nt; ++t) {
        const float kmx = kmx_next, vmx = vmx_next;
        if (t + 1 < nt) {
            kmx_next = __ldg(tmax_k + t + 1);
            vmx_next = __ldg(tmax_v + t + 1);
        }
        const int buf = t % kBufs;
        const int j0 = t * kKeys;
        const uint32_t s_addr = lane_base + kColX + buf * kKeys;
        wait(&s_full[t % KST], phn(t, KST), 1);      // S(t) is in TMEM
        tc_fence_after();
        const int wrow0 = q0 + wq * 32;              // first row of this warp
        // columns of this tile that the row sees; the warp's last row sees the most, its first row the fewest
        const int ncols = min(kKeys, S - j0);
        const int nvalid = CAUSAL ? max(0, min(ncols, row - j0 + 1)) : ncols;
        const int nwarp = CAUSAL ? max(0, min(ncols, wrow0 + 31 - j0 + 1)) : ncols;
        const int nmin = CAUSAL ? max(0, min(ncols, wrow0 - j0 + 1)) : ncols;
        const int nch = (nwarp + 31) >> 5;           // 32-column chunks with any visible key (0: the tile is above the diagonal for the warp)

        // ---- the tile's scores are read once and stay in registers for both sweeps -------------------
        // (chunks of 32 columns; a chunk that no row of the warp sees is not read)
        float v0[32], v1[32];
        if (nch > 0) tmem_ld32(s_addr, v0);
        if (nch > 1) tmem_ld32(s_addr + 32, v1);
        tmem_wait_ld();
        // ---- first sweep: the row's largest score of this tile (hidden scores become -inf here) ------
        float mx = -INFINITY;
        if (nch > 0) mx = chunk_max(v0, 0, nvalid, 32 > nmin);
        if (nch > 1) mx = fmaxf(mx, chunk_max(v1, 32, nvalid, 64 > nmin));
        const float tfac = sfac / range_scale(kmx);   // what this tile's scores carry too much: the row's and the tile's factors
        mx *= tfac;                                  // the row's largest true score (tfac > 0)
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
                wait(&o_done[(t - 1) % VST], phn(t - 1, VST), 2);    // P V(t-1) has completed
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
        const float vrel = fminf(vhs / range_scale(vmx), 1.0f);   // <= 1: this V tile's factor against the head's (a tile of zeros: 1)
        const float nm = kPShift - m_ref + log2_of_pow2(vrel);
        float psum = 0.0f;
        if (nch > 0) psum = chunk_exp(v0, s_addr, tfac, nm);
        else tmem_zero32(s_addr);
        if (nch > 1) psum += chunk_exp(v1, s_addr + 32, tfac, nm);
        else tmem_zero32(s_addr + 32);               // a chunk that no row of this warp sees
        l += psum / vrel;                            // the row sum counts the probabilities themselves (a power of two: exact)
        tmem_wait_st();
        tc_fence_before();
        arrive(&p_full[buf]);
    }

    {
        wait(&o_done[(nt - 1) % VST], phn(nt - 1, VST), 3);
        tc_fence_after();
        const float linv = 1.0f / fmaxf(l, 1e-20f);  // for the probabilities
        const float inv = linv * vinv;
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
                const float tfac2 = sfac / range_scale(__ldg(tmax_k + (u - nt)));
                const uint32_t s_addr = lane_base + kColX + buf * kKeys;
                wait(&s_full[u % KST], phn(u, KST), 1);
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
                        o[i] = c < nvalid ? ex2_approx(fmaf(sc, tfac2, kPShift - m_ref)) * linv : 0.0f;
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
}

// The packed operands of a call live in a buffer of the library, one per device and stream (a call's kernels read it
// after the call has returned; calls on different streams must not share it).  It grows to the largest call.
struct PackScratch {
    std::mutex mu;
    // side: the stream on which the groups after the first are packed while the group before them is attended to;
    // entered: the caller's stream has reached the call; packed[i], attended[i]: buffer i has been written / read
    struct Entry { int dev; cudaStream_t st; uint8_t *buf; size_t cap; cudaStream_t side; cudaEvent_t entered, packed[2], attended[2]; };
    std::vector<Entry> entries;
    int get(int dev, cudaStream_t st, size_t need, uint8_t **out, Entry **entry = nullptr)
    {
        std::lock_guard<std::mutex> lock(mu);
        Entry *e = nullptr;
        for (auto &x : entries) if (x.dev == dev && x.st == st) e = &x;
        if (!e) { entries.push_back({dev, st, nullptr, 0, nullptr, nullptr, {nullptr, nullptr}, {nullptr, nullptr}}); e = &entries.back(); }
        if (entry) {
            *entry = e;                              // entries are only appended, and only under the lock: take care below
            if (!e->side) {
                cudaError_t err = cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking);
                if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->entered, cudaEventDisableTiming);
                for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
                    err = cudaEventCreateWithFlags(&e->packed[i], cudaEventDisableTiming);
                    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&e->attended[i], cudaEventDisableTiming);
                }
                if (err != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "stream or event for the packing: %s", cudaGetErrorString(err));
            }
        }
        if (e->cap < need) {
            if (e->buf) cudaFree(e->buf);        // waits for the kernels that read it
            e->buf = nullptr;
            e->cap = 0;
            const cudaError_t err = cudaMalloc(&e->buf, need);
            if (err != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMalloc(%zu) for the packed K and V: %s", need, cudaGetErrorString(err));
            e->cap = need;
        }
        *out = e->buf;
        return HIPGPT_OK;
    }
    void release()
    {
        std::lock_guard<std::mutex> lock(mu);
        for (auto &x : entries) {
            if (x.buf) cudaFree(x.buf);
            if (x.side) cudaStreamDestroy(x.side);
            if (x.entered) cudaEventDestroy(x.entered);
            for (int i = 0; i < 2; ++i) {
                if (x.packed[i]) cudaEventDestroy(x.packed[i]);
                if (x.attended[i]) cudaEventDestroy(x.attended[i]);
            }
        }
        entries.clear();
    }
};
PackScratch g_pack;

template <int D, bool CAUSAL, bool PROBS>
int launch_tc16_cfg(const float *q, const float *k, const float *v, float *out, float *probs, int B, int S, int E, int H, cudaStream_t st)
{
    using C = Tc16Cfg<D>;
    auto kern = mha_tc16_kernel<D, CAUSAL, PROBS>;
    // two blocks per SM (256 TMEM columns each): at least 100 KB, so that a third block never shares the SM
    size_t smem = C::kSmemBytes + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    static_assert(C::kSmemBytes + 1024 + 2048 <= 232448 / C::BLOCKS_PER_SM, "shared memory of a block");
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kRows - 1) / kRows;
    const int ntk = (S + kKeys - 1) / kKeys;
    // The call is cut into groups of batches whose packed K and V (as many bytes as the fp32 K and V) stay in L2
    // between the kernel that writes them and the kernel that reads them; the scratch buffer is one group's size.
    const size_t per_batch = (size_t)H * ntk * (C::kK16Stage + C::kV16Stage);
    size_t group_bytes = 96u << 20;
    if (const char *env = getenv("HIPGPT_PACK_GROUP_MB")) { const long v = atol(env); if (v > 0) group_bytes = (size_t)v << 20; }
    long long gb = (long long)(group_bytes / per_batch);
    if (gb < 1) gb = 1;
    // A call of several groups can pack group g + 1 on a second stream while group g is attended to: two buffers of half
    // a group each (the same footprint in L2), events in both directions.  Measured at B=64 H=16 S=2048 head_dim 64:
    // unmasked 292 -> 309 TFLOP/s; causal 256 -> 249 (half-size groups leave the causal kernel, whose blocks differ in
    // length, a longer tail per launch, and 128 - 192 MB of buffers do not help either: 252 - 254).  So it is the default
    // for unmasked calls only; HIPGPT_PACK_OVERLAP=0 / 1 forces it off / on for both.
    static const int overlap_env = [] { const char *e = getenv("HIPGPT_PACK_OVERLAP"); return (!e || !*e) ? -1 : (*e != '0' ? 1 : 0); }();
    const bool overlap = (overlap_env < 0 ? !CAUSAL : overlap_env == 1) && B > gb && gb >= 2;
    if (overlap) gb = gb / 2;
    if (gb > B) gb = B;
    while (gb * H > 65535) --gb;                     // grid.y of the pack kernel
    if (gb < 1) return fail(HIPGPT_ERR_BAD_ARG, "%d heads are too many", H);
    if (gb * H * (long long)nqblk > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", gb * H * (long long)nqblk);
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    const size_t kbytes = (size_t)gb * H * ntk * C::kK16Stage, vbytes = (size_t)gb * H * ntk * C::kV16Stage;
    const size_t gtiles = (size_t)gb * H * ntk;
    const size_t one = (kbytes + vbytes + 2 * gtiles * sizeof(float) + 1023) & ~(size_t)1023;      // one buffer: K images, V images, the tiles' maxima
    uint8_t *scratch = nullptr;
    PackScratch::Entry *ent = nullptr;
    int rc = g_pack.get(dev, st, overlap ? 2 * one : one, &scratch, overlap ? &ent : nullptr);
    if (rc != HIPGPT_OK) return rc;
    cudaStream_t side = nullptr;
    cudaEvent_t entered = nullptr, packed[2] = {nullptr, nullptr}, attended[2] = {nullptr, nullptr};
    if (overlap) {                                   // copies: the vector of entries may move
        side = ent->side; entered = ent->entered;
        for (int i = 0; i < 2; ++i) { packed[i] = ent->packed[i]; attended[i] = ent->attended[i]; }
        e = cudaEventRecord(entered, st);            // K and V are valid from here on, and earlier calls have read the buffers
        if (e == cudaSuccess) e = cudaStreamWaitEvent(side, entered, 0);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
    }
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    int g = 0;
    for (long long b0 = 0; b0 < B; b0 += gb, ++g) {
        const int nb = (int)(B - b0 < gb ? B - b0 : gb);
        const size_t off = (size_t)b0 * S * E;       // the group's first token in every plane and in the output
        const int ntiles = nb * H * ntk;
        uint8_t *buf = scratch + (overlap ? (size_t)(g & 1) * one : 0);
        float *tmax = reinterpret_cast<float *>(buf + kbytes + vbytes);      // [2][group's tiles]: largest |K|, |V| of every tile
        const cudaStream_t ps = overlap ? side : st;
        if (overlap && g >= 2) {
            e = cudaStreamWaitEvent(side, attended[g & 1], 0);               // the group that used this buffer has been attended to
            if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
        }
        kv_pack_kernel<D><<<dim3((unsigned)ntk, (unsigned)(nb * H)), kPackThreads, 0, ps>>>(k + off, v + off, tmax, buf, buf + kbytes, S, E, H, ntk, ntiles);
        rc = check_launch("kv_pack_kernel");
        if (rc != HIPGPT_OK) return rc;
        if (overlap) {
            e = cudaEventRecord(packed[g & 1], side);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(st, packed[g & 1], 0);
            if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
        }
        // (one stream:) the attention kernel's blocks start, and stage their query rows, while the pack kernel's last blocks run
        e = launch_overlapped(kern, dim3((unsigned)(nb * H * nqblk)), dim3(C::THREADS), smem, st, (const uint8_t *)buf, (const uint8_t *)(buf + kbytes),
                              (const float *)tmax, ntiles, q + off, out + off, probs ? probs + (size_t)b0 * H * S * S : nullptr, S, E, H, nb * H, nqblk, ntk, qscale);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "mha_tc16_kernel launch: %s", cudaGetErrorString(e));
        rc = check_launch("mha_tc16_kernel");
        if (rc != HIPGPT_OK) return rc;
        if (overlap) {
            e = cudaEventRecord(attended[g & 1], st);
            if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
        }
    }
    return HIPGPT_OK;
}

}  // namespace

bool mha_tc16_supports(int head_dim) { return head_dim == 32 || head_dim == 64; }

// Frees the packed-operand buffers (hipgpt_release_workspace).
void tc16_release_scratch() { g_pack.release(); }

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
