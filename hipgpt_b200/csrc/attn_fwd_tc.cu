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
// One thread block = 128 query rows of one (batch, head): 256 worker threads plus one warp
// whose single elected lane issues the MMAs.  Worker warp w works on TMEM lanes 32*(w%4)..,
// i.e. worker (w%4)*32+lane owns query row q0 + that index, and the two workers of a row
// (warps w and w+4) split the 64 keys of a tile and the head dimension of the output.
// A tcgen05.mma with M=128, K=8 costs 64 cycles for any N up to 128 (measured), so operands
// are concatenated along N where the split allows it.  Per tile of 64 keys:
//   stage   K and V are read from global with coalesced 128-bit loads one tile ahead (they wait
//           in registers), split into hi / lo and written to shared memory in the tensor
//           core's canonical 128-byte-swizzled layouts (K: K-major SWIZZLE_128B, hi rows then
//           lo rows; V: N-major, which for 32-bit operands must be SWIZZLE_128B with a
//           32-byte base, hi blocks then lo blocks);
//   S_ext   = Q_hi [K_hi; K_lo]^T (one N=128 product: columns 0-63 main term, 64-127 first
//           correction) and Q_lo K_hi^T added to columns 64-127, accumulators in TMEM;
//   softmax each worker reads its 32 scores (main + corrections) with tcgen05.ld, the two
//           halves of a row exchange their maxima through shared memory, running maximum
//           and sum are kept in the log2 domain (one ex2 per score); P is split into hi / lo
//           and written back to TMEM (P_hi over S in place, P_lo beside it);
//   O_ext   = P_hi [V_hi | V_lo] (N = 2D) and P_lo V_hi added to its second half, A = P from
//           TMEM, fresh accumulator per tile; it is collected one iteration later;
//   update  o = o * alpha + (both halves of O_ext) in registers.
// The issuing lane runs P V(t) then Q K(t+1)^T back to back; meanwhile the workers of the
// other resident block do their softmax, so two blocks per SM keep the tensor pipe busy.
// Hand-offs use mbarriers (tcgen05.commit for the MMAs, 256 arrivals for the workers).  Every
// wait is bounded: on expiry the block raises a flag that cuts all its later waits short,
// records a status code, skips its stores, frees its TMEM and returns.  No probabilities are
// written by this kernel; callers that want them get the FFMA rows kernel.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kM = 128;          // query rows per block
constexpr int kN = 64;           // keys per tile
constexpr int kWorkers = 256;      // softmax / staging threads
constexpr int kThreads = kWorkers + 32;   // plus the warp that issues the MMAs
constexpr long long kSpinLimit = 1LL << 24;      // polls per wait, and
constexpr long long kCycleLimit = 1LL << 31;     // SM cycles per wait (about one second)

__device__ int g_tc_status = 0;   // 0 ok; 1 = an mbarrier wait ran out

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    const long long deadline = clock64() + kCycleLimit;
    for (long long i = 0; i < kSpinLimit && clock64() < deadline; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor for a tile made of 128-byte rows.
//   K-major operands (Q, K): layout 2 = SWIZZLE_128B, rows grouped by 8 (1024 bytes); sbo = bytes
//     between groups, lbo unused (16).
//   N-major operand (V): 32-bit operands that are contiguous along N must use layout 1,
//     SWIZZLE_128B with a 32-byte base: reduction rows grouped by 4 (512 bytes); sbo = bytes
//     between groups, lbo = bytes between 32-float column blocks.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version of sm_100
    d |= (uint64_t)layout_type << 61;   // 2 = SWIZZLE_128B, 1 = SWIZZLE_128B with 32-byte base
    return d;
}

// Instruction descriptor: fp32 accumulator, TF32 operands, A K-major, B K- or N-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_n_major)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_n_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32])
{
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t addr, const float (&v)[32])
{
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16])
{
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float (&v)[16])
{
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// Writes one 16-byte chunk of a row, split into hi and lo, at its swizzled place:
// chunk c of row r of a [rows][128 B] block lands at r*128 + ((c ^ (r & 7)) * 16).
__device__ __forceinline__ void store_split(float *hi_blk, float *lo_blk, int row, int chunk, float4 x)
{
    const int off = row * 32 + ((chunk ^ (row & 7)) << 2);
    const float4 h = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
    *reinterpret_cast<float4 *>(hi_blk + off) = h;
    *reinterpret_cast<float4 *>(lo_blk + off) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
}

// The same for the N-major operand: 32-byte pieces of a row are permuted by the row index
// modulo 4; the 16-byte half inside a piece keeps its place.
__device__ __forceinline__ void store_split_nmajor(float *hi_blk, float *lo_blk, int row, int chunk, float4 x)
{
    const int piece = (chunk >> 1) ^ (row & 3);
    const int off = row * 32 + (((piece << 1) | (chunk & 1)) << 2);
    const float4 h = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
    *reinterpret_cast<float4 *>(hi_blk + off) = h;
    *reinterpret_cast<float4 *>(lo_blk + off) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
}

template <int D>
struct TcCfg {
    static constexpr int DB = D / 32;                     // 32-float column blocks per row
    static constexpr int QBLK = kM * 32;                  // floats per [128][32] block
    static constexpr int KBLK = kN * 32;                  // floats per [64][32] block
    // TMEM columns: S_ext | P_lo | O_ext
    static constexpr uint32_t kColS = 0;                  // [0,64): Q_hi K_hi (later P_hi), [64,128): Q_hi K_lo + Q_lo K_hi
    static constexpr uint32_t kColPlo = 128;              // 64 columns
    static constexpr uint32_t kColO = 192;                // [0,D): P_hi V_hi, [D,2D): P_hi V_lo + P_lo V_hi
    static constexpr uint32_t kTmemCols = (192 + 2 * D) <= 256 ? 256 : 512;
    static constexpr size_t kSmemFloats = (size_t)2 * DB * QBLK + 4 * DB * KBLK;
};

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kThreads, D == 32 ? 2 : 1)   // head_dim 32: two blocks per SM
mha_tc_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
              float *__restrict__ O, int S, int E, int H, int BH, int nqblk, float qscale)
{
    using C = TcCfg<D>;
    constexpr int DB = C::DB, QBLK = C::QBLK, KBLK = C::KBLK;
    constexpr int DH = D / 2;                    // output columns per worker thread
    constexpr int CPR = D / 4;                   // 16-byte chunks per row
    constexpr int RPP = kWorkers / CPR;          // K/V rows staged per pass
    constexpr int NP = kN / RPP;                 // passes = float4 registers per staged tile
    constexpr uint32_t kColS = C::kColS, kColPlo = C::kColPlo, kColO = C::kColO;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment is what the swizzled layouts assume
    float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *q_hi = base, *q_lo = q_hi + DB * QBLK;        // [DB][128][32] each
    float *k_s = q_lo + DB * QBLK;                       // [DB][hi, lo][64][32]: hi and lo rows form one 128-row operand
    float *v_s = k_s + 2 * DB * KBLK;                    // [hi, lo][DB][64][32]: hi and lo blocks form one 2D-column operand
    __shared__ uint64_t mbar_s, mbar_p, mbar_o;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;
    __shared__ float xchg[2][kM];                // row maxima (later: row sums) of the two halves

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_mma_warp = warp == kWorkers / 32;
    const int half = (warp >> 2) & 1;            // which 32 keys of a tile / which output columns
    const int rloc = (warp & 3) * 32 + lane;     // row inside the block = TMEM lane
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);   // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * kM;
    const int row = q0 + rloc;                   // this worker's query

    const int kend = CAUSAL ? min(S, q0 + kM) : S;
    const int ntiles = (kend + kN - 1) / kN;

    if (tid == 0) {
        abort_flag = 0;
        mbar_init(&mbar_s, 1);                   // tcgen05.commit after Q K^T
        mbar_init(&mbar_p, kWorkers);            // every worker: P written, K and V staged
        mbar_init(&mbar_o, 1);                   // tcgen05.commit after P V
    }

    // Bounded wait that gives up at once when another thread already gave up.
    auto wait = [&](uint64_t *bar, uint32_t parity) {
        if (abort_flag) return;
        if (!mbar_wait(bar, parity)) abort_flag = 1;
    };

    // K/V staging role of a worker: chunk sc of rows sr0 + p*RPP
    const int sc = tid % CPR, sr0 = (tid % kWorkers) / CPR;
    auto load_tile = [&](const float *__restrict__ plane, int t, float4 (&regs)[NP]) {
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            const int j = t * kN + sr0 + p * RPP;
            const bool ok = t < ntiles && j < S;
            regs[p] = ok ? __ldg(reinterpret_cast<const float4 *>(plane + (tok0 + j) * (size_t)E + hcol + sc * 4))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto store_k = [&](const float4 (&regs)[NP]) {
        float *blk = k_s + (sc >> 3) * 2 * KBLK;
#pragma unroll
        for (int p = 0; p < NP; ++p) store_split(blk, blk + KBLK, sr0 + p * RPP, sc & 7, regs[p]);
    };
    auto store_v = [&](const float4 (&regs)[NP]) {
        float *blk = v_s + (sc >> 3) * KBLK;
#pragma unroll
        for (int p = 0; p < NP; ++p) store_split_nmajor(blk, blk + DB * KBLK, sr0 + p * RPP, sc & 7, regs[p]);
    };

    // ---- prologue ------------------------------------------------------------------------------
    float4 kreg[NP], vreg[NP];
    if (!is_mma_warp) {
        constexpr int QC = CPR / 2;              // Q chunks per worker (two workers per row)
        float4 qreg[QC];
        const bool ok = row < S;
        const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol) + half * QC;
#pragma unroll
        for (int c = 0; c < QC; ++c) qreg[c] = ok ? __ldg(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        load_tile(K, 0, kreg);
        load_tile(V, 0, vreg);
#pragma unroll
        for (int c = 0; c < QC; ++c) {
            float4 x = qreg[c];
            x.x *= qscale; x.y *= qscale; x.z *= qscale; x.w *= qscale;
            const int cc = half * QC + c;
            store_split(q_hi + (cc >> 3) * QBLK, q_lo + (cc >> 3) * QBLK, rloc, cc & 7, x);
        }
        store_k(kreg);
        load_tile(K, 1, kreg);                   // in flight until Q K(0)^T has completed
        proxy_fence();                           // generic-proxy writes -> visible to the tensor core's reads
    } else {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;

    if (is_mma_warp) {
        // ================= the issuing warp: one lane feeds the tensor core ====================
        if (lane == 0) {
            constexpr uint32_t idesc_qk1 = make_idesc(kM, 2 * kN, 0);    // Q_hi  x [K_hi; K_lo]
            constexpr uint32_t idesc_qk2 = make_idesc(kM, kN, 0);        // Q_lo  x K_hi
            constexpr uint32_t idesc_pv1 = make_idesc(kM, 2 * D, 1);     // P_hi  x [V_hi | V_lo]
            constexpr uint32_t idesc_pv2 = make_idesc(kM, D, 1);         // P_lo  x V_hi
            auto issue_qk = [&]() {
                uint32_t acc = 0;
#pragma unroll
                for (int db = 0; db < DB; ++db) {
                    const uint64_t da = make_desc(smem_u32(q_hi + db * QBLK), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(k_s + db * 2 * KBLK), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {            // 8 floats = 32 bytes per instruction
                        mma_ss(tmem + kColS, da + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk1, acc);
                        acc = 1;
                    }
                }
                // the second correction term joins the first one in columns [64,128): both are
                // small, so the tensor core's truncating adds cost no accuracy there
#pragma unroll
                for (int db = 0; db < DB; ++db) {
                    const uint64_t da = make_desc(smem_u32(q_lo + db * QBLK), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(k_s + db * 2 * KBLK), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_ss(tmem + kColS + kN, da + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk2, 1);
                }
                tc_commit(&mbar_s);
            };
            auto issue_pv = [&]() {
                // N-major B: 8 reduction rows (keys) of 128 bytes per instruction = 1024 bytes
                const uint64_t dv = make_desc(smem_u32(v_s), KBLK * 4, 512, 1);
#pragma unroll
                for (int k = 0; k < kN / 8; ++k)
                    mma_ts(tmem + kColO, tmem + kColS + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv1, k ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < kN / 8; ++k)
                    mma_ts(tmem + kColO + D, tmem + kColPlo + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv2, 1);
                tc_commit(&mbar_o);
            };
            if (ntiles > 0) issue_qk();
            for (int t = 0; t < ntiles; ++t) {
                wait(&mbar_p, (uint32_t)(t & 1));        // P(t) in TMEM, V(t) and K(t+1) in shared memory
                tc_fence_after();
                issue_pv();
                if (t + 1 < ntiles) issue_qk();          // runs after P V(t): MMAs of one thread execute in order
            }
        }
        __syncwarp();
    } else {
        // ================= the 256 workers: softmax, staging, output ===========================
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);   // this warp's 32 TMEM lanes
        float o[DH];
#pragma unroll
        for (int d = 0; d < DH; ++d) o[d] = 0.0f;
        float m = -1e30f, l = 0.0f, alpha_prev = 1.0f;

        // o = o * alpha_prev + (both parts of) O_tile of the previous tile, this worker's DH columns
        auto collect_o = [&]() {
            if (DH == 16) {
                float a[16], c[16];
                tmem_ld16(lane_base + kColO + half * 16, a);
                tmem_ld16(lane_base + kColO + D + half * 16, c);
                tmem_wait_ld();
#pragma unroll
                for (int d = 0; d < 16; ++d) o[d] = fmaf(o[d], alpha_prev, a[d] + c[d]);
            } else {
                float a[32], c[32];
                tmem_ld32(lane_base + kColO + half * 32, a);
                tmem_ld32(lane_base + kColO + D + half * 32, c);
                tmem_wait_ld();
#pragma unroll
                for (int d = 0; d < 32; ++d) o[d % DH] = fmaf(o[d % DH], alpha_prev, a[d] + c[d]);
            }
        };

        for (int t = 0; t < ntiles; ++t) {
            const int j0 = t * kN + half * 32;        // first key of this worker's 32 columns
            wait(&mbar_s, (uint32_t)(t & 1));         // S(t) is in TMEM; the K buffer is free again
            tc_fence_after();
            if (t + 1 < ntiles) store_k(kreg);        // K(t+1) for the product that follows P V(t)
            load_tile(K, t + 2, kreg);

            // ---- softmax of this worker's 32 scores (tcgen05 ops are warp-wide: uniform control) ----
            float s[32];
            const bool warp_dead = CAUSAL && j0 > q0 + (warp & 3) * 32 + 31;   // all above the diagonal
            float mx = -INFINITY;
            if (!warp_dead) {
                tmem_ld32(lane_base + kColS + half * 32, s);
                {
                    float c0[16], c1[16];
                    tmem_ld16(lane_base + kColS + kN + half * 32, c0);
                    tmem_ld16(lane_base + kColS + kN + half * 32 + 16, c1);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 16; ++c) { s[c] += c0[c]; s[16 + c] += c1[c]; }
                }
                if ((CAUSAL && j0 + 31 > q0 + (warp & 3) * 32) || j0 + 32 > S) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int j = j0 + c;
                        if (j >= S || (CAUSAL && j > row)) s[c] = -INFINITY;
                    }
                }
#pragma unroll
                for (int c = 0; c < 32; ++c) mx = fmaxf(mx, s[c]);
            }
            xchg[half][rloc] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");   // the two warps of these rows
            mx = fmaxf(mx, xchg[half ^ 1][rloc]);
            const float mn = fmaxf(m, mx);            // m is finite (-1e30f at worst), so is mn
            const float alpha = ex2_approx(m - mn);
            m = mn;

            // ---- the previous tile's P V: collect it; P_lo and the V buffer are free afterwards ----
            if (t > 0) {
                wait(&mbar_o, (uint32_t)((t - 1) & 1));
                tc_fence_after();
                collect_o();
            }
            alpha_prev = alpha;
            store_v(vreg);                            // V(t)
            load_tile(V, t + 1, vreg);

            float psum = 0.0f;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                float lo[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float p = warp_dead ? 0.0f : ex2_approx(s[g * 16 + c] - mn);   // masked scores give exactly 0
                    psum += p;
                    const float ph = tf32_hi(p);
                    s[g * 16 + c] = ph;
                    lo[c] = p - ph;
                }
                tmem_st16(lane_base + kColPlo + half * 32 + g * 16, lo);
            }
            l = fmaf(l, alpha, psum);
            tmem_st32(lane_base + kColS + half * 32, s);       // P_hi over S, in place
            tmem_wait_st();
            proxy_fence();
            tc_fence_before();
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&mbar_p)) : "memory");
            // the exchange slots are reused next iteration: the partner has read them before it
            // arrives here, and nobody passes the next wait on mbar_s before all have arrived
        }
        if (ntiles > 0) {
            wait(&mbar_o, (uint32_t)((ntiles - 1) & 1));
            tc_fence_after();
            collect_o();
        }
        xchg[half][rloc] = l;                     // row sums of the two halves
        asm volatile("bar.sync 5, %0;" ::"r"(kWorkers) : "memory");
        if (!abort_flag && row < S) {
            const float inv = 1.0f / fmaxf(l + xchg[half ^ 1][rloc], 1e-20f);
            float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + row) * (size_t)E + hcol + half * DH);
#pragma unroll
            for (int c = 0; c < DH / 4; ++c)
                dst[c] = make_float4(o[c * 4 + 0] * inv, o[c * 4 + 1] * inv, o[c * 4 + 2] * inv, o[c * 4 + 3] * inv);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (abort_flag && tid == 0) atomicExch(&g_tc_status, 1);
    if (is_mma_warp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
    }
}

template <int D, bool CAUSAL>
int launch_tc_cfg(const float *q, const float *k, const float *v, float *out, int B, int S, int E, int H, cudaStream_t st)
{
    auto kern = mha_tc_kernel<D, CAUSAL>;
    // operands + alignment slack; never less than 100 KB, so that at most two blocks share an
    // SM and their two 256-column TMEM allocations always fit in the 512 columns
    size_t smem = TcCfg<D>::kSmemFloats * sizeof(float) + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kM - 1) / kM;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(q, k, v, out, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_tc_kernel");
}

}  // namespace

bool mha_tc_supports(int D) { return D == 32 || D == 64; }

int launch_mha_tc(const float *q, const float *k, const float *v, float *out,
                  int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (D == 32) return causal ? launch_tc_cfg<32, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<32, false>(q, k, v, out, B, S, E, H, st);
    if (D == 64) return causal ? launch_tc_cfg<64, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<64, false>(q, k, v, out, B, S, E, H, st);
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
