// tcgen05 / TMEM / mbarrier primitives shared by the tensor-core attention kernels (sm_100a).
#pragma once

#include "attn_common.cuh"

namespace hipgpt {

constexpr long long kSpinLimit = 1LL << 24;      // polls per wait, and
constexpr long long kCycleLimit = 1LL << 31;     // SM cycles per wait (about one second)
constexpr uint32_t kSuspendHintNs = 20000;       // how long one try_wait may sleep before it returns unsatisfied

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Non-blocking test: has the phase with the given parity completed?
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}

// Bounded wait for the phase with the given parity; false when the limit (SM cycles, and a number of
// polls) ran out.  A phase that has already completed is recognised by one non-blocking test,
// without reading the clock.
__device__ __forceinline__ bool mbar_wait_for(uint64_t *bar, uint32_t parity, long long cycle_limit, long long poll_limit)
{
    const uint32_t addr = smem_u32(bar);
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    const long long deadline = clock64() + cycle_limit;
    for (long long i = 0; i < poll_limit; ++i) {
        // the thread sleeps inside the instruction until the phase completes or the hinted time (ns) has passed
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity), "r"(kSuspendHintNs) : "memory");
        if (done) return true;
        if ((i & 3) == 3 && clock64() > deadline) break;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) { return mbar_wait_for(bar, parity, kCycleLimit, kSpinLimit); }

// One arrival that also announces `bytes` of asynchronous copies which will complete on this barrier.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// TMA: one box of a rank-3 tensor map (this GPU's own memory; no multicast) into shared memory; the
// bytes count towards `bar`.  c0 is the innermost coordinate: c0 * element size must be a multiple
// of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tensor_map, int c0, int c1, int c2, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}

// Plain bulk copy global -> shared (both 16-byte aligned, a multiple of 16 bytes), completion counted on the mbarrier.
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gmem_src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Asks L2 for one box of a rank-3 tensor map; nothing is written to shared memory and nothing signals completion.
__device__ __forceinline__ void tma_prefetch_3d(const void *tensor_map, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
                 ::"l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One lane of the (converged) warp: true for the elected lane only.  The hardware picks the same lane every
// time for the same set of lanes, so the instructions a warp issues under this test come from one thread and
// run in program order, and a tcgen05.commit issued under it covers them.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, px;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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

// tcgen05.ld / st, shape 32x32b: thread i of the warp moves N consecutive 32-bit columns of TMEM
// lane (base lane + i).  Values pass through plain registers (no address is taken).
__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32])
{
    uint32_t r0, r1, r2, r3, r4, r5, r6, r7, r8, r9, r10, r11, r12, r13, r14, r15, r16, r17, r18, r19, r20, r21, r22, r23, r24, r25, r26, r27, r28, r29, r30, r31;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3), "=r"(r4), "=r"(r5), "=r"(r6), "=r"(r7), "=r"(r8), "=r"(r9), "=r"(r10), "=r"(r11), "=r"(r12), "=r"(r13), "=r"(r14), "=r"(r15), "=r"(r16), "=r"(r17), "=r"(r18), "=r"(r19), "=r"(r20), "=r"(r21), "=r"(r22), "=r"(r23), "=r"(r24), "=r"(r25), "=r"(r26), "=r"(r27), "=r"(r28), "=r"(r29), "=r"(r30), "=r"(r31)
                 : "r"(addr) : "memory");
    v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3); v[4] = __uint_as_float(r4); v[5] = __uint_as_float(r5); v[6] = __uint_as_float(r6); v[7] = __uint_as_float(r7); v[8] = __uint_as_float(r8); v[9] = __uint_as_float(r9); v[10] = __uint_as_float(r10); v[11] = __uint_as_float(r11); v[12] = __uint_as_float(r12); v[13] = __uint_as_float(r13); v[14] = __uint_as_float(r14); v[15] = __uint_as_float(r15); v[16] = __uint_as_float(r16); v[17] = __uint_as_float(r17); v[18] = __uint_as_float(r18); v[19] = __uint_as_float(r19); v[20] = __uint_as_float(r20); v[21] = __uint_as_float(r21); v[22] = __uint_as_float(r22); v[23] = __uint_as_float(r23); v[24] = __uint_as_float(r24); v[25] = __uint_as_float(r25); v[26] = __uint_as_float(r26); v[27] = __uint_as_float(r27); v[28] = __uint_as_float(r28); v[29] = __uint_as_float(r29); v[30] = __uint_as_float(r30); v[31] = __uint_as_float(r31);
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16])
{
    uint32_t r0, r1, r2, r3, r4, r5, r6, r7, r8, r9, r10, r11, r12, r13, r14, r15;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3), "=r"(r4), "=r"(r5), "=r"(r6), "=r"(r7), "=r"(r8), "=r"(r9), "=r"(r10), "=r"(r11), "=r"(r12), "=r"(r13), "=r"(r14), "=r"(r15)
                 : "r"(addr) : "memory");
    v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3); v[4] = __uint_as_float(r4); v[5] = __uint_as_float(r5); v[6] = __uint_as_float(r6); v[7] = __uint_as_float(r7); v[8] = __uint_as_float(r8); v[9] = __uint_as_float(r9); v[10] = __uint_as_float(r10); v[11] = __uint_as_float(r11); v[12] = __uint_as_float(r12); v[13] = __uint_as_float(r13); v[14] = __uint_as_float(r14); v[15] = __uint_as_float(r15);
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const float (&v)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 16 packed 32-bit words (e.g. 32 bf16 values) to 16 consecutive TMEM columns of this thread's lane.
__device__ __forceinline__ void tmem_st16_u32(uint32_t addr, const uint32_t (&v)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}

// ---- split-TF32 helpers (fp32 operands cut into a TF32-exact hi part and the remainder) ----

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

// Instruction descriptor: fp32 accumulator, TF32 operands, A K-major, B K- or N-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_n_major)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_n_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

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

// ---- fp16 products (kind::f16) used for the correction terms and the all-fp16 P V product ----

// fp32 accumulator, fp16 A and B, both K-major
__host__ __device__ constexpr uint32_t idesc_f16(int m, int n)
{
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void mma_h_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_h_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// two floats -> one word of two fp16 (round to nearest, saturating), `lo` in the low half
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void tmem_st8_u32(uint32_t addr, const uint32_t (&v)[8])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}

__device__ __forceinline__ float4 hi4(float4 x) { return make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w)); }

// Two fp32 operations in one instruction (sm_100 has fused multiply-add and add on pairs of registers), and the
// three-input maximum: the softmax sweeps are bound by the instructions they issue.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<const uint64_t *>(&a)), "l"(*reinterpret_cast<const uint64_t *>(&b)), "l"(*reinterpret_cast<const uint64_t *>(&c)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<const uint64_t *>(&a)), "l"(*reinterpret_cast<const uint64_t *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// byte offset of 16-byte chunk c of row r in a tile of 128-byte rows, SWIZZLE_128B
__device__ __forceinline__ int sw128(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

}  // namespace hipgpt
