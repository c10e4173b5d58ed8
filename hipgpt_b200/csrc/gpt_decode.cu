// Greedy generation with HipGPT's model shape on one GPU, KV-cache form (sm_100a).
//
// This is the host driver and the plain, parity-first kernels around the attention path for the
// whole-model benchmark shape (E=256, L=8, H=8, F=1024, V=5000, S=256 by default).  Operators
// and wiring follow the reference (paths relative to the HipGPT tree):
//   embedding      src/hip_kernels.cpp:537-581      layer norm   src/hip_kernels.cpp:757-836
//   matmul(+bias)  src/hip_kernels.cpp:69-100, :113-145           relu  src/hip_kernels.cpp:249-252
//   block          src/transformer_layer.cpp:232-253 (pre-LN, two residual adds)
//   logits         src/gpt_model.cpp:117 (x * Wout, no final layer norm)
//   weights        checkpoint order of src/gpt_model.cpp:355-420 / src/transformer_layer.cpp:312-405
// What replaces the reference's loop (src/gpt_model.cpp:248-353: a full left-padded, unmasked
// window re-run per token, host sampling): every token runs once at its own position against
// cached K/V (hipgpt's split-context decode kernel), no dropout, Q/K/V are the column thirds
// of the projection, the next id is the first maximum of the logits and stays on the device.
//
// Arithmetic is fixed so that a CPU restatement can follow it bit for bit outside the
// attention: matmuls accumulate k ascending with fused multiply-add inside 16 equal segments of K
// whose partial sums are added in ascending order;
// layer-norm sums are 32 lane-strided partial sums joined by a butterfly; nothing else is
// contracted (explicit __fmul_rn / __fadd_rn), divisions and square roots are IEEE.
#include "attn_common.cuh"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

namespace hipgpt {
namespace {

constexpr int kRowsPerBlock = 8;     // activation rows a matmul block keeps in shared memory

// running (max, sum, weighted V) of the split-context attention, as in attn_decode.cu
struct Partial4f {
    float m, l;
    float4 o;
};
__device__ __forceinline__ void merge_partial(Partial4f &a, float m2, float l2, const float4 &o2)
{
    const float mn = fmaxf(a.m, m2);
    const float a1 = ex2_approx(a.m - mn), a2 = ex2_approx(m2 - mn);
    a.l = a.l * a1 + l2 * a2;
    a.o.x = a.o.x * a1 + o2.x * a2;
    a.o.y = a.o.y * a1 + o2.y * a2;
    a.o.z = a.o.z * a1 + o2.z * a2;
    a.o.w = a.o.w * a1 + o2.w * a2;
    a.m = mn;
}

// x[b] = tok[id] + pos[p]; the id is the prompt's while p is inside it, afterwards the id picked
// by the previous step.  p is read from device memory so that one captured step serves all.
__global__ void embed_kernel(const int *__restrict__ prompts, int n_prompt, const int *__restrict__ ids,
                             const int *__restrict__ pos_ptr, const float *__restrict__ tok, const float *__restrict__ pos,
                             float *__restrict__ x, int E, int V)
{
    dependency_wait();                               // overlapped launch: nothing is read before the kernel before this one has completed
    dependents_may_start();
    const int b = blockIdx.x;
    const int p = *pos_ptr;
    const int id = p < n_prompt ? prompts[(size_t)b * n_prompt + p] : ids[b];
    const bool ok = id >= 0 && id < V;
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        x[(size_t)b * E + e] = ok ? __fadd_rn(tok[(size_t)id * E + e], pos[(size_t)p * E + e]) : 0.0f;
}

// Layer norm of one row held in shared memory, by one warp, in place.  Sums are 32 lane-strided
// partial sums joined by a butterfly; nothing is contracted.
__device__ __forceinline__ void layernorm_row(float *row, const float *__restrict__ g, const float *__restrict__ b, int E, int lane)
{
    float s = 0.0f;
    for (int i = lane; i < E; i += 32) s = __fadd_rn(s, row[i]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    const float mean = __fdiv_rn(s, (float)E);
    float q = 0.0f;
    for (int i = lane; i < E; i += 32) {
        const float v = __fsub_rn(row[i], mean);
        q = __fadd_rn(q, __fmul_rn(v, v));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) q = __fadd_rn(q, __shfl_xor_sync(0xffffffffu, q, off));
    const float var = __fdiv_rn(q, (float)E);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, 1e-5f)));
    for (int i = lane; i < E; i += 32)
        row[i] = __fadd_rn(__fmul_rn(__fmul_rn(g[i], __fsub_rn(row[i], mean)), inv), b[i]);
}

// Where a matmul's outputs go: plain [M][ldo] (with optional residual), or the Q/K/V scatter of
// the attention projection (columns [0,E) -> q[m], [E,2E) -> K cache row p, [2E,3E) -> V cache row p).
struct MatmulOut {
    float *out;
    int ldo;
    const float *res;
    float *q, *kc, *vc;          // non-null q selects the scatter
    const int *pos_ptr;          // position of the scatter, read from the device ...
    int cap, E;
    int p_fixed;                 // ... or, when pos_ptr is NULL, given here
};

// y = relu?( LN?(A) * W + bias ) (+ res) for up to kRowsPerBlock rows.  A block owns 32 columns; its
// 16 warps split K into 16 equal segments (kSeg), lane = column, so a warp reads 128 contiguous
// bytes of W per k.  Inside a segment the terms are accumulated k ascending into one accumulator
// with fused multiply-add; the 16 partial sums are then added in ascending segment order.  (The
// reference's kernel keeps a single accumulator over all of K, src/hip_kernels.cpp:127-140; the
// fixed 16-way split trades that order for sixteen times the loads in flight, and the CPU oracle of
// the generation path follows the same order.)  With ln_g the rows are layer-normalised in
// shared memory first (one warp per row; every block repeats it, which is cheaper than a launch).
constexpr int kSeg = 16;
// One block's share of the matmul: column block bx, row block by.  FUSED = called from the
// persistent generation kernel, where the activations (A, the residual) were written earlier in
// the same launch by other blocks: they are read past L1 (ld.global.cg), never through the
// read-only path.
template <bool FUSED>
__device__ __forceinline__ void matmul_rows_body(int bx, int by, float *a_s, const float *A, int lda,
                                                 const float *__restrict__ ln_g, const float *__restrict__ ln_b,
                                                 const float *__restrict__ W, const float *__restrict__ bias, const MatmulOut &o,
                                                 int M, int K, int N, int relu)
{
    const int m0 = by * kRowsPerBlock;
    const int rows = min(kRowsPerBlock, M - m0);
    float *part = a_s + kRowsPerBlock * K;          // a_s: [rows][K] activations, then [kSeg][rows][32] partial sums
    const int seg = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < rows * K; i += blockDim.x)
        a_s[i] = FUSED ? __ldcg(A + (size_t)(m0 + i / K) * lda + i % K) : A[(size_t)(m0 + i / K) * lda + i % K];
    __syncthreads();
    if (ln_g) {
        if (seg < rows) layernorm_row(a_s + seg * K, ln_g, ln_b, K, lane);
        __syncthreads();
    }
    const int n = bx * 32 + lane;
    const int klen = K / kSeg, k0 = seg * klen;
    float acc[kRowsPerBlock];
#pragma unroll
    for (int m = 0; m < kRowsPerBlock; ++m) acc[m] = 0.0f;
    if (n < N) {
        const float *wp = W + (size_t)k0 * N + n;
        int k = 0;
        for (; k + 16 <= klen; k += 16) {
            float w[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) w[u] = __ldg(wp + (size_t)(k + u) * N);     // sixteen loads in flight
#pragma unroll
            for (int u = 0; u < 16; ++u)
#pragma unroll
                for (int m = 0; m < kRowsPerBlock; ++m)
                    if (m < rows) acc[m] = fmaf(a_s[m * K + k0 + k + u], w[u], acc[m]);
        }
        for (; k < klen; ++k) {
            const float w = __ldg(wp + (size_t)k * N);
#pragma unroll
            for (int m = 0; m < kRowsPerBlock; ++m)
                if (m < rows) acc[m] = fmaf(a_s[m * K + k0 + k], w, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < kRowsPerBlock; ++m) part[(seg * kRowsPerBlock + m) * 32 + lane] = acc[m];
    __syncthreads();
    // the first 256 threads finish the 8 x 32 outputs of the block: thread -> (row, column)
    const int m = threadIdx.x >> 5;
    if (m < kRowsPerBlock && m < rows && n < N) {
        float v = part[m * 32 + lane];
#pragma unroll
        for (int s2 = 1; s2 < kSeg; ++s2) v = __fadd_rn(v, part[(s2 * kRowsPerBlock + m) * 32 + lane]);
        if (bias) v = __fadd_rn(v, bias[n]);
        if (relu) v = fmaxf(0.0f, v);
        const int row = m0 + m;
        if (o.q) {
            const int p = o.pos_ptr ? *o.pos_ptr : o.p_fixed;
            if (n < o.E) o.q[(size_t)row * o.E + n] = v;
            else if (n < 2 * o.E) o.kc[((size_t)row * o.cap + p) * o.E + (n - o.E)] = v;
            else o.vc[((size_t)row * o.cap + p) * o.E + (n - 2 * o.E)] = v;
        } else {
            if (o.res) v = __fadd_rn(FUSED ? __ldcg(o.res + (size_t)row * o.ldo + n) : o.res[(size_t)row * o.ldo + n], v);
            o.out[(size_t)row * o.ldo + n] = v;
        }
    }
}

__global__ void __launch_bounds__(32 * kSeg)
matmul_rows_kernel(const float *__restrict__ A, int lda, const float *__restrict__ ln_g, const float *__restrict__ ln_b,
                   const float *__restrict__ W, const float *__restrict__ bias, MatmulOut o, int M, int K, int N, int relu)
{
    extern __shared__ float a_s[];
    dependency_wait();
    dependents_may_start();
    matmul_rows_body<false>(blockIdx.x, blockIdx.y, a_s, A, lda, ln_g, ln_b, W, bias, o, M, K, N, relu);
}

// first maximum of each row (lowest index wins ties) -> ids_next[b]; recorded in out_ids once the
// prompt's last position has been reached
__global__ void __launch_bounds__(256)
argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ ids_next, int *__restrict__ out_ids, int n_new,
              int n_prompt, const int *__restrict__ pos_ptr)
{
    __shared__ float sv[256];
    __shared__ int si[256];
    dependency_wait();
    dependents_may_start();
    const int b = blockIdx.x;
    const float *row = logits + (size_t)b * V;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v = threadIdx.x; v < V; v += blockDim.x) {
        const float x = row[v];
        if (x > best || bi == 0x7fffffff) { best = x; bi = v; }     // ascending v per thread: strict > keeps the first
    }
    sv[threadIdx.x] = best;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = sv[threadIdx.x + s];
            const int oi = si[threadIdx.x + s];
            if (oi != 0x7fffffff && (si[threadIdx.x] == 0x7fffffff || ov > sv[threadIdx.x] ||
                                     (ov == sv[threadIdx.x] && oi < si[threadIdx.x]))) {
                sv[threadIdx.x] = ov;
                si[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        ids_next[b] = si[0];
        const int col = *pos_ptr - (n_prompt - 1);
        if (col >= 0 && col < n_new) out_ids[(size_t)b * n_new + col] = si[0];
    }
}

__global__ void advance_pos_kernel(int *pos_ptr)
{
    dependency_wait();
    dependents_may_start();
    *pos_ptr += 1;
}

struct LayerW {
    const float *wqkv, *wo, *w1, *w2, *bqkv, *bo, *b1, *b2, *g1, *be1, *g2, *be2;
};

// ------------------------------------------------------------------------------------------------
// The persistent form: ONE cooperative launch runs `nsteps` token positions.  A step of the graph
// form is 52 launches of a few microseconds each; here the same phases (the same device
// functions, the same arithmetic; the split of a (batch, head) that finishes last merges the
// attention partials instead of a kernel of its own) follow one another inside the kernel,
// separated by a barrier over the grid.  Measured on B200 at the default model, batch 8: 335 us
// per step against 327 us of the replayed graph - a barrier over 148 blocks costs about what a
// launch inside a graph costs, and the phases themselves (a few blocks each, chains of L2 round
// trips) are the larger part of both.  Selectable (hipgpt_gpt_set_mode), not the default.  The grid is one
// block per SM, co-resident by the cooperative launch.  The barrier is a counter and a
// generation word in global memory; its wait is bounded: when it runs out, the block raises the
// error word, every other block sees it in its own wait, and all of them return.
struct FusedArgs {
    const float *tok, *pos, *wout;
    const LayerW *layers;            // device copy, L entries
    int V, S, E, L, H, F;
    float *kc, *vc;                  // [L][max_batch][S][E]
    size_t layer_stride;             // floats between the caches of two layers
    float *x, *q, *att, *ff, *logits, *scratch;
    int *ids, *out_ids, *pos_ptr;
    const int *prompts;
    int B, n_prompt, n_new, nsteps, ns;
    unsigned *bar;                   // [0] arrivals, [1] generation
    long long bar_limit;             // SM cycles a block waits at the barrier before it gives up
    unsigned *cnt;                   // [B*H] splits of a (batch, head) that have finished, zero between phases
    int *err;
};

constexpr long long kBarrierLimitCycles = 4000000000LL;     // about two seconds

__device__ __forceinline__ bool grid_barrier(const FusedArgs &a, unsigned &gen, int *ok_s)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        const unsigned target = gen + 1;
        // the arrival releases this block's writes (the other threads' through the barrier above) and
        // acquires those of the blocks that arrived before; the last one publishes the generation
        unsigned old;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.bar) : "memory");
        if (old == gridDim.x - 1) {
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(a.bar), "r"(0u) : "memory");
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.bar + 1), "r"(target) : "memory");
        } else {
            const long long t0 = clock64();
            unsigned seen, spins = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.bar + 1) : "memory");
                if (seen == target) break;
                if ((++spins & 63u) == 0u) {
                    if (*reinterpret_cast<volatile int *>(a.err) != 0) { ok = 0; break; }
                    if (clock64() - t0 > a.bar_limit) { atomicExch(a.err, 1); ok = 0; break; }
                }
            }
        }
        *ok_s = ok;
    }
    __syncthreads();
    gen += 1;
    return *ok_s != 0;
}

// the arithmetic of decode_split_vec_kernel<LPK> (attn_decode.cu) for four of its 128-thread
// blocks at a time; q and the caches were written earlier in this launch and are read past L1
template <int LPK>
__device__ __forceinline__ void attn_split_phase(const FusedArgs &a, const float *kc, const float *vc, int ctx, float *sm)
{
    constexpr int KPW = 32 / LPK, W4 = 4;
    const int H = a.H, E = a.E, D = E / H, cap = a.S, ns = a.ns;
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    const int sub = threadIdx.x >> 7, t = threadIdx.x & 127, warp = t >> 5, lane = t & 31;
    const int lik = lane % LPK, kg = lane / LPK;
    const bool act = lik * 4 < D;
    const int stride = ((D + 3) / 4) * 4 + 4;
    float *smb = sm + sub * (W4 * LPK * 6);          // [warp][lik][6]
    const int nvb = ns * a.B * H;
    for (int vb0 = blockIdx.x * 4; vb0 < nvb; vb0 += gridDim.x * 4) {
        const int vb = vb0 + sub;
        const bool live = vb < nvb;
        const int split = live ? vb % ns : 0, bh = live ? vb / ns : 0;
        const int b = bh / H, h = bh % H;
        const size_t col = (size_t)h * D + lik * 4;
        const int per = (ctx + ns - 1) / ns;
        const int k0 = split * per, k1 = min(ctx, k0 + per);
        Partial4f acc{-1e30f, 0.0f, make_float4(0.f, 0.f, 0.f, 0.f)};
        if (live) {
            float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (act) {
                q4 = __ldcg(reinterpret_cast<const float4 *>(a.q + (size_t)b * E + col));
                q4.x *= qscale; q4.y *= qscale; q4.z *= qscale; q4.w *= qscale;
            }
            const int steps = (max(k1 - k0, 0) + W4 * KPW - 1) / (W4 * KPW);
            for (int it = 0; it < steps; ++it) {
                const int j = k0 + (it * W4 + warp) * KPW + kg;
                const bool valid = j < k1;
                float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), v4 = k4;
                if (valid && act) {
                    const size_t off = ((size_t)b * cap + j) * (size_t)E + col;
                    k4 = __ldcg(reinterpret_cast<const float4 *>(kc + off));
                    v4 = __ldcg(reinterpret_cast<const float4 *>(vc + off));
                }
                float s = q4.x * k4.x;
                s = fmaf(q4.y, k4.y, s);
                s = fmaf(q4.z, k4.z, s);
                s = fmaf(q4.w, k4.w, s);
#pragma unroll
                for (int off = 1; off < LPK; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
                if (!valid) s = -INFINITY;
                const float mn = fmaxf(acc.m, s);
                const float alpha = ex2_approx(acc.m - mn), pr = ex2_approx(s - mn);
                acc.l = fmaf(acc.l, alpha, pr);
                acc.o.x = fmaf(pr, v4.x, acc.o.x * alpha);
                acc.o.y = fmaf(pr, v4.y, acc.o.y * alpha);
                acc.o.z = fmaf(pr, v4.z, acc.o.z * alpha);
                acc.o.w = fmaf(pr, v4.w, acc.o.w * alpha);
                acc.m = mn;
            }
#pragma unroll
            for (int off = LPK; off < 32; off <<= 1) {
                const float m2 = __shfl_xor_sync(0xffffffffu, acc.m, off);
                const float l2 = __shfl_xor_sync(0xffffffffu, acc.l, off);
                float4 o2;
                o2.x = __shfl_xor_sync(0xffffffffu, acc.o.x, off);
                o2.y = __shfl_xor_sync(0xffffffffu, acc.o.y, off);
                o2.z = __shfl_xor_sync(0xffffffffu, acc.o.z, off);
                o2.w = __shfl_xor_sync(0xffffffffu, acc.o.w, off);
                merge_partial(acc, m2, l2, o2);
            }
            if (kg == 0) {
                float *r = smb + (warp * LPK + lik) * 6;
                r[0] = acc.m; r[1] = acc.l; r[2] = acc.o.x; r[3] = acc.o.y; r[4] = acc.o.z; r[5] = acc.o.w;
            }
        }
        __syncthreads();
        if (live && warp == 0) {
            if (lane < LPK) {
                const float *r0 = smb + lane * 6;
                Partial4f tt{r0[0], r0[1], make_float4(r0[2], r0[3], r0[4], r0[5])};
#pragma unroll
                for (int w = 1; w < W4; ++w) {
                    const float *r = smb + (w * LPK + lane) * 6;
                    merge_partial(tt, r[0], r[1], make_float4(r[2], r[3], r[4], r[5]));
                }
                if (lane * 4 < D) {
                    if (ns == 1) {
                        const float inv = 1.0f / fmaxf(tt.l, 1e-20f);
                        *reinterpret_cast<float4 *>(a.att + (size_t)b * E + (size_t)h * D + lane * 4) =
                            make_float4(tt.o.x * inv, tt.o.y * inv, tt.o.z * inv, tt.o.w * inv);
                    } else {
                        float *rec = a.scratch + ((size_t)bh * ns + split) * stride;
                        *reinterpret_cast<float4 *>(rec + lane * 4) = tt.o;
                        if (lane == 0) { rec[stride - 4] = tt.m; rec[stride - 3] = tt.l; }
                    }
                }
            }
            if (ns > 1) {
                // the split that finishes last for this (batch, head) merges the ns records: what
                // decode_combine_kernel (attn_decode.cu) computes, element d by lane d, d + 32, ...
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    unsigned old;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.cnt + bh) : "memory");
                    last = old == (unsigned)(ns - 1);
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    const float *rec = a.scratch + (size_t)bh * ns * stride;
                    float M = -1e30f, L = 0.0f;
                    if (ns <= 8) {                   // all loads of a pass in flight at once
                        float ms[8], ls[8];
#pragma unroll
                        for (int s = 0; s < 8; ++s)
                            if (s < ns) { ms[s] = __ldcg(rec + (size_t)s * stride + stride - 4); ls[s] = __ldcg(rec + (size_t)s * stride + stride - 3); }
#pragma unroll
                        for (int s = 0; s < 8; ++s) if (s < ns) M = fmaxf(M, ms[s]);
#pragma unroll
                        for (int s = 0; s < 8; ++s) if (s < ns) L += ls[s] * ex2_approx(ms[s] - M);
                        const float inv = 1.0f / fmaxf(L, 1e-20f);
                        for (int d = lane; d < D; d += 32) {
                            float os[8];
#pragma unroll
                            for (int s = 0; s < 8; ++s) if (s < ns) os[s] = __ldcg(rec + (size_t)s * stride + d);
                            float av = 0.0f;
#pragma unroll
                            for (int s = 0; s < 8; ++s) if (s < ns) av += os[s] * ex2_approx(ms[s] - M);
                            a.att[(size_t)b * E + (size_t)h * D + d] = av * inv;
                        }
                    } else {
                        for (int s = 0; s < ns; ++s) M = fmaxf(M, __ldcg(rec + (size_t)s * stride + stride - 4));
                        for (int s = 0; s < ns; ++s)
                            L += __ldcg(rec + (size_t)s * stride + stride - 3) * ex2_approx(__ldcg(rec + (size_t)s * stride + stride - 4) - M);
                        const float inv = 1.0f / fmaxf(L, 1e-20f);
                        for (int d = lane; d < D; d += 32) {
                            float av = 0.0f;
                            for (int s = 0; s < ns; ++s)
                                av += __ldcg(rec + (size_t)s * stride + d) * ex2_approx(__ldcg(rec + (size_t)s * stride + stride - 4) - M);
                            a.att[(size_t)b * E + (size_t)h * D + d] = av * inv;
                        }
                    }
                    if (lane == 0) a.cnt[bh] = 0u;   // next used after a barrier over the grid
                }
            }
        }
        __syncthreads();
    }
}


__global__ void __launch_bounds__(32 * kSeg, 1)
gpt_steps_kernel(const FusedArgs a)
{
    extern __shared__ float dsm[];                   // the matmul's rows and partial sums; the other phases' scratch
    __shared__ int ok_s;
    const int B = a.B, E = a.E, F = a.F, V = a.V, D = a.E / a.H;
    unsigned gen = *reinterpret_cast<volatile unsigned *>(a.bar + 1);   // read before this block's first arrival: cannot move yet
    const int p0 = __ldcg(a.pos_ptr);
    const int mrows = (B + kRowsPerBlock - 1) / kRowsPerBlock;
    // one matmul phase: its blocks (column block, row block) are dealt out over the grid
    auto matmul_phase = [&](const float *A, int lda, const float *ln_g, const float *ln_b, const float *W,
                            const float *bias, const MatmulOut &o, int K, int N, int relu) {
        const int nbx = (N + 31) / 32;
        for (int vb = blockIdx.x; vb < nbx * mrows; vb += gridDim.x) {
            matmul_rows_body<true>(vb % nbx, vb / nbx, dsm, A, lda, ln_g, ln_b, W, bias, o, B, K, N, relu);
            __syncthreads();                         // the rows and partial sums are reused by the next block of work
        }
    };
    for (int step = 0; step < a.nsteps; ++step) {
        const int p = p0 + step;
        // embedding: x[b] = tok[id] + pos[p]
        for (int b = blockIdx.x; b < B; b += gridDim.x) {
            const int id = p < a.n_prompt ? a.prompts[(size_t)b * a.n_prompt + p] : __ldcg(a.ids + b);
            const bool ok = id >= 0 && id < V;
            for (int e = threadIdx.x; e < E; e += blockDim.x)
                a.x[(size_t)b * E + e] = ok ? __fadd_rn(a.tok[(size_t)id * E + e], a.pos[(size_t)p * E + e]) : 0.0f;
        }
        if (!grid_barrier(a, gen, &ok_s)) return;
        for (int l = 0; l < a.L; ++l) {
            const LayerW w = a.layers[l];
            float *kc = a.kc + (size_t)l * a.layer_stride, *vc = a.vc + (size_t)l * a.layer_stride;
            const MatmulOut scatter{nullptr, 0, nullptr, a.q, kc, vc, nullptr, a.S, E, p};
            matmul_phase(a.x, E, w.g1, w.be1, w.wqkv, w.bqkv, scatter, E, 3 * E, 0);
            if (!grid_barrier(a, gen, &ok_s)) return;
            if (D <= 32) attn_split_phase<8>(a, kc, vc, p + 1, dsm);
            else if (D <= 64) attn_split_phase<16>(a, kc, vc, p + 1, dsm);
            else attn_split_phase<32>(a, kc, vc, p + 1, dsm);
            if (!grid_barrier(a, gen, &ok_s)) return;
            const MatmulOut to_x{a.x, E, a.x, nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
            matmul_phase(a.att, E, nullptr, nullptr, w.wo, w.bo, to_x, E, E, 0);
            if (!grid_barrier(a, gen, &ok_s)) return;
            const MatmulOut to_ff{a.ff, F, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
            matmul_phase(a.x, E, w.g2, w.be2, w.w1, w.b1, to_ff, E, F, 1);
            if (!grid_barrier(a, gen, &ok_s)) return;
            matmul_phase(a.ff, F, nullptr, nullptr, w.w2, w.b2, to_x, F, E, 0);
            if (!grid_barrier(a, gen, &ok_s)) return;
        }
        const MatmulOut to_logits{a.logits, V, nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, 0};
        matmul_phase(a.x, E, nullptr, nullptr, a.wout, nullptr, to_logits, E, V, 0);
        if (!grid_barrier(a, gen, &ok_s)) return;
        // first maximum of each row of the logits (lowest index wins ties)
        for (int b = blockIdx.x; b < B; b += gridDim.x) {
            float *sv = dsm;
            int *si = reinterpret_cast<int *>(dsm + blockDim.x);
            const float *row = a.logits + (size_t)b * V;
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int v = threadIdx.x; v < V; v += blockDim.x) {
                const float xv = __ldcg(row + v);
                if (xv > best || bi == 0x7fffffff) { best = xv; bi = v; }
            }
            sv[threadIdx.x] = best;
            si[threadIdx.x] = bi;
            __syncthreads();
            for (int s2 = blockDim.x >> 1; s2 > 0; s2 >>= 1) {
                if ((int)threadIdx.x < s2) {
                    const float ov = sv[threadIdx.x + s2];
                    const int oi = si[threadIdx.x + s2];
                    if (oi != 0x7fffffff && (si[threadIdx.x] == 0x7fffffff || ov > sv[threadIdx.x] ||
                                             (ov == sv[threadIdx.x] && oi < si[threadIdx.x]))) {
                        sv[threadIdx.x] = ov;
                        si[threadIdx.x] = oi;
                    }
                }
                __syncthreads();
            }
            if (threadIdx.x == 0) {
                a.ids[b] = si[0];
                const int col = p - (a.n_prompt - 1);
                if (col >= 0 && col < a.n_new) a.out_ids[(size_t)b * a.n_new + col] = si[0];
            }
            __syncthreads();
        }
        if (!grid_barrier(a, gen, &ok_s)) return;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.pos_ptr = p0 + a.nsteps;
}

}  // namespace

struct GptDecoder {
    int V, S, E, L, H, F, max_batch;
    float *d_weights = nullptr;
    const float *tok = nullptr, *pos = nullptr, *wout = nullptr;
    std::vector<LayerW> lw;
    float *d_kc = nullptr, *d_vc = nullptr;        // [L][max_batch][S][E]
    float *d_x = nullptr, *d_h = nullptr, *d_qkv = nullptr, *d_q = nullptr, *d_att = nullptr, *d_ff = nullptr, *d_logits = nullptr;
    float *d_scratch = nullptr;
    size_t scratch_bytes = 0;
    int *d_ids = nullptr, *d_out = nullptr, *d_pos = nullptr, *d_prompts = nullptr;
    int out_cap = 0, prompt_cap = 0;
    cudaStream_t stream = nullptr;
    // one step of generation captured as a CUDA graph; valid for (graph_B, graph_n_prompt, graph_n_new)
    cudaGraphExec_t graph = nullptr;
    int graph_B = 0, graph_n_prompt = 0, graph_n_new = 0;
    // the persistent form (gpt_steps_kernel): device copy of the layer table, barrier words, error word
    LayerW *d_layers = nullptr;
    unsigned *d_bar = nullptr, *d_cnt = nullptr;
    int *d_err = nullptr;
    int mode = HIPGPT_GPT_MODE_GRAPH;                // measured: the persistent form is no faster (335 against 327 us per step)
    bool persistent_ok = false;                      // head_dim, shared memory and co-residency allow it
    int grid_blocks = 0;
    size_t fused_smem = 0;
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};   // start, prompt done, all done
    // test hook (hipgpt_gpt_debug_stall_barrier): the next persistent call starts with an arrival counter
    // that can never complete and this wait limit, so that the barrier's give-up path runs
    bool stall_next = false;
    long long stall_limit = 0;
};

namespace {

#define CUDA_OK(call)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

long long weight_count(int V, int S, int E, int L, int F)
{
    const long long per_layer = (long long)E * 3 * E + (long long)E * E + (long long)E * F + (long long)F * E +
                                3LL * E + E + F + E + 4LL * E;
    return (long long)V * E + (long long)S * E + L * per_layer + (long long)E * V;
}

int matmul(const GptDecoder &g, const float *A, int lda, const float *ln_g, const float *ln_b, const float *W,
           const float *bias, const MatmulOut &o, int M, int K, int N, int relu)
{
    const dim3 grid((N + 31) / 32, (M + kRowsPerBlock - 1) / kRowsPerBlock);
    const size_t smem = (size_t)kRowsPerBlock * (K + kSeg * 32) * sizeof(float);
    const cudaError_t le = launch_overlapped(matmul_rows_kernel, grid, dim3(32 * kSeg), smem, g.stream, A, lda, ln_g, ln_b, W, bias, o, M, K, N, relu);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "matmul_rows_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("matmul_rows_kernel");
}

MatmulOut plain_out(float *out, int ldo, const float *res) { return MatmulOut{out, ldo, res, nullptr, nullptr, nullptr, nullptr, 0, 0, 0}; }

// One token position for all B sequences, every launch reading the position from g.d_pos: embed,
// L x {LN+QKV projection scattered into q and the caches, split-context attention, output
// projection + residual, LN+FF1+ReLU, FF2 + residual}, logits, first-maximum pick, position + 1.
int enqueue_step(GptDecoder &g, int B, int n_prompt, int n_new)
{
    const int E = g.E, F = g.F, V = g.V, D = g.E / g.H;
    // every launch of the step is an overlapped one (captured into the graph as programmatic dependencies): a kernel's
    // blocks are placed while the kernel before it drains and wait for it before their first read
    cudaError_t le = launch_overlapped(embed_kernel, dim3(B), dim3(128), 0, g.stream, (const int *)g.d_prompts, n_prompt, (const int *)g.d_ids, (const int *)g.d_pos,
                                       (const float *)g.tok, (const float *)g.pos, g.d_x, E, V);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "embed_kernel launch: %s", cudaGetErrorString(le));
    int rc = check_launch("embed_kernel");
    if (rc) return rc;
    const int ns = decode_splits(B, g.H, D, g.S);        // fixed for the whole graph; short contexts leave splits empty
    for (int l = 0; l < g.L; ++l) {
        const LayerW &w = g.lw[l];
        float *kc = g.d_kc + (size_t)l * g.max_batch * g.S * E;
        float *vc = g.d_vc + (size_t)l * g.max_batch * g.S * E;
        const MatmulOut scatter{nullptr, 0, nullptr, g.d_q, kc, vc, g.d_pos, g.S, E, 0};
        if ((rc = matmul(g, g.d_x, E, w.g1, w.be1, w.wqkv, w.bqkv, scatter, B, E, 3 * E, 0))) return rc;
        if ((rc = launch_decode(g.d_q, kc, vc, g.d_att, g.d_scratch, B, g.H, D, 1, g.S, ns, g.stream, g.d_pos))) return rc;
        if ((rc = matmul(g, g.d_att, E, nullptr, nullptr, w.wo, w.bo, plain_out(g.d_x, E, g.d_x), B, E, E, 0))) return rc;
        if ((rc = matmul(g, g.d_x, E, w.g2, w.be2, w.w1, w.b1, plain_out(g.d_ff, F, nullptr), B, E, F, 1))) return rc;
        if ((rc = matmul(g, g.d_ff, F, nullptr, nullptr, w.w2, w.b2, plain_out(g.d_x, E, g.d_x), B, F, E, 0))) return rc;
    }
    if ((rc = matmul(g, g.d_x, E, nullptr, nullptr, g.wout, nullptr, plain_out(g.d_logits, V, nullptr), B, E, V, 0))) return rc;
    le = launch_overlapped(argmax_kernel, dim3(B), dim3(256), 0, g.stream, (const float *)g.d_logits, V, g.d_ids, g.d_out, n_new, n_prompt, (const int *)g.d_pos);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "argmax_kernel launch: %s", cudaGetErrorString(le));
    if ((rc = check_launch("argmax_kernel"))) return rc;
    le = launch_overlapped(advance_pos_kernel, dim3(1), dim3(1), 0, g.stream, g.d_pos);
    if (le != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "advance_pos_kernel launch: %s", cudaGetErrorString(le));
    return check_launch("advance_pos_kernel");
}

int build_graph(GptDecoder &g, int B, int n_prompt, int n_new)
{
    if (g.graph && g.graph_B == B && g.graph_n_prompt == n_prompt && g.graph_n_new == n_new) return HIPGPT_OK;
    if (g.graph) { cudaGraphExecDestroy(g.graph); g.graph = nullptr; }
    cudaGraph_t captured = nullptr;
    CUDA_OK(cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_step(g, B, n_prompt, n_new);
    const cudaError_t e = cudaStreamEndCapture(g.stream, &captured);
    if (rc != HIPGPT_OK) { if (captured) cudaGraphDestroy(captured); return rc; }
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    const cudaError_t e2 = cudaGraphInstantiate(&g.graph, captured, 0);
    cudaGraphDestroy(captured);
    if (e2 != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e2));
    g.graph_B = B; g.graph_n_prompt = n_prompt; g.graph_n_new = n_new;
    return HIPGPT_OK;
}

}  // namespace
}  // namespace hipgpt

using namespace hipgpt;

extern "C" {

long long hipgpt_gpt_weight_count(int V, int S, int E, int L, int H, int F)
{
    (void)H;
    return weight_count(V, S, E, L, F);
}

int hipgpt_gpt_create(hipgpt_gpt **out, const float *h_weights, int V, int S, int E, int L, int H, int F, int max_batch)
{
    if (!out || !h_weights) return fail(HIPGPT_ERR_NULL, "out and h_weights must not be NULL");
    if (V <= 0 || S <= 0 || E <= 0 || L <= 0 || H <= 0 || F <= 0 || E % H || max_batch <= 0 || E % 16 || F % 16 || F > 6000 || E > 6000)
        return fail(HIPGPT_ERR_BAD_ARG, "bad model shape V=%d S=%d E=%d L=%d H=%d F=%d batch=%d", V, S, E, L, H, F, max_batch);
    GptDecoder *g = new (std::nothrow) GptDecoder();
    if (!g) return fail(HIPGPT_ERR_CUDA, "out of host memory");
    g->V = V; g->S = S; g->E = E; g->L = L; g->H = H; g->F = F; g->max_batch = max_batch;
    const long long nw = weight_count(V, S, E, L, F);
    auto bail = [&](int rc) { hipgpt_gpt_destroy(reinterpret_cast<hipgpt_gpt *>(g)); return rc; };
#define TRY(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return bail(fail(HIPGPT_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_))); } while (0)
    TRY(cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking));
    TRY(cudaMalloc(&g->d_weights, (size_t)nw * sizeof(float)));
    TRY(cudaMemcpyAsync(g->d_weights, h_weights, (size_t)nw * sizeof(float), cudaMemcpyHostToDevice, g->stream));
    const float *p = g->d_weights;
    auto take = [&](long long n) { const float *r = p; p += n; return r; };
    g->tok = take((long long)V * E);
    g->pos = take((long long)S * E);
    g->lw.resize(L);
    for (int l = 0; l < L; ++l) {
        LayerW &w = g->lw[l];
        w.wqkv = take((long long)E * 3 * E); w.wo = take((long long)E * E); w.w1 = take((long long)E * F); w.w2 = take((long long)F * E);
        w.bqkv = take(3LL * E); w.bo = take(E); w.b1 = take(F); w.b2 = take(E);
        w.g1 = take(E); w.be1 = take(E); w.g2 = take(E); w.be2 = take(E);
    }
    g->wout = take((long long)E * V);
    const size_t cache = (size_t)L * max_batch * S * E * sizeof(float);
    TRY(cudaMalloc(&g->d_kc, cache));
    TRY(cudaMalloc(&g->d_vc, cache));
    TRY(cudaMalloc(&g->d_x, (size_t)max_batch * E * sizeof(float)));
    TRY(cudaMalloc(&g->d_h, (size_t)max_batch * E * sizeof(float)));
    TRY(cudaMalloc(&g->d_qkv, (size_t)max_batch * 3 * E * sizeof(float)));
    TRY(cudaMalloc(&g->d_q, (size_t)max_batch * E * sizeof(float)));
    TRY(cudaMalloc(&g->d_att, (size_t)max_batch * E * sizeof(float)));
    TRY(cudaMalloc(&g->d_ff, (size_t)max_batch * F * sizeof(float)));
    TRY(cudaMalloc(&g->d_logits, (size_t)max_batch * V * sizeof(float)));
    TRY(cudaMalloc(&g->d_ids, (size_t)max_batch * sizeof(int)));
    TRY(cudaMalloc(&g->d_pos, sizeof(int)));
    TRY(cudaMemsetAsync(g->d_ids, 0, (size_t)max_batch * sizeof(int), g->stream));
    size_t sb = 0;
    for (int ctx = 1; ctx <= S; ++ctx) {
        const size_t b = hipgpt_mha_decode_scratch_bytes(max_batch, H, E / H, ctx);
        if (b > sb) sb = b;
    }
    for (int b2 = 1; b2 < max_batch; ++b2)
        for (int ctx = 32; ctx <= S; ctx += 32) {
            const size_t b = hipgpt_mha_decode_scratch_bytes(b2, H, E / H, ctx);
            if (b > sb) sb = b;
        }
    g->scratch_bytes = sb ? sb : 16;
    TRY(cudaMalloc(&g->d_scratch, g->scratch_bytes));
    {
        const int need = kRowsPerBlock * ((E > F ? E : F) + kSeg * 32) * (int)sizeof(float);   // activation rows of the widest matmul + partial sums
        if (need > 48 * 1024) TRY(cudaFuncSetAttribute(matmul_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, need));
    }
    {
        // the persistent kernel: one block per SM, all resident at once (checked here, enforced by the cooperative launch)
        const int D = E / H;
        int dev = 0, sms = 0, coop = 0, per_sm = 0;
        TRY(cudaGetDevice(&dev));
        TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        g->fused_smem = (size_t)kRowsPerBlock * ((E > F ? E : F) + kSeg * 32) * sizeof(float);
        if (g->fused_smem < 16 * 1024) g->fused_smem = 16 * 1024;      // the attention and first-maximum phases' scratch
        TRY(cudaFuncSetAttribute(gpt_steps_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g->fused_smem));
        TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gpt_steps_kernel, 32 * kSeg, g->fused_smem));
        g->persistent_ok = coop && per_sm >= 1 && D % 4 == 0 && D <= 128;
        g->grid_blocks = sms;
        TRY(cudaMalloc(&g->d_layers, (size_t)L * sizeof(LayerW)));
        TRY(cudaMemcpyAsync(g->d_layers, g->lw.data(), (size_t)L * sizeof(LayerW), cudaMemcpyHostToDevice, g->stream));
        TRY(cudaMalloc(&g->d_bar, 2 * sizeof(unsigned)));
        TRY(cudaMemsetAsync(g->d_bar, 0, 2 * sizeof(unsigned), g->stream));
        TRY(cudaMalloc(&g->d_cnt, (size_t)max_batch * H * sizeof(unsigned)));
        TRY(cudaMemsetAsync(g->d_cnt, 0, (size_t)max_batch * H * sizeof(unsigned), g->stream));
        TRY(cudaMalloc(&g->d_err, sizeof(int)));
        TRY(cudaMemsetAsync(g->d_err, 0, sizeof(int), g->stream));
    }
    TRY(cudaStreamSynchronize(g->stream));
#undef TRY
    *out = reinterpret_cast<hipgpt_gpt *>(g);
    return HIPGPT_OK;
}

int hipgpt_gpt_generate(hipgpt_gpt *handle, const int *h_prompts, int B, int n_prompt, int n_new, int *h_out_ids,
                        float *h_logits_last, float *ms_prompt, float *ms_decode)
{
    GptDecoder *g = reinterpret_cast<GptDecoder *>(handle);
    if (!g || !h_prompts || !h_out_ids) return fail(HIPGPT_ERR_NULL, "handle, prompts and out_ids must not be NULL");
    if (B <= 0 || B > g->max_batch || n_prompt <= 0 || n_new <= 0 || n_prompt + n_new - 1 > g->S)
        return fail(HIPGPT_ERR_BAD_ARG, "bad request: B=%d (max %d) n_prompt=%d n_new=%d S=%d", B, g->max_batch, n_prompt, n_new, g->S);
    if (g->out_cap < B * n_new) {
        if (g->d_out) cudaFree(g->d_out);
        g->d_out = nullptr;
        g->graph_B = 0;                      // the captured step holds the old pointer
        CUDA_OK(cudaMalloc(&g->d_out, (size_t)B * n_new * sizeof(int)));
        g->out_cap = B * n_new;
    }
    if (g->prompt_cap < B * n_prompt) {
        if (g->d_prompts) cudaFree(g->d_prompts);
        g->d_prompts = nullptr;
        g->graph_B = 0;
        CUDA_OK(cudaMalloc(&g->d_prompts, (size_t)B * n_prompt * sizeof(int)));
        g->prompt_cap = B * n_prompt;
    }
    const bool persistent = g->mode == HIPGPT_GPT_MODE_PERSISTENT && g->persistent_ok;
    int rc = persistent ? HIPGPT_OK : build_graph(*g, B, n_prompt, n_new);
    if (rc != HIPGPT_OK) return rc;
    CUDA_OK(cudaMemcpyAsync(g->d_prompts, h_prompts, (size_t)B * n_prompt * sizeof(int), cudaMemcpyHostToDevice, g->stream));
    CUDA_OK(cudaMemsetAsync(g->d_pos, 0, sizeof(int), g->stream));
    for (cudaEvent_t &ev : g->ev)
        if (!ev) CUDA_OK(cudaEventCreate(&ev));
    const cudaEvent_t e0 = g->ev[0], e1 = g->ev[1], e2 = g->ev[2];
    CUDA_OK(cudaEventRecord(e0, g->stream));
    if (persistent) {
        FusedArgs a{};
        a.tok = g->tok; a.pos = g->pos; a.wout = g->wout; a.layers = g->d_layers;
        a.V = g->V; a.S = g->S; a.E = g->E; a.L = g->L; a.H = g->H; a.F = g->F;
        a.kc = g->d_kc; a.vc = g->d_vc; a.layer_stride = (size_t)g->max_batch * g->S * g->E;
        a.x = g->d_x; a.q = g->d_q; a.att = g->d_att; a.ff = g->d_ff; a.logits = g->d_logits; a.scratch = g->d_scratch;
        a.ids = g->d_ids; a.out_ids = g->d_out; a.pos_ptr = g->d_pos; a.prompts = g->d_prompts;
        a.B = B; a.n_prompt = n_prompt; a.n_new = n_new; a.ns = decode_splits(B, g->H, g->E / g->H, g->S);
        a.bar = g->d_bar; a.cnt = g->d_cnt; a.err = g->d_err;
        a.bar_limit = kBarrierLimitCycles;
        if (g->stall_next) {
            // arrivals start at the grid size: no block ever sees itself as the last one
            const unsigned poisoned = (unsigned)g->grid_blocks;
            CUDA_OK(cudaMemcpyAsync(g->d_bar, &poisoned, sizeof(unsigned), cudaMemcpyHostToDevice, g->stream));
            CUDA_OK(cudaStreamSynchronize(g->stream));
            a.bar_limit = g->stall_limit;
            g->stall_next = false;
        }
        void *params[] = {&a};
        a.nsteps = n_prompt;                         // the prompt positions, then the remaining new tokens
        CUDA_OK(cudaLaunchCooperativeKernel((const void *)gpt_steps_kernel, dim3(g->grid_blocks), dim3(32 * kSeg), params, g->fused_smem, g->stream));
        CUDA_OK(cudaEventRecord(e1, g->stream));
        a.nsteps = n_new - 1;
        if (a.nsteps > 0)
            CUDA_OK(cudaLaunchCooperativeKernel((const void *)gpt_steps_kernel, dim3(g->grid_blocks), dim3(32 * kSeg), params, g->fused_smem, g->stream));
    } else {
        for (int p = 0; p < n_prompt; ++p) CUDA_OK(cudaGraphLaunch(g->graph, g->stream));
        CUDA_OK(cudaEventRecord(e1, g->stream));
        for (int i = 1; i < n_new; ++i) CUDA_OK(cudaGraphLaunch(g->graph, g->stream));
    }
    CUDA_OK(cudaEventRecord(e2, g->stream));
    CUDA_OK(cudaMemcpyAsync(h_out_ids, g->d_out, (size_t)B * n_new * sizeof(int), cudaMemcpyDeviceToHost, g->stream));
    if (h_logits_last)
        CUDA_OK(cudaMemcpyAsync(h_logits_last, g->d_logits, (size_t)B * g->V * sizeof(float), cudaMemcpyDeviceToHost, g->stream));
    int h_err = 0;
    if (persistent) CUDA_OK(cudaMemcpyAsync(&h_err, g->d_err, sizeof(int), cudaMemcpyDeviceToHost, g->stream));
    CUDA_OK(cudaStreamSynchronize(g->stream));
    if (h_err) {
        cudaMemsetAsync(g->d_err, 0, sizeof(int), g->stream);
        cudaMemsetAsync(g->d_bar, 0, 2 * sizeof(unsigned), g->stream);
        cudaMemsetAsync(g->d_cnt, 0, (size_t)g->max_batch * g->H * sizeof(unsigned), g->stream);
        cudaStreamSynchronize(g->stream);
        rc = fail(HIPGPT_ERR_CUDA, "persistent generation kernel: a wait at the grid barrier ran out");
    }
    float a = 0.f, b = 0.f;
    cudaEventElapsedTime(&a, e0, e1);
    cudaEventElapsedTime(&b, e1, e2);
    if (ms_prompt) *ms_prompt = a;
    if (ms_decode) *ms_decode = b;
    return rc;
}

int hipgpt_gpt_set_mode(hipgpt_gpt *handle, int mode)
{
    GptDecoder *g = reinterpret_cast<GptDecoder *>(handle);
    if (!g) return fail(HIPGPT_ERR_NULL, "handle must not be NULL");
    if (mode != HIPGPT_GPT_MODE_PERSISTENT && mode != HIPGPT_GPT_MODE_GRAPH) return fail(HIPGPT_ERR_BAD_ARG, "unknown mode %d", mode);
    if (mode == HIPGPT_GPT_MODE_PERSISTENT && !g->persistent_ok)
        return fail(HIPGPT_ERR_UNSUPPORTED, "persistent form needs head_dim %% 4 == 0, head_dim <= 128 and cooperative launch");
    g->mode = mode;
    return HIPGPT_OK;
}

int hipgpt_gpt_debug_stall_barrier(hipgpt_gpt *handle, long long limit_cycles)
{
    GptDecoder *g = reinterpret_cast<GptDecoder *>(handle);
    if (!g) return fail(HIPGPT_ERR_NULL, "handle must not be NULL");
    if (limit_cycles <= 0 || limit_cycles > kBarrierLimitCycles) return fail(HIPGPT_ERR_BAD_ARG, "limit of %lld cycles out of range", limit_cycles);
    if (!(g->mode == HIPGPT_GPT_MODE_PERSISTENT && g->persistent_ok)) return fail(HIPGPT_ERR_UNSUPPORTED, "the handle is not in the persistent mode");
    g->stall_next = true;
    g->stall_limit = limit_cycles;
    return HIPGPT_OK;
}

void hipgpt_gpt_destroy(hipgpt_gpt *handle)
{
    GptDecoder *g = reinterpret_cast<GptDecoder *>(handle);
    if (!g) return;
    float *bufs[] = {g->d_weights, g->d_kc, g->d_vc, g->d_x, g->d_h, g->d_qkv, g->d_q, g->d_att, g->d_ff, g->d_logits, g->d_scratch};
    for (float *b : bufs) if (b) cudaFree(b);
    if (g->graph) cudaGraphExecDestroy(g->graph);
    if (g->d_ids) cudaFree(g->d_ids);
    if (g->d_out) cudaFree(g->d_out);
    if (g->d_pos) cudaFree(g->d_pos);
    if (g->d_prompts) cudaFree(g->d_prompts);
    if (g->d_layers) cudaFree(g->d_layers);
    if (g->d_bar) cudaFree(g->d_bar);
    if (g->d_cnt) cudaFree(g->d_cnt);
    if (g->d_err) cudaFree(g->d_err);
    for (cudaEvent_t ev : g->ev) if (ev) cudaEventDestroy(ev);
    if (g->stream) cudaStreamDestroy(g->stream);
    delete g;
}

}  // extern "C"
