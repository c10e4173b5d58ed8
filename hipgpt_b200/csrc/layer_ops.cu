// The launchers that stand either side of attention in HipGPT's TransformerLayer::forward and
// GPTModel::forward (src/transformer_layer.cpp:214-253, src/gpt_model.cpp:97-118): projections,
// layer norm, dropout, residual add, ReLU, embedding lookup.  Plain sm_100a CUDA with the
// reference's arithmetic restated exactly, so that an unchanged HipGPT layer runs on this library.
//
//   matmul(+bias)   C[M][K] = A[M][N] B[N][K] (+ bias[K]): HipGPT's argument order, N is the inner
//                   dimension (src/hip_kernels.cpp:69-154).  One accumulator per output, terms added
//                   k ascending with fused multiply-add, the bias added once at the end: the
//                   summation order of the reference kernel, hence bit-identical to its arithmetic.
//                   Register-tiled (each thread 64 outputs), operands staged through shared memory.
//   layer norm      src/hip_kernels.cpp:757-848: mean, variance about the mean, 1/sqrt(var + 1e-5),
//                   gamma (x - mean) inv + beta.  One warp per row; the reference reduces in 64-lane
//                   waves, so sums agree to rounding (about 1e-7), not bitwise.
//   dropout         src/hip_kernels.cpp:944-970 with the generator at :24-42: the mask is a pure function
//                   of the element index; restated in integer arithmetic, bit-identical.
//   add, ReLU, embedding lookup   src/hip_kernels.cpp:721-730, :248-258, :537-599; bit-identical.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kGemmThreads = 256;
constexpr int kBK = 16;

// C tile of BM x BN per block, 16 x 16 threads, TM x TN outputs per thread.  A thread's rows are
// contiguous (ty * TM ...), its columns come in groups of four, 64 apart (tx * 4 + 64 j), so that the
// shared-memory reads of a warp are either broadcasts (A) or 256 contiguous bytes (B).
template <int BM, int BN>
__global__ void __launch_bounds__(kGemmThreads)
matmul_exact_kernel(const float *A, const float *__restrict__ B, const float *__restrict__ bias,
                    float *C, int M, int N, int K)          // A and C may be the same buffer (see the launcher)
{
    constexpr int TM = BM / 16, TN = BN / 16, NJ = TN / 4;
    constexpr int A4 = (BM * kBK / 4) / kGemmThreads;      // float4 loads of A per thread and tile
    constexpr int B4 = (kBK * BN / 4) / kGemmThreads;
    __shared__ __align__(16) float As[2][kBK][BM + 4];     // transposed: As[k][m]
    __shared__ __align__(16) float Bs[2][kBK][BN];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    float4 ra[A4], rb[B4];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < A4; ++i) {
            const int f = tid + i * kGemmThreads;            // float4 index inside the A tile: 4 per row
            const int r = row0 + (f >> 2), k = k0 + (f & 3) * 4;
            ra[i] = (r < M && k < N) ? *reinterpret_cast<const float4 *>(A + (size_t)r * N + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < B4; ++i) {
            const int f = tid + i * kGemmThreads;            // BN / 4 per row
            const int k = k0 + f / (BN / 4), c = col0 + (f % (BN / 4)) * 4;
            rb[i] = (k < N && c < K) ? *reinterpret_cast<const float4 *>(B + (size_t)k * K + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A4; ++i) {
            const int f = tid + i * kGemmThreads;
            const int m = f >> 2, k = (f & 3) * 4;
            As[buf][k][m] = ra[i].x; As[buf][k + 1][m] = ra[i].y; As[buf][k + 2][m] = ra[i].z; As[buf][k + 3][m] = ra[i].w;
        }
#pragma unroll
        for (int i = 0; i < B4; ++i) {
            const int f = tid + i * kGemmThreads;
            *reinterpret_cast<float4 *>(&Bs[buf][f / (BN / 4)][(f % (BN / 4)) * 4]) = rb[i];
        }
    };

    const int ntiles = (N + kBK - 1) / kBK;
    fetch(0);
    stash(0);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
        const int buf = t & 1;
        if (t + 1 < ntiles) fetch((t + 1) * kBK);            // global loads in flight during the products
#pragma unroll
        for (int k = 0; k < kBK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; i += 4)
                *reinterpret_cast<float4 *>(&a[i]) = *reinterpret_cast<const float4 *>(&As[buf][k][ty * TM + i]);
#pragma unroll
            for (int j = 0; j < NJ; ++j)
                *reinterpret_cast<float4 *>(&b[4 * j]) = *reinterpret_cast<const float4 *>(&Bs[buf][k][tx * 4 + 64 * j]);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (t + 1 < ntiles) {
            stash(buf ^ 1);                                  // the other buffer was last read two tiles ago
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + ty * TM + i;
        if (r >= M) continue;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int c = col0 + tx * 4 + 64 * j;
            if (c >= K) continue;                            // K % 4 == 0 on this path: a group of four is in or out
            float4 v = make_float4(acc[i][4 * j], acc[i][4 * j + 1], acc[i][4 * j + 2], acc[i][4 * j + 3]);
            if (bias) {
                const float4 bb = *reinterpret_cast<const float4 *>(bias + c);
                v.x += bb.x; v.y += bb.y; v.z += bb.z; v.w += bb.w;
            }
            *reinterpret_cast<float4 *>(C + (size_t)r * K + c) = v;
        }
    }
}

// Any sizes and alignments: one thread per output, the same order of additions.
__global__ void matmul_plain_kernel(const float *__restrict__ A, const float *__restrict__ B, const float *__restrict__ bias,
                                    float *__restrict__ C, int M, int N, int K)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * K) return;
    const int r = (int)(idx / K), c = (int)(idx % K);
    float s = 0.0f;
    for (int k = 0; k < N; ++k) s = fmaf(A[(size_t)r * N + k], B[(size_t)k * K + c], s);
    C[idx] = bias ? s + bias[c] : s;
}

// One warp per row.  Sums: lane l adds elements l, l + 32, ... ascending, then a butterfly over the lanes.
// Separately rounded multiplies and adds (no contraction), IEEE division and square root: the CPU oracle
// built without contraction reproduces every bit.
__global__ void layer_norm_rows_kernel(const float *x, float *y, const float *__restrict__ g,
                                       const float *__restrict__ b, int rows, int E)
{
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float *xr = x + (size_t)row * E;
    float s = 0.0f;
    for (int e = lane; e < E; e += 32) s = __fadd_rn(s, xr[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
    const float mean = __fdiv_rn(s, (float)E);
    float v = 0.0f;
    for (int e = lane; e < E; e += 32) {
        const float d = __fsub_rn(xr[e], mean);
        v = __fadd_rn(v, __fmul_rn(d, d));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(v, (float)E), 1e-5f)));
    float *yr = y + (size_t)row * E;
    for (int e = lane; e < E; e += 32)
        yr[e] = __fadd_rn(__fmul_rn(__fmul_rn(g[e], __fsub_rn(xr[e], mean)), inv), b[e]);
}

// The reference seeds a xorwow state from the element index, its 256-thread block and its thread
// (a = idx + 1, b = block + 1, c = thread + 1, d = idx * block + 1) and draws once: only a and d reach
// that first draw.  u = (t + 1) / 2^32; the element is dropped when u < p, else divided by (1 - p).
__global__ void dropout_index_kernel(const float *in, float *out, float *__restrict__ mask, float p, unsigned n)   // in == out allowed
{
    const unsigned idx = blockIdx.x * 256u + threadIdx.x;
    if (idx >= n) return;
    const unsigned s = idx + 1u;
    unsigned t = idx * blockIdx.x + 1u;
    t ^= t >> 2;
    t ^= t << 1;
    t ^= s ^ (s << 4);
    const float u = __fdiv_rn((float)(t + 1u), 4294967296.0f);
    const bool drop = u < p;
    out[idx] = drop ? 0.0f : __fdiv_rn(in[idx], __fsub_rn(1.0f, p));
    if (mask) mask[idx] = drop ? 0.0f : 1.0f;
}

// out = residual + dropout(in): the sub-layer tail of the reference's block (dropout in place, then the residual
// add, src/transformer_layer.cpp:242-244 and :250-252) in one pass over memory instead of three.  The same generator,
// the same division, the same addition: bit-identical to hipgpt_dropout followed by hipgpt_add_inplace.  Four
// consecutive elements per thread when the count and the pointers allow 16-byte accesses.
__device__ __forceinline__ bool dropped(unsigned idx, float p)
{
    const unsigned s = idx + 1u;
    unsigned t = idx * (idx >> 8) + 1u;          // the reference's block of an element is idx / 256
    t ^= t >> 2;
    t ^= t << 1;
    t ^= s ^ (s << 4);
    return __fdiv_rn((float)(t + 1u), 4294967296.0f) < p;
}

__global__ void __launch_bounds__(256)
dropout_residual_kernel(const float *in, const float *residual, float *out, float *__restrict__ mask, float p, unsigned n, int vec)   // out may be in or residual
{
    const float keep = __fsub_rn(1.0f, p);
    if (vec) {
        const unsigned i4 = (blockIdx.x * 256u + threadIdx.x) * 4u;
        if (i4 >= n) return;
        const float4 x = *reinterpret_cast<const float4 *>(in + i4), r = *reinterpret_cast<const float4 *>(residual + i4);
        const bool d0 = dropped(i4, p), d1 = dropped(i4 + 1u, p), d2 = dropped(i4 + 2u, p), d3 = dropped(i4 + 3u, p);
        float4 o;
        o.x = __fadd_rn(r.x, d0 ? 0.0f : __fdiv_rn(x.x, keep));
        o.y = __fadd_rn(r.y, d1 ? 0.0f : __fdiv_rn(x.y, keep));
        o.z = __fadd_rn(r.z, d2 ? 0.0f : __fdiv_rn(x.z, keep));
        o.w = __fadd_rn(r.w, d3 ? 0.0f : __fdiv_rn(x.w, keep));
        *reinterpret_cast<float4 *>(out + i4) = o;
        if (mask) *reinterpret_cast<float4 *>(mask + i4) = make_float4(d0 ? 0.f : 1.f, d1 ? 0.f : 1.f, d2 ? 0.f : 1.f, d3 ? 0.f : 1.f);
    } else {
        const unsigned idx = blockIdx.x * 256u + threadIdx.x;
        if (idx >= n) return;
        const bool d = dropped(idx, p);
        out[idx] = __fadd_rn(residual[idx], d ? 0.0f : __fdiv_rn(in[idx], keep));
        if (mask) mask[idx] = d ? 0.0f : 1.0f;
    }
}

__global__ void add_inplace_kernel(float *__restrict__ a, const float *__restrict__ b, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = __fadd_rn(a[i], b[i]);
}

__global__ void relu_kernel(float *a, long long n)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] = fmaxf(0.0f, a[i]);
}

// out[t][e] = tok[id_t][e] + pos[t mod S][e]; an id outside [0, V) gives a row of zeros.
__global__ void embedding_kernel(const int *__restrict__ ids, const float *__restrict__ tok, const float *__restrict__ pos,
                                 float *__restrict__ out, long long T, int S, int V, int E)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * E) return;
    const long long t = i / E;
    const int e = (int)(i % E), id = ids[t];
    out[i] = (id < 0 || id >= V) ? 0.0f : __fadd_rn(tok[(size_t)id * E + e], pos[(size_t)(t % S) * E + e]);
}

bool overlap(const void *a, size_t na, const void *b, size_t nb)
{
    const uintptr_t a0 = reinterpret_cast<uintptr_t>(a), b0 = reinterpret_cast<uintptr_t>(b);
    return a0 < b0 + nb && b0 < a0 + na;
}

}  // namespace

int launch_matmul_exact(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, cudaStream_t st)
{
    if (M == 0 || K == 0) return HIPGPT_OK;
    const bool vec = (N % 4 == 0) && (K % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
                       reinterpret_cast<uintptr_t>(bias)) & 15) == 0;
    // HipGPT's layer projects in place (src/transformer_layer.cpp:220 passes the same buffer as A and C).  That is
    // safe when one block holds whole rows of C: it reads its rows of A completely before it stores.
    const bool alias = overlap(A, (size_t)M * N * 4, C, (size_t)M * K * 4);
    if (vec && K <= 256) {
        const dim3 grid(1, (M + 63) / 64);
        matmul_exact_kernel<64, 256><<<grid, kGemmThreads, 0, st>>>(A, B, bias, C, M, N, K);
        return check_launch("matmul_exact_kernel");
    }
    if (alias) return fail(HIPGPT_ERR_UNSUPPORTED, "matmul in place needs an output of at most 256 columns, a multiple of 4 (K=%d)", K);
    if (vec) {
        const dim3 grid((K + 127) / 128, (M + 127) / 128);
        matmul_exact_kernel<128, 128><<<grid, kGemmThreads, 0, st>>>(A, B, bias, C, M, N, K);
        return check_launch("matmul_exact_kernel");
    }
    const long long n = (long long)M * K;
    matmul_plain_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(A, B, bias, C, M, N, K);
    return check_launch("matmul_plain_kernel");
}

int launch_layer_norm_rows(const float *x, float *y, const float *g, const float *b, int rows, int E, cudaStream_t st)
{
    if (rows == 0 || E == 0) return HIPGPT_OK;
    layer_norm_rows_kernel<<<(rows + 7) / 8, 256, 0, st>>>(x, y, g, b, rows, E);
    return check_launch("layer_norm_rows_kernel");
}

int launch_dropout_index(const float *in, float *out, float *mask, float p, long long n, cudaStream_t st)
{
    if (n == 0) return HIPGPT_OK;
    if (n > 0xffffffffLL) return fail(HIPGPT_ERR_BAD_ARG, "dropout over %lld elements: the reference's index is 32 bits wide", n);
    dropout_index_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, mask, p, (unsigned)n);
    return check_launch("dropout_index_kernel");
}

int launch_dropout_residual(const float *in, const float *residual, float *out, float *mask, float p, long long n, cudaStream_t st)
{
    if (n == 0) return HIPGPT_OK;
    if (n > 0xffffffffLL) return fail(HIPGPT_ERR_BAD_ARG, "dropout over %lld elements: the reference's index is 32 bits wide", n);
    const uintptr_t all = reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(mask);
    const int vec = (n % 4 == 0) && (all & 15) == 0;
    const long long threads = vec ? n / 4 : n;
    dropout_residual_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(in, residual, out, mask, p, (unsigned)n, vec);
    return check_launch("dropout_residual_kernel");
}

int launch_add_inplace_n(float *a, const float *b, long long n, cudaStream_t st)
{
    if (n == 0) return HIPGPT_OK;
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a, b, n);
    return check_launch("add_inplace_kernel");
}

int launch_relu_n(float *a, long long n, cudaStream_t st)
{
    if (n == 0) return HIPGPT_OK;
    relu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a, n);
    return check_launch("relu_kernel");
}

int launch_embedding_rows(const int *ids, const float *tok, const float *pos, float *out, int B, int S, int V, int E, cudaStream_t st)
{
    const long long n = (long long)B * S * E;
    if (n == 0) return HIPGPT_OK;
    embedding_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(ids, tok, pos, out, (long long)B * S, S, V, E);
    return check_launch("embedding_kernel");
}

}  // namespace hipgpt

using namespace hipgpt;

extern "C" {

int hipgpt_matmul(const float *d_A, const float *d_B, const float *d_bias, float *d_C, int M, int N, int K, void *stream)
{
    if (M < 0 || N < 0 || K < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: M=%d N=%d K=%d", M, N, K);
    if (M == 0 || K == 0) return HIPGPT_OK;
    if (!d_C || (N > 0 && (!d_A || !d_B))) return fail(HIPGPT_ERR_NULL, "A, B and C must not be NULL");
    return launch_matmul_exact(d_A, d_B, d_bias, d_C, M, N, K, static_cast<cudaStream_t>(stream));
}

int hipgpt_matmul_tc(const float *d_A, const float *d_B, const float *d_bias, float *d_C, int M, int N, int K, void *stream)
{
    if (M < 0 || N < 0 || K < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: M=%d N=%d K=%d", M, N, K);
    if (M == 0 || K == 0) return HIPGPT_OK;
    if (!d_C || (N > 0 && (!d_A || !d_B))) return fail(HIPGPT_ERR_NULL, "A, B and C must not be NULL");
    if (N == 0) return launch_matmul_exact(d_A, d_B, d_bias, d_C, M, N, K, static_cast<cudaStream_t>(stream));   // bias (or zeros) only
    if (d_C == d_A || d_C == d_B) return fail(HIPGPT_ERR_UNSUPPORTED, "the tensor-core product does not work in place; hipgpt_matmul does (K <= 256)");
    return launch_matmul_tc(d_A, d_B, d_bias, d_C, M, N, K, static_cast<cudaStream_t>(stream));
}

int hipgpt_matmul_tc_prepare(const float *d_B, int N, int K, hipgpt_packed_matrix **out, void *stream)
{
    if (!out || !d_B) return fail(HIPGPT_ERR_NULL, "B and out must not be NULL");
    if (N <= 0 || K <= 0) return fail(HIPGPT_ERR_BAD_ARG, "bad size: N=%d K=%d", N, K);
    PackedB *p = nullptr;
    const int rc = matmul_tc_prepare(d_B, N, K, &p, static_cast<cudaStream_t>(stream));
    if (rc == HIPGPT_OK) *out = reinterpret_cast<hipgpt_packed_matrix *>(p);
    return rc;
}

int hipgpt_matmul_tc_prepared(const float *d_A, const hipgpt_packed_matrix *b, const float *d_bias, float *d_C, int M, void *stream)
{
    if (!b) return fail(HIPGPT_ERR_NULL, "the packed right-hand side must not be NULL");
    if (M < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: M=%d", M);
    if (M == 0) return HIPGPT_OK;
    if (!d_A || !d_C) return fail(HIPGPT_ERR_NULL, "A and C must not be NULL");
    if (d_A == d_C) return fail(HIPGPT_ERR_UNSUPPORTED, "the tensor-core product does not work in place");
    return launch_matmul_tc_prepared(d_A, reinterpret_cast<const PackedB *>(b), d_bias, d_C, M, static_cast<cudaStream_t>(stream));
}

void hipgpt_matmul_tc_release(hipgpt_packed_matrix *b) { matmul_tc_release(reinterpret_cast<PackedB *>(b)); }

int hipgpt_ln_matmul_tc(const float *d_A, const float *d_gamma, const float *d_beta, const float *d_B, const float *d_bias, float *d_C,
                        int M, int N, int K, void *stream)
{
    if (M < 0 || N <= 0 || K < 0) return fail(HIPGPT_ERR_BAD_ARG, "bad size: M=%d N=%d K=%d", M, N, K);
    if (M == 0 || K == 0) return HIPGPT_OK;
    if (!d_A || !d_B || !d_C || !d_gamma || !d_beta) return fail(HIPGPT_ERR_NULL, "A, gamma, beta, B and C must not be NULL");
    if (d_C == d_A || d_C == d_B) return fail(HIPGPT_ERR_UNSUPPORTED, "the tensor-core product does not work in place");
    return launch_matmul_tc(d_A, d_B, d_bias, d_C, M, N, K, static_cast<cudaStream_t>(stream), d_gamma, d_beta);
}

int hipgpt_ln_matmul_tc_prepared(const float *d_A, const float *d_gamma, const float *d_beta, const hipgpt_packed_matrix *b, const float *d_bias,
                                 float *d_C, int M, void *stream)
{
    if (!b) return fail(HIPGPT_ERR_NULL, "the packed right-hand side must not be NULL");
    if (M < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: M=%d", M);
    if (M == 0) return HIPGPT_OK;
    if (!d_A || !d_C || !d_gamma || !d_beta) return fail(HIPGPT_ERR_NULL, "A, gamma, beta and C must not be NULL");
    if (d_A == d_C) return fail(HIPGPT_ERR_UNSUPPORTED, "the tensor-core product does not work in place");
    return launch_matmul_tc_prepared(d_A, reinterpret_cast<const PackedB *>(b), d_bias, d_C, M, static_cast<cudaStream_t>(stream), d_gamma, d_beta);
}

int hipgpt_layer_norm(const float *d_in, float *d_out, const float *d_gamma, const float *d_beta, int rows, int E, void *stream)
{
    if (rows < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: rows=%d E=%d", rows, E);
    if (rows == 0 || E == 0) return HIPGPT_OK;
    if (!d_in || !d_out || !d_gamma || !d_beta) return fail(HIPGPT_ERR_NULL, "input, output, gamma and beta must not be NULL");
    return launch_layer_norm_rows(d_in, d_out, d_gamma, d_beta, rows, E, static_cast<cudaStream_t>(stream));
}

int hipgpt_dropout(const float *d_in, float *d_out, float *d_mask, float p, int rows, int E, void *stream)
{
    if (rows < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: rows=%d E=%d", rows, E);
    if (!(p >= 0.0f && p < 1.0f)) return fail(HIPGPT_ERR_BAD_ARG, "dropout probability %g outside [0, 1)", (double)p);
    if (rows == 0 || E == 0) return HIPGPT_OK;
    if (!d_in || !d_out) return fail(HIPGPT_ERR_NULL, "input and output must not be NULL");
    return launch_dropout_index(d_in, d_out, d_mask, p, (long long)rows * E, static_cast<cudaStream_t>(stream));
}

int hipgpt_dropout_residual(const float *d_in, const float *d_residual, float *d_out, float *d_mask, float p, int rows, int E, void *stream)
{
    if (rows < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: rows=%d E=%d", rows, E);
    if (!(p >= 0.0f && p < 1.0f)) return fail(HIPGPT_ERR_BAD_ARG, "dropout probability %g outside [0, 1)", (double)p);
    if (rows == 0 || E == 0) return HIPGPT_OK;
    if (!d_in || !d_residual || !d_out) return fail(HIPGPT_ERR_NULL, "input, residual and output must not be NULL");
    return launch_dropout_residual(d_in, d_residual, d_out, d_mask, p, (long long)rows * E, static_cast<cudaStream_t>(stream));
}

int hipgpt_add_inplace(float *d_a, const float *d_b, long long n, void *stream)
{
    if (n < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: n=%lld", n);
    if (n == 0) return HIPGPT_OK;
    if (!d_a || !d_b) return fail(HIPGPT_ERR_NULL, "a and b must not be NULL");
    return launch_add_inplace_n(d_a, d_b, n, static_cast<cudaStream_t>(stream));
}

int hipgpt_relu(float *d_a, long long n, void *stream)
{
    if (n < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: n=%lld", n);
    if (n == 0) return HIPGPT_OK;
    if (!d_a) return fail(HIPGPT_ERR_NULL, "a must not be NULL");
    return launch_relu_n(d_a, n, static_cast<cudaStream_t>(stream));
}

int hipgpt_embedding_lookup(const int *d_ids, const float *d_tok, const float *d_pos, float *d_out, int B, int S, int V, int E, void *stream)
{
    if (B < 0 || S < 0 || V < 0 || E < 0) return fail(HIPGPT_ERR_BAD_ARG, "negative size: B=%d S=%d V=%d E=%d", B, S, V, E);
    if (B == 0 || S == 0 || E == 0) return HIPGPT_OK;
    if (!d_ids || !d_tok || !d_pos || !d_out) return fail(HIPGPT_ERR_NULL, "ids, embeddings and output must not be NULL");
    return launch_embedding_rows(d_ids, d_tok, d_pos, d_out, B, S, V, E, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
