/*
 * CPU oracle for HipGPT's multi-head-attention forward path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a scalar restatement, in plain C, of the arithmetic of the reference's
 * attention kernels (paths are relative to the HipGPT source tree):
 *
 *   oracle_mha_flash        src/hip_kernels.cpp:263-325  flash_attention_kernel<HEAD_DIM>
 *   oracle_mha_fallback     src/hip_kernels.cpp:329-402  multihead_attention_kernel_fallback
 *   oracle_mha_dispatch     src/hip_kernels.cpp:404-451  launch_multihead_attention
 *   oracle_sdp              src/hip_kernels.cpp:455-473  scaled_dot_product_kernel
 *   oracle_softmax          src/hip_kernels.cpp:478-511  softmax_kernel
 *   oracle_weighted_sum     src/hip_kernels.cpp:514-532  attention_weighted_sum_kernel
 *   oracle_mha_backward     src/hip_kernels.cpp:1162-1272  multihead_attention_backward_kernel
 *   oracle_decode_row       (extension) one query row over a key/value cache, same
 *                           arithmetic as the flash kernel restricted to one row.
 *
 * Every loop keeps the reference's order (d ascending, j ascending, one accumulator that
 * starts at 0.0f) so that, compiled like the reference source built through the host shim
 * (oracle/ref_shim; both with -ffp-contract=off), results are equal bit for bit.
 * The reference launches up to 32 threads that compute the same query row
 * (src/hip_kernels.cpp:271 against :423-424); one evaluation per row gives the same bits.
 *
 * `causal` is an extension that the reference does not have: with causal != 0 every loop
 * over keys j stops at j <= query index, and stored probabilities above the diagonal are 0.
 * With causal == 0 the functions are the reference's semantics (no mask at all).
 *
 * Parity pin: oracle/Makefile compiles the reference's own hip_kernels.cpp, where it is
 * mounted, into oracle/_ref/libhipgpt_ref.so; tests/test_oracle.py asserts
 * bit equality, and tests/golden/ holds outputs of that reference build.
 *
 * Only tests/, the smoke check and bench.py's CPU-baseline leg may call this file.
 * The product library never links or loads it.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* acc + a*b.  The library is built twice (oracle/Makefile):
 *   libattn_oracle.so      ORACLE_FMA=0, -ffp-contract=off: separately rounded multiply and
 *                          add everywhere.  With the reference source built the same way this
 *                          variant is equal to it bit for bit; it is the pinned oracle.
 *   libattn_oracle_fma.so  ORACLE_FMA=1: the multiply-accumulates are single-rounded fmaf,
 *                          which is what a GPU compiler (hipcc, nvcc) makes of the same source
 *                          lines.  Used where a GPU result is compared bit for bit. */
#ifndef ORACLE_FMA
#define ORACLE_FMA 0
#endif
#if ORACLE_FMA
#define MAC(acc, a, b) fmaf((a), (b), (acc))
#else
#define MAC(acc, a, b) ((acc) + (a) * (b))
#endif

static float inv_sqrtf(float x) { return 1.0f / sqrtf(x); } /* rsqrtf on the host */

/* One query row of the flash kernel (src/hip_kernels.cpp:279-324).  `scores` is scratch of
 * S floats.  probs_row may be NULL (the reference always stores; NULL skips the store and
 * keeps the normalised value in `scores`, which is what the stored value would be). */
static void flash_row(const float *Q, const float *K, const float *V, float *out, float *probs_row,
                      float *scores, int S, int E, int D, size_t tok0, int qi, int h, int causal)
{
    const float scale = inv_sqrtf((float)D);
    const size_t q_off = (tok0 + (size_t)qi) * (size_t)E + (size_t)h * D;
    const int jend = causal ? qi + 1 : S;
    float max_score = -1e30f;
    float sum_exp = 0.0f;
    for (int j = 0; j < jend; ++j) {                         /* :287-296 */
        const float *k_vec = K + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        float score = 0.0f;
        for (int d = 0; d < D; ++d) score = MAC(score, Q[q_off + d], k_vec[d]);
        score *= scale;
        scores[j] = score;
        max_score = fmaxf(max_score, score);
    }
    for (int j = 0; j < jend; ++j) {                         /* :299-303 */
        float prob = expf(scores[j] - max_score);
        scores[j] = prob;
        sum_exp += prob;
    }
    sum_exp = fmaxf(sum_exp, 1e-20f);                        /* :304 */
    for (int j = 0; j < jend; ++j) scores[j] = scores[j] / sum_exp;   /* :308-310 */
    if (probs_row) {
        memcpy(probs_row, scores, (size_t)jend * sizeof(float));
        for (int j = jend; j < S; ++j) probs_row[j] = 0.0f;
    }
    /* :313-319 — j outer, d inner, accumulating into D independent sums */
    float acc[512];
    for (int d = 0; d < D; ++d) acc[d] = 0.0f;
    for (int j = 0; j < jend; ++j) {
        const float *v_vec = V + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        const float p = scores[j];
        for (int d = 0; d < D; ++d) acc[d] = MAC(acc[d], p, v_vec[d]);
    }
    for (int d = 0; d < D; ++d) out[q_off + d] = acc[d];     /* :322-324 */
}

/* Flash-kernel math for every (batch, head, query).  Q, K, V, out are [B*S][E] with head h
 * of token t at t*E + h*D (src/hip_kernels.cpp:276,289,314); probs is [B][H][S][S] (:277)
 * or NULL.  Returns 0, or -1 for a bad shape (D > 512 would overflow the row scratch). */
ORACLE_API int oracle_mha_flash(const float *Q, const float *K, const float *V, float *out, float *probs,
                                int B, int S, int E, int H, int causal)
{
    if (B < 0 || S < 0 || H <= 0 || E % H != 0) return -1;
    const int D = E / H;
    if (D > 512) return -1;
    const long long rows = (long long)B * H * S;
#pragma omp parallel
    {
        float *scores = (float *)malloc((size_t)(S > 0 ? S : 1) * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (long long r = 0; r < rows; ++r) {
            const int qi = (int)(r % S);
            const int h = (int)((r / S) % H);
            const int b = (int)(r / ((long long)S * H));
            float *prow = probs ? probs + (((size_t)b * H + h) * (size_t)S + (size_t)qi) * (size_t)S : NULL;
            flash_row(Q, K, V, out, prow, scores, S, E, D, (size_t)b * S, qi, h, causal);
        }
        free(scores);
    }
    return 0;
}

/* One query row of the fallback kernel (src/hip_kernels.cpp:341-401): three passes that each
 * recompute q.k, probability = exp(s - max) * (1 / sum), accumulation straight into out. */
static void fallback_row(const float *Q, const float *K, const float *V, float *out, float *probs_row,
                         int S, int E, int D, size_t tok0, int qi, int h, int causal)
{
    const float inv_sqrt = inv_sqrtf((float)D);
    const float *q_vec = Q + (tok0 + (size_t)qi) * (size_t)E + (size_t)h * D;
    float *out_vec = out + (tok0 + (size_t)qi) * (size_t)E + (size_t)h * D;
    const int jend = causal ? qi + 1 : S;
    float max_score = -1e30f;
    for (int j = 0; j < jend; ++j) {                         /* :353-360 */
        const float *k_vec = K + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = MAC(dot, q_vec[d], k_vec[d]);
        float s = dot * inv_sqrt;
        if (s > max_score) max_score = s;
    }
    float sum_exp = 0.f;
    for (int j = 0; j < jend; ++j) {                         /* :366-372 */
        const float *k_vec = K + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = MAC(dot, q_vec[d], k_vec[d]);
        sum_exp += expf(dot * inv_sqrt - max_score);         /* __expf on the GPU */
    }
    sum_exp = fmaxf(sum_exp, 1e-20f);                        /* :373 */
    const float inv_sum = 1.0f / sum_exp;                    /* :374 */
    for (int d = 0; d < D; ++d) out_vec[d] = 0.f;            /* :379 */
    for (int j = 0; j < jend; ++j) {                         /* :386-401 */
        const float *k_vec = K + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        const float *v_vec = V + (tok0 + (size_t)j) * (size_t)E + (size_t)h * D;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = MAC(dot, q_vec[d], k_vec[d]);
        float p = expf(dot * inv_sqrt - max_score) * inv_sum;
        if (probs_row) probs_row[j] = p;
        for (int d = 0; d < D; ++d) out_vec[d] = MAC(out_vec[d], p, v_vec[d]);
    }
    if (probs_row) for (int j = jend; j < S; ++j) probs_row[j] = 0.0f;
}

ORACLE_API int oracle_mha_fallback(const float *Q, const float *K, const float *V, float *out, float *probs,
                                   int B, int S, int E, int H, int causal)
{
    if (B < 0 || S < 0 || H <= 0 || E % H != 0) return -1;
    const int D = E / H;
    const long long rows = (long long)B * H * S;
#pragma omp parallel for schedule(dynamic, 16)
    for (long long r = 0; r < rows; ++r) {
        const int qi = (int)(r % S);
        const int h = (int)((r / S) % H);
        const int b = (int)(r / ((long long)S * H));
        float *prow = probs ? probs + (((size_t)b * H + h) * (size_t)S + (size_t)qi) * (size_t)S : NULL;
        fallback_row(Q, K, V, out, prow, S, E, D, (size_t)b * S, qi, h, causal);
    }
    return 0;
}

/* The launcher's plane view and dispatch rule (src/hip_kernels.cpp:415-422): d_qkv holds
 * three stacked [B*S][E] planes; flash math when head_dim is 32 or 64 and S <= 512, the
 * fallback math otherwise.  Returns which path ran (1 flash, 2 fallback) or -1. */
ORACLE_API int oracle_mha_dispatch(const float *qkv, float *out, float *probs,
                                   int B, int S, int E, int H, int causal)
{
    if (H <= 0 || (E % H) != 0) return -1;                   /* :410-413 aborts there */
    const size_t plane = (size_t)B * S * E;
    const float *Q = qkv, *K = qkv + plane, *V = qkv + 2 * plane;
    const int D = E / H;
    if ((D == 64 || D == 32) && S <= 512) {
        return oracle_mha_flash(Q, K, V, out, probs, B, S, E, H, causal) == 0 ? 1 : -1;
    }
    return oracle_mha_fallback(Q, K, V, out, probs, B, S, E, H, causal) == 0 ? 2 : -1;
}

/* scores[t*S + j] = (sum_d Q[t*D+d] * K[(t/S)*S*D + j*D + d]) * rsqrt(D)   (:455-466) */
ORACLE_API int oracle_sdp(const float *Q, const float *K, float *scores, int B, int S, int D)
{
    const long long total = (long long)B * S;
    const float inv = inv_sqrtf((float)D);
#pragma omp parallel for schedule(static)
    for (long long t = 0; t < total; ++t) {
        const size_t kb = (size_t)(t / S) * (size_t)S * D;
        for (int j = 0; j < S; ++j) {
            float sum = 0.0f;
            for (int d = 0; d < D; ++d) sum = MAC(sum, Q[(size_t)t * D + d], K[kb + (size_t)j * D + d]);
            scores[(size_t)t * S + j] = sum * inv;
        }
    }
    return 0;
}

/* Row softmax: max from -1e30f, expf(x - max) stored and summed ascending, then every entry
 * times 1 / max(sum, 1e-20f)   (:478-504) */
ORACLE_API int oracle_softmax(const float *scores, float *softmax_out, int B, int S)
{
    const long long total = (long long)B * S;
#pragma omp parallel for schedule(static)
    for (long long t = 0; t < total; ++t) {
        const float *row = scores + (size_t)t * S;
        float *orow = softmax_out + (size_t)t * S;
        float max_score = -1e30f;
        for (int i = 0; i < S; ++i) max_score = fmaxf(max_score, row[i]);
        float sum_exp = 0.0f;
        for (int i = 0; i < S; ++i) {
            float e = expf(row[i] - max_score);
            orow[i] = e;
            sum_exp += e;
        }
        float inv_sum = 1.0f / fmaxf(sum_exp, 1e-20f);
        for (int i = 0; i < S; ++i) orow[i] *= inv_sum;
    }
    return 0;
}

/* out[t*D+d] = sum_j P[t*S+j] * V[(t/S)*S*D + j*D + d], j ascending per d   (:514-525) */
ORACLE_API int oracle_weighted_sum(const float *P, const float *V, float *out, int B, int S, int D)
{
    const long long total = (long long)B * S;
#pragma omp parallel for schedule(static)
    for (long long t = 0; t < total; ++t) {
        const size_t vb = (size_t)(t / S) * (size_t)S * D;
        for (int d = 0; d < D; ++d) {
            float sum = 0.0f;
            for (int j = 0; j < S; ++j) sum = MAC(sum, P[(size_t)t * S + j], V[vb + (size_t)j * D + d]);
            out[(size_t)t * D + d] = sum;
        }
    }
    return 0;
}

/* Extension (no reference counterpart): attention of ONE new query row per (batch, head)
 * over the first `ctx` rows of a key/value cache.  q and out are [B][E]; the caches are
 * [B][cap][E] with head h of position j at (b*cap + j)*E + h*D.  The arithmetic is the flash
 * kernel's row (src/hip_kernels.cpp:287-319) with S := ctx. */
ORACLE_API int oracle_decode_row(const float *q, const float *kcache, const float *vcache, float *out,
                                 int B, int H, int D, int ctx, int cap)
{
    if (ctx < 0 || ctx > cap || D > 512) return -1;
    const int E = H * D;
    const long long rows = (long long)B * H;
#pragma omp parallel
    {
        float *scores = (float *)malloc((size_t)(ctx > 0 ? ctx : 1) * sizeof(float));
#pragma omp for schedule(static)
        for (long long r = 0; r < rows; ++r) {
            const int h = (int)(r % H);
            const int b = (int)(r / H);
            const float scale = inv_sqrtf((float)D);
            const float *qv = q + (size_t)b * E + (size_t)h * D;
            float max_score = -1e30f, sum_exp = 0.0f;
            for (int j = 0; j < ctx; ++j) {
                const float *k_vec = kcache + ((size_t)b * cap + j) * (size_t)E + (size_t)h * D;
                float score = 0.0f;
                for (int d = 0; d < D; ++d) score = MAC(score, qv[d], k_vec[d]);
                score *= scale;
                scores[j] = score;
                max_score = fmaxf(max_score, score);
            }
            for (int j = 0; j < ctx; ++j) {
                float p = expf(scores[j] - max_score);
                scores[j] = p;
                sum_exp += p;
            }
            sum_exp = fmaxf(sum_exp, 1e-20f);
            float acc[512];
            for (int d = 0; d < D; ++d) acc[d] = 0.0f;
            for (int j = 0; j < ctx; ++j) {
                const float *v_vec = vcache + ((size_t)b * cap + j) * (size_t)E + (size_t)h * D;
                const float p = scores[j] / sum_exp;
                for (int d = 0; d < D; ++d) acc[d] = MAC(acc[d], p, v_vec[d]);
            }
            for (int d = 0; d < D; ++d) out[(size_t)b * E + (size_t)h * D + d] = acc[d];
        }
        free(scores);
    }
    return 0;
}

/* Host threads the parallel loops will use (for the CPU-baseline report). */
ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* dQ, dK, dV as three stacked planes (launcher view, src/hip_kernels.cpp:1242-1255), from dO, the stacked
 * Q, K, V planes and the stored probabilities.  Loop order of the kernel (:1190-1239): per (token, head) first
 * w = sum_j p_ij (g . V_j), then for j ascending: dV_j += p_ij g; dQ_i += ds k_j / sqrt(D); dK_j += ds q_i / sqrt(D)
 * with ds = p_ij ((g . V_j) - w).  The reference's threads add into dK and dV with atomicAdd in whatever
 * order they run; here queries are visited in ascending order, which is also what the reference source
 * does when it is run on one host thread through the host stand-in (the pin in tests/test_oracle.py).
 * `probs` NULL (extension): the probabilities are formed from Q and K by the flash arithmetic above.
 * `causal` (extension): keys j > i are skipped. */
ORACLE_API int oracle_mha_backward(const float *gout, const float *qkv, const float *probs, float *gqkv,
                                   int B, int S, int E, int H, int causal)
{
    if (H <= 0 || (E % H) != 0) return -1;
    const int D = E / H;
    const size_t plane = (size_t)B * S * E;
    const float *Q = qkv, *K = qkv + plane, *V = qkv + 2 * plane;
    float *dQ = gqkv, *dK = gqkv + plane, *dV = gqkv + 2 * plane;
    const float inv = inv_sqrtf((float)D);
    memset(gqkv, 0, 3 * plane * sizeof(float));
    float *prow = probs ? NULL : (float *)malloc(sizeof(float) * (size_t)S);
    float *scratch = probs ? NULL : (float *)malloc(sizeof(float) * plane);      /* the forward output, unused */
    for (int h = 0; h < H; ++h)
        for (long long t = 0; t < (long long)B * S; ++t) {
            const int b = (int)(t / S), i = (int)(t % S);
            const float *q = Q + (size_t)t * E + (size_t)h * D, *g = gout + (size_t)t * E + (size_t)h * D;
            float *dq = dQ + (size_t)t * E + (size_t)h * D;
            const float *p;
            if (probs) {
                p = probs + (((size_t)b * H + h) * (size_t)S + (size_t)i) * (size_t)S;
            } else {
                flash_row(Q, K, V, scratch, NULL, prow, S, E, D, (size_t)b * S, i, h, causal);
                for (int j = causal ? i + 1 : S; j < S; ++j) prow[j] = 0.0f;
                p = prow;
            }
            const int jend = causal ? i + 1 : S;
            float w = 0.0f;
            for (int j = 0; j < jend; ++j) {
                const float *v = V + ((size_t)b * S + j) * E + (size_t)h * D;
                float vdot = 0.0f;
                for (int d = 0; d < D; ++d) vdot = MAC(vdot, g[d], v[d]);
                w = MAC(w, p[j], vdot);
            }
            for (int d = 0; d < D; ++d) dq[d] = 0.0f;
            for (int j = 0; j < jend; ++j) {
                const float pij = p[j];
                const float *k = K + ((size_t)b * S + j) * E + (size_t)h * D, *v = V + ((size_t)b * S + j) * E + (size_t)h * D;
                float *dk = dK + ((size_t)b * S + j) * E + (size_t)h * D, *dv = dV + ((size_t)b * S + j) * E + (size_t)h * D;
                float vdot = 0.0f;
                for (int d = 0; d < D; ++d) vdot = MAC(vdot, g[d], v[d]);
                const float ds = pij * (vdot - w);
                for (int d = 0; d < D; ++d) dv[d] = MAC(dv[d], pij, g[d]);
                for (int d = 0; d < D; ++d) dq[d] += ds * k[d] * inv;
                for (int d = 0; d < D; ++d) dk[d] += ds * q[d] * inv;
            }
        }
    free(prow);
    free(scratch);
    return 0;
}
