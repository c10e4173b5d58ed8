// Measurement helper: a register-resident FFMA loop that gives the fp32 FMA-pipe ceiling of
// the GPU it runs on, at the clocks of the moment.  The exact-fp32 attention kernels are bound
// by that pipe, not by HBM, so benchmarks divide by this figure measured in the same run.
// No counterpart in the reference.
#include "attn_common.cuh"

namespace hipgpt {
namespace {

constexpr int kChains = 16;

__global__ void __launch_bounds__(256)
fma_probe_kernel(float *sink, int iters, float x, float y)
{
    float a[kChains];
#pragma unroll
    for (int j = 0; j < kChains; ++j) a[j] = (float)(threadIdx.x + j) * 1e-3f;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int j = 0; j < kChains; ++j) a[j] = fmaf(a[j], x, y);
    }
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kChains; ++j) s += a[j];
    if (s == 123456.789f) sink[0] = s;      // never true for these operands; keeps the loop alive
}

}  // namespace
}  // namespace hipgpt

extern "C" int hipgpt_probe_fma(float *d_sink, int blocks, int iters, double *flops, void *stream)
{
    using namespace hipgpt;
    if (!d_sink || !flops) return fail(HIPGPT_ERR_NULL, "d_sink and flops must not be NULL");
    if (blocks <= 0 || iters <= 0) return fail(HIPGPT_ERR_BAD_ARG, "bad probe size: blocks=%d iters=%d", blocks, iters);
    fma_probe_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_sink, iters, 0.999999f, 1e-7f);
    *flops = 2.0 * kChains * (double)iters * 256.0 * (double)blocks;
    return check_launch("fma_probe_kernel");
}
