// Test hook for the bounded waits of the tensor-core kernels (no counterpart in the reference).
//
// Those kernels never spin without a limit: every wait on an mbarrier goes through mbar_wait_for()
// (tc_primitives.cuh), and a wait that runs out makes the block raise its abort flag, record the site
// of the wait in a status word, skip its stores and return.  On a healthy GPU that path never runs.
// The kernel below runs the same protocol on a barrier at which nothing ever arrives, with a limit
// of the caller's choosing (a fraction of a millisecond in the tests), so that the give-up path, the
// status word and the "nothing stored" promise can be checked without hanging or faulting anything.
#include "tc_primitives.cuh"

namespace hipgpt {
namespace {

__device__ int g_probe_status = 0;

constexpr int kProbeSite = 7;

__global__ void wait_expiry_kernel(float *canary, int n, long long limit_cycles)
{
    __shared__ uint64_t never;                   // nothing arrives here
    __shared__ uint64_t once;                    // thread 0 arrives here: a wait that completes
    __shared__ volatile int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(&never, 1);
        mbar_init(&once, 1);
    }
    __syncthreads();
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag) return;
        if (!mbar_wait_for(bar, parity, limit_cycles, kSpinLimit)) { abort_flag = 1; atomicCAS(&g_probe_status, 0, site); }
    };
    if (threadIdx.x == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&once)) : "memory");
    wait(&once, 0, 1);                           // completes: site 1 must not show up
    wait(&never, 0, kProbeSite);                 // runs out after limit_cycles
    wait(&never, 0, kProbeSite + 1);             // cut short by the flag: site 8 must not show up either
    __syncthreads();
    if (!abort_flag)
        for (int i = threadIdx.x; i < n; i += blockDim.x) canary[i] = 1.0f;
}

}  // namespace

int probe_status_fetch(int *status)
{
    int s = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&s, g_probe_status, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (s != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_probe_status, &zero, sizeof(int));
    }
    *status = s;
    return HIPGPT_OK;
}

}  // namespace hipgpt

extern "C" int hipgpt_debug_wait_expiry(float *d_canary, int n, long long limit_cycles, void *stream)
{
    using namespace hipgpt;
    if (!d_canary || n <= 0) return fail(HIPGPT_ERR_NULL, "canary buffer missing");
    if (limit_cycles <= 0 || limit_cycles > (1LL << 24)) return fail(HIPGPT_ERR_BAD_ARG, "limit of %lld cycles out of range (1 .. 2^24)", limit_cycles);
    wait_expiry_kernel<<<2, 128, 0, static_cast<cudaStream_t>(stream)>>>(d_canary, n, limit_cycles);
    return check_launch("wait_expiry_kernel");
}
