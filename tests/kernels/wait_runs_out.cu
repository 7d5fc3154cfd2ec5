// A kernel for the tests only: one thread waits, with the package's own bounded
// wait (tc::mbar_wait), on an mbarrier that nothing will ever complete. The
// limit is passed in and short (about 50 microseconds), so the wait runs out,
// records `code` in *status and returns false; the kernel then writes what the
// wait returned to *returned and ends like any other. It shows that a wait that
// cannot be satisfied ends in a status code and a usable context, not in a hang.
#include "tcgen05.cuh"

namespace {

__global__ void wait_runs_out_kernel(int* status, int code, long long limit_cycles, int* returned) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        stride::tc::mbar_init(stride::tc::smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = stride::tc::mbar_wait(stride::tc::smem_u32(&bar), 0, status, code, limit_cycles);
        *returned = ok ? 1 : 0;
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(stride::tc::smem_u32(&bar)) : "memory");
    }
}

}  // namespace

extern "C" int test_wait_runs_out(int* status, int code, long long limit_cycles, int* returned, cudaStream_t stream) {
    if (status == nullptr || returned == nullptr || limit_cycles <= 0 || limit_cycles > 100000000LL) return STRIDE_BAD_ARGUMENT;
    wait_runs_out_kernel<<<1, 32, 0, stream>>>(status, code, limit_cycles, returned);
    return STRIDE_LAUNCH_STATUS();
}
