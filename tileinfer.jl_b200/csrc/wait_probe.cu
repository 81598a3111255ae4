// A wait that runs out, on purpose and harmlessly: the error path of the bounded waits, for the tests.
//
// The tensor-core kernels wait on mbarriers with a limit of attempts; when a wait runs out they set a bit
// in a status word, let what is in flight land and return, so that the host sees an error instead of a
// hung device (AntoineBut/TileInfer.jl dropped a device-side spin-wait for the same reason,
// docs/src/performance.md:89-90). This entry point runs exactly that path and nothing else: one block
// initialises one mbarrier on which nobody ever arrives, waits on it with a small limit through the same
// `tc::mbar_wait`, and returns. It touches no TMA copy, no MMA and no tensor memory.
#include "tcgen05.cuh"

namespace {

__global__ void wait_probe_kernel(int* status, int code, unsigned limit, int* result) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(tc::smem_addr(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool done = tc::mbar_wait(tc::smem_addr(&bar), 0, status, code, limit);
        if (!done) tc::drain_after_timeout();
        *result = done ? 1 : 2;                       // 2: the wait gave up, as it must here
    }
}

}  // namespace

// Waits at most `limit` attempts (clamped to 1..65536) on a barrier that nothing completes; sets bit `code`
// of *status and writes 2 to *result when it gives up.
extern "C" int ti_wait_probe(int* status, int code, int limit, int* result, cudaStream_t stream) {
    TI_REQUIRE(status != nullptr && result != nullptr && code >= 0 && code < 31, "wait_probe: bad arguments");
    if (limit < 1) limit = 1;
    if (limit > 65536) limit = 65536;
    ti_launch(wait_probe_kernel, dim3(1), dim3(32), 0, stream, status, code, (unsigned)limit, result);
    return ti_check_launch("wait_probe");
}
