// Self-test of the bounded waits (cuvdia_selftest_bounded_wait): shows, without any fault, what a kernel of this
// library does when an asynchronous copy never completes.
#include "cuvdia_internal.cuh"

namespace cuvdia {

// One warp polls an mbarrier that is initialised for one arrival and never gets it, the way the TMA kernels
// poll theirs, and gives up after max_polls polls with a code in the health word.
__global__ void selftest_wait_kernel(int* status, unsigned max_polls) {
    __shared__ unsigned long long bar;
    const unsigned b = (unsigned)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    bool done = false;
    for (unsigned it = 0; it < max_polls && !done; it++) {
        unsigned d;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(d) : "r"(b), "r"(0u) : "memory");
        done = d != 0;
    }
    if (!done && threadIdx.x == 0 && status) *status = 9;
}

int launch_selftest_wait(int* status, unsigned max_polls, cudaStream_t st) {
    selftest_wait_kernel<<<1, 32, 0, st>>>(status, max_polls);
    count_launch();
    return check_launch("selftest_wait_kernel");
}

}  // namespace cuvdia
