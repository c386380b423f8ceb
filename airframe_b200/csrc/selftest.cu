// A self-test of the library's bounded waits: a kernel that waits on a barrier nobody arrives on, with
// a short limit, so that the give-up path of mbar_wait (timer, error word, orderly return) runs for
// real.  The product kernels take the same path after their limit of two seconds; nothing else in the
// library can make them take it without starving them.
#include "tma.cuh"

namespace {

__global__ void wait_runs_out_kernel(int* err, unsigned long long limit_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t bar;
  __shared__ int give_up_s;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    give_up_s = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long t0 = now_ns();
    const bool done = mbar_wait(&bar, 0, &give_up_s, limit_ns);     // no arrival will ever come
    if (waited_ns) *waited_ns = now_ns() - t0;
    if (!done && give_up_s && err) atomicExch(err, 1);
  }
}

}  // namespace

// Launches one block whose wait on an mbarrier runs out after limit_ns (at most 100 ms): *err becomes 1,
// *waited_ns (optional) the time the wait took.  For tests of the give-up path.
AF_EXPORT int af_selftest_wait_runs_out(int* err, unsigned long long limit_ns, unsigned long long* waited_ns,
                                        cudaStream_t stream) {
  AF_REQUIRE(err != nullptr && limit_ns > 0 && limit_ns <= 100000000ull,
             "af_selftest_wait_runs_out: a limit of up to 100 ms");
  af_launch(wait_runs_out_kernel, dim3(1), dim3(32), 0, stream, err, limit_ns, waited_ns);
  AF_CHECK_LAUNCH("af_selftest_wait_runs_out");
}
