// A launch that lets a bounded wait run out, so that the path every kernel of the package takes when a barrier never
// completes can be seen to work: the wait gives up after its cycle limit, the error word receives 5, the block still
// reaches its end (block-wide barriers stay matched), and the context stays usable.  Nothing here faults or hangs: the
// barrier simply has no arrival coming, and the wait is the same mbar_wait_cycles that the kernels' waits go through.
#include "sm100.cuh"

namespace cvb {

__global__ void wait_runs_out_kernel(int* err, int* finished, long long limit_cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool completed = mbar_wait_cycles(&bar, 0, err, limit_cycles);       // nothing ever arrives on `bar`
    __syncthreads();
    if (threadIdx.x == 0) *finished = completed ? 2 : 1;
}

}  // namespace cvb

// finished receives 1 when the wait ran out and the kernel went on to its end (2 if the wait completed, which it cannot).
extern "C" int cvb_selftest_wait_runs_out(int* err_flag, int* finished, long long limit_cycles, cudaStream_t stream) {
    if (err_flag == nullptr || finished == nullptr) return CVB_E_SHAPE;
    if (limit_cycles <= 0 || limit_cycles > 40000000LL) return CVB_E_SIZE;   // never longer than the kernels' own limit (about 20 ms)
    cvb::wait_runs_out_kernel<<<1, 64, 0, stream>>>(err_flag, finished, limit_cycles);
    return cvb::launch_status();
}
