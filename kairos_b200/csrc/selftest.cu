// Self-test of the bounded device-side wait: the path every pipeline kernel of this library takes when a
// barrier it waits on is never completed.  One CTA initialises an mbarrier that nothing arrives on, waits
// on it with a limit of about a millisecond through the same routine the kernels use, and -- when the
// limit runs out -- raises the device status word and returns.  Nothing faults and nothing spins without
// a limit; the context stays usable.  The host then reads KAIROS_ERR_DEVICE from kairos_device_status().
#include "common.cuh"

namespace kairos {

int* device_status_word();   // api.cu

__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    // phase 0 of the barrier never completes: no thread arrives and no copy is in flight
    const bool ok = mbar_wait_limit(&bar, 0, &abort_flag, limit_cycles);
    __syncthreads();
    if (!ok && threadIdx.x == 0) atomicExch(status, KAIROS_ERR_DEVICE);
}

}  // namespace kairos

extern "C" int kairos_selftest_bounded_wait(kairos_stream_t stream) {
    using namespace kairos;
    int* status = device_status_word();
    if (!status) return KAIROS_ERR_CUDA;
    bounded_wait_selftest_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, 2000000LL);
    return launch_status();
}
