// Times the grid-wide barrier that the fused decode kernel is built on: `rounds` barriers over one
// CTA per SM, nothing in between.
#include "common.cuh"
#include "grid_sync.cuh"

namespace {

__global__ void __launch_bounds__(256) grid_barrier_probe_kernel(unsigned* counter, int rounds, int* error_flag) {
    unsigned arrivals = 0;
    for (int r = 0; r < rounds; ++r)
        if (!grid_sync::barrier(counter, arrivals)) {
            if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 1);
            return;
        }
}

}  // namespace

// counter: one zeroed 32-bit word in device memory (zeroed again here, on the stream, before the launch).
LLM_EXPORT int llm_grid_barrier_probe(unsigned* counter, int rounds, int* error_flag, cudaStream_t stream) {
    int dev = 0, sms = 0, coop = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    if (!coop || sms <= 0) return LLM_ERR_UNSUPPORTED;
    cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned), stream);
    if (e != cudaSuccess) return (int)e;
    void* args[] = {&counter, &rounds, &error_flag};
    return (int)cudaLaunchCooperativeKernel((void*)grid_barrier_probe_kernel, dim3(sms), dim3(256), args, 0, stream);
}
