// A barrier over all CTAs of a cooperatively launched kernel (every CTA is resident, so the wait
// cannot starve), with a bounded wait: a CTA that does not see the others arrive within the limit
// reports failure instead of spinning for ever.
#pragma once

#include <cuda_runtime.h>

namespace grid_sync {

constexpr int SPIN_LIMIT = 1 << 22;  // polls of the counter before giving up (on the order of a second)

// `counter` starts at zero for the launch and only grows; `arrivals_so_far` is gridDim.x times the number of
// barriers this CTA has passed before.  Returns false if the wait gave up.
__device__ __forceinline__ bool barrier(unsigned* counter, unsigned& arrivals_so_far) {
    __shared__ int ok_s;
    __syncthreads();
    arrivals_so_far += gridDim.x;
    if (threadIdx.x == 0) {
        __threadfence();  // this CTA's writes are visible before its arrival is
        atomicAdd(counter, 1u);
        int ok = 0;
        for (int i = 0; i < SPIN_LIMIT; ++i) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(counter) : "memory");
            if (seen >= arrivals_so_far) {
                ok = 1;
                break;
            }
        }
        ok_s = ok;
    }
    __syncthreads();
    return ok_s != 0;
}

}  // namespace grid_sync
