// Small host-buffer calls without the copy engines.  A blocking call with host activations in and a host result out
// spends most of its time in latencies around the kernel: a DMA copy in, a DMA copy out and the wake-up of the
// waiting thread cost ~8 us each, the kernel itself ~8.  For calls whose tables, activations and result fit a pinned
// block of the calling thread, two one-CTA kernels replace the copies: stage_in reads the block (pinned host memory
// the GPU addresses directly) into the device staging area -- one pass over PCIe, so that the GEMM's CTAs do not each
// fetch their rows across the bus -- and stage_out writes the result into the block with coalesced 16-byte stores,
// then the status word and, behind a system-scope fence, a sequence number the host thread polls.  Both are launched
// with programmatic stream serialization, so their launch latencies overlap their neighbours.
#pragma once

#include "common.cuh"

namespace gnf4b {

constexpr int kHostStageThreads = 1024;

__global__ void __launch_bounds__(kHostStageThreads, 1)
host_stage_in_kernel(const uint4* __restrict__ src_host, uint4* __restrict__ dst, int32_t n16, uint4* zero_a, int32_t zero_a_n16,
                     uint4* zero_b, int32_t zero_b_n16) {
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < n16; i += kHostStageThreads) dst[i] = __ldg(src_host + i);
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < zero_a_n16; i += kHostStageThreads) zero_a[i] = z;     // counters that must start at zero
    for (int i = threadIdx.x; i < zero_b_n16; i += kHostStageThreads) zero_b[i] = z;
}

// tail_host[0] = sequence number (written last), tail_host[1] = the device status word of the call
__global__ void __launch_bounds__(kHostStageThreads, 1)
host_stage_out_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst_host, int32_t n16, const int32_t* __restrict__ d_status,
                      volatile uint32_t* tail_host, uint32_t seq) {
    pdl_launch_dependents();
    pdl_wait();
    for (int i = threadIdx.x; i < n16; i += kHostStageThreads) dst_host[i] = __ldcg(src + i);
    __syncthreads();            // orders the CTA's stores before thread 0, whose fence then orders them before the flag
    if (threadIdx.x == 0) {
        tail_host[1] = (uint32_t)__ldcg(d_status);
        __threadfence_system();
        tail_host[0] = seq;
    }
}

}  // namespace gnf4b
