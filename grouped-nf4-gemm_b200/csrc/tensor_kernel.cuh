// tcgen05 / TMEM grouped GEMM for prefill-sized groups (placeholder until the kernel lands).
#pragma once
#include "common.cuh"
namespace gnf4b {
static int launch_tensor(int fmt, int op, int s_dtype, const GemmArgs& g, int max_rows, int sm_count,
                         int smem_optin, cudaStream_t st) {
    (void)fmt; (void)op; (void)s_dtype; (void)g; (void)max_rows; (void)sm_count; (void)smem_optin; (void)st;
    return GNF4B_EUNSUPPORTED;
}
}  // namespace gnf4b
