// Shared device helpers: codebooks, scale conversion, mbarrier / bulk-copy PTX wrappers
// with bounded waits.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gnf4b.h"

namespace gnf4b {

// ---- codebooks (values identical to NF4_LUT / FP4_VALUES of the reference,
//      kernel/nf4_grouped.py:53-70 and kernel/mxfp4_grouped.py:34-35) ----
__device__ __constant__ float kNf4Lut[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
    0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
    0.7229568362236023f, 1.0f};
__device__ __constant__ float kFp4Lut[16] = {
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

// Both codebook values of one packed byte, in ELEMENT order (even element first).
// NF4 keeps the even element in the high nibble, MXFP4 in the low nibble.
// MXFP4 values come back DOUBLED (0, 1, 2, 3, 4, 6, 8, 12) and load_scale returns
// 2^(e-128): the product is the same number, every step is exact, and the largest block
// exponent (e = 255, i.e. 2^128, not an fp32 value) needs no special case -- 0.5 * 2^128
// is the finite 2^127, larger magnitudes overflow to inf and zeros stay zero, exactly as
// ldexp(value, e - 127) does.
template <int FMT>
__device__ __forceinline__ float2 byte_pair(uint32_t b) {
    if (FMT == GNF4B_FMT_NF4) return make_float2(kNf4Lut[b >> 4], kNf4Lut[b & 15]);
    return make_float2(2.0f * kFp4Lut[b & 15], 2.0f * kFp4Lut[b >> 4]);
}

// The same pair with the codebook values taken from instruction immediates (a select chain) instead of constant
// memory: a kernel that decodes only while it builds a lookup table would otherwise start with a constant-cache
// miss (about a microsecond before its first table row is written).  MXFP4 doubled as above.
template <int FMT>
__device__ __forceinline__ float code_value_imm(uint32_t c) {
    constexpr uint32_t nf4[16] = {0xbf800000u, 0xbf3239b1u, 0xbf066b30u, 0xbeca32a0u, 0xbe91a24du, 0xbe3d353fu, 0xbdba7871u, 0x0u,
                                  0x3da2faffu, 0x3e24cae3u, 0x3e7c04ddu, 0x3ead033au, 0x3ee1a4b8u, 0x3f1007abu, 0x3f3913b3u, 0x3f800000u};
    if (FMT == GNF4B_FMT_NF4) {
        uint32_t v = nf4[15];
#pragma unroll
        for (int i = 14; i >= 0; --i) v = (c == (uint32_t)i) ? nf4[i] : v;
        return __uint_as_float(v);
    }
    // doubled e2m1 magnitudes 0, 1, 2, 3, 4, 6, 8, 12: small integers, exact in every float format
    const uint32_t m = c & 7u;
    const uint32_t v = __float_as_uint((float)(m < 4u ? m : (2u + (m & 1u)) << ((m >> 1) - 1u)));
    return __uint_as_float(v | ((c & 8u) << 28));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t h) { return __uint_as_float(h << 16); }

// One block scale as fp32.  NF4: the absmax itself (bf16 widened exactly).  MXFP4:
// 2^(e-128) (see byte_pair): subnormal for e < 2, always finite.
template <int SDT>
__device__ __forceinline__ float load_scale(const void* base, int64_t idx) {
    if (SDT == GNF4B_S_F32) return __ldg(reinterpret_cast<const float*>(base) + idx);
    if (SDT == GNF4B_S_BF16)
        return bf16_bits_to_float(__ldg(reinterpret_cast<const unsigned short*>(base) + idx));
    const uint32_t e = __ldg(reinterpret_cast<const unsigned char*>(base) + idx);
    return __uint_as_float(e >= 2 ? (e - 1) << 23 : 0x00200000u << e);
}

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrive without ordering earlier memory operations.  For "this warp has finished READING a ring stage": the
// reads have completed when their values were used, and a release arrive would also wait for the
// acknowledgement of every global store the thread issued before it (half a microsecond per output row).
__device__ __forceinline__ void mbar_arrive_relaxed(uint64_t* bar) {
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Every wait in these kernels is bounded: after kWaitLimitCycles SM cycles (about two
// seconds) without progress the waiter raises *abort_flag (shared memory), every other
// waiter of the CTA sees it and leaves too; the kernel then records GNF4B_ST_TIMEOUT and
// returns.  The SM cycle counter is used because it is cheap to read.
constexpr long long kWaitLimitCycles = 4000000000ll;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may
// start while the previous kernel of the stream is still running: everything up to pdl_wait() (barrier
// set-up, lookup tables) overlaps that kernel's tail; pdl_wait() returns once all earlier grids have
// completed and their writes are visible, so it must precede the first read of anything an earlier
// kernel may have written and every global write.  pdl_launch_dependents() lets the NEXT kernel start
// the same way.  Both are no-ops for a kernel launched without the attribute.
// Timeline of a chain of kernels, for development builds only (-DGNF4B_EP_TRACE; the shipped library compiles
// EPT() to nothing): thread 0 of CTA 0 appends (mark, %globaltimer) pairs to a device array that
// gnf4b_ep_trace_read() copies out.  The marks are the numbers at the EPT() sites (tens = kernel, units = phase).
#ifdef GNF4B_EP_TRACE
__device__ unsigned long long g_ep_trace[8192];
__device__ unsigned int g_ep_trace_n;
#define EPT(id) do { if (threadIdx.x == 0 && blockIdx.x == 0) { unsigned i_ = atomicAdd(&g_ep_trace_n, 1u); if (i_ < 4096u) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_ep_trace[2 * i_] = (id); g_ep_trace[2 * i_ + 1] = t_; } } } while (0)
#else
#define EPT(id) do { } while (0)
#endif
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 1-D bulk copy global -> shared, completion counted on an mbarrier (TMA engine).
// Both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 ld_shared_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 ld_shared_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ld_shared_u32x4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

// The GLU of gpt-oss on one (gate, up) pair of bf16 values: gate clamped from above at 7, up clamped to [-7, 7],
// (up + 1) * gate * sigmoid(1.702 gate) -- evaluated the way the reference evaluates it, as a chain of bf16 tensor
// operations (kernel/mxfp4_pipelined.py:453-461): every intermediate is computed in fp32 and rounded to bf16.
// Returns the bf16-representable result as a float.
__device__ __forceinline__ float glu_gpt_oss(float gate, float up) {
    const float g = fminf(gate, 7.0f);
    const float u = fminf(fmaxf(up, -7.0f), 7.0f);
    const float t1 = bf16_round(__fmul_rn(g, 1.702f));
    const float t2 = bf16_round(1.0f / (1.0f + expf(-t1)));
    const float t3 = bf16_round(__fmul_rn(g, t2));
    const float t4 = bf16_round(__fadd_rn(u, 1.0f));
    return bf16_round(__fmul_rn(t4, t3));
}

// Problem description shared by all GEMM kernels.
struct GemmArgs {
    const void* x;          // activations / grad rows
    const uint8_t* W;       // packed nibbles
    const void* S;          // scales
    const int32_t* off;     // [G+1]
    const int32_t* eids;    // [G]
    void* out;              // bf16
    float* ws;              // split-K partials [split][T][N]
    int32_t* counters;      // split-K arrival counters, one per (group, n-tile)
    int32_t* status;        // optional
    int64_t w_se, w_sn;     // bytes
    int64_t s_se, s_sn;     // elements
    int64_t T, N, K;
    int32_t G, E;
    int32_t x_dtype;
    int32_t split_k;
};

}  // namespace gnf4b
