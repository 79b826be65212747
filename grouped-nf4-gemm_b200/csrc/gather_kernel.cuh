// Residency feeders: byte movers that put an expert's packed row-block into a device slot, selected on the device --
// by expert id from one stack (gather_rows_by_id, the reference's kernel/host_gather.py:33-54), by absolute address
// per slot (gather_rows_addr, kernel/mxfp4_pipelined.py:48-60) or by absolute address with the row's segments landing
// in a different order (the piece table of kernel/mxfp4_residency.py:117-134).  A slot whose wanted row is the one it
// already holds is skipped without touching the source: that is the residency engines' miss correction.  The source
// may be device memory or pinned host memory the GPU addresses directly (zero-copy reads over PCIe).
//
// Format-agnostic: bytes in, the same bytes out.  HBM/PCIe-bound; no shared-memory staging is needed because every
// byte is read once and written once: each thread keeps four 16-byte loads in flight, a CTA covers 32 KiB of one
// slot, the grid is (chunks, slots) so that a 17 MB row spreads over hundreds of CTAs.  Rows and pieces are multiples
// of 8 bytes (the reference moves int64 words); 16-byte accesses are used where source, destination and length allow.
#pragma once

#include "common.cuh"

namespace gnf4b {

constexpr int kGatherThreads = 256;
constexpr int kGatherUnroll = 4;
constexpr int64_t kGatherChunk = (int64_t)kGatherThreads * kGatherUnroll * 16 * 2;     // 32 KiB per CTA

// streaming load: read-only data that is used once (nothing is kept in L1 for it)
__device__ __forceinline__ uint4 ld_nc_na_16(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void gather_span(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int64_t lo, int64_t hi) {
    const int t = threadIdx.x;
    if ((((uintptr_t)dst | (uintptr_t)src | (uint64_t)lo | (uint64_t)hi) & 15) == 0) {
        const uint4* s = reinterpret_cast<const uint4*>(src + lo);
        uint4* d = reinterpret_cast<uint4*>(dst + lo);
        const int64_t n = (hi - lo) >> 4;
        for (int64_t i = t; i < n; i += (int64_t)kGatherThreads * kGatherUnroll) {
            uint4 v[kGatherUnroll];
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i + (int64_t)u * kGatherThreads < n) v[u] = ld_nc_na_16(s + i + (int64_t)u * kGatherThreads);
#pragma unroll
            for (int u = 0; u < kGatherUnroll; ++u)
                if (i + (int64_t)u * kGatherThreads < n) d[i + (int64_t)u * kGatherThreads] = v[u];
        }
    } else {
        const uint2* s = reinterpret_cast<const uint2*>(src + lo);
        uint2* d = reinterpret_cast<uint2*>(dst + lo);
        const int64_t n = (hi - lo) >> 3;
        for (int64_t i = t; i < n; i += kGatherThreads) d[i] = s[i];
    }
}

// MODE 0: want = src_base + ids[slot] * row_bytes (ids int32, have_ids int32 optional)
// MODE 1: want = want_addr[slot] (int64 absolute addresses, have_addr optional)
template <int MODE>
__global__ void __launch_bounds__(kGatherThreads)
gather_rows_kernel(uint8_t* __restrict__ dst, int64_t row_bytes, const uint8_t* src_base, const int32_t* __restrict__ ids,
                   const int32_t* __restrict__ have_ids, const int64_t* __restrict__ want_addr,
                   const int64_t* __restrict__ have_addr, int32_t n_rows_src, int32_t* status) {
    const int slot = blockIdx.y;
    const uint8_t* src;
    if (MODE == 0) {
        const int32_t want = __ldg(ids + slot);
        if (have_ids && __ldg(have_ids + slot) == want) return;
        if (want < 0 || (n_rows_src > 0 && want >= n_rows_src)) {       // never dereferenced
            if (status && blockIdx.x == 0 && threadIdx.x == 0) atomicOr(status, GNF4B_ST_BAD_EXPERT);
            return;
        }
        src = src_base + (int64_t)want * row_bytes;
    } else {
        const int64_t want = __ldg(want_addr + slot);
        if (have_addr && __ldg(have_addr + slot) == want) return;
        if (want == 0) return;
        src = reinterpret_cast<const uint8_t*>(want);
    }
    const int64_t lo = (int64_t)blockIdx.x * kGatherChunk;
    gather_span(dst + (int64_t)slot * row_bytes, src, lo, min(row_bytes, lo + kGatherChunk));
}

// Absolute address per slot plus a piece table: piece p copies pieces[3p + 2] bytes from source offset pieces[3p] to
// slot offset pieces[3p + 1].  grid = (chunks of the longest piece, pieces, slots).
__global__ void __launch_bounds__(kGatherThreads)
gather_rows_pieces_kernel(uint8_t* __restrict__ dst, int64_t row_bytes, const int64_t* __restrict__ want_addr,
                          const int64_t* __restrict__ have_addr, const int64_t* __restrict__ pieces) {
    const int slot = blockIdx.z, piece = blockIdx.y;
    const int64_t want = __ldg(want_addr + slot);
    if ((have_addr && __ldg(have_addr + slot) == want) || want == 0) return;
    const int64_t so = __ldg(pieces + 3 * piece), d_o = __ldg(pieces + 3 * piece + 1), n = __ldg(pieces + 3 * piece + 2);
    const int64_t lo = (int64_t)blockIdx.x * kGatherChunk;
    if (lo >= n) return;
    gather_span(dst + (int64_t)slot * row_bytes + d_o, reinterpret_cast<const uint8_t*>(want) + so, lo, min(n, lo + kGatherChunk));
}

}  // namespace gnf4b
