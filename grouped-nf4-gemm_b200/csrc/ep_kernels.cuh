// Row-wise helpers of the expert-parallel layer: the two elementwise passes that sit between the
// grouped GEMMs and the exchanges.  Both are HBM-bound (read once, write once, 16-byte accesses)
// and deterministic.
#pragma once

#include "common.cuh"

namespace gnf4b {

// out[r, c] = bf16( silu(gate[r, c]) * up[r, c] ), gate = gu[:, :h], up = gu[:, h:], fp32 math.
// VEC = 8 (h % 8 == 0, 16-byte aligned rows) or 1.
template <int VEC>
__global__ void silu_glu_kernel(const uint16_t* __restrict__ gu, int64_t rows, int64_t h, uint16_t* __restrict__ out) {
    const int64_t per_row = h / VEC;
    const int64_t total = rows * per_row;
    EPT(50);
    pdl_launch_dependents();          // launched with programmatic stream serialization: the next kernel may set up now
    pdl_wait();                       // and this one reads nothing before the kernel that wrote gu has finished
    EPT(51);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = (i - r * per_row) * VEC;
        const uint16_t* g = gu + r * 2 * h + c;
        if (VEC == 8) {
            const uint4 gv = __ldg(reinterpret_cast<const uint4*>(g));
            const uint4 uv = __ldg(reinterpret_cast<const uint4*>(g + h));
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
                const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
                ow[j] = (uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g0), u0)) |
                        ((uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g1), u1)) << 16);
            }
            *reinterpret_cast<uint4*>(out + r * h + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        } else {
            const float gf = bf16_bits_to_float(g[0]), uf = bf16_bits_to_float(g[h]);
            out[r * h + c] = f32_to_bf16_bits(__fmul_rn(silu_f32(gf), uf));
        }
    }
}

// out[r, c] = glu_gpt_oss(gu[r, 2c] (+ bias[e, 2c]), gu[r, 2c + 1] (+ bias[e, 2c + 1])), e = row_expert[r]: the
// activation of gpt-oss between its two expert GEMMs, gate and up interleaved in the columns.  The optional
// per-expert bias is added first, in bf16 like the reference does (kernel/mxfp4_pipelined.py:441-442).
__global__ void glu_gpt_oss_kernel(const uint16_t* __restrict__ gu, int64_t rows, int64_t h, const uint16_t* __restrict__ bias,
                                   const int32_t* __restrict__ row_expert, uint16_t* __restrict__ out) {
    const int64_t total = rows * h;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / h, c = i - r * h;
        const uint32_t pair = __ldg(reinterpret_cast<const uint32_t*>(gu + r * 2 * h) + c);
        float g = __uint_as_float(pair << 16), u = __uint_as_float(pair & 0xffff0000u);
        if (bias) {
            const uint32_t bp = __ldg(reinterpret_cast<const uint32_t*>(bias + (int64_t)__ldg(row_expert + r) * 2 * h) + c);
            g = bf16_round(__fadd_rn(g, __uint_as_float(bp << 16)));
            u = bf16_round(__fadd_rn(u, __uint_as_float(bp & 0xffff0000u)));
        }
        out[i] = f32_to_bf16_bits(glu_gpt_oss(g, u));
    }
}

// out[m, :] = bf16( sum_j w[m, j] * rows[pos[m, j], :] ), j = 0..k-1 in order, fp32, multiply and add
// rounded separately (no fused multiply-add) so that a plain loop of tensor operations gives the same bits.
// One thread = 8 consecutive columns of one token (VEC = 8) or one column (VEC = 1).
template <int VEC>
__global__ void combine_rows_kernel(const uint16_t* __restrict__ rows, const int64_t* __restrict__ pos,
                                    const float* __restrict__ w, int32_t k, int64_t M, int64_t H, int64_t P,
                                    uint16_t* __restrict__ out, int32_t* status) {
    const int64_t per_row = H / VEC;
    const int64_t total = M * per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / per_row, c = (i - m * per_row) * VEC;
        float acc[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
        for (int j = 0; j < k; ++j) {
            const int64_t p = __ldg(pos + m * k + j);
            if (p < 0 || p >= P) {                     // never dereferenced
                if (status) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
                continue;
            }
            const float wj = __ldg(w + m * k + j);
            const uint16_t* src = rows + p * H + c;
            if (VEC == 8) {
                const uint4 rv = __ldg(reinterpret_cast<const uint4*>(src));
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(__uint_as_float(rw[q] << 16), wj));
                    acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(__uint_as_float(rw[q] & 0xffff0000u), wj));
                }
            } else {
                acc[0] = __fadd_rn(acc[0], __fmul_rn(bf16_bits_to_float(src[0]), wj));
            }
        }
        if (VEC == 8) {
            uint32_t ow[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
                ow[q] = (uint32_t)f32_to_bf16_bits(acc[2 * q]) | ((uint32_t)f32_to_bf16_bits(acc[2 * q + 1]) << 16);
            *reinterpret_cast<uint4*>(out + m * H + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        } else {
            out[m * H + c] = f32_to_bf16_bits(acc[0]);
        }
    }
}

}  // namespace gnf4b

namespace gnf4b {

// Routing plan of the fixed-capacity exchange for a small batch, ONE CTA: per-expert counts, the row of
// every (token, choice) pair in the send buffer -- destination rank d = expert / experts_per_rank gets
// rows [d * cap, d * cap + ...) ordered by local expert, pairs of one expert in pair order -- and the
// copy of the pairs' hidden rows into those slots.  P = tokens * top_k <= 1024, n_experts <= 1024.
// A pair whose expert id is out of range gets slot -1, is not sent and is flagged (GNF4B_ST_BAD_EXPERT);
// so does a pair beyond the cap rows of its destination rank (GNF4B_ST_BAD_OFFSETS).
constexpr int kEpPlanThreads = 256;
constexpr int kEpPlanMax = 1024;

__global__ void __launch_bounds__(kEpPlanThreads, 1)
ep_plan_kernel(const int64_t* __restrict__ idx, int32_t P, int32_t k, int32_t n_experts, int32_t e_local, int32_t cap,
               const uint16_t* __restrict__ hidden, int64_t H, int32_t* __restrict__ counts, int64_t* __restrict__ slot,
               uint16_t* __restrict__ send, int32_t* status) {
    __shared__ int32_t s_e[kEpPlanMax];        // expert of pair p (-1: invalid)
    __shared__ int32_t s_hist[kEpPlanMax];     // pairs per expert
    __shared__ int32_t s_base[kEpPlanMax];     // pairs of lower experts on the same destination rank
    __shared__ int64_t s_slot[kEpPlanMax];
    const int t = threadIdx.x;
    for (int e = t; e < n_experts; e += kEpPlanThreads) s_hist[e] = 0;
    __syncthreads();
    for (int p = t; p < P; p += kEpPlanThreads) {
        const int64_t e = idx[p];
        const bool ok = e >= 0 && e < n_experts;
        s_e[p] = ok ? (int32_t)e : -1;
        if (ok) atomicAdd(&s_hist[e], 1);
        else if (status) atomicOr(status, GNF4B_ST_BAD_EXPERT);
    }
    __syncthreads();
    for (int e = t; e < n_experts; e += kEpPlanThreads) {
        int32_t b = 0;
        for (int q = (e / e_local) * e_local; q < e; ++q) b += s_hist[q];
        s_base[e] = b;
        counts[e] = s_hist[e];
    }
    __syncthreads();
    for (int p = t; p < P; p += kEpPlanThreads) {
        const int32_t e = s_e[p];
        int64_t s = -1;
        if (e >= 0) {
            int32_t rank = 0;
            for (int q = 0; q < p; ++q) rank += (s_e[q] == e);
            // a destination rank that would get more than cap pairs: the pair is not sent and the call is
            // flagged, never written into the next rank's block (or past the end of send)
            if (s_base[e] + rank < cap) s = (int64_t)(e / e_local) * cap + s_base[e] + rank;
            else if (status) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
        }
        s_slot[p] = s;
        slot[p] = s;
    }
    __syncthreads();
    // copy the rows: 16 bytes per thread and step when the rows allow it
    const bool vec = (H % 8) == 0 && ((reinterpret_cast<uintptr_t>(hidden) | reinterpret_cast<uintptr_t>(send)) & 15) == 0;
    if (vec) {
        const int64_t per_row = H / 8;
        for (int64_t i = t; i < (int64_t)P * per_row; i += kEpPlanThreads) {
            const int p = (int)(i / per_row);
            const int64_t c = (i - (int64_t)p * per_row) * 8;
            if (s_slot[p] >= 0)
                *reinterpret_cast<uint4*>(send + s_slot[p] * H + c) =
                    __ldg(reinterpret_cast<const uint4*>(hidden + (int64_t)(p / k) * H + c));
        }
    } else {
        for (int64_t i = t; i < (int64_t)P * H; i += kEpPlanThreads) {
            const int p = (int)(i / H);
            const int64_t c = i - (int64_t)p * H;
            if (s_slot[p] >= 0) send[s_slot[p] * H + c] = hidden[(int64_t)(p / k) * H + c];
        }
    }
}

}  // namespace gnf4b

namespace gnf4b {

// Router selection, one warp per token: the k largest logits in descending order, ties to the lower
// expert index, and their weights -- mode 0: softmax over all E experts (norm: renormalised over the k),
// mode 1: softmax over the k selected.  Same rule as the reference's CPU router
// (gnf4_native/cpu_kernels.c:1408-1471).  k <= 32.
__global__ void route_topk_kernel(const float* __restrict__ logits, int64_t T, int32_t E, int32_t k, int32_t mode,
                                  int32_t norm, int64_t* __restrict__ idx, float* __restrict__ w) {
    const int lane = threadIdx.x & 31;
    const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* lg = logits + t * E;
    // each lane keeps the position of its own last pick so it never offers an element twice
    float sel_v = 0.f;            // value of the pick with rank == lane
    int32_t sel_i = 0;
    float prev_v = INFINITY;
    int32_t prev_i = -1;
    for (int j = 0; j < k; ++j) {
        // best remaining element: smaller than the previous pick, or equal with a larger index
        float bv = -INFINITY;
        int32_t bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = __ldg(lg + e);
            const bool after_prev = v < prev_v || (v == prev_v && e > prev_i);
            if (after_prev && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == j) { sel_v = bv; sel_i = bi; }
        prev_v = bv;
        prev_i = bi;
    }
    const float top = __shfl_sync(0xffffffffu, sel_v, 0);
    float wj;
    if (mode == 0) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, __ldg(lg + e));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float z = 0.f;
        for (int e = lane; e < E; e += 32) z += expf(__ldg(lg + e) - m);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        wj = (lane < k) ? expf(sel_v - m) / z : 0.f;
        if (norm) {
            float s = wj;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            wj /= s;
        }
    } else {
        const float ej = (lane < k) ? expf(sel_v - top) : 0.f;
        float z = ej;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        wj = ej / z;
    }
    if (lane < k) {
        idx[t * k + lane] = sel_i;
        w[t * k + lane] = wj;
    }
}

}  // namespace gnf4b

namespace gnf4b {

// Routing plan of a LARGE batch (any number of pairs): the stable sort of the (token, choice) pairs by
// (half, global expert id) as a counting sort over several CTAs, and the gather of the pairs' hidden rows into that
// order.  half = 1 for experts whose local index (id % e_local) is >= cut, so that with cut < e_local every rank's
// lower experts come first (the layer pipelined over two halves of the local experts); cut = e_local: one half.
// Three small kernels and one copy:
//   hist    CTA b counts the bins of its chunk of kEpChunk pairs                       -> hist[b][bin]
//   starts  one CTA: per bin the pairs of lower bins and of lower CTAs                  -> hist[b][bin] = first position,
//           per expert the number of pairs                                              -> counts[e]
//   place   CTA b: position of each of its pairs = first position of (b, bin) + the pair's rank among the
//           chunk's earlier pairs of the same bin (stable)                              -> pos[p]
//   rows    send[pos[p], :] = hidden[p / k, :], 16 bytes per thread and step
// Same order as a stable argsort of the keys; an expert id outside [0, n_experts) is flagged and its pair is placed
// after all valid pairs (never sent: it is counted by no expert).
constexpr int kEpChunk = 512;
constexpr int kEpLargeThreads = 256;
constexpr int kEpMaxBins = 2048 + 1;          // 2 halves x 1024 experts + the bin of invalid ids

__device__ __forceinline__ int32_t ep_bin(int64_t e, int32_t n_experts, int32_t e_local, int32_t cut) {
    if (e < 0 || e >= n_experts) return 2 * n_experts;
    return (int32_t)e + (((int32_t)e % e_local) >= cut ? n_experts : 0);
}

__global__ void __launch_bounds__(kEpLargeThreads)
ep_large_hist_kernel(const int64_t* __restrict__ idx, int64_t P, int32_t n_experts, int32_t e_local, int32_t cut,
                     int32_t* __restrict__ hist, int32_t* status) {
    __shared__ int32_t s_h[kEpMaxBins];
    const int n_bins = 2 * n_experts + 1;
    for (int i = threadIdx.x; i < n_bins; i += kEpLargeThreads) s_h[i] = 0;
    __syncthreads();
    const int64_t lo = (int64_t)blockIdx.x * kEpChunk;
    for (int i = threadIdx.x; i < kEpChunk && lo + i < P; i += kEpLargeThreads) {
        const int32_t b = ep_bin(__ldg(idx + lo + i), n_experts, e_local, cut);
        if (b == 2 * n_experts && status) atomicOr(status, GNF4B_ST_BAD_EXPERT);
        atomicAdd(&s_h[b], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_bins; i += kEpLargeThreads) hist[(int64_t)blockIdx.x * n_bins + i] = s_h[i];
}

__global__ void __launch_bounds__(1024, 1)
ep_large_starts_kernel(int32_t* __restrict__ hist, int32_t n_ctas, int32_t n_experts, int32_t* __restrict__ counts) {
    __shared__ int32_t s_tot[kEpMaxBins];
    __shared__ int32_t s_start[kEpMaxBins];
    const int n_bins = 2 * n_experts + 1;
    for (int b = threadIdx.x; b < n_bins; b += blockDim.x) {
        int32_t n = 0;
        for (int c = 0; c < n_ctas; ++c) n += hist[(int64_t)c * n_bins + b];
        s_tot[b] = n;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t at = 0;
        for (int b = 0; b < n_bins; ++b) { s_start[b] = at; at += s_tot[b]; }
    }
    __syncthreads();
    for (int b = threadIdx.x; b < n_bins; b += blockDim.x) {
        int32_t at = s_start[b];
        for (int c = 0; c < n_ctas; ++c) {
            const int32_t n = hist[(int64_t)c * n_bins + b];
            hist[(int64_t)c * n_bins + b] = at;
            at += n;
        }
    }
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = s_tot[e] + s_tot[e + n_experts];
}

__global__ void __launch_bounds__(kEpLargeThreads)
ep_large_place_kernel(const int64_t* __restrict__ idx, int64_t P, int32_t n_experts, int32_t e_local, int32_t cut,
                      const int32_t* __restrict__ hist, int64_t* __restrict__ pos) {
    __shared__ int32_t s_bin[kEpChunk];
    const int n_bins = 2 * n_experts + 1;
    const int64_t lo = (int64_t)blockIdx.x * kEpChunk;
    const int n = (int)min((int64_t)kEpChunk, P - lo);
    for (int i = threadIdx.x; i < n; i += kEpLargeThreads) s_bin[i] = ep_bin(__ldg(idx + lo + i), n_experts, e_local, cut);
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kEpLargeThreads) {
        const int32_t b = s_bin[i];
        int32_t rank = 0;
        for (int q = 0; q < i; ++q) rank += (s_bin[q] == b);
        pos[lo + i] = (int64_t)__ldg(hist + (int64_t)blockIdx.x * n_bins + b) + rank;
    }
}

__global__ void __launch_bounds__(kEpLargeThreads)
ep_large_rows_kernel(const uint16_t* __restrict__ hidden, int64_t P, int32_t k, int64_t H, const int64_t* __restrict__ pos,
                     uint16_t* __restrict__ send) {
    const int64_t per_row = H / 8;
    for (int64_t i = (int64_t)blockIdx.x * kEpLargeThreads + threadIdx.x; i < P * per_row; i += (int64_t)gridDim.x * kEpLargeThreads) {
        const int64_t p = i / per_row, c = (i - p * per_row) * 8;
        *reinterpret_cast<uint4*>(send + __ldg(pos + p) * H + c) = __ldg(reinterpret_cast<const uint4*>(hidden + (p / k) * H + c));
    }
}

}  // namespace gnf4b
