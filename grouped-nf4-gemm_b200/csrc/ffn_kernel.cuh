// Fused expert FFN for decode-sized batches (every group has ONE row): gate_up GEMV -> GLU -> down GEMV in ONE
// persistent launch.  The GPU counterpart of the reference's fused CPU entry point gnf4_gemv_nf4_ffn_grouped
// (gnf4_native/cpu_kernels.c:763-986); the activation is SiLU(gate) * up with gate = the first half of the
// gate_up columns (ACT 0, the reference's CPU FFN and bench/phase3/offload_decode_235b.py:232-233), or the
// interleaved clamped GLU of gpt-oss (ACT 1, kernel/mxfp4_pipelined.py:453-461).
//
// One CTA per SM, the warps of the decode kernel (16 consumers + 1 producer), its lookup table and its ring.
// The work list is every (group, weight-row tile) of gate_up followed by every (group, tile) of down; each CTA
// takes an even, contiguous share of both.  The producer lane streams its gate_up share and then its down share
// through the same ring without a pause -- weights depend on nothing -- so the down weights are already in shared
// memory when the gate_up phase ends.  Consumers write gate_up results (bf16) to a scratch matrix in global
// memory; when a CTA leaves a group it adds the rows it finished to that group's counter (barrier, fence, atomic
// add by one thread).  A down item of group g waits -- bounded, one polling thread per CTA -- until the counter
// says all N_gu gate_up columns of g exist; the CTA then builds h = act(gate, up) once in shared memory (fp32
// math, one rounding to bf16: bit for bit what the separate GLU kernel writes), every warp takes its lanes'
// share of it into registers and runs the same GEMV.  Results equal the three-launch composition gate_up GEMM
// -> GLU -> down GEMM exactly.
//
// What it buys, measured on B200 at the Qwen3-30B-A3B layer with 8 one-row groups: 16.5 us against 18.1 us for
// the three programmatically chained launches, and one launch instead of three for the host.  Not more, because
// the hand-over between the phases is a grid-wide dependency through global memory (fence, atomic, poll, reload:
// each a round trip of most of a microsecond) -- about what the start of a chained kernel costs -- and the time
// is dominated by the consumers' table lookups either way.  Building h once per CTA (not once per warp, which
// cost 9 us) and polling with one thread (not 512) are what made it faster than the three launches at all.
//
// All CTAs are resident at once (grid <= SM count, one CTA per SM), which the waits rely on; every wait is
// bounded and raises GNF4B_ST_TIMEOUT instead of hanging.  The counters must be zero when the kernel starts: the
// last CTA to finish clears them again.
#pragma once

#include "common.cuh"
#include "decode_kernel.cuh"

namespace gnf4b {

constexpr int kFfnCW = 16;                       // consumer warps
constexpr int kFfnThreads = (kFfnCW + 1) * 32;

struct FfnPhase {
    const uint8_t* W;
    const void* S;
    int64_t w_se, s_se;         // expert strides: bytes / scale elements (rows are contiguous)
    int32_t N;                  // weight rows (output columns) of this projection
    int32_t rows_per_stage;     // R
    int32_t tiles_per_group;    // ceil(N / R)
    int32_t row_bytes, scale_row_bytes;
    int32_t items_per_cta, items_extra;      // G * tiles_per_group dealt over the grid
};

struct FfnArgs {
    const void* x;              // [T, K_gu] bf16
    FfnPhase ph[2];             // gate_up, down
    const int32_t* off;         // [G + 1]
    const int32_t* eids;        // [G]
    const uint16_t* bias_gu;    // optional bf16 [E, N_gu], added to gate_up (in bf16) before the activation
    uint16_t* gu;               // scratch, bf16 [T, N_gu]
    uint16_t* out;              // bf16 [T, N_dn]
    int32_t* counters;          // [G] gate_up columns finished per group, [G] = CTAs finished; zero at launch
    int32_t* status;
    int64_t T;
    int32_t G, E;
    int32_t K_gu, H;            // H = N_gu / 2 = the contraction length of down
    int32_t slot_bytes, stages;
    int32_t tables_ready;
};

// Dynamic shared memory: [slack][table 64 KiB][ring][barriers, abort flag: 256 B][h row: H bf16]
__host__ __device__ inline size_t ffn_smem_bytes(int slot_bytes, int stages, int H) {
    return (size_t)kDTabAbs + (size_t)kSTableBytes + (size_t)stages * slot_bytes + 256 + (size_t)H * 2;
}

__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct FfnGroup {
    int32_t row0, eid;
    bool valid;
};

__device__ __forceinline__ FfnGroup ffn_group(const FfnArgs& a, int g, bool flag) {
    const int32_t row0 = __ldg(a.off + g), end = __ldg(a.off + g + 1), eid = __ldg(a.eids + g);
    FfnGroup d;
    d.row0 = row0;
    d.eid = eid;
    const bool bad_e = eid < 0 || eid >= a.E;
    const bool bad_o = end < row0 || row0 < 0 || end > a.T || end - row0 > 1;     // this kernel takes one-row groups
    d.valid = !bad_e && !bad_o && end > row0;
    const bool pad = eid == GNF4B_PAD_EXPERT;
    if (flag && ((bad_e && !pad) || bad_o) && end != row0 && a.status && (threadIdx.x & 31) == 0)
        atomicOr(a.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
    return d;
}

// AU: 16-byte units per lane of the longer of the two contractions (K_gu, H <= AU * 1024).  RW, XF as in the decode
// kernel.  ACT: 0 SiLU(gate) * up over column halves; 1 gpt-oss: gate / up interleaved, clamped, (up + 1) * gate *
// sigmoid(1.702 gate).
template <int FMT, int SDT, int AU, int RW, int XF, int ACT>
__global__ void __launch_bounds__(kFfnThreads, 1) ffn_decode_kernel(const FfnArgs a) {
    constexpr int kXN = XF == 1 ? AU * 32 : AU * 16;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* tab_raw = smem + ((uint32_t)kDTabAbs - smem_base);
    uint8_t* ring = tab_raw + kSTableBytes;
    uint8_t* tail = ring + (size_t)a.stages * a.slot_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kDMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kDMaxStages);
    uint4* h_s = reinterpret_cast<uint4*>(tail + 256);      // the current group's h row, bf16

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bid = (int)blockIdx.x;

    pdl_launch_dependents();
    if (smem_base > (uint32_t)kDTabAbs) {
        if (threadIdx.x == 0 && a.status) atomicOr(a.status, GNF4B_ST_TIMEOUT);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kFfnCW);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    int32_t lo[2], hi[2];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        lo[p] = bid * a.ph[p].items_per_cta + min(bid, a.ph[p].items_extra);
        hi[p] = lo[p] + a.ph[p].items_per_cta + (bid < a.ph[p].items_extra ? 1 : 0);
    }

    if (warp == kFfnCW) {
        // ------------------------------------------------------------ producer (two lanes), both phases back to back
        if (lane < 2) {
            if (!a.tables_ready) pdl_wait();
            const int elt = (SDT == GNF4B_S_F32) ? 4 : (SDT == GNF4B_S_BF16 ? 2 : 1);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int p = 0; p < 2 && ok; ++p) {
                const FfnPhase& ph = a.ph[p];
                const uint8_t* Sb = reinterpret_cast<const uint8_t*>(ph.S);
                int g = lo[p] / ph.tiles_per_group, tile = lo[p] - g * ph.tiles_per_group, cur_g = -1;
                FfnGroup grp;
                grp.valid = false;
                for (int item = lo[p]; item < hi[p]; ++item) {
                    if (cur_g != g) { grp = ffn_group(a, g, false); cur_g = g; }
                    ok = mbar_wait_bounded(empty_bar + stage, phase ^ 1, abort_flag);
                    if (!ok) break;
                    if (grp.valid) {
                        uint8_t* st = ring + (size_t)stage * a.slot_bytes;
                        const int n0 = tile * ph.rows_per_stage;
                        const int rows = min(ph.rows_per_stage, ph.N - n0);
                        const uint32_t wb = (uint32_t)rows * (uint32_t)ph.row_bytes;
                        const uint32_t sb = (uint32_t)rows * (uint32_t)ph.scale_row_bytes;
                        if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, wb + sb);
                        __syncwarp(0x3u);
                        const uint8_t* src = (lane == 0)
                            ? ph.W + (int64_t)grp.eid * ph.w_se + (int64_t)n0 * ph.row_bytes
                            : Sb + ((int64_t)grp.eid * ph.s_se) * elt + (int64_t)n0 * ph.scale_row_bytes;
                        bulk_g2s(lane == 0 ? st : st + (size_t)ph.rows_per_stage * ph.row_bytes, src, lane == 0 ? wb : sb,
                                 full_bar + stage);
                    } else if (lane == 0) {
                        mbar_arrive(full_bar + stage);
                    }
                    if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
                    if (++tile == ph.tiles_per_group) { tile = 0; ++g; }
                }
            }
            if (!ok && lane == 0 && a.status) atomicOr(a.status, GNF4B_ST_TIMEOUT);
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    // With ready tables the first group of either phase is read before the dependency wait (the loads fly while
    // the table is built), and a hint brings the first activation row's lines into L2.
    const bool early = a.tables_ready != 0;
    FfnGroup first[2];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        first[p].valid = false;
        first[p].row0 = 0;
        first[p].eid = 0;
        if (early && lo[p] < hi[p]) first[p] = ffn_group(a, lo[p] / a.ph[p].tiles_per_group, false);
    }
    build_lookup_table<FMT, XF, kFfnCW>(warp, lane);
    if (early && warp == 0 && first[0].valid) {
        const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.x) + (int64_t)first[0].row0 * a.K_gu * 2;
        for (int o = lane * 128; o < a.K_gu * 2; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(xrow + o));
    }
    pdl_wait();
    named_bar_sync(1, kFfnCW * 32);

    const uint32_t lane8 = (uint32_t)lane * (XF == 2 ? 4u : 8u);
    uint32_t xr[1][kXN];
    uint32_t stage = 0, phase = 0;
    bool poisoned = false;

    // One bf16 pair (elements 2j, 2j + 1 of this lane's unit) into the register form of the activations
    auto put_pair = [&](int q, int v, int j, uint32_t pair) {
        if (XF == 1) {
            xr[0][q * 32 + v * 8 + 2 * j] = pair << 16;
            xr[0][q * 32 + v * 8 + 2 * j + 1] = pair & 0xffff0000u;
        } else {
            xr[0][q * 16 + v * 4 + j] = pair;
        }
    };

    for (int p = 0; p < 2; ++p) {
        const FfnPhase& ph = a.ph[p];
        const int n_units = ph.row_bytes >> 4;
        int g = lo[p] / ph.tiles_per_group, tile = lo[p] - g * ph.tiles_per_group, cur_g = -1;
        int done_in_group = 0;         // gate_up columns this CTA finished in the current group
        FfnGroup grp;
        grp.valid = false;
        grp.row0 = 0;
        uint16_t* dst = p == 0 ? a.gu : a.out;

        // leaving a group of the gate_up phase: publish what this CTA finished of it
        auto publish = [&]() {
            if (p == 0 && cur_g >= 0 && done_in_group > 0) {
                named_bar_sync(1, kFfnCW * 32);          // every warp's rows of the group are written
                if (threadIdx.x == 0) {
                    __threadfence();
                    atomicAdd(a.counters + cur_g, done_in_group);
                }
            }
            done_in_group = 0;
        };

        for (int item = lo[p]; item < hi[p]; ++item) {
            if (cur_g != g) {
                publish();
                if (early && item == lo[p]) {
                    grp = first[p];
                    if (p == 0 && tile == 0) (void)ffn_group(a, g, true);      // for its flags only
                } else {
                    grp = ffn_group(a, g, p == 0 && tile == 0);
                }
                cur_g = g;
                if (p == 0) {
                    // the group's activation row
                    const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.x) + (int64_t)grp.row0 * a.K_gu * 2;
#pragma unroll
                    for (int q = 0; q < AU; ++q) {
                        const int U = lane + 32 * q;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const uint4 raw = (grp.valid && U < n_units)
                                                  ? __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)U * 64 + v * 16))
                                                  : make_uint4(0, 0, 0, 0);
                            put_pair(q, v, 0, raw.x);
                            put_pair(q, v, 1, raw.y);
                            put_pair(q, v, 2, raw.z);
                            put_pair(q, v, 3, raw.w);
                        }
                    }
                } else {
                    // Every warp is done with the previous group's h row; one thread waits (bounded, pauses between
                    // reads) until every gate_up column of this group exists; then the whole CTA builds the group's
                    // h row once in shared memory and every warp takes its lanes' share into registers.  grp.valid
                    // is the same in every warp, so all of them take these barriers.
                    named_bar_sync(1, kFfnCW * 32);
                    if (grp.valid && threadIdx.x == 0) {
                        const long long t0 = clock64();
                        uint32_t spins = 0;
                        while (ld_acquire_gpu(a.counters + g) < a.ph[0].N) {
                            __nanosleep(32);
                            if ((++spins & 63u) == 0 && (*abort_flag || clock64() - t0 > kWaitLimitCycles)) {
                                *abort_flag = 1;
                                break;
                            }
                        }
                    }
                    named_bar_sync(1, kFfnCW * 32);
                    if (*abort_flag) poisoned = true;
                    const uint16_t* gurow = a.gu + (int64_t)grp.row0 * a.ph[0].N;
                    for (int c = threadIdx.x; c < a.H / 8 && grp.valid && !poisoned; c += kFfnCW * 32) {
                        const int e0 = c * 8;                  // 8 h elements per thread and step
                        uint32_t hw[4];
                        if (ACT == 0) {
                            const uint4 gv = __ldcg(reinterpret_cast<const uint4*>(gurow + e0));
                            const uint4 uv = __ldcg(reinterpret_cast<const uint4*>(gurow + a.H + e0));
                            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
                                const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
                                hw[j] = (uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g0), u0)) |
                                        ((uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g1), u1)) << 16);
                            }
                        } else {
                            // gate = column 2e, up = column 2e + 1: 16 consecutive bf16 give 8 h elements
                            const uint4 c0 = __ldcg(reinterpret_cast<const uint4*>(gurow + 2 * e0));
                            const uint4 c1 = __ldcg(reinterpret_cast<const uint4*>(gurow + 2 * e0 + 8));
                            const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                            uint32_t bw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                            if (a.bias_gu) {
                                const uint16_t* brow = a.bias_gu + (int64_t)grp.eid * a.ph[0].N + 2 * e0;
                                const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(brow));
                                const uint4 b1 = __ldg(reinterpret_cast<const uint4*>(brow + 8));
                                bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w;
                                bw[4] = b1.x; bw[5] = b1.y; bw[6] = b1.z; bw[7] = b1.w;
                            }
                            float hv[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                float gt = __uint_as_float(cw[j] << 16), up = __uint_as_float(cw[j] & 0xffff0000u);
                                if (a.bias_gu) {
                                    gt = bf16_round(__fadd_rn(gt, __uint_as_float(bw[j] << 16)));
                                    up = bf16_round(__fadd_rn(up, __uint_as_float(bw[j] & 0xffff0000u)));
                                }
                                hv[j] = glu_gpt_oss(gt, up);
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                hw[j] = (uint32_t)f32_to_bf16_bits(hv[2 * j]) | ((uint32_t)f32_to_bf16_bits(hv[2 * j + 1]) << 16);
                        }
                        h_s[c] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                    }
                    named_bar_sync(1, kFfnCW * 32);
#pragma unroll
                    for (int q = 0; q < AU; ++q) {
                        const int U = lane + 32 * q;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            const uint4 raw = (grp.valid && !poisoned && U < n_units) ? h_s[U * 4 + v] : make_uint4(0, 0, 0, 0);
                            put_pair(q, v, 0, raw.x);
                            put_pair(q, v, 1, raw.y);
                            put_pair(q, v, 2, raw.z);
                            put_pair(q, v, 3, raw.w);
                        }
                    }
                }
            }
            if (!poisoned && !mbar_wait_bounded(full_bar + stage, phase, abort_flag)) poisoned = true;
            const int n0 = tile * ph.rows_per_stage;
            const int rows = min(ph.rows_per_stage, ph.N - n0);
            if (!poisoned && grp.valid)
                consume_rows<FMT, SDT, AU, 1, RW, XF, kFfnCW, kXN>(
                    smem_u32(ring + (size_t)stage * a.slot_bytes), ph.rows_per_stage, rows, ph.row_bytes,
                    ph.scale_row_bytes, n_units, warp, lane, lane8, xr, dst + (int64_t)grp.row0 * ph.N + n0, ph.N, 1);
            // counted whether or not a wait gave up, so that every warp takes the same barriers (the status word
            // tells the caller that the results are void)
            if (grp.valid) done_in_group += rows;
            __syncwarp();
            if (!poisoned && lane == 0) mbar_arrive_relaxed(empty_bar + stage);
            if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
            if (++tile == ph.tiles_per_group) { tile = 0; ++g; }
        }
        publish();
    }

    // the last CTA to finish leaves the counters zeroed for the next launch
    named_bar_sync(1, kFfnCW * 32);
    if (threadIdx.x == 0) {
        __threadfence();
        const int old = atomicAdd(a.counters + a.G, 1);
        if (old == (int)gridDim.x - 1) {
            for (int i = 0; i <= a.G; ++i) a.counters[i] = 0;
        }
    }
    if (poisoned && threadIdx.x == 0 && a.status) atomicOr(a.status, GNF4B_ST_TIMEOUT);
}

}  // namespace gnf4b
