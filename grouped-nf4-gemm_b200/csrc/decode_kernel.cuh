// Decode kernel: every group has ONE activation row (RM = 1), or a few: then RM = 2 rows at a time, the
// weights streamed once per pair of rows and decoded once for both.
//
// The tight special case of the streaming path, taken when the host knows that no group has
// more than 16 rows, K <= 7168 (beyond 3072 one row per pass), N % 8 == 0 and the stack is laid out so that consecutive
// weight rows (and their scale rows) are contiguous and 16-byte aligned.  Then a work item
// (group, tile of R weight rows) is ONE contiguous span of packed bytes and ONE
// contiguous span of scale bytes, so a stage of the ring is filled by two bulk copies
// (TMA engine) issued by a single producer lane -- no per-row copies, no register-staged
// scale loads -- and the stage index is a closed-form function of the item index.
//
//   warp 16      producer: two lanes walk this CTA's contiguous item range and issue, per
//                item, cp.async.bulk(weights) + cp.async.bulk(raw scales) on full[stage]
//   warps 0..15  consumers: warp w owns rows w, w + 16, ... of the stage; a lane owns the
//                16-byte units lane, lane + 32, ... of a row, decodes through the
//                conflict-free byte-pair table, FMAs against the activation row it keeps in
//                registers as bf16 pairs, applies the block scale once per unit, warp-shuffle
//                reduces.  Sixteen warps because the loop is latency-bound, not issue-bound.
//                RM > 1: eight consumer warps (the RM activation rows need RM x 32 registers per
//                1024 columns); the table lookups of a unit are shared by the group's rows.
//
// Summation order per output element is the same as in stream_kernel.cuh, so both kernels
// give bit-identical results.
#pragma once

#include "common.cuh"
#include "stream_kernel.cuh"

namespace gnf4b {

// consumer warps: sixteen while a lane's share of the activation rows is small (one row, K <= 3072), fewer
// when it needs the registers (two rows: 8 warps; one row of up to 7168 columns: 6 warps)
// (two rows per pass: 12 warps while a row's activations fit 32 registers per row (AU <= 2: 128 registers per
// thread, no spills; the 8-warp form was issue-bound at 14 % warp occupancy), 8 warps at AU = 3)
__host__ __device__ constexpr int decode_consumer_warps(int rm, int au) {
    return au > 3 ? 6 : (rm == 1 ? 16 : (au <= 2 ? 12 : 8));
}
__host__ __device__ constexpr int decode_threads(int rm, int au) { return (decode_consumer_warps(rm, au) + 1) * 32; }
constexpr int kDMaxStages = 8;

struct DecodeArgs {
    GemmArgs g;
    int32_t rows_per_stage;     // R, a multiple of 4 or 8 (so that every scale span stays 16-byte aligned)
    int32_t tiles_per_group;    // ceil(N / R)
    int32_t row_bytes;          // K / 2
    int32_t scale_row_bytes;    // (K / block) * sizeof(scale)
    int32_t slot_bytes;         // ring slot, >= R * (row_bytes + scale_row_bytes), multiple of 128
    int32_t g_cache;
    int32_t stages;             // ring depth, 3..8, as many slots as shared memory holds
    int32_t items_per_cta;      // total_items / grid
    int32_t items_extra;        // total_items % grid: the first items_extra CTAs take one more
    int64_t total_items;        // G * row_chunks * tiles_per_group
    int32_t row_chunks;         // a group's rows are taken rows_per_pass at a time: ceil(max_rows / rows_per_pass)
    int32_t rows_per_pass;      // RM of the kernel instance
    int32_t compact;            // work list holds only (group, chunk) pairs that exist (prefix sum in shared memory)
};

__host__ __device__ inline size_t decode_smem_bytes(int slot_bytes, int stages, int g_cache) {
    return (size_t)kSTableBytes + (size_t)stages * slot_bytes + 256 + (size_t)(2 * g_cache + 1) * 4;
}

// One unit (16 packed bytes = 32 elements) against the activation row kept in registers as
// 16 bf16 pairs (widened on use: a bf16 is the top half of its fp32).  Same four partial
// sums and the same order as unit_dot_regs of the streaming kernel, so the bits agree.
__device__ __forceinline__ float2 ld_table(uint32_t addr) {
    // the pair table is written once before the consumers' barrier and never again, so this
    // load may be scheduled freely (no volatile, no memory clobber)
    float2 v;
    asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ void unit_lookup(const uint4 wv, uint32_t tab_lane, float2* p) {
    const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int b = 0; b < 4; ++b) p[i * 4 + b] = ld_table(tab_lane + prmt(words[i], 0u, 0x4404u | (b << 4)));
}

__device__ __forceinline__ float unit_fma_bf16(const float2* p, const uint32_t* a16) {
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t ab = a16[i * 4 + b];
            part[b] = fmaf(p[i * 4 + b].x, __uint_as_float(ab << 16), part[b]);
            part[b] = fmaf(p[i * 4 + b].y, __uint_as_float(ab & 0xffff0000u), part[b]);
        }
    }
    return (part[0] + part[1]) + (part[2] + part[3]);
}

__device__ __forceinline__ float unit_dot_bf16(const uint4 wv, const uint32_t* a16, uint32_t tab_lane) {
    float2 p[16];
    unit_lookup(wv, tab_lane, p);
    return unit_fma_bf16(p, a16);
}

template <int SDT>
__device__ __forceinline__ float ld_shared_scale(uint32_t row_addr, int idx) {
    if (SDT == GNF4B_S_F32) return ld_shared_f32(row_addr + idx * 4);
    if (SDT == GNF4B_S_BF16) {
        uint32_t h;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(h) : "r"(row_addr + idx * 2));
        return __uint_as_float(h << 16);
    }
    uint32_t e;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(e) : "r"(row_addr + idx));
    return __uint_as_float(e >= 2 ? (e - 1) << 23 : 0x00200000u << e);
}

struct DGroup {
    int32_t row0, eid, rows;
    bool valid;
};

// Rows [c * RM, c * RM + RM) of group g.  With row_chunks > 1 a group's rows are taken RM at a time:
// the work list is (group, row chunk, tile) with the tile fastest, so a CTA keeps one chunk's activation
// rows in registers for a run of tiles, and the group's weights are streamed once per chunk (the later
// passes mostly from L2).  Chunks that a group does not have are not in the list (see GroupWalk).
__device__ __forceinline__ DGroup decode_group(const DecodeArgs& a, int g, int c) {
    // a group changes once per N / R items, so its three ints come straight from global
    // memory (L1-cached) instead of a shared-memory copy that every thread would wait for
    const int32_t row0 = __ldg(a.g.off + g);
    const int32_t end = __ldg(a.g.off + g + 1);
    const int32_t eid = __ldg(a.g.eids + g);
    DGroup d;
    d.row0 = row0 + c * a.rows_per_pass;
    d.eid = eid;
    d.rows = min(end - d.row0, a.rows_per_pass);
    const bool bad_e = eid < 0 || eid >= a.g.E;
    const bool bad_o = end < row0 || row0 < 0 || end > a.g.T;
    d.valid = !bad_e && !bad_o && d.rows > 0;
    const bool pad = eid == GNF4B_PAD_EXPERT;        // padding group: skipped, not an error
    if (((bad_e && !pad) || bad_o) && end != row0 && c == 0 && a.g.status && (threadIdx.x & 31) == 0)
        atomicOr(a.g.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
    // a group with more rows than the caller's max_rows promised: the rows beyond are not visited
    if (d.valid && c == 0 && end - row0 > a.row_chunks * a.rows_per_pass && a.g.status && (threadIdx.x & 31) == 0)
        atomicOr(a.g.status, GNF4B_ST_BAD_OFFSETS);
    return d;
}

// Position in the list of (group, row chunk) pairs.  Plain mode: pair v is group v.
// Compact mode (groups taken in row chunks, or a group list that is mostly empty or padding): vb[g] = number of pairs before group g (a prefix sum in shared memory, groups that are
// empty or flagged have none), so the list holds only chunks that exist.
struct GroupWalk {
    int v, g, c;
};
__device__ __forceinline__ void walk_to(const DecodeArgs& a, const int32_t* vb, GroupWalk& w, int v) {
    w.v = v;
    if (!a.compact) {
        w.g = v;
        w.c = 0;
        return;
    }
    while (w.g + 1 < a.g.G && vb[w.g + 1] <= v) ++w.g;      // v only ever grows
    w.c = v - vb[w.g];
}

template <int FMT, int SDT, int AU, int RM>
__global__ void __launch_bounds__(decode_threads(RM, AU), 1) decode_gemv_kernel(const DecodeArgs a) {
    constexpr int kDConsumerWarps = decode_consumer_warps(RM, AU);
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* tab_raw = smem;
    uint8_t* ring = smem + kSTableBytes;
    uint8_t* tail = ring + (size_t)a.stages * a.slot_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kDMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kDMaxStages);
    int32_t* s_grp = reinterpret_cast<int32_t*>(tail + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kDConsumerWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    const int bid = (int)blockIdx.x;
    int64_t item_lo = (int64_t)bid * a.items_per_cta + min(bid, a.items_extra);
    int64_t item_hi = item_lo + a.items_per_cta + (bid < a.items_extra ? 1 : 0);
    const int32_t* vb = s_grp;
    if (a.compact) {
        // compact mode (row chunks, or far more groups than rows): build the prefix sum of the groups' chunk counts (one warp, ordered scan),
        // then cut the list of existing items evenly over the CTAs
        pdl_wait();
        if (warp == 0) {
            int32_t carry = 0;
            if (lane == 0) s_grp[0] = 0;
            for (int base = 0; base < a.g.G; base += 32) {
                const int gi = base + lane;
                int32_t n = 0;
                if (gi < a.g.G) {
                    const int32_t r0 = __ldg(a.g.off + gi), r1 = __ldg(a.g.off + gi + 1), e = __ldg(a.g.eids + gi);
                    const bool bad = e < 0 || e >= a.g.E || r1 < r0 || r0 < 0 || r1 > a.g.T;
                    const bool bad_off = r1 < r0 || r0 < 0 || r1 > a.g.T;
                    if (bad && r1 != r0 && (bad_off || e != GNF4B_PAD_EXPERT) && a.g.status && bid == 0)
                        atomicOr(a.g.status, bad_off ? GNF4B_ST_BAD_OFFSETS : GNF4B_ST_BAD_EXPERT);
                    n = bad ? 0 : min((r1 - r0 + a.rows_per_pass - 1) / a.rows_per_pass, a.row_chunks);
                }
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int32_t t = __shfl_up_sync(0xffffffffu, n, o);
                    if (lane >= o) n += t;
                }
                if (gi < a.g.G) s_grp[gi + 1] = carry + n;
                carry += __shfl_sync(0xffffffffu, n, 31);
            }
        }
        __syncthreads();
        const int64_t total = (int64_t)vb[a.g.G] * a.tiles_per_group;
        const int64_t per = total / gridDim.x, extra = total % gridDim.x;
        item_lo = (int64_t)bid * per + min((int64_t)bid, extra);
        item_hi = item_lo + per + (bid < extra ? 1 : 0);
    }
    const int R = a.rows_per_stage;
    GroupWalk w{0, 0, 0};
    walk_to(a, vb, w, (int)((uint32_t)item_lo / (uint32_t)a.tiles_per_group));
    int tile = (int)((uint32_t)item_lo - (uint32_t)w.v * (uint32_t)a.tiles_per_group);

    if (warp == kDConsumerWarps) {
        // ------------------------------------------------------------ producer (two lanes)
        // lane 0 copies the packed rows, lane 1 the scale rows of the same stage
        if (lane < 2) {
            pdl_wait();             // group tables (and, for the consumers, activations) may come from the previous kernel
            const int elt = (SDT == GNF4B_S_F32) ? 4 : (SDT == GNF4B_S_BF16 ? 2 : 1);
            const uint8_t* Sb = reinterpret_cast<const uint8_t*>(a.g.S);
            uint32_t stage = 0, phase = 0;
            int cur_v = -1;
            DGroup grp;
            grp.valid = false;
            bool ok = true;
            for (int64_t item = item_lo; item < item_hi && ok; ++item) {
                if (cur_v != w.v) { grp = decode_group(a, w.g, w.c); cur_v = w.v; }
                ok = mbar_wait_bounded(empty_bar + stage, phase ^ 1, abort_flag);
                if (!ok) break;
                if (grp.valid) {
                    uint8_t* st = ring + (size_t)stage * a.slot_bytes;
                    const int n0 = tile * R;
                    const int rows = min(R, (int)(a.g.N - n0));
                    const uint32_t wb = (uint32_t)rows * (uint32_t)a.row_bytes;
                    const uint32_t sb = (uint32_t)rows * (uint32_t)a.scale_row_bytes;
                    if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, wb + sb);
                    __syncwarp(0x3u);
                    const uint8_t* src = (lane == 0)
                        ? a.g.W + (int64_t)grp.eid * a.g.w_se + (int64_t)n0 * a.row_bytes
                        : Sb + ((int64_t)grp.eid * a.g.s_se + (int64_t)n0 * a.g.s_sn) * elt;
                    bulk_g2s(lane == 0 ? st : st + (size_t)R * a.row_bytes, src, lane == 0 ? wb : sb, full_bar + stage);
                } else if (lane == 0) {
                    mbar_arrive(full_bar + stage);      // empty group: the stage carries nothing
                }
                if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
                if (++tile == a.tiles_per_group) { tile = 0; walk_to(a, vb, w, w.v + 1); }
            }
            if (!ok && lane == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int n_units = a.row_bytes >> 4;
    int cur_v = -1;
    DGroup grp;
    grp.valid = false;
    grp.row0 = 0;
    grp.rows = 0;
    uint32_t a16[RM][AU * 16];     // the group's activation rows, bf16 pairs, units lane, lane + 32, ...

    auto load_a = [&](const DGroup& gr) {
#pragma unroll
        for (int m = 0; m < RM; ++m) {
            const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)(gr.row0 + m) * a.g.K * 2;
            const bool have = gr.valid && m < gr.rows;
#pragma unroll
            for (int q = 0; q < AU; ++q) {
                const int U = lane + 32 * q;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const uint4 raw = (have && U < n_units)
                                          ? __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)U * 64 + v * 16))
                                          : make_uint4(0, 0, 0, 0);
                    a16[m][q * 16 + v * 4 + 0] = raw.x;
                    a16[m][q * 16 + v * 4 + 1] = raw.y;
                    a16[m][q * 16 + v * 4 + 2] = raw.z;
                    a16[m][q * 16 + v * 4 + 3] = raw.w;
                }
            }
        }
    };
    {
        // pair table: tab[byte][slot], 32 slots of float2 per byte, all holding the same pair,
        // so a lane reading slot == its lane id never conflicts with another lane.  A half
        // warp writes one byte's 256-byte row per step with 16-byte stores.  Built before
        // pdl_wait(): it overlaps the tail of the previous kernel.
        const int half = lane >> 4, hl = lane & 15;
#pragma unroll 4
        for (int b = warp * 2 + half; b < 256; b += kDConsumerWarps * 2) {
            const float2 p = byte_pair<FMT>(b);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(smem_u32(tab_raw) + b * 256 + hl * 16),
                         "f"(p.x), "f"(p.y), "f"(p.x), "f"(p.y)
                         : "memory");
        }
    }
    pdl_wait();
    if (item_lo < item_hi) {
        grp = decode_group(a, w.g, w.c);
        cur_v = w.v;
    }
    load_a(grp);
    named_bar_sync(1, kDConsumerWarps * 32);

    const uint32_t tab_lane = smem_u32(tab_raw) + lane * 8;
    uint16_t* out_bf = reinterpret_cast<uint16_t*>(a.g.out);
    uint32_t stage = 0, phase = 0;
    bool poisoned = false;

    for (int64_t item = item_lo; item < item_hi; ++item) {
        if (cur_v != w.v) {
            grp = decode_group(a, w.g, w.c);
            cur_v = w.v;
            load_a(grp);
        }
        if (!poisoned && !mbar_wait_bounded(full_bar + stage, phase, abort_flag)) poisoned = true;
        if (!poisoned && grp.valid) {
            const uint32_t st = smem_u32(ring + (size_t)stage * a.slot_bytes);
            const int n0 = tile * R;
            const int rows = min(R, (int)(a.g.N - n0));
            for (int r = warp; r < rows; r += kDConsumerWarps) {
                const uint32_t wrow = st + (uint32_t)(r * a.row_bytes);
                const uint32_t srow = st + (uint32_t)(R * a.row_bytes + r * a.scale_row_bytes);
                float acc[RM];
#pragma unroll
                for (int m = 0; m < RM; ++m) acc[m] = 0.f;
#pragma unroll
                for (int q = 0; q < AU; ++q) {
                    const int u = lane + 32 * q;
                    if (u < n_units) {
                        const uint4 wv = ld_shared_u32x4(wrow + u * 16);
                        const float sc = ld_shared_scale<SDT>(srow, (FMT == GNF4B_FMT_NF4) ? (u >> 1) : u);
                        if (RM == 1) {
                            acc[0] += unit_dot_bf16(wv, &a16[0][q * 16], tab_lane) * sc;
                        } else {
                            // one table lookup per byte for all rows of the group; word by word to keep
                            // the live registers down; per row the same four chains and the same order
                            // as unit_fma_bf16
                            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                            float part[RM][4];
#pragma unroll
                            for (int m = 0; m < RM; ++m)
#pragma unroll
                                for (int b = 0; b < 4; ++b) part[m][b] = 0.f;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float2 p[4];
#pragma unroll
                                for (int b = 0; b < 4; ++b) p[b] = ld_table(tab_lane + prmt(words[i], 0u, 0x4404u | (b << 4)));
#pragma unroll
                                for (int m = 0; m < RM; ++m) {
#pragma unroll
                                    for (int b = 0; b < 4; ++b) {
                                        const uint32_t ab = a16[m][q * 16 + i * 4 + b];
                                        part[m][b] = fmaf(p[b].x, __uint_as_float(ab << 16), part[m][b]);
                                        part[m][b] = fmaf(p[b].y, __uint_as_float(ab & 0xffff0000u), part[m][b]);
                                    }
                                }
                            }
#pragma unroll
                            for (int m = 0; m < RM; ++m)
                                acc[m] += ((part[m][0] + part[m][1]) + (part[m][2] + part[m][3])) * sc;
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < RM; ++m) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
                    if (lane == 0 && m < grp.rows)
                        out_bf[(int64_t)(grp.row0 + m) * a.g.N + n0 + r] = f32_to_bf16_bits(acc[m]);
                }
            }
        }
        __syncwarp();
        if (!poisoned && lane == 0) mbar_arrive(empty_bar + stage);
        if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
        if (++tile == a.tiles_per_group) { tile = 0; walk_to(a, vb, w, w.v + 1); }
    }
    if (poisoned && threadIdx.x == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
}

}  // namespace gnf4b
