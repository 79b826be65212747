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
//   last warp      producer: two lanes walk this CTA's contiguous item range and issue, per
//                  item, cp.async.bulk(weights) + cp.async.bulk(raw scales) on full[stage]
//   warps 0..CW-1  consumers: warp w owns rows w, w + CW, ... of the stage, RW of them in flight at a
//                  time; a lane owns the 16-byte units lane, lane + 32, ... of a row, decodes through a
//                  conflict-free lookup table indexed by the packed byte, FMAs against the activation row
//                  it keeps in registers, applies the block scale once per unit, warp-shuffle reduces.
//
// What bounds it (measured on B200 with the consumer loop alone, weights already in shared memory): every
// element costs one table read of 4 bytes (fp32 codebook value) through the 128 B/clk shared-memory pipe, so
// NF4 tops out at about 23 weight rows of 2048 elements per microsecond and SM, 3.9 TB/s of packed bytes
// chip-wide, before HBM does.  MXFP4 values are exact in bf16: 2 bytes per element and the mixed-precision FMA
// take it to 5.5 TB/s.
//
// Summation order per output element is the same as in stream_kernel.cuh, so both kernels
// give bit-identical results.
#pragma once

#include "common.cuh"
#include "stream_kernel.cuh"

namespace gnf4b {

// consumer warps: sixteen while a lane's share of the activation rows is small (one row, K <= 3072), fewer
// when it needs the registers (one row of up to 7168 columns: 6 warps; two rows per pass: 12 warps while a
// row's activations fit 32 registers per row (AU <= 2), 8 warps at AU = 3)
__host__ __device__ constexpr int decode_consumer_warps(int rm, int au) {
    return au > 3 ? 6 : (rm == 1 ? 16 : (au <= 2 ? 12 : 8));
}
__host__ __device__ constexpr int decode_threads(int rm, int au) { return (decode_consumer_warps(rm, au) + 1) * 32; }
// Long rows (K > 3072), chained pairs: a weight row is shared by TWO warps -- the first takes the lower half of the
// row's 1024-element units and hands its per-lane partial sums to the second through shared memory, which goes on
// from them with the upper half, reduces and stores.  The per-lane order of additions is the one a single warp
// would use, so the bits do not change, but a warp holds only half of the activation row in registers: twelve
// consumer warps (six pairs, one row per pair and stage) instead of six.
constexpr int kDChainPairs = 6;
constexpr int kDChainWarps = 2 * kDChainPairs;
constexpr int kDChainRowsMax = 2 * kDChainPairs;                 // rows of a ring stage: one or two per pair
constexpr int kDChainPartialBytes = kDChainRowsMax * 32 * 4;     // per ring stage: one partial sum per lane and row
constexpr int kDMaxStages = 8;

// The lookup table sits at a FIXED address of the CTA's shared-memory window (dynamic shared memory
// starts below it: the kernel checks), so the address of a lookup is one PRMT -- (byte << 8) | lane * 8
// -- plus the load's immediate offset: two instructions per packed byte, no address arithmetic.
constexpr int kDTabAbs = 2048;

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
    int32_t tables_ready;       // group_offsets / expert_ids were NOT written by the kernel launched just before
    int32_t x_act;              // 0: x [T, K].  1 / 2: x is the gate_up output [T, 2K], SiLU-GLU / gpt-oss GLU applied on load
    int32_t h_bytes;            // x_act: shared memory behind the group prefix for the activated rows (rows_per_pass * K * 2)
};


// Dynamic shared memory: [slack up to kDTabAbs][table 64 KiB][ring][barriers, abort flag: 256 B][group prefix]
__host__ __device__ inline size_t decode_smem_bytes(int slot_bytes, int stages, int g_cache) {
    return (size_t)kDTabAbs + (size_t)kSTableBytes + (size_t)stages * slot_bytes + 256 + (size_t)(2 * g_cache + 1) * 4;
}

// (byte B of w) << 8 | lane8, with lane8 = lane * 8 < 256
template <int B>
__device__ __forceinline__ uint32_t tab_index(uint32_t w, uint32_t lane8) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(w), "r"(lane8), "n"(0x7604 | (B << 4)));
    return d;
}
__device__ __forceinline__ float2 ld_table(uint32_t idx) {
    // the pair table is written once before the consumers' barrier and never again, so this
    // load may be scheduled freely (no volatile, no memory clobber)
    float2 v;
    asm("ld.shared.v2.f32 {%0, %1}, [%2 + %3];" : "=f"(v.x), "=f"(v.y) : "r"(idx), "n"(kDTabAbs));
    return v;
}

__device__ __forceinline__ uint32_t ld_table_b32(uint32_t idx) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1 + %2];" : "=r"(v) : "r"(idx), "n"(kDTabAbs));
    return v;
}
// acc += w.lo * x.lo, then acc += w.hi * x.hi, w and x pairs of bf16: the mixed-precision FMA of sm_100 (bf16
// operands, fp32 addend and result, one rounding), i.e. exactly fmaf() on the widened values.
__device__ __forceinline__ void fma_bf16_pair(float& acc, uint32_t w, uint32_t x) {
    asm("{ .reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %1;\n\t"
        "mov.b32 {xl, xh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.bf16 %0, wh, xh, %0; }"
        : "+f"(acc)
        : "r"(w), "r"(x));
}

// One word (4 packed bytes = 8 elements) of a unit against RM activation rows.  part[m][b] is the partial
// sum of byte position b: the same four chains and the same order as unit_dot_regs of the streaming
// kernel, so the bits agree.
//   XF = 1: activations as fp32 bits (x[m][base + e], e = 0..7), table of float2 pairs.
//   XF = 0: activations as bf16 pairs (x[m][base + b] holds elements 2b, 2b + 1), widened on use -- a bf16 is
//           the top half of its fp32 --, table of float2 pairs.
//   XF = 2: codebooks whose values are exact in bf16 (MXFP4): table of bf16 pairs (4 bytes per packed byte: half
//           the shared-memory traffic of the float2 table), activations as bf16 pairs, mixed-precision FMA (no
//           widening instructions at all).  lane8 is then lane * 4.
template <int RM, int XF, int XN>
__device__ __forceinline__ void word_fma(uint32_t w, uint32_t lane8, const uint32_t (&x)[RM][XN], int base,
                                         float (&part)[RM][4]) {
    if (XF == 2) {
        uint32_t p[4];
        p[0] = ld_table_b32(tab_index<0>(w, lane8));
        p[1] = ld_table_b32(tab_index<1>(w, lane8));
        p[2] = ld_table_b32(tab_index<2>(w, lane8));
        p[3] = ld_table_b32(tab_index<3>(w, lane8));
#pragma unroll
        for (int m = 0; m < RM; ++m)
#pragma unroll
            for (int b = 0; b < 4; ++b) fma_bf16_pair(part[m][b], p[b], x[m][base + b]);
        return;
    }
    float2 p[4];
    p[0] = ld_table(tab_index<0>(w, lane8));
    p[1] = ld_table(tab_index<1>(w, lane8));
    p[2] = ld_table(tab_index<2>(w, lane8));
    p[3] = ld_table(tab_index<3>(w, lane8));
#pragma unroll
    for (int m = 0; m < RM; ++m) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float x0, x1;
            if (XF == 1) {
                x0 = __uint_as_float(x[m][base + 2 * b]);
                x1 = __uint_as_float(x[m][base + 2 * b + 1]);
            } else {
                const uint32_t ab = x[m][base + b];
                x0 = __uint_as_float(ab << 16);
                x1 = __uint_as_float(ab & 0xffff0000u);
            }
            part[m][b] = fmaf(p[b].x, x0, part[m][b]);
            part[m][b] = fmaf(p[b].y, x1, part[m][b]);
        }
    }
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

// The rows of one ring stage that belong to this warp (w, w + CW, ..., RW of them in flight at a time), each
// against the RM activation rows in xr: decode, FMA, block scale per unit, warp-shuffle reduce, one bf16 store per
// (activation row, weight row) by lane 0 at out0[m * out_stride + r] for m < m_valid.  `st` is the shared-window
// address of the stage: `rows` packed rows of row_bytes, then (from R * row_bytes on) their scale rows.
template <int FMT, int SDT, int AU, int RM, int RW, int XF, int CW, int XN>
__device__ __forceinline__ void consume_rows(uint32_t st, int R, int rows, int row_bytes, int scale_row_bytes, int n_units,
                                             int warp, int lane, uint32_t lane8, const uint32_t (&xr)[RM][XN],
                                             uint16_t* out0, int64_t out_stride, int m_valid) {
    for (int r = warp; r < rows; r += CW * RW) {
        // RW rows of the stage: r, r + CW, ...; one past the end repeats the last valid row (its result is not
        // stored)
        uint32_t wrow[RW], srow[RW];
        float acc[RW][RM];
#pragma unroll
        for (int j = 0; j < RW; ++j) {
            const int rj = min(r + j * CW, rows - 1);
            wrow[j] = st + (uint32_t)(rj * row_bytes);
            srow[j] = st + (uint32_t)(R * row_bytes + rj * scale_row_bytes);
#pragma unroll
            for (int m = 0; m < RM; ++m) acc[j][m] = 0.f;
        }
#pragma unroll
        for (int q = 0; q < AU; ++q) {
            const int u = lane + 32 * q;
            if (u < n_units) {
                constexpr int kPerUnit = XN / AU, kPerWord = kPerUnit / 4;
                uint4 wv[RW];
                float sc[RW];
                float part[RW][RM][4];
#pragma unroll
                for (int j = 0; j < RW; ++j) {
                    wv[j] = ld_shared_u32x4(wrow[j] + u * 16);
                    sc[j] = ld_shared_scale<SDT>(srow[j], (FMT == GNF4B_FMT_NF4) ? (u >> 1) : u);
#pragma unroll
                    for (int m = 0; m < RM; ++m)
#pragma unroll
                        for (int b = 0; b < 4; ++b) part[j][m][b] = 0.f;
                }
                // one table lookup per byte serves all activation rows of the pass; word by word and row by
                // row, so that few looked-up pairs are live at a time
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int j = 0; j < RW; ++j) {
                        const uint32_t word = i == 0 ? wv[j].x : i == 1 ? wv[j].y : i == 2 ? wv[j].z : wv[j].w;
                        word_fma<RM, XF, XN>(word, lane8, xr, q * kPerUnit + i * kPerWord, part[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < RW; ++j)
#pragma unroll
                    for (int m = 0; m < RM; ++m)
                        acc[j][m] += ((part[j][m][0] + part[j][m][1]) + (part[j][m][2] + part[j][m][3])) * sc[j];
            }
        }
#pragma unroll
        for (int j = 0; j < RW; ++j) {
#pragma unroll
            for (int m = 0; m < RM; ++m) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc[j][m] += __shfl_xor_sync(0xffffffffu, acc[j][m], o);
                if (lane == 0 && m < m_valid && r + j * CW < rows)
                    out0[(int64_t)m * out_stride + r + j * CW] = f32_to_bf16_bits(acc[j][m]);
            }
        }
    }
}

// Chained pairs (see kDChainPairs): the rows of one ring stage, row r by pair r % kDChainPairs.  Warp 2p is the
// first half of pair p (units q_base = 0 ..), warp 2p + 1 the second (units AU ..): it waits for part_bar (one arrival
// per first-half warp and ring pass) before it reads the partial sums.  AU = units per warp.  Returns false when
// that wait ran out.
template <int FMT, int SDT, int AU, int XF, int XN>
__device__ __forceinline__ bool consume_rows_chain(uint32_t st, int R, int rows, int row_bytes, int scale_row_bytes, int n_units,
                                                   int warp, int lane, uint32_t lane8, const uint32_t (&xr)[1][XN],
                                                   uint16_t* out0, float* partial, uint64_t* part_bar, uint32_t phase,
                                                   volatile int* abort_flag) {
    const int pair = warp >> 1, second = warp & 1;
    const int q_base = second * AU;
    if (second && !mbar_wait_bounded(part_bar, phase, abort_flag)) return false;
    for (int r = pair; r < rows; r += kDChainPairs) {
        const uint32_t wrow = st + (uint32_t)(r * row_bytes);
        const uint32_t srow = st + (uint32_t)(R * row_bytes + r * scale_row_bytes);
        float acc = second ? partial[r * 32 + lane] : 0.f;
#pragma unroll
        for (int q = 0; q < AU; ++q) {
            const int u = lane + 32 * (q + q_base);
            if (u < n_units) {
                constexpr int kPerUnit = XN / AU, kPerWord = kPerUnit / 4;
                const uint4 wv = ld_shared_u32x4(wrow + u * 16);
                const float sc = ld_shared_scale<SDT>(srow, (FMT == GNF4B_FMT_NF4) ? (u >> 1) : u);
                float part[1][4] = {{0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t word = i == 0 ? wv.x : i == 1 ? wv.y : i == 2 ? wv.z : wv.w;
                    word_fma<1, XF, XN>(word, lane8, xr, q * kPerUnit + i * kPerWord, part);
                }
                acc += ((part[0][0] + part[0][1]) + (part[0][2] + part[0][3])) * sc;
            }
        }
        if (!second) {
            partial[r * 32 + lane] = acc;
        } else {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) out0[r] = f32_to_bf16_bits(acc);
        }
    }
    if (!second) {
        __syncwarp();
        if (lane == 0) mbar_arrive(part_bar);        // release: this warp's partial sums of the stage are written
    }
    return true;
}

// The lookup table of word_fma, one 256-byte row per packed byte value, built by CW warps from instruction
// immediates (no constant memory).  XF < 2: 32 slots of float2, all holding the byte's pair of codebook values, so
// a lane reading slot == its lane id never conflicts with another lane; a half warp writes one row per step with
// 16-byte stores.  XF = 2: 32 slots of bf16 pairs in the first 128 bytes of the row.
template <int FMT, int XF, int CW>
__device__ __forceinline__ void build_lookup_table(int warp, int lane) {
    const float mine = code_value_imm<FMT>((uint32_t)lane & 15u);
    if (XF == 2) {
        for (int b = warp; b < 256; b += CW) {
            const float e0 = __shfl_sync(0xffffffffu, mine, (FMT == GNF4B_FMT_NF4) ? (b >> 4) : (b & 15));
            const float e1 = __shfl_sync(0xffffffffu, mine, (FMT == GNF4B_FMT_NF4) ? (b & 15) : (b >> 4));
            const uint32_t v = (__float_as_uint(e0) >> 16) | (__float_as_uint(e1) & 0xffff0000u);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"((uint32_t)kDTabAbs + b * 256 + lane * 4), "r"(v) : "memory");
        }
    } else {
        const int half = lane >> 4, hl = lane & 15;
#pragma unroll 4
        for (int b0 = warp * 2; b0 < 256; b0 += CW * 2) {
            const int b = b0 + half;
            const float e0 = __shfl_sync(0xffffffffu, mine, (FMT == GNF4B_FMT_NF4) ? (b >> 4) : (b & 15));
            const float e1 = __shfl_sync(0xffffffffu, mine, (FMT == GNF4B_FMT_NF4) ? (b & 15) : (b >> 4));
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"((uint32_t)kDTabAbs + b * 256 + hl * 16),
                         "f"(e0), "f"(e1), "f"(e0), "f"(e1)
                         : "memory");
        }
    }
}

// Eight consecutive activations (columns k0 .. k0 + 7, bf16 pairs in four words) of a row that holds the gate_up
// output: act 1 = SiLU(gate) * up with gate = columns [0, K), up = [K, 2K) (the arithmetic of silu_glu_kernel);
// act 2 = the gpt-oss form on interleaved columns (gate 2k, up 2k + 1; glu_gpt_oss_kernel without bias).
__device__ __forceinline__ uint4 load_glu8(int act, const uint8_t* xrow, int k0, int64_t K) {
    uint32_t ow[4];
    if (act == 1) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)k0 * 2));
        const uint4 uv = __ldg(reinterpret_cast<const uint4*>(xrow + (K + k0) * 2));
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
            ow[j] = (uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g0), u0)) |
                    ((uint32_t)f32_to_bf16_bits(__fmul_rn(silu_f32(g1), u1)) << 16);
        }
    } else {
        const uint4 p0 = __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)k0 * 4));
        const uint4 p1 = __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)k0 * 4 + 16));
        const uint32_t pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t a0 = pw[2 * j], a1 = pw[2 * j + 1];
            ow[j] = (uint32_t)f32_to_bf16_bits(glu_gpt_oss(__uint_as_float(a0 << 16), __uint_as_float(a0 & 0xffff0000u))) |
                    ((uint32_t)f32_to_bf16_bits(glu_gpt_oss(__uint_as_float(a1 << 16), __uint_as_float(a1 & 0xffff0000u))) << 16);
        }
    }
    return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

struct DGroup {
    int32_t row0, eid, rows;
    bool valid;
};

// Rows [c * RM, c * RM + RM) of group g.  With row_chunks > 1 a group's rows are taken RM at a time:
// the work list is (group, row chunk, tile) with the tile fastest, so a CTA keeps one chunk's activation
// rows in registers for a run of tiles, and the group's weights are streamed once per chunk (the later
// passes mostly from L2).  Chunks that a group does not have are not in the list (see GroupWalk).
struct DGroupRaw {
    int32_t row0, end, eid;
};
// a group changes once per N / R items, so its three ints come straight from global memory (L1-cached) instead
// of a shared-memory copy that every thread would wait for
__device__ __forceinline__ DGroupRaw decode_group_load(const DecodeArgs& a, int g) {
    DGroupRaw r;
    r.row0 = __ldg(a.g.off + g);
    r.end = __ldg(a.g.off + g + 1);
    r.eid = __ldg(a.g.eids + g);
    return r;
}
__device__ __forceinline__ DGroup decode_group_check(const DecodeArgs& a, const DGroupRaw& r, int c) {
    const int32_t row0 = r.row0, end = r.end, eid = r.eid;
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
__device__ __forceinline__ DGroup decode_group(const DecodeArgs& a, int g, int c) {
    return decode_group_check(a, decode_group_load(a, g), c);
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

// FMT, SDT: weight format and scale dtype.  AU: 16-byte units of a row per lane (K <= AU * 1024).
// RM: activation rows per pass.  RW: weight rows of a stage that a warp works on at the same time (two
// independent streams of lookups and FMAs hide the table-read latency that one leaves exposed).  XF: form of the
// activations in registers and of the lookup table (see word_fma).
// Compact mode: the prefix sum of the groups' chunk counts in shared memory (s_grp[g + 1] = chunks of groups 0..g).
// Every thread fetches the tables of its groups (one memory round trip for the whole list, not one per 32 groups),
// then one warp turns the counts into the prefix sum in place.  Out of line: it runs once, before the kernel's
// register-heavy part, and must not weigh on that part's register allocation.
// When the tables may have been written by the kernel launched just before, that kernel has to be waited for first
// of all; the lookup table, which depends on nothing, is then built here before the wait (and not again later).
// (Arguments by value: a reference to the kernel's parameter block would move the whole block to local memory.)
template <int FMT, int XF, int CW>
__device__ __noinline__ void decode_compact_scan(const int32_t* __restrict__ off, const int32_t* __restrict__ eids, int32_t G,
                                                 int32_t E, int64_t T, int32_t* status, int32_t rows_per_pass,
                                                 int32_t row_chunks, int32_t tables_ready, int32_t* s_grp) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, bid = (int)blockIdx.x;
    if (!tables_ready) {
        if (warp < CW) build_lookup_table<FMT, XF, CW>(warp, lane);
        pdl_wait();
    }
    for (int gi = threadIdx.x; gi < G; gi += blockDim.x) {
        const int32_t r0 = __ldg(off + gi), r1 = __ldg(off + gi + 1), e = __ldg(eids + gi);
        const bool bad = e < 0 || e >= E || r1 < r0 || r0 < 0 || r1 > T;
        const bool bad_off = r1 < r0 || r0 < 0 || r1 > T;
        if (bad && r1 != r0 && (bad_off || e != GNF4B_PAD_EXPERT) && status && bid == 0)
            atomicOr(status, bad_off ? GNF4B_ST_BAD_OFFSETS : GNF4B_ST_BAD_EXPERT);
        s_grp[gi + 1] = bad ? 0 : min((r1 - r0 + rows_per_pass - 1) / rows_per_pass, row_chunks);
    }
    __syncthreads();
    if (warp == 0) {
        int32_t carry = 0;
        if (lane == 0) s_grp[0] = 0;
        for (int base = 0; base < G; base += 32) {
            const int gi = base + lane;
            int32_t n = gi < G ? s_grp[gi + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t t = __shfl_up_sync(0xffffffffu, n, o);
                if (lane >= o) n += t;
            }
            if (gi < G) s_grp[gi + 1] = carry + n;
            carry += __shfl_sync(0xffffffffu, n, 31);
        }
    }
}

// XA = 1: the instance that can apply the FFN's activation while it loads its activation rows (DecodeArgs.x_act);
// a separate instance so that the plain one keeps its registers.
// CH = 1: long rows as chained pairs; AU is then the units per WARP (half of the row's), RM = RW = 1.
template <int FMT, int SDT, int AU, int RM, int RW, int XF, int XA = 0, int CH = 0>
__global__ void __launch_bounds__(CH ? (kDChainWarps + 1) * 32 : decode_threads(RM, AU), 1) decode_gemv_kernel(const DecodeArgs a) {
    constexpr int kCW = CH ? kDChainWarps : decode_consumer_warps(RM, AU);
    constexpr int kXN = XF == 1 ? AU * 32 : AU * 16;     // registers per activation row
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* tab_raw = smem + ((uint32_t)kDTabAbs - smem_base);     // window address kDTabAbs
    uint8_t* ring = tab_raw + kSTableBytes;
    uint8_t* tail = ring + (size_t)a.stages * a.slot_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kDMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kDMaxStages);
    uint64_t* part_bar = empty_bar + kDMaxStages + 1;       // CH: "first halves written", one per ring stage
    int32_t* s_grp = reinterpret_cast<int32_t*>(tail + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    EPT(60);
    pdl_launch_dependents();
    if (smem_base > (uint32_t)kDTabAbs) {
        // dynamic shared memory starts beyond the table's fixed address (never seen): nothing is computed
        if (threadIdx.x == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kCW);
            if (CH) mbar_init(part_bar + s, kDChainPairs);
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
        decode_compact_scan<FMT, XF, kCW>(a.g.off, a.g.eids, a.g.G, a.g.E, a.g.T, a.g.status, a.rows_per_pass, a.row_chunks,
                                          a.tables_ready, s_grp);
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

    if (warp == kCW) {
        // ------------------------------------------------------------ producer (two lanes)
        // lane 0 copies the packed rows, lane 1 the scale rows of the same stage
        if (lane < 2) {
            // The group tables may have been written by the kernel launched just before this one: wait for
            // it, unless the caller said they were not.  The packed weights never are, so with ready tables
            // the ring fills while the previous kernel of the stream is still running.
            if (!a.tables_ready) pdl_wait();
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
    uint32_t xr[RM][kXN];     // the group's activation rows: units lane, lane + 32, ... (fp32 bits or bf16 pairs)

    // XA: the rows of x are gate_up outputs (2K wide).  The consumer warps compute the group's activated rows ONCE,
    // together, into shared memory (every warp needs the whole row: computed per warp, the activation would be done
    // kCW times over), then each takes its lanes' share from there.  All consumer warps walk the same items, so
    // they reach every group change together and the two barriers are safe.
    const int64_t x_pitch = (XA ? 2 : 1) * a.g.K * 2;
    uint4* h_s = reinterpret_cast<uint4*>(tail + 256 + (((size_t)(2 * a.g_cache + 1) * 4 + 15) & ~(size_t)15));
    auto load_a = [&](const DGroup& gr) {
        if (XA) {
            named_bar_sync(2, kCW * 32);              // the previous group's rows have been taken by every warp
            const int per_row = (int)(a.g.K >> 3);
#pragma unroll 1
            for (int m = 0; m < RM; ++m) {
                if (!(gr.valid && m < gr.rows)) break;
                const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)(gr.row0 + m) * x_pitch;
#pragma unroll 1
                for (int c8 = (int)threadIdx.x; c8 < per_row; c8 += kCW * 32)
                    h_s[m * per_row + c8] = load_glu8(a.x_act, xrow, c8 * 8, a.g.K);
            }
            named_bar_sync(3, kCW * 32);
        }
#pragma unroll
        for (int m = 0; m < RM; ++m) {
            const uint8_t* xrow = XA ? reinterpret_cast<const uint8_t*>(h_s) + (size_t)m * a.g.K * 2
                                     : reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)(gr.row0 + m) * x_pitch;
            const bool have = gr.valid && m < gr.rows;
#pragma unroll
            for (int q = 0; q < AU; ++q) {
                const int U = lane + 32 * (q + (CH ? (warp & 1) * AU : 0));
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const uint4 raw = !(have && U < n_units) ? make_uint4(0, 0, 0, 0)
                                      : XA == 0 ? __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)U * 64 + v * 16))
                                                : *reinterpret_cast<const uint4*>(xrow + (size_t)U * 64 + v * 16);
                    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (XF == 1) {
                            xr[m][q * 32 + v * 8 + 2 * j] = rw[j] << 16;
                            xr[m][q * 32 + v * 8 + 2 * j + 1] = rw[j] & 0xffff0000u;
                        } else {
                            xr[m][q * 16 + v * 4 + j] = rw[j];
                        }
                    }
                }
            }
        }
    };
    // Before waiting for the previous kernel: with ready tables, the loads of this CTA's first group (three ints
    // that the activation row's address depends on) go out now and are used after the table is built.
    const bool early = a.tables_ready != 0 && item_lo < item_hi;
    DGroupRaw raw0 = {0, 0, 0};
    if (early) raw0 = decode_group_load(a, w.g);
    // built before pdl_wait(): it overlaps the tail of the previous kernel
    if (!(a.compact && !a.tables_ready)) build_lookup_table<FMT, XF, kCW>(warp, lane);
    if (early) {
        grp = decode_group_check(a, raw0, w.c);
        cur_v = w.v;
        if (warp == 0 && grp.valid) {       // a hint that brings the activation rows' lines into L2
            const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)grp.row0 * x_pitch;
            const int64_t bytes = (int64_t)min(grp.rows, RM) * x_pitch;
            for (int64_t o = (int64_t)lane * 128; o < bytes; o += 32 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(xrow + o));
        }
    }
    EPT(61);
    pdl_wait();
    EPT(62);
    if (!early && item_lo < item_hi) {
        grp = decode_group(a, w.g, w.c);
        cur_v = w.v;
    }
    load_a(grp);
    named_bar_sync(1, kCW * 32);

    const uint32_t lane8 = (uint32_t)lane * (XF == 2 ? 4u : 8u);     // slot of this lane in a table row
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
        if constexpr (CH != 0) {
            if (!poisoned) {
                // (every stage, also of an empty group: the pairs' hand-over barrier counts ring passes)
                const int n0 = tile * R;
                float* partial = reinterpret_cast<float*>(h_s) + (size_t)stage * (kDChainPartialBytes / 4);
                if (!consume_rows_chain<FMT, SDT, AU, XF, kXN>(
                        smem_u32(ring + (size_t)stage * a.slot_bytes), R, grp.valid ? min(R, (int)(a.g.N - n0)) : 0, a.row_bytes,
                        a.scale_row_bytes, n_units, warp, lane, lane8, xr, out_bf + (int64_t)grp.row0 * a.g.N + n0, partial,
                        part_bar + stage, phase, abort_flag))
                    poisoned = true;
            }
        } else if (!poisoned && grp.valid) {     // NOLINT(readability-misleading-indentation): the plain instances
            const int n0 = tile * R;
            consume_rows<FMT, SDT, AU, RM, RW, XF, kCW, kXN>(
                smem_u32(ring + (size_t)stage * a.slot_bytes), R, min(R, (int)(a.g.N - n0)), a.row_bytes,
                a.scale_row_bytes, n_units, warp, lane, lane8, xr, out_bf + (int64_t)grp.row0 * a.g.N + n0, a.g.N, grp.rows);
        }
        __syncwarp();
        if (!poisoned && lane == 0) mbar_arrive_relaxed(empty_bar + stage);
        if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
        if (++tile == a.tiles_per_group) { tile = 0; walk_to(a, vb, w, w.v + 1); }
    }
    if (poisoned && threadIdx.x == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
    EPT(63);
}

}  // namespace gnf4b
