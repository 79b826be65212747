// Streaming (CUDA-core) grouped GEMM for decode-sized groups.
//
// One persistent CTA per SM.  Warps 8..11 are producers: they walk this CTA's contiguous
// range of work items and stream each item's packed rows from HBM into an 8-stage
// shared-memory ring with 1-D bulk copies (TMA engine) counted on mbarriers, and stage
// the block scales beside them.  Stage number q belongs to producer warp q % 4, so four
// global-memory latencies of the scale loads are in flight at once.  Warps 0..7 are consumers: consumer w owns weight row
// (tile*8 + w); its lanes split the row into 16-byte units (32 elements), decode each
// byte through a bank-conflict-free 256-entry pair table, multiply-accumulate in fp32
// against the activation rows, apply the block scale once per unit, and reduce with
// warp shuffles.  Split-K partials meet in a workspace and are summed in split order by
// the last CTA to arrive, so results are deterministic.
//
// Work item = (group, 8-row tile of N, K split).  Groups, their row ranges and expert ids
// are read on the device from group_offsets / expert_ids: there is no host-built tile
// table.  Stands in for _gemv_nf4_grouped, _gemv_nf4_grouped_splitk and
// _gemv_mxfp4_grouped (kernel/nf4_grouped.py:465-574, kernel/mxfp4_grouped.py:100-131)
// and is correct for any group size (larger groups loop over row chunks).
#pragma once

#include "common.cuh"

namespace gnf4b {

constexpr int kSConsumerWarps = 8;
constexpr int kSProducerWarps = 4;
constexpr int kSThreads = (kSConsumerWarps + kSProducerWarps) * 32;
constexpr int kSTileN = 8;              // weight rows per stage (one per consumer warp)
constexpr int kSRowPitch = 1024;        // bytes of one row slot in a stage
constexpr int kSStages = 8;
constexpr int kSScaleSlots = 64;        // fp32 scale slots per row per stage (MXFP4: 2048/32)
constexpr int kSStageBytes = kSTileN * kSRowPitch + kSTileN * kSScaleSlots * 4;
constexpr int kSTableBytes = 256 * 32 * 8;   // pair table: [byte][lane] float2
constexpr int kSRowsMax = 4;            // activation rows accumulated at once

struct StreamArgs {
    GemmArgs g;
    int32_t n_tiles;        // ceil(N / 8)
    int32_t chunk_bytes;    // packed bytes of one K chunk per row (<= 1024, multiple of 16)
    int32_t n_chunks;       // ceil(K/2 / chunk_bytes)
    int32_t chunks_per_split;
    int32_t rows_cap;       // activation rows staged at once (1..kSRowsMax)
    int32_t a_units_pad;    // 16-byte units of one activation row, rounded up to 32
    int32_t w_align;        // 16: bulk copies; 8 / 4 / 1: plain loads of that width
    int64_t total_items;
};

__host__ __device__ inline size_t stream_smem_bytes(int rows_cap, int a_units_pad) {
    return (size_t)kSTableBytes + (size_t)kSStages * kSStageBytes +
           (size_t)rows_cap * a_units_pad * 128 + 256;
}

// Decoded item shared by producer and consumers (they must agree exactly).
struct StreamItem {
    int32_t g, tile, split, row0, rows, eid, c0, c1;
    bool valid;
};

__device__ __forceinline__ StreamItem stream_decode_item(const StreamArgs& a, int64_t item) {
    StreamItem it;
    const int32_t S = a.g.split_k;
    const int64_t per_group = (int64_t)a.n_tiles * S;
    it.g = (int32_t)(item / per_group);
    const int32_t rem = (int32_t)(item - (int64_t)it.g * per_group);
    it.tile = rem / S;
    it.split = rem - it.tile * S;
    it.row0 = __ldg(a.g.off + it.g);
    it.rows = __ldg(a.g.off + it.g + 1) - it.row0;
    it.eid = __ldg(a.g.eids + it.g);
    it.c0 = it.split * a.chunks_per_split;
    it.c1 = min(a.n_chunks, it.c0 + a.chunks_per_split);
    const bool bad_e = it.eid < 0 || it.eid >= a.g.E;
    const bool bad_o = it.rows < 0 || it.row0 < 0 || (int64_t)it.row0 + it.rows > a.g.T;
    it.valid = !bad_e && !bad_o && it.rows > 0;
    if ((bad_e || bad_o) && a.g.status && it.rows != 0)
        atomicOr(a.g.status, bad_e ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
    return it;
}

template <int VEC>
__device__ __forceinline__ void plain_copy_row(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
    if (VEC == 8) {
        for (int i = lane * 8; i < bytes; i += 256)
            *reinterpret_cast<uint2*>(dst + i) = __ldg(reinterpret_cast<const uint2*>(src + i));
    } else if (VEC == 4) {
        for (int i = lane * 4; i < bytes; i += 128)
            *reinterpret_cast<uint32_t*>(dst + i) = __ldg(reinterpret_cast<const uint32_t*>(src + i));
    } else {
        for (int i = lane; i < bytes; i += 32) dst[i] = __ldg(src + i);
    }
}

// Activation element k of staged row m lives at float index
//   ((m*UPG + U/32)*8 + f)*32 + U%32)*4 + c   with U = k/32, f = (k%32)/4, c = k%4
// so that the 32 lanes of a warp, each reading float4 number f of its own unit,
// touch 32 consecutive 16-byte words.
__device__ __forceinline__ uint32_t a_f4_offset(int m, int upg, int U, int f) {
    return (uint32_t)((((m * upg + (U >> 5)) * 8 + f) * 32 + (U & 31)) * 16);
}

__device__ __forceinline__ void cvt8(const uint4 raw, int x_dtype, float* o) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (x_dtype == GNF4B_X_BF16) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            const float2 f = __half22float2(h);
            o[2 * i] = f.x;
            o[2 * i + 1] = f.y;
        }
    }
}

// FMT: weight format.  SDT: scale dtype.  AU: activation units (of 32 elements) a lane
// keeps in registers for single-row groups (0 = always read activations from shared memory).
template <int FMT, int SDT, int AU>
__global__ void __launch_bounds__(kSThreads, 1) stream_gemm_kernel(const StreamArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* tab_raw = smem;
    uint8_t* ring = smem + kSTableBytes;
    float* a_smem = reinterpret_cast<float*>(ring + kSStages * kSStageBytes);
    uint8_t* tail = reinterpret_cast<uint8_t*>(a_smem) + (size_t)a.rows_cap * a.a_units_pad * 128;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kSStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kSStages);
    volatile int* last_flag = abort_flag + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSStages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kSConsumerWarps);
        }
        *abort_flag = 0;
        *last_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    const int64_t item_lo = a.total_items * blockIdx.x / gridDim.x;
    const int64_t item_hi = a.total_items * (blockIdx.x + 1) / gridDim.x;
    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;
    const int scales_per_chunk = a.chunk_bytes * 2 / (int)scale_blk;
    const int64_t row_bytes = a.g.K / 2;

    if (warp >= kSConsumerWarps) {
        // ------------------------------------------------------------ producers
        const uint32_t pw = (uint32_t)(warp - kSConsumerWarps);
        uint32_t stage = 0, phase = 0, seq = 0;
        bool poisoned = false;
        for (int64_t item = item_lo; item < item_hi; ++item) {
            const StreamItem it = stream_decode_item(a, item);
            if (!it.valid) continue;
            const int row_chunks = (it.rows + a.rows_cap - 1) / a.rows_cap;
            const uint8_t* w_e = a.g.W + (int64_t)it.eid * a.g.w_se;
            const int n0 = it.tile * kSTileN;
            const int n_valid = min(kSTileN, (int)(a.g.N - n0));
            for (int rc = 0; rc < row_chunks; ++rc) {
                for (int c = it.c0; c < it.c1; ++c) {
                    const bool mine = (seq++ % kSProducerWarps) == pw;
                    if (mine && !poisoned && !mbar_wait_bounded(empty_bar + stage, phase ^ 1, abort_flag))
                        poisoned = true;
                    if (mine && !poisoned) {
                        uint8_t* st = ring + stage * kSStageBytes;
                        float* st_sc = reinterpret_cast<float*>(st + kSTileN * kSRowPitch);
                        const int64_t boff = (int64_t)c * a.chunk_bytes;
                        const int cbytes = (int)min((int64_t)a.chunk_bytes, row_bytes - boff);
                        // block scales of this chunk, widened to fp32
                        const int nsc = cbytes * 2 / (int)scale_blk;
                        for (int i = lane; i < n_valid * scales_per_chunk; i += 32) {
                            const int r = i / scales_per_chunk, j = i - r * scales_per_chunk;
                            if (j < nsc)
                                st_sc[r * kSScaleSlots + j] = load_scale<SDT>(
                                    a.g.S, (int64_t)it.eid * a.g.s_se + (int64_t)(n0 + r) * a.g.s_sn +
                                               (int64_t)c * scales_per_chunk + j);
                        }
                        if (a.w_align == 16) {
                            __syncwarp();
                            if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, (uint32_t)(n_valid * cbytes));
                            __syncwarp();
                            if (lane < n_valid)
                                bulk_g2s(st + lane * kSRowPitch,
                                         w_e + (int64_t)(n0 + lane) * a.g.w_sn + boff, (uint32_t)cbytes,
                                         full_bar + stage);
                        } else {
                            for (int r = 0; r < n_valid; ++r) {
                                const uint8_t* src = w_e + (int64_t)(n0 + r) * a.g.w_sn + boff;
                                if (a.w_align == 8) plain_copy_row<8>(st + r * kSRowPitch, src, cbytes, lane);
                                else if (a.w_align == 4) plain_copy_row<4>(st + r * kSRowPitch, src, cbytes, lane);
                                else plain_copy_row<1>(st + r * kSRowPitch, src, cbytes, lane);
                            }
                            __syncwarp();
                            if (lane == 0) mbar_arrive(full_bar + stage);
                        }
                    }
                    if (++stage == kSStages) { stage = 0; phase ^= 1; }
                }
            }
        }
        if (poisoned && lane == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
        return;
    }

    // ---------------------------------------------------------------- consumers
    // pair table: tab[byte][slot] for slot 0..31, every slot holds the same float2, so a
    // lane reading slot == its lane id never conflicts with another lane.
    {
        float2* tab = reinterpret_cast<float2*>(tab_raw);
        for (int i = threadIdx.x; i < 256 * 32; i += kSConsumerWarps * 32) tab[i] = byte_pair<FMT>(i >> 5);
    }
    named_bar_sync(1, kSConsumerWarps * 32);

    const uint32_t tab_lane = smem_u32(tab_raw) + lane * 8;
    const uint32_t a_base = smem_u32(a_smem);
    const int upg = a.a_units_pad >> 5;
    const int units_per_chunk = a.chunk_bytes >> 4;
    const int64_t n_units = a.g.K / 32;
    const bool bf16_out_direct = a.g.split_k == 1;
    uint16_t* out_bf = reinterpret_cast<uint16_t*>(a.g.out);

    uint32_t stage = 0, phase = 0;
    bool poisoned = false;
    int staged_g = -1, staged_rc = -1;   // what a_smem currently holds
    int reg_g = -1;                      // which group's row the a registers hold
    float a_reg[AU > 0 ? AU * 32 : 1];

    for (int64_t item = item_lo; item < item_hi; ++item) {
        const StreamItem it = stream_decode_item(a, item);
        if (!it.valid) continue;
        const int n = it.tile * kSTileN + warp;
        const bool active = n < a.g.N;
        const int row_chunks = (it.rows + a.rows_cap - 1) / a.rows_cap;
        const bool fast = AU > 0 && it.rows == 1 && a.chunk_bytes == kSRowPitch && n_units <= AU * 32;

        for (int rc = 0; rc < row_chunks; ++rc) {
            const int r_lo = rc * a.rows_cap;
            const int rm = min(a.rows_cap, it.rows - r_lo);
            float acc[kSRowsMax] = {0.f, 0.f, 0.f, 0.f};

            if (fast) {
                if (AU > 0 && reg_g != it.g) {
                    const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)it.row0 * a.g.K * 2;
#pragma unroll
                    for (int q = 0; q < AU; ++q) {
                        const int U = lane + 32 * q;
                        if (U < n_units) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)U * 64 + v * 16));
                                cvt8(raw, a.g.x_dtype, &a_reg[q * 32 + v * 8]);
                            }
                        } else {
#pragma unroll
                            for (int v = 0; v < 32; ++v) a_reg[q * 32 + v] = 0.f;
                        }
                    }
                    reg_g = it.g;
                }
            } else if (staged_g != it.g || staged_rc != rc) {
                // all consumers finished with the previous rows before they are replaced
                named_bar_sync(1, kSConsumerWarps * 32);
                const uint8_t* xb = reinterpret_cast<const uint8_t*>(a.g.x);
                const int per_row = upg * 8;   // (unit group, float4) pairs per row
                for (int w = warp; w < rm * per_row; w += kSConsumerWarps) {
                    const int m = w / per_row, r2 = w - m * per_row;
                    const int ug = r2 >> 3, f = r2 & 7;
                    const int U = ug * 32 + lane;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (U < n_units) {
                        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(
                            xb + ((int64_t)(it.row0 + r_lo + m) * a.g.K + (int64_t)U * 32 + f * 4) * 2));
                        if (a.g.x_dtype == GNF4B_X_BF16) {
                            v.x = __uint_as_float(raw.x << 16);
                            v.y = __uint_as_float(raw.x & 0xffff0000u);
                            v.z = __uint_as_float(raw.y << 16);
                            v.w = __uint_as_float(raw.y & 0xffff0000u);
                        } else {
                            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                            v = make_float4(f0.x, f0.y, f1.x, f1.y);
                        }
                    }
                    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a_base + a_f4_offset(m, upg, U, f)),
                                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                                 : "memory");
                }
                named_bar_sync(1, kSConsumerWarps * 32);
                staged_g = it.g;
                staged_rc = rc;
            }

            for (int c = it.c0; c < it.c1; ++c) {
                if (!poisoned && !mbar_wait_bounded(full_bar + stage, phase, abort_flag)) poisoned = true;
                if (!poisoned && active) {
                    const uint32_t st = smem_u32(ring + stage * kSStageBytes);
                    const uint32_t wrow = st + warp * kSRowPitch;
                    const uint32_t srow = st + kSTileN * kSRowPitch + warp * kSScaleSlots * 4;
                    const int cbytes = (int)min((int64_t)a.chunk_bytes, row_bytes - (int64_t)c * a.chunk_bytes);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int u = lane + 32 * j;
                        if (u * 16 < cbytes) {
                            const uint4 wv = ld_shared_u32x4(wrow + u * 16);
                            const float sc = ld_shared_f32(srow + ((FMT == GNF4B_FMT_NF4) ? (u >> 1) : u) * 4);
                            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                            if (fast) {
                                // q is a compile-time index only when the chunk loop is short;
                                // the switch keeps a_reg in registers.
                                float part = 0.f;
                                const int q = c * 2 + j;   // global 32-lane unit group of this lane's unit
#pragma unroll
                                for (int qq = 0; qq < (AU > 0 ? AU : 1); ++qq) {
                                    if (AU > 0 && qq == q) {
#pragma unroll
                                        for (int i = 0; i < 4; ++i) {
#pragma unroll
                                            for (int b = 0; b < 4; ++b) {
                                                const uint32_t off = prmt(words[i], 0u, 0x4404u | (b << 4));  // byte b -> bits 8..15
                                                const float2 p = ld_shared_f32x2(tab_lane + off);
                                                part = fmaf(p.x, a_reg[qq * 32 + i * 8 + b * 2], part);
                                                part = fmaf(p.y, a_reg[qq * 32 + i * 8 + b * 2 + 1], part);
                                            }
                                        }
                                    }
                                }
                                acc[0] += part * sc;
                            } else {
                                const int U = c * units_per_chunk + u;
                                float part[kSRowsMax] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    float wf[8];
#pragma unroll
                                    for (int b = 0; b < 4; ++b) {
                                        const uint32_t off = prmt(words[i], 0u, 0x4404u | (b << 4));  // byte b -> bits 8..15
                                        const float2 p = ld_shared_f32x2(tab_lane + off);
                                        wf[2 * b] = p.x;
                                        wf[2 * b + 1] = p.y;
                                    }
#pragma unroll
                                    for (int m = 0; m < kSRowsMax; ++m) {
                                        if (m < rm) {
                                            const float4 lo = ld_shared_f32x4(a_base + a_f4_offset(m, upg, U, 2 * i));
                                            const float4 hi = ld_shared_f32x4(a_base + a_f4_offset(m, upg, U, 2 * i + 1));
                                            float s = part[m];
                                            s = fmaf(wf[0], lo.x, s);
                                            s = fmaf(wf[1], lo.y, s);
                                            s = fmaf(wf[2], lo.z, s);
                                            s = fmaf(wf[3], lo.w, s);
                                            s = fmaf(wf[4], hi.x, s);
                                            s = fmaf(wf[5], hi.y, s);
                                            s = fmaf(wf[6], hi.z, s);
                                            s = fmaf(wf[7], hi.w, s);
                                            part[m] = s;
                                        }
                                    }
                                }
#pragma unroll
                                for (int m = 0; m < kSRowsMax; ++m)
                                    acc[m] += part[m] * sc;
                            }
                        }
                    }
                }
                __syncwarp();
                if (!poisoned && lane == 0) mbar_arrive(empty_bar + stage);
                if (++stage == kSStages) { stage = 0; phase ^= 1; }
            }

            // warp reduction, one value per activation row
#pragma unroll
            for (int m = 0; m < kSRowsMax; ++m) {
                float v = acc[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                acc[m] = v;
            }
            if (active && !poisoned && lane == 0) {
#pragma unroll
                for (int m = 0; m < kSRowsMax; ++m) {
                    if (m < rm) {
                        const int64_t row = (int64_t)it.row0 + r_lo + m;
                        if (bf16_out_direct) out_bf[row * a.g.N + n] = f32_to_bf16_bits(acc[m]);
                        else a.g.ws[((int64_t)it.split * a.g.T + row) * a.g.N + n] = acc[m];
                    }
                }
            }
        }

        if (!bf16_out_direct) {
            // ordered split-K finish: the CTA that arrives last sums the partials of this
            // (group, tile) in split order 0..S-1 and writes bf16.
            __threadfence();
            named_bar_sync(1, kSConsumerWarps * 32);
            int32_t* cnt = a.g.counters + (int64_t)it.g * a.n_tiles + it.tile;
            if (threadIdx.x == 0) {
                const int old = atomicAdd(cnt, 1);
                *last_flag = (old == a.g.split_k - 1) ? 1 : 0;
            }
            named_bar_sync(1, kSConsumerWarps * 32);
            if (*last_flag && !poisoned) {
                __threadfence();
                const int n0 = it.tile * kSTileN;
                for (int i = threadIdx.x; i < it.rows * kSTileN; i += kSConsumerWarps * 32) {
                    const int r = i / kSTileN, cidx = i - r * kSTileN;
                    if (n0 + cidx < a.g.N) {
                        const int64_t row = (int64_t)it.row0 + r;
                        float s = 0.f;
                        for (int sp = 0; sp < a.g.split_k; ++sp)
                            s += __ldcg(a.g.ws + ((int64_t)sp * a.g.T + row) * a.g.N + n0 + cidx);
                        out_bf[row * a.g.N + n0 + cidx] = f32_to_bf16_bits(s);
                    }
                }
                if (threadIdx.x == 0) *cnt = 0;   // leave the workspace zeroed for the next call
            }
            named_bar_sync(1, kSConsumerWarps * 32);
        }
    }
    if (poisoned && threadIdx.x == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
}

}  // namespace gnf4b
