// Streaming (CUDA-core) grouped GEMM for decode-sized groups.
//
// One persistent CTA per SM.  Warps 8..11 are producers: they walk this CTA's contiguous
// range of work items and stream each item's packed rows from HBM into an 8-stage
// shared-memory ring with 1-D bulk copies (TMA engine) counted on mbarriers, and stage
// the block scales beside them.  Stage number q belongs to producer warp q % 4 and each
// warp keeps its next stage's scale loads in flight, so eight global-memory latencies
// overlap per CTA.  Warps 0..7 are consumers: consumer w owns weight row
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
    int32_t g_cache;        // groups whose offsets / expert ids are cached in shared memory
    int64_t total_items;
};

__host__ __device__ inline size_t stream_smem_bytes(int rows_cap, int a_units_pad, int g_cache) {
    return (size_t)kSTableBytes + (size_t)kSStages * kSStageBytes +
           (size_t)rows_cap * a_units_pad * 128 + 256 + (size_t)(2 * g_cache + 1) * 4;
}

// Decoded item shared by producer and consumers (they must agree exactly).
struct StreamItem {
    int32_t g, tile, split, row0, rows, eid, c0, c1;
    bool valid;
};

// Position in the item space plus the current group's row range and expert id.  Consecutive
// items of a CTA are reached by incrementing (split, tile, group) counters; the group table
// is read from shared memory (the first g_cache groups) so the hot loop has no global load
// and no division.
struct ItemWalker {
    int32_t g, tile, split;
    int32_t loaded_g;
    int32_t row0, rows, eid;
    bool gvalid;
};

__device__ __forceinline__ void walker_seek(const StreamArgs& a, ItemWalker& w, int64_t item) {
    const int64_t per_group = (int64_t)a.n_tiles * a.g.split_k;
    w.g = (int32_t)(item / per_group);
    const int32_t rem = (int32_t)(item - (int64_t)w.g * per_group);
    w.tile = rem / a.g.split_k;
    w.split = rem - w.tile * a.g.split_k;
    w.loaded_g = -1;
}

__device__ __forceinline__ void walker_step(const StreamArgs& a, ItemWalker& w) {
    if (++w.split == a.g.split_k) {
        w.split = 0;
        if (++w.tile == a.n_tiles) { w.tile = 0; ++w.g; }
    }
}

__device__ __forceinline__ StreamItem walker_item(const StreamArgs& a, const int32_t* s_grp, ItemWalker& w) {
    if (w.loaded_g != w.g) {
        int32_t end;
        if (w.g < a.g_cache) {
            w.row0 = s_grp[w.g];
            end = s_grp[w.g + 1];
            w.eid = s_grp[a.g_cache + 1 + w.g];
        } else {
            w.row0 = __ldg(a.g.off + w.g);
            end = __ldg(a.g.off + w.g + 1);
            w.eid = __ldg(a.g.eids + w.g);
        }
        w.rows = end - w.row0;
        const bool bad_e = w.eid < 0 || w.eid >= a.g.E;
        const bool bad_o = w.rows < 0 || w.row0 < 0 || (int64_t)w.row0 + w.rows > a.g.T;
        w.gvalid = !bad_e && !bad_o && w.rows > 0;
        const bool pad = w.eid == GNF4B_PAD_EXPERT;      // padding group: skipped, not an error
        if (((bad_e && !pad) || bad_o) && w.rows != 0 && a.g.status && (threadIdx.x & 31) == 0)
            atomicOr(a.g.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
        w.loaded_g = w.g;
    }
    StreamItem it;
    it.g = w.g; it.tile = w.tile; it.split = w.split;
    it.row0 = w.row0; it.rows = w.rows; it.eid = w.eid; it.valid = w.gvalid;
    it.c0 = w.split * a.chunks_per_split;
    it.c1 = min(a.n_chunks, it.c0 + a.chunks_per_split);
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

// One ring stage = (item, row chunk, K chunk).  Producers and consumers enumerate the
// stages of a CTA in the same order: items ascending, row chunks, then K chunks.
struct StageCursor {
    int64_t item;
    int32_t rc, c, row_chunks;
    bool in_item;
    ItemWalker w;
    StreamItem it;
};

// Advance to the next stage; returns false past the end.  cursor_init first.
__device__ __forceinline__ void cursor_init(const StreamArgs& a, StageCursor& cur, int64_t item_lo) {
    cur.item = item_lo - 1;
    cur.in_item = false;
    walker_seek(a, cur.w, item_lo);
}

__device__ __forceinline__ bool cursor_next(const StreamArgs& a, const int32_t* s_grp, StageCursor& cur,
                                            int64_t item_lo, int64_t item_hi) {
    if (cur.in_item) {                         // inside an item: next K chunk, then next row chunk
        if (++cur.c < cur.it.c1) return true;
        if (++cur.rc < cur.row_chunks) { cur.c = cur.it.c0; return true; }
    }
    while (++cur.item < item_hi) {
        if (cur.item > item_lo) walker_step(a, cur.w);
        cur.it = walker_item(a, s_grp, cur.w);
        if (cur.it.valid) {
            cur.row_chunks = (cur.it.rows + a.rows_cap - 1) / a.rows_cap;
            cur.rc = 0;
            cur.c = cur.it.c0;
            cur.in_item = true;
            return true;
        }
    }
    cur.in_item = false;
    return false;
}

// Block scales of one stage, widened to fp32, 16 per lane: slot (r, j) = (i / 64, i % 64) for
// i = lane + 32 t.  Slots past the chunk or past N read nothing (0).
template <int FMT, int SDT>
__device__ __forceinline__ void producer_fetch_scales(const StreamArgs& a, int eid, int tile, int c,
                                                      int scales_per_chunk, int lane, float* v) {
    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;
    const int64_t boff = (int64_t)c * a.chunk_bytes;
    const int cbytes = (int)min((int64_t)a.chunk_bytes, a.g.K / 2 - boff);
    const int nsc = cbytes * 2 / (int)scale_blk;
    const int n0 = tile * kSTileN;
    const int64_t base = (int64_t)eid * a.g.s_se + (int64_t)c * scales_per_chunk;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const int i = lane + 32 * t;
        const int r = i >> 6, j = i & 63;
        v[t] = (j < nsc && n0 + r < a.g.N) ? load_scale<SDT>(a.g.S, base + (int64_t)(n0 + r) * a.g.s_sn + j) : 0.f;
    }
}

// Warm L2 (and the TLB) with the block scales of one stage: lanes 0..15 each touch one of
// the at most two 128-byte lines of one of the eight rows.
template <int FMT, int SDT>
__device__ __forceinline__ void producer_prefetch_scales(const StreamArgs& a, int eid, int tile, int c,
                                                         int scales_per_chunk, int lane) {
    if (lane >= 16) return;
    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;
    const int elt = (SDT == GNF4B_S_F32) ? 4 : (SDT == GNF4B_S_BF16 ? 2 : 1);
    const int64_t boff = (int64_t)c * a.chunk_bytes;
    const int cbytes = (int)min((int64_t)a.chunk_bytes, a.g.K / 2 - boff);
    const int nsc = cbytes * 2 / (int)scale_blk;
    const int n = tile * kSTileN + (lane >> 1);
    if (n >= a.g.N) return;
    const uintptr_t first = reinterpret_cast<uintptr_t>(a.g.S) +
        (uintptr_t)(((int64_t)eid * a.g.s_se + (int64_t)n * a.g.s_sn + (int64_t)c * scales_per_chunk) * elt);
    const uintptr_t last = first + (uintptr_t)(nsc * elt) - 1;
    const uintptr_t line = (first & ~(uintptr_t)127) + (uintptr_t)(lane & 1) * 128;
    if (line <= last) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
}

// One unit (16 packed bytes = 32 elements) against one activation row held in registers.
// Four partial sums, one per byte position of a word, keep the FMA chains short; every
// path of this file sums a unit in this same order.
__device__ __forceinline__ float unit_dot_regs(const uint4 wv, const float* a32, uint32_t tab_lane) {
    const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
    float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t off = prmt(words[i], 0u, 0x4404u | (b << 4));      // byte b -> bits 8..15
            const float2 p = ld_shared_f32x2(tab_lane + off);
            part[b] = fmaf(p.x, a32[i * 8 + b * 2], part[b]);
            part[b] = fmaf(p.y, a32[i * 8 + b * 2 + 1], part[b]);
        }
    }
    return (part[0] + part[1]) + (part[2] + part[3]);
}

// FMT: weight format.  SDT: scale dtype.  AU > 0: decode specialisation -- every group has at
// most one row and K <= AU * 1024, the activation row lives in registers (AU units of 32
// elements per lane), no split-K.  AU == 0: any group size, activations staged in shared
// memory, optional split-K.
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
    int32_t* s_grp = reinterpret_cast<int32_t*>(tail + 256);     // [g_cache + 1 offsets][g_cache expert ids]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSStages; ++s) {
            mbar_init(full_bar + s, 2);      // weights published + scales published
            mbar_init(empty_bar + s, kSConsumerWarps);
        }
        *abort_flag = 0;
        *last_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < 2 * a.g_cache + 1; i += kSThreads)
        s_grp[i] = (i <= a.g_cache) ? __ldg(a.g.off + i) : __ldg(a.g.eids + (i - a.g_cache - 1));
    __syncthreads();

    const int64_t item_lo = a.total_items * blockIdx.x / gridDim.x;
    const int64_t item_hi = a.total_items * (blockIdx.x + 1) / gridDim.x;
    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;
    const int scales_per_chunk = a.chunk_bytes * 2 / (int)scale_blk;
    const int64_t row_bytes = a.g.K / 2;

    if (warp >= kSConsumerWarps && AU > 0) {
        // ------------------------------------------------------------ producers, decode form
        // Every item takes exactly n_chunks ring stages whether its group is empty or not, so
        // stage q of this CTA is (item_lo + q / n_chunks, q % n_chunks) in closed form and a
        // producer warp reaches its stages q = pw, pw + 4, ... without walking the ones between.
        // A four-deep register queue of stage descriptors lets a warp prefetch the scales of a
        // stage into L2 three of its turns ahead, load them one turn ahead and publish them now.
        const uint32_t pw = (uint32_t)(warp - kSConsumerWarps);
        const uint32_t nc = (uint32_t)a.n_chunks;
        const uint32_t ns = (uint32_t)(item_hi - item_lo) * nc;
        struct DStage { int32_t eid, tile, c; bool valid; };
        // generator state: next stage index to describe and the (group, tile) of its item
        uint32_t gq = pw;
        uint32_t g_item = gq / nc;                       // item index relative to item_lo
        int32_t gg, gtile;
        {
            const uint32_t it0 = (uint32_t)item_lo + g_item;
            gg = (int32_t)(it0 / (uint32_t)a.n_tiles);
            gtile = (int32_t)(it0 - (uint32_t)gg * (uint32_t)a.n_tiles);
        }
        auto gen = [&]() -> DStage {
            DStage d;
            d.valid = false; d.eid = 0; d.tile = gtile; d.c = (int32_t)(gq - g_item * nc);
            if (gq < ns) {
                int32_t row0, end;
                if (gg < a.g_cache) { row0 = s_grp[gg]; end = s_grp[gg + 1]; d.eid = s_grp[a.g_cache + 1 + gg]; }
                else { row0 = __ldg(a.g.off + gg); end = __ldg(a.g.off + gg + 1); d.eid = __ldg(a.g.eids + gg); }
                d.valid = end > row0 && row0 >= 0 && end <= a.g.T && d.eid >= 0 && d.eid < a.g.E;
                if (d.valid) producer_prefetch_scales<FMT, SDT>(a, d.eid, d.tile, d.c, scales_per_chunk, lane);
            }
            gq += kSProducerWarps;
            const uint32_t ni = gq / nc;
            gtile += (int32_t)(ni - g_item);
            g_item = ni;
            while (gtile >= a.n_tiles) { gtile -= a.n_tiles; ++gg; }
            return d;
        };
        DStage f0 = gen(), f1 = gen(), f2 = gen(), f3 = gen();
        float v_cur[16], v_nxt[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) { v_cur[t] = 0.f; v_nxt[t] = 0.f; }
        if (f0.valid) producer_fetch_scales<FMT, SDT>(a, f0.eid, f0.tile, f0.c, scales_per_chunk, lane, v_cur);
        bool poisoned = false;
        for (uint32_t q = pw; q < ns; q += kSProducerWarps) {
            const uint32_t stage = q % kSStages, phase = (q / kSStages) & 1;
            if (!poisoned && !mbar_wait_bounded(empty_bar + stage, phase ^ 1, abort_flag)) poisoned = true;
            uint8_t* st = ring + stage * kSStageBytes;
            if (!poisoned) {
                if (f0.valid && a.w_align == 16) {
                    const int n0 = f0.tile * kSTileN;
                    const int n_valid = min(kSTileN, (int)(a.g.N - n0));
                    const int64_t boff = (int64_t)f0.c * kSRowPitch;
                    const int cbytes = (int)min((int64_t)kSRowPitch, row_bytes - boff);
                    if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, (uint32_t)(n_valid * cbytes));
                    __syncwarp();
                    if (lane < n_valid)
                        bulk_g2s(st + lane * kSRowPitch,
                                 a.g.W + (int64_t)f0.eid * a.g.w_se + (int64_t)(n0 + lane) * a.g.w_sn + boff,
                                 (uint32_t)cbytes, full_bar + stage);
                } else {
                    if (f0.valid) {
                        const int n0 = f0.tile * kSTileN;
                        const int n_valid = min(kSTileN, (int)(a.g.N - n0));
                        const int64_t boff = (int64_t)f0.c * kSRowPitch;
                        const int cbytes = (int)min((int64_t)kSRowPitch, row_bytes - boff);
                        for (int r = 0; r < n_valid; ++r) {
                            const uint8_t* src = a.g.W + (int64_t)f0.eid * a.g.w_se + (int64_t)(n0 + r) * a.g.w_sn + boff;
                            if (a.w_align == 8) plain_copy_row<8>(st + r * kSRowPitch, src, cbytes, lane);
                            else if (a.w_align == 4) plain_copy_row<4>(st + r * kSRowPitch, src, cbytes, lane);
                            else plain_copy_row<1>(st + r * kSRowPitch, src, cbytes, lane);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar + stage);
                }
            }
            if (f1.valid) producer_fetch_scales<FMT, SDT>(a, f1.eid, f1.tile, f1.c, scales_per_chunk, lane, v_nxt);
            if (!poisoned) {
                float* st_sc = reinterpret_cast<float*>(st + kSTileN * kSRowPitch);
                if (f0.valid) {
#pragma unroll
                    for (int t = 0; t < 16; ++t) st_sc[lane + 32 * t] = v_cur[t];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar + stage);
            }
            f0 = f1; f1 = f2; f2 = f3; f3 = gen();
#pragma unroll
            for (int t = 0; t < 16; ++t) v_cur[t] = v_nxt[t];
        }
        if (poisoned && lane == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
        return;
    }
    if (warp >= kSConsumerWarps) {
        // ------------------------------------------------------------ producers
        // Stage q of this CTA belongs to producer warp q % 4.  Per stage a warp (1) issues the
        // bulk copies of the packed rows, (2) stores the block scales it loaded one iteration
        // earlier, (3) starts the loads of its next stage's scales and (4) prefetches into L2
        // the scales of the stage three of its turns ahead, so what it waits for is an L2 hit.
        constexpr int kFar = 3;
        const uint32_t pw = (uint32_t)(warp - kSConsumerWarps);
        StageCursor cur;
        cursor_init(a, cur, item_lo);
        uint32_t q = 0;                       // stage sequence number of `cur`
        bool have = cursor_next(a, s_grp, cur, item_lo, item_hi);
        for (uint32_t i = 0; have && i < pw; ++i, ++q) have = cursor_next(a, s_grp, cur, item_lo, item_hi);
        float v_cur[16], v_nxt[16];
        if (have) producer_fetch_scales<FMT, SDT>(a, cur.it.eid, cur.it.tile, cur.c, scales_per_chunk, lane, v_cur);
        StageCursor far = cur;
        bool have_far = have;
        for (int d = 0; d < kFar; ++d) {
            for (int i = 0; have_far && i < kSProducerWarps; ++i) have_far = cursor_next(a, s_grp, far, item_lo, item_hi);
            if (have_far) producer_prefetch_scales<FMT, SDT>(a, far.it.eid, far.it.tile, far.c, scales_per_chunk, lane);
        }
        bool poisoned = false;
        while (have) {
            const uint32_t stage = q % kSStages, phase = (q / kSStages) & 1;
            if (!poisoned && !mbar_wait_bounded(empty_bar + stage, phase ^ 1, abort_flag)) poisoned = true;
            uint8_t* st = ring + stage * kSStageBytes;
            if (!poisoned) {
                const uint8_t* w_e = a.g.W + (int64_t)cur.it.eid * a.g.w_se;
                const int n0 = cur.it.tile * kSTileN;
                const int n_valid = min(kSTileN, (int)(a.g.N - n0));
                const int64_t boff = (int64_t)cur.c * a.chunk_bytes;
                const int cbytes = (int)min((int64_t)a.chunk_bytes, row_bytes - boff);
                if (a.w_align == 16) {
                    if (lane == 0) mbar_arrive_expect_tx(full_bar + stage, (uint32_t)(n_valid * cbytes));
                    __syncwarp();
                    if (lane < n_valid)
                        bulk_g2s(st + lane * kSRowPitch, w_e + (int64_t)(n0 + lane) * a.g.w_sn + boff,
                                 (uint32_t)cbytes, full_bar + stage);
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
            StageCursor nxt = cur;
            bool have_nxt = true;
            for (int i = 0; have_nxt && i < kSProducerWarps; ++i) have_nxt = cursor_next(a, s_grp, nxt, item_lo, item_hi);
            if (have_nxt) producer_fetch_scales<FMT, SDT>(a, nxt.it.eid, nxt.it.tile, nxt.c, scales_per_chunk, lane, v_nxt);
            for (int i = 0; have_far && i < kSProducerWarps; ++i) have_far = cursor_next(a, s_grp, far, item_lo, item_hi);
            if (have_far) producer_prefetch_scales<FMT, SDT>(a, far.it.eid, far.it.tile, far.c, scales_per_chunk, lane);
            if (!poisoned) {
                // scale slot (r, j) of the stage lives at st_sc[r * 64 + j]; a lane owns slots
                // lane, lane + 32, ... of the 8 x 64 grid
                float* st_sc = reinterpret_cast<float*>(st + kSTileN * kSRowPitch);
#pragma unroll
                for (int t = 0; t < 16; ++t) st_sc[lane + 32 * t] = v_cur[t];
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar + stage);
            }
            cur = nxt;
            have = have_nxt;
            q += kSProducerWarps;
#pragma unroll
            for (int t = 0; t < 16; ++t) v_cur[t] = v_nxt[t];
        }
        if (poisoned && lane == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
        return;
    }

    // ---------------------------------------------------------------- consumers
    // pair table: tab[byte][slot] for slot 0..31, every slot holds the same float2, so a
    // lane reading slot == its lane id never conflicts with another lane.  Warp w fills the
    // rows of bytes 32w..32w+31: each lane looks one byte up once, shuffles spread it.
    {
        float2* tab = reinterpret_cast<float2*>(tab_raw);
        const float2 mine = byte_pair<FMT>(warp * 32 + lane);
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
            float2 p;
            p.x = __shfl_sync(0xffffffffu, mine.x, j);
            p.y = __shfl_sync(0xffffffffu, mine.y, j);
            tab[(warp * 32 + j) * 32 + lane] = p;
        }
    }
    named_bar_sync(1, kSConsumerWarps * 32);

    const uint32_t tab_lane = smem_u32(tab_raw) + lane * 8;
    uint16_t* out_bf = reinterpret_cast<uint16_t*>(a.g.out);
    uint32_t stage = 0, phase = 0;
    bool poisoned = false;
    ItemWalker walker;
    walker_seek(a, walker, item_lo);

    if constexpr (AU > 0) {
        // ------------------------------------------------ decode: one row per group
        float a_reg[AU * 32];
        int reg_g = -1;
        for (int64_t item = item_lo; item < item_hi; ++item) {
            if (item > item_lo) walker_step(a, walker);
            const StreamItem it = walker_item(a, s_grp, walker);
            const int n = it.tile * kSTileN + warp;
            const bool active = it.valid && n < a.g.N;      // empty groups still take their stages
            if (active && reg_g != it.g) {
                const uint8_t* xrow = reinterpret_cast<const uint8_t*>(a.g.x) + (int64_t)it.row0 * a.g.K * 2;
#pragma unroll
                for (int q = 0; q < AU; ++q) {
                    const int U = lane + 32 * q;
                    if (U * 32 < a.g.K) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            cvt8(__ldg(reinterpret_cast<const uint4*>(xrow + (int64_t)U * 64 + v * 16)), a.g.x_dtype,
                                 &a_reg[q * 32 + v * 8]);
                    } else {
#pragma unroll
                        for (int v = 0; v < 32; ++v) a_reg[q * 32 + v] = 0.f;
                    }
                }
                reg_g = it.g;
            }
            float acc = 0.f;
#pragma unroll
            for (int c = 0; c < (AU + 1) / 2; ++c) {
                if (c < a.n_chunks) {
                    if (!poisoned && !mbar_wait_bounded(full_bar + stage, phase, abort_flag)) poisoned = true;
                    if (!poisoned && active) {
                        const uint32_t st = smem_u32(ring + stage * kSStageBytes);
                        const uint32_t wrow = st + warp * kSRowPitch;
                        const uint32_t srow = st + kSTileN * kSRowPitch + warp * kSScaleSlots * 4;
                        const int cbytes = (int)min((int64_t)kSRowPitch, row_bytes - (int64_t)c * kSRowPitch);
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            if (c * 2 + j < AU) {
                                const int u = lane + 32 * j;
                                if (u * 16 < cbytes) {
                                    const uint4 wv = ld_shared_u32x4(wrow + u * 16);
                                    const float sc = ld_shared_f32(srow + ((FMT == GNF4B_FMT_NF4) ? (u >> 1) : u) * 4);
                                    acc += unit_dot_regs(wv, &a_reg[(c * 2 + j) * 32], tab_lane) * sc;
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (!poisoned && lane == 0) mbar_arrive(empty_bar + stage);
                    if (++stage == kSStages) { stage = 0; phase ^= 1; }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (active && !poisoned && lane == 0) out_bf[(int64_t)it.row0 * a.g.N + n] = f32_to_bf16_bits(acc);
        }
    } else {
        // ------------------------------------------------ any group size
        const uint32_t a_base = smem_u32(a_smem);
        const int upg = a.a_units_pad >> 5;
        const int units_per_chunk = a.chunk_bytes >> 4;
        const int64_t n_units = a.g.K / 32;
        const bool bf16_out_direct = a.g.split_k == 1;
        int staged_g = -1, staged_rc = -1;   // what a_smem currently holds
        for (int64_t item = item_lo; item < item_hi; ++item) {
            if (item > item_lo) walker_step(a, walker);
            const StreamItem it = walker_item(a, s_grp, walker);
            if (!it.valid) continue;
            const int n = it.tile * kSTileN + warp;
            const bool active = n < a.g.N;
            const int row_chunks = (it.rows + a.rows_cap - 1) / a.rows_cap;

            for (int rc = 0; rc < row_chunks; ++rc) {
                const int r_lo = rc * a.rows_cap;
                const int rm = min(a.rows_cap, it.rows - r_lo);
                float acc[kSRowsMax] = {0.f, 0.f, 0.f, 0.f};

                if (staged_g != it.g || staged_rc != rc) {
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
                                const int U = c * units_per_chunk + u;
                                float part[kSRowsMax][4];
#pragma unroll
                                for (int m = 0; m < kSRowsMax; ++m)
#pragma unroll
                                    for (int b = 0; b < 4; ++b) part[m][b] = 0.f;
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    float wf[8];
#pragma unroll
                                    for (int b = 0; b < 4; ++b) {
                                        const uint32_t off = prmt(words[i], 0u, 0x4404u | (b << 4));
                                        const float2 p = ld_shared_f32x2(tab_lane + off);
                                        wf[2 * b] = p.x;
                                        wf[2 * b + 1] = p.y;
                                    }
#pragma unroll
                                    for (int m = 0; m < kSRowsMax; ++m) {
                                        if (m < rm) {
                                            const float4 lo = ld_shared_f32x4(a_base + a_f4_offset(m, upg, U, 2 * i));
                                            const float4 hi = ld_shared_f32x4(a_base + a_f4_offset(m, upg, U, 2 * i + 1));
                                            part[m][0] = fmaf(wf[1], lo.y, fmaf(wf[0], lo.x, part[m][0]));
                                            part[m][1] = fmaf(wf[3], lo.w, fmaf(wf[2], lo.z, part[m][1]));
                                            part[m][2] = fmaf(wf[5], hi.y, fmaf(wf[4], hi.x, part[m][2]));
                                            part[m][3] = fmaf(wf[7], hi.w, fmaf(wf[6], hi.z, part[m][3]));
                                        }
                                    }
                                }
#pragma unroll
                                for (int m = 0; m < kSRowsMax; ++m)
                                    acc[m] += ((part[m][0] + part[m][1]) + (part[m][2] + part[m][3])) * sc;
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
    }
    if (poisoned && threadIdx.x == 0 && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
}

}  // namespace gnf4b
