// tcgen05 / TMEM grouped GEMM for prefill-sized groups, forward and dgrad.
//
// Persistent, warp-specialised, one CTA per SM (704 threads):
//   warp 0      TMA producer: activation tiles [128 rows x 64 contraction] per stage via
//               cp.async.bulk.tensor (128-byte swizzle), counted on full_a[stage]
//   warp 1      MMA issuer: one lane issues tcgen05.mma (M=128, N=128, K=16, bf16 x bf16,
//               fp32 accumulate in TMEM); tcgen05.commit frees the stage / publishes the tile
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (one TMEM lane quarter per warp),
//               one bf16 rounding, masked stores for ragged rows / columns
//   warps 6-21  weight decode: packed nibbles + block scales straight from global memory
//               (prefetched two stages ahead) -> bf16 tiles written into shared memory in the
//               UMMA canonical 128-byte-swizzled layout.  MXFP4 decodes exactly to one bf16
//               tile.  NF4 writes hi = bf16(w) and lo = bf16(w - hi) with w = fp32(LUT*absmax)
//               and the issuer runs two MMAs per step, so the product keeps ~16 mantissa bits.
//
// Work item = (group, chunk of up to two 128-row tiles, 128-column tile of the output); the
// decoded weight tile of a stage is shared by both row tiles.  Items are enumerated on the
// device from group_offsets (column tile fastest, so concurrently running CTAs read the same
// activation rows); there is no host-built tile table.  Accumulators are double-buffered in
// TMEM (2 buffers x 2 row tiles x 128 columns = all 512 columns).
//
//   forward  out[T, N] = x[T, K] . W^T : stage = 128 weight rows x 64 k, K-major B operand
//   dgrad    out[T, K] = x[T, N] . W   : stage = 64 weight rows x 128 k, the decoded tile is
//            k-contiguous and is used as an MN-major B operand, so nothing is transposed
//
// Stands in for _gemm_nf4_grouped, _dgrad_nf4_grouped and _gemm_mxfp4_grouped
// (kernel/nf4_grouped.py:365-462, 953-1023; kernel/mxfp4_grouped.py:51-97).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace gnf4b {

constexpr int kTBM = 128;             // rows per row tile (UMMA M)
constexpr int kTBC = 128;             // output columns per item (UMMA N)
constexpr int kTBR = 64;              // contraction elements per stage
constexpr int kTMT = 2;               // row tiles per item
constexpr int kTDecodeWarps = 16;
constexpr int kTThreads = (2 + 4 + kTDecodeWarps) * 32;
constexpr int kTATile = kTBM * kTBR * 2;        // 16 KiB
constexpr int kTBTile = kTBC * kTBR * 2;        // 16 KiB
constexpr int kTTableBytes = 32768;
constexpr int kTMaxStages = 4;
constexpr int kTTmemCols = 512;

struct TensorArgs {
    GemmArgs g;
    int64_t C;          // output columns (N forward, K dgrad)
    int64_t R;          // contraction length (K forward, N dgrad)
    int32_t c_tiles;    // ceil(C / 128)
    int32_t r_blocks;   // ceil(R / 64)
    int32_t stages;
    int32_t w_align;
};

__host__ __device__ inline int tensor_stage_bytes(int fmt) {
    return kTMT * kTATile + (fmt == GNF4B_FMT_NF4 ? 2 : 1) * kTBTile;
}
__host__ __device__ inline size_t tensor_smem_bytes(int fmt, int stages) {
    return (size_t)stages * tensor_stage_bytes(fmt) + kTTableBytes + 1024 /*barriers*/ + 1024 /*alignment*/;
}

// ------------------------------------------------------------------ tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int32_t c0, int32_t c1,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor of a bf16 tile in the 128-byte-swizzled canonical layout
// (rows of 128 bytes, 8-row groups of 1024 bytes).  lbo / sbo in bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)((lbo >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;      // descriptor version of this architecture
    d |= (uint64_t)2 << 61;      // SWIZZLE_128B
    return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 A and B, A K-major, M = 128, N = 128.
__host__ __device__ constexpr uint32_t umma_idesc(int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((kTBC >> 3) << 17) |
           ((kTBM >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float hi_elem, float lo_elem) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_elem), "f"(lo_elem));
    return d;
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Group table in shared memory (NF4 only: its lookup table leaves 30 KiB of the table region free; at most
// kTTabGroups groups): row range, expert id and the number of items before the group.  Without it every
// role walks the groups through global memory -- three dependent loads per group, a dozen groups per step
// of a CTA -- which costs the MMA issuer thousands of cycles between two items.
constexpr int kTTabGroups = 640;
struct TGrp {
    int32_t row0, rows, eid, base;
};

// Walks the item space in increasing item id.  Every role of a CTA runs the same walk.
struct ItemCursor {
    int32_t g = 0;
    int64_t base = 0;       // first item id of group g
    int32_t row0 = 0, rows = 0, eid = 0, chunks = 0;
    bool loaded = false;
};

struct TItem {
    int32_t row0;      // first row of this item's first row tile
    int32_t row_end;   // end of the group
    int32_t eid;
    int32_t c0;        // first output column
    int32_t mts;       // row tiles in this item (1..kTMT)
};

__device__ __forceinline__ bool next_item(const TensorArgs& a, ItemCursor& cur, int64_t id, TItem* it,
                                          const TGrp* tab = nullptr) {
    if (tab) {
        while (cur.g < a.g.G && id >= tab[cur.g + 1].base) cur.g++;
        if (cur.g >= a.g.G) return false;
        const TGrp gr = tab[cur.g];
        const int32_t local = (int32_t)(id - gr.base);
        const int32_t mc = local / a.c_tiles;
        const int32_t ct = local - mc * a.c_tiles;
        it->row0 = gr.row0 + mc * kTBM * kTMT;
        it->row_end = gr.row0 + gr.rows;
        it->eid = gr.eid;
        it->c0 = ct * kTBC;
        it->mts = min(kTMT, (it->row_end - it->row0 + kTBM - 1) / kTBM);
        return true;
    }
    while (cur.g < a.g.G) {
        if (!cur.loaded) {
            cur.row0 = __ldg(a.g.off + cur.g);
            cur.rows = __ldg(a.g.off + cur.g + 1) - cur.row0;
            cur.eid = __ldg(a.g.eids + cur.g);
            const bool bad_e = cur.eid < 0 || cur.eid >= a.g.E;
            const bool bad_o = cur.rows < 0 || cur.row0 < 0 || (int64_t)cur.row0 + cur.rows > a.g.T;
            const bool pad = cur.eid == GNF4B_PAD_EXPERT;    // padding group: skipped, not an error
            if (((bad_e && !pad) || bad_o) && cur.rows != 0 && a.g.status && threadIdx.x == 0 && blockIdx.x == 0)
                atomicOr(a.g.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
            cur.chunks = (bad_e || bad_o || cur.rows <= 0) ? 0 : (cur.rows + kTBM * kTMT - 1) / (kTBM * kTMT);
            cur.loaded = true;
        }
        const int64_t n_items = (int64_t)cur.chunks * a.c_tiles;
        if (id < cur.base + n_items) {
            const int32_t local = (int32_t)(id - cur.base);
            const int32_t mc = local / a.c_tiles;
            const int32_t ct = local - mc * a.c_tiles;
            it->row0 = cur.row0 + mc * kTBM * kTMT;
            it->row_end = cur.row0 + cur.rows;
            it->eid = cur.eid;
            it->c0 = ct * kTBC;
            it->mts = min(kTMT, (it->row_end - it->row0 + kTBM - 1) / kTBM);
            return true;
        }
        cur.base += n_items;
        cur.g++;
        cur.loaded = false;
    }
    return false;
}

// 8 packed bytes (16 elements) of one weight row.
__device__ __forceinline__ uint2 load_packed8(const uint8_t* p, int w_align) {
    if (w_align >= 8) return __ldg(reinterpret_cast<const uint2*>(p));
    uint2 v;
    if (w_align >= 4) {
        const uint32_t* q = reinterpret_cast<const uint32_t*>(p);
        v.x = __ldg(q);
        v.y = __ldg(q + 1);
    } else {
        uint32_t w[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
            w[i] = (uint32_t)__ldg(p + 4 * i) | ((uint32_t)__ldg(p + 4 * i + 1) << 8) |
                   ((uint32_t)__ldg(p + 4 * i + 2) << 16) | ((uint32_t)__ldg(p + 4 * i + 3) << 24);
        v = make_uint2(w[0], w[1]);
    }
    return v;
}

// Decode 16 elements and store them as two 16-byte chunks (8 bf16 each) of a swizzled
// 128-byte row.  row_addr = shared address of the row, chunk0 = first chunk index, r7 =
// row & 7 (the swizzle key), lo_delta = byte distance from the hi tile to the lo tile.
// Padding (rows past N, columns past K) arrives with scale 0 and decodes to zeros; it must
// not be produced from zero BYTES, which are code 0 = -1.0 in NF4.
//   NF4 table: lut[code][lane] fp32 (one copy of the 16-entry codebook per lane).
//   MXFP4 table: tab[byte][lane] bf16x2 of the doubled e2m1 pair.
template <int FMT>
__device__ __forceinline__ void decode_store16(const uint2 pk, float scale, uint32_t tab_lane, uint32_t row_addr,
                                               int chunk0, int r7, uint32_t lo_delta) {
    const uint32_t w[2] = {pk.x, pk.y};
    if (FMT == GNF4B_FMT_NF4) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                // even element = high nibble of byte b, odd element = low nibble; offset = code * 128
                const uint32_t off_e = (b == 0) ? ((w[i] << 3) & 0x780u) : ((w[i] >> (8 * b - 3)) & 0x780u);
                const uint32_t off_o = (b == 0) ? ((w[i] << 7) & 0x780u) : ((w[i] >> (8 * b - 7)) & 0x780u);
                const float w0 = ld_shared_f32(tab_lane + off_e) * scale;
                const float w1 = ld_shared_f32(tab_lane + off_o) * scale;
                hi[b] = pack_bf16x2(w1, w0);
                const float r0 = w0 - __uint_as_float(hi[b] << 16);
                const float r1 = w1 - __uint_as_float(hi[b] & 0xffff0000u);
                lo[b] = pack_bf16x2(r1, r0);
            }
            const uint32_t addr = row_addr + (uint32_t)(((chunk0 + i) ^ r7) << 4);
            st_shared_v4(addr, hi[0], hi[1], hi[2], hi[3]);
            st_shared_v4(addr + lo_delta, lo[0], lo[1], lo[2], lo[3]);
        }
    } else {
        // scale = 2^(e-128) as a bf16 pair (0 for padding); the table holds the doubled e2m1
        // values, so the bf16 product is exactly value * 2^(e-127)
        const uint32_t s16 = __float_as_uint(scale) >> 16;
        const uint32_t s2 = s16 | (s16 << 16);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint32_t v[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t off = (b == 0) ? ((w[i] << 7) & 0x7f80u) : ((w[i] >> (8 * b - 7)) & 0x7f80u);
                v[b] = mul_bf16x2(ld_shared_u32(tab_lane + off), s2);
            }
            st_shared_v4(row_addr + (uint32_t)(((chunk0 + i) ^ r7) << 4), v[0], v[1], v[2], v[3]);
        }
    }
}

template <int FMT, int SDT, int OP>
__global__ void __launch_bounds__(kTThreads, 1)
tensor_gemm_kernel(const TensorArgs a, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int kStageBytes = kTMT * kTATile + (FMT == GNF4B_FMT_NF4 ? 2 : 1) * kTBTile;
    constexpr uint32_t kLoDelta = kTBTile;
    uint8_t* tab_raw = smem + (size_t)a.stages * kStageBytes;
    uint64_t* full_a = reinterpret_cast<uint64_t*>(tab_raw + kTTableBytes);
    uint64_t* full_b = full_a + kTMaxStages;
    uint64_t* empty = full_b + kTMaxStages;
    uint64_t* acc_full = empty + kTMaxStages;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(full_a + s, 1);
            mbar_init(full_b + s, kTDecodeWarps);
            mbar_init(empty + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, 4);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTTmemCols);
        tmem_relinquish();
    }
    // decode table, one copy per lane so lookups never conflict: NF4 lut[code][lane] fp32,
    // MXFP4 tab[byte][lane] bf16x2 (doubled e2m1 pair).
    const TGrp* gtab = nullptr;
    if (FMT == GNF4B_FMT_NF4) {
        float* tab = reinterpret_cast<float*>(tab_raw);
        for (int i = threadIdx.x; i < 16 * 32; i += kTThreads) tab[i] = kNf4Lut[i >> 5];
        if (a.g.G <= kTTabGroups && a.g.G <= kTThreads) {
            // one thread per group, block-wide inclusive scan of the item counts
            TGrp* gt = reinterpret_cast<TGrp*>(tab_raw + 2048);
            int32_t* wtot = reinterpret_cast<int32_t*>(tab_raw + 2048 + (kTTabGroups + 1) * 16);
            const int t = threadIdx.x;
            int32_t items = 0;
            TGrp gr{0, 0, 0, 0};
            if (t < a.g.G) {
                gr.row0 = __ldg(a.g.off + t);
                gr.rows = __ldg(a.g.off + t + 1) - gr.row0;
                gr.eid = __ldg(a.g.eids + t);
                const bool bad_e = gr.eid < 0 || gr.eid >= a.g.E;
                const bool bad_o = gr.rows < 0 || gr.row0 < 0 || (int64_t)gr.row0 + gr.rows > a.g.T;
                const bool pad = gr.eid == GNF4B_PAD_EXPERT;
                if (((bad_e && !pad) || bad_o) && gr.rows != 0 && a.g.status && blockIdx.x == 0)
                    atomicOr(a.g.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
                const int32_t chunks = (bad_e || bad_o || gr.rows <= 0) ? 0 : (gr.rows + kTBM * kTMT - 1) / (kTBM * kTMT);
                items = chunks * a.c_tiles;
            }
            int32_t incl = items;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int32_t up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            if (lane == 31) wtot[warp] = incl;
            __syncthreads();
            int32_t before = 0;
            for (int v = 0; v < warp; ++v) before += wtot[v];
            if (t < a.g.G) {
                gr.base = before + incl - items;
                gt[t] = gr;
                if (t == a.g.G - 1) gt[a.g.G] = TGrp{0, 0, 0, before + incl};
            }
            gtab = gt;
        }
    } else {
        uint32_t* tab = reinterpret_cast<uint32_t*>(tab_raw);
        for (int i = threadIdx.x; i < 256 * 32; i += kTThreads) {
            const float2 p = byte_pair<FMT>(i >> 5);
            tab[i] = pack_bf16x2(p.y, p.x);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ItemCursor cur;
            TItem it;
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int64_t id = blockIdx.x; ok && next_item(a, cur, id, &it, gtab); id += gridDim.x) {
                for (int rb = 0; rb < a.r_blocks && ok; ++rb) {
                    ok = mbar_wait_bounded(empty + stage, phase ^ 1, abort_flag);
                    if (!ok) break;
                    uint8_t* st = smem + (size_t)stage * kStageBytes;
                    mbar_arrive_expect_tx(full_a + stage, (uint32_t)(it.mts * kTATile));
                    for (int mt = 0; mt < it.mts; ++mt)
                        tma_load_2d(st + mt * kTATile, &x_map, rb * kTBR, it.row0 + mt * kTBM, full_a + stage);
                    if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            ItemCursor cur;
            TItem it;
            uint32_t stage = 0, phase = 0, buf = 0, acc_phase = 0;
            bool ok = true;
            constexpr uint32_t idesc = umma_idesc(OP == GNF4B_OP_DGRAD ? 1 : 0);
            for (int64_t id = blockIdx.x; ok && next_item(a, cur, id, &it, gtab); id += gridDim.x) {
                ok = mbar_wait_bounded(acc_empty + buf, acc_phase ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                for (int rb = 0; rb < a.r_blocks && ok; ++rb) {
                    ok = mbar_wait_bounded(full_a + stage, phase, abort_flag) &&
                         mbar_wait_bounded(full_b + stage, phase, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)stage * kStageBytes);
                    const uint32_t b_hi = st + kTMT * kTATile;
#pragma unroll
                    for (int mt = 0; mt < kTMT; ++mt) {
                        if (mt < it.mts) {
                            const uint32_t d = tmem_base + (uint32_t)((buf * kTMT + mt) * kTBC);
#pragma unroll
                            for (int j = 0; j < kTBR / 16; ++j) {
                                const uint64_t da = umma_desc(st + mt * kTATile + j * 32, 16, 1024);
                                // forward: K-major tile, 32 bytes per 16 k.  dgrad: MN-major tile
                                // [64 n][128 k]: two 64-column blocks 8192 bytes apart (LBO),
                                // 8-row groups 1024 bytes apart (SBO), 16 n = 2048 bytes per step.
                                const uint64_t dbh = (OP == GNF4B_OP_FWD) ? umma_desc(b_hi + j * 32, 16, 1024)
                                                                          : umma_desc(b_hi + j * 2048, 8192, 1024);
                                tc_mma_bf16(d, da, dbh, idesc, (rb > 0 || j > 0) ? 1u : 0u);
                                if (FMT == GNF4B_FMT_NF4) {
                                    const uint64_t dbl = (OP == GNF4B_OP_FWD)
                                                             ? umma_desc(b_hi + kLoDelta + j * 32, 16, 1024)
                                                             : umma_desc(b_hi + kLoDelta + j * 2048, 8192, 1024);
                                    tc_mma_bf16(d, da, dbl, idesc, 1u);
                                }
                            }
                        }
                    }
                    tc_commit(empty + stage);
                    if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(acc_full + buf);
                if (++buf == 2) { buf = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        ItemCursor cur;
        TItem it;
        uint32_t buf = 0, acc_phase = 0;
        bool ok = true;
        uint16_t* out = reinterpret_cast<uint16_t*>(a.g.out);
        const bool vec_ok = (a.C % 8) == 0;
        for (int64_t id = blockIdx.x; ok && next_item(a, cur, id, &it, gtab); id += gridDim.x) {
            ok = mbar_wait_bounded(acc_full + buf, acc_phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            for (int mt = 0; mt < it.mts; ++mt) {
                const int64_t row = (int64_t)it.row0 + mt * kTBM + q * 32 + lane;
                const bool row_ok = row < it.row_end;
#pragma unroll 1
                for (int c = 0; c < kTBC / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((buf * kTMT + mt) * kTBC + c * 32), r);
                    tmem_ld_wait();
                    const int64_t col = (int64_t)it.c0 + c * 32;
                    if (row_ok && col < a.C) {
                        uint16_t* dst = out + row * a.C + col;
                        if (vec_ok && col + 32 <= a.C) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(r[8 * v + 1]), __uint_as_float(r[8 * v + 0]));
                                o.y = pack_bf16x2(__uint_as_float(r[8 * v + 3]), __uint_as_float(r[8 * v + 2]));
                                o.z = pack_bf16x2(__uint_as_float(r[8 * v + 5]), __uint_as_float(r[8 * v + 4]));
                                o.w = pack_bf16x2(__uint_as_float(r[8 * v + 7]), __uint_as_float(r[8 * v + 6]));
                                *reinterpret_cast<uint4*>(dst + 8 * v) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < a.C) dst[j] = f32_to_bf16_bits(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + buf);
            if (++buf == 2) { buf = 0; acc_phase ^= 1; }
        }
    } else {
        // ------------------------------------------------------------ weight decode
        const int dt = threadIdx.x - 6 * 32;       // 0..511, 16 elements (8 packed bytes) each
        // forward: stage tile = 128 weight rows x 64 k.  row = dt / 4, k offset = (dt % 4) * 16.
        // dgrad:   stage tile = 64 weight rows x 128 k, stored as two 64-column blocks of 8 KiB.
        //          block = dt / 256, row = (dt % 256) / 4, k offset = block * 64 + (dt % 4) * 16.
        // Either way a quarter warp covers two rows x four 32-byte pieces, whose swizzled
        // 16-byte chunks fall into eight different bank groups.
        const int blk = (OP == GNF4B_OP_FWD) ? 0 : (dt >> 8);
        const int trow = (OP == GNF4B_OP_FWD) ? (dt >> 2) : ((dt & 255) >> 2);
        const int koff = blk * 64 + (dt & 3) * 16;
        const int chunk0 = (dt & 3) * 2;
        const uint32_t tile_off = (uint32_t)(blk * 8192 + trow * 128);
        const int r7 = trow & 7;
        const uint32_t tab_lane = smem_u32(tab_raw) + lane * 4;
        ItemCursor cur;
        TItem it;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int64_t id = blockIdx.x; ok && next_item(a, cur, id, &it, gtab); id += gridDim.x) {
            const uint8_t* w_e = a.g.W + (int64_t)it.eid * a.g.w_se;
            const int64_t s_e = (int64_t)it.eid * a.g.s_se;
            // Element coordinates of this thread's 16 elements in stage rb:
            //   forward: n = c0 + trow,        k = rb*64 + koff
            //   dgrad:   n = rb*64 + trow,     k = c0 + koff
            auto fetch = [&](int rb, uint2* pk, float* sc) {
                const int64_t n = (OP == GNF4B_OP_FWD) ? (int64_t)it.c0 + trow : (int64_t)rb * kTBR + trow;
                const int64_t k = (OP == GNF4B_OP_FWD) ? (int64_t)rb * kTBR + koff : (int64_t)it.c0 + koff;
                if (rb < a.r_blocks && n < a.g.N && k < a.g.K) {
                    *pk = load_packed8(w_e + n * a.g.w_sn + (k >> 1), a.w_align);
                    *sc = load_scale<SDT>(a.g.S, s_e + n * a.g.s_sn + k / scale_blk);
                } else {
                    *pk = make_uint2(0, 0);
                    *sc = 0.f;                 // padding decodes to zeros
                }
            };
            uint2 pk0, pk1;
            float sc0, sc1;
            fetch(0, &pk0, &sc0);
            fetch(1, &pk1, &sc1);
            for (int rb = 0; rb < a.r_blocks && ok; rb += 2) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (rb + u < a.r_blocks && ok) {
                        ok = mbar_wait_bounded(empty + stage, phase ^ 1, abort_flag);
                        if (ok) {
                            const uint32_t row_addr =
                                smem_u32(smem + (size_t)stage * kStageBytes) + kTMT * kTATile + tile_off;
                            if (u == 0) {
                                decode_store16<FMT>(pk0, sc0, tab_lane, row_addr, chunk0, r7, kLoDelta);
                                fetch(rb + 2, &pk0, &sc0);
                            } else {
                                decode_store16<FMT>(pk1, sc1, tab_lane, row_addr, chunk0, r7, kLoDelta);
                                fetch(rb + 3, &pk1, &sc1);
                            }
                            fence_proxy_async();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(full_b + stage);
                            if (++stage == (uint32_t)a.stages) { stage = 0; phase ^= 1; }
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

template <int FMT, int SDT, int OP>
static int launch_tensor_t(const TensorArgs& ta, const CUtensorMap& map, int sm_count, size_t smem, cudaStream_t st) {
    auto kfn = tensor_gemm_kernel<FMT, SDT, OP>;
    static int granted[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GNF4B_ECUDA;
    dev &= 63;
    if ((int)smem > granted[dev]) {
        if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GNF4B_ECUDA;
        granted[dev] = (int)smem;
    }
    kfn<<<sm_count, kTThreads, smem, st>>>(ta, map);
    return cudaPeekAtLastError() == cudaSuccess ? GNF4B_OK : GNF4B_ECUDA;
}

static int launch_tensor(int fmt, int op, int s_dtype, const GemmArgs& g, int max_rows, int sm_count,
                         int smem_optin, int w_align, cudaStream_t st) {
    (void)max_rows;
    if (g.x_dtype != GNF4B_X_BF16) return GNF4B_EUNSUPPORTED;      // the MMA runs bf16 x bf16
    TensorArgs ta;
    ta.g = g;
    ta.C = (op == GNF4B_OP_FWD) ? g.N : g.K;
    ta.R = (op == GNF4B_OP_FWD) ? g.K : g.N;
    if ((ta.R * 2) % 16) return GNF4B_EUNSUPPORTED;                // TMA row pitch must be a multiple of 16 bytes
    ta.c_tiles = (int32_t)((ta.C + kTBC - 1) / kTBC);
    ta.r_blocks = (int32_t)((ta.R + kTBR - 1) / kTBR);
    ta.w_align = w_align;
    int stages = kTMaxStages;
    while (stages > 2 && tensor_smem_bytes(fmt, stages) > (size_t)smem_optin) --stages;
    if (tensor_smem_bytes(fmt, stages) > (size_t)smem_optin) return GNF4B_EUNSUPPORTED;
    ta.stages = stages;
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return GNF4B_EUNSUPPORTED;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)ta.R, (cuuint64_t)g.T};
    const cuuint64_t strides[1] = {(cuuint64_t)ta.R * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTBR, (cuuint32_t)kTBM};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(g.x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return GNF4B_EUNSUPPORTED;
    const size_t smem = tensor_smem_bytes(fmt, stages);
#define GNF4B_T(F, S, O) return launch_tensor_t<F, S, O>(ta, map, sm_count, smem, st)
    if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32) {
        if (op == GNF4B_OP_FWD) GNF4B_T(GNF4B_FMT_NF4, GNF4B_S_F32, GNF4B_OP_FWD);
        GNF4B_T(GNF4B_FMT_NF4, GNF4B_S_F32, GNF4B_OP_DGRAD);
    }
    if (fmt == GNF4B_FMT_NF4) {
        if (op == GNF4B_OP_FWD) GNF4B_T(GNF4B_FMT_NF4, GNF4B_S_BF16, GNF4B_OP_FWD);
        GNF4B_T(GNF4B_FMT_NF4, GNF4B_S_BF16, GNF4B_OP_DGRAD);
    }
    if (op == GNF4B_OP_FWD) GNF4B_T(GNF4B_FMT_MXFP4, GNF4B_S_E8M0, GNF4B_OP_FWD);
    GNF4B_T(GNF4B_FMT_MXFP4, GNF4B_S_E8M0, GNF4B_OP_DGRAD);
#undef GNF4B_T
}

}  // namespace gnf4b
