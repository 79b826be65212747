// tcgen05 / TMEM grouped GEMM, forward only, weight tile resident in TENSOR MEMORY.
//
// The first tensor kernel (tensor_kernel.cuh) keeps both MMA operands in shared memory and is
// bound by shared-memory bandwidth: per k-step the MMAs read their operands, the decode warps
// read codebook entries and write hi/lo tiles, TMA writes activations -- all through the same
// 128 B/clk.  Here the decoded weights never touch shared memory:
//
//   out^T[n, t] = sum_k W[n, k] * x[t, k]      (accumulator lane = weight row n, column = token t)
//
//   operand A = decoded weight tile [128 n x 16 k] bf16 in TMEM, written by the decode warps with
//               tcgen05.st straight from registers (hi and, for NF4, lo = bf16(w - hi))
//   operand B = activation tile [<=256 tokens x 16 k] bf16, K-major, 128-byte swizzled, in
//               shared memory by TMA -- the only MMA operand read from shared memory
//   D         = fp32 [128 lanes x <=256 columns] in TMEM
//
// Roles (832 threads, one CTA per SM, persistent):
//   warp 0      TMA producer of activation tiles (two 128-row boxes per stage)
//   warp 1      MMA issuer (one lane): per stage 4 k-steps x (hi [, lo]) tcgen05.mma with A in TMEM
//   warps 2-9   epilogue, two per TMEM lane quarter taking alternate 32-token chunks: tcgen05.ld,
//               neighbour lanes exchange one value so each writes a bf16 pair, stores are 64-byte
//               coalesced along n (the output is transposed back here).  One warp needs ~700 cycles
//               per chunk (it is bound by its own instruction latency), the tensor pipe idles
//               until the last chunk is in registers: hence two warps per quarter
//   warps 10-25 decode, two groups of 8 warps that take alternate stages: thread = (weight row,
//               32 k): 16 packed bytes + one block scale from global memory (prefetched one own
//               stage = two pipeline stages ahead, across item boundaries), one table lookup per
//               byte, tcgen05.st of 16 columns (hi) + 16 columns (lo)
//
// TMEM budget (512 columns): 256 accumulator columns + 4 stages x 64 columns of A (hi 32 + lo 32).
// Work item = (group, balanced chunk of <= 256 rows, 128-column tile of N), column tile fastest.
// Barriers: one ring of 8 slots, full[s] (TMA bytes + one arrival per decode warp of the stage's group)
// and done[s] (tcgen05.commit: the stage's MMAs have completed, its two slots may be refilled); the
// accumulator is handed over with acc_full / acc_empty once per item.
//
// CG = 2 (optional): a cluster of two CTAs shares every item -- same row chunk, neighbouring column
// tiles; the leader issues tcgen05.mma.cta_group::2 for both, each CTA loads half of the activation
// tile and decodes its own weight tile, the peer's warps arrive on the leader's barriers remotely.
//
// What bounds it: issuing one tcgen05.mma occupies the issuing thread for 100-125 cycles whatever the
// shape, and NF4 needs two per k-step; a 64-k stage of 8 MMAs (1024 pipe cycles at N = 256) takes about
// 1450 cycles including that thread's barrier wait, fence and loop and the accumulator hand-over.
#pragma once

#include "tensor_kernel.cuh"

namespace gnf4b {

constexpr int kFStages = 4;                     // tensor-memory slots of decoded weights
constexpr int kFRing = 8;                       // barrier ring
constexpr int kFTok = 256;                     // tokens per item (UMMA N)
constexpr int kFXTile = kFTok * kTBR * 2;      // 32 KiB of activations per stage
constexpr int kFAcols = 64;                    // TMEM columns of A per stage (hi 32 + lo 32)
constexpr int kFEpiWarps = 8;                  // two per TMEM lane quarter, alternate 32-token chunks
constexpr int kFDecWarp0 = 2 + kFEpiWarps;     // first decode warp
constexpr int kFThreads = (2 + kFEpiWarps + 16) * 32;
constexpr int kFGroupBytes = 512 * 16 + 513 * 8 + 16 * 8 + 8;   // FGroup[512], base[513], warp totals[16]

// Lookup tables, one copy per lane so that no two lanes share a bank:
//   NF4   tab[byte][lane] float2 = codebook values of the byte's two elements (64 KiB)
//   MXFP4 tab[byte][lane] bf16x2 = doubled e2m1 values of the byte's two elements (32 KiB)
__host__ __device__ inline size_t tensor_fwd_table_bytes(int fmt) { return fmt == GNF4B_FMT_NF4 ? 65536 : 32768; }
__host__ __device__ inline size_t tensor_fwd_smem_bytes(int fmt) {
    return (size_t)kFStages * kFXTile + tensor_fwd_table_bytes(fmt) + kFGroupBytes + 1024 + 1024;
}

__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, "
                 "%13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- CTA-pair (cta_group::2) helpers.  A pair is a cluster of two CTAs on the two SMs of a TPC.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory location in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// Arrive on a barrier of the peer CTA.  Relaxed on purpose: a release at cluster scope costs a
// cluster-wide fence per arrival (measured: 25 % of the kernel's time), and nothing here publishes
// ordinary memory.  What the arrival announces is complete before it is issued -- tensor-memory
// stores behind tcgen05.wait::st and tcgen05.fence::before_thread_sync, accumulator reads behind
// tcgen05.wait::ld, a landed TMA copy observed on the local barrier -- and the waiter acquires at
// cluster scope and fences tcgen05 after it.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded like mbar_wait_bounded; acquires at cluster scope (the arrival came from the peer CTA)
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tcgen05.mma over the CTA pair: M = 256 (128 rows of A and D in each CTA's tensor memory),
// each CTA supplies half of B's rows from its own shared memory at the same offset
__device__ __forceinline__ void tc_mma_bf16_ts2(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive on a barrier (shared::cluster address, this CTA's or the peer's) when every MMA issued so far is done
__device__ __forceinline__ void tc_commit2(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}

struct FItem {
    int32_t row0;      // first row of the chunk
    int32_t tokens;    // rows in the chunk (1..256)
    int32_t eid;
    int32_t c0;        // first output column (weight row) of the tile
};

// The group table lives in shared memory: every role walks the item list, and the MMA issuer does
// so between two items with the tensor pipe idle -- a walk through global memory (three dependent
// loads per group, a dozen groups per step) cost it thousands of cycles per item.
constexpr int kFMaxGroups = 512;
struct FGroup {
    int32_t row0, rows, eid, chunk_rows;
};
struct FTable {
    const FGroup* grp;       // [G]
    const int64_t* base;     // [G + 1] items before group g
};
struct FCursor {
    int32_t g = 0;
};

// Item id -> (group, balanced row chunk, column tile); column tile fastest.
// `tiles` = column tiles (CG = 1) or column-tile pairs (CG = 2) per row chunk; `tile_mul`, `tile_add`
// turn the item's tile index into this CTA's 128-column tile.
__device__ __forceinline__ bool next_fitem(const TensorArgs& a, const FTable& tb, FCursor& cur, int64_t id, FItem* it,
                                           int32_t tiles, int32_t tile_mul, int32_t tile_add) {
    while (cur.g < a.g.G && id >= tb.base[cur.g + 1]) cur.g++;
    if (cur.g >= a.g.G) return false;
    const FGroup gr = tb.grp[cur.g];
    const int32_t local = (int32_t)(id - tb.base[cur.g]);
    const int32_t mc = local / tiles;
    const int32_t ct = local - mc * tiles;
    it->row0 = gr.row0 + mc * gr.chunk_rows;
    it->tokens = min(gr.chunk_rows, gr.row0 + gr.rows - it->row0);
    it->eid = gr.eid;
    it->c0 = (ct * tile_mul + tile_add) * kTBC;
    return true;
}

// Build the table: one thread per group, then a block-wide inclusive scan of the item counts.
// Groups with a bad expert id or bad offsets are flagged in the status word and get no items.
__device__ __forceinline__ void build_ftable(const TensorArgs& a, FGroup* grp, int64_t* base, int64_t* warp_tot,
                                             int32_t tiles) {
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    int64_t items = 0;
    if (t < a.g.G) {
        FGroup gr;
        gr.row0 = __ldg(a.g.off + t);
        gr.rows = __ldg(a.g.off + t + 1) - gr.row0;
        gr.eid = __ldg(a.g.eids + t);
        const bool bad_e = gr.eid < 0 || gr.eid >= a.g.E;
        const bool bad_o = gr.rows < 0 || gr.row0 < 0 || (int64_t)gr.row0 + gr.rows > a.g.T;
        const bool pad = gr.eid == GNF4B_PAD_EXPERT;     // padding group: skipped, not an error
        if (((bad_e && !pad) || bad_o) && gr.rows != 0 && a.g.status && blockIdx.x == 0)
            atomicOr(a.g.status, (bad_e && !pad) ? GNF4B_ST_BAD_EXPERT : GNF4B_ST_BAD_OFFSETS);
        const int32_t chunks = (bad_e || bad_o || gr.rows <= 0) ? 0 : (gr.rows + kFTok - 1) / kFTok;
        // equal chunks, a multiple of 16 rows each (the MMA's N granularity)
        gr.chunk_rows = chunks ? (((gr.rows + chunks - 1) / chunks + 15) & ~15) : 0;
        grp[t] = gr;
        items = (int64_t)chunks * tiles;
    }
    int64_t incl = items;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int64_t up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31 && w < kFMaxGroups / 32) warp_tot[w] = incl;
    __syncthreads();
    if (t < a.g.G) {
        int64_t before = 0;
        for (int v = 0; v < w; ++v) before += warp_tot[v];
        base[t + 1] = before + incl;
    }
    if (t == 0) base[0] = 0;
}

// 16 packed bytes (32 elements) of one weight row.
// A thread walks its weight row 16 bytes per own stage; on an L2 miss the load asks L2 for the whole
// 256 bytes around it, so the next stages of the row hit L2 instead of waiting on HBM each time (the
// register prefetch is only one own stage deep).
__device__ __forceinline__ uint4 load_packed16(const uint8_t* p, int w_align) {
    if (w_align >= 16) {
        uint4 v;
        asm volatile("ld.global.nc.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(p));
        return v;
    }
    const uint2 lo = load_packed8(p, w_align), hi = load_packed8(p + 8, w_align);
    return make_uint4(lo.x, lo.y, hi.x, hi.y);
}

// Decode the 8 elements of one packed word into 4 bf16x2 words of hi (and lo for NF4): per byte
// one table read, NF4 then scales in fp32 and splits hi = bf16(w), lo = bf16(w - hi); MXFP4
// multiplies the exact bf16 pair by the power-of-two scale (exact).  Same arithmetic as
// decode_store16 of tensor_kernel.cuh.
template <int FMT>
__device__ __forceinline__ void decode8_regs(const uint32_t w, float scale, uint32_t s2, uint32_t tab_lane,
                                             uint32_t* hi, uint32_t* lo) {
    uint64_t scale2;
    asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "r"(__float_as_uint(scale)));
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint32_t byte = (b == 0) ? (w & 0xffu) : (b == 3) ? (w >> 24) : prmt(w, 0u, 0x4440u | b);
        if (FMT == GNF4B_FMT_NF4) {
            // both elements of the byte at once with the packed fp32 pair instructions of sm_100 (the same IEEE
            // multiply and subtract per element, half the instructions)
            uint64_t pq, w2, r2;
            asm volatile("ld.shared.b64 %0, [%1];" : "=l"(pq) : "r"(tab_lane + (byte << 8)));
            asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(w2) : "l"(pq), "l"(scale2));
            uint32_t w0b, w1b;
            asm("mov.b64 {%0, %1}, %2;" : "=r"(w0b), "=r"(w1b) : "l"(w2));
            const uint32_t h = pack_bf16x2(__uint_as_float(w1b), __uint_as_float(w0b));
            hi[b] = h;
            uint64_t h2;
            asm("mov.b64 %0, {%1, %2};" : "=l"(h2) : "r"(h << 16), "r"(h & 0xffff0000u));
            asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r2) : "l"(w2), "l"(h2));
            uint32_t r0b, r1b;
            asm("mov.b64 {%0, %1}, %2;" : "=r"(r0b), "=r"(r1b) : "l"(r2));
            lo[b] = pack_bf16x2(__uint_as_float(r1b), __uint_as_float(r0b));
        } else {
            hi[b] = mul_bf16x2(ld_shared_u32(tab_lane + (byte << 7)), s2);
        }
    }
}

template <int FMT, int SDT, int CG>
__global__ void __launch_bounds__(kFThreads, 1)
tensor_fwd_kernel(const TensorArgs a, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tab_raw = smem + (size_t)kFStages * kFXTile;
    uint8_t* grp_raw = tab_raw + tensor_fwd_table_bytes(FMT);
    FGroup* s_grp = reinterpret_cast<FGroup*>(grp_raw);
    int64_t* s_base = reinterpret_cast<int64_t*>(grp_raw + kFMaxGroups * 16);
    int64_t* s_wtot = s_base + kFMaxGroups + 1;
    // full[s]: the stage's activations (TMA transaction bytes + the producer's arrival) and its decoded
    // weights (one arrival per decode warp of the group) are in place
    // One barrier ring of kFRing slots serves both pipelines; stage number seq uses slot seq % kFRing,
    // tensor-memory slot seq % kFStages for its decoded weights and shared-memory slot seq % XS for
    // its activations (XS = 4 tiles of 32 KiB, or 8 half tiles of 16 KiB in a CTA pair).
    //   full[slot]  activations landed (TMA bytes + the producer's arrival) and weights decoded
    //               (one arrival per decode warp); in a pair only the leader's is used and the
    //               peer's warps arrive on it remotely
    //   done[slot]  the stage's MMAs have completed: its two slots may be refilled
    //   x_local[slot]  peer CTA only: its own TMA landed (the relay forwards this to the leader)
    uint64_t* full = reinterpret_cast<uint64_t*>(grp_raw + kFGroupBytes);
    uint64_t* done = full + kFRing;
    uint64_t* x_local = done + kFRing;
    uint64_t* acc_full = x_local + kFRing;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // CG = 2: the two CTAs of a cluster share every item -- same row chunk, neighbouring column
    // tiles; rank 0 (the leader) issues the MMAs for both
    const uint32_t rank = (CG == 2) ? cluster_ctarank() : 0u;
    const int64_t worker = (CG == 2) ? (blockIdx.x >> 1) : blockIdx.x;
    const int64_t workers = (CG == 2) ? (gridDim.x >> 1) : gridDim.x;
    const int32_t tiles = (CG == 2) ? (a.c_tiles + 1) / 2 : a.c_tiles;
    constexpr uint32_t XS = (CG == 2) ? 8 : 4;                  // activation slots
    constexpr uint32_t kXBytes = (CG == 2) ? kTATile : kFXTile; // bytes per activation slot

    if (threadIdx.x == 0) {
        for (int s = 0; s < kFRing; ++s) {
            mbar_init(full + s, CG == 2 ? 2 * (1 + 8) : 1 + 8);
            mbar_init(done + s, 1);
            mbar_init(x_local + s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, kFEpiWarps * CG);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTTmemCols);
        tmem_relinquish();
    }
    if (FMT == GNF4B_FMT_NF4) {
        float2* tab = reinterpret_cast<float2*>(tab_raw);
        for (int i = threadIdx.x; i < 256 * 32; i += kFThreads) tab[i] = byte_pair<FMT>(i >> 5);
    } else {
        uint32_t* tab = reinterpret_cast<uint32_t*>(tab_raw);
        for (int i = threadIdx.x; i < 256 * 32; i += kFThreads) {
            const float2 p = byte_pair<FMT>(i >> 5);
            tab[i] = pack_bf16x2(p.y, p.x);
        }
    }
    build_ftable(a, s_grp, s_base, s_wtot, tiles);
    const FTable tb{s_grp, s_base};
    tc_fence_before();
    if (CG == 2) cluster_sync_all();      // the peer's barriers exist before anything arrives on them
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a0 = tmem_base + kFTok;          // A stages start after the 256 accumulator columns
    const int64_t scale_blk = (FMT == GNF4B_FMT_NF4) ? 64 : 32;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            FCursor cur;
            FItem it;
            uint32_t seq = 0;
            bool ok = true;
            for (int64_t id = worker; ok && next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank); id += workers) {
                // CG = 1: the whole chunk, two 128-row boxes when it has more than 128 rows.
                // CG = 2: this CTA's half of the MMA's N = round_up(tokens, 16) rows, one box.
                const int boxes = (CG == 1 && it.tokens > kTBM) ? 2 : 1;
                const int row_first = it.row0 + (CG == 2 ? (int)rank * (((it.tokens + 15) & ~15) >> 1) : 0);
                for (int rb = 0; rb < a.r_blocks && ok; ++rb, ++seq) {
                    if (seq >= XS) {             // the slot's previous stage has been multiplied
                        ok = mbar_wait_bounded(done + ((seq - XS) & (kFRing - 1)), ((seq - XS) / kFRing) & 1, abort_flag);
                        if (!ok) break;
                    }
                    uint8_t* st = smem + (size_t)(seq % XS) * kXBytes;
                    uint64_t* bar = ((CG == 2 && rank == 1) ? x_local : full) + (seq & (kFRing - 1));
                    mbar_arrive_expect_tx(bar, (uint32_t)(boxes * kTATile));
                    for (int b = 0; b < boxes; ++b)
                        tma_load_2d(st + b * kTATile, &x_map, rb * kTBR, row_first + b * kTBM, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            FCursor cur;
            FItem it;
            uint32_t seq = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t peer_done = (CG == 2) ? map_to_cta(smem_u32(done), 1) : 0u;
            const uint32_t peer_acc_full = (CG == 2) ? map_to_cta(smem_u32(acc_full), 1) : 0u;
            auto wait_full = [&](uint32_t q_) {
                uint64_t* bar = full + (q_ & (kFRing - 1));
                const uint32_t par = (q_ / kFRing) & 1;
                return (CG == 2) ? mbar_wait_bounded_cluster(bar, par, abort_flag) : mbar_wait_bounded(bar, par, abort_flag);
            };
            for (int64_t id = worker; ok && next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank); id += workers) {
                const uint32_t n_umma = (uint32_t)((it.tokens + 15) & ~15);
                // kind::f16: fp32 accumulate, bf16 x bf16, both K-major, M = 128 per CTA, N = n_umma
                const uint32_t idesc =
                    (1u << 4) | (1u << 7) | (1u << 10) | ((n_umma >> 3) << 17) | (((uint32_t)(kTBM * CG) >> 4) << 24);
                ok = (CG == 2) ? mbar_wait_bounded_cluster(acc_empty, acc_phase ^ 1, abort_flag)
                               : mbar_wait_bounded(acc_empty, acc_phase ^ 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                // Between the last MMA of a stage and the first of the next this thread does nothing but
                // address arithmetic: the tensor pipe keeps only a short queue, so every cycle spent
                // there on a barrier, a fence or a commit is a cycle the pipe idles.  Hence the wait
                // (and fence) for stage s + 1 sits before the last k-step of stage s, and the commit
                // of stage s after the first k-step of stage s + 1 (it then also covers that k-step,
                // which frees the slots of stage s one MMA later -- harmless).
                bool primed = false, pending = false;
                uint32_t pending_slot = 0;
                auto commit_done = [&](uint32_t slot) {
                    if (CG == 2) {
                        tc_commit2(smem_u32(done + slot));
                        tc_commit2(peer_done + slot * 8);
                    } else {
                        tc_commit(done + slot);
                    }
                };
                for (int rb = 0; rb < a.r_blocks && ok; ++rb, ++seq) {
                    if (!primed) {
                        ok = wait_full(seq);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    primed = false;
                    const uint32_t xs = smem_u32(smem + (size_t)(seq % XS) * kXBytes);
                    const uint32_t a_hi = tmem_a0 + (seq & (kFStages - 1)) * kFAcols;
#pragma unroll
                    for (int j = 0; j < kTBR / 16; ++j) {
                        if (j == kTBR / 16 - 1 && rb + 1 < a.r_blocks) {
                            ok = wait_full(seq + 1);
                            tc_fence_after();
                            primed = true;
                        }
                        const uint64_t db = umma_desc(xs + j * 32, 16, 1024);
                        const uint32_t acc = (rb > 0 || j > 0) ? 1u : 0u;
                        if (CG == 2) {
                            tc_mma_bf16_ts2(tmem_base, a_hi + j * 8, db, idesc, acc);
                            if (FMT == GNF4B_FMT_NF4) tc_mma_bf16_ts2(tmem_base, a_hi + 32 + j * 8, db, idesc, 1u);
                        } else {
                            tc_mma_bf16_ts(tmem_base, a_hi + j * 8, db, idesc, acc);
                            if (FMT == GNF4B_FMT_NF4) tc_mma_bf16_ts(tmem_base, a_hi + 32 + j * 8, db, idesc, 1u);
                        }
                        if (j == 0 && pending) {
                            commit_done(pending_slot);
                            pending = false;
                        }
                    }
                    pending = true;
                    pending_slot = seq & (kFRing - 1);
                }
                if (pending) commit_done(pending_slot);
                if (ok) {
                    if (CG == 2) {
                        tc_commit2(smem_u32(acc_full));
                        tc_commit2(peer_acc_full);
                    } else {
                        tc_commit(acc_full);
                    }
                }
                acc_phase ^= 1;
            }
        } else if (lane == 0 && CG == 2) {
            // -------------------------------------------------------- relay (rank 1): forward "my
            // activations have landed" to the leader's full barrier
            FCursor cur;
            FItem it;
            uint32_t seq = 0;
            bool ok = true;
            const uint32_t leader_full = map_to_cta(smem_u32(full), 0);
            for (int64_t id = worker; ok && next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank); id += workers) {
                for (int rb = 0; rb < a.r_blocks && ok; ++rb, ++seq) {
                    ok = mbar_wait_bounded(x_local + (seq & (kFRing - 1)), (seq / kFRing) & 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_cluster(leader_full + (seq & (kFRing - 1)) * 8);
                }
            }
        }
    } else if (warp < kFDecWarp0) {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;
        const int e = (warp - 2) >> 2;              // takes chunks e, e + 2, ...
        FCursor cur;
        FItem it;
        uint32_t acc_phase = 0;
        bool ok = true;
        uint16_t* out = reinterpret_cast<uint16_t*>(a.g.out);
        const uint32_t leader_acc_empty = (CG == 2) ? map_to_cta(smem_u32(acc_empty), 0) : 0u;
        auto release_acc = [&]() {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2) mbar_arrive_cluster(leader_acc_empty);
                else mbar_arrive(acc_empty);
            }
        };
        const bool pair_ok = (a.C % 2) == 0;
        for (int64_t id = worker; ok && next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank); id += workers) {
            ok = mbar_wait_bounded(acc_full, acc_phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const int64_t n = (int64_t)it.c0 + q * 32 + lane;          // this lane's output column
            const int chunks = (it.tokens + 31) >> 5;
            if (e >= chunks) release_acc();              // nothing to drain for this warp
            for (int c = e; c < chunks; c += 2) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), r);
                tmem_ld_wait();
                if (c + 2 >= chunks) release_acc();      // all this warp needs is in registers
                const int t0 = c * 32;
                if (pair_ok) {
                    // lanes 2i and 2i+1 swap one value: the even lane stores (n, n+1) of token j,
                    // the odd lane (n-1, n) of token j+1 -- 4-byte stores, 64 bytes per half warp
                    const int odd = lane & 1;
                    const int left = (n - odd < a.C) ? it.tokens - t0 - odd : 0;     // store while j < left
                    uint16_t* p = out + (int64_t)(it.row0 + t0 + odd) * a.C + (n - odd);
                    const int64_t step = 2 * a.C;
                    uint32_t v[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float mine0 = __uint_as_float(r[j]), mine1 = __uint_as_float(r[j + 1]);
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? mine0 : mine1, 1);
                        v[j >> 1] = odd ? pack_bf16x2(mine1, got) : pack_bf16x2(got, mine0);
                    }
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        if (j < left) *reinterpret_cast<uint32_t*>(p) = v[j >> 1];
                        p += step;
                    }
                } else {
                    const int left = (n < a.C) ? it.tokens - t0 : 0;
                    uint16_t* p = out + (int64_t)(it.row0 + t0) * a.C + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < left) *p = f32_to_bf16_bits(__uint_as_float(r[j]));
                        p += a.C;
                    }
                }
            }
            acc_phase ^= 1;
        }
    } else {
        // ------------------------------------------------------------ weight decode -> TMEM
        const int dw = warp - kFDecWarp0;
        const int grp = dw >> 3;                   // this group takes pipeline stages grp, grp + 2, ...
        const int hf = (dw >> 2) & 1;              // which 32 k of the stage's 64
        const int q = warp & 3;                    // TMEM lane quarter this warp may write
        const int n_local = q * 32 + lane;
        const uint32_t tab_lane = smem_u32(tab_raw) + lane * (FMT == GNF4B_FMT_NF4 ? 8 : 4);
        const uint32_t col0 = tmem_a0 + ((uint32_t)(q * 32) << 16) + hf * 16;
        // the fetch cursor runs one own stage ahead of the stage being decoded and crosses items
        FCursor cur;
        FItem it;
        int64_t id = worker;
        bool have = next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank);
        int rb = grp;
        uint4 pk_n = make_uint4(0, 0, 0, 0);
        float sc_n = 0.f;
        auto settle = [&]() {                      // bring (it, rb) to the next existing stage
            while (have && rb >= a.r_blocks) {
                rb -= a.r_blocks;
                id += workers;
                have = next_fitem(a, tb, cur, id, &it, tiles, CG, (int32_t)rank);
            }
        };
        auto fetch = [&]() {
            const int64_t n = (int64_t)it.c0 + n_local;
            const int64_t k = (int64_t)rb * kTBR + hf * 32;
            if (n < a.g.N && k < a.g.K) {
                pk_n = load_packed16(a.g.W + (int64_t)it.eid * a.g.w_se + n * a.g.w_sn + (k >> 1), a.w_align);
                sc_n = load_scale<SDT>(a.g.S, (int64_t)it.eid * a.g.s_se + n * a.g.s_sn + k / scale_blk);
            } else {
                pk_n = make_uint4(0, 0, 0, 0);
                sc_n = 0.f;                        // padding decodes to zeros
            }
        };
        settle();
        if (have) fetch();
        uint32_t seq = grp;
        bool ok = true;
        const uint32_t leader_full = (CG == 2) ? map_to_cta(smem_u32(full), 0) : 0u;
        while (have && ok) {
            const uint4 pk = pk_n;
            const float sc = sc_n;
            rb += 2;
            settle();
            if (have) fetch();
            const bool more = have;
            if (seq >= kFStages)             // the tensor-memory slot's previous stage has been multiplied
                ok = mbar_wait_bounded(done + ((seq - kFStages) & (kFRing - 1)), ((seq - kFStages) / kFRing) & 1, abort_flag);
            if (ok) {
                const uint32_t s16 = __float_as_uint(sc) >> 16;
                const uint32_t s2 = s16 | (s16 << 16);
                const uint32_t col = col0 + (seq & (kFStages - 1)) * kFAcols;
                const uint32_t w4[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t hi[8], lo[8];
                    decode8_regs<FMT>(w4[2 * h], sc, s2, tab_lane, hi, lo);
                    decode8_regs<FMT>(w4[2 * h + 1], sc, s2, tab_lane, hi + 4, lo + 4);
                    tmem_st8(col + h * 8, hi);
                    if (FMT == GNF4B_FMT_NF4) tmem_st8(col + 32 + h * 8, lo);
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (CG == 2) mbar_arrive_cluster(leader_full + (seq & (kFRing - 1)) * 8);
                    else mbar_arrive(full + (seq & (kFRing - 1)));
                }
                seq += 2;
            }
            have = more;
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    // CG = 2: neither CTA may free its tensor memory or leave while the pair's MMAs can still read it
    if (CG == 2) cluster_sync_all();
    else __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, kTTmemCols);
    }
    if (threadIdx.x == 0 && *abort_flag && a.g.status) atomicOr(a.g.status, GNF4B_ST_TIMEOUT);
}

template <int FMT, int SDT, int CG>
static int launch_tensor_fwd_t(const TensorArgs& ta, const CUtensorMap& map, int sm_count, size_t smem, cudaStream_t st) {
    auto kfn = tensor_fwd_kernel<FMT, SDT, CG>;
    static int granted[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GNF4B_ECUDA;
    dev &= 63;
    if ((int)smem > granted[dev]) {
        if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GNF4B_ECUDA;
        granted[dev] = (int)smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(CG == 2 ? (sm_count & ~1) : sm_count));
    cfg.blockDim = dim3(kFThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kfn, ta, map) != cudaSuccess) return GNF4B_ECUDA;
    return GNF4B_OK;
}

template <int CG>
static int launch_tensor_fwd_cg(int fmt, int s_dtype, const TensorArgs& ta, const CUtensorMap& map, int sm_count,
                                size_t smem, cudaStream_t st) {
    if (fmt == GNF4B_FMT_NF4 && s_dtype == GNF4B_S_F32)
        return launch_tensor_fwd_t<GNF4B_FMT_NF4, GNF4B_S_F32, CG>(ta, map, sm_count, smem, st);
    if (fmt == GNF4B_FMT_NF4)
        return launch_tensor_fwd_t<GNF4B_FMT_NF4, GNF4B_S_BF16, CG>(ta, map, sm_count, smem, st);
    return launch_tensor_fwd_t<GNF4B_FMT_MXFP4, GNF4B_S_E8M0, CG>(ta, map, sm_count, smem, st);
}

// Forward with the weight tile in tensor memory.  Same preconditions as launch_tensor.
// `pair` = run as CTA pairs (cta_group::2 MMAs, each CTA loads half of the activation tile).
static int launch_tensor_fwd(int fmt, int s_dtype, const GemmArgs& g, int sm_count, int smem_optin, int w_align,
                             bool pair, cudaStream_t st) {
    if (g.x_dtype != GNF4B_X_BF16) return GNF4B_EUNSUPPORTED;
    TensorArgs ta;
    ta.g = g;
    ta.C = g.N;
    ta.R = g.K;
    if ((ta.R * 2) % 16 || g.G > kFMaxGroups) return GNF4B_EUNSUPPORTED;
    ta.c_tiles = (int32_t)((ta.C + kTBC - 1) / kTBC);
    ta.r_blocks = (int32_t)((ta.R + kTBR - 1) / kTBR);
    ta.w_align = w_align;
    ta.stages = kFStages;
    const size_t smem = tensor_fwd_smem_bytes(fmt);
    if (smem > (size_t)smem_optin) return GNF4B_EUNSUPPORTED;
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
    if (pair && sm_count >= 2) return launch_tensor_fwd_cg<2>(fmt, s_dtype, ta, map, sm_count, smem, st);
    return launch_tensor_fwd_cg<1>(fmt, s_dtype, ta, map, sm_count, smem, st);
}

}  // namespace gnf4b
