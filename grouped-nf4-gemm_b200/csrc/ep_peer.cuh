// Small-batch expert-parallel exchange without a collective library and without a memory fence: every rank writes
// the rows it routes to a peer straight into that peer's exchange buffer over NVLink, each 8 bytes carrying 4 bytes
// of payload and the 4-byte number of the current step.  An 8-byte store is delivered whole, so a reader that finds
// the step number it expects has the payload beside it: no fence on the writer's side (a system-scope fence costs
// microseconds), no separate flag, one NVLink traversal of latency.  The price is twice the bytes, which at these
// sizes (tens of KB per rank) is nothing.  Two kernels per layer around the grouped GEMMs, each of which first sends
// and then receives (so no rank waits before it has sent, and the waits cannot form a cycle):
//
//   dispatch   SEND: routing plan (as ep_plan_kernel); rows and per-expert counts into the destinations' buffers.
//              RECEIVE: waits for every source's counts, orders the announced rows expert-major (all rows of a local
//              expert next to each other, whatever their source), waits for them and unpacks them into that order in
//              a plain row matrix; writes the group tables of the GEMMs and the map back to (source, row).
//   combine    SEND: result rows back into the sources' buffers, and one word to EVERY rank ("this rank has consumed
//              what you sent this step").  RECEIVE: waits for that word from every rank and for the rows it expects,
//              routing-weight sum (the arithmetic of combine_rows_kernel).
//
// One buffer per rank, the same layout everywhere (ep_peer_layout), one set of row slots.  That is enough because the
// steps interlock: a rank starts dispatch n + 1 only after its combine n heard from every peer's combine n, whose
// sending half follows that peer's dispatch n, which has read everything sent to it in step n; a peer's combine
// n + 1 follows its dispatch n + 1, which needs this rank's dispatch n + 1 and so this rank's combine n.  Each kernel
// keeps its own step number in the rank's buffer (all ranks make the same calls, so the numbers agree), so a
// captured sequence of launches can be replayed as it is.
//
// Both kernels are launched with programmatic stream serialization: each lets its successor start at once
// (pdl_launch_dependents) and touches nothing before pdl_wait(), so launch latencies overlap along the chain.  Their
// code is kept small (waits out of line, loops rolled): a kernel that runs for two microseconds once per layer pays
// for every instruction-cache line it has to fetch.
// No multicast, no multimem: unicast stores and loads only.  Every wait is bounded (kEpPeerWaitNs); when it runs
// out the kernel raises GNF4B_ST_TIMEOUT and goes on with what is there (stale rows, never a bad address).
#pragma once

#include "common.cuh"
#include "ep_kernels.cuh"

namespace gnf4b {

constexpr int kEpPeerMaxWorld = 16;
constexpr int kEpPeerThreads = 256;
constexpr int kEpOffsetsThreads = 128;
constexpr int kEpPeerMaxRows = 1024;      // world * cap: the placement tables live in shared memory
constexpr unsigned long long kEpPeerWaitNs = 2000000000ull;     // 2 s

struct EpPeerLayout {
    int64_t local;               // uint32[8], this rank only: step numbers of the two kernels [0..1], their finished-CTA counters [4..5]
    int64_t ret_word;            // uint2[kEpPeerMaxWorld]: {1, step} from every rank's combine kernel
    int64_t used;                // int32[kEpPeerMaxWorld], this rank only: rows received from every source this step
    int64_t counts;              // uint2[world * e_local]: {rows, step} per (source, local expert)
    int64_t row_map;             // int32[world * cap_max], this rank only: row of the matrix that holds (source, row of its block)
    int64_t recv_rows;           // bf16[world * cap_max * H], this rank only: the received rows unpacked, source-major
    int64_t recv_ll;             // received rows, 8 bytes per 4 bytes of row, source-major
    int64_t ret_ll;              // returned result rows, same form, destination-major
    int64_t total;
};

__host__ __device__ inline EpPeerLayout ep_peer_layout(int32_t world, int32_t e_local, int32_t cap_max, int64_t H) {
    EpPeerLayout L;
    L.local = 0;
    L.ret_word = 64;
    L.used = 192;
    L.counts = 256;
    const int64_t cnt_bytes = ((int64_t)world * e_local * 8 + 255) / 256 * 256;
    L.row_map = L.counts + cnt_bytes;
    L.recv_rows = L.row_map + ((int64_t)world * cap_max * 4 + 255) / 256 * 256;
    const int64_t row_bytes = ((int64_t)world * cap_max * H * 2 + 255) / 256 * 256;
    L.recv_ll = L.recv_rows + row_bytes;
    L.ret_ll = L.recv_ll + 2 * row_bytes;
    L.total = L.ret_ll + 2 * row_bytes;
    return L;
}

struct EpPeerCtx {
    int32_t world, rank, e_local, cap_max;
    int64_t H;
    uint8_t* peers[kEpPeerMaxWorld];      // exchange buffer of every rank as this GPU addresses it
};

__device__ __forceinline__ uint4 ld_volatile_16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_volatile_8(const void* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_16(void* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_volatile_8(void* p, uint2 v) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// The waits, out of line.  {payload, step} once the step number is there; false in `ok` when the limit ran out.
// The first polls follow each other directly (over NVLink the payload is normally a few microseconds away); after
// that the thread sleeps between polls and looks at the clock now and then -- reading the global timer is itself
// slow, so it stays out of the common case.
__device__ __noinline__ uint2 ep_peer_wait8(const void* p, uint32_t step, bool* ok) {
    uint2 v = ld_volatile_8(p);
    uint64_t t0 = 0;
    for (uint32_t it = 0; v.y != step && it < (1u << 28); ++it) {
        if (it >= 64) {
            __nanosleep(100);
            if (it == 64) t0 = global_timer_ns();
            else if ((it & 255) == 0 && global_timer_ns() - t0 > kEpPeerWaitNs) break;
        }
        v = ld_volatile_8(p);
    }
    if (v.y != step) *ok = false;
    return v;
}
__device__ __noinline__ uint4 ep_peer_wait16(const void* p, uint32_t step, bool* ok) {
    uint4 v = ld_volatile_16(p);
    uint64_t t0 = 0;
    for (uint32_t it = 0; (v.y != step || v.w != step) && it < (1u << 28); ++it) {
        if (it >= 64) {
            __nanosleep(100);
            if (it == 64) t0 = global_timer_ns();
            else if ((it & 255) == 0 && global_timer_ns() - t0 > kEpPeerWaitNs) break;
        }
        v = ld_volatile_16(p);
    }
    if (v.y != step || v.w != step) *ok = false;
    return v;
}
// `ok` is sticky: after one wait has run out in this thread the later ones take what is there.
__device__ __forceinline__ uint2 ep_peer_poll8(const void* p, uint32_t step, bool& ok) {
    const uint2 v = ld_volatile_8(p);
    return (v.y == step || !ok) ? v : ep_peer_wait8(p, step, &ok);
}
__device__ __forceinline__ uint4 ep_peer_settle16(uint4 v, const void* p, uint32_t step, bool& ok) {
    return ((v.y == step && v.w == step) || !ok) ? v : ep_peer_wait16(p, step, &ok);
}

// The step number of kernel `which` (0 dispatch, 1 combine) for this launch; never 0, so a zeroed buffer matches
// no step.
__device__ __forceinline__ uint32_t ep_peer_step(const uint32_t* local, int which) {
    const uint32_t s = __ldcv(local + which) + 1u;
    return s == 0u ? 1u : s;
}
// The last CTA of the grid to get here records the step as done (nothing else of this launch reads it any more).
__device__ __forceinline__ void ep_peer_step_done(uint32_t* local, int which, uint32_t step) {
    __syncthreads();
    if (threadIdx.x != 0) return;
    if (gridDim.x > 1) {
        const uint32_t prev = atomicAdd(local + 4 + which, 1u);
        if (prev != gridDim.x - 1) return;
        local[4 + which] = 0;
    }
    local[which] = step;
}

// 8 bf16 of a row (16 bytes) -> 32 bytes at q in the peer's buffer
__device__ __forceinline__ void ep_peer_put_row16(uint8_t* q, uint4 d, uint32_t step) {
    st_volatile_16(q, make_uint4(d.x, step, d.y, step));
    st_volatile_16(q + 16, make_uint4(d.z, step, d.w, step));
}

// Source of the q-th row when the sources' rows are numbered through in rank order (first[s] = rows before s).
__device__ __forceinline__ int ep_peer_source_of(const int32_t* first, int world, int32_t q) {
    int s = 0;
#pragma unroll 1
    while (s + 1 < world && q >= first[s + 1]) ++s;
    return s;
}

// Group offsets of a received fixed-capacity buffer whose counts came through a collective (recv_counts[world,
// e_local] in this GPU's memory): per source its e_local expert blocks and the unused capacity as one padding group,
// world * (e_local + 1) + 1 offsets.  The counts are fetched by all threads at once (a serial loop of loads costs a
// memory round trip each); counts that do not fit the capacity are clamped and flagged.
__global__ void __launch_bounds__(kEpOffsetsThreads, 1)
ep_offsets_kernel(const int32_t* __restrict__ recv_counts, int32_t world, int32_t e_local, int32_t cap,
                  int32_t* __restrict__ offsets, int32_t* status) {
    __shared__ int32_t s_cnt[kEpPlanMax];
    for (int i = threadIdx.x; i < world * e_local; i += blockDim.x) s_cnt[i] = __ldg(recv_counts + i);
    __syncthreads();
    if (threadIdx.x != 0) return;
    int32_t off = 0, g = 0;
    bool bad = false;
    offsets[0] = 0;
    for (int s = 0; s < world; ++s) {
        int32_t used = 0;
        for (int e = 0; e < e_local; ++e) {
            int32_t c = s_cnt[s * e_local + e];
            if (c < 0 || used + c > cap) {
                bad = true;
                c = c < 0 ? 0 : cap - used;
            }
            used += c;
            off += c;
            offsets[++g] = off;
        }
        off += cap - used;
        offsets[++g] = off;
    }
    if (bad && status) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
}

// dispatch.  SEND: the plan in every CTA (P <= 1024 pairs, the same result in each); CTA 0 writes the slots
// (slot[p] = d * cap + row inside rank d's block, -1: not sent) and the counts, all CTAs copy their share of the
// rows.  RECEIVE: every CTA waits for all sources' counts and derives the same placement from them in shared memory:
// the rows of local expert e from all sources are consecutive, experts ascending, sources in rank order inside an
// expert, a source's rows of one expert in the order it sent them.  CTA 0 writes the tables:
//   one_row = 0   offsets[e_local + 1] (rows per local expert; the caller's expert ids are 0 .. e_local - 1)
//   one_row = 1   every row is its own group: offsets[g] = min(g, rows), eids[g] = the row's expert or
//                 GNF4B_PAD_EXPERT beyond the rows, for g < n_groups (the caller's world * cap).  Batches of a few
//                 rows, where no two rows share an expert often enough to matter and the one-row kernels are faster.
//   row_map[s * cap + j] = the matrix row of the j-th row source s sent, used[s] = its rows (this rank's buffer,
//   read by combine).
// Then the rows are awaited and unpacked to their places, 32 bytes of the buffer into 16 bytes of the matrix per
// thread and step, shared among the CTAs.  world * cap <= kEpPeerMaxRows.
__global__ void __launch_bounds__(kEpPeerThreads, 1)
ep_peer_dispatch_kernel(EpPeerCtx cx, const int64_t* __restrict__ idx, int32_t P, int32_t k, int32_t n_experts, int32_t cap,
                        const uint16_t* __restrict__ hidden, int64_t* __restrict__ slot, int32_t one_row, int32_t n_groups,
                        int32_t* __restrict__ offsets, int32_t* __restrict__ eids, int32_t* status) {
    __shared__ int32_t s_e[kEpPlanMax];          // send: expert of pair p.  receive: rows per (source, expert), then first row
    __shared__ int32_t s_hist[kEpPlanMax + 1];   // send: pairs per expert.  receive: first matrix row of local expert e
    __shared__ int32_t s_base[kEpPlanMax];       // send: pairs of lower experts on the same rank.  receive: s_map
    __shared__ int32_t s_slot[kEpPlanMax];       // send: row inside the destination's block, -1: not sent
    __shared__ int32_t s_first[kEpPeerMaxWorld + 1];
    __shared__ int32_t s_bad;
    const EpPeerLayout L = ep_peer_layout(cx.world, cx.e_local, cx.cap_max, cx.H);
    uint8_t* mine = cx.peers[cx.rank];
    uint32_t* local = reinterpret_cast<uint32_t*>(mine + L.local);
    const int t = threadIdx.x;
    const int W = cx.world, El = cx.e_local;
    const bool lead = blockIdx.x == 0;
    const int64_t H = cx.H, per_row = H / 8;     // H % 8 == 0 is checked by the host entry
    EPT(10);
    pdl_launch_dependents();
    pdl_wait();
    EPT(11);
    const uint32_t step = ep_peer_step(local, 0);
    // ------------------------------------------------------------------ send
#pragma unroll 1
    for (int e = t; e < n_experts; e += kEpPeerThreads) s_hist[e] = 0;
    if (t == 0) s_bad = 0;
    __syncthreads();
#pragma unroll 1
    for (int p = t; p < P; p += kEpPeerThreads) {
        const int64_t e = idx[p];
        const bool ok = e >= 0 && e < n_experts;
        s_e[p] = ok ? (int32_t)e : -1;
        if (ok) atomicAdd(&s_hist[e], 1);
        else if (status && lead) atomicOr(status, GNF4B_ST_BAD_EXPERT);
    }
    __syncthreads();
#pragma unroll 1
    for (int e = t; e < n_experts; e += kEpPeerThreads) {
        int32_t b = 0;
#pragma unroll 1
        for (int q = (e / El) * El; q < e; ++q) b += s_hist[q];
        s_base[e] = b;
        if (lead) {
            // rows of this expert that fit the capacity: the receiver lays its groups out from these
            int32_t n = s_hist[e];
            if (b + n > cap) n = b < cap ? cap - b : 0;
            st_volatile_8(cx.peers[e / El] + L.counts + (int64_t)(cx.rank * El + (e % El)) * 8, make_uint2((uint32_t)n, step));
        }
    }
    __syncthreads();
#pragma unroll 1
    for (int p = t; p < P; p += kEpPeerThreads) {
        const int32_t e = s_e[p];
        int32_t s = -1;
        if (e >= 0) {
            int32_t rank = 0;
#pragma unroll 1
            for (int q = 0; q < p; ++q) rank += (s_e[q] == e);
            if (s_base[e] + rank < cap) s = s_base[e] + rank;
            else if (status && lead) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
        }
        s_slot[p] = s;
        if (lead) slot[p] = s < 0 ? -1 : (int64_t)(e / El) * cap + s;
    }
    __syncthreads();
#pragma unroll 1
    for (int64_t i = (int64_t)blockIdx.x * kEpPeerThreads + t; i < (int64_t)P * per_row; i += (int64_t)gridDim.x * kEpPeerThreads) {
        const int p = (int)(i / per_row);
        const int64_t c = (i - (int64_t)p * per_row) * 8;
        if (s_slot[p] < 0) continue;
        uint8_t* dst = cx.peers[s_e[p] / El] + L.recv_ll + (((int64_t)cx.rank * cap + s_slot[p]) * H + c) * 4;
        ep_peer_put_row16(dst, __ldg(reinterpret_cast<const uint4*>(hidden + (int64_t)(p / k) * H + c)), step);
    }
    EPT(12);
    __syncthreads();                    // the plan's tables are done with: the placement reuses them
    // --------------------------------------------------------------- receive
    int32_t* s_cnt = s_e;
    int32_t* s_estart = s_hist;
    int32_t* s_map = s_base;
    bool ok = true;
#pragma unroll 1
    for (int i = t; i < W * El; i += kEpPeerThreads)
        s_cnt[i] = (int32_t)ep_peer_poll8(mine + L.counts + (int64_t)i * 8, step, ok).x;
    __syncthreads();
    if (t < W) {
        // rows of source t; counts are never trusted beyond the capacity
        int32_t used = 0;
#pragma unroll 1
        for (int e = 0; e < El; ++e) {
            int32_t c = s_cnt[t * El + e];
            if (c < 0 || used + c > cap) {
                s_bad = 1;
                c = c < 0 ? 0 : cap - used;
                s_cnt[t * El + e] = c;
            }
            used += c;
        }
        s_first[t + 1] = used;
    }
    __syncthreads();
    // rows per expert over all sources; then (one warp) the first row of every expert and of every source
#pragma unroll 1
    for (int e = t; e < El; e += kEpPeerThreads) {
        int32_t n = 0;
#pragma unroll 1
        for (int s = 0; s < W; ++s) n += s_cnt[s * El + e];
        s_estart[e + 1] = n;
    }
    __syncthreads();
    if (t < 32) {
        int32_t carry = 0;
        if (t == 0) s_estart[0] = 0;
#pragma unroll 1
        for (int base = 0; base < El; base += 32) {
            const int e = base + t;
            int32_t n = e < El ? s_estart[e + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int32_t u = __shfl_up_sync(0xffffffffu, n, o);
                if (t >= o) n += u;
            }
            if (e < El) s_estart[e + 1] = carry + n;
            carry += __shfl_sync(0xffffffffu, n, 31);
        }
        int32_t u = t < W ? s_first[t + 1] : 0;          // W <= 16: one pass
        const int32_t mine_u = u;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t v = __shfl_up_sync(0xffffffffu, u, o);
            if (t >= o) u += v;
        }
        __syncwarp();
        if (t < W) s_first[t] = u - mine_u;
        if (t == W - 1) s_first[W] = u;
    }
    __syncthreads();
    const int32_t n_rows = s_first[W];
    // block (s, e): its first matrix row (the expert's start plus the rows of lower sources) and the place of its
    // rows in source s's block (the rows of s's lower experts); one thread per block
#pragma unroll 1
    for (int i = t; i < W * El; i += kEpPeerThreads) {
        const int s = i / El, e = i - s * El;
        const int32_t c = s_cnt[i];
        if (c == 0) continue;
        int32_t at = s_estart[e], j0 = 0;
#pragma unroll 1
        for (int q = 0; q < s; ++q) at += s_cnt[q * El + e];
#pragma unroll 1
        for (int q = 0; q < e; ++q) j0 += s_cnt[s * El + q];
#pragma unroll 1
        for (int32_t r = 0; r < c; ++r) s_map[s * cap + j0 + r] = at + r;
        if (lead && one_row)
#pragma unroll 1
            for (int32_t r = 0; r < c; ++r)
                if (at + r < n_groups) eids[at + r] = e;
    }
    __syncthreads();
    EPT(22);
    if (lead) {
        int32_t* row_map = reinterpret_cast<int32_t*>(mine + L.row_map);
        if (t < W) reinterpret_cast<int32_t*>(mine + L.used)[t] = s_first[t + 1] - s_first[t];
#pragma unroll 1
        for (int q = t; q < n_rows; q += kEpPeerThreads) {
            const int s = ep_peer_source_of(s_first, W, q);
            const int32_t j = q - s_first[s];
            row_map[s * cap + j] = s_map[s * cap + j];
        }
        if (one_row) {
#pragma unroll 1
            for (int g = t; g <= n_groups; g += kEpPeerThreads) offsets[g] = min(g, n_rows);
#pragma unroll 1
            for (int g = n_rows + t; g < n_groups; g += kEpPeerThreads) eids[g] = GNF4B_PAD_EXPERT;
        } else {
#pragma unroll 1
            for (int e = t; e <= El; e += kEpPeerThreads) offsets[e] = s_estart[e];
        }
        if (t == 0 && s_bad && status) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
    }
    uint16_t* rows = reinterpret_cast<uint16_t*>(mine + L.recv_rows);
#pragma unroll 1
    for (int64_t i = (int64_t)blockIdx.x * kEpPeerThreads + t; i < (int64_t)n_rows * per_row; i += (int64_t)gridDim.x * kEpPeerThreads) {
        const int32_t q = (int32_t)(i / per_row);
        const int64_t c = (i - (int64_t)q * per_row) * 8;
        const int s = ep_peer_source_of(s_first, W, q);
        const int32_t j = q - s_first[s];
        const uint8_t* src = mine + L.recv_ll + (((int64_t)s * cap + j) * H + c) * 4;
        uint4 a, b;
        bool both = false;
#pragma unroll 1
        for (int attempt = 0; attempt < 64 && !both; ++attempt) {
            a = ld_volatile_16(src);
            b = ld_volatile_16(src + 16);
            both = a.y == step && a.w == step && b.y == step && b.w == step;
        }
        if (!both) {
            a = ep_peer_settle16(a, src, step, ok);
            b = ep_peer_settle16(b, src + 16, step, ok);
        }
        *reinterpret_cast<uint4*>(rows + (int64_t)s_map[s * cap + j] * H + c) = make_uint4(a.x, a.z, b.x, b.z);
    }
    if (!ok && status) atomicOr(status, GNF4B_ST_TIMEOUT);
    ep_peer_step_done(local, 0, step);
    EPT(13);
}

// combine.  SEND: result row row_map[s * cap + j] of y goes back to rank s as the j-th row of block `rank` of its
// return slots (used[s] rows, both as this rank's dispatch left them); every rank gets the word that says this rank
// is through with what it received this step.  RECEIVE: every CTA waits for that word from every rank, then
// out[m, :] = bf16( sum_j w[m, j] * returned[slot[m, j], :] ) with the arithmetic of combine_rows_kernel<8>, the
// loads of four choices in flight together and each 16 bytes of a returned row awaited where it is read.
__global__ void __launch_bounds__(kEpPeerThreads, 1)
ep_peer_combine_kernel(EpPeerCtx cx, int32_t cap, const uint16_t* __restrict__ y, const int64_t* __restrict__ slot,
                       const float* __restrict__ w, int32_t k, int64_t M, uint16_t* __restrict__ out, int32_t* status) {
    __shared__ int32_t s_first[kEpPeerMaxWorld + 1];
    const EpPeerLayout L = ep_peer_layout(cx.world, cx.e_local, cx.cap_max, cx.H);
    uint8_t* mine = cx.peers[cx.rank];
    uint32_t* local = reinterpret_cast<uint32_t*>(mine + L.local);
    const int64_t H = cx.H, per_row = H / 8, Pmax = (int64_t)cx.world * cap;
    EPT(40);
    pdl_launch_dependents();
    pdl_wait();
    EPT(41);
    const uint32_t step = ep_peer_step(local, 1);
    // ------------------------------------------------------------------ send
    if (threadIdx.x == 0) {
        const int32_t* used = reinterpret_cast<const int32_t*>(mine + L.used);
        int32_t n = 0;
#pragma unroll 1
        for (int s = 0; s < cx.world; ++s) {
            s_first[s] = n;
            n += min(max(__ldg(used + s), 0), cap);
        }
        s_first[cx.world] = n;
    }
    if (blockIdx.x == 0 && (int)threadIdx.x < cx.world)
        st_volatile_8(cx.peers[threadIdx.x] + L.ret_word + (int64_t)cx.rank * 8, make_uint2(1u, step));
    __syncthreads();
    const int32_t* row_map = reinterpret_cast<const int32_t*>(mine + L.row_map);
#pragma unroll 1
    for (int64_t i = (int64_t)blockIdx.x * kEpPeerThreads + threadIdx.x; i < (int64_t)s_first[cx.world] * per_row;
         i += (int64_t)gridDim.x * kEpPeerThreads) {
        const int32_t q = (int32_t)(i / per_row);
        const int64_t c = (i - (int64_t)q * per_row) * 8;
        const int s = ep_peer_source_of(s_first, cx.world, q);
        const int32_t j = q - s_first[s];
        const int32_t r = __ldg(row_map + s * cap + j);
        uint8_t* dst = cx.peers[s] + L.ret_ll + (((int64_t)cx.rank * cap + j) * H + c) * 4;
        ep_peer_put_row16(dst, __ldg(reinterpret_cast<const uint4*>(y + (int64_t)r * H + c)), step);
    }
    EPT(42);
    // --------------------------------------------------------------- receive
    bool ok = true;
    if ((int)threadIdx.x < cx.world) ep_peer_poll8(mine + L.ret_word + (int64_t)threadIdx.x * 8, step, ok);
    __syncthreads();
    const uint8_t* rows = mine + L.ret_ll;
#pragma unroll 1
    for (int64_t i = (int64_t)blockIdx.x * kEpPeerThreads + threadIdx.x; i < M * per_row; i += (int64_t)gridDim.x * kEpPeerThreads) {
        const int64_t m = i / per_row, c = (i - m * per_row) * 8;
        float acc[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] = 0.f;
#pragma unroll 1
        for (int j0 = 0; j0 < k; j0 += 4) {
            int64_t p[4];
            float wj[4];
            uint4 a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                p[u] = (j0 + u < k) ? __ldg(slot + m * k + j0 + u) : -1;
                wj[u] = (j0 + u < k) ? __ldg(w + m * k + j0 + u) : 0.f;
            }
            // all eight loads go out together and are repeated together until every word carries the step (a word
            // that is late costs one more round of loads for the batch, not a round trip of its own)
            bool all = false;
#pragma unroll 1
            for (int attempt = 0; attempt < 64 && !all; ++attempt) {
                all = true;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool have = p[u] >= 0 && p[u] < Pmax;
                    const uint8_t* src = rows + ((have ? p[u] : 0) * H + c) * 4;
                    a[u] = ld_volatile_16(src);
                    b[u] = ld_volatile_16(src + 16);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (p[u] >= 0 && p[u] < Pmax)
                        all = all && a[u].y == step && a[u].w == step && b[u].y == step && b[u].w == step;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (j0 + u >= k) continue;
                if (p[u] < 0 || p[u] >= Pmax) {
                    if (status) atomicOr(status, GNF4B_ST_BAD_OFFSETS);
                    continue;
                }
                if (!all) {         // still missing after the quick rounds: the bounded wait, word by word
                    const uint8_t* src = rows + (p[u] * H + c) * 4;
                    a[u] = ep_peer_settle16(a[u], src, step, ok);
                    b[u] = ep_peer_settle16(b[u], src + 16, step, ok);
                }
                const uint32_t rw[4] = {a[u].x, a[u].z, b[u].x, b[u].z};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(__uint_as_float(rw[q] << 16), wj[u]));
                    acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(__uint_as_float(rw[q] & 0xffff0000u), wj[u]));
                }
            }
        }
        uint32_t ow[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
            ow[q] = (uint32_t)f32_to_bf16_bits(acc[2 * q]) | ((uint32_t)f32_to_bf16_bits(acc[2 * q + 1]) << 16);
        *reinterpret_cast<uint4*>(out + m * H + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
    if (!ok && status) atomicOr(status, GNF4B_ST_TIMEOUT);
    ep_peer_step_done(local, 1, step);
    EPT(43);
}

}  // namespace gnf4b

namespace gnf4b {

// Large batches: blocks of rows pushed into the peers' buffers by all SMs with plain 16-byte stores, then one flag per
// destination behind a system-scope fence (at these sizes the fence is noise); the receiver waits on its flags before
// its GEMMs read the rows.  The host knows every block's place (it has read the counts of all ranks), so the kernel
// is a list of up to kEpPeerMaxWorld copies.  Flags carry the caller's step number and only grow.
struct EpPushArgs {
    const uint8_t* src[kEpPeerMaxWorld];
    uint8_t* dst[kEpPeerMaxWorld];
    int64_t bytes[kEpPeerMaxWorld];            // multiples of 16
    int32_t* flag[kEpPeerMaxWorld];            // this rank's flag word in every peer's buffer (null: no flag)
    int32_t* done_counter;                     // this rank only: finished-CTA counter, left at zero
    int32_t n, step, rot;
};

constexpr int64_t kEpPushChunk = 64 << 10;     // bytes of one block a CTA takes at a time

__global__ void __launch_bounds__(kEpPeerThreads)
ep_push_blocks_kernel(const EpPushArgs a) {
    // Chunks are taken round by round over the blocks -- chunk r of every block before chunk r + 1 of any -- and the
    // round starts at block `rot` (the caller's rank): a rank then writes to all its peers at once, and no two ranks
    // start on the same peer.  (Block after block, every rank would first pour into peer 0's links, then peer 1's.)
    int64_t rounds = 0;
    for (int b = 0; b < a.n; ++b) rounds = max(rounds, (a.bytes[b] + kEpPushChunk - 1) / kEpPushChunk);
    for (int64_t c = blockIdx.x; c < rounds * a.n; c += gridDim.x) {
        const int64_t r = c / a.n;
        const int b = (int)((c - r * a.n + a.rot) % a.n);
        const int64_t lo = r * kEpPushChunk, hi = min(a.bytes[b], lo + kEpPushChunk);
        if (lo >= hi) continue;
        const uint4* s = reinterpret_cast<const uint4*>(a.src[b] + lo);
        uint4* d = reinterpret_cast<uint4*>(a.dst[b] + lo);
        const int64_t n16 = (hi - lo) >> 4;
        for (int64_t i = threadIdx.x; i < n16; i += (int64_t)kEpPeerThreads * 4) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + (int64_t)u * kEpPeerThreads < n16) v[u] = __ldg(s + i + (int64_t)u * kEpPeerThreads);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (i + (int64_t)u * kEpPeerThreads < n16) d[i + (int64_t)u * kEpPeerThreads] = v[u];
        }
    }
    // the CTA's stores are ordered before thread 0 by the barrier, its fence orders them before its count; the CTA
    // that finds all others counted raises the flags
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence_system();
    if (atomicAdd(a.done_counter, 1) != (int32_t)gridDim.x - 1) return;
    __threadfence_system();
    *a.done_counter = 0;
    for (int b = 0; b < a.n; ++b)
        if (a.flag[b]) asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(a.flag[b]), "r"(a.step) : "memory");
}

// Wait until every one of `world` flag words has reached `step` (bounded: limit_ns; GNF4B_ST_TIMEOUT on expiry).
__global__ void ep_wait_flags_kernel(const int32_t* flags, int32_t world, int32_t step, uint64_t limit_ns, int32_t* status) {
    if ((int)threadIdx.x >= world) return;
    const int32_t* f = flags + threadIdx.x;
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    uint64_t t0 = 0;
    for (uint32_t it = 0; (int32_t)(v - step) < 0; ++it) {
        if (it >= 64) {
            __nanosleep(200);
            if (it == 64) t0 = global_timer_ns();
            else if ((it & 255) == 0 && global_timer_ns() - t0 > limit_ns) {
                if (status) atomicOr(status, GNF4B_ST_TIMEOUT);
                break;
            }
        }
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    }
}

}  // namespace gnf4b
