"""Expert-parallel MoE layer around the grouped 4-bit GEMM (one process per GPU).

The reference project is single-GPU; its 128- and 256-expert configurations are sharded
here the way its routing producers lay tokens out (stable sort of token-expert pairs by
expert, ``kernel/mxfp4_qlora.py:294-329``), with one exchange each way:

  rank r owns experts [r*E/W, (r+1)*E/W) as a contiguous slice of every stack;
  1. top-k ids per token -> stable sort of the pairs by global expert id (= by destination
     rank, then local expert), per-(rank, expert) counts;
  2. counts exchanged with all_to_all_single (int32 [W * E/W]) -> receive splits and the
     local group sizes;
  3. DISPATCH: all_to_all_single of the bf16 hidden rows (they land in this GPU's HBM
     before any kernel reads them);
  4. received rows regrouped expert-major, then grouped gate_up -> GLU -> grouped down,
     each ONE launch over all local experts;
  5. COMBINE: the reverse all_to_all_single of the bf16 output rows;
  6. un-sort and routing-weight sum in fp32.

Small batches (decode) take a FIXED-CAPACITY exchange instead: every rank sends every rank a buffer
of C = tokens * top_k rows (the most one destination can get), counts travel in a second equal-split
exchange, and the received buffer is multiplied where it lies -- one group per (source, expert) plus one
padding group per source for the unused capacity (expert id -1: skipped by the kernels).  Nothing is read
back to the host, so the layer is a fixed sequence of launches.

On GPUs of one node the fixed-capacity exchange does not go through a collective library at all
(``PeerExchange``): each rank's routing kernel stores the rows and their per-expert counts straight into the
destination ranks' buffers over NVLink (symmetric memory, plain peer stores, one flag per source and
destination), the result rows come back the same way, and the waits are bounded polls inside the two small kernels
either side of the GEMMs: four launches per layer and no collective.  Large batches move their rows the same way
in bulk (``LargePeerExchange``: every rank gathers all ranks' counts, one host read, then blocks of rows are stored
into the peers' buffers by all SMs with one flag per destination); NCCL's all-to-all is the fallback.

Otherwise the collectives are NCCL over NVLink/NVSwitch on GPUs and gloo in the CPU tests; the GEMM is
injectable (``grouped_fn``) so the exchange logic can be tested on CPU ranks against the
oracle.  There is no TMA multicast anywhere on this path.
"""
from __future__ import annotations

import os
import statistics
import time

import torch
import torch.distributed as dist


def silu_glu(gu: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with gate = first half, up = second half of the gate_up output
    (the split of the reference's offload decode, bench/phase3/offload_decode_235b.py:232-233).
    fp32 math, one bf16 rounding.  On a GPU this is one kernel of the library (gnf4b_silu_glu)."""
    h = gu.shape[1] // 2
    if gu.is_cuda and gu.dtype == torch.bfloat16 and gu.is_contiguous():
        import _gnf4b
        out = torch.empty(gu.shape[0], h, dtype=gu.dtype, device=gu.device)
        with torch.cuda.device(gu.device):
            rc = _gnf4b.load().gnf4b_silu_glu(gu.data_ptr(), gu.shape[0], h, out.data_ptr(),
                                              torch.cuda.current_stream(gu.device).cuda_stream)
        _gnf4b.check(rc, "gnf4b_silu_glu")
        return out
    g, u = gu[:, :h].float(), gu[:, h:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(gu.dtype)


def combine_rows(rows: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out[m] = sum_j weights[m, j] * rows[pos[m, j]], j in order, fp32 (multiply and add rounded
    separately), one rounding to the row dtype.  Deterministic -- unlike an index_add of the pairs.
    On a GPU one kernel of the library (gnf4b_combine_rows); the loop below gives the same bits."""
    M, k = pos.shape
    H = rows.shape[1]
    if rows.is_cuda and rows.dtype == torch.bfloat16 and rows.is_contiguous():
        import _gnf4b
        import nf4_grouped
        out = torch.empty(M, H, dtype=rows.dtype, device=rows.device)
        pos64 = pos.to(torch.int64).contiguous()
        w32 = weights.to(torch.float32).contiguous()
        with torch.cuda.device(rows.device):
            rc = _gnf4b.load().gnf4b_combine_rows(rows.data_ptr(), rows.shape[0], pos64.data_ptr(), w32.data_ptr(), k, M, H,
                                                  out.data_ptr(), nf4_grouped._status_word(rows.device).data_ptr(),
                                                  torch.cuda.current_stream(rows.device).cuda_stream)
        _gnf4b.check(rc, "gnf4b_combine_rows")
        return out
    acc = torch.zeros(M, H, dtype=torch.float32, device=rows.device)
    for j in range(k):
        acc = acc + rows[pos[:, j]].float() * weights[:, j].to(torch.float32)[:, None]
    return acc.to(rows.dtype)


def route_topk(logits: torch.Tensor, k: int, mode: int = 0, norm: bool = False):
    """Router selection: logits [M, E] -> (idx [M, k] int64, weights [M, k] fp32): the k largest logits in
    descending order, ties to the lower expert index; weights = softmax over all experts (``mode`` 0,
    ``norm`` renormalises over the k) or over the k selected (``mode`` 1) -- the rule of the reference's CPU
    router (gnf4_native/cpu_kernels.c:1408-1471).  On a GPU one kernel (gnf4b_route_topk), no host read."""
    lg = logits.float().contiguous()
    M, E = lg.shape
    if lg.is_cuda and k <= 32:
        import _gnf4b
        idx = torch.empty(M, k, dtype=torch.int64, device=lg.device)
        w = torch.empty(M, k, dtype=torch.float32, device=lg.device)
        with torch.cuda.device(lg.device):
            rc = _gnf4b.load().gnf4b_route_topk(lg.data_ptr(), M, E, k, mode, int(norm), idx.data_ptr(), w.data_ptr(),
                                                torch.cuda.current_stream(lg.device).cuda_stream)
        _gnf4b.check(rc, "gnf4b_route_topk")
        return idx, w
    idx = torch.argsort(-lg, dim=-1, stable=True)[:, :k]
    top = torch.gather(lg, 1, idx)
    if mode == 0:
        w = torch.gather(torch.softmax(lg, dim=-1), 1, idx)
        if norm:
            w = w / w.sum(1, keepdim=True)
    else:
        w = torch.softmax(top, dim=-1)
    return idx, w


def plan_dispatch(idx: torch.Tensor, n_experts: int, world: int):
    """Routing ids [M, k] (global expert ids) -> (order [P], tok_of_pair [P], counts [W, E/W]).
    ``order`` is the stable argsort of the flattened ids, so pairs are grouped by destination
    rank, then by local expert, and keep token order inside an expert."""
    k = idx.shape[1]
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    # scatter_add, not bincount: bincount reads its maximum back to the host
    counts = torch.zeros(n_experts, dtype=torch.int64, device=flat.device).scatter_add_(
        0, flat.to(torch.int64), torch.ones_like(flat, dtype=torch.int64)).reshape(world, n_experts // world)
    return order, order // k, counts


def regroup_index(recv_counts: torch.Tensor, total: int | None = None):
    """recv_counts [W, E_local]: rows arrive source-major (source rank, then local expert).
    Returns (perm, sizes): ``recv[perm]`` is expert-major (expert, then source rank, token
    order kept) and ``sizes[e]`` the rows of local expert e.  ``total`` = the row count when the
    caller already has it on the host (saves a device read)."""
    W, E = recv_counts.shape
    rc = recv_counts.to(torch.int64)
    start = (torch.cumsum(rc.reshape(-1), 0) - rc.reshape(-1)).reshape(W, E)   # block starts, source-major
    blk_start = start.t().reshape(-1)                                         # expert-major block order
    blk_len = rc.t().reshape(-1)
    if total is None:
        total = int(blk_len.sum())
    if total == 0:
        return torch.empty(0, dtype=torch.int64, device=rc.device), rc.sum(0)
    within = torch.arange(total, device=rc.device) - torch.repeat_interleave(torch.cumsum(blk_len, 0) - blk_len, blk_len,
                                                                               output_size=total)
    perm = torch.repeat_interleave(blk_start, blk_len, output_size=total) + within
    return perm, rc.sum(0)


#: bytes of exchange buffer (world * capacity * hidden * 2) up to which the fixed-capacity, host-sync-free
#: exchange is used; above it the exact-size exchange (one host read per layer) moves fewer bytes
FIXED_CAPACITY_MAX_BYTES = 4 << 20

#: row slots (world * capacity) up to which the peer-memory exchange makes every received row its own group -- while a
#: local expert gets a few rows at most on average (capacity <= ONE_ROW_MAX_PER_EXPERT * local experts).  Measured
#: with 512 slots on the DeepSeek-V3 shape at 8 tokens per GPU (64 rows per rank): 1036 against 982 us/layer for one
#: group per expert on the tensor kernel, so the bound stays at 128
ONE_ROW_MAX_ROWS = 128
ONE_ROW_MAX_PER_EXPERT = 4

#: tokens per rank from which the exact-size layer is pipelined over two halves of the local experts (below, two more
#: collectives cost more than the overlap brings)
SPLIT_MIN_TOKENS = 512

#: expert id of a padding group (include/gnf4b.h: GNF4B_PAD_EXPERT)
PAD_EXPERT = -1


#: mean rows per (source rank, local expert) block from which the blocks are multiplied where they
#: landed -- each block its own group, the expert id repeated per source -- instead of being gathered
#: expert-major first.  Big blocks lose nothing in the GEMM and save two passes over the rows.
BLOCK_GROUPS_MIN_ROWS = 64


class PeerExchange:
    """This rank's exchange buffer (include/gnf4b.h: gnf4b_ep_peer_ctx) and every peer's address of it.

    The buffer comes from torch's symmetric memory (``torch.distributed._symmetric_memory``): one allocation
    per rank, mapped into every rank of the group by ``rendezvous``; the kernels of the library then use plain
    stores and loads on the peers' addresses.  Building it is a collective: all ranks of the group construct it
    at the same point.  One rank alone needs no mapping and takes ordinary device memory."""

    def __init__(self, group, world: int, rank: int, e_local: int, cap_max: int, H: int, device):
        import ctypes
        import _gnf4b
        lib = _gnf4b.load()
        lay = (ctypes.c_int64 * 3)()
        _gnf4b.check(lib.gnf4b_ep_peer_layout(world, e_local, cap_max, H, lay), "gnf4b_ep_peer_layout")
        self.total, self.recv_off, self.ret_off = int(lay[0]), int(lay[1]), int(lay[2])
        self.world, self.cap_max, self.H = world, cap_max, H
        if world == 1:
            self.handle = None
            self.buf = torch.zeros(self.total, dtype=torch.uint8, device=device)
            ptrs = [self.buf.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm
            pg = group if group is not None else dist.group.WORLD
            self.buf = symm.empty(self.total, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm.rendezvous(self.buf, pg)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            torch.cuda.synchronize(device)
            dist.barrier(group)          # every buffer is zeroed before any rank stores into a peer's
        self.ctx = _gnf4b.EpPeerCtx(world, rank, e_local, cap_max, H)
        for r in range(world):
            self.ctx.peers[r] = ptrs[r]
        self.ref = ctypes.byref(self.ctx)

    _shared = {}

    @classmethod
    def shared(cls, group, world, rank, e_local, cap_max, H, device):
        """One buffer per (group, shape, device) for all layers of a process: the layers run one after the other
        on one stream and every rank uses the buffer in the same order, which is all the exchange needs."""
        key = (id(group) if group is not None else 0, world, rank, e_local, cap_max, H, str(device))
        px = cls._shared.get(key)
        if px is None:
            px = cls._shared[key] = cls(group, world, rank, e_local, cap_max, H, device)
        return px

    def recv_rows(self, cap: int) -> torch.Tensor:
        """The row matrix [world * cap, H] bf16 the arrive kernel unpacks the received rows into."""
        n = self.world * cap * self.H * 2
        return self.buf[self.recv_off:self.recv_off + n].view(torch.bfloat16).view(self.world * cap, self.H)


class LargePeerExchange:
    """Symmetric buffers of the large-batch exchange: [flags of dispatch | flags of combine | counter | received rows
    (cap_recv x H) | returned rows (cap_ret x H)], one per rank, mapped into every rank.  Built collectively."""

    def __init__(self, group, world, rank, cap_recv, cap_ret, H, device):
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank, self.H = world, rank, H
        self.cap_recv, self.cap_ret = int(cap_recv), int(cap_ret)
        self.flags_dispatch_off, self.flags_combine_off, self.done_off = 0, 64, 128
        self.recv_off = 256
        self.ret_off = self.recv_off + (self.cap_recv * H * 2 + 255) // 256 * 256
        total = self.ret_off + (self.cap_ret * H * 2 + 255) // 256 * 256
        pg = group if group is not None else dist.group.WORLD
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.buf[:256].zero_()
        self.handle = symm.rendezvous(self.buf, pg)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)              # every header is zeroed before any rank raises a flag in it
        self.step = 0
        self.timeout_ms = 10000

    _shared = {}

    @classmethod
    def shared(cls, group, world, rank, cap_recv, cap_ret, H, device):
        """One set of buffers per (group, capacity, device) for all layers of a process (they run one after the other
        on one stream, and every rank uses the buffers in the same order)."""
        key = (id(group) if group is not None else 0, world, rank, int(cap_recv), int(cap_ret), H, str(device))
        px = cls._shared.get(key)
        if px is None:
            px = cls._shared[key] = cls(group, world, rank, cap_recv, cap_ret, H, device)
        return px

    def next_step(self) -> int:
        self.step += 1
        return self.step

    def view(self, off, rows, H):
        return self.buf[off:off + rows * H * 2].view(torch.bfloat16).view(rows, H)


class EPGroupedMoE:
    """One expert-parallel MoE layer.  ``gate_up`` / ``down`` are this rank's shards
    ``(W [E/W, N, K/2] u8, S scales)``; ``grouped_fn(a_cat, W, S, sizes, expert_ids)`` is the
    grouped GEMM (the CUDA op by default)."""

    def __init__(self, n_experts: int, gate_up, down, group=None, grouped_fn=None, fmt: str = "nf4",
                 peer_exchange: bool | None = None, split_experts: bool | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_experts = n_experts
        self.e_local = n_experts // self.world
        assert self.e_local * self.world == n_experts, "experts must divide evenly over the ranks"
        self.gate_up, self.down = gate_up, down
        self._own_gemm = grouped_fn is None          # the library's GEMM (not an injected one): fused forms apply
        self._fmt_id = 0 if fmt == "nf4" else 1      # GNF4B_FMT_NF4 / GNF4B_FMT_MXFP4
        if grouped_fn is None:
            if fmt == "nf4":
                from nf4_grouped import gemm_4bit_grouped as grouped_fn
            else:
                from mxfp4_grouped import gemm_mxfp4_grouped as grouped_fn
        self.grouped_fn = grouped_fn
        self.timers = None           # set to a dict of CUDA-event lists to get a phase breakdown
        self._fixed_eids = None      # expert ids of the fixed-capacity path's groups (built once per device)
        # small batches on GPUs: rows cross NVLink by the library's own peer stores (PeerExchange) unless this is
        # False or GNF4B_EP_PEER=0, in which case the same exchange runs as collectives
        if peer_exchange is None:
            peer_exchange = os.environ.get("GNF4B_EP_PEER", "1") != "0"
        self.peer_exchange = bool(peer_exchange) and self.world <= 16
        self._peer = {}              # (hidden size, device) -> PeerExchange
        # large batches: the layer pipelined over the two halves of the local experts on two streams, on request
        # (split_experts=True or GNF4B_EP_SPLIT=1).  Off by default: on 2 GPUs at 4096 tokens per GPU it measured
        # 1832 against 1597 us/layer -- there the exchange phases are the routing plan's sort and gather kernels and
        # the host read, not time on NVLink, and two more collectives and smaller GEMMs cost more than the overlap brings
        self.split_experts = (os.environ.get("GNF4B_EP_SPLIT", "0") == "1") if split_experts is None else bool(split_experts)
        self._streams = None
        self._host_counts = None     # pinned landing buffer of the large-batch path's one host read
        self._host_all = None
        # large batches over the library's own stores into symmetric buffers (GNF4B_EP_PEER_LARGE=0: NCCL all-to-all)
        self.peer_large = os.environ.get("GNF4B_EP_PEER_LARGE", "1") != "0"
        self._peer_large_buf = {}
        self._peer_recv_counts = None
        self._local_eids = None
        self.last_rows = 0

    # -- helpers ---------------------------------------------------------------
    def _a2a(self, out, inp, out_splits, in_splits):
        if self.world == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out, inp, out_splits, in_splits, group=self.group)

    def _mark(self, name):
        if self.timers is not None and torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.timers.setdefault(name, []).append(e)

    # -- the layer ---------------------------------------------------------------
    def forward(self, hidden: torch.Tensor, idx: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """hidden [M, H] bf16, idx [M, k] global expert ids, weights [M, k] fp32 -> [M, H] bf16.
        A collective call: every rank of the group calls it with the same M and k (the choice between the
        fixed-capacity and the exact-size exchange, and the capacity itself, follow from them)."""
        W, El = self.world, self.e_local
        dev = hidden.device
        self._mark("start")
        cap = idx.numel()                    # rows one destination can get from this rank at most
        # (a single rank takes it too: routing plan, groups and combine without a host read)
        if W * cap * hidden.shape[1] * hidden.element_size() <= FIXED_CAPACITY_MAX_BYTES:
            return self._forward_fixed(hidden, idx, weights, cap)
        halves = 2 if (self.split_experts and W > 1 and El >= 2 and self.timers is None
                       and hidden.shape[0] >= SPLIT_MIN_TOKENS) else 1
        return self._forward_exact(hidden, idx, weights, halves)

    def _forward_exact(self, hidden, idx, weights, halves: int = 1):
        """The exact-size layer.  ``halves`` = 2 pipelines it over the two halves of every rank's local experts on
        two streams: rows for the lower half are dispatched first, their GEMMs run while the upper half's rows
        cross NVLink, and the lower half's results travel back under the upper half's GEMMs.  The split is by
        EXPERT, not by token, because the grouped GEMM's cost at these sizes is per expert (every active expert's
        4-bit weights are decoded once whatever its rows): token chunks would pay it once per chunk.  One routing
        plan, one counts exchange and one host read serve both halves, and the returned rows land in one buffer in
        the order they left, so the weighted sum -- and the result -- is the same as without the split.  The
        collectives of one communicator run in the order they are issued, the same on every rank:
        dispatch(0), dispatch(1), combine(0), combine(1)."""
        W, El = self.world, self.e_local
        dev = hidden.device
        H = hidden.shape[1]
        k = idx.shape[1]
        flat = idx.reshape(-1).to(torch.int64)
        cut = El - El // 2 if halves == 2 else El                       # local experts [0, cut) are half 0
        both = torch.empty(2, W, El, dtype=torch.int32, device=dev)     # [0] what this rank sends, [1] what it receives
        counts32, recv_counts = both[0], both[1]
        use_lib = (hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.is_contiguous() and H % 8 == 0
                   and self.n_experts <= 1024 and self._own_gemm)
        if use_lib:
            # the stable sort by (half, global expert id), the per-expert counts and the row gather as four small
            # kernels of the library (a counting sort; the tensor operations below take ~150 us more at 32768 pairs)
            import _gnf4b
            import nf4_grouped
            lib = _gnf4b.load()
            P = flat.numel()
            need = lib.gnf4b_ep_plan_large_scratch_bytes(P, self.n_experts)
            scratch = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
            pos = torch.empty(P, dtype=torch.int64, device=dev)
            send = torch.empty(P, H, dtype=hidden.dtype, device=dev)
            with torch.cuda.device(dev):
                _gnf4b.check(lib.gnf4b_ep_plan_large(flat.data_ptr(), P, k, self.n_experts, El, cut, hidden.data_ptr(), H,
                                                     counts32.data_ptr(), pos.data_ptr(), send.data_ptr(), scratch.data_ptr(),
                                                     need, nf4_grouped._status_word(dev).data_ptr(),
                                                     torch.cuda.current_stream(dev).cuda_stream), "gnf4b_ep_plan_large")
            if self.peer_exchange and self.peer_large and halves == 1 and W > 1:
                out = self._exact_peer(hidden, idx, weights, counts32, pos, send)
                if out is not None:
                    return out
                # (capacity of the symmetric buffers exceeded: this step goes over NCCL; recv_counts was filled)
                recv_counts = self._peer_recv_counts
                both = torch.stack((counts32, recv_counts))
            else:
                self._a2a(recv_counts.reshape(-1), counts32.reshape(-1), None, None)
        else:
            # stable sort by (half, global expert id) = (half, destination rank, local expert), token order kept
            key = flat if halves == 1 else flat + ((flat % El) >= cut).to(torch.int64) * self.n_experts
            order = torch.argsort(key, stable=True)
            tok = order // k
            counts = torch.zeros(self.n_experts, dtype=torch.int64, device=dev).scatter_add_(
                0, flat, torch.ones_like(flat)).reshape(W, El)
            counts32.copy_(counts)
            self._a2a(recv_counts.reshape(-1), counts32.reshape(-1), None, None)
            # work that does not depend on the counts is queued before the host waits for them
            send = hidden[tok]
            pos = torch.empty_like(order)        # pair (m, j) sits at sorted position pos[m * k + j]
            pos[order] = torch.arange(order.numel(), device=dev)
        # the exchange needs its split sizes on the host: ONE small read per layer brings both count
        # tables, everything else about the layer's shape is derived from them on the host.  On a GPU the read
        # lands in a pinned buffer (a copy to pageable memory costs ~150 us more)
        if hidden.is_cuda:
            if self._host_counts is None or self._host_counts.shape != both.shape:
                self._host_counts = torch.empty(both.shape, dtype=torch.int32).pin_memory()
            self._host_counts.copy_(both, non_blocking=True)
            torch.cuda.current_stream(dev).synchronize()
            host = self._host_counts.clone()
        else:
            host = both.clone()
        ret = torch.empty_like(send)
        self.last_rows = int(host[1].sum())
        if halves == 1:
            self._exact_part(send, ret, host, recv_counts, 0, El, H)
        else:
            n0 = int(host[0][:, :cut].sum())                            # rows of half 0 in send / ret
            parts = ((send[:n0], ret[:n0], 0, cut), (send[n0:], ret[n0:], cut, El))
            if hidden.is_cuda:
                cur = torch.cuda.current_stream(dev)
                if self._streams is None:
                    self._streams = [torch.cuda.Stream(dev) for _ in range(2)]
                staged = []
                for st, (sp, rp, lo, hi) in zip(self._streams, parts):      # dispatch(0), dispatch(1)
                    st.wait_stream(cur)
                    with torch.cuda.stream(st):
                        staged.append(self._exact_dispatch(sp, host, lo, hi, H))
                for st, (sp, rp, lo, hi), stg in zip(self._streams, parts, staged):     # GEMMs + combine per half
                    with torch.cuda.stream(st):
                        self._exact_compute_return(stg, rp, host, recv_counts, lo, hi)
                for st in self._streams:
                    cur.wait_stream(st)
                for t in staged:
                    t["recv"].record_stream(cur)
            else:           # CPU ranks (tests): the same sequence of exchanges without streams
                staged = [self._exact_dispatch(sp, host, lo, hi, H) for sp, rp, lo, hi in parts]
                for (sp, rp, lo, hi), stg in zip(parts, staged):
                    self._exact_compute_return(stg, rp, host, recv_counts, lo, hi)
        self._mark("combine")
        out = combine_rows(ret, pos.reshape(idx.shape), weights)     # the k copies are summed in j order
        self._mark("sum")
        return out

    def _exact_peer(self, hidden, idx, weights, counts32, pos, send):
        """The exact-size layer with the rows moved by the library's own stores into symmetric buffers
        (gnf4b_ep_push_blocks / gnf4b_ep_wait_flags) instead of NCCL's all-to-all, which reaches about a third of
        a peer copy's bandwidth at these sizes.  Every rank gathers ALL ranks' per-(destination, expert) counts
        (one small all_gather, then the layer's one host read), so each knows where its blocks start in every
        peer's receive buffer and where every peer's results start in its own return buffer.  Returns None when the
        rows of this step do not fit the buffers (every rank sees the same table and decides the same)."""
        import ctypes
        import _gnf4b
        import nf4_grouped
        W, El, rank = self.world, self.e_local, self.rank
        dev = hidden.device
        H = hidden.shape[1]
        P = send.shape[0]
        all_counts = torch.empty(W, W, El, dtype=torch.int32, device=dev)            # [source, destination, expert]
        dist.all_gather_into_tensor(all_counts.reshape(-1), counts32.reshape(-1), group=self.group)
        if self._host_all is None or self._host_all.shape != all_counts.shape:
            self._host_all = torch.empty(all_counts.shape, dtype=torch.int32).pin_memory()
        self._host_all.copy_(all_counts, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        tab = self._host_all.clone()
        # (numpy for the few dozen integers: the GPU waits while the host does this arithmetic)
        tot = tab.numpy().sum(-1, dtype="int64")                                     # rows [source, destination]
        self._peer_recv_counts = all_counts[:, rank, :].contiguous()
        px = self._peer_large_buf.get((H, dev))
        if px is None:
            rows = int(tot.sum(1).max())            # the most pairs any rank holds: the same number on every rank
            px = self._peer_large_buf[(H, dev)] = LargePeerExchange.shared(self.group, W, rank, 2 * rows, rows, H, dev)
        n_recv_all = tot.sum(0)
        if int(n_recv_all.max()) > px.cap_recv or int(tot.sum(1).max()) > px.cap_ret:
            return None
        lib = _gnf4b.load()
        stream = torch.cuda.current_stream(dev).cuda_stream
        status = nf4_grouped._status_word(dev).data_ptr()
        row = H * 2
        send_tot, recv_tot = tot[rank].tolist(), tot[:, rank].tolist()
        send_start = (tot[rank].cumsum() - tot[rank]).tolist()
        recv_start = (tot[:, rank].cumsum() - tot[:, rank]).tolist()
        n_recv = sum(recv_tot)
        start_in_dest = tot[:rank].sum(0).tolist()                                 # my block in d's receive buffer
        ret_start_in_src = tot[:, :rank].sum(1).tolist()                           # my results in s's return buffer
        step = px.next_step()
        vp = ctypes.c_void_p

        def push(srcs, dsts, sizes, flag_off):
            a_src = (vp * W)(*srcs)
            a_dst = (vp * W)(*dsts)
            a_len = (ctypes.c_int64 * W)(*sizes)
            a_flag = (vp * W)(*[px.ptrs[r] + flag_off + rank * 4 for r in range(W)])
            _gnf4b.check(lib.gnf4b_ep_push_blocks(W, a_src, a_dst, a_len, a_flag, step, rank, px.ptrs[rank] + px.done_off, stream),
                         "gnf4b_ep_push_blocks")

        with torch.cuda.device(dev):
            push([send.data_ptr() + send_start[d] * row for d in range(W)],
                 [px.ptrs[d] + px.recv_off + start_in_dest[d] * row for d in range(W)],
                 [send_tot[d] * row for d in range(W)], px.flags_dispatch_off)
            _gnf4b.check(lib.gnf4b_ep_wait_flags(px.ptrs[rank] + px.flags_dispatch_off, W, step, px.timeout_ms, status, stream),
                         "gnf4b_ep_wait_flags")
        self._mark("dispatch")
        recv = px.view(px.recv_off, n_recv, H)
        stg = dict(recv=recv)
        host = torch.stack((tab[rank], tab[:, rank]))
        self.last_rows = n_recv
        back = self._exact_compute(stg, host, self._peer_recv_counts, 0, El)
        with torch.cuda.device(dev):
            push([back.data_ptr() + recv_start[s] * row for s in range(W)],
                 [px.ptrs[s] + px.ret_off + ret_start_in_src[s] * row for s in range(W)],
                 [recv_tot[s] * row for s in range(W)], px.flags_combine_off)
            _gnf4b.check(lib.gnf4b_ep_wait_flags(px.ptrs[rank] + px.flags_combine_off, W, step, px.timeout_ms, status, stream),
                         "gnf4b_ep_wait_flags")
        self._mark("combine")
        out = combine_rows(px.view(px.ret_off, P, H), pos.reshape(idx.shape), weights)
        self._mark("sum")
        return out

    def _exact_dispatch(self, send_part, host, lo, hi, H):
        """Rows for local experts [lo, hi) of every rank: one all_to_all with the split sizes from the host counts."""
        send_splits = host[0][:, lo:hi].sum(1).tolist()
        recv_splits = host[1][:, lo:hi].sum(1).tolist()
        recv = torch.empty(sum(recv_splits), H, dtype=send_part.dtype, device=send_part.device)
        self._a2a(recv, send_part, recv_splits, send_splits)
        self._mark("dispatch")
        return dict(recv=recv, send_splits=send_splits, recv_splits=recv_splits)

    def _exact_compute_return(self, stg, ret_part, host, recv_counts, lo, hi):
        """The grouped GEMMs and the activation on the received rows of local experts [lo, hi), results back."""
        back = self._exact_compute(stg, host, recv_counts, lo, hi)
        self._a2a(ret_part, back, stg["send_splits"], stg["recv_splits"])

    def _exact_compute(self, stg, host, recv_counts, lo, hi):
        """The grouped GEMMs and the activation on the received rows of local experts [lo, hi); returns the result
        rows in the order the rows arrived."""
        W, El = self.world, self.e_local
        recv = stg["recv"]
        n_recv = recv.shape[0]
        if W > 1 and n_recv >= BLOCK_GROUPS_MIN_ROWS * W * (hi - lo):
            perm = None                     # groups = the (source, expert) blocks as they arrived
            a_cat = recv
            sizes_l = host[1][:, lo:hi].reshape(-1).tolist()
            eids = list(range(lo, hi)) * W
        else:
            perm, _ = regroup_index(recv_counts[:, lo:hi], n_recv)
            a_cat = recv[perm]
            sizes_l = host[1][:, lo:hi].sum(0).tolist()
            eids = list(range(lo, hi))
        gu = self.grouped_fn(a_cat, self.gate_up[0], self.gate_up[1], sizes_l, eids)
        self._mark("gate_up")
        h = silu_glu(gu)
        self._mark("glu")
        y = self.grouped_fn(h, self.down[0], self.down[1], sizes_l, eids)
        self._mark("down")
        if perm is None:
            return y
        # back[perm[i]] = y[i] as a gather through the inverse permutation (an index_put of whole rows is several
        # times slower than a gather)
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel(), device=perm.device)
        return y[inv]

    def _exact_part(self, send, ret, host, recv_counts, lo, hi, H):
        self._exact_compute_return(self._exact_dispatch(send, host, lo, hi, H), ret, host, recv_counts, lo, hi)

    def forward_logits(self, hidden: torch.Tensor, logits: torch.Tensor, k: int, mode: int = 0, norm: bool = False):
        """Router included: ``logits [M, E]`` -> top-k ids and weights on the device, then ``forward``."""
        idx, w = route_topk(logits, k, mode, norm)
        return self.forward(hidden, idx, w)

    def _forward_fixed(self, hidden, idx, weights, cap):
        """The layer with fixed-capacity exchanges: no host read, a fixed sequence of launches.  On a GPU
        the routing plan (counts, slots, row scatter) and the group offsets are one small kernel each
        (gnf4b_ep_plan, gnf4b_ep_offsets); the tensor-operation form below them is the same computation
        (it serves CPU ranks and batches beyond the kernels' 1024 pairs)."""
        W, El = self.world, self.e_local
        dev = hidden.device
        H = hidden.shape[1]
        n_groups = W * (El + 1)
        if self._fixed_eids is None or self._fixed_eids.device != dev:
            self._fixed_eids = torch.tensor((list(range(El)) + [PAD_EXPERT]) * W, dtype=torch.int32, device=dev)
        use_lib = (hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.is_contiguous() and cap <= 1024
                   and self.n_experts <= 1024)
        if use_lib and self.peer_exchange and H % 8 == 0 and W * cap <= 1024:
            return self._forward_peer(hidden, idx, weights, cap)
        if use_lib:
            import _gnf4b
            import nf4_grouped
            lib = _gnf4b.load()
            stream = torch.cuda.current_stream(dev).cuda_stream
            status = nf4_grouped._status_word(dev).data_ptr()
            idx64 = idx.to(torch.int64).contiguous()
            counts32 = torch.empty(W, El, dtype=torch.int32, device=dev)
            slot = torch.empty(cap, dtype=torch.int64, device=dev)
            send = torch.empty(W * cap, H, dtype=hidden.dtype, device=dev)
            with torch.cuda.device(dev):
                _gnf4b.check(lib.gnf4b_ep_plan(idx64.data_ptr(), cap, idx.shape[1], self.n_experts, El, cap, hidden.data_ptr(), H,
                                               counts32.data_ptr(), slot.data_ptr(), send.data_ptr(), status, stream),
                             "gnf4b_ep_plan")
        else:
            order, tok, counts = plan_dispatch(idx, self.n_experts, W)          # counts [W, El]
            counts32 = counts.to(torch.int32).contiguous()
            # pair p (sorted order) goes to rank d(p) at row p - start[d] of that rank's buffer
            per_dest = counts.sum(1)
            start = torch.cumsum(per_dest, 0) - per_dest
            dest = torch.repeat_interleave(torch.arange(W, device=dev), per_dest, output_size=order.numel())
            slot_sorted = dest * cap + (torch.arange(order.numel(), device=dev) - start[dest])
            send = torch.zeros(W * cap, H, dtype=hidden.dtype, device=dev)
            send[slot_sorted] = hidden[tok]
            slot = torch.empty_like(order)
            slot[order] = slot_sorted                # pair (m, j) comes back at the row it was sent from
        if W == 1:                      # one rank: what it would send is what it receives
            recv_counts, recv = counts32, send
        else:
            recv_counts = torch.empty_like(counts32)
            self._a2a(recv_counts.reshape(-1), counts32.reshape(-1), None, None)
            recv = torch.empty_like(send)
            self._a2a(recv, send, None, None)
        self._mark("dispatch")
        # groups as the rows lie: per source its El expert blocks, then the unused capacity as padding
        if use_lib:
            offsets = torch.empty(n_groups + 1, dtype=torch.int32, device=dev)
            with torch.cuda.device(dev):
                _gnf4b.check(lib.gnf4b_ep_offsets(recv_counts.data_ptr(), W, El, cap, offsets.data_ptr(), status, stream),
                             "gnf4b_ep_offsets")
        else:
            rc = recv_counts.to(torch.int64)
            sizes = torch.cat((rc, (cap - rc.sum(1, keepdim=True))), 1).reshape(-1)         # [W * (El + 1)]
            offsets = torch.zeros(n_groups + 1, dtype=torch.int32, device=dev)
            offsets[1:] = torch.cumsum(sizes, 0).to(torch.int32)
        self.last_rows = W * cap
        # a (source, expert) block has at most one row per token of the source: the row bound of the
        # real groups is the token count, not the capacity (padding groups are skipped whatever their size)
        max_rows = idx.shape[0]
        gu = self.grouped_fn(recv, self.gate_up[0], self.gate_up[1], None, self._fixed_eids,
                             group_offsets=offsets, max_rows=max_rows)
        self._mark("gate_up")
        h = silu_glu(gu)
        self._mark("glu")
        y = self.grouped_fn(h, self.down[0], self.down[1], None, self._fixed_eids, group_offsets=offsets,
                            max_rows=max_rows)
        self._mark("down")
        if W == 1:
            ret = y
        else:
            ret = torch.empty_like(y)
            self._a2a(ret, y, None, None)
        self._mark("combine")
        out = combine_rows(ret, slot.reshape(idx.shape), weights)
        self._mark("sum")
        return out


    def _forward_peer(self, hidden, idx, weights, cap):
        """The fixed-capacity layer with the rows carried by the library's own kernels over peer memory: dispatch
        (plan + stores into the destinations' buffers, then bounded wait, rows unpacked expert-major, group tables),
        the two grouped GEMMs and the activation, combine (stores back, then bounded wait + routing-weight sum).
        Four launches (the activation is applied by the second GEMM), no collective, no fence, no host read.  Up to ONE_ROW_MAX_ROWS row
        slots every received row is its own group (the one-row kernels); beyond, the groups are the local experts."""
        import _gnf4b
        import nf4_grouped
        W, El = self.world, self.e_local
        dev = hidden.device
        H = hidden.shape[1]
        px = self._peer.get((H, dev))
        if px is None:
            cap_max = max(1, min(1024 // W, FIXED_CAPACITY_MAX_BYTES // (W * H * hidden.element_size())))
            with torch.cuda.device(dev):
                px = self._peer[(H, dev)] = PeerExchange.shared(self.group, W, self.rank, El, cap_max, H, dev)
        one_row = W * cap <= ONE_ROW_MAX_ROWS and cap <= ONE_ROW_MAX_PER_EXPERT * El
        n_groups = W * cap if one_row else El
        lib = _gnf4b.load()
        stream = torch.cuda.current_stream(dev).cuda_stream
        status = nf4_grouped._status_word(dev).data_ptr()
        idx64 = idx.to(torch.int64).contiguous()
        w32 = weights.to(torch.float32).contiguous()
        M, k = idx.shape
        slot = torch.empty(cap, dtype=torch.int64, device=dev)
        offsets = torch.empty(n_groups + 1, dtype=torch.int32, device=dev)
        if one_row:
            eids = torch.empty(n_groups, dtype=torch.int32, device=dev)
        else:
            if self._local_eids is None or self._local_eids.device != dev:
                self._local_eids = torch.arange(El, dtype=torch.int32, device=dev)
            eids = self._local_eids
        out = torch.empty(M, H, dtype=hidden.dtype, device=dev)
        with torch.cuda.device(dev):
            _gnf4b.check(lib.gnf4b_ep_peer_dispatch(px.ref, idx64.data_ptr(), cap, k, self.n_experts, cap, hidden.data_ptr(),
                                                    slot.data_ptr(), int(one_row), offsets.data_ptr(), eids.data_ptr(), status,
                                                    stream), "gnf4b_ep_peer_dispatch")
        self._mark("dispatch")
        recv = px.recv_rows(cap)
        self.last_rows = W * cap
        max_rows = 1 if one_row else W * M          # an expert can get every token of every rank
        # one-row groups: a list of world * cap groups of which the first few exist -- the kernels deal out only those
        sparse = {"path": _gnf4b.FLAG_SPARSE_GROUPS} if (one_row and self._own_gemm) else {}
        gu = self.grouped_fn(recv, self.gate_up[0], self.gate_up[1], None, eids, group_offsets=offsets, max_rows=max_rows,
                             **sparse)
        self._mark("gate_up")
        if self._own_gemm:
            # small groups: the second GEMM applies the activation while it loads the first one's output
            self._mark("glu")
            y = nf4_grouped.gemm_after_glu(self._fmt_id, gu, self.down[0], self.down[1], eids, offsets, max_rows,
                                           path=sparse.get("path", 0))
        else:
            h = silu_glu(gu)
            self._mark("glu")
            y = self.grouped_fn(h, self.down[0], self.down[1], None, eids, group_offsets=offsets, max_rows=max_rows)
        self._mark("down")
        with torch.cuda.device(dev):
            _gnf4b.check(lib.gnf4b_ep_peer_combine(px.ref, cap, y.data_ptr(), slot.data_ptr(), w32.data_ptr(), k, M,
                                                   out.data_ptr(), status, stream), "gnf4b_ep_peer_combine")
        self._mark("combine")
        self._mark("sum")
        return out

# --------------------------------------------------------------------------- benchmark leg
def bench_ep(args, shape, rank, world, B):
    """Expert-parallel leg of bench.py: ``args.tokens`` tokens per rank, experts sharded over
    the ranks, one EP layer per step (dispatch, gate_up, GLU, down, combine, weighted sum).
    Times K steps with CUDA events, max over ranks."""
    import os

    import nf4_grouped
    import synth
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    K, Wm = args.steps, args.warmup
    e_local = shape.experts // world
    n_layers = max(2, min(args.layers, 8))
    # this rank's expert shards (seeded per global expert slice)
    gen = torch.Generator().manual_seed(4321 + rank)
    layers = []
    for _ in range(n_layers):
        (n1, k1), (n2, k2) = shape.gate_up, shape.down
        mk = synth.nf4_stack if shape.fmt == "nf4" else synth.mxfp4_stack
        layers.append((mk(e_local, n1, k1, gen, device=dev, fast=True), mk(e_local, n2, k2, gen, device=dev, fast=True)))
    zipf = 1.1 if shape.name == "deepseek_v3" else None
    gen2 = torch.Generator().manual_seed(777 + rank)
    steps = []
    for _ in range(K + Wm):
        x, idx, w = synth.routed_batch(shape, args.tokens, gen2, zipf)
        steps.append((x.pin_memory(), idx.pin_memory(), w.pin_memory()))
    dsteps = [(x.to(dev), idx.to(dev), w.to(dev)) for x, idx, w in steps]
    mods = [EPGroupedMoE(shape.experts, gu, dn, fmt=shape.fmt) for gu, dn in layers]

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def run(i, host):
        m = mods[i % n_layers]
        if host:
            x, idx, w = (t.to(dev, non_blocking=True) for t in steps[i])
            return m.forward(x, idx, w).to("cpu")
        return m.forward(*dsteps[i])

    for i in range(Wm):
        run(i, False)
    # The fixed-capacity path reads nothing back to the host, so the K steps can be one CUDA graph
    # (collectives included), like the single-GPU arm; the exact-size path is timed eagerly.
    cap_bytes = world * args.tokens * shape.top_k * shape.hidden * 2
    graph, timing = None, "K eager steps, CUDA events, max over ranks"
    if cap_bytes <= FIXED_CAPACITY_MAX_BYTES and os.environ.get("GNF4B_EP_GRAPH", "1") != "0":
        try:
            barrier()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(Wm, Wm + K):
                    run(i, False)
            torch.cuda.current_stream().wait_stream(side)
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(Wm, Wm + K):
                    run(i, False)
            graph.replay()
            barrier()
            timing = "K steps (fixed-capacity exchange, no host read) in one CUDA graph incl. the exchanges, CUDA events, max over ranks"
        except Exception as exc:      # capture of the collectives not available: time eagerly
            if os.environ.get("GNF4B_EP_DEBUG"):
                import traceback
                traceback.print_exc()
            graph = None
            timing += f" (graph capture failed: {type(exc).__name__}: {str(exc)[:160]})"
            torch.cuda.synchronize()
    with B.ClockSampler(dev.index) as clk:
        t_res = []
        # at least repeats // 2 timed passes, and more of them until 0.5 s of this load have passed, so
        # that the 100 ms clock sampler sees the GPU under it (the same count on every rank)
        n_pass, extended = max(1, args.repeats // 2), False
        t_begin = time.perf_counter()
        while True:
            if len(t_res) >= n_pass:
                if extended:
                    break
                extended = True
                per = (time.perf_counter() - t_begin) / len(t_res)
                want = torch.tensor([min(500.0, max(float(n_pass), 0.5 / max(per, 1e-6)))], device=dev)
                dist.all_reduce(want, op=dist.ReduceOp.MAX)
                n_pass = int(want.item())
                if len(t_res) >= n_pass:
                    break
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if graph is not None:
                graph.replay()
            else:
                for i in range(Wm, Wm + K):
                    run(i, False)
            e1.record()
            barrier()
            t_res.append(e0.elapsed_time(e1))
        for i in range(Wm):
            run(i, True)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(Wm, Wm + K):
            run(i, True)
        e1.record()
        barrier()
        t_e2e = e0.elapsed_time(e1)
        # phase breakdown and per-rank load, one instrumented pass
        for m in mods:
            m.timers = {}
        rows = []
        for i in range(Wm, Wm + K):
            run(i, False)
            rows.append(mods[i % n_layers].last_rows)
        torch.cuda.synchronize()
        names = ["dispatch", "gate_up", "glu", "down", "combine", "sum"]
        phase = {n: [] for n in names}
        for m in mods:
            ev = m.timers
            for j in range(len(ev.get("start", []))):
                prev = ev["start"][j]
                for n in names:
                    phase[n].append(prev.elapsed_time(ev[n][j]) * 1e3)
                    prev = ev[n][j]
            m.timers = None
    # parity on the real collectives: this rank's result of one step against the same layer computed WITHOUT any
    # exchange from the gathered expert shards (a one-rank process group), same seeds
    parity = None
    single_us = None
    try:
        own = None
        for r in range(world):
            grp = dist.new_group([r])
            if r == rank:
                own = grp
        (gu0, dn0) = layers[0]
        full = []
        for (Wl, Sl) in (gu0, dn0):
            parts_w = [torch.empty_like(Wl) for _ in range(world)]
            parts_s = [torch.empty_like(Sl) for _ in range(world)]
            dist.all_gather(parts_w, Wl.contiguous())
            dist.all_gather(parts_s, Sl.contiguous())
            full.append((torch.cat(parts_w), torch.cat(parts_s)))
        single = EPGroupedMoE(shape.experts, full[0], full[1], group=own, fmt=shape.fmt)
        got = mods[0].forward(*dsteps[Wm]).float()
        want = single.forward(*dsteps[Wm]).float()
        lim = 2 * 2 ** -8 * want.abs().max()
        ratio = torch.stack(((got - want).abs().max() / lim.clamp_min(1e-30), want.abs().max()))
        dist.all_reduce(ratio, op=dist.ReduceOp.MAX)
        parity = {"max_abs_diff_over_limit": ratio[0].item(), "limit": "2 * 2^-8 * max|reference| per rank",
                  "ok": bool(ratio[0].item() <= 1.0),
                  "what": "EP layer output of one step vs the same layer on one rank from the gathered shards, max over ranks"}
        # the same layer WITHOUT any exchange partner (all experts on this GPU, this rank's tokens): what one GPU
        # needs for the layer code itself, the denominator of the efficiency figure below
        if graph is not None:
            mine_us, fine = 0.0, 1.0
            try:
                for i in range(Wm, Wm + K):
                    single.forward(*dsteps[i])
                g1 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1):
                    for i in range(Wm, Wm + K):
                        single.forward(*dsteps[i])
                ts1 = []
                for _ in range(5):
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g1.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts1.append(e0.elapsed_time(e1) * 1e3 / K)
                mine_us = statistics.median(ts1)
                del g1
            except Exception:
                fine = 0.0
                torch.cuda.synchronize()
            both = torch.tensor([mine_us, -fine], device=dev)       # every rank reaches this reduction
            dist.all_reduce(both, op=dist.ReduceOp.MAX)
            single_us = both[0].item() if both[1].item() == -1.0 else None
        del single, full
    except Exception as exc:      # never at the cost of the timing
        parity = {"ok": None, "error": f"{type(exc).__name__}: {str(exc)[:200]}"}
    t = torch.tensor([statistics.median(t_res), t_e2e, float(statistics.mean(rows))], device=dev)
    tmax = t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone()
    dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    ms_layer, ms_e2e = tmax[0].item(), tmax[1].item()
    us_layer = ms_layer * 1e3 / K
    rows_mean = tsum[2].item() / world
    pairs = args.tokens * shape.top_k
    fl = sum(2 * pairs * n * k for n, k in (shape.gate_up, shape.down)) * world
    peaks = B.measured_peaks()
    us_gu = statistics.median(phase["gate_up"])
    fl_gu_rank = 2 * rows_mean * shape.gate_up[0] * shape.gate_up[1]
    hbm_bound = pairs / shape.experts <= 16
    if hbm_bound:
        # decode-sized groups: the weights of the experts that received rows are streamed once.  The number of
        # distinct local experts is the expectation for rows_mean uniformly routed rows over e_local experts.
        active_est = e_local * (1.0 - (1.0 - 1.0 / e_local) ** rows_mean)
        by_gu_rank = B.algorithmic(shape, "gate_up", rows_mean, active_est)[0]
        ach = by_gu_rank / (us_gu * 1e-6) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "active_experts_per_rank_expected": active_est}
    else:
        ach = fl_gu_rank / (us_gu * 1e-6) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"]}
    roof.update(traffic=None, kernel="gate_up grouped GEMM (per rank, timed eagerly between events)", us_per_launch=us_gu,
                peak_source=peaks["source"])
    # this library's kernels per layer pass.  Fixed-capacity path over peer memory: dispatch, gate_up, down (activation
    # applied on load), combine; over collectives: plan, offsets, gate_up, GLU, down, combine (torch index kernels and
    # NCCL's are not counted); exact-size path: gate_up, GLU, down, combine
    peer = any(m._peer for m in mods)
    # (large batches over peer memory: 4 plan kernels, push + wait each way, gate_up, GLU, down, combine = 12)
    launches_per_layer = (4 if peer else 6) if graph is not None else (12 if any(m._peer_large_buf for m in mods) else 4)
    peer_large = any(m._peer_large_buf for m in mods)
    exchange = ("peer memory: rows and counts stored straight into the destination ranks' buffers over NVLink by this "
                "library's kernels (8-byte words of payload + step number, bounded polls), no collective"
                if peer else
                "peer memory: blocks of rows stored into the destination ranks' symmetric buffers by this library's "
                "kernels (flags behind a fence, bounded waits); counts by one small all_gather and one host read"
                if peer_large else "collectives (all_to_all_single)")
    line = {
        "metric": "grouped 4-bit MoE GEMM us/layer", "value": us_layer, "unit": "us/layer", "n_gpus": world,
        "steps": K, "warmup": Wm, "ms_per_step": ms_layer / K, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 activations x 4-bit weights, fp32 accumulate", "data": "synthetic",
        "config": B.workload_config(shape, args.tokens, args.layers, world),
        "method": {"layers_resident": n_layers, "zipf": zipf, "timing": timing, "exchange": exchange},
        "e2e": {"value": ms_e2e * 1e3 / K, "unit": "us/layer",
                "h2d_bytes_per_step": args.tokens * (shape.hidden * 2 + shape.top_k * 12),
                "d2h_bytes_per_step": args.tokens * shape.hidden * 2},
        "gpu_launches": launches_per_layer * K,
        "roofline": roof,
        "ep": {"parity": parity, "phase_us_median": {n: statistics.median(v) for n, v in phase.items()},
               "rows_per_rank_mean": rows_mean, "rows_per_rank_max": tmax[2].item(),
               "imbalance_max_over_mean": tmax[2].item() / max(rows_mean, 1e-9),
               "aggregate_tflops": fl / (us_layer * 1e-6) / 1e12,
               # the layer on ONE GPU that holds all experts and has no partner (one resident layer, K steps in a
               # graph, max over ranks), and what fraction of the N-GPU layer time that is
               "single_gpu_layer_us": single_us,
               "efficiency_vs_single_gpu": (single_us / us_layer) if single_us else None},
        "clocks": clk.summary(), "device_status": nf4_grouped.last_status(dev),
    }
    return line
