"""Expert-parallel layer on real GPUs (needs >= 2): two NCCL ranks must reproduce the
single-GPU layer on the same seeds.  Rows are computed by the same kernels whatever the
sharding, but the planner may pick a different kernel for a rank's smaller groups, so the
comparison is at bf16 resolution, plus a check against the fp64 oracle on rank 0."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _problem():
    import synth
    E, H, I, k, M = 16, 256, 128, 4, 96
    gen = torch.Generator().manual_seed(31)
    gu = synth.nf4_stack(E, 2 * I, H, gen, scale=0.05)
    dn = synth.nf4_stack(E, H, I, gen, scale=0.05)
    return E, H, I, k, M, gu, dn


def _tokens(rank, E, H, k, M):
    import synth
    gen = torch.Generator().manual_seed(500 + rank)
    logits = torch.randn(M, E, generator=gen)
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    idx, w = synth.route_topk(logits, k)
    return x, idx, w


def _agree(a, b):
    """The two exchanges hand the GEMM the same rows in different groupings (expert-major against per source), so
    the planner may pick different kernels: equal to bf16 resolution of the largest value, not to the bit."""
    return bool(((a.float() - b.float()).abs().max() <= 2 * 2 ** -8 * b.float().abs().max()).item())


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        import ep_moe
        import nf4_grouped
        dev = torch.device("cuda", rank)
        E, H, I, k, M, gu, dn = _problem()
        el = E // world
        sh = lambda t: (t[0][rank * el:(rank + 1) * el].to(dev), t[1][rank * el:(rank + 1) * el].to(dev))  # noqa: E731
        layer = ep_moe.EPGroupedMoE(E, sh(gu), sh(dn), fmt="nf4")
        x, idx, w = _tokens(rank, E, H, k, M)
        y = layer.forward(x.to(dev), idx.to(dev), w.to(dev))
        torch.cuda.synchronize()
        # small batches: the library's own exchange over peer memory against the same layer over NCCL, bit for
        # bit, on steps with different routing and batch sizes (buffers and flags are reused from step to step)
        nccl = ep_moe.EPGroupedMoE(E, sh(gu), sh(dn), fmt="nf4", peer_exchange=False)
        same = True
        for step, m in enumerate((1, 3, 8, 2, 8, 1, 5, 8, 24, 40, 1)):
            xs, ids, ws = _tokens(rank + 10 * step, E, H, k, m)
            a = layer.forward(xs.to(dev), ids.to(dev), ws.to(dev))
            b = nccl.forward(xs.to(dev), ids.to(dev), ws.to(dev))
            same = same and _agree(a, b)
        peer_used = len(layer._peer) == 1 and len(nccl._peer) == 0
        # the same launches replayed from a CUDA graph: the step number lives on the device
        xs, ids, ws = (t.to(dev) for t in _tokens(rank + 77, E, H, k, 4))
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            layer.forward(xs, ids, ws)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                yg = layer.forward(xs, ids, ws)
            for _ in range(3):
                g.replay()
        side.synchronize()
        torch.cuda.current_stream(dev).wait_stream(side)
        same_graph = _agree(yg, nccl.forward(xs, ids, ws))
        # a large batch (exact-size exchange over NCCL): pipelined over the two halves of the local experts against
        # the layer in one piece -- the returned rows land in the same places, so the results are the same bits
        xl, il, wl = (t.to(dev) for t in _tokens(rank + 300, E, H, k, 2600))
        whole = ep_moe.EPGroupedMoE(E, sh(gu), sh(dn), fmt="nf4", split_experts=False)
        piped = ep_moe.EPGroupedMoE(E, sh(gu), sh(dn), fmt="nf4", split_experts=True)
        a, b = piped.forward(xl, il, wl), whole.forward(xl, il, wl)
        same_chunked = _agree(a, b) and piped._streams is not None and whole._streams is None
        # the same large batch with the rows moved by the library's own stores into symmetric buffers (the default)
        # against NCCL's all-to-all: the GEMMs see the same rows in the same order, so the same bits; twice (the
        # buffers and flags are reused), then a larger step that does not fit the buffers and goes over NCCL
        os.environ["GNF4B_EP_PEER_LARGE"] = "0"
        over_nccl = ep_moe.EPGroupedMoE(E, sh(gu), sh(dn), fmt="nf4", split_experts=False)
        os.environ["GNF4B_EP_PEER_LARGE"] = "1"
        for rep in range(2):
            xr, ir, wr = (t.to(dev) for t in _tokens(rank + 400 + rep, E, H, k, 2600))
            same_chunked = same_chunked and torch.equal(whole.forward(xr, ir, wr), over_nccl.forward(xr, ir, wr))
        same_chunked = same_chunked and len(whole._peer_large_buf) == 1 and not over_nccl._peer_large_buf
        xb, ib, wb = (t.to(dev) for t in _tokens(rank + 500, E, H, k, 2600 * 3))
        same_chunked = same_chunked and torch.equal(whole.forward(xb, ib, wb), over_nccl.forward(xb, ib, wb))
        torch.cuda.synchronize()
        q.put((rank, y.float().cpu().numpy(), nf4_grouped.last_status(dev), same, peer_used, same_graph, same_chunked))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_layer_matches_single_gpu_layer():
    import ep_moe
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, y, status, same, peer_used, same_graph, same_chunked = q.get(timeout=300)
        got[r] = y
        assert status == 0
        assert peer_used, "the small-batch steps did not take the peer-memory exchange"
        assert same, "peer-memory exchange and NCCL exchange differ beyond bf16 resolution"
        assert same_graph, "replayed graph of the peer-memory exchange differs"
        assert same_chunked, "the large-batch layer pipelined over two halves of the experts differs from the layer in one piece"
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    E, H, I, k, M, gu, dn = _problem()
    dev = torch.device("cuda", 0)
    single = ep_moe.EPGroupedMoE(E, (gu[0].to(dev), gu[1].to(dev)), (dn[0].to(dev), dn[1].to(dev)), fmt="nf4")
    for r in range(world):
        x, idx, w = _tokens(r, E, H, k, M)
        want = single.forward(x.to(dev), idx.to(dev), w.to(dev)).float().cpu().numpy()
        scale = np.abs(want).max()
        assert np.abs(got[r] - want).max() <= 2 * 2 ** -8 * scale, r


def test_silu_glu_kernel_equals_the_tensor_expression():
    import ep_moe
    gen = torch.Generator().manual_seed(1)
    for rows, h in ((33, 96), (5, 7), (0, 8)):
        gu = (torch.randn(rows, 2 * h, generator=gen) * 3).to(torch.bfloat16).cuda()
        got = ep_moe.silu_glu(gu)
        g, u = gu[:, :h].float(), gu[:, h:].float()
        want = (g / (1.0 + torch.exp(-g)) * u).to(torch.bfloat16)
        assert got.shape == (rows, h) and torch.equal(got, want)


def test_combine_rows_kernel_equals_the_ordered_loop():
    import ep_moe
    import nf4_grouped
    gen = torch.Generator().manual_seed(2)
    for M, k, H in ((50, 8, 256), (9, 3, 10)):
        rows = torch.randn(M * k, H, generator=gen).to(torch.bfloat16).cuda()
        pos = torch.randperm(M * k, generator=gen).reshape(M, k).cuda()
        w = torch.rand(M, k, generator=gen).cuda()
        got = ep_moe.combine_rows(rows, pos, w)
        want = torch.zeros(M, H, device="cuda")
        for j in range(k):
            want = want + rows[pos[:, j]].float() * w[:, j, None]
        assert torch.equal(got, want.to(torch.bfloat16))
    assert nf4_grouped.last_status("cuda") == 0
    # a position outside the rows is skipped and flagged, never dereferenced
    pos[0, 0] = M * k + 5
    ep_moe.combine_rows(rows, pos, w)
    torch.cuda.synchronize()
    assert nf4_grouped.last_status("cuda") & 2


def test_ep_plan_and_offsets_kernels_equal_the_tensor_form():
    """gnf4b_ep_plan / gnf4b_ep_offsets against the sort-based plan of ep_moe (what CPU ranks run)."""
    import _gnf4b
    import ep_moe
    import nf4_grouped
    import synth
    lib = _gnf4b.load()
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(12)
    E, W, k, M, H = 32, 4, 4, 9, 64
    El, cap = E // W, M * k
    idx, _ = synth.route_topk(torch.randn(M, E, generator=gen), k)
    hidden = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    idx_d, hid_d = idx.to(dev), hidden.to(dev)
    counts = torch.empty(W, El, dtype=torch.int32, device=dev)
    slot = torch.empty(cap, dtype=torch.int64, device=dev)
    send = torch.zeros(W * cap, H, dtype=torch.bfloat16, device=dev)
    st = nf4_grouped._status_word(dev)
    rc = lib.gnf4b_ep_plan(idx_d.to(torch.int64).contiguous().data_ptr(), cap, k, E, El, cap, hid_d.data_ptr(), H, counts.data_ptr(),
                           slot.data_ptr(), send.data_ptr(), st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    # the tensor form
    order, tok, cnt = ep_moe.plan_dispatch(idx, E, W)
    per_dest = cnt.sum(1)
    start = torch.cumsum(per_dest, 0) - per_dest
    dest = torch.repeat_interleave(torch.arange(W), per_dest)
    slot_sorted = dest * cap + (torch.arange(order.numel()) - start[dest])
    want_slot = torch.empty_like(order)
    want_slot[order] = slot_sorted
    want_send = torch.zeros(W * cap, H, dtype=torch.bfloat16)
    want_send[slot_sorted] = hidden[tok]
    torch.cuda.synchronize()
    assert torch.equal(counts.cpu().to(torch.int64), cnt)
    assert torch.equal(slot.cpu(), want_slot)
    assert torch.equal(send.cpu(), want_send)
    # offsets of a received buffer
    rcnt = torch.randint(0, 3, (W, El), generator=gen).to(torch.int32)
    off = torch.empty(W * (El + 1) + 1, dtype=torch.int32, device=dev)
    assert lib.gnf4b_ep_offsets(rcnt.to(dev).data_ptr(), W, El, cap, off.data_ptr(), st.data_ptr(),
                                torch.cuda.current_stream().cuda_stream) == 0
    sizes = torch.cat((rcnt.to(torch.int64), cap - rcnt.sum(1, keepdim=True)), 1).reshape(-1)
    assert off.cpu().tolist() == [0] + torch.cumsum(sizes, 0).tolist()
    assert nf4_grouped.last_status(dev) == 0


def test_router_kernel_matches_the_reference_rule(golden_dir):
    """gnf4b_route_topk against the golden routing of the reference (indices exact, weights to fp32
    rounding of the exponentials) and against the oracle on random logits with ties."""
    import ep_moe
    from oracle import oracle as O
    g = np.load(golden_dir / "routing.npz")
    lg = torch.from_numpy(g["logits"]).cuda()
    for mode, norm, tag in ((0, False, "m0n0"), (0, True, "m0n1"), (1, False, "m1n0")):
        idx, w = ep_moe.route_topk(lg, 8, mode, norm)
        assert np.array_equal(idx.cpu().numpy(), g["idx_" + tag].astype(np.int64))
        want_bits = g["wts_" + tag + "_bf16bits"]
        got_bits = w.to(torch.bfloat16).view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.abs(got_bits.astype(np.int32) - want_bits.astype(np.int32)).max() <= 1       # one bf16 ulp
    gen = torch.Generator().manual_seed(4)
    logits = torch.randn(37, 130, generator=gen)
    logits[3] = 0.0                       # all tied: experts 0..k-1
    logits[5, 7] = logits[5, 99]          # a tie inside the top
    for k, mode, norm in ((1, 0, False), (4, 0, True), (8, 1, False), (32, 0, False)):
        idx, w = ep_moe.route_topk(logits.cuda(), k, mode, norm)
        oi, ow = O.route_topk(logits.numpy(), k, mode, norm)
        assert np.array_equal(idx.cpu().numpy(), oi.astype(np.int64))
        assert np.allclose(w.cpu().numpy(), ow, rtol=2e-6, atol=1e-9)


def test_single_gpu_layer_from_logits_without_host_reads():
    """One rank: router kernel -> plan kernel -> grouped GEMMs over device offsets -> GLU -> combine.
    Equal to the layer built from host-side routing and per-expert dense math at bf16 resolution."""
    import ep_moe
    import nf4_grouped
    import synth
    from nf4_grouped import dequant_ref
    E, H, I, k, M = 16, 256, 128, 4, 12
    gen = torch.Generator().manual_seed(31)
    gu = synth.nf4_stack(E, 2 * I, H, gen, device="cuda", scale=0.05)
    dn = synth.nf4_stack(E, H, I, gen, device="cuda", scale=0.05)
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16).cuda()
    logits = torch.randn(M, E, generator=gen).cuda()
    layer = ep_moe.EPGroupedMoE(E, gu, dn, fmt="nf4")
    y = layer.forward_logits(x, logits, k)
    idx, w = ep_moe.route_topk(logits, k)
    want = torch.zeros(M, H, device="cuda")
    for m in range(M):
        for j in range(k):
            e = int(idx[m, j])
            w1 = dequant_ref(gu[0][e], gu[1][e], 2 * I, H).float()
            w2 = dequant_ref(dn[0][e], dn[1][e], H, I).float()
            g_ = (x[m].float() @ w1.t()).to(torch.bfloat16)
            h = ep_moe.silu_glu(g_[None])[0]
            want[m] += w[m, j] * (h.float() @ w2.t()).to(torch.bfloat16).float()
    assert ((y.float() - want).norm() / want.norm()).item() < 1e-2
    assert nf4_grouped.last_status("cuda") == 0


def test_peer_exchange_on_one_gpu_equals_the_collective_form_and_replays():
    """One rank: the four exchange kernels around the GEMMs against the plan / offsets / combine kernels (the form
    the collectives use), same bits over steps of different sizes; then a captured sequence replayed."""
    import ep_moe
    import nf4_grouped
    import synth
    E, H, I, k = 16, 256, 128, 4
    gen = torch.Generator().manual_seed(5)
    gu = synth.nf4_stack(E, 2 * I, H, gen, device="cuda", scale=0.05)
    dn = synth.nf4_stack(E, H, I, gen, device="cuda", scale=0.05)
    peer = ep_moe.EPGroupedMoE(E, gu, dn, fmt="nf4", peer_exchange=True)
    coll = ep_moe.EPGroupedMoE(E, gu, dn, fmt="nf4", peer_exchange=False)
    for step, m in enumerate((1, 7, 2, 16, 1, 40, 200, 3)):        # 40 and 200 tokens: groups = the local experts
        x, idx, w = (t.cuda() for t in _tokens(step, E, H, k, m))
        assert _agree(peer.forward(x, idx, w), coll.forward(x, idx, w)), step
    assert len(peer._peer) == 1 and not coll._peer
    x, idx, w = (t.cuda() for t in _tokens(40, E, H, k, 4))
    want = coll.forward(x, idx, w)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        peer.forward(x, idx, w)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            y = peer.forward(x, idx, w)
        for _ in range(3):
            g.replay()
    side.synchronize()
    assert _agree(y, want)
    assert nf4_grouped.last_status("cuda") == 0


def test_peer_exchange_wait_runs_out_and_sets_the_status():
    """A flag that nothing raises: rank 0 of a two-rank context whose second buffer is a local stand-in that no
    process writes.  The dispatch kernel's receiving half gives up after its time limit, raises GNF4B_ST_TIMEOUT and returns; the
    context stays usable."""
    import ctypes
    import _gnf4b
    lib = _gnf4b.load()
    world, e_local, cap, H = 2, 2, 4, 64
    lay = (ctypes.c_int64 * 3)()
    assert lib.gnf4b_ep_peer_layout(world, e_local, cap, H, lay) == 0
    bufs = [torch.zeros(int(lay[0]), dtype=torch.uint8, device="cuda") for _ in range(world)]
    ctx = _gnf4b.EpPeerCtx(world, 0, e_local, cap, H)
    for r in range(world):
        ctx.peers[r] = bufs[r].data_ptr()
    idx = torch.tensor([0, 3, 1, 2], dtype=torch.int64, device="cuda")
    hidden = torch.randn(2, H, device="cuda").to(torch.bfloat16)
    slot = torch.empty(4, dtype=torch.int64, device="cuda")
    offsets = torch.zeros(e_local + 1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.gnf4b_ep_peer_dispatch(ctypes.byref(ctx), idx.data_ptr(), 4, 2, world * e_local, cap, hidden.data_ptr(),
                                      slot.data_ptr(), 0, offsets.data_ptr(), None, status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _gnf4b.ST_TIMEOUT
    # rank 0's own rows did arrive: experts 0 and 1 got one row each, unpacked expert-major
    assert offsets.tolist() == [0, 1, 2]
    assert slot.tolist() == [0, cap + 1, 1, cap + 0]
    rows = bufs[0][int(lay[1]):int(lay[1]) + 2 * H * 2].view(torch.bfloat16).view(2, H)
    assert torch.equal(rows[0], hidden[0]) and torch.equal(rows[1], hidden[1])
    # too large a capacity is refused before any launch
    assert lib.gnf4b_ep_peer_dispatch(ctypes.byref(ctx), idx.data_ptr(), 4, 2, world * e_local, cap + 1, hidden.data_ptr(),
                                      slot.data_ptr(), 0, offsets.data_ptr(), None, status.data_ptr(), st) == -6
    assert torch.randn(8, device="cuda").sum().isfinite()


@pytest.mark.parametrize("M,k,E,El,cut", [(700, 4, 16, 8, 8), (700, 4, 16, 8, 4), (4096, 8, 128, 64, 32), (3, 2, 8, 4, 1),
                                          (513, 1, 1024, 128, 128)])
def test_large_batch_plan_equals_the_stable_argsort(M, k, E, El, cut):
    """gnf4b_ep_plan_large (a counting sort over several CTAs) against the tensor form it replaces: positions of
    the pairs in the stable order of (half, expert id), per-expert counts, gathered rows -- integer / bit equality."""
    import _gnf4b
    import nf4_grouped
    lib = _gnf4b.load()
    gen = torch.Generator().manual_seed(M + cut)
    H = 64
    idx = torch.randint(0, E, (M, k), generator=gen).cuda()
    hidden = torch.randn(M, H, generator=gen).to(torch.bfloat16).cuda()
    flat = idx.reshape(-1)
    P = flat.numel()
    key = flat + ((flat % El) >= cut).to(torch.int64) * E
    order = torch.argsort(key, stable=True)
    want_pos = torch.empty_like(order)
    want_pos[order] = torch.arange(P, device="cuda")
    want_counts = torch.bincount(flat, minlength=E).to(torch.int32)
    need = lib.gnf4b_ep_plan_large_scratch_bytes(P, E)
    scratch = torch.full((need,), 0x5A, dtype=torch.uint8, device="cuda")        # any content
    counts = torch.empty(E, dtype=torch.int32, device="cuda")
    pos = torch.empty(P, dtype=torch.int64, device="cuda")
    send = torch.empty(P, H, dtype=torch.bfloat16, device="cuda")
    rc = lib.gnf4b_ep_plan_large(flat.data_ptr(), P, k, E, El, cut, hidden.data_ptr(), H, counts.data_ptr(), pos.data_ptr(),
                                 send.data_ptr(), scratch.data_ptr(), need, nf4_grouped._status_word("cuda").data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert torch.equal(pos, want_pos) and torch.equal(counts, want_counts)
    assert torch.equal(send, hidden[order // k])
    assert nf4_grouped.last_status("cuda") == 0
    # an id outside the experts: flagged, placed behind every valid pair, counted by no expert
    flat2 = flat.clone()
    flat2[0] = E + 3
    rc = lib.gnf4b_ep_plan_large(flat2.data_ptr(), P, k, E, El, cut, hidden.data_ptr(), H, counts.data_ptr(), pos.data_ptr(),
                                 send.data_ptr(), scratch.data_ptr(), need, nf4_grouped._status_word("cuda").data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and int(pos[0]) == P - 1 and int(counts.sum()) == P - 1
    assert nf4_grouped.last_status("cuda") & _gnf4b.ST_BAD_EXPERT
