"""Expert-parallel exchange logic on two CPU ranks (gloo): routing sort, count exchange,
dispatch, expert-major regroup, combine and weighted sum must reproduce the single-process
layer bit for bit.  The grouped GEMM is replaced by the CPU oracle here (the product has no
CPU path); the exchange code is the same code the GPUs run."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import ep_moe
import synth
from oracle import oracle as O


def _oracle_grouped(fmt):
    """The grouped GEMM's contract on the CPU: groups by sizes or by offsets, padding groups (expert id -1)
    skipped with their output rows left alone (zero here)."""
    def fn(a_cat, W, S, sizes, eids, group_offsets=None, max_rows=None):
        if group_offsets is not None:
            off = group_offsets.tolist()
            sizes = [off[i + 1] - off[i] for i in range(len(off) - 1)]
        sizes = [int(v) for v in sizes]
        eids = [int(v) for v in (eids.tolist() if torch.is_tensor(eids) else eids)]
        out = torch.zeros(a_cat.shape[0], W.shape[1], dtype=torch.bfloat16)
        row = 0
        for n, e in zip(sizes, eids):
            if n and e != ep_moe.PAD_EXPERT:
                ref = O.gemm_grouped_f64(fmt, a_cat[row:row + n].float().numpy(), W.numpy(), S.numpy(), [n], [e])
                out[row:row + n] = torch.from_numpy(ref).to(torch.float32).to(torch.bfloat16)
            row += n
        return out
    return fn


def _problem(fmt="nf4"):
    E, H, I, k, M = 8, 128, 64, 2, 24
    gen = torch.Generator().manual_seed(3)
    if fmt == "nf4":
        gu = synth.nf4_stack(E, 2 * I, H, gen, scale=0.5)
        dn = synth.nf4_stack(E, H, I, gen, scale=0.5)
    else:
        gu = synth.mxfp4_stack(E, 2 * I, H, gen, e_lo=124, e_hi=127)
        dn = synth.mxfp4_stack(E, H, I, gen, e_lo=124, e_hi=127)
    return E, H, I, k, M, gu, dn


def _tokens(rank, E, H, k, M):
    gen = torch.Generator().manual_seed(100 + rank)
    logits = torch.randn(M, E, generator=gen)
    logits[0] = 0.0                                   # ties -> lowest expert ids
    x = torch.randn(M, H, generator=gen).to(torch.bfloat16)
    idx, w = synth.route_topk(logits, k)
    return x, idx, w


def _worker(rank, world, port, fmt, out_q, mode="regroup"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if mode != "fixed":
        ep_moe.FIXED_CAPACITY_MAX_BYTES = 0       # exact-size exchange (one host read per layer)
    if mode in ("blocks", "split_blocks"):
        ep_moe.BLOCK_GROUPS_MIN_ROWS = 0          # multiply the (source, expert) blocks where they landed
    if mode.startswith("split"):
        ep_moe.SPLIT_MIN_TOKENS = 1               # the layer pipelined over the two halves of the local experts
    try:
        E, H, I, k, M, gu, dn = _problem(fmt)
        el = E // world

        def shard(t):
            return t[0][rank * el:(rank + 1) * el].contiguous(), t[1][rank * el:(rank + 1) * el].contiguous()

        layer = ep_moe.EPGroupedMoE(E, shard(gu), shard(dn), grouped_fn=_oracle_grouped(fmt), fmt=fmt,
                                    split_experts=mode.startswith("split"))
        x, idx, w = _tokens(rank, E, H, k, M)
        y = layer.forward(x, idx, w)
        out_q.put((rank, y.view(torch.int16).numpy().copy(), layer.last_rows))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("fmt,mode", [("nf4", "regroup"), ("mxfp4", "regroup"), ("nf4", "blocks"), ("nf4", "fixed"),
                                      ("mxfp4", "fixed"), ("nf4", "split_regroup"), ("nf4", "split_blocks")])
def test_two_rank_layer_equals_single_process_layer(fmt, mode):
    """All ways of exchanging and grouping -- exact-size exchange with rows regrouped expert-major, the same with
    one group per (source rank, expert) block as the rows arrived, both again as two exchanges over the two halves
    of the local experts, and the fixed-capacity exchange with padding groups and no host read -- must reproduce
    the single-process layer bit for bit."""
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fmt, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(world):
        r, y, rows = q.get(timeout=180)
        got[r] = (y, rows)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-process layer over the full stacks, same tokens
    E, H, I, k, M, gu, dn = _problem(fmt)
    single = ep_moe.EPGroupedMoE(E, gu, dn, grouped_fn=_oracle_grouped(fmt), fmt=fmt)
    total_rows = 0
    for r in range(world):
        x, idx, w = _tokens(r, E, H, k, M)
        want = single.forward(x, idx, w)
        assert np.array_equal(got[r][0], want.view(torch.int16).numpy()), f"rank {r}"
        total_rows += got[r][1]
    if mode != "fixed":
        assert total_rows == world * M * k      # every pair landed on exactly one rank


def test_plan_and_regroup_are_exact():
    """Integer bookkeeping against the oracle's routing restatement."""
    gen = torch.Generator().manual_seed(5)
    E, Wn, k = 16, 4, 3
    logits = torch.randn(40, E, generator=gen)
    idx, _ = synth.route_topk(logits, k)
    order, tok, counts = ep_moe.plan_dispatch(idx, E, Wn)
    o_ref, c_ref = O.sort_pairs(idx.reshape(-1).numpy(), E)
    assert np.array_equal(order.numpy(), o_ref) and np.array_equal(counts.reshape(-1).numpy(), c_ref)
    assert np.array_equal(tok.numpy(), o_ref // k)
    oi, _ = O.route_topk(logits.numpy(), k)
    assert np.array_equal(idx.numpy(), oi)
    rc = torch.tensor([[2, 0, 1], [1, 3, 0]], dtype=torch.int32)       # 2 sources, 3 local experts
    perm, sizes = ep_moe.regroup_index(rc)
    # source-major rows: s0:[e0,e0,e2] s1:[e0,e1,e1,e1]  -> expert-major: e0:{0,1,3} e1:{4,5,6} e2:{2}
    assert perm.tolist() == [0, 1, 3, 4, 5, 6, 2] and sizes.tolist() == [3, 3, 1]
    perm0, sizes0 = ep_moe.regroup_index(torch.zeros(2, 3, dtype=torch.int32))
    assert perm0.numel() == 0 and sizes0.tolist() == [0, 0, 0]


def test_combine_rows_is_the_ordered_weighted_sum():
    gen = torch.Generator().manual_seed(9)
    M, k, H = 7, 3, 16
    rows = torch.randn(M * k, H, generator=gen).to(torch.bfloat16)
    pos = torch.randperm(M * k, generator=gen).reshape(M, k)
    w = torch.rand(M, k, generator=gen)
    got = ep_moe.combine_rows(rows, pos, w)
    want = torch.zeros(M, H)
    for j in range(k):
        want = want + rows[pos[:, j]].float() * w[:, j, None]
    assert torch.equal(got, want.to(torch.bfloat16))
