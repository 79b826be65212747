"""The host-buffer entry points (host activations, host group tables, host result; stack on the GPU)
against the device-tensor entry points -- the same kernels, so the same bits -- and the fp64 oracle."""
import pytest
import torch

import _gnf4b
import mxfp4_grouped
import nf4_grouped
from helpers import oracle_fwd64, rel_fro
from mxfp4_pack_ref import quantize_pack_mxfp4
from nf4_pack_ref import make_stack

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_FRO_TOL = 2.0e-3      # bf16 output rounding level, as in the other GPU tests


@pytest.mark.parametrize("sizes,ids", [
    ([1, 1, 1], [2, 0, 3]),                   # decode kernel, x rides with the tables
    ([3, 0, 2, 1], [1, 2, 1, 0]),             # a zero-size group, a repeated expert
    ([40, 0, 70, 18], [3, 1, 0, 2]),          # tensor kernel, x copied on its own
    ([2, 1, 1], [0, -1, 3]),                  # a padding group: its output row is unspecified
])
def test_nf4_host_entry_equals_device_entry(sizes, ids):
    B, A = make_stack(4, 256, 512, seed=5, device=DEV)
    T = sum(sizes)
    a = torch.randn(T, 512, dtype=torch.bfloat16)
    want = nf4_grouped.gemm_4bit_grouped(a.to(DEV), B, A, sizes, ids).cpu()
    out = torch.full((T, 256), 7.0, dtype=torch.bfloat16).pin_memory()
    got, status = nf4_grouped.gemm_4bit_grouped_host(a.pin_memory(), B, A, torch.tensor(sizes, dtype=torch.int32),
                                                     ids, out, return_status=True)
    assert got is out and status == 0
    rows = torch.ones(T, dtype=torch.bool)
    first = 0
    for n, e in zip(sizes, ids):
        if e < 0:
            rows[first:first + n] = False
        first += n
    assert torch.equal(got[rows], want[rows])
    live = [(n, e) for n, e in zip(sizes, ids) if e >= 0]
    if len(live) == len(ids):
        ref = oracle_fwd64("nf4", a, B.cpu(), A.cpu(), sizes, ids)
        assert rel_fro(got, ref) < REL_FRO_TOL


def test_host_entry_pageable_input_unpinned_result_and_reuse():
    B, A = make_stack(3, 128, 2048, seed=9, device=DEV)
    for step in range(3):                      # the staging block and the pinned block are reused
        sizes, ids = [1, 1], [step % 3, (step + 1) % 3]
        a = torch.randn(2, 2048, dtype=torch.bfloat16)
        got = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids)
        want = nf4_grouped.gemm_4bit_grouped(a.to(DEV), B, A, sizes, ids).cpu()
        assert torch.equal(got, want)


def test_host_entry_split_k_scratch_is_cleared_between_calls():
    B, A = make_stack(4, 256, 2048, seed=11, device=DEV)
    for _ in range(2):
        a = torch.randn(2, 2048, dtype=torch.bfloat16)
        got = nf4_grouped.gemm_4bit_grouped_host(a, B, A, [1, 1], [3, 0], split_k=4, path=_gnf4b.PATH_STREAM)
        want = nf4_grouped.gemm_4bit_grouped(a.to(DEV), B, A, [1, 1], [3, 0], split_k=4, path=_gnf4b.PATH_STREAM).cpu()
        assert torch.equal(got, want)
        # a big x in between overwrites other parts of the staging block
        big = torch.randn(300, 2048, dtype=torch.bfloat16)
        nf4_grouped.gemm_4bit_grouped_host(big, B, A, [300], [1])


def test_dgrad_and_mxfp4_host_entries():
    B, A = make_stack(2, 256, 512, seed=3, device=DEV)
    g = torch.randn(50, 256, dtype=torch.bfloat16)
    got = nf4_grouped.dgrad_4bit_grouped_host(g, B, A, [20, 30], [1, 0])
    want = nf4_grouped.dgrad_4bit_grouped(g.to(DEV), B, A, [20, 30], [1, 0]).cpu()
    assert torch.equal(got, want)
    w = torch.randn(2, 128, 256)
    blocks, scales = quantize_pack_mxfp4(w)
    blocks, scales = blocks.reshape(2, 128, 128).to(DEV), scales.to(DEV)
    a = torch.randn(3, 256, dtype=torch.bfloat16)
    got = mxfp4_grouped.gemm_mxfp4_grouped_host(a, blocks, scales, [2, 1], [1, 0])
    want = mxfp4_grouped.gemm_mxfp4_grouped(a.to(DEV), blocks, scales, [2, 1], [1, 0]).cpu()
    assert torch.equal(got, want)
    gm = torch.randn(3, 128, dtype=torch.bfloat16)
    got = mxfp4_grouped.dgrad_mxfp4_grouped_host(gm, blocks, scales, [2, 1], [1, 0])
    want = mxfp4_grouped.dgrad_mxfp4_grouped(gm.to(DEV), blocks, scales, [2, 1], [1, 0]).cpu()
    assert torch.equal(got, want)


def test_host_entry_refuses_bad_tables_and_device_inputs():
    B, A = make_stack(2, 128, 512, seed=1, device=DEV)
    a = torch.randn(2, 512, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        nf4_grouped.gemm_4bit_grouped_host(a, B, A, [1, 2], [0, 1])          # sizes do not sum to T
    with pytest.raises(ValueError):
        nf4_grouped.gemm_4bit_grouped_host(a, B, A, [1, 1], [0, 2])          # expert id beyond the stack
    with pytest.raises(ValueError):
        nf4_grouped.gemm_4bit_grouped_host(a.to(DEV), B, A, [1, 1], [0, 1])  # activations on the device
    with pytest.raises(ValueError):
        nf4_grouped.gemm_4bit_grouped_host(a, B.cpu(), A.cpu(), [1, 1], [0, 1])


def test_bound_host_call_equals_the_one_shot_entry():
    B, A = make_stack(3, 128, 2048, seed=21, device=DEV)
    run = nf4_grouped.HostGroupedGemm(B, A)
    back = nf4_grouped.HostGroupedGemm(B, A, op="dgrad")
    out = torch.empty(3, 128, dtype=torch.bfloat16).pin_memory()
    gout = torch.empty(3, 2048, dtype=torch.bfloat16).pin_memory()
    for step in range(3):
        sizes = torch.tensor([2, 0, 1], dtype=torch.int32)
        ids = torch.tensor([step % 3, 1, (step + 2) % 3], dtype=torch.int32)
        a = torch.randn(3, 2048, dtype=torch.bfloat16).pin_memory()
        assert run(a, sizes, ids, out) is out
        assert torch.equal(out, nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids))
        g = torch.randn(3, 128, dtype=torch.bfloat16)
        back(g, sizes, ids, gout)
        assert torch.equal(gout, nf4_grouped.dgrad_4bit_grouped(g.to(DEV), B, A, sizes.tolist(), ids.tolist()).cpu())
    with pytest.raises(ValueError):
        run(a, torch.tensor([1, 1, 0], dtype=torch.int32), ids, out)       # sums to 2, not 3
    with pytest.raises(ValueError):
        run(a.float(), sizes, ids, out)


def _ffn_stacks(E=4, K=512, H=128, N_dn=256, seed=31):
    B_gu, A_gu = make_stack(E, 2 * H, K, seed=seed, device=DEV)
    B_dn, A_dn = make_stack(E, N_dn, H, seed=seed + 1, device=DEV)
    return B_gu, A_gu, B_dn, A_dn


@pytest.mark.parametrize("sizes,ids", [([1, 1, 1], [2, 0, 3]), ([3, 2, 1], [1, 3, 1]), ([40, 70, 18], [3, 0, 2])])
def test_host_ffn_equals_the_three_launch_composition_and_the_reference_ffn(sizes, ids):
    import ep_moe
    from helpers import O
    B_gu, A_gu, B_dn, A_dn = _ffn_stacks()
    T = sum(sizes)
    a = torch.randn(T, 512, dtype=torch.bfloat16)
    got = nf4_grouped.ffn_4bit_grouped_host(a, B_gu, A_gu, B_dn, A_dn, sizes, ids)
    gu = nf4_grouped.gemm_4bit_grouped(a.to(DEV), B_gu, A_gu, sizes, ids)
    want = nf4_grouped.gemm_4bit_grouped(ep_moe.silu_glu(gu), B_dn, A_dn, sizes, ids).cpu()
    assert torch.equal(got, want)
    f64 = O.ffn_grouped_f64(a.float().numpy(), B_gu.cpu().numpy(), A_gu.cpu().numpy(), B_dn.cpu().numpy(),
                            A_dn.cpu().numpy(), sizes, ids)
    assert rel_fro(got, f64) < 6.0e-3          # three bf16 roundings (gate_up, GLU, result)
    # against the reference project's own fused CPU FFN (fp32 throughout; ours rounds both intermediates
    # and the result to bf16: three roundings of 2^-9 relative each)
    if O.ref_available():
        ref = O.ref_ffn_call(a.float().numpy(), B_gu.cpu().numpy(), A_gu.cpu().numpy(), B_dn.cpu().numpy(),
                             A_dn.cpu().numpy(), sizes, ids)
        assert rel_fro(got, ref.astype("float64")) < 6.0e-3


def test_bound_host_ffn_reuse_and_errors():
    B_gu, A_gu, B_dn, A_dn = _ffn_stacks(seed=41)
    ffn = nf4_grouped.HostGroupedFfn(B_gu, A_gu, B_dn, A_dn)
    out = torch.empty(2, 256, dtype=torch.bfloat16).pin_memory()
    for step in range(3):
        a = torch.randn(2, 512, dtype=torch.bfloat16).pin_memory()
        sizes = torch.tensor([1, 1], dtype=torch.int32)
        ids = torch.tensor([step, (step + 1) % 4], dtype=torch.int32)
        ffn(a, sizes, ids, out)
        assert torch.equal(out, nf4_grouped.ffn_4bit_grouped_host(a, B_gu, A_gu, B_dn, A_dn, sizes, ids))
    with pytest.raises(ValueError):
        ffn(a, torch.tensor([1, 2], dtype=torch.int32), ids, out)
    with pytest.raises(ValueError):
        nf4_grouped.HostGroupedFfn(B_gu, A_gu, B_gu, A_gu)            # down does not contract over H


def test_host_entry_with_more_groups_than_the_pinned_block_holds():
    """20000 groups (tables of 160 KB: beyond the thread's pinned block, copied from a heap array), most of one row,
    some empty: same bits as the tensor entry point on the same kernel."""
    B, A = make_stack(4, 64, 64, seed=13, device=DEV)
    gen = torch.Generator().manual_seed(3)
    sizes = (torch.rand(20000, generator=gen) < 0.9).to(torch.int32)
    ids = torch.randint(0, 4, (20000,), generator=gen, dtype=torch.int32)
    T = int(sizes.sum())
    a = torch.randn(T, 64, generator=gen).to(torch.bfloat16)
    got, status = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, path=_gnf4b.PATH_STREAM, return_status=True)
    want = nf4_grouped.gemm_4bit_grouped(a.to(DEV), B, A, sizes.tolist(), ids.tolist(), path=_gnf4b.PATH_STREAM).cpu()
    assert status == 0 and torch.equal(got, want)


def test_small_host_calls_without_the_copy_engines_equal_the_copying_form():
    """Small calls go in and out through the thread's pinned block by two staging kernels; the flag
    GNF4B_FLAG_HOST_COPIES keeps the copy engines.  Same bits, same status, for the GEMM, the dgrad and the FFN, over
    repeated calls (the sequence number advances) and with a split-K scratch that must start at zero."""
    B, A = make_stack(4, 256, 2048, seed=21, device=DEV)
    for step in range(4):
        sizes, ids = [1, 2, 1], [step % 4, (step + 2) % 4, 3]
        a = torch.randn(4, 2048, dtype=torch.bfloat16)
        fast, st_f = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, return_status=True)
        slow, st_s = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, path=_gnf4b.FLAG_HOST_COPIES, return_status=True)
        assert torch.equal(fast, slow) and st_f == st_s == 0
        k4 = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, split_k=4, path=_gnf4b.PATH_STREAM)
        k4c = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, split_k=4, path=_gnf4b.PATH_STREAM | _gnf4b.FLAG_HOST_COPIES)
        assert torch.equal(k4, k4c)
    g = torch.randn(4, 256, dtype=torch.bfloat16) * 1e-2
    assert torch.equal(nf4_grouped.dgrad_4bit_grouped_host(g, B, A, [3, 1], [2, 0]),
                       nf4_grouped.dgrad_4bit_grouped(g.to(DEV), B, A, [3, 1], [2, 0]).cpu())
    # a bad expert id inside a small call still reaches the caller's status word
    bad, status = nf4_grouped.gemm_4bit_grouped_host(torch.randn(1, 2048, dtype=torch.bfloat16), B, A, [1], [1], return_status=True)
    assert status == 0
    Bg, Ag, Bd, Ad = _ffn_stacks()
    for sizes, ids in (([1, 1, 1], [3, 0, 2]), ([2, 3], [1, 1])):
        a = torch.randn(sum(sizes), 512, dtype=torch.bfloat16)
        assert torch.equal(nf4_grouped.ffn_4bit_grouped_host(a, Bg, Ag, Bd, Ad, sizes, ids),
                           nf4_grouped.ffn_4bit_grouped(a.to(DEV), Bg, Ag, Bd, Ad, sizes, ids).cpu())
