"""The expert FFN (gate_up GEMM -> activation -> down GEMM) as ONE fused launch for one-row groups, against the
three-launch composition (bit for bit: that is its contract), the reference's own fused CPU FFN and the fp64
FFN oracle; the gpt-oss activation against the reference's chain of bf16 tensor operations
(kernel/mxfp4_pipelined.py:453-461)."""
import numpy as np
import pytest
import torch

import _gnf4b
import ep_moe
import mxfp4_grouped
import nf4_grouped
import synth
from mxfp4_pack_ref import dequant_mxfp4
from nf4_grouped import dequant_ref, ffn_4bit_grouped, gemm_4bit_grouped
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_FRO_TOL = 4.0e-3      # three bf16 roundings in sequence (gate_up, activation, result), ~1.65e-3 each


def _clean():
    assert nf4_grouped.last_status(DEV) == 0


def _nf4_pair(E, N_gu, K_gu, N_dn, seed, bf16_absmax=False):
    gen = torch.Generator().manual_seed(seed)
    gu = synth.nf4_stack(E, N_gu, K_gu, gen, scale=0.05, device=DEV, fast=True, bf16_absmax=bf16_absmax)
    dn = synth.nf4_stack(E, N_dn, N_gu // 2, gen, scale=0.05, device=DEV, fast=True, bf16_absmax=bf16_absmax)
    return gu, dn


@pytest.mark.parametrize("N_gu,K_gu,N_dn,G", [(1536, 2048, 2048, 8), (256, 128, 64, 3), (512, 3072, 1024, 5),
                                              (4096, 1024, 512, 40), (128, 64, 8, 1)])
def test_fused_ffn_equals_three_launches_bitwise(N_gu, K_gu, N_dn, G):
    """Qwen3's layer shape at batch 1 and smaller / longer shapes; G one-row groups with repeated and unsorted
    experts.  The fused launch, the forced three-launch form and the explicit composition give the same bits."""
    E = 6
    (Bg, Ag), (Bd, Ad) = _nf4_pair(E, N_gu, K_gu, N_dn, seed=N_gu + G)
    gen = torch.Generator().manual_seed(G)
    ids = [int(v) for v in torch.randint(0, E, (G,), generator=gen)]
    sizes = [1] * G
    a = torch.randn(G, K_gu, generator=gen).to(torch.bfloat16).to(DEV)
    fused = ffn_4bit_grouped(a, Bg, Ag, Bd, Ad, sizes, ids)
    three = ffn_4bit_grouped(a, Bg, Ag, Bd, Ad, sizes, ids, fused=False)
    comp = gemm_4bit_grouped(ep_moe.silu_glu(gemm_4bit_grouped(a, Bg, Ag, sizes, ids)), Bd, Ad, sizes, ids)
    assert torch.equal(three, comp)
    assert torch.equal(fused, comp)
    # twice more on the same workspace: the kernel must have left its counters zeroed
    assert torch.equal(ffn_4bit_grouped(a, Bg, Ag, Bd, Ad, sizes, ids), comp)
    assert torch.equal(ffn_4bit_grouped(a, Bg, Ag, Bd, Ad, sizes, ids), comp)
    want = O.ffn_grouped_f64(a.float().cpu().numpy(), Bg.cpu().numpy(), Ag.cpu().numpy(), Bd.cpu().numpy(),
                             Ad.cpu().numpy(), sizes, ids)
    assert O.rel_frobenius(fused.double().cpu().numpy(), want) <= REL_FRO_TOL
    _clean()


def test_fused_ffn_device_tables_empty_and_padding_groups():
    """Device-side group tables (no host read), an empty group and a padding group in the list: the rows of real
    groups equal the composition, the padded row is left untouched."""
    E, N_gu, K_gu, N_dn = 4, 512, 256, 256
    (Bg, Ag), (Bd, Ad) = _nf4_pair(E, N_gu, K_gu, N_dn, seed=3, bf16_absmax=True)
    a = torch.randn(4, K_gu, device=DEV, dtype=torch.bfloat16)
    off = torch.tensor([0, 1, 1, 2, 3, 4], dtype=torch.int32, device=DEV)          # sizes 1, 0, 1, 1, 1
    ids = torch.tensor([2, 0, nf4_grouped.PAD_EXPERT, 3, 2], dtype=torch.int32, device=DEV)
    out = ffn_4bit_grouped(a, Bg, Ag, Bd, Ad, None, ids, group_offsets=off, max_rows=1)
    for row, e in ((0, 2), (2, 3), (3, 2)):
        comp = gemm_4bit_grouped(ep_moe.silu_glu(gemm_4bit_grouped(a[row:row + 1], Bg, Ag, [1], [e])), Bd, Ad, [1], [e])
        assert torch.equal(out[row:row + 1], comp), row
    _clean()


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (no reference checkout)")
def test_fused_ffn_against_the_reference_cpu_ffn():
    """The reference's own fused CPU kernel (fp32 in, fp32 out) on the same stacks: agreement at the level of the
    two bf16 roundings of the GPU path."""
    E, N_gu, K_gu, N_dn = 3, 256, 128, 64
    (Bg, Ag), (Bd, Ad) = _nf4_pair(E, N_gu, K_gu, N_dn, seed=51)
    sizes, ids = [1, 1, 1, 1], [2, 0, 1, 2]
    a = torch.randn(4, K_gu).to(torch.bfloat16)
    ref = O.ref_ffn_call(a.float().numpy(), Bg.cpu().numpy(), Ag.cpu().numpy(), Bd.cpu().numpy(), Ad.cpu().numpy(), sizes, ids)
    out = ffn_4bit_grouped(a.to(DEV), Bg, Ag, Bd, Ad, sizes, ids)
    assert O.rel_frobenius(out.double().cpu().numpy(), ref.astype(np.float64)) <= 2 ** -7
    _clean()


def _torch_glu_gpt_oss(gu, alpha=1.702, limit=7.0):
    """The reference's _glu, verbatim semantics: bf16 tensor operations."""
    gate, up = gu[..., ::2], gu[..., 1::2]
    gate = gate.clamp(max=limit)
    up = up.clamp(min=-limit, max=limit)
    return (up + 1) * (gate * torch.sigmoid(gate * alpha))


def test_glu_gpt_oss_kernel_equals_the_bf16_tensor_chain():
    gen = torch.Generator().manual_seed(9)
    gu = (torch.randn(37, 2 * 96, generator=gen) * 4).to(torch.bfloat16).to(DEV)
    gu[0, :8] = torch.tensor([9, -9, 7, 7.5, -7.5, 0, 100, -100], dtype=torch.bfloat16)
    got = mxfp4_grouped.glu_gpt_oss(gu)
    want = _torch_glu_gpt_oss(gu)
    diff = (got.float() - want.float()).abs()
    # the device exp and torch's may differ in the last fp32 bit: at most one bf16 ulp, and almost nowhere
    assert (diff <= 2 ** -7 * want.float().abs() + 1e-30).all()
    assert (got != want).float().mean().item() < 0.01
    bias = (torch.randn(5, 2 * 96, generator=gen)).to(torch.bfloat16).to(DEV)
    rows = torch.randint(0, 5, (37,), generator=gen).to(DEV)
    got_b = mxfp4_grouped.glu_gpt_oss(gu, bias, rows)
    want_b = _torch_glu_gpt_oss(gu + bias.index_select(0, rows))
    assert ((got_b.float() - want_b.float()).abs() <= 2 ** -7 * want_b.float().abs() + 1e-30).all()


@pytest.mark.parametrize("N_gu,K,N_dn,G,with_bias", [(5760, 2880, 2880, 4, True), (256, 96, 64, 3, False), (512, 1024, 128, 9, True)])
def test_fused_mxfp4_ffn_gpt_oss(N_gu, K, N_dn, G, with_bias):
    """gpt-oss-20b's expert FFN at batch 1 (4 experts of 32) and small shapes: the fused launch against the
    composition gemm -> (+ bias) -> gpt-oss GLU kernel -> gemm (same bits), and against an fp64 evaluation of the
    same formula (tolerance of the bf16 chain)."""
    E = 5
    gen = torch.Generator().manual_seed(N_gu + G)
    Wg, Sg = synth.mxfp4_stack(E, N_gu, K, gen, device=DEV, e_lo=118, e_hi=122)
    Wd, Sd = synth.mxfp4_stack(E, N_dn, N_gu // 2, gen, device=DEV, e_lo=118, e_hi=122)
    ids = [int(v) for v in torch.randint(0, E, (G,), generator=gen)]
    sizes = [1] * G
    a = torch.randn(G, K, generator=gen).to(torch.bfloat16).to(DEV)
    bias = (torch.randn(E, N_gu, generator=gen) * 0.5).to(torch.bfloat16).to(DEV) if with_bias else None
    fused = mxfp4_grouped.ffn_mxfp4_grouped(a, Wg, Sg, Wd, Sd, sizes, ids, bias_gu=bias)
    gu = mxfp4_grouped.gemm_mxfp4_grouped(a, Wg, Sg, sizes, ids)
    h = mxfp4_grouped.glu_gpt_oss(gu, bias, torch.tensor(ids, device=DEV) if with_bias else None)
    comp = mxfp4_grouped.gemm_mxfp4_grouped(h, Wd, Sd, sizes, ids)
    assert torch.equal(fused, comp)
    if not with_bias:
        assert torch.equal(mxfp4_grouped.ffn_mxfp4_grouped(a, Wg, Sg, Wd, Sd, sizes, ids, fused=False), comp)
    # silu form on MXFP4 stacks as well
    fs = mxfp4_grouped.ffn_mxfp4_grouped(a, Wg, Sg, Wd, Sd, sizes, ids, act="silu")
    cs = mxfp4_grouped.gemm_mxfp4_grouped(ep_moe.silu_glu(gu), Wd, Sd, sizes, ids)
    assert torch.equal(fs, cs)
    # fp64 evaluation of the gpt-oss formula from the decoded weights
    for i, e in enumerate(ids[:2]):
        wg = dequant_mxfp4(Wg[e].reshape(N_gu, K // 32, 16), Sg[e]).double()
        wd = dequant_mxfp4(Wd[e].reshape(N_dn, N_gu // 64, 16), Sd[e]).double()
        g64 = a[i].double() @ wg.t()
        if with_bias:
            g64 = g64 + bias[e].double()
        gate, up = g64[::2].clamp(max=7.0), g64[1::2].clamp(-7.0, 7.0)
        ref = ((up + 1) * gate * torch.sigmoid(gate * 1.702)) @ wd.t()
        err = ((fused[i].double() - ref).norm() / ref.norm()).item()
        assert err <= 1.5e-2, err          # five bf16 roundings inside the activation
    _clean()


def test_host_ffn_entry_uses_the_fused_launch_and_keeps_its_results():
    E, N_gu, K_gu, N_dn = 8, 1536, 2048, 2048
    (Bg, Ag), (Bd, Ad) = _nf4_pair(E, N_gu, K_gu, N_dn, seed=77)
    sizes, ids = [1] * 8, [7, 0, 3, 3, 1, 6, 2, 5]
    a = torch.randn(8, K_gu).to(torch.bfloat16)
    out_h = nf4_grouped.ffn_4bit_grouped_host(a, Bg, Ag, Bd, Ad, sizes, ids)
    out_d = ffn_4bit_grouped(a.to(DEV), Bg, Ag, Bd, Ad, sizes, ids)
    assert torch.equal(out_h, out_d.cpu())
    # larger groups: three launches behind the same entry
    sizes2, ids2 = [3, 5], [1, 4]
    a2 = torch.randn(8, K_gu).to(torch.bfloat16)
    out2 = nf4_grouped.ffn_4bit_grouped_host(a2, Bg, Ag, Bd, Ad, sizes2, ids2)
    comp = gemm_4bit_grouped(ep_moe.silu_glu(gemm_4bit_grouped(a2.to(DEV), Bg, Ag, sizes2, ids2)), Bd, Ad, sizes2, ids2)
    assert torch.equal(out2, comp.cpu())
    _clean()


@pytest.mark.parametrize("N_gu,K_gu,N_dn,G,rows", [(1536, 2048, 2048, 8, 1), (512, 256, 256, 5, 2), (4096, 1024, 512, 12, 1),
                                                   (256, 128, 64, 3, 5)])
def test_second_gemm_applies_the_activation_on_load(N_gu, K_gu, N_dn, G, rows):
    """gemm_after_glu: the down GEMM reads the gate_up output and applies SiLU-GLU while it loads its rows.  Same
    bits as the activation kernel followed by the plain GEMM, for one-row groups and for groups of a few rows."""
    E = 6
    (Bg, Ag), (Bd, Ad) = _nf4_pair(E, N_gu, K_gu, N_dn, seed=N_gu + rows)
    gen = torch.Generator().manual_seed(G)
    ids = torch.tensor([int(v) for v in torch.randint(0, E, (G,), generator=gen)], dtype=torch.int32, device=DEV)
    sizes = [int(v) for v in torch.randint(0, rows + 1, (G,), generator=gen)]
    sizes[0] = rows
    off = torch.tensor([0] + list(np.cumsum(sizes)), dtype=torch.int32, device=DEV)
    T = int(sum(sizes))
    gu = (torch.randn(T, N_gu, generator=gen) * 2).to(torch.bfloat16).to(DEV)
    got = nf4_grouped.gemm_after_glu(_gnf4b.FMT_NF4, gu, Bd, Ad, ids, off, rows)
    want = gemm_4bit_grouped(ep_moe.silu_glu(gu), Bd, Ad, None, ids, group_offsets=off, max_rows=rows)
    assert torch.equal(got, want)
    # the library did take the fused form (no silent detour through the activation kernel)
    direct = nf4_grouped._launch(_gnf4b.FMT_NF4, _gnf4b.OP_FWD, gu, Bd, Ad, None, ids, N_dn, group_offsets=off,
                                 max_rows=rows, x_glu=_gnf4b.FLAG_X_SILU_GLU)
    assert direct is not None and torch.equal(direct, want)
    _clean()


def test_second_gemm_gpt_oss_activation_on_load():
    E, N_gu, K, N_dn, G = 4, 5760, 2880, 2880, 4
    gen = torch.Generator().manual_seed(2)
    Wd, Sd = synth.mxfp4_stack(E, N_dn, N_gu // 2, gen, device=DEV, e_lo=118, e_hi=122)
    ids = torch.tensor([3, 0, 2, 3], dtype=torch.int32, device=DEV)
    off = torch.arange(G + 1, dtype=torch.int32, device=DEV)
    gu = (torch.randn(G, N_gu, generator=gen) * 3).to(torch.bfloat16).to(DEV)
    got = nf4_grouped.gemm_after_glu(_gnf4b.FMT_MXFP4, gu, Wd, Sd, ids, off, 1, act="gpt_oss")
    want = mxfp4_grouped.gemm_mxfp4_grouped(mxfp4_grouped.glu_gpt_oss(gu), Wd, Sd, None, ids, group_offsets=off, max_rows=1)
    assert torch.equal(got, want)
    # large groups: no kernel applies the activation on load, the same entry runs the activation kernel first
    gu2 = (torch.randn(64, N_gu, generator=gen)).to(torch.bfloat16).to(DEV)
    off2 = torch.tensor([0, 40, 64], dtype=torch.int32, device=DEV)
    ids2 = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    got2 = nf4_grouped.gemm_after_glu(_gnf4b.FMT_MXFP4, gu2, Wd, Sd, ids2, off2, 40, act="gpt_oss")
    want2 = mxfp4_grouped.gemm_mxfp4_grouped(mxfp4_grouped.glu_gpt_oss(gu2), Wd, Sd, None, ids2, group_offsets=off2, max_rows=40)
    assert torch.equal(got2, want2)
    _clean()
