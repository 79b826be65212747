"""The benchmark configurations themselves on the CUDA kernels, plus the planner cases that only those sizes
reach.  Config 1 is replayed from its golden fixture (inputs regenerated from the seed, checked by hash);
the prefill shapes of configs 3 and 5 run on the tensor-core kernel at their real N and K with a few experts;
config 4's gate_up dgrad runs full size (sampled rows + an exact permutation property).  fp16 activations are
driven through every entry point at a shape where the planner wants the tensor kernel and must take the
split-K streaming kernel instead."""
import hashlib

import numpy as np
import pytest
import torch

import _gnf4b
import mxfp4_grouped
import nf4_grouped
import synth
from helpers import max_rel, oracle_fwd64, rel_fro
from mxfp4_pack_ref import dequant_mxfp4
from nf4_grouped import dequant_ref, dgrad_4bit_grouped, gemm_4bit_grouped
from nf4_pack_ref import make_stack, quantize_pack_nf4

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_FRO_TOL = 2.0e-3      # bf16 output rounding level (reference fused path: 1.66e-3 - 1.70e-3)
MX_MAXREL = 2e-2          # kernel/test_mxfp4_grouped.py:58 of the reference
T = _gnf4b.PATH_TENSOR
S = _gnf4b.PATH_STREAM


def _clean():
    assert nf4_grouped.last_status(DEV) == 0


# ------------------------------------------------------------------ config 1
def test_config1_fixture_through_every_kernel(golden_dir):
    """BASELINE config 1 (E=8, N=512, K=1024, 64 tokens top-2): the fixture's inputs through the planner's
    choice, the streaming kernel and the tensor kernel.  `out_cpu_bits` is the reference's own CPU result
    (fp32, locked order): the kernels must equal it at bf16 resolution and stay within tolerance of fp64."""
    g = np.load(golden_dir / "config1.npz")
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()  # noqa: E731
    E, N, K, M, k = 8, 512, 1024, 64, 2
    gen = torch.Generator(device="cpu").manual_seed(int(g["seed"]))
    B = torch.empty(E, N, K // 2, dtype=torch.uint8)
    A = torch.empty(E, N, K // 64)
    for e in range(E):
        B[e], A[e] = quantize_pack_nf4(torch.randn(N, K, generator=gen) * 0.02)
    logits = torch.randn(M, E, generator=gen)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    assert sha(B.numpy()) == str(g["sha_B"]) and sha(A.numpy()) == str(g["sha_A"])
    idx, _ = synth.route_topk(logits, k)
    tok, sizes, eids, _ = synth.dispatch(idx, E)
    assert sizes == g["sizes"].tolist() and eids == g["eids"].tolist()
    a_cat = x[tok].contiguous().to(DEV)
    Bd, Ad = B.to(DEV), A.to(DEV)
    cpu = torch.from_numpy(g["out_cpu_bits"].view(np.float32).copy())          # [128, 512] fp32
    ref64 = oracle_fwd64("nf4", a_cat, Bd, Ad, sizes, eids)
    lim = 2 ** -8 * float(np.abs(ref64).max())
    for path in (0, S, T):
        out = gemm_4bit_grouped(a_cat, Bd, Ad, sizes, eids, path=path)
        assert out.shape == (128, 512) and out.dtype == torch.bfloat16
        assert rel_fro(out, ref64) <= REL_FRO_TOL, (path, rel_fro(out, ref64))
        # against the reference's CPU output: equal up to the one bf16 rounding of the result
        assert (out.float().cpu() - cpu).abs().max().item() <= lim, path
    # the streaming kernel accumulates in the CPU tier's precision class: its bf16 result is the bf16 rounding
    # of the CPU result except where fp32 summation order moves a value across a rounding boundary
    st = gemm_4bit_grouped(a_cat, Bd, Ad, sizes, eids, path=S).cpu()
    same = (st.view(torch.int16) == cpu.to(torch.bfloat16).view(torch.int16)).float().mean().item()
    assert same >= 0.99, same
    _clean()


# ------------------------------------------------------------------ config 5 / config 3 prefill shapes
@pytest.mark.parametrize("N,K", [(4096, 7168), (7168, 2048)])
def test_config5_shapes_on_the_tensor_kernel(N, K):
    """DeepSeek-V3 projections (BASELINE config 5) at their real N and K: 112 / 32 k-stages per item, groups
    of >= 300 rows (two chunks of the 256-row accumulator) and of 17 - 64 rows, 4 experts."""
    E = 4
    gen = torch.Generator().manual_seed(N + K)
    W, Sc = synth.mxfp4_stack(E, N, K, gen, device=DEV)
    sizes, ids = [300, 17, 64, 0, 333, 40], [2, 0, 3, 1, 1, 2]
    a = torch.randn(sum(sizes), K, generator=gen).to(torch.bfloat16).to(DEV)
    out = mxfp4_grouped.gemm_mxfp4_grouped(a, W, Sc, sizes, ids, path=T)
    r = 0
    for m, e in zip(sizes, ids):
        if m:
            w = dequant_mxfp4(W[e].reshape(N, K // 32, 16), Sc[e]).double()
            ref = a[r:r + m].double() @ w.t()
            err = ((out[r:r + m].double() - ref).abs().max() / ref.abs().max()).item()
            assert err < MX_MAXREL, (m, e, err)
            assert ((out[r:r + m].double() - ref).norm() / ref.norm()).item() <= REL_FRO_TOL
        r += m
    # the planner's choice (tensor kernel at these sizes) gives the same bits
    assert torch.equal(mxfp4_grouped.gemm_mxfp4_grouped(a, W, Sc, sizes, ids), out)
    _clean()


def test_config3_gate_up_on_the_tensor_kernel():
    """gpt-oss-20b gate_up (BASELINE config 3): N = 5760, K = 2880 = 45 x 64, a ragged last k-stage and 45 column
    tiles, on the tensor kernel."""
    N, K, E = 5760, 2880, 4
    gen = torch.Generator().manual_seed(3)
    W, Sc = synth.mxfp4_stack(E, N, K, gen, device=DEV)
    sizes, ids = [256, 31, 130], [3, 1, 0]
    a = torch.randn(sum(sizes), K, generator=gen).to(torch.bfloat16).to(DEV)
    out = mxfp4_grouped.gemm_mxfp4_grouped(a, W, Sc, sizes, ids, path=T)
    ref = oracle_fwd64("mxfp4", a, W, Sc, sizes, ids)
    assert rel_fro(out, ref) <= REL_FRO_TOL and max_rel(out, ref) < MX_MAXREL
    _clean()


def test_config4_gate_up_dgrad_full_size():
    """BASELINE config 4, the larger of its two problems: dX [32768, 2048] for the Qwen3 gate_up stack
    [128, 1536, 1024] from dY [32768, 1536] ~ N(0, 1e-3); sampled rows against the fp64 decode, and reversing
    the group order must permute the result rows exactly."""
    shape = synth.CONFIGS["qwen3_30b_a3b"]
    gen = torch.Generator().manual_seed(44)
    N, K = shape.gate_up
    B, A = synth.nf4_stack(shape.experts, N, K, gen, device=DEV, fast=True)
    _, idx, _ = synth.routed_batch(shape, 4096, gen)
    tok, sizes, ids, _ = synth.dispatch(idx, shape.experts)
    go = (torch.randn(len(tok), N, generator=gen) * 1e-3).to(torch.bfloat16).to(DEV)
    dx = dgrad_4bit_grouped(go, B, A, sizes, ids)
    assert dx.shape == (32768, K)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    for r in np.random.default_rng(2).integers(0, go.shape[0], 24):
        gi = int(np.searchsorted(offs, r, side="right") - 1)
        ref = go[r].double() @ dequant_ref(B[ids[gi]], A[ids[gi]], N, K).double()
        assert ((dx[r].double() - ref).norm() / ref.norm()).item() <= REL_FRO_TOL
    order = list(range(len(sizes)))[::-1]
    rows = torch.cat([torch.arange(offs[g], offs[g + 1]) for g in order]).to(DEV)
    assert torch.equal(dgrad_4bit_grouped(go[rows], B, A, [sizes[g] for g in order], [ids[g] for g in order]), dx[rows])
    _clean()


# ------------------------------------------------------------------ fp16 activations where the planner wants tensor cores
def _fp16_case():
    """One group of 32 fp16 rows, N = 1024, K = 4096: the planner's first choice is the tensor kernel (which
    multiplies bf16 only), the streaming kernel that takes the call splits K (128 items < 2 x SMs)."""
    B, A = make_stack(1, 1024, 4096, seed=77, device=DEV)
    gen = torch.Generator().manual_seed(78)
    a = torch.randn(32, 4096, generator=gen).to(torch.float16)
    return a, B, A, [32], [0]


def test_fp16_activations_take_split_k_streaming_kernel_through_every_entry_point():
    lib = _gnf4b.load()
    a, B, A, sizes, ids = _fp16_case()
    ref = oracle_fwd64("nf4", a, B, A, sizes, ids)
    assert lib.gnf4b_workspace_bytes(_gnf4b.FMT_NF4, _gnf4b.OP_FWD, 32, 1, 1024, 4096, 32, 0) > 0
    ad = a.to(DEV)
    out = gemm_4bit_grouped(ad, B, A, sizes, ids)
    assert rel_fro(out, ref) <= REL_FRO_TOL, rel_fro(out, ref)
    # the host-buffer entry point
    out_h, status = nf4_grouped.gemm_4bit_grouped_host(a, B, A, sizes, ids, return_status=True)
    assert status == 0 and torch.equal(out_h, out.cpu())
    # the allocation-free entry point, after a call whose fp32 partials cover this call's counter span
    off = torch.tensor([0, 32], dtype=torch.int32, device=DEV)
    eid = torch.tensor([0], dtype=torch.int32, device=DEV)
    status_w = nf4_grouped._status_word(DEV)
    stream = torch.cuda.current_stream().cuda_stream

    def noalloc(x, xdt, Bx, Ax, offx, idx, G, N, K, max_rows, flags):
        o = torch.full((x.shape[0], N), float("nan"), dtype=torch.bfloat16, device=DEV)
        rc = lib.gnf4b_gemm_grouped_noalloc(
            _gnf4b.FMT_NF4, _gnf4b.OP_FWD, x.data_ptr(), xdt, x.shape[0], Bx.data_ptr(), Bx.stride(0), Bx.stride(1),
            Ax.data_ptr(), _gnf4b.S_F32, Ax.stride(0), Ax.stride(1), offx.data_ptr(), idx.data_ptr(), G, Bx.shape[0],
            N, K, max_rows, o.data_ptr(), status_w.data_ptr(), flags, stream)
        assert rc == 0, rc
        return o

    # dirty the array: 2 groups x 32 tiles of counters (256 bytes), then fp32 partials of [4][2][256] right behind
    B2, A2 = make_stack(4, 256, 2048, seed=11, device=DEV)
    a2 = torch.randn(2, 2048, device=DEV, dtype=torch.bfloat16) * 100
    noalloc(a2, _gnf4b.X_BF16, B2, A2, torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV),
            torch.tensor([3, 0], dtype=torch.int32, device=DEV), 2, 256, 2048, 1, S | (4 << _gnf4b.SPLITK_SHIFT))
    got = noalloc(ad, _gnf4b.X_FP16, B, A, off, eid, 1, 1024, 4096, 32, 0)
    torch.cuda.synchronize()
    assert torch.equal(got, out)
    _clean()


def test_noalloc_call_allocates_no_device_memory():
    """The property the entry point exists for: around a warmed-up call neither torch's allocator nor the
    driver's free-memory figure moves."""
    lib = _gnf4b.load()
    B, A = make_stack(4, 256, 2048, seed=11, device=DEV)
    a = torch.randn(2, 2048, device=DEV, dtype=torch.bfloat16)
    off = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    ids = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(2, 256, dtype=torch.bfloat16, device=DEV)
    status_w = nf4_grouped._status_word(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    args = (_gnf4b.FMT_NF4, _gnf4b.OP_FWD, a.data_ptr(), _gnf4b.X_BF16, 2, B.data_ptr(), B.stride(0), B.stride(1),
            A.data_ptr(), _gnf4b.S_F32, A.stride(0), A.stride(1), off.data_ptr(), ids.data_ptr(), 2, 4, 256, 2048, 1,
            out.data_ptr(), status_w.data_ptr(), S | (4 << _gnf4b.SPLITK_SHIFT), stream)
    assert lib.gnf4b_gemm_grouped_noalloc(*args) == 0          # warm-up: module load, symbol address
    torch.cuda.synchronize()
    free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    for _ in range(3):
        assert lib.gnf4b_gemm_grouped_noalloc(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == alloc0
    _clean()


# ------------------------------------------------------------------ contract edges found by review
def test_dgrad_with_n_not_a_multiple_of_8_is_ineligible_not_a_runtime_error():
    B, A = make_stack(2, 132, 128, seed=5, device=DEV)
    go = torch.randn(6, 132, device=DEV, dtype=torch.bfloat16)
    why = nf4_grouped.dgrad_eligible(go, B, A)
    assert why is not None and "multiple of 8" in why
    with pytest.raises(ValueError, match="cannot run this problem"):
        dgrad_4bit_grouped(go, B, A, [3, 3], [0, 1])


def test_understated_max_rows_is_flagged():
    """max_rows promises the largest group; the decode kernel visits only that many rows of a group, so a group
    that is larger must raise the offsets flag instead of silently leaving rows unwritten."""
    B, A = make_stack(2, 64, 256, seed=9, device=DEV)
    a = torch.randn(5, 256, device=DEV, dtype=torch.bfloat16)
    off = torch.tensor([0, 1, 5], dtype=torch.int32, device=DEV)
    ids = torch.tensor([1, 0], dtype=torch.int32, device=DEV)
    assert nf4_grouped.last_status(DEV) == 0
    gemm_4bit_grouped(a, B, A, None, ids, group_offsets=off, max_rows=2, path=S)
    assert nf4_grouped.last_status(DEV) & _gnf4b.ST_BAD_OFFSETS
    full = gemm_4bit_grouped(a, B, A, None, ids, group_offsets=off, max_rows=4, path=S)
    assert rel_fro(full, oracle_fwd64("nf4", a, B, A, [1, 4], [1, 0])) <= 2 ** -8
    _clean()


def test_ep_plan_pairs_beyond_the_capacity_are_dropped_and_flagged():
    """gnf4b_ep_plan with cap smaller than the pairs one rank receives: the surplus pair gets slot -1, nothing
    is written outside that rank's cap rows, GNF4B_ST_BAD_OFFSETS is raised."""
    lib = _gnf4b.load()
    P, k, n_experts, e_local, cap, H = 6, 1, 4, 2, 2, 16
    idx = torch.tensor([3, 3, 2, 0, 3, 1], dtype=torch.int64, device=DEV)        # rank 1 gets 4 pairs, cap is 2
    hidden = torch.arange(P * H, device=DEV, dtype=torch.float32).reshape(P, H).to(torch.bfloat16)
    counts = torch.zeros(n_experts, dtype=torch.int32, device=DEV)
    slot = torch.full((P,), -7, dtype=torch.int64, device=DEV)
    guard = 4
    send = torch.full((2 * cap + guard, H), -1.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.gnf4b_ep_plan(idx.data_ptr(), P, k, n_experts, e_local, cap, hidden.data_ptr(), H, counts.data_ptr(),
                           slot.data_ptr(), send.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _gnf4b.ST_BAD_OFFSETS
    assert counts.tolist() == [1, 1, 1, 3]
    s = slot.tolist()
    assert s[3] == 0 and s[5] == 1                     # rank 0: experts 0 then 1
    assert s[2] == cap + 0 and s[0] == cap + 1         # rank 1: expert 2 first, then the first pair of expert 3
    assert s[1] == -1 and s[4] == -1                   # no room left on rank 1
    assert (send[2 * cap:] == -1).all()                # nothing past the end of rank 1's block
    assert torch.equal(send[cap + 1], hidden[0])
