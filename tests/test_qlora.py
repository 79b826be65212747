"""Autograd layer over the grouped 4-bit GEMMs (nf4_qlora): what the reference checks in
kernel/test_nf4_qlora_grad.py -- the input gradient against dequantise-then-matmul autograd, the exact
per-expert loop, the low-rank delta batched vs looped, the composition, and that nothing but the
callable is retained when ``weights_fn`` is given."""
import pytest
import torch

import nf4_qlora


def _lora_case(seed, sizes, E=5, K=48, N=40, r=4, device="cpu", dtype=torch.float32):
    gen = torch.Generator().manual_seed(seed)
    T = sum(sizes)
    a = torch.randn(T, K, generator=gen).to(device, dtype)
    A = (torch.randn(E, r, K, generator=gen) * 0.2).to(device, dtype)
    B = (torch.randn(E, N, r, generator=gen) * 0.2).to(device, dtype)
    ids = [int(v) for v in torch.randint(0, E, (len(sizes),), generator=gen)]
    return a, A, B, ids


@pytest.mark.parametrize("sizes", [[3, 0, 5, 1], [1, 1, 1, 1, 1], [0, 0], [40, 1, 0, 1, 1, 1, 1, 1, 1, 1, 1, 1]])
def test_lora_delta_batched_equals_loop_and_propagates_gradients(sizes):
    a, A, B, ids = _lora_case(len(sizes) + sum(sizes), sizes)
    A.requires_grad_(True)
    B.requires_grad_(True)
    got = nf4_qlora.lora_delta_grouped(a, A, B, sizes, ids, scaling=2.0)
    want = nf4_qlora._lora_delta_grouped_loop(a, A.detach(), B.detach(), sizes, ids, scaling=2.0)
    if sum(sizes) == 0:
        assert got is None and want is None
        return
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    got.square().sum().backward()
    A2, B2 = A.detach().clone().requires_grad_(True), B.detach().clone().requires_grad_(True)
    nf4_qlora._lora_delta_grouped_loop(a, A2, B2, sizes, ids, scaling=2.0).square().sum().backward()
    assert torch.allclose(A.grad, A2.grad, rtol=1e-3, atol=1e-4) and torch.allclose(B.grad, B2.grad, rtol=1e-3, atol=1e-4)


def test_lora_delta_accepts_tensor_carriers():
    sizes = [2, 3, 0, 1]
    a, A, B, ids = _lora_case(9, sizes)
    want = nf4_qlora.lora_delta_grouped(a, A, B, sizes, ids)
    got = nf4_qlora.lora_delta_grouped(a, A, B, torch.tensor(sizes), torch.tensor(ids, dtype=torch.int32))
    assert torch.equal(got, want)


# ------------------------------------------------------------------------------------------- GPU
def _nf4_case(sizes, N=128, K=256, E=6, seed=3):
    import synth
    gen = torch.Generator().manual_seed(seed)
    W, S = synth.nf4_stack(E, N, K, gen, device="cuda", scale=0.05)
    ids = [int(v) for v in torch.randint(0, E, (len(sizes),), generator=gen)]
    a = torch.randn(sum(sizes), K, generator=gen).to(torch.bfloat16).cuda()
    return W, S, ids, a


def _dense_reference(a, W, S, sizes, ids, grad_out):
    """Dequantise-then-matmul in fp32 with autograd: output and input gradient."""
    from nf4_grouped import dequant_ref
    x = a.detach().float().requires_grad_(True)
    outs, first = [], 0
    for rows, e in zip(sizes, ids):
        w = dequant_ref(W[e], S[e], W.shape[1], W.shape[2] * 2).float()
        outs.append(x[first:first + rows] @ w.t())
        first += rows
    out = torch.cat(outs)
    out.backward(grad_out.float())
    return out.detach(), x.grad


@pytest.mark.gpu
@pytest.mark.parametrize("dgrad_kernel", [True, False])
@pytest.mark.parametrize("sizes", [[5, 0, 130, 1], [1, 1, 1]])
def test_input_gradient_matches_dense_autograd(sizes, dgrad_kernel):
    W, S, ids, a = _nf4_case(sizes)
    a.requires_grad_(True)
    out = nf4_qlora.gemm_4bit_grouped_train(a, W, S, sizes, ids, dgrad_kernel=dgrad_kernel)
    g = (torch.randn(out.shape, device="cuda") * 1e-3).to(torch.bfloat16)
    out.backward(g)
    ref_out, ref_grad = _dense_reference(a, W, S, sizes, ids, g)
    rel = lambda x, y: ((x.float() - y).norm() / y.norm()).item()  # noqa: E731
    assert rel(out, ref_out) < 1e-2 and rel(a.grad, ref_grad) < 1e-2      # the reference's bf16 budget


@pytest.mark.gpu
def test_weights_fn_is_called_at_backward_and_no_stack_is_retained():
    sizes = [4, 2]
    W, S, ids, a = _nf4_case(sizes)
    a.requires_grad_(True)
    calls = []

    def staged():
        calls.append(1)
        return W, S

    out = nf4_qlora.gemm_4bit_grouped_train(a, W, S, sizes, ids, weights_fn=staged)
    assert out.grad_fn.stack is None and not calls
    out.sum().backward()
    assert calls == [1] and a.grad is not None


@pytest.mark.gpu
def test_fused_grouped_lora_is_projection_plus_delta_and_trains_the_adapters():
    sizes = [3, 0, 6]
    W, S, ids, a = _nf4_case(sizes)
    _, A, B, _ = _lora_case(1, sizes, E=6, K=256, N=128, r=8, device="cuda", dtype=torch.bfloat16)
    A.requires_grad_(True)
    B.requires_grad_(True)
    a.requires_grad_(True)
    y = nf4_qlora.fused_grouped_lora(a, W, S, sizes, ids, A, B, scaling=2.0)
    base = nf4_qlora.gemm_4bit_grouped_train(a.detach(), W, S, sizes, ids)
    delta = nf4_qlora._lora_delta_grouped_loop(a.detach(), A.detach(), B.detach(), sizes, ids, 2.0)
    assert torch.allclose(y.float(), base.float() + delta.float(), rtol=2e-2, atol=2e-2)
    y.float().square().mean().backward()
    assert a.grad is not None and A.grad.abs().sum() > 0 and B.grad.abs().sum() > 0
    assert nf4_qlora.fused_grouped_lora(a.detach(), W, S, sizes, ids).shape == y.shape


@pytest.mark.gpu
def test_mxfp4_input_gradient_matches_dense_autograd():
    import synth
    from mxfp4_pack_ref import dequant_mxfp4
    gen = torch.Generator().manual_seed(8)
    E, N, K = 4, 96, 128
    Wm, Sm = synth.mxfp4_stack(E, N, K, gen, device="cuda", e_lo=120, e_hi=124)
    sizes, ids = [7, 0, 2], [3, 1, 0]
    a = torch.randn(sum(sizes), K, generator=gen).to(torch.bfloat16).cuda().requires_grad_(True)
    out = nf4_qlora.gemm_mxfp4_grouped_train(a, Wm, Sm, sizes, ids)
    g = (torch.randn(out.shape, device="cuda") * 1e-2).to(torch.bfloat16)
    out.backward(g)
    x = a.detach().float().requires_grad_(True)
    outs, first = [], 0
    for rows, e in zip(sizes, ids):
        w = dequant_mxfp4(Wm[e].reshape(N, K // 32, 16).cpu(), Sm[e].cpu()).reshape(N, K).float().cuda()
        outs.append(x[first:first + rows] @ w.t())
        first += rows
    torch.cat(outs).backward(g.float())
    assert ((a.grad.float() - x.grad).norm() / x.grad.norm()).item() < 1e-2
