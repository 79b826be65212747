"""Differentiable grouped 4-bit GEMMs for QLoRA-style training on top of the CUDA op.

Mirror of the reference's autograd layer (``kernel/nf4_qlora.py:32-305`` for NF4 and the
``_FusedGroupedMxfp4`` function of ``kernel/mxfp4_qlora.py:98-122`` for MXFP4): the packed base weight is
frozen, so the only gradient is the input gradient ``grad_out @ W`` -- one launch of the dgrad kernel -- and
nothing decoded survives from forward to backward.  The trainable part is the per-expert low-rank delta,
added to the projection BEFORE any activation (``act(Wx + BAx) != act(Wx) + d``).

Same names, argument meaning and defaults as the reference:

    gemm_4bit_grouped_train(a_cat, packed, absmax, sizes, expert_ids, weights_fn=None, dgrad_kernel=True)
    lora_delta_grouped(a_cat, lora_A, lora_B, sizes, expert_ids, scaling=1.0)
    fused_grouped_lora(a_cat, packed, absmax, sizes, expert_ids, lora_A=None, lora_B=None, weights_fn=None,
                       scaling=1.0, dgrad_kernel=True)

plus ``gemm_mxfp4_grouped_train`` (the reference's MXFP4 backward is a Python loop over experts; here it is
the same dgrad kernel with the MXFP4 decode).
"""
from __future__ import annotations

import torch

#: the batched low-rank delta pads every group to the widest one; beyond this ratio of padded to real rows
#: (a very hot expert) the per-expert loop is used instead (reference: ``_PAD_WASTE_LIMIT``)
_PAD_WASTE_LIMIT = 4.0


def _host_ints(v):
    return [int(x) for x in (v.tolist() if torch.is_tensor(v) else v)]


class FusedGroupedNf4(torch.autograd.Function):
    """``out = gemm_4bit_grouped(a_cat, packed, absmax, sizes, expert_ids)`` with
    ``grad_a = dgrad_4bit_grouped(grad_out, ...)``.

    ``weights_fn`` (optional, zero arguments, returns ``(packed, absmax)``) is called at backward time
    instead of keeping the two tensors on the context: an offloading caller re-stages a layer by replacing
    storage, and a tensor held here would keep the evicted storage alive (ref ``:54-72``).
    ``dgrad_kernel=False`` takes the exact per-expert loop (decode one expert, one matmul per group) -- the
    form to use when a gradient has to be compared bit for bit with a dequantise-then-matmul trainer; the
    loop is also the fallback when the kernel cannot take the problem (``dgrad_eligible``) or the stack
    lives on another device.
    """

    @staticmethod
    def forward(ctx, a_cat, packed, absmax, sizes, expert_ids, weights_fn=None, dgrad_kernel=True):
        from nf4_grouped import gemm_4bit_grouped
        ctx.use_kernel = bool(dgrad_kernel)
        ctx.weights_fn = weights_fn
        ctx.stack = None if weights_fn is not None else (packed, absmax)
        ctx.sizes, ctx.expert_ids = sizes, expert_ids       # kept as given: no host read of device ids here
        return gemm_4bit_grouped(a_cat, packed, absmax, sizes, expert_ids)

    @staticmethod
    def backward(ctx, grad_out):
        if not ctx.needs_input_grad[0]:
            return (None,) * 7
        from nf4_grouped import dequant_ref, dgrad_4bit_grouped, dgrad_eligible
        packed, absmax = ctx.stack if ctx.weights_fn is None else ctx.weights_fn()
        grad_out = grad_out.contiguous()
        if ctx.use_kernel and packed.device == grad_out.device and dgrad_eligible(grad_out, packed, absmax) is None:
            return (dgrad_4bit_grouped(grad_out, packed, absmax, ctx.sizes, ctx.expert_ids),) + (None,) * 6
        n_out, k_in = packed.shape[1], packed.shape[2] * 2
        grad_a = torch.zeros(grad_out.shape[0], k_in, dtype=grad_out.dtype, device=grad_out.device)
        first = 0
        for rows, e in zip(_host_ints(ctx.sizes), _host_ints(ctx.expert_ids)):
            if rows:
                w = dequant_ref(packed[e].to(grad_out.device), absmax[e].to(grad_out.device), n_out, k_in)
                grad_a[first:first + rows] = grad_out[first:first + rows] @ w.to(grad_out.dtype)
            first += rows
        return (grad_a,) + (None,) * 6


def gemm_4bit_grouped_train(a_cat, packed, absmax, sizes, expert_ids, weights_fn=None, dgrad_kernel=True):
    """``gemm_4bit_grouped`` that ``a_cat`` may require a gradient through (ref ``:161-171``)."""
    return FusedGroupedNf4.apply(a_cat, packed, absmax, sizes, expert_ids, weights_fn, dgrad_kernel)


class FusedGroupedMxfp4(torch.autograd.Function):
    """The MXFP4 counterpart: forward ``gemm_mxfp4_grouped``, backward ``dgrad_mxfp4_grouped``."""

    @staticmethod
    def forward(ctx, a_cat, blocks, scales, sizes, expert_ids):
        from mxfp4_grouped import gemm_mxfp4_grouped
        ctx.stack = (blocks, scales)
        ctx.sizes, ctx.expert_ids = sizes, expert_ids
        return gemm_mxfp4_grouped(a_cat, blocks, scales, sizes, expert_ids)

    @staticmethod
    def backward(ctx, grad_out):
        if not ctx.needs_input_grad[0]:
            return (None,) * 5
        from mxfp4_grouped import dgrad_mxfp4_grouped
        blocks, scales = ctx.stack
        return (dgrad_mxfp4_grouped(grad_out.contiguous(), blocks, scales, ctx.sizes, ctx.expert_ids),) + (None,) * 4


def gemm_mxfp4_grouped_train(a_cat, blocks, scales, sizes, expert_ids):
    return FusedGroupedMxfp4.apply(a_cat, blocks, scales, sizes, expert_ids)


def _lora_delta_grouped_loop(a_cat, lora_A, lora_B, sizes, expert_ids, scaling=1.0):
    """One pair of matmuls per non-empty group: the fallback for skewed routing and the form the batched
    path is tested against.  ``None`` when there are no rows."""
    out, first = None, 0
    for rows, e in zip(_host_ints(sizes), _host_ints(expert_ids)):
        if rows:
            x = a_cat[first:first + rows].to(lora_A.dtype)
            d = scaling * ((x @ lora_A[e].t()) @ lora_B[e].t())
            if out is None:
                out = torch.zeros(a_cat.shape[0], lora_B.shape[1], dtype=d.dtype, device=a_cat.device)
            out[first:first + rows] = d
        first += rows
    return out


def lora_delta_grouped(a_cat, lora_A, lora_B, sizes, expert_ids, scaling=1.0):
    """``scaling * B_e (A_e x)`` for every row x of every group (``lora_A [E, r, K]``, ``lora_B [E, N, r]``)
    -> ``[T, N]``; ``None`` when all groups are empty (ref ``:174-248``).  ``scaling`` is LoRA's alpha / r.

    Batched: the non-empty groups are padded to the widest one and run as two ``bmm``s, so the autograd
    graph has two nodes per projection instead of two per expert; when padding would multiply the rows by
    more than ``_PAD_WASTE_LIMIT`` the per-expert loop is used."""
    size_list = _host_ints(sizes)
    live = [g for g, n in enumerate(size_list) if n > 0]
    if not live:
        return None
    rows = [size_list[g] for g in live]
    total, widest = sum(rows), max(rows)
    if len(live) * widest > _PAD_WASTE_LIMIT * total:
        return _lora_delta_grouped_loop(a_cat, lora_A, lora_B, sizes, expert_ids, scaling)
    dev = a_cat.device
    if torch.is_tensor(expert_ids) and expert_ids.device.type != "cpu":
        experts = expert_ids.to(torch.int64)[torch.tensor(live, dtype=torch.int64, device=expert_ids.device)]
    else:
        ids = _host_ints(expert_ids)
        experts = torch.tensor([ids[g] for g in live], dtype=torch.int64, device=dev)
    # row t of the live rows belongs to live group grp[t], at position pos[t] inside it
    counts = torch.tensor(rows, dtype=torch.int64, device=dev)
    starts = torch.cumsum(counts, 0) - counts
    grp = torch.repeat_interleave(torch.arange(len(live), device=dev), counts, output_size=total)
    pos = torch.arange(total, device=dev) - starts[grp]
    # live rows in a_cat: the groups are contiguous, empty groups take no rows, so they are rows [0, total)
    x = torch.zeros(len(live), widest, a_cat.shape[1], dtype=lora_A.dtype, device=dev)
    x[grp, pos] = a_cat[:total].to(lora_A.dtype)
    low = torch.bmm(x, lora_A[experts].transpose(1, 2))                        # [G, widest, r]
    d = scaling * torch.bmm(low, lora_B[experts].transpose(1, 2))              # [G, widest, N]
    out = torch.zeros(a_cat.shape[0], lora_B.shape[1], dtype=d.dtype, device=dev)
    out[:total] = d[grp, pos]
    return out


def fused_grouped_lora(a_cat, packed, absmax, sizes, expert_ids, lora_A=None, lora_B=None, weights_fn=None,
                       scaling=1.0, dgrad_kernel=True):
    """Frozen 4-bit projection (differentiable in ``a_cat``) plus the trainable low-rank delta
    (differentiable in ``lora_A`` / ``lora_B``), summed before any activation (ref ``:286-305``)."""
    out = gemm_4bit_grouped_train(a_cat, packed, absmax, sizes, expert_ids, weights_fn=weights_fn,
                                  dgrad_kernel=dgrad_kernel)
    if lora_A is None or lora_B is None:
        return out
    delta = lora_delta_grouped(a_cat, lora_A, lora_B, sizes, expert_ids, scaling)
    return out if delta is None else out + delta.to(out.dtype)
