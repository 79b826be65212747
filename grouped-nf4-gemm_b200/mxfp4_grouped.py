"""Grouped W4A16 GEMM over native MXFP4 expert stacks on NVIDIA B200 -- the drop-in for
the reference module of the same name (pjordanandrsn/grouped-nf4-gemm,
kernel/mxfp4_grouped.py:134-172).

``out[t] = a[t] @ dequant_mxfp4(blocks[e(t)]).T`` for rows grouped by expert, one launch of
the sm_100a kernels in ``libgnf4b.so``.  Decode rules (ref :7-16): e2m1 codebook, element
2j in the LOW nibble of byte j, one e8m0 scale byte per 32 elements with value 2^(e-127).
The decode follows the ``ldexp`` semantics of ``mxfp4_pack_ref.dequant_mxfp4`` (a zero
element times the 0xFF scale stays zero).  Offsets are 64-bit throughout, so stacks beyond
2 GiB are fine (the reference's Triton kernel multiplies ``eid * stride`` in int32,
ref :65, 73).
"""
from __future__ import annotations

import torch

import _gnf4b
from nf4_grouped import (_dispatch, _launch, _launch_ffn, _launch_host, _prefill_block_m, _require_cuda,  # noqa: F401  (re-exported names)
                         build_group_tiles)

# e2m1 codebook, index = (sign << 3) | magnitude (ref :34-35)
FP4_VALUES = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
              -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
MX_BLOCK = 32
E8M0_BIAS = 127

_LUT_CACHE: dict = {}


def _lut(device):
    key = str(device)
    if key not in _LUT_CACHE:
        _LUT_CACHE[key] = torch.tensor(FP4_VALUES, dtype=torch.float32, device=device)
    return _LUT_CACHE[key]


def gemm_mxfp4_grouped(a_cat, blocks, scales, sizes, expert_ids,
                       block_m: int | None = None, prefill_variant: int | None = None, *,
                       group_offsets=None, max_rows=None, path: int = 0, tables_ready: bool | None = None):
    """Single-launch grouped MXFP4 GEMM (ref :134-172).  ``a_cat [T,K]`` bf16/fp16 rows
    sorted by group; ``blocks [E,N,K//2]`` uint8; ``scales [E,N,K//32]`` uint8 (e8m0);
    ``sizes`` per-group row counts; ``expert_ids [G]`` list / CPU / CUDA int tensor.
    Returns ``[T,N]`` bf16 in the same row order.  ``block_m`` and ``prefill_variant`` are
    Triton knobs of the reference, accepted and ignored.  ``group_offsets`` / ``max_rows`` /
    ``path`` / ``tables_ready`` are the keyword-only additions described at ``nf4_grouped.gemm_4bit_grouped``."""
    E, N, _ = blocks.shape
    T, K = a_cat.shape
    assert scales.shape == (E, N, K // MX_BLOCK), (scales.shape, (E, N, K // MX_BLOCK))
    assert blocks.dtype == torch.uint8 and scales.dtype == torch.uint8
    _require_cuda(a_cat, "gemm_mxfp4_grouped",
                  "For a CPU-checkable decode of the same MXFP4 bytes, use "
                  "mxfp4_pack_ref.dequant_mxfp4(blocks, scales).")
    if blocks.shape[2] * 2 != K:
        raise ValueError(f"a_cat has K={K} but blocks pack K={blocks.shape[2] * 2}")
    return _dispatch(_gnf4b.FMT_MXFP4, _gnf4b.OP_FWD, a_cat, blocks, scales, sizes, expert_ids, N,
                     group_offsets=group_offsets, max_rows=max_rows, path=path, tables_ready=tables_ready)


def ffn_mxfp4_grouped(a_cat, blocks_gu, scales_gu, blocks_dn, scales_dn, sizes, expert_ids, *, act: str = "gpt_oss",
                      bias_gu=None, group_offsets=None, max_rows=None, tables_ready: bool | None = None,
                      fused: bool = True):
    """One MXFP4 expert FFN per row on CUDA tensors: ``act(a @ W_gu[e].T (+ bias_gu[e])) @ W_dn[e].T``.
    ``act="gpt_oss"``: gate and up interleaved in the gate_up columns, the clamped GLU of gpt-oss evaluated as the
    reference's chain of bf16 tensor operations (``kernel/mxfp4_pipelined.py:440-445, 453-461``); ``act="silu"``:
    SiLU(gate) * up over column halves.  ``bias_gu`` is an optional bf16 ``[E, N_gu]``.  Batch-1 decode (every group
    one row) runs as ONE kernel launch; the down bias and the router-weighted sum stay with the caller (fp32 there)."""
    if act not in ("gpt_oss", "silu"):
        raise ValueError("act is 'gpt_oss' or 'silu'")
    assert blocks_gu.dtype == torch.uint8 and scales_gu.dtype == torch.uint8
    assert blocks_dn.dtype == torch.uint8 and scales_dn.dtype == torch.uint8
    _require_cuda(a_cat, "ffn_mxfp4_grouped", "The CPU-checkable equivalent composes mxfp4_pack_ref.dequant_mxfp4 per expert.")
    return _launch_ffn(_gnf4b.FMT_MXFP4, _gnf4b.ACT_GPT_OSS_GLU if act == "gpt_oss" else _gnf4b.ACT_SILU_GLU, a_cat,
                       blocks_gu, scales_gu, blocks_dn, scales_dn, sizes, expert_ids, bias_gu=bias_gu,
                       group_offsets=group_offsets, max_rows=max_rows, tables_ready=tables_ready, fused=fused)


def glu_gpt_oss(gate_up, bias=None, row_expert=None):
    """The activation of gpt-oss between its expert GEMMs as one kernel: ``gate_up [rows, 2h]`` bf16 (gate and up
    interleaved) -> ``[rows, h]`` bf16; ``bias`` bf16 ``[E, 2h]`` is added first (row r takes ``bias[row_expert[r]]``)."""
    _require_cuda(gate_up, "glu_gpt_oss", "")
    gate_up = gate_up.contiguous()
    rows, two_h = gate_up.shape
    out = torch.empty(rows, two_h // 2, dtype=torch.bfloat16, device=gate_up.device)
    if bias is not None:
        bias = bias.contiguous()
        row_expert = row_expert.to(torch.int32).contiguous()
    lib = _gnf4b.load()
    with torch.cuda.device(gate_up.device):
        rc = lib.gnf4b_glu_gpt_oss(gate_up.data_ptr(), rows, two_h // 2, bias.data_ptr() if bias is not None else None,
                                   row_expert.data_ptr() if bias is not None else None, out.data_ptr(),
                                   torch.cuda.current_stream(gate_up.device).cuda_stream)
    _gnf4b.check(rc, "gnf4b_glu_gpt_oss")
    return out


def gemm_mxfp4_grouped_host(a_host, blocks, scales, sizes, expert_ids, out=None, *, path: int = 0,
                            return_status: bool = False):
    """``gemm_mxfp4_grouped`` with host activations, host group tables and a host result, the stack resident on
    the GPU: the calling convention of the reference's native CPU kernel
    (``gnf4_native/cpu_kernels.c:1097``).  See ``nf4_grouped.gemm_4bit_grouped_host``."""
    assert blocks.dtype == torch.uint8 and scales.dtype == torch.uint8
    return _launch_host(_gnf4b.FMT_MXFP4, _gnf4b.OP_FWD, a_host, blocks, scales, sizes, expert_ids,
                        blocks.shape[1], out, path=path, return_status=return_status)


def dgrad_mxfp4_grouped_host(grad_host, blocks, scales, sizes, expert_ids, out=None, *, return_status: bool = False):
    """``dgrad_mxfp4_grouped`` with host buffers (``gnf4_native/cpu_kernels.c:1386-1397``)."""
    return _launch_host(_gnf4b.FMT_MXFP4, _gnf4b.OP_DGRAD, grad_host, blocks, scales, sizes, expert_ids,
                        blocks.shape[2] * 2, out, return_status=return_status)


def dgrad_mxfp4_grouped(grad_out, blocks, scales, sizes, expert_ids, *, group_offsets=None, max_rows=None):
    """``grad_a[t,:] = grad_out[t,:] @ dequant_mxfp4(blocks[e(t)])`` in one launch, ``[T,K]``
    bf16.  The reference has this only as a per-expert Python loop on the GPU
    (kernel/mxfp4_qlora.py:105-122) and as a CPU kernel (gnf4_native/cpu_kernels.c:1386-1397)."""
    E, N, half = blocks.shape
    _require_cuda(grad_out, "dgrad_mxfp4_grouped",
                  "The CPU-checkable equivalent is grad_out @ dequant_mxfp4(blocks, scales) per group.")
    if grad_out.dtype != torch.bfloat16:
        raise ValueError(f"dgrad_mxfp4_grouped cannot run this problem: grad_out dtype {grad_out.dtype} is not bfloat16")
    if grad_out.shape[1] != N:
        raise ValueError(f"grad_out has {grad_out.shape[1]} columns but the stack has N={N}")
    return _launch(_gnf4b.FMT_MXFP4, _gnf4b.OP_DGRAD, grad_out, blocks, scales, sizes, expert_ids, half * 2,
                   group_offsets=group_offsets, max_rows=max_rows)


def dequant_stack_cuda(blocks, scales):
    """Element decode of a whole MXFP4 stack by the CUDA library's decode routines ->
    ``[E,N,K]`` fp32, for bit-for-bit comparison with ``mxfp4_pack_ref.dequant_mxfp4``."""
    _require_cuda(blocks, "dequant_stack_cuda", "Use mxfp4_pack_ref.dequant_mxfp4 on CPU tensors.")
    E, N, half = blocks.shape
    if blocks.stride(2) != 1:
        blocks = blocks.contiguous()
    if scales.stride(2) != 1:
        scales = scales.contiguous()
    out = torch.empty(E, N, half * 2, dtype=torch.float32, device=blocks.device)
    lib = _gnf4b.load()
    with torch.cuda.device(blocks.device):
        rc = lib.gnf4b_dequant(_gnf4b.FMT_MXFP4, blocks.data_ptr(), blocks.stride(0), blocks.stride(1),
                               scales.data_ptr(), _gnf4b.S_E8M0, scales.stride(0), scales.stride(1),
                               E, N, half * 2, out.data_ptr(),
                               torch.cuda.current_stream(blocks.device).cuda_stream)
    _gnf4b.check(rc, "gnf4b_dequant")
    return out
