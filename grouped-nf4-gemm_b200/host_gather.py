"""Residency feeders: device-side gathers of packed expert row-blocks into slot buffers.

Replaces the Triton byte movers of the reference's residency engines on the path that feeds the grouped GEMM:
``gather_expert_rows`` (``kernel/host_gather.py:73-95``: rows of one stack selected by device-resident expert ids, read
straight from pinned host memory), the per-slot absolute-address gather (``kernel/mxfp4_pipelined.py:48-60``) and its
permuting form with a piece table (``kernel/mxfp4_residency.py:117-170``).  Same semantics: bytes in, the same bytes
out; a slot that already holds the wanted row is skipped (no traffic); all launch parameters are independent of the
ids, so the host never reads them and nothing synchronises.  One hand-written CUDA kernel family behind the C ABI
(``gnf4b_gather_rows_by_id`` / ``gnf4b_gather_rows_addr``); 16-byte aligned rows take 16-byte accesses, so the slots
the engines hand to the grouped GEMM can sit on 16-byte boundaries and take its bulk-copy loaders.
"""
from __future__ import annotations

import torch

import _gnf4b


def _row_bytes(t: torch.Tensor) -> int:
    nbytes = t[0].numel() * t[0].element_size()
    if nbytes % 8:
        raise ValueError(f"row-block of {nbytes} bytes is not 8-byte aligned; the gather moves 8-byte words")
    return nbytes


def _check_dst(dst: torch.Tensor):
    if not dst.is_cuda:
        raise RuntimeError("the gather writes device slots: dst must be a CUDA tensor")
    if not dst.is_contiguous():
        raise ValueError("dst must be contiguous (slot j is rows [j] of one buffer)")


def gather_expert_rows(dst: torch.Tensor, host: torch.Tensor, ids: torch.Tensor, have: torch.Tensor | None = None,
                       block: int = 2048):
    """``dst [k, ...]`` cuda <- ``host [E, ...]`` rows selected by ``ids`` (cuda int32 ``[k]``).  ``host`` is pinned
    host memory (read by the GPU over PCIe) or a device tensor.  ``have`` (cuda int32 ``[k]``, optional): what the
    slots hold now; matching slots are skipped.  ``block`` is a Triton launch knob of the reference, accepted and
    ignored.  Enqueues on the current stream and returns."""
    _check_dst(dst)
    k = dst.shape[0]
    row = _row_bytes(dst)
    if _row_bytes(host) != row:
        raise ValueError(f"host rows are {_row_bytes(host)} bytes, slots {row}")
    if not host.is_cuda and not host.is_pinned():
        raise RuntimeError("host rows must be pinned (cudaHostAlloc / pin_memory) to be addressable from the device")
    if not host.is_contiguous():
        raise ValueError("host must be contiguous")
    if ids.dtype != torch.int32 or not ids.is_cuda or (have is not None and (have.dtype != torch.int32 or not have.is_cuda)):
        raise TypeError("ids / have must be CUDA int32 tensors")
    import nf4_grouped
    with torch.cuda.device(dst.device):
        rc = _gnf4b.load().gnf4b_gather_rows_by_id(dst.data_ptr(), row, k, host.data_ptr(), host.shape[0], ids.data_ptr(),
                                                   have.data_ptr() if have is not None else None,
                                                   nf4_grouped._status_word(dst.device).data_ptr(),
                                                   torch.cuda.current_stream(dst.device).cuda_stream)
    _gnf4b.check(rc, "gnf4b_gather_rows_by_id")
    return dst


def piece_table(pieces, device) -> tuple[torch.Tensor, int]:
    """``(src_off, dst_off, length)`` byte triples -> (cuda int64 ``[n, 3]``, longest length).  Every offset and
    length must be a multiple of 8 (``ValueError`` otherwise, as the reference's chunk table refuses them)."""
    flat = []
    longest = 0
    for s_off, d_off, n in pieces:
        for bad, name in ((s_off, "src_off"), (d_off, "dst_off"), (n, "length")):
            if bad % 8:
                raise ValueError(f"{name}={bad} is not 8-byte aligned; the gather moves 8-byte words, so every segment "
                                 "offset and length must be. Re-bake with 8-aligned segments.")
        flat += [int(s_off), int(d_off), int(n)]
        longest = max(longest, int(n))
    return torch.tensor(flat, dtype=torch.int64, device=device).reshape(-1, 3), longest


def gather_rows_addr(dst: torch.Tensor, want_addr: torch.Tensor, have_addr: torch.Tensor | None = None, pieces=None):
    """``dst [k, ...]`` cuda <- the row-block at absolute address ``want_addr[j]`` (cuda int64 ``[k]``: device memory
    or pinned host memory), skipped where ``have_addr[j] == want_addr[j]``.  ``pieces``: the result of ``piece_table``
    when the row's segments land in a different order in the slot."""
    _check_dst(dst)
    k = dst.shape[0]
    row = _row_bytes(dst)
    if want_addr.dtype != torch.int64 or not want_addr.is_cuda or \
            (have_addr is not None and (have_addr.dtype != torch.int64 or not have_addr.is_cuda)):
        raise TypeError("want_addr / have_addr must be CUDA int64 tensors")
    tab, longest = (pieces if pieces is not None else (None, 0))
    with torch.cuda.device(dst.device):
        rc = _gnf4b.load().gnf4b_gather_rows_addr(dst.data_ptr(), row, k, want_addr.data_ptr(),
                                                  have_addr.data_ptr() if have_addr is not None else None,
                                                  tab.data_ptr() if tab is not None else None,
                                                  tab.shape[0] if tab is not None else 0, longest,
                                                  torch.cuda.current_stream(dst.device).cuda_stream)
    _gnf4b.check(rc, "gnf4b_gather_rows_addr")
    return dst
