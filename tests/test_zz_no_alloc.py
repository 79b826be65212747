"""The allocation-free entry point, gnf4b_gemm_grouped_noalloc, against the ordinary one.

Some hosts of this library may not allocate device memory while they run: a serving loop
whose memory plan is frozen, a plugin inside a runtime that owns every byte of the GPU, a
latency-critical path that cannot afford an allocator call or its failure.  For them the
split-K scratch comes from a fixed array inside the library instead of a caller buffer.
This test drives both entry points through the C ABI on the same inputs, twice in a row
(the second call meets whatever the first left in the shared array), and expects the same
bits -- it is the same kernel -- and the usual tolerance against the fp64 oracle.  It also
checks that a problem whose scratch exceeds the array is refused, not launched.

The file name keeps it last in collection order, so a run that stops at the first failure
has already been through every other test.
"""
import pytest
import torch

import _gnf4b
import nf4_grouped
from helpers import oracle_fwd64, rel_fro
from nf4_pack_ref import make_stack

pytestmark = pytest.mark.gpu
DEV = "cuda"
REL_FRO_TOL = 2.0e-3      # bf16 output rounding level, as in the other GPU tests


def _call(lib, entry, a, B, A, off, ids, out, split_k, ws=None):
    E, N, half = B.shape
    K = half * 2
    T = a.shape[0]
    G = ids.numel()
    flags = _gnf4b.PATH_STREAM | (split_k << _gnf4b.SPLITK_SHIFT)
    stream = torch.cuda.current_stream().cuda_stream
    status = nf4_grouped._status_word(DEV)
    common = (_gnf4b.FMT_NF4, _gnf4b.OP_FWD, a.data_ptr(), _gnf4b.X_BF16, T, B.data_ptr(), B.stride(0), B.stride(1),
              A.data_ptr(), _gnf4b.S_F32, A.stride(0), A.stride(1), off.data_ptr(), ids.data_ptr(), G, E, N, K, 1,
              out.data_ptr())
    if entry == "noalloc":
        return lib.gnf4b_gemm_grouped_noalloc(*common, status.data_ptr(), flags, stream)
    return lib.gnf4b_gemm_grouped(*common, ws.data_ptr(), ws.numel(), status.data_ptr(), flags, stream)


def test_noalloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    lib = _gnf4b.load()
    B, A = make_stack(4, 256, 2048, seed=11, device=DEV)
    ids = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    off = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    split_k = 4
    need = lib.gnf4b_workspace_bytes(_gnf4b.FMT_NF4, _gnf4b.OP_FWD, 2, 2, 256, 2048, 1,
                                     _gnf4b.PATH_STREAM | (split_k << _gnf4b.SPLITK_SHIFT))
    assert 0 < need <= _gnf4b.NOALLOC_SCRATCH_BYTES          # the split-K (scratch-using) kernel is what runs
    for round_ in range(2):
        a = torch.randn(2, 2048, device=DEV, dtype=torch.bfloat16)
        want = torch.empty(2, 256, dtype=torch.bfloat16, device=DEV)
        ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
        assert _call(lib, "alloc", a, B, A, off, ids, want, split_k, ws) == 0
        got = torch.full((2, 256), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert _call(lib, "noalloc", a, B, A, off, ids, got, split_k) == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"round {round_}"
        assert rel_fro(got, oracle_fwd64("nf4", a, B, A, [1, 1], [3, 0])) <= REL_FRO_TOL
    assert nf4_grouped.last_status(DEV) == 0
    # the headline property, around a warmed-up call: no device memory is allocated or freed by it
    a = torch.randn(2, 2048, device=DEV, dtype=torch.bfloat16)
    got = torch.empty(2, 256, dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    assert _call(lib, "noalloc", a, B, A, off, ids, got, split_k) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before


def test_noalloc_entry_point_refuses_scratch_beyond_its_array():
    lib = _gnf4b.load()
    # split-K partials of 8 x 4096 rows x 1024 columns x 4 bytes = 128 MiB: far beyond the array
    T, N, K, E = 4096, 1024, 8192, 1
    B = torch.zeros(E, N, K // 2, dtype=torch.uint8, device=DEV)
    A = torch.ones(E, N, K // 64, dtype=torch.float32, device=DEV)
    a = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
    off = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    ids = torch.tensor([0], dtype=torch.int32, device=DEV)
    flags = _gnf4b.PATH_STREAM | (8 << _gnf4b.SPLITK_SHIFT)
    rc = lib.gnf4b_gemm_grouped_noalloc(
        _gnf4b.FMT_NF4, _gnf4b.OP_FWD, a.data_ptr(), _gnf4b.X_BF16, T, B.data_ptr(), B.stride(0), B.stride(1),
        A.data_ptr(), _gnf4b.S_F32, A.stride(0), A.stride(1), off.data_ptr(), ids.data_ptr(), 1, E, N, K, T,
        out.data_ptr(), None, flags, torch.cuda.current_stream().cuda_stream)
    assert rc == -6
    with pytest.raises(ValueError, match="maximum"):
        _gnf4b.check(rc, "gnf4b_gemm_grouped_noalloc")
    torch.cuda.synchronize()
    assert not out.any()                                     # nothing ran
