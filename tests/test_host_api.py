"""Host-side behaviour of the drop-in modules that needs no GPU: importability, the
planning helpers' values (pinned to the reference's answers), error behaviour, and that
the C-ABI library loads and exports every symbol the header declares."""
import ctypes
import json
import re
from pathlib import Path

import pytest
import torch

import _gnf4b
import mxfp4_grouped
import nf4_grouped
from mxfp4_pack_ref import dequant_mxfp4, quantize_pack_mxfp4
from nf4_pack_ref import make_stack

ROOT = Path(__file__).resolve().parents[1]


def test_modules_import_without_gpu_and_export_reference_names():
    for name in ("gemm_4bit_grouped", "dgrad_4bit_grouped", "dgrad_eligible", "dequant_ref", "repack_from_bnb",
                 "build_group_tiles", "to_device_i32", "decode_dispatch", "_decode_plan", "_prefill_block_m",
                 "_sm_count", "_DGRAD_DEFAULT", "_lut", "_arena", "_ARENAS", "_PinnedIndexArena", "NF4_LUT",
                 "BLOCKSIZE", "DECODE_MIN_FUSED_BYTES", "SPLITK_MIN_BLOCKS"):
        assert hasattr(nf4_grouped, name), name
    for name in ("gemm_mxfp4_grouped", "FP4_VALUES", "MX_BLOCK", "E8M0_BIAS", "build_group_tiles", "_prefill_block_m"):
        assert hasattr(mxfp4_grouped, name), name


def test_constants_and_plans_match_reference(golden_dir):
    rec = json.loads((golden_dir / "plans.json").read_text())
    c = rec["constants"]
    assert nf4_grouped.NF4_LUT == c["NF4_LUT"] and nf4_grouped.BLOCKSIZE == c["BLOCKSIZE"]
    assert mxfp4_grouped.FP4_VALUES == c["FP4_VALUES"] and mxfp4_grouped.MX_BLOCK == c["MX_BLOCK"]
    assert mxfp4_grouped.E8M0_BIAS == c["E8M0_BIAS"]
    assert nf4_grouped.DECODE_MIN_FUSED_BYTES == c["DECODE_MIN_FUSED_BYTES"]
    assert nf4_grouped.SPLITK_MIN_BLOCKS == c["SPLITK_MIN_BLOCKS"]
    assert list(nf4_grouped._DGRAD_DEFAULT) == c["DGRAD_DEFAULT"]
    for args, want in rec["decode_plan"]:
        assert list(nf4_grouped._decode_plan(*args)) == want, args
    for args, want in rec["decode_dispatch"]:
        assert list(nf4_grouped.decode_dispatch(*args)) == want, args
    for m, want in rec["prefill_block_m"]:
        assert nf4_grouped._prefill_block_m(m) == want
    for sizes, bm, r0, rows, grp in rec["group_tiles"]:
        a, b, c_ = nf4_grouped.build_group_tiles(sizes, bm, "cpu")
        assert (a.tolist(), b.tolist(), c_.tolist()) == (r0, rows, grp)
        assert a.dtype == torch.int32


def test_build_group_tiles_does_not_mutate_tensor_sizes():
    t = torch.tensor([3, 2, 0, 5], dtype=torch.int32)
    nf4_grouped.build_group_tiles(t, 2, "cpu")
    nf4_grouped.build_group_tiles(t, 2, "cpu")
    assert t.tolist() == [3, 2, 0, 5]


def test_dequant_ref_matches_golden(golden_dir):
    import numpy as np
    g = np.load(golden_dir / "decode.npz")
    B = torch.from_numpy(g["nf4_packed"])
    am = torch.from_numpy(g["nf4_absmax"])
    w = nf4_grouped.dequant_ref(B, am, *B.shape[:1], B.shape[1] * 2)
    assert np.array_equal(w.view(torch.int32).numpy().view(np.uint32), g["nf4_w_bits"])
    B2, S2 = torch.from_numpy(g["mx_packed"]), torch.from_numpy(g["mx_scales"])
    w2 = dequant_mxfp4(B2.reshape(B2.shape[0], -1, 16), S2)
    assert np.array_equal(w2.view(torch.int32).numpy().view(np.uint32), g["mx_w_bits"])


def test_pack_round_trip():
    B, A = make_stack(2, 16, 128, seed=3)
    w = nf4_grouped.dequant_ref(B[0], A[0], 16, 128)
    assert w.shape == (16, 128) and torch.isfinite(w).all()
    blocks, scales = quantize_pack_mxfp4(torch.randn(8, 64))
    assert blocks.shape == (8, 2, 16) and scales.shape == (8, 2)
    w2 = dequant_mxfp4(blocks, scales)
    b2, s2 = quantize_pack_mxfp4(w2)          # decoded values re-quantise to the same bytes
    assert torch.equal(dequant_mxfp4(b2, s2), w2)


def test_cpu_tensors_are_refused_with_the_taught_error():
    B, A = make_stack(2, 16, 64)
    a = torch.randn(2, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="requires CUDA tensors.*dequant_ref"):
        nf4_grouped.gemm_4bit_grouped(a, B, A, [1, 1], [0, 1])
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        nf4_grouped.dgrad_4bit_grouped(torch.randn(2, 16, dtype=torch.bfloat16), B, A, [1, 1], [0, 1])
    blocks, scales = quantize_pack_mxfp4(torch.randn(1, 16, 64))
    with pytest.raises(RuntimeError, match="requires CUDA tensors.*dequant_mxfp4"):
        mxfp4_grouped.gemm_mxfp4_grouped(a, blocks.reshape(1, 16, 32), scales, [2], [0])


def test_dgrad_eligibility_rules():
    B, A = make_stack(2, 16, 128)
    go = torch.randn(3, 16, dtype=torch.bfloat16)
    assert nf4_grouped.dgrad_eligible(go, B, A) is None
    assert "bfloat16" in nf4_grouped.dgrad_eligible(go.to(torch.float16), B, A)
    assert "does not divide" in nf4_grouped.dgrad_eligible(go, B, A, block_k=48)
    assert "do not tile" in nf4_grouped.dgrad_eligible(go, B, A[:, :, :1])
    assert "empty" in nf4_grouped.dgrad_eligible(go, B[:0], A)


def test_to_device_i32_cpu_path_keeps_values_and_order():
    a, b, c = nf4_grouped.to_device_i32(([1, 2, 3], [], torch.tensor([7, 8])), "cpu")
    assert a.tolist() == [1, 2, 3] and b.numel() == 0 and c.tolist() == [7, 8]
    assert a.dtype == torch.int32


def test_header_symbols_are_exported_by_the_built_library():
    """include/gnf4b.h is the contract: the loader's EXPORTS list must name every function
    it declares, and the built library must export each one (no compute call here)."""
    header = (ROOT / "include" / "gnf4b.h").read_text()
    declared = set(re.findall(r"\b(gnf4b_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_gnf4b.EXPORTS), declared ^ set(_gnf4b.EXPORTS)
    if not _gnf4b.LIB_PATH.exists():
        _gnf4b.build()
    lib = ctypes.CDLL(str(_gnf4b.LIB_PATH))
    for sym in declared:
        assert hasattr(lib, sym), sym
    lib.gnf4b_abi_version.restype = ctypes.c_int
    assert lib.gnf4b_abi_version() == 1
    lib.gnf4b_strerror.restype = ctypes.c_char_p
    assert b"workspace" in lib.gnf4b_strerror(-3)


def test_c_abi_rejects_contract_violations_without_a_gpu():
    if not _gnf4b.LIB_PATH.exists():
        _gnf4b.build()
    lib = _gnf4b.load()
    # K not a multiple of 64 for NF4 -> ESHAPE, before any CUDA call
    rc = lib.gnf4b_gemm_grouped(0, 0, None, 0, 4, None, 0, 0, None, 0, 0, 0, None, None, 1, 1, 16, 96, 1,
                                None, None, 0, None, 0, None)
    assert rc == -2
    rc = lib.gnf4b_gemm_grouped(7, 0, None, 0, 4, None, 0, 0, None, 0, 0, 0, None, None, 1, 1, 16, 128, 1,
                                None, None, 0, None, 0, None)
    assert rc == -1
    with pytest.raises(ValueError):
        _gnf4b.check(-2, "x")
    with pytest.raises(RuntimeError):
        _gnf4b.check(-5, "x")
    # the host-buffer entry point checks its group tables on the host, before any CUDA call:
    # sizes that do not sum to T, a negative size, an expert id outside the stack
    def host(sizes, ids, T, E=4):
        sz = (ctypes.c_int32 * len(sizes))(*sizes)
        ii = (ctypes.c_int32 * len(ids))(*ids)
        st = ctypes.c_int32(99)
        rc = lib.gnf4b_gemm_grouped_host(0, 0, None, 0, T, None, 0, 0, None, 0, 0, 0, ctypes.addressof(sz),
                                         ctypes.addressof(ii), len(sizes), E, 16, 128, None, None, 0,
                                         ctypes.addressof(st), 0, None)
        return rc, st.value
    assert host([1, 2], [0, 1], 4) == (-1, 0)
    assert host([-1, 5], [0, 1], 4) == (-1, 0)
    assert host([2, 2], [0, 4], 4) == (-1, 0)
    assert host([2, 2], [0, -2], 4) == (-1, 0)
    assert host([0, 0], [0, -1], 0) == (0, 0)            # nothing to do: OK without touching the device


def test_repack_from_bnb_with_stand_in_state_objects(monkeypatch):
    """repack_from_bnb (kernel/nf4_grouped.py:74-96 of the reference) on hand-made stand-ins for bitsandbytes'
    per-expert outputs -- bitsandbytes itself is not installable here: packed bytes land as [E, N, K/2], absmax as
    fp32 [E, N, K/64], and nested statistics (compress_statistics=True) are de-nested through
    bitsandbytes.functional.dequantize_blockwise + offset."""
    import sys
    import types

    E, N, K = 3, 8, 128
    gen = torch.Generator().manual_seed(5)
    packed = [torch.randint(0, 256, (N * K // 2, 1), dtype=torch.uint8, generator=gen) for _ in range(E)]
    absmax = [torch.rand(N * K // 64, generator=gen) + 0.1 for _ in range(E)]

    class State:
        def __init__(self, am, nested=False, state2=None, offset=None):
            self.absmax, self.nested, self.state2, self.offset = am, nested, state2, offset

    # plain statistics
    B, A = nf4_grouped.repack_from_bnb(packed, [State(a) for a in absmax], N, K)
    assert B.shape == (E, N, K // 2) and B.dtype == torch.uint8 and A.shape == (E, N, K // 64) and A.dtype == torch.float32
    for e in range(E):
        assert torch.equal(B[e].reshape(-1), packed[e].reshape(-1))
        assert torch.equal(A[e].reshape(-1), absmax[e])
    # nested statistics: absmax stored as uint8 codes of (absmax - offset), decoded by a second-level quantiser
    calls = []

    def dequantize_blockwise(q, state2):
        calls.append(state2)
        return q.float() * state2["scale"]

    fake = types.ModuleType("bitsandbytes")
    fake.functional = types.ModuleType("bitsandbytes.functional")
    fake.functional.dequantize_blockwise = dequantize_blockwise
    monkeypatch.setitem(sys.modules, "bitsandbytes", fake)
    monkeypatch.setitem(sys.modules, "bitsandbytes.functional", fake.functional)
    offset = torch.tensor(0.25)
    codes = [torch.randint(0, 256, (N * K // 64,), dtype=torch.uint8, generator=gen) for _ in range(E)]
    states = [State(c, nested=True, state2={"scale": 1.0 / 512 * (e + 1)}, offset=offset) for e, c in enumerate(codes)]
    B2, A2 = nf4_grouped.repack_from_bnb(packed, states, N, K)
    assert len(calls) == E and torch.equal(B2, B)
    for e in range(E):
        want = (codes[e].float() * (1.0 / 512 * (e + 1)) + 0.25).reshape(N, K // 64)
        assert torch.equal(A2[e], want)
    with pytest.raises(AssertionError):
        nf4_grouped.repack_from_bnb(packed, states, N, 100)        # K must be a multiple of the blocksize


def test_custom_operator_is_registered_with_a_fake_kernel():
    """torch.ops.gnf4b.grouped_gemm exists and its fake kernel gives shape, dtype and device of the result without
    touching a GPU (what torch.compile / torch.export need to trace through the entry points)."""
    assert hasattr(torch.ops.gnf4b, "grouped_gemm")
    x = torch.empty(5, 128, dtype=torch.bfloat16, device="meta")
    W = torch.empty(4, 64, 64, dtype=torch.uint8, device="meta")
    S = torch.empty(4, 64, 2, dtype=torch.float32, device="meta")
    out = torch.ops.gnf4b.grouped_gemm(x, W, S, None, None, [2, 3], [0, 1], 0, 0, 64, 3, 0, 0, True)
    assert out.shape == (5, 64) and out.dtype == torch.bfloat16 and out.device.type == "meta"
    go = torch.empty(5, 64, dtype=torch.bfloat16, device="meta")
    dx = torch.ops.gnf4b.grouped_gemm(go, W, S, None, None, [2, 3], [0, 1], 0, 1, 128, 3, 0, 0, True)
    assert dx.shape == (5, 128)


def test_gather_oracle_and_piece_table_rules():
    """The byte-level restatement of the residency feeders (skip rule, piece order) and the alignment rule of the
    piece table, without a GPU."""
    import numpy as np
    from oracle import oracle as O
    src = np.arange(4 * 32, dtype=np.uint8).reshape(4, 32)
    dst = np.full((3, 32), 255, np.uint8)
    out = O.gather_rows_ref(dst, src, [2, 0, 3], have=[2, 1, -1])
    assert (out[0] == 255).all() and np.array_equal(out[1], src[0]) and np.array_equal(out[2], src[3])
    out = O.gather_rows_ref(dst, src, [1, 1, 9], pieces=[(0, 24, 8), (8, 0, 24)])
    assert np.array_equal(out[0, 24:], src[1, :8]) and np.array_equal(out[0, :24], src[1, 8:]) and (out[2] == 255).all()
    import host_gather
    with pytest.raises(ValueError, match="8-byte aligned"):
        host_gather.piece_table([(8, 8, 12)], "cpu")
    tab, longest = host_gather.piece_table([(0, 16, 8), (8, 0, 16)], "cpu")
    assert tab.tolist() == [[0, 16, 8], [8, 0, 16]] and longest == 16


def test_exchange_and_feeder_entry_points_check_their_arguments_on_the_host():
    """Layout arithmetic and argument checks of the entry points added around the GEMM (no launch is reached)."""
    import ctypes
    import _gnf4b
    lib = _gnf4b.load()
    lay = (ctypes.c_int64 * 3)()
    assert lib.gnf4b_ep_peer_layout(8, 16, 8, 2048, lay) == 0
    total, rows_off, ret_off = int(lay[0]), int(lay[1]), int(lay[2])
    row_bytes = 8 * 8 * 2048 * 2
    assert rows_off % 256 == 0 and ret_off % 256 == 0
    assert ret_off >= rows_off + 3 * row_bytes and total >= ret_off + 2 * row_bytes      # plain rows, then two 8-byte-per-4 areas
    assert lib.gnf4b_ep_peer_layout(17, 16, 8, 2048, lay) == -1                          # more ranks than the context holds
    assert lib.gnf4b_ep_peer_layout(8, 16, 8, 2050, lay) == -1                           # H not a multiple of 8
    assert lib.gnf4b_ep_plan_large_scratch_bytes(32768, 128) == (32768 // 512) * 257 * 4
    assert lib.gnf4b_ep_plan_large_scratch_bytes(1, 2048) == 0                           # more experts than the kernels' bins
    # feeders: rows are 8-byte words
    assert lib.gnf4b_gather_rows_by_id(None, 12, 2, None, 4, None, None, None, None) == -2
    assert lib.gnf4b_gather_rows_by_id(None, 16, 0, None, 4, None, None, None, None) == 0   # nothing to do
    assert lib.gnf4b_gather_rows_by_id(None, 16, 2, None, 4, None, None, None, None) == -1  # null pointers
    assert lib.gnf4b_gather_rows_addr(None, 16, 2, None, None, None, 0, 0, None) == -1
    assert lib.gnf4b_gather_rows_addr(None, 16, 2, None, None, None, 0, 12, None) == -2
    # push: at most 16 blocks, byte counts multiples of 16
    assert lib.gnf4b_ep_push_blocks(17, None, None, None, None, 1, 0, None, None) == -1
    ctx = _gnf4b.EpPeerCtx(2, 0, 4, 8, 64)
    assert lib.gnf4b_ep_peer_dispatch(ctypes.byref(ctx), None, 0, 2, 8, 4, None, None, 0, None, None, None, None) == -1   # no buffers
