"""numpy front end of the CPU oracle (TEST INFRASTRUCTURE, never the product).

Only the test suite, the smoke check and the benchmark's CPU legs import this
module.  It wraps ``libgnf4_oracle.so`` (the C restatement, ``gnf4_oracle.c``)
and, when present, the reference project's own CPU kernels compiled into
``oracle/_ref/`` (see ``build.py``).  Parity status: pinned -- see the header of
``gnf4_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
FMT = {"nf4": 0, "mxfp4": 1}
S_F32, S_BF16, S_E8M0 = 0, 1, 2

_LIB = None
_REF = None


def _vp(a):
    return C.c_void_p(a.ctypes.data)


def lib():
    """The C restatement, built on first use when a compiler is present."""
    global _LIB
    if _LIB is None:
        so = HERE / "libgnf4_oracle.so"
        src = HERE / "gnf4_oracle.c"
        if (not so.exists()) or so.stat().st_mtime < src.stat().st_mtime:
            from . import build as _b  # type: ignore
            _b.build_oracle()
        L = C.CDLL(str(so))
        i32, i64, vp = C.c_int32, C.c_int64, C.c_void_p
        common = [C.c_int, vp, i64, vp, vp, C.c_int, vp, vp, i32, i32, i64, i64, vp]
        for name in ("gnf4o_gemm_grouped_f64", "gnf4o_dgrad_grouped_f64",
                     "gnf4o_gemv_grouped_locked", "gnf4o_dgrad_grouped_locked"):
            f = getattr(L, name)
            f.restype, f.argtypes = C.c_int, common
        L.gnf4o_decode_stack.restype = C.c_int
        L.gnf4o_decode_stack.argtypes = [C.c_int, vp, vp, C.c_int, i64, i64, i64, vp]
        L.gnf4o_round_bf16.restype = None
        L.gnf4o_round_bf16.argtypes = [vp, i64, vp]
        L.gnf4o_group_offsets.restype = C.c_int
        L.gnf4o_group_offsets.argtypes = [vp, i32, vp]
        L.gnf4o_group_tiles.restype = i64
        L.gnf4o_group_tiles.argtypes = [vp, i32, i32, vp, vp, vp]
        L.gnf4o_route_topk.restype = C.c_int
        L.gnf4o_route_topk.argtypes = [vp, i64, i64, i64, C.c_int, C.c_int, vp, vp]
        L.gnf4o_sort_pairs.restype = C.c_int
        L.gnf4o_sort_pairs.argtypes = [vp, i64, i32, vp, vp]
        L.gnf4o_luts.restype = None
        L.gnf4o_luts.argtypes = [vp, vp]
        _LIB = L
    return _LIB


def luts():
    nf4 = np.empty(16, np.float32)
    fp4 = np.empty(16, np.float32)
    lib().gnf4o_luts(_vp(nf4), _vp(fp4))
    return nf4, fp4


def _scale_dtype(fmt, S):
    if fmt == "mxfp4":
        assert S.dtype == np.uint8
        return S_E8M0
    if S.dtype == np.float32:
        return S_F32
    assert S.dtype == np.uint16, "bf16 absmax is passed as its uint16 bit pattern"
    return S_BF16


def _prep(fmt, x, W, S, sizes, expert_ids):
    x = np.ascontiguousarray(x, np.float32)
    W = np.ascontiguousarray(W, np.uint8)
    S = np.ascontiguousarray(S)
    sizes = np.ascontiguousarray(sizes, np.int32)
    eids = np.ascontiguousarray(expert_ids, np.int32)
    E, N, half = W.shape
    return x, W, S, sizes, eids, E, N, half * 2


def decode_stack(fmt, W, S):
    """[E,N,K/2] u8 + scales -> [E,N,K] fp32, bit-exact element decode."""
    W = np.ascontiguousarray(W, np.uint8)
    S = np.ascontiguousarray(S)
    E, N, half = W.shape
    out = np.empty((E, N, half * 2), np.float32)
    rc = lib().gnf4o_decode_stack(FMT[fmt], _vp(W), _vp(S), _scale_dtype(fmt, S), E, N, half * 2, _vp(out))
    if rc:
        raise ValueError(f"decode_stack rc={rc}")
    return out


def _call(name, out_dtype, out_cols, fmt, x, W, S, sizes, expert_ids):
    x, W, S, sizes, eids, E, N, K = _prep(fmt, x, W, S, sizes, expert_ids)
    T = x.shape[0]
    cols = N if out_cols == "N" else K
    out = np.empty((T, cols), out_dtype)
    rc = getattr(lib(), name)(FMT[fmt], _vp(x), T, _vp(W), _vp(S), _scale_dtype(fmt, S),
                              _vp(sizes), _vp(eids), len(sizes), E, N, K, _vp(out))
    if rc:
        raise ValueError(f"{name} rc={rc}")
    return out


def gemm_grouped_f64(fmt, a, W, S, sizes, expert_ids):
    """fp64 oracle of the forward: [T,K] x stack -> [T,N] float64."""
    return _call("gnf4o_gemm_grouped_f64", np.float64, "N", fmt, a, W, S, sizes, expert_ids)


def dgrad_grouped_f64(fmt, g, W, S, sizes, expert_ids):
    """fp64 oracle of the dgrad: [T,N] x stack -> [T,K] float64."""
    return _call("gnf4o_dgrad_grouped_f64", np.float64, "K", fmt, g, W, S, sizes, expert_ids)


def gemv_grouped_locked(fmt, a, W, S, sizes, expert_ids):
    """fp32 forward in the CPU tier's locked summation order."""
    return _call("gnf4o_gemv_grouped_locked", np.float32, "N", fmt, a, W, S, sizes, expert_ids)


def dgrad_grouped_locked(fmt, g, W, S, sizes, expert_ids):
    return _call("gnf4o_dgrad_grouped_locked", np.float32, "K", fmt, g, W, S, sizes, expert_ids)


def round_bf16_bits(x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().gnf4o_round_bf16(_vp(x), x.size, _vp(out))
    return out


def bf16_bits_to_f32(bits):
    return (np.ascontiguousarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def group_offsets(sizes):
    sizes = np.ascontiguousarray(sizes, np.int32)
    out = np.empty(len(sizes) + 1, np.int32)
    if lib().gnf4o_group_offsets(_vp(sizes), len(sizes), _vp(out)):
        raise ValueError("bad sizes")
    return out


def group_tiles(sizes, block_m):
    sizes = np.ascontiguousarray(sizes, np.int32)
    n = lib().gnf4o_group_tiles(_vp(sizes), len(sizes), block_m, None, None, None)
    a, b, c = (np.empty(n, np.int32) for _ in range(3))
    lib().gnf4o_group_tiles(_vp(sizes), len(sizes), block_m, _vp(a), _vp(b), _vp(c))
    return a, b, c


def route_topk(logits, k, mode=0, norm=False):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    if lib().gnf4o_route_topk(_vp(logits), T, E, k, mode, int(norm), _vp(idx), _vp(w)):
        raise ValueError("bad k")
    return idx, w


def sort_pairs(flat, E):
    flat = np.ascontiguousarray(flat, np.int32).reshape(-1)
    order = np.empty(flat.size, np.int32)
    counts = np.empty(E, np.int32)
    if lib().gnf4o_sort_pairs(_vp(flat), flat.size, E, _vp(order), _vp(counts)):
        raise ValueError("expert id out of range")
    return order, counts


def rel_frobenius(out, ref64):
    """||out - ref|| / ||ref|| in fp64 (the reference's err_vs_fp64 metric,
    kernel/test_nf4_grouped.py:50-59)."""
    d = np.asarray(out, np.float64) - ref64
    return float(np.sqrt((d * d).sum()) / max(np.sqrt((ref64 * ref64).sum()), 1e-30))


def max_rel(out, ref64):
    """max|out - ref| / max|ref| (kernel/test_mxfp4_grouped.py:58)."""
    return float(np.abs(np.asarray(out, np.float64) - ref64).max() / max(np.abs(ref64).max(), 1e-30))


# --------------------------------------------------------------------------- #
# the reference project's own CPU kernels (oracle/_ref), when built
# --------------------------------------------------------------------------- #

def _cpu_flags():
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_available() -> bool:
    return any((HERE / "_ref").glob("cpu_kernels-*.so"))


def load_ref():
    """ctypes handle on the reference's compiled cpu_kernels (best ISA variant the
    running CPU supports), or None when oracle/_ref was never built."""
    global _REF
    if _REF is not None:
        return _REF
    flags = _cpu_flags()
    want = []
    if {"avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512cd"} <= flags:
        want.append("avx512")
    if {"avx2", "fma", "bmi2"} <= flags:
        want.append("avx2")
    want.append("base")
    for name in want:
        so = HERE / "_ref" / f"cpu_kernels-{name}.so"
        if so.exists():
            L = C.CDLL(str(so))
            vp, i64 = C.c_void_p, C.c_int64
            sig = [vp, vp, vp, vp, vp, C.c_int, i64, i64, vp, C.c_int]
            for fn in ("gnf4_gemv_nf4_grouped", "gnf4_gemv_mxfp4_grouped",
                       "gnf4_dgrad_nf4_grouped", "gnf4_dgrad_mxfp4_grouped"):
                getattr(L, fn).restype = C.c_int
                getattr(L, fn).argtypes = sig
            L.gnf4_gemv_nf4_ffn_grouped.restype = C.c_int
            L.gnf4_gemv_nf4_ffn_grouped.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_int, i64, i64, i64, vp, C.c_int]
            L.gnf4_pool_start.restype = C.c_int
            L.gnf4_pool_start.argtypes = [C.c_int]
            L.gnf4_pool_stop.restype = None
            L.gnf4_cpu_features.restype = C.c_int
            L.variant = name
            _REF = L
            return L
    return None


def ref_call(kind, fmt, x, W, S, sizes, expert_ids, threads=0):
    """Run the reference's native kernel.  kind: 'gemv' (x [R,K] -> [R,N]) or
    'dgrad' (x [R,N] -> [R,K]).  fp32 in/out, sizes >= 1, G <= 512 (its limits,
    gnf4_native/cpu_kernels.c:755)."""
    L = load_ref()
    if L is None:
        raise RuntimeError("oracle/_ref is not built")
    x, W, S, sizes, eids, E, N, K = _prep(fmt, x, W, S, sizes, expert_ids)
    assert S.dtype == (np.float32 if fmt == "nf4" else np.uint8)
    e64 = eids.astype(np.int64)
    if kind == "gemv":
        out = np.empty((x.shape[0], N), np.float32)
    else:
        out = np.zeros((x.shape[0], K), np.float32)   # it accumulates into zeros
    fn = getattr(L, f"gnf4_{kind}_{fmt}_grouped")
    rc = fn(_vp(x), _vp(W), _vp(S), _vp(e64), _vp(sizes), len(sizes), N, K, _vp(out), threads)
    if rc:
        raise ValueError(f"reference kernel rejected the call rc={rc}")
    return out


def ref_ffn_call(x, W_gu, S_gu, W_dn, S_dn, sizes, expert_ids, threads=0):
    """The reference's fused NF4 expert FFN (gnf4_native/cpu_kernels.c:947-986): x [R,K] fp32 ->
    (silu(gate) * up) @ W_dn^T, [R, N_dn] fp32, gate/up the two halves of x @ W_gu^T.  sizes >= 1, G <= 512."""
    L = load_ref()
    if L is None:
        raise RuntimeError("oracle/_ref is not built")
    x, W_gu, S_gu, sizes, eids, E, N_gu, K_gu = _prep("nf4", x, W_gu, S_gu, sizes, expert_ids)
    W_dn = np.ascontiguousarray(W_dn, np.uint8)
    S_dn = np.ascontiguousarray(S_dn, np.float32)
    assert S_gu.dtype == np.float32 and W_dn.shape[2] * 2 == N_gu // 2
    N_dn = W_dn.shape[1]
    e64 = eids.astype(np.int64)
    out = np.empty((x.shape[0], N_dn), np.float32)
    rc = L.gnf4_gemv_nf4_ffn_grouped(_vp(x), _vp(W_gu), _vp(S_gu), _vp(W_dn), _vp(S_dn), _vp(e64), _vp(sizes),
                                     len(sizes), N_gu, K_gu, N_dn, _vp(out), threads)
    if rc:
        raise ValueError(f"reference FFN kernel rejected the call rc={rc}")
    return out


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def ffn_grouped_f64(a, W_gu, S_gu, W_dn, S_dn, sizes, expert_ids, fmt="nf4"):
    """fp64 oracle of the expert FFN (the computation of gnf4_native/cpu_kernels.c:947-986): gate_up GEMM,
    h = silu(gate) * up over the two halves of its columns, down GEMM; nothing rounded in between."""
    gu = gemm_grouped_f64(fmt, a, W_gu, S_gu, sizes, expert_ids)
    H = gu.shape[1] // 2
    gate, up = gu[:, :H], gu[:, H:]
    h = gate / (1.0 + np.exp(-gate)) * up
    # the second GEMM through the same fp64 routine: its input is taken as float32 there, so feed the
    # high and the residual parts separately and add (exact split of a float64 into two float32)
    hi = h.astype(np.float32)
    lo = (h - hi.astype(np.float64)).astype(np.float32)
    return (gemm_grouped_f64(fmt, hi, W_dn, S_dn, sizes, expert_ids)
            + gemm_grouped_f64(fmt, lo, W_dn, S_dn, sizes, expert_ids))


def gather_rows_ref(dst, src_rows, ids, have=None, pieces=None):
    """Byte-level restatement of the residency feeders: ``dst [k, row_bytes]`` uint8 (its current content) with slot j
    overwritten by ``src_rows[ids[j]]`` unless ``have[j] == ids[j]`` -- kernel/host_gather.py:33-54 (selection by
    id), kernel/mxfp4_pipelined.py:48-60 (the same with one absolute address per slot: here the address is the row
    index) -- and, with ``pieces`` = (src_off, dst_off, length) byte triples, only those spans, each landing at its
    own offset of the slot (kernel/mxfp4_residency.py:117-134).  Returns a new array."""
    out = np.array(dst, dtype=np.uint8, copy=True)
    src_rows = np.asarray(src_rows, dtype=np.uint8)
    for j, want in enumerate(np.asarray(ids).tolist()):
        if have is not None and int(np.asarray(have)[j]) == want:
            continue
        if want < 0 or want >= src_rows.shape[0]:
            continue
        if pieces is None:
            out[j] = src_rows[want]
        else:
            for s_off, d_off, n in pieces:
                out[j, d_off:d_off + n] = src_rows[want, s_off:s_off + n]
    return out
