"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

The reference project is Python (+ one C file); it cannot travel to the GPU
box, so its answers on small seeded inputs are frozen here as .npz/.json files
that the tests compare the oracle (and through it the CUDA path) against.

What is run, all imported from the reference checkout, nothing re-implemented:
  * ``nf4_grouped.dequant_ref``, ``mxfp4_pack_ref.dequant_mxfp4``       (decode)
  * ``nf4_pack_ref.quantize_pack_nf4``, ``mxfp4_pack_ref.quantize_pack_mxfp4``
  * ``cpu_grouped.ref_gemv_grouped`` / ``ordered_dgrad_ref`` (numpy spec) and the
    native ``gemv_*_grouped_cpu`` / ``dgrad_*_grouped_cpu``           (locked order)
  * ``gemm_4bit_grouped`` / ``dgrad_4bit_grouped`` / ``gemm_mxfp4_grouped`` -- the
    reference's Triton kernels, executed by the Triton interpreter on CPU
  * ``build_group_tiles``, ``_decode_plan``, ``decode_dispatch``, ``_prefill_block_m``
  * ``cpu_grouped.route_epilogue_bf16`` and the stable-argsort dispatch producer
    of ``mxfp4_qlora._forward_fused`` (restated inline from its five lines,
    kernel/mxfp4_qlora.py:294-329, because that module needs a model to import)

Usage (in a container that has the reference checkout):
    TRITON_INTERPRET=1 CC=/usr/bin/gcc GNF4_NATIVE_CACHE=/tmp/gnf4cache \
    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [REFERENCE_CHECKOUT]
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
if os.path.exists("/usr/bin/gcc"):      # the image default CC has no OpenMP spec file
    os.environ["CC"] = "/usr/bin/gcc"
os.environ.setdefault("GNF4_NATIVE_CACHE", "/tmp/gnf4_native_cache")
sys.dont_write_bytecode = True

# the reference checkout: first argument, else GNF4_REFERENCE_ROOT, else a directory named `reference` beside this repository
REF = Path(sys.argv[1] if len(sys.argv) > 1 else
           os.environ.get("GNF4_REFERENCE_ROOT") or Path(__file__).resolve().parents[3] / "reference")
sys.path[:0] = [str(REF / "kernel"), str(REF)]
OUT = Path(__file__).resolve().parent

import numpy as np  # noqa: E402
import torch  # noqa: E402

import cpu_grouped as cg  # noqa: E402
import mxfp4_grouped  # noqa: E402
import nf4_grouped  # noqa: E402
from mxfp4_pack_ref import dequant_mxfp4, quantize_pack_mxfp4  # noqa: E402
from nf4_pack_ref import quantize_pack_nf4  # noqa: E402


def bits32(t):
    return t.contiguous().view(torch.int32).numpy().astype(np.uint32)


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


# --------------------------------------------------------------------------- #
def golden_decode():
    g = torch.Generator().manual_seed(11)
    # NF4: rows 0..15 = every code in both nibble positions; rest random
    N, K = 48, 256
    B = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    for c in range(16):
        B[c, :] = (c << 4) | (15 - c)
    am = torch.rand(N, K // 64, generator=g) * 3 + 0.01
    am[16] = 1e-30
    am[17] = 1e30
    am[18] = 1e-38
    am[19, 0::2] = 1e30
    am[19, 1::2] = 1e-30
    am[20] = 1.0
    w = nf4_grouped.dequant_ref(B, am, N, K)
    am16 = am.to(torch.bfloat16)
    w16 = nf4_grouped.dequant_ref(B, am16, N, K)    # bf16 absmax widened by the ref
    # MXFP4: all scale edge bytes, all 256 byte values
    N2, K2 = 40, 256
    B2 = torch.randint(0, 256, (N2, K2 // 2), dtype=torch.uint8, generator=g)
    B2[0, :] = torch.arange(128, dtype=torch.uint8)
    B2[1, :] = torch.arange(128, 256).to(torch.uint8)
    S2 = torch.randint(100, 140, (N2, K2 // 32), dtype=torch.uint8, generator=g)
    edge = [0, 1, 2, 119, 120, 121, 122, 123, 124, 125, 126, 127, 128, 253, 254, 255]
    for i, e in enumerate(edge):
        S2[2 + i, :] = e
    S2[0, :] = 127
    S2[1, :] = 127
    w2 = dequant_mxfp4(B2.reshape(N2, K2 // 32, 16), S2)
    np.savez_compressed(
        OUT / "decode.npz",
        nf4_packed=B.numpy(), nf4_absmax=am.numpy(), nf4_w_bits=bits32(w),
        nf4_absmax_bf16_bits=bits16(am16), nf4_w_bf16am_bits=bits32(w16),
        mx_packed=B2.numpy(), mx_scales=S2.numpy(), mx_w_bits=bits32(w2),
    )


# --------------------------------------------------------------------------- #
def golden_locked():
    rng = np.random.default_rng(0)
    E, N, K = 4, 24, 128
    sizes, eids = [1, 2, 1], [2, 0, 3]
    out = {}
    packed = rng.integers(0, 256, size=(E, N, K // 2), dtype=np.uint8)
    absmax = rng.random(size=(E, N, K // 64), dtype=np.float32) + 0.5
    scales = rng.integers(100, 140, size=(E, N, K // 32), dtype=np.uint8)
    scales[0, 0, 0] = 0xFF
    scales[0, 0, 1] = 0
    scales[3, 3, 2] = 0xFF
    a = rng.standard_normal((sum(sizes), K), dtype=np.float32)
    gr = rng.standard_normal((sum(sizes), N), dtype=np.float32)
    out.update(packed=packed, absmax=absmax, scales=scales, a=a, g=gr,
               sizes=np.asarray(sizes, np.int32), eids=np.asarray(eids, np.int32))
    spec_nf4 = cg.ref_gemv_grouped(a, packed, absmax, sizes, eids, fmt="nf4")
    spec_mx = cg.ref_gemv_grouped(a, packed, scales, sizes, eids, fmt="mxfp4")
    dg_nf4 = cg.ordered_dgrad_ref(gr, packed, absmax, sizes, eids, fmt="nf4")
    dg_mx = cg.ordered_dgrad_ref(gr, packed, scales, sizes, eids, fmt="mxfp4")
    assert cg.cpu_kernels_available(), "reference native CPU kernels did not build"
    t = torch.from_numpy
    nat_nf4 = cg.gemv_nf4_grouped_cpu(t(a), t(packed), t(absmax), sizes, eids).numpy()
    nat_mx = cg.gemv_mxfp4_grouped_cpu(t(a), t(packed), t(scales), sizes, eids).numpy()
    nat_dg = cg.dgrad_nf4_grouped_cpu(t(gr), t(packed), t(absmax), sizes, eids).numpy()
    nat_dgm = cg.dgrad_mxfp4_grouped_cpu(t(gr), t(packed), t(scales), sizes, eids).numpy()
    same = lambda x, y: np.array_equal(x.view(np.uint32), y.view(np.uint32))  # noqa: E731
    assert same(spec_nf4, nat_nf4) and same(spec_mx, nat_mx)
    assert same(dg_nf4, nat_dg) and same(dg_mx, nat_dgm)
    out.update(fwd_nf4_bits=spec_nf4.view(np.uint32), fwd_mx_bits=spec_mx.view(np.uint32),
               dgrad_nf4_bits=dg_nf4.view(np.uint32), dgrad_mx_bits=dg_mx.view(np.uint32))
    np.savez_compressed(OUT / "locked_order.npz", **out)


# --------------------------------------------------------------------------- #
def _nf4_stack(E, N, K, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    B = torch.empty(E, N, K // 2, dtype=torch.uint8)
    A = torch.empty(E, N, K // 64, dtype=torch.float32)
    for e in range(E):
        B[e], A[e] = quantize_pack_nf4(torch.randn(N, K, generator=g) * scale)
    return B, A


def _mx_stack(E, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    B = torch.empty(E, N, K // 2, dtype=torch.uint8)
    S = torch.empty(E, N, K // 32, dtype=torch.uint8)
    for e in range(E):
        b, s = quantize_pack_mxfp4(torch.randn(N, K, generator=g) * 0.3)
        B[e], S[e] = b.reshape(N, K // 2), s
    return B, S


def golden_interp():
    """The reference's Triton kernels, run by the Triton interpreter, on cases
    that cover decode, split-K decode, the M-tile path, ragged N, repeated and
    unsorted experts, and dgrad."""
    cases = [  # name, fmt, E, N, K, sizes, eids, kwargs
        ("nf4_decode", "nf4", 4, 128, 256, [1, 1, 1], [1, 3, 0], {}),
        ("nf4_decode_splitk", "nf4", 2, 64, 512, [1, 1], [1, 0], {"split_k": 4}),
        ("nf4_prefill", "nf4", 4, 128, 128, [65, 1, 17], [2, 0, 3], {"prefill_variant": 0}),
        ("nf4_ragged_n", "nf4", 3, 130, 128, [1, 1], [0, 2], {}),
        ("nf4_same_expert", "nf4", 2, 96, 128, [1] * 12, [0] * 12, {}),
        ("nf4_mixed", "nf4", 5, 72, 192, [3, 2, 1, 3], [4, 4, 0, 2], {"prefill_variant": 0}),
        ("mx_decode", "mxfp4", 4, 128, 256, [1, 1, 1, 1], [0, 1, 2, 3], {}),
        ("mx_prefill", "mxfp4", 4, 128, 128, [3, 1, 4, 2], [1, 0, 3, 2], {"prefill_variant": 0}),
        ("mx_ragged", "mxfp4", 3, 96, 160, [2, 5], [2, 0], {"prefill_variant": 0}),
    ]
    out = {}
    meta = {}
    for i, (name, fmt, E, N, K, sizes, eids, kw) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        a = torch.randn(sum(sizes), K, generator=g).to(torch.bfloat16)
        ids_t = torch.tensor(eids, dtype=torch.int32)
        if fmt == "nf4":
            B, S = _nf4_stack(E, N, K, seed=i)
            got = nf4_grouped.gemm_4bit_grouped(a, B, S, sizes, ids_t, **kw)
        else:
            B, S = _mx_stack(E, N, K, seed=i)
            got = mxfp4_grouped.gemm_mxfp4_grouped(a, B, S, sizes, ids_t, **kw)
        out[f"{name}.W"] = B.numpy()
        out[f"{name}.S"] = S.numpy()
        out[f"{name}.a_bits"] = bits16(a)
        out[f"{name}.out_bits"] = bits16(got)
        meta[name] = dict(fmt=fmt, E=E, N=N, K=K, sizes=sizes, eids=eids)
    # dgrad (NF4 only in the reference's GPU path)
    for j, rows in enumerate([(3, 3, 3, 3), (1, 7, 2, 5), (33, 1, 1, 1)]):
        name = f"nf4_dgrad_{j}"
        E, N, K = 4, 128, 128
        B, S = _nf4_stack(E, N, K, seed=50 + j)
        g = torch.Generator().manual_seed(200 + j)
        go = torch.randn(sum(rows), N, generator=g).to(torch.bfloat16)
        got = nf4_grouped.dgrad_4bit_grouped(go, B, S, list(rows), list(range(E)))
        out[f"{name}.W"] = B.numpy()
        out[f"{name}.S"] = S.numpy()
        out[f"{name}.a_bits"] = bits16(go)
        out[f"{name}.out_bits"] = bits16(got)
        meta[name] = dict(fmt="nf4", op="dgrad", E=E, N=N, K=K, sizes=list(rows), eids=list(range(E)))
    np.savez_compressed(OUT / "reference_kernels_interp.npz", **out)
    (OUT / "reference_kernels_interp.json").write_text(json.dumps(meta, indent=1))


# --------------------------------------------------------------------------- #
def golden_plans():
    rec = {"decode_plan": [], "decode_dispatch": [], "prefill_block_m": [], "group_tiles": []}
    for (N, K, T, sm) in [(2048, 768, 8, 26), (2048, 768, 8, 64), (5120, 8192, 1, 64),
                          (2048, 2048, 8, 26), (1408, 2816, 8, 64), (1536, 2048, 8, 148),
                          (2880, 2880, 8, 64), (64, 64, 1, 64), (6144, 768, 1, 64),
                          (64, 8192, 1, 64), (1024, 4096, 1, 148), (1536, 2048, 1, 148),
                          (5760, 2880, 4, 148), (128, 16384, 1, 148)]:
        rec["decode_plan"].append([[N, K, T, sm], list(nf4_grouped._decode_plan(N, K, T, sm))])
        rec["decode_dispatch"].append([[N, K, T, sm], list(nf4_grouped.decode_dispatch(N, K, T, sm))])
    for m in (1, 15, 16, 17, 32, 33, 64, 65, 128, 129, 256, 4096):
        rec["prefill_block_m"].append([m, nf4_grouped._prefill_block_m(m)])
    for sizes, bm in [([3, 1, 0, 5, 2], 4), ([65, 17], 64), ([1, 1, 1], 16), ([200], 128),
                      ([0, 0, 7], 16), ([129, 128, 127], 128), ([], 16)]:
        a, b, c = nf4_grouped.build_group_tiles(sizes, bm, "cpu")
        rec["group_tiles"].append([sizes, bm, a.tolist(), b.tolist(), c.tolist()])
    # tensor-valued sizes must not be mutated (kernel/test_group_tiles_readonly.py)
    t = torch.tensor([3, 2], dtype=torch.int32)
    nf4_grouped.build_group_tiles(t, 2, "cpu")
    assert t.tolist() == [3, 2]
    rec["constants"] = dict(NF4_LUT=nf4_grouped.NF4_LUT, BLOCKSIZE=nf4_grouped.BLOCKSIZE,
                            FP4_VALUES=mxfp4_grouped.FP4_VALUES, MX_BLOCK=mxfp4_grouped.MX_BLOCK,
                            E8M0_BIAS=mxfp4_grouped.E8M0_BIAS,
                            DECODE_MIN_FUSED_BYTES=nf4_grouped.DECODE_MIN_FUSED_BYTES,
                            SPLITK_MIN_BLOCKS=nf4_grouped.SPLITK_MIN_BLOCKS,
                            DGRAD_DEFAULT=list(nf4_grouped._DGRAD_DEFAULT))
    (OUT / "plans.json").write_text(json.dumps(rec, indent=1))


# --------------------------------------------------------------------------- #
def golden_routing():
    rng = np.random.default_rng(5)
    T, E, k = 6, 64, 8
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0, 5] = logits[0, 11] = logits[0, 3]
    logits[1, :] = 0.25                       # all tied -> ids 0..k-1
    out = dict(logits=logits)
    for mode, norm in ((0, False), (0, True), (1, False)):
        idx = np.zeros((T, k), np.int64)
        wts = np.zeros((T, k), np.uint16)
        cg.route_epilogue_bf16(logits, k, mode, norm, idx, wts)
        out[f"idx_m{mode}n{int(norm)}"] = idx.astype(np.int32)
        out[f"wts_m{mode}n{int(norm)}_bf16bits"] = wts
    # dispatch producer: stable sort of token-expert pairs by expert
    ri = torch.from_numpy(out["idx_m0n0"].astype(np.int64))
    flat = ri.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok_of_pair = order // k
    uniq, counts = torch.unique_consecutive(flat[order], return_counts=True)
    out.update(order=order.numpy().astype(np.int32), tok_of_pair=tok_of_pair.numpy().astype(np.int32),
               uniq=uniq.numpy().astype(np.int32), counts=counts.numpy().astype(np.int32))
    np.savez_compressed(OUT / "routing.npz", **out)


# --------------------------------------------------------------------------- #
def golden_config1():
    """BASELINE config 1 (E=8, N=512, K=1024, 64 tokens, top-2): the reference's
    packer + its CPU path.  Inputs are regenerated from the seeds by the tests'
    own generator; this file pins their hashes and the reference's answer."""
    E, N, K, M, k = 8, 512, 1024, 64, 2
    g = torch.Generator(device="cpu").manual_seed(2026)
    B = torch.empty(E, N, K // 2, dtype=torch.uint8)
    A = torch.empty(E, N, K // 64, dtype=torch.float32)
    for e in range(E):
        B[e], A[e] = quantize_pack_nf4(torch.randn(N, K, generator=g) * 0.02)
    logits = torch.randn(M, E, generator=g)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    probs = torch.softmax(logits, dim=-1)
    idx = np.zeros((M, k), np.int64)
    wts = np.zeros((M, k), np.uint16)
    cg.route_epilogue_bf16(logits.numpy(), k, 0, False, idx, wts)
    flat = torch.from_numpy(idx).reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    uniq, counts = torch.unique_consecutive(flat[order], return_counts=True)
    a_cat = x[tok]
    sizes, eids = counts.tolist(), uniq.tolist()
    out_cpu = cg.gemv_nf4_grouped_cpu(a_cat.float(), B, A, sizes, eids)
    np.savez_compressed(
        OUT / "config1.npz",
        seed=np.int64(2026), sha_B=sha(B.numpy()), sha_A=sha(A.numpy()),
        sha_x=sha(bits16(x)), sha_probs=sha(probs.numpy()),
        sizes=np.asarray(sizes, np.int32), eids=np.asarray(eids, np.int32),
        tok_of_pair=tok.numpy().astype(np.int32),
        out_cpu_bits=out_cpu.numpy().view(np.uint32),
    )


if __name__ == "__main__":
    golden_decode()
    golden_locked()
    golden_interp()
    golden_plans()
    golden_routing()
    golden_config1()
    for p in sorted(OUT.glob("*.np*")) + sorted(OUT.glob("*.json")):
        print(p.name, p.stat().st_size)
