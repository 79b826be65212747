"""The oracle is only trusted once it reproduces the reference: every fixture below was
produced by running the reference project's own code (tests/golden/make_golden.py)."""
import json

import numpy as np
import pytest

from oracle import oracle as O


def test_codebooks_match_reference_constants(golden_dir):
    c = json.loads((golden_dir / "plans.json").read_text())["constants"]
    nf4, fp4 = O.luts()
    assert np.array_equal(nf4, np.asarray(c["NF4_LUT"], np.float32))
    assert np.array_equal(fp4.view(np.uint32), np.asarray(c["FP4_VALUES"], np.float32).view(np.uint32))
    assert nf4[7] == 0.0 and c["BLOCKSIZE"] == 64 and c["MX_BLOCK"] == 32 and c["E8M0_BIAS"] == 127


def test_nf4_decode_is_bit_exact(golden_dir):
    g = np.load(golden_dir / "decode.npz")
    w = O.decode_stack("nf4", g["nf4_packed"][None], g["nf4_absmax"][None])[0]
    assert np.array_equal(w.view(np.uint32), g["nf4_w_bits"])
    # bf16 absmax widened exactly
    w16 = O.decode_stack("nf4", g["nf4_packed"][None], g["nf4_absmax_bf16_bits"][None])[0]
    assert np.array_equal(w16.view(np.uint32), g["nf4_w_bf16am_bits"])
    # every code in both nibble positions (rows 0..15: code c high, 15-c low), absmax row 20 == 1
    nf4, _ = O.luts()
    B = np.zeros((1, 16, 32), np.uint8)
    for c in range(16):
        B[0, c] = (c << 4) | (15 - c)
    one = O.decode_stack("nf4", B, np.ones((1, 16, 1), np.float32))[0]
    for c in range(16):
        assert np.all(one[c, 0::2] == nf4[c]) and np.all(one[c, 1::2] == nf4[15 - c])


def test_mxfp4_decode_is_bit_exact_including_scale_edges(golden_dir):
    g = np.load(golden_dir / "decode.npz")
    w = O.decode_stack("mxfp4", g["mx_packed"][None], g["mx_scales"][None])[0]
    assert np.array_equal(w.view(np.uint32), g["mx_w_bits"])
    # known answer: byte 0x21 under scale 127 -> (0.5, 1.0): low nibble is the even element
    B = np.full((1, 1, 16), 0x21, np.uint8)
    S = np.full((1, 1, 1), 127, np.uint8)
    w = O.decode_stack("mxfp4", B, S)[0, 0]
    assert w[0] == 0.5 and w[1] == 1.0
    # 0xFF scale (2^128): zeros stay zero (ldexp), 0.5 becomes the finite 2^127, 1.0 overflows
    B = np.full((1, 1, 16), 0x10, np.uint8)      # even element code 0 (0.0), odd code 1 (0.5)
    B[0, 0, 1] = 0x2A                            # even code 10 (-1.0), odd code 2 (1.0)
    w = O.decode_stack("mxfp4", B, np.full((1, 1, 1), 255, np.uint8))[0, 0]
    assert w[0] == 0.0 and w[1] == np.float32(2.0) ** 127 and w[2] == -np.inf and w[3] == np.inf


@pytest.mark.parametrize("fmt,skey,fkey,dkey", [("nf4", "absmax", "fwd_nf4_bits", "dgrad_nf4_bits"),
                                                ("mxfp4", "scales", "fwd_mx_bits", "dgrad_mx_bits")])
def test_locked_order_matches_reference_spec_and_native(golden_dir, fmt, skey, fkey, dkey):
    g = np.load(golden_dir / "locked_order.npz")
    with np.errstate(all="ignore"):
        fwd = O.gemv_grouped_locked(fmt, g["a"], g["packed"], g[skey], g["sizes"], g["eids"])
        dg = O.dgrad_grouped_locked(fmt, g["g"], g["packed"], g[skey], g["sizes"], g["eids"])

    def same(a, bits):
        a = a.view(np.uint32)
        nan_a = np.isnan(a.view(np.float32))
        nan_b = np.isnan(bits.view(np.float32))
        return np.array_equal(nan_a, nan_b) and np.array_equal(a[~nan_a], bits[~nan_b])

    assert same(fwd, g[fkey])
    assert same(dg, g[dkey])


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (no reference checkout)")
@pytest.mark.parametrize("fmt", ["nf4", "mxfp4"])
def test_oracle_equals_compiled_reference_kernels_bitwise(fmt):
    """oracle/_ref is the reference's cpu_kernels.c compiled as-is; the restated locked
    order must give the same bits on fresh random inputs, forward and dgrad."""
    rng = np.random.default_rng(42)
    E, N, K = 5, 40, 256
    sizes, eids = [2, 1, 9, 3], [4, 0, 0, 2]
    W = rng.integers(0, 256, size=(E, N, K // 2), dtype=np.uint8)
    if fmt == "nf4":
        S = (rng.random(size=(E, N, K // 64), dtype=np.float32) + 0.25)
    else:
        S = rng.integers(110, 135, size=(E, N, K // 32), dtype=np.uint8)
    a = rng.standard_normal((sum(sizes), K), dtype=np.float32)
    gr = rng.standard_normal((sum(sizes), N), dtype=np.float32)
    for threads in (1, 4):
        ref = O.ref_call("gemv", fmt, a, W, S, sizes, eids, threads=threads)
        assert np.array_equal(ref.view(np.uint32), O.gemv_grouped_locked(fmt, a, W, S, sizes, eids).view(np.uint32))
        refd = O.ref_call("dgrad", fmt, gr, W, S, sizes, eids, threads=threads)
        assert np.array_equal(refd.view(np.uint32), O.dgrad_grouped_locked(fmt, gr, W, S, sizes, eids).view(np.uint32))


def test_fp64_oracle_brackets_the_reference_triton_kernels(golden_dir):
    """The reference's own kernels (run by the Triton interpreter) against the fp64 oracle:
    their bf16 outputs must sit within bf16 resolution of it (the interpreter truncates
    fp32 -> bf16 instead of rounding, so the bound is one bf16 ulp, up to 2^-7 relative, not half of
    one).  This pins the oracle's grouping semantics (row ranges, expert indexing, nibble
    order, dgrad orientation) on the reference's actual outputs."""
    meta = json.loads((golden_dir / "reference_kernels_interp.json").read_text())
    g = np.load(golden_dir / "reference_kernels_interp.npz")
    for name, m in meta.items():
        x = O.bf16_bits_to_f32(g[f"{name}.a_bits"])
        out = O.bf16_bits_to_f32(g[f"{name}.out_bits"])
        fn = O.dgrad_grouped_f64 if m.get("op") == "dgrad" else O.gemm_grouped_f64
        ref = fn(m["fmt"], x, g[f"{name}.W"], g[f"{name}.S"], m["sizes"], m["eids"])
        assert out.shape == ref.shape, name
        assert O.rel_frobenius(out, ref) < 4e-3, (name, O.rel_frobenius(out, ref))
        assert O.max_rel(out, ref) < 2 ** -7, (name, O.max_rel(out, ref))


def test_group_tiles_and_offsets_match_reference(golden_dir):
    rec = json.loads((golden_dir / "plans.json").read_text())
    for sizes, bm, r0, rows, grp in rec["group_tiles"]:
        a, b, c = O.group_tiles(sizes, bm)
        assert a.tolist() == r0 and b.tolist() == rows and c.tolist() == grp
        off = O.group_offsets(sizes)
        assert off.tolist() == np.concatenate([[0], np.cumsum(sizes)]).astype(int).tolist()


def test_router_rule_matches_reference_epilogue(golden_dir):
    g = np.load(golden_dir / "routing.npz")
    for mode, norm in ((0, False), (0, True), (1, False)):
        idx, w = O.route_topk(g["logits"], 8, mode, norm)
        assert np.array_equal(idx, g[f"idx_m{mode}n{int(norm)}"])
        assert np.array_equal(O.round_bf16_bits(w), g[f"wts_m{mode}n{int(norm)}_bf16bits"])
    order, counts = O.sort_pairs(g["idx_m0n0"].reshape(-1), 64)
    assert np.array_equal(order, g["order"])
    assert np.array_equal(order // 8, g["tok_of_pair"])
    assert np.array_equal(np.nonzero(counts)[0], g["uniq"])
    assert np.array_equal(counts[counts > 0], g["counts"])


def test_config1_reference_cpu_path(golden_dir):
    """BASELINE config 1 end to end on the CPU: same packer bytes, same routing, and the
    locked-order oracle reproduces the reference's native output bit for bit."""
    import hashlib
    import torch
    import synth
    from nf4_pack_ref import quantize_pack_nf4

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
    assert sha(x.view(torch.int16).numpy().view(np.uint16)) == str(g["sha_x"])
    idx, _ = synth.route_topk(logits, k)
    tok, sizes, eids, _ = synth.dispatch(idx, E)
    assert sizes == g["sizes"].tolist() and eids == g["eids"].tolist()
    assert np.array_equal(tok.numpy(), g["tok_of_pair"])
    out = O.gemv_grouped_locked("nf4", x[tok].float().numpy(), B.numpy(), A.numpy(), sizes, eids)
    assert np.array_equal(out.view(np.uint32), g["out_cpu_bits"])


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (no reference checkout)")
def test_ffn_oracle_brackets_the_compiled_reference_ffn():
    """The restated expert FFN (fp64) against the reference project's own fused CPU kernel (fp32, its
    polynomial SiLU): agreement at fp32 accumulation level pins gate/up halves, SiLU-GLU and operand order."""
    from nf4_pack_ref import make_stack
    B_gu, A_gu = make_stack(3, 256, 128, seed=51)
    B_dn, A_dn = make_stack(3, 64, 128, seed=52)
    rng = np.random.default_rng(5)
    for sizes, ids in (([1, 1], [2, 0]), ([3, 5, 2], [1, 0, 1])):
        a = rng.standard_normal((sum(sizes), 128)).astype(np.float32)
        ref = O.ref_ffn_call(a, B_gu.numpy(), A_gu.numpy(), B_dn.numpy(), A_dn.numpy(), sizes, ids)
        want = O.ffn_grouped_f64(a, B_gu.numpy(), A_gu.numpy(), B_dn.numpy(), A_dn.numpy(), sizes, ids)
        assert O.rel_frobenius(ref.astype(np.float64), want) < 2e-5
