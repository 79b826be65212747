"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (weights N(0, 0.02) quantised to NF4, or uniform e2m1 nibbles with e8m0
exponents uniform in [119, 125]; bf16 N(0, 1) activations; top-k routing from seeded
N(0, 1) router logits, optionally with a Zipf expert-popularity skew).

Used by the tests, the smoke check and bench.py.  Generation order is fixed
(weights -> router logits -> activations) and everything is drawn from a CPU
``torch.Generator`` so the same seed gives the same bytes on any machine; large stacks
are quantised on the GPU in expert chunks from CPU-drawn normals only when ``fast=True``
(then the draw itself happens on the device and the bytes depend on the device RNG).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from mxfp4_pack_ref import MX_BLOCK
from nf4_grouped import BLOCKSIZE
from nf4_pack_ref import quantize_pack_nf4


@dataclass
class LayerShape:
    name: str
    fmt: str          # "nf4" | "mxfp4"
    experts: int
    hidden: int
    inter: int        # moe intermediate size; gate_up has N = 2*inter
    top_k: int

    @property
    def gate_up(self):   # (N, K)
        return 2 * self.inter, self.hidden

    @property
    def down(self):
        return self.hidden, self.inter


CONFIGS = {
    "c1_cpu": LayerShape("c1_cpu", "nf4", 8, 1024, 256, 2),          # E=8, N=512, K=1024
    "qwen3_30b_a3b": LayerShape("qwen3_30b_a3b", "nf4", 128, 2048, 768, 8),
    "gpt_oss_20b": LayerShape("gpt_oss_20b", "mxfp4", 32, 2880, 2880, 4),
    "deepseek_v3": LayerShape("deepseek_v3", "mxfp4", 256, 7168, 2048, 8),
}


def nf4_stack(E, N, K, gen, scale=0.02, device="cpu", bf16_absmax=False, fast=False):
    """[E,N,K/2] u8 + [E,N,K/64] absmax.  ``bf16_absmax`` quantises bf16-rounded weights so
    the absmax is exactly representable in bf16 and returns it in that dtype."""
    dev = torch.device(device)
    B = torch.empty(E, N, K // 2, dtype=torch.uint8, device=dev)
    A = torch.empty(E, N, K // BLOCKSIZE, dtype=torch.float32, device=dev)
    for e in range(E):
        if fast and dev.type == "cuda":
            w = torch.randn(N, K, device=dev, dtype=torch.float32) * scale
        else:
            w = (torch.randn(N, K, generator=gen, dtype=torch.float32) * scale).to(dev)
        if bf16_absmax:
            w = w.to(torch.bfloat16).float()
        B[e], A[e] = quantize_pack_nf4(w)
    return B, (A.to(torch.bfloat16) if bf16_absmax else A)


def mxfp4_stack(E, N, K, gen, device="cpu", e_lo=119, e_hi=125, fast=False):
    """Uniform nibbles and uniform exponents in [e_lo, e_hi]: [E,N,K/2] u8 + [E,N,K/32] u8."""
    dev = torch.device(device)
    if fast and dev.type == "cuda":
        B = torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, device=dev)
        S = torch.randint(e_lo, e_hi + 1, (E, N, K // MX_BLOCK), dtype=torch.uint8, device=dev)
        return B, S
    B = torch.randint(0, 256, (E, N, K // 2), dtype=torch.uint8, generator=gen)
    S = torch.randint(e_lo, e_hi + 1, (E, N, K // MX_BLOCK), dtype=torch.uint8, generator=gen)
    return B.to(dev), S.to(dev)


def route_topk(logits: torch.Tensor, k: int):
    """Softmax then top-k; ties go to the lower expert index (stable descending sort).
    Returns (idx [M,k] int64, weights [M,k] fp32)."""
    probs = torch.softmax(logits.float(), dim=-1)
    order = torch.argsort(-logits.float(), dim=-1, stable=True)[:, :k]
    return order, torch.gather(probs, 1, order)


def dispatch(idx: torch.Tensor, n_experts: int):
    """Token-expert pairs -> expert-sorted layout: (tok_of_pair [P], sizes list over the
    ACTIVE experts, expert_ids list, order [P]).  Stable sort, so pairs of one expert keep
    token order."""
    k = idx.shape[1]
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    uniq, counts = torch.unique_consecutive(flat[order], return_counts=True)
    return tok, counts.tolist(), uniq.tolist(), order


def zipf_logit_bias(n_experts: int, gen, alpha: float = 1.1):
    """log p_e with p_e proportional to rank(e)^-alpha under a seeded expert permutation."""
    perm = torch.randperm(n_experts, generator=gen)
    rank = torch.empty(n_experts)
    rank[perm] = torch.arange(1, n_experts + 1, dtype=torch.float32)
    p = rank.pow(-alpha)
    return torch.log(p / p.sum())


def routed_batch(shape: LayerShape, tokens: int, gen, zipf: float | None = None):
    """Router logits and bf16 activations for ``tokens`` tokens -> (x [M,hidden] bf16 CPU,
    idx [M,k], weights [M,k])."""
    logits = torch.randn(tokens, shape.experts, generator=gen)
    if zipf:
        logits = logits + zipf_logit_bias(shape.experts, gen, zipf)
    x = torch.randn(tokens, shape.hidden, generator=gen).to(torch.bfloat16)
    idx, w = route_topk(logits, shape.top_k)
    return x, idx, w
