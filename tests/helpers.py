"""Shared test helpers: torch <-> numpy views, fp64 references through the oracle."""
import numpy as np
import torch

from oracle import oracle as O


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def from_bf16_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16)


def f32_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int32).numpy().view(np.uint32)


def scales_np(S: torch.Tensor) -> np.ndarray:
    """Scale tensor as the oracle takes it (bf16 absmax as its uint16 bit pattern)."""
    S = S.detach().cpu().contiguous()
    if S.dtype == torch.bfloat16:
        return S.view(torch.int16).numpy().view(np.uint16)
    return S.numpy()


def oracle_fwd64(fmt, a, W, S, sizes, eids):
    return O.gemm_grouped_f64(fmt, a.detach().cpu().float().numpy(), W.detach().cpu().numpy(), scales_np(S),
                              list(sizes), list(eids))


def oracle_dgrad64(fmt, g, W, S, sizes, eids):
    return O.dgrad_grouped_f64(fmt, g.detach().cpu().float().numpy(), W.detach().cpu().numpy(), scales_np(S),
                               list(sizes), list(eids))


def rel_fro(out: torch.Tensor, ref64: np.ndarray) -> float:
    return O.rel_frobenius(out.detach().cpu().double().numpy(), ref64)


def max_rel(out: torch.Tensor, ref64: np.ndarray) -> float:
    return O.max_rel(out.detach().cpu().double().numpy(), ref64)


def bf16_round(ref64: np.ndarray) -> torch.Tensor:
    """fp64 reference rounded once to bf16 (what an exact kernel would return)."""
    return torch.from_numpy(ref64).to(torch.float32).to(torch.bfloat16)
