"""Pure-torch NF4 quantise + pack for synthetic fixtures (no bitsandbytes), the drop-in for
the reference's ``kernel/nf4_pack_ref.py:20-57``.

Storage rule: per 64-element block of a row, ``absmax = max|w|`` (floored at 1e-12); every
element becomes the index of the codebook entry nearest to ``w / absmax`` (first index on a
tie); element 2j goes to the HIGH nibble of byte j, element 2j+1 to the LOW nibble.
Runs on any torch device; results are device-independent because every step is an exact
elementwise fp32 operation or an argmin.
"""
import torch

from nf4_grouped import BLOCKSIZE, NF4_LUT


def quantize_pack_nf4(w: torch.Tensor, chunk_rows: int = 256):
    """w [N, K] float -> (packed [N, K//2] uint8, absmax [N, K//64] fp32)."""
    if w.dim() != 2:
        raise ValueError(
            f"expected 2-D [N, K] per-expert weight; got shape {tuple(w.shape)} -- "
            "pack per-expert and stack, or use make_stack() for synthetic fixtures.")
    N, K = w.shape
    assert K % BLOCKSIZE == 0, f"K={K} must be a multiple of {BLOCKSIZE}"
    lut = torch.tensor(NF4_LUT, dtype=torch.float32, device=w.device)
    blocks = w.float().reshape(N, K // BLOCKSIZE, BLOCKSIZE)
    absmax = blocks.abs().amax(dim=2).clamp_min(1e-12)
    scaled = (blocks / absmax[:, :, None]).reshape(N, K)
    codes = torch.empty(N, K, dtype=torch.uint8, device=w.device)
    for r in range(0, N, chunk_rows):                      # bound the [rows, K, 16] temporary
        s = scaled[r:r + chunk_rows]
        codes[r:r + chunk_rows] = (s.unsqueeze(-1) - lut).abs().argmin(dim=-1).to(torch.uint8)
    packed = (codes[:, 0::2] << 4) | codes[:, 1::2]
    return packed.contiguous(), absmax.to(torch.float32).contiguous()


def make_stack(E: int, N: int, K: int, seed: int = 0, device: str = "cpu"):
    """E experts of seeded N(0,1) weights -> (B [E,N,K/2] u8, absmax [E,N,K/64] f32)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    B = torch.empty(E, N, K // 2, dtype=torch.uint8)
    A = torch.empty(E, N, K // BLOCKSIZE, dtype=torch.float32)
    for e in range(E):
        B[e], A[e] = quantize_pack_nf4(torch.randn(N, K, generator=g, dtype=torch.float32))
    return B.to(device), A.to(device)
