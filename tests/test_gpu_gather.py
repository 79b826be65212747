"""Residency feeders (device-side gathers of packed expert row-blocks into slots) against the byte-level oracle:
bit-exact, from device memory and from pinned host memory, with the have-skip, 8-byte (not 16-byte) aligned rows,
the permuting piece table, a bad id, and rows that span many CTAs; then a gathered slot buffer fed to the grouped GEMM."""
import numpy as np
import pytest
import torch

import _gnf4b
import host_gather
import nf4_grouped
import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rows(E, row_bytes, seed):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (E, row_bytes), dtype=torch.uint8, generator=gen)


@pytest.mark.parametrize("row_bytes", [8, 24, 4096, 70000 * 8, 3 * 1024 * 1024 + 16])
@pytest.mark.parametrize("where", ["device", "pinned"])
def test_gather_by_id_is_byte_exact_and_skips_resident_slots(row_bytes, where):
    E, k = 7, 5
    src = _rows(E, row_bytes, seed=row_bytes % 97)
    store = src.to(DEV) if where == "device" else src.pin_memory()
    ids = torch.tensor([3, 0, 6, 3, 1], dtype=torch.int32, device=DEV)
    have = torch.tensor([3, 5, -1, 2, 1], dtype=torch.int32, device=DEV)        # slots 0 and 4 already hold their rows
    dst = torch.full((k, row_bytes), 0xAB, dtype=torch.uint8, device=DEV)
    host_gather.gather_expert_rows(dst, store, ids)
    want = O.gather_rows_ref(np.full((k, row_bytes), 0xAB, np.uint8), src.numpy(), ids.cpu().numpy())
    assert np.array_equal(dst.cpu().numpy(), want)
    dst.fill_(0xCD)
    host_gather.gather_expert_rows(dst, store, ids, have)
    want = O.gather_rows_ref(np.full((k, row_bytes), 0xCD, np.uint8), src.numpy(), ids.cpu().numpy(), have.cpu().numpy())
    assert np.array_equal(dst.cpu().numpy(), want)
    assert (dst[0] == 0xCD).all() and (dst[4] == 0xCD).all()                     # skipped slots were not touched
    assert nf4_grouped.last_status(DEV) == 0


def test_gather_by_id_flags_an_id_outside_the_stack():
    src = _rows(4, 256, seed=1).to(DEV)
    ids = torch.tensor([1, 9, -2], dtype=torch.int32, device=DEV)
    dst = torch.zeros(3, 256, dtype=torch.uint8, device=DEV)
    host_gather.gather_expert_rows(dst, src, ids)
    assert torch.equal(dst[0], src[1]) and not dst[1].any() and not dst[2].any()
    assert nf4_grouped.last_status(DEV) & _gnf4b.ST_BAD_EXPERT


@pytest.mark.parametrize("where", ["device", "pinned"])
def test_gather_by_address_with_and_without_a_piece_table(where):
    """Absolute addresses per slot (rows of two different stores), the have-skip on addresses, and a piece table that
    lands the row's three segments in a different order (8-byte aligned offsets that are not 16-byte aligned)."""
    row_bytes = 40 + 4096 + 808
    a = _rows(3, row_bytes, seed=5)
    b = _rows(2, row_bytes, seed=6)
    sa, sb = (a.to(DEV), b.to(DEV)) if where == "device" else (a.pin_memory(), b.pin_memory())
    picks = [(sa, a, 2), (sb, b, 0), (sa, a, 0), (sb, b, 1)]
    want_addr = torch.tensor([s.data_ptr() + i * row_bytes for s, _, i in picks], dtype=torch.int64, device=DEV)
    dst = torch.full((4, row_bytes), 0x11, dtype=torch.uint8, device=DEV)
    host_gather.gather_rows_addr(dst, want_addr)
    for j, (_, host_rows, i) in enumerate(picks):
        assert torch.equal(dst[j].cpu(), host_rows[i]), j
    have_addr = want_addr.clone()
    have_addr[1] = 0
    dst.fill_(0x22)
    host_gather.gather_rows_addr(dst, want_addr, have_addr)
    assert (dst[0] == 0x22).all() and torch.equal(dst[1].cpu(), b[0]) and (dst[2] == 0x22).all()
    # segments [0, 40) [40, 4136) [4136, 4944) of the source land as [4904, 4944) [808, 4904) [0, 808)
    pieces = [(0, 4904, 40), (40, 808, 4096), (4136, 0, 808)]
    tab = host_gather.piece_table(pieces, DEV)
    dst.fill_(0x33)
    host_gather.gather_rows_addr(dst, want_addr, None, tab)
    for j, (_, host_rows, i) in enumerate(picks):
        ref = O.gather_rows_ref(np.full((1, row_bytes), 0x33, np.uint8), host_rows.numpy(), [i], None, pieces)[0]
        assert np.array_equal(dst[j].cpu().numpy(), ref), j


def test_gathered_slots_feed_the_grouped_gemm():
    """The use the feeders exist for: experts' packed rows and scales gathered from a pinned host store into device
    slots by device-resident ids, then multiplied where they lie (expert id = slot index)."""
    E, N, K, k = 6, 256, 512, 3
    gen = torch.Generator().manual_seed(8)
    B, A = synth.nf4_stack(E, N, K, gen)
    Bh, Ah = B.pin_memory(), A.pin_memory()
    ids = torch.tensor([4, 1, 5], dtype=torch.int32, device=DEV)
    slots_B = torch.empty(k, N, K // 2, dtype=torch.uint8, device=DEV)
    slots_A = torch.empty(k, N, K // 64, dtype=torch.float32, device=DEV)
    host_gather.gather_expert_rows(slots_B, Bh, ids)
    host_gather.gather_expert_rows(slots_A, Ah, ids)
    x = torch.randn(k, K, generator=gen).to(torch.bfloat16).to(DEV)
    got = nf4_grouped.gemm_4bit_grouped(x, slots_B, slots_A, [1, 1, 1], [0, 1, 2])
    want = nf4_grouped.gemm_4bit_grouped(x, B.to(DEV), A.to(DEV), [1, 1, 1], ids.tolist())
    assert torch.equal(got, want)


def test_gather_refuses_what_it_cannot_move():
    dst = torch.zeros(2, 12, dtype=torch.uint8, device=DEV)           # 12-byte rows: not 8-byte words
    with pytest.raises(ValueError):
        host_gather.gather_expert_rows(dst, torch.zeros(3, 12, dtype=torch.uint8, device=DEV),
                                       torch.zeros(2, dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError):                                  # pageable host memory is not addressable
        host_gather.gather_expert_rows(torch.zeros(2, 16, dtype=torch.uint8, device=DEV), torch.zeros(3, 16, dtype=torch.uint8),
                                       torch.zeros(2, dtype=torch.int32, device=DEV))
    with pytest.raises(ValueError):
        host_gather.piece_table([(0, 4, 8)], DEV)
