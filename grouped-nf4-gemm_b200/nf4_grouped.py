"""Grouped W4A16 GEMM over NF4 expert stacks on NVIDIA B200 -- the drop-in for the
reference module of the same name (pjordanandrsn/grouped-nf4-gemm, kernel/nf4_grouped.py).

Same entry points, argument meaning and error behaviour:

    gemm_4bit_grouped(a_cat, B, absmax, sizes, expert_ids, ...)   -> [T, N] bf16   (ref :697-907)
    dgrad_4bit_grouped(grad_out, B, absmax, sizes, expert_ids)    -> [T, K] bf16   (ref :1056-1121)

What differs is everything below the call: no Triton, no backend detection.  Each call is
one launch of a hand-written sm_100a kernel from ``libgnf4b.so`` (C ABI in
``include/gnf4b.h``) that walks a device-side schedule built from ``group_offsets`` and
``expert_ids``; the host never builds a tile table.  There is no CPU fallback: tensors that
are not on a CUDA device raise the same taught ``RuntimeError`` as the reference
(ref :732-738), and a missing library raises at the first launch.

Helpers that other layers of the reference import from this module keep their names and
values: ``dequant_ref``, ``repack_from_bnb``, ``build_group_tiles``, ``to_device_i32``,
``decode_dispatch``, ``_decode_plan``, ``_prefill_block_m``, ``dgrad_eligible``,
``_DGRAD_DEFAULT``, ``_sm_count``, ``_lut``, ``_arena``, ``_ARENAS``, ``_PinnedIndexArena``,
``NF4_LUT``, ``BLOCKSIZE``.  The Triton-specific tuning keywords are accepted and do not
change results.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

import _gnf4b

# bitsandbytes / QLoRA NF4 codebook; code 7 is exactly 0.0 (ref :53-70).
NF4_LUT = [
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
]
BLOCKSIZE = 64
#: expert id of a padding group: its rows are skipped and its output rows left untouched
#: (include/gnf4b.h GNF4B_PAD_EXPERT; no counterpart in the reference)
PAD_EXPERT = -1

# Product-layer hints of the reference (ref :605-606); kept so callers that consult
# decode_dispatch() keep working.  They were measured on sm_86 and do not steer this op.
DECODE_MIN_FUSED_BYTES = 3_000_000
SPLITK_MIN_BLOCKS = 32
_DGRAD_DEFAULT = (32, 64, 64, 2)

_LUT_CACHE: dict = {}
_SM_CACHE: dict = {}
_STATUS: dict = {}


# --------------------------------------------------------------------------- #
# small-int transfers (capture-legal), ref :99-331
# --------------------------------------------------------------------------- #
class _PinnedIndexArena:
    """Pinned host staging for the small int32 tensors a call needs (group offsets,
    expert ids).

    Two regions.  ``take`` hands out PERMANENT slices and is what a call uses while the
    current stream is being captured into a CUDA graph: a captured host-to-device copy
    re-reads its pinned source on every replay, so those bytes may never be reused, the
    watermark never rewinds, and the arena refuses to grow inside a capture (allocating
    pinned memory there breaks the capture) -- the semantics of the reference's arena
    (ref :99-217).  Outside a capture ``stage`` cycles through a small ring of slots, each
    guarded by an event recorded after its copy, so an eager call pays one asynchronous
    pinned copy and no stream synchronisation.
    """

    DEFAULT_INTS = int(os.environ.get("GNF4_PIN_ARENA_INTS", 1 << 20))
    RING_SLOTS = 64
    RING_SLOT_INTS = 8192

    def __init__(self, device, n: int | None = None):
        self.device = device
        self.host = torch.empty(n or self.DEFAULT_INTS, dtype=torch.int32, pin_memory=True)
        self.off = 0
        self._retired: list = []
        self._ring = torch.empty(self.RING_SLOTS * self.RING_SLOT_INTS, dtype=torch.int32, pin_memory=True)
        self._ring_np = self._ring.numpy()          # same memory; list -> pinned bytes without a torch op
        self._ring_evt = [None] * self.RING_SLOTS
        self._ring_next = 0

    @staticmethod
    def _capturing() -> bool:
        try:
            return torch.cuda.is_current_stream_capturing()
        except Exception:
            return False

    def take(self, n: int):
        capturing = self._capturing()
        if self.off + n > self.host.numel():
            if capturing:
                need = 2 * (self.off + n)
                raise RuntimeError(
                    f"grouped-nf4: the pinned index arena ({self.host.numel()} int32, {self.off} already "
                    f"owned by this process's captures) cannot hold {n} more ints, and growing it would "
                    "allocate pinned memory inside the capture region, which is not capturable. Slices "
                    "taken under capture are permanent (replays re-read them): set GNF4_PIN_ARENA_INTS "
                    f"to at least {need} ({need * 4 / 2**20:.1f} MiB pinned) or call reserve() before capturing.")
            self._grow(self.off + n)
        view = self.host[self.off:self.off + n]
        self.off += n
        return view, capturing

    def _grow(self, need: int):
        self._retired.append(self.host)          # live graphs may still read it
        fresh = torch.empty(max(2 * self.host.numel(), need), dtype=torch.int32, pin_memory=True)
        fresh[: self.off] = self.host[: self.off]
        self.host = fresh

    def reserve(self, n_more: int):
        if self._capturing():
            raise RuntimeError("reserve() inside a capture would allocate pinned memory in the region; "
                               "call it before capturing.")
        if self.off + n_more > self.host.numel():
            self._grow(self.off + n_more)

    def mark(self):
        """Kept for call-site compatibility; permanence made it a no-op."""

    def stage(self, n: int):
        """A reusable pinned slot of n ints for an eager (uncaptured) call, or None when n
        does not fit a slot."""
        if n > self.RING_SLOT_INTS:
            return None, -1
        i = self._ring_next
        self._ring_next = (i + 1) % self.RING_SLOTS
        evt = self._ring_evt[i]
        if evt is not None:
            evt.synchronize()
        lo = i * self.RING_SLOT_INTS
        return self._ring[lo: lo + n], i

    def staged(self, slot: int):
        if self._ring_evt[slot] is None:
            self._ring_evt[slot] = torch.cuda.Event()
        self._ring_evt[slot].record()


_ARENAS: dict = {}


def _arena(device) -> _PinnedIndexArena:
    key = str(device)
    if key not in _ARENAS:
        _ARENAS[key] = _PinnedIndexArena(device)
    return _ARENAS[key]


class _IndexRing:
    """Per (device, stream) staging for the group tables of eager calls: a pinned host ring
    and a device ring of the same shape.  A call writes its ints into the next host slot
    (numpy view, no torch op), issues ONE asynchronous copy to the matching device slot on
    the call's stream and hands the kernel the device slot's address.  Slots are recycled
    in blocks of eight; a block is reused only after the event recorded behind its last
    copy has completed, and copies and kernels of one stream are ordered, so neither side
    of a slot is overwritten while something still reads it."""

    SLOTS, SLOT_INTS, BLOCK = 64, 4096, 8

    def __init__(self, dev):
        self.host = torch.empty(self.SLOTS * self.SLOT_INTS, dtype=torch.int32, pin_memory=True)
        self.np = self.host.numpy()
        self.dev = torch.empty(self.SLOTS * self.SLOT_INTS, dtype=torch.int32, device=dev)
        self.host_ptr, self.dev_ptr = self.host.data_ptr(), self.dev.data_ptr()
        self.events = [None] * (self.SLOTS // self.BLOCK)
        self.next = 0

    def upload(self, flat, lib, stream_ptr):
        """-> device address of the uploaded ints, or 0 when they do not fit a slot."""
        n = len(flat)
        if n > self.SLOT_INTS:
            return 0
        i = self.next
        self.next = (i + 1) % self.SLOTS
        blk = i // self.BLOCK
        if i % self.BLOCK == 0 and self.events[blk] is not None:
            self.events[blk].synchronize()
        lo = i * self.SLOT_INTS
        self.np[lo: lo + n] = flat
        rc = lib.gnf4b_upload_i32(self.host_ptr + lo * 4, self.dev_ptr + lo * 4, n, stream_ptr)
        if rc:
            _gnf4b.check(rc, "gnf4b_upload_i32")
        if i % self.BLOCK == self.BLOCK - 1:
            if self.events[blk] is None:
                self.events[blk] = torch.cuda.Event()
            self.events[blk].record()
        return self.dev_ptr + lo * 4


_RINGS: dict = {}          # (device index, stream) -> _IndexRing, most recently used last
_RINGS_MAX = 8             # 1 MiB pinned + 1 MiB device each: a process that cycles through streams keeps only these


def _index_ring(dev, stream_ptr):
    key = (dev.index, stream_ptr)
    r = _RINGS.pop(key, None)
    if r is None:
        while len(_RINGS) >= _RINGS_MAX:
            # retire the least recently used ring once nothing can still read it
            old = _RINGS.pop(next(iter(_RINGS)))
            with torch.cuda.device(old.dev.device):
                torch.cuda.synchronize()
        r = _IndexRing(dev)
    _RINGS[key] = r
    return r


def _flat_ints(seqs):
    flat = []
    for s in seqs:
        if torch.is_tensor(s):
            flat.extend(int(v) for v in s.reshape(-1).tolist())
        else:
            flat.extend(int(v) for v in s)
    return flat


def to_device_i32(seqs, device):
    """Small host integer sequences -> one int32 device view per input, identical values
    on every path, in ONE transfer (ref :229-331).  Under CUDA-graph capture the source is
    a permanent slice of the pinned arena and the copy is asynchronous (a pageable build
    synchronises, which is illegal in a capture); otherwise a recycled pinned slot."""
    lens = [len(s) for s in seqs]
    total = sum(lens)
    dev = torch.device(device)
    if total == 0:
        return [torch.empty(0, dtype=torch.int32, device=dev) for _ in seqs]
    if dev.type != "cuda" or not torch.cuda.is_available():
        packed = torch.tensor(_flat_ints(seqs), dtype=torch.int32, device=dev)
    else:
        ar = _arena(dev)
        flat = _flat_ints(seqs)
        if ar._capturing():
            host, _ = ar.take(total)
            host.copy_(torch.tensor(flat, dtype=torch.int32))
            packed = host.to(dev, non_blocking=True)
        else:
            host, slot = ar.stage(total)
            if host is None:
                packed = torch.tensor(flat, dtype=torch.int32).to(dev)
            else:
                lo = slot * ar.RING_SLOT_INTS
                ar._ring_np[lo: lo + total] = flat
                packed = host.to(dev, non_blocking=True)
                ar.staged(slot)
    out, o = [], 0
    for n in lens:
        out.append(packed[o:o + n])
        o += n
    return out


def build_group_tiles(sizes, block_m: int, device):
    """Jagged group sizes -> fixed-height M-tiles ``(row0, valid_rows, group)`` as three
    int32 tensors on ``device`` (ref :334-362).  The CUDA kernels here do not consume this
    table (they schedule from group offsets on the device); it stays for callers and tests
    that import it.  ``sizes`` is never modified, including when it is a tensor."""
    t_row0, t_rows, t_group = [], [], []
    row = 0
    for g, m in enumerate(sizes):
        m = int(m)
        for done in range(0, m, block_m):
            t_row0.append(row + done)
            t_rows.append(min(block_m, m - done))
            t_group.append(g)
        row += m
    a, b, c = to_device_i32((t_row0, t_rows, t_group), device)
    return a, b, c


# --------------------------------------------------------------------------- #
# planning helpers kept for API parity
# --------------------------------------------------------------------------- #
def _sm_count(device) -> int:
    key = str(device)
    if key not in _SM_CACHE:
        if torch.cuda.is_available() and "cuda" in key:
            _SM_CACHE[key] = torch.cuda.get_device_properties(device).multi_processor_count
        else:
            _SM_CACHE[key] = 64
    return _SM_CACHE[key]


def _decode_plan(N: int, K: int, T: int, sm_count: int):
    """The reference's decode launch plan ``(BLOCK_N, num_warps, split_k)`` (ref :609-632):
    constant (64, 2); split-K only for starved grids (programs < 2*SM), power of two up to
    8, each split owning at least SPLITK_MIN_BLOCKS absmax blocks.  Pure function, kept so
    integrations that consult it see the same answers; the sm_100a kernel plans for itself
    (``gnf4b_plan_split_k``)."""
    bn, warps = 64, 2
    programs = T * -(-N // bn)
    split_k = 1
    if programs < 2 * sm_count:
        want = -(-(4 * sm_count) // programs)
        while split_k < want and split_k < 8:
            split_k *= 2
        kblocks = max(K // BLOCKSIZE, 1)
        while split_k > 1 and kblocks // split_k < SPLITK_MIN_BLOCKS:
            split_k //= 2
    return bn, warps, split_k


def decode_dispatch(N: int, K: int, T: int, sm_count: int):
    """Product-layer hint (ref :635-649): ``("dequant",)`` below the fused-traffic floor,
    else ``("fused", BLOCK_N, num_warps, split_k)``.  The op itself always runs fused."""
    traffic = T * N * (K // 2 + K // 16)
    if traffic < DECODE_MIN_FUSED_BYTES:
        return ("dequant",)
    return ("fused", *_decode_plan(N, K, T, sm_count))


def _prefill_block_m(max_rows: int) -> int:
    """M-tile height rule of the reference (ref :686-694)."""
    for bm in (16, 32, 64):
        if max_rows <= bm:
            return bm
    return 128


def _lut(device):
    key = str(device)
    if key not in _LUT_CACHE:
        _LUT_CACHE[key] = torch.tensor(NF4_LUT, dtype=torch.float32, device=device)
    return _LUT_CACHE[key]


def repack_from_bnb(packed_list, states, N: int, K: int):
    """bitsandbytes per-expert ``quantize_4bit`` outputs -> ``B [E,N,K/2] u8`` and
    ``absmax [E,N,K/64] fp32`` (ref :74-96); nested statistics are de-nested here."""
    assert K % BLOCKSIZE == 0, f"K={K} not a multiple of blocksize {BLOCKSIZE}"
    E, dev = len(packed_list), packed_list[0].device
    B = torch.empty(E, N, K // 2, dtype=torch.uint8, device=dev)
    A = torch.empty(E, N, K // BLOCKSIZE, dtype=torch.float32, device=dev)
    for e, (q, st) in enumerate(zip(packed_list, states)):
        B[e] = q.reshape(N, K // 2)
        am = st.absmax
        if getattr(st, "nested", False):
            from bitsandbytes import functional as F
            am = F.dequantize_blockwise(st.absmax, st.state2) + st.offset
        A[e] = am.to(torch.float32).reshape(N, K // BLOCKSIZE)
    return B, A


def dequant_ref(packed_row_major: torch.Tensor, absmax: torch.Tensor, N: int, K: int):
    """Pure-torch element decode, any device: ``w = fp32(LUT[code]) * fp32(absmax)``, element
    2j in the HIGH nibble of byte j (ref :910-929).  The CPU-checkable counterpart of what
    the kernels decode in registers."""
    lut = _lut(packed_row_major.device)
    b = packed_row_major.reshape(-1).to(torch.int64)
    codes = torch.stack((b >> 4, b & 15), dim=1).reshape(-1)
    am = absmax.to(torch.float32).reshape(-1).repeat_interleave(BLOCKSIZE)
    return (lut[codes] * am).reshape(N, K)


# --------------------------------------------------------------------------- #
# launch plumbing shared with mxfp4_grouped
# --------------------------------------------------------------------------- #
_WS_BYTES = {}       # (device, fmt, op, T, G, N, K, max_rows, flags) -> scratch bytes the planner asks for
_STATUS_PTR = {}     # device index -> address of the status word


def _raw_stream(dev) -> int:
    """Address of torch's current stream on ``dev`` (the cheap accessor when this torch has it)."""
    get = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if get is not None and dev.index is not None:
        return get(dev.index)
    return torch.cuda.current_stream(dev).cuda_stream


def _status_ptr(dev) -> int:
    ptr = _STATUS_PTR.get(dev.index)
    if ptr is None:
        ptr = _status_word(dev).data_ptr()
        if dev.index is not None:
            _STATUS_PTR[dev.index] = ptr
    return ptr


def _status_word(dev):
    dev = torch.device(dev)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    key = str(dev)
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _STATUS[key]


def last_status(device) -> int:
    """OR of the GNF4B_ST_* bits kernels on ``device`` have raised since the last call of
    this function (synchronises).  0 = nothing skipped, no wait timed out."""
    w = _status_word(torch.device(device))
    v = int(w.item())
    if v:
        w.zero_()
    return v


def _group_tables(sizes, expert_ids, T: int, E: int, dev, group_offsets=None, max_rows=None, stream_ptr=0):
    """-> (group_offsets[G+1] dev, expert_ids[G] dev, G, max_rows); the first two are tensors,
    or plain device addresses on the eager host-list fast path.  Host inputs are checked and
    travel in one transfer; device inputs are used where they are, with no host read."""
    ids_dev = torch.is_tensor(expert_ids) and expert_ids.is_cuda
    if group_offsets is not None:
        # caller-built device prefix sum: nothing to transfer, nothing to read back
        if not (torch.is_tensor(group_offsets) and group_offsets.is_cuda and group_offsets.dtype == torch.int32):
            raise TypeError("group_offsets must be a CUDA int32 tensor of G+1 entries")
        G = int(group_offsets.numel()) - 1
        ids_t = (expert_ids.to(torch.int32).contiguous() if ids_dev
                 else to_device_i32(([int(v) for v in expert_ids],), dev)[0])
        if ids_t.numel() != G:
            raise ValueError(f"group_offsets has {G} groups but expert_ids has {ids_t.numel()}")
        return group_offsets.contiguous(), ids_t, G, int(max_rows) if max_rows else -1
    sz_dev = torch.is_tensor(sizes) and sizes.is_cuda
    if sz_dev:
        G = int(sizes.numel())
        max_rows = -1
    else:
        sz = [int(v) for v in (sizes.tolist() if torch.is_tensor(sizes) else sizes)]
        G = len(sz)
        assert sum(sz) == T, (sum(sz), T)
        if any(v < 0 for v in sz):
            raise ValueError("negative group size")
        max_rows = max(sz) if sz else 0
        offs = [0] * (G + 1)
        for i, v in enumerate(sz):
            offs[i + 1] = offs[i] + v
    if not ids_dev:
        ids = [int(v) for v in (expert_ids.tolist() if torch.is_tensor(expert_ids) else expert_ids)]
        if len(ids) != G:
            raise ValueError(f"sizes has {G} groups but expert_ids has {len(ids)}")
        if any((v < 0 and v != PAD_EXPERT) or v >= E for v in ids):
            raise ValueError(f"expert id out of range for a stack of {E} experts")
    else:
        if expert_ids.numel() != G:
            raise ValueError(f"sizes has {G} groups but expert_ids has {expert_ids.numel()}")
    if not sz_dev and not ids_dev:
        capturing = False
        try:
            capturing = torch.cuda.is_current_stream_capturing()
        except Exception:
            pass
        base = 0 if capturing else _index_ring(dev, stream_ptr).upload(offs + ids, _gnf4b.load(), stream_ptr)
        if base:
            return base, base + 4 * (G + 1), G, max_rows
        off_t, ids_t = to_device_i32((offs, ids), dev)
    elif not sz_dev:
        off_t = to_device_i32((offs,), dev)[0]
        ids_t = expert_ids.to(torch.int32).contiguous()
    else:
        lib = _gnf4b.load()
        sz_t = sizes.to(torch.int32).contiguous()
        off_t = torch.empty(G + 1, dtype=torch.int32, device=dev)
        _gnf4b.check(lib.gnf4b_build_offsets(sz_t.data_ptr(), G, off_t.data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream),
                     "gnf4b_build_offsets")
        ids_t = (expert_ids.to(torch.int32).contiguous() if ids_dev else to_device_i32((ids,), dev)[0])
    return off_t, ids_t, G, max_rows


def _launch(fmt, op, x, W, S, sizes, expert_ids, n_out, *, split_k=None, path=_gnf4b.PATH_AUTO,
            group_offsets=None, max_rows=None, tables_ready=None, x_glu: int = 0):
    """One grouped launch.  x [T, C] bf16/fp16, W [E, N, K/2] u8, S scales -> bf16 [T, n_out].
    ``x_glu`` (FLAG_X_SILU_GLU / FLAG_X_GPT_OSS_GLU): x is the gate_up output [T, 2K]; returns None when the
    library has no kernel that applies the activation on load for this problem."""
    dev = x.device
    E, N, half = W.shape
    K = half * 2
    T = x.shape[0]
    if x.dtype == torch.bfloat16:
        xdt = _gnf4b.X_BF16
    elif x.dtype == torch.float16:
        xdt = _gnf4b.X_FP16
    else:
        raise TypeError(f"activations must be bfloat16 or float16, got {x.dtype}")
    if W.dtype != torch.uint8:
        raise TypeError(f"packed weights must be uint8, got {W.dtype}")
    if W.device != dev or S.device != dev:
        raise ValueError("activations, packed weights and scales must live on the same device")
    if not x.is_contiguous():
        x = x.contiguous()
    if x.data_ptr() % 16:
        x = x.clone()
    if W.stride(2) != 1:
        W = W.contiguous()
    if fmt == _gnf4b.FMT_NF4:
        if S.dtype == torch.float32:
            sdt = _gnf4b.S_F32
        elif S.dtype == torch.bfloat16:
            sdt = _gnf4b.S_BF16
        else:
            S, sdt = S.to(torch.float32), _gnf4b.S_F32
    else:
        sdt = _gnf4b.S_E8M0
    if S.stride(2) != 1:
        S = S.contiguous()
    out = torch.empty(T, n_out, dtype=torch.bfloat16, device=dev)
    if T == 0:
        return out
    lib = _gnf4b.load()
    prev = -1
    if dev.index is not None and dev.index != torch.cuda.current_device():
        prev = torch.cuda.current_device()          # the C library launches on the current device
        torch.cuda.set_device(dev)
    try:
        stream_ptr = _raw_stream(dev)
        off_t, ids_t, G, max_rows = _group_tables(sizes, expert_ids, T, E, dev, group_offsets, max_rows, stream_ptr)
        if G == 0:
            return out
        off_p = off_t if isinstance(off_t, int) else off_t.data_ptr()
        ids_p = ids_t if isinstance(ids_t, int) else ids_t.data_ptr()
        flags = path | x_glu
        if split_k is not None:
            flags |= max(1, int(split_k)) << _gnf4b.SPLITK_SHIFT
        # Group tables that this call uploaded from host lists travel by a stream-ordered copy, which no kernel
        # overtakes: they are ready when the kernel starts.  Device tables may have been written by the kernel
        # launched just before (a router, a prefix sum): only the caller can say that they were not.
        if tables_ready is None:
            tables_ready = group_offsets is None and not (torch.is_tensor(sizes) and sizes.is_cuda) \
                and not (torch.is_tensor(expert_ids) and expert_ids.is_cuda)
        if tables_ready:
            flags |= _gnf4b.FLAG_TABLES_READY
        key = (dev.index, fmt, op, T, G, N, K, max_rows, flags)        # the plan depends on the device's SM count
        need = _WS_BYTES.get(key)
        if need is None:
            need = lib.gnf4b_workspace_bytes(*key[1:])
            if len(_WS_BYTES) < 4096:
                _WS_BYTES[key] = need
        ws = torch.zeros(need, dtype=torch.uint8, device=dev) if need else None
        rc = lib.gnf4b_gemm_grouped(
            fmt, op, x.data_ptr(), xdt, T, W.data_ptr(), W.stride(0), W.stride(1),
            S.data_ptr(), sdt, S.stride(0), S.stride(1), off_p, ids_p,
            G, E, N, K, max_rows, out.data_ptr(), ws.data_ptr() if ws is not None else None,
            need, _status_ptr(dev), flags, stream_ptr)
    finally:
        if prev >= 0:
            torch.cuda.set_device(prev)
    if rc == _gnf4b.EUNSUPPORTED and x_glu:
        return None
    if rc:
        _gnf4b.check(rc, "gnf4b_gemm_grouped")
    return out


def gemm_after_glu(fmt, gate_up, W, S, expert_ids, group_offsets, max_rows, act: str = "silu", path: int = 0):
    """The FFN's second GEMM on the OUTPUT of its first: ``gate_up [T, 2K]`` bf16 -> ``[T, N]``, the activation
    (``"silu"``: SiLU(gate_up[:, :K]) * gate_up[:, K:]; ``"gpt_oss"``: the clamped form on interleaved columns)
    applied inside the GEMM kernel while it loads its rows, where a kernel for that exists (small groups), else by
    the activation kernel first.  Same bits either way."""
    flag = _gnf4b.FLAG_X_SILU_GLU if act == "silu" else _gnf4b.FLAG_X_GPT_OSS_GLU
    out = None
    if max_rows and max_rows <= 16 and gate_up.dtype == torch.bfloat16:
        out = _launch(fmt, _gnf4b.OP_FWD, gate_up, W, S, None, expert_ids, W.shape[1], group_offsets=group_offsets,
                      max_rows=max_rows, x_glu=flag, path=path)
    if out is None:
        if act == "silu":
            import ep_moe
            h = ep_moe.silu_glu(gate_up)
        else:
            import mxfp4_grouped
            h = mxfp4_grouped.glu_gpt_oss(gate_up)
        out = _launch(fmt, _gnf4b.OP_FWD, h, W, S, None, expert_ids, W.shape[1], group_offsets=group_offsets,
                      max_rows=max_rows, path=path)
    return out


# --------------------------------------------------------------------------- #
# torch.library registration: the grouped GEMM as a custom operator with a fake (meta) kernel, so that callers that
# trace these entry points (torch.compile, torch.export) get one opaque node instead of a graph break
# --------------------------------------------------------------------------- #
try:
    from typing import List, Optional

    @torch.library.custom_op("gnf4b::grouped_gemm", mutates_args=())
    def _grouped_gemm_op(x: torch.Tensor, W: torch.Tensor, S: torch.Tensor, group_offsets: Optional[torch.Tensor],
                         expert_ids_t: Optional[torch.Tensor], sizes: Optional[List[int]], expert_ids: Optional[List[int]],
                         fmt: int, op: int, n_out: int, max_rows: int, path: int, split_k: int,
                         tables_ready: bool) -> torch.Tensor:
        return _launch(fmt, op, x, W, S, sizes, expert_ids_t if expert_ids_t is not None else expert_ids, n_out,
                       split_k=split_k if split_k > 0 else None, path=path, group_offsets=group_offsets,
                       max_rows=max_rows if max_rows > 0 else None, tables_ready=tables_ready)

    @_grouped_gemm_op.register_fake
    def _grouped_gemm_fake(x, W, S, group_offsets, expert_ids_t, sizes, expert_ids, fmt, op, n_out, max_rows, path,
                           split_k, tables_ready):
        return x.new_empty((x.shape[0], n_out), dtype=torch.bfloat16)

    _HAVE_OP = True
except Exception:      # an older torch without torch.library.custom_op: the plain functions still work
    _HAVE_OP = False


def _tracing() -> bool:
    try:
        return _HAVE_OP and torch.compiler.is_compiling()
    except Exception:
        return False


def _dispatch(fmt, op, x, W, S, sizes, expert_ids, n_out, *, split_k=None, path=_gnf4b.PATH_AUTO, group_offsets=None,
              max_rows=None, tables_ready=None):
    """_launch directly in eager mode (no dispatcher overhead on the decode path); through the registered operator
    ``torch.ops.gnf4b.grouped_gemm`` while a compiler is tracing."""
    if not _tracing():
        return _launch(fmt, op, x, W, S, sizes, expert_ids, n_out, split_k=split_k, path=path,
                       group_offsets=group_offsets, max_rows=max_rows, tables_ready=tables_ready)
    ids_t = expert_ids if torch.is_tensor(expert_ids) else None
    ids_l = None if ids_t is not None else [int(v) for v in expert_ids]
    if torch.is_tensor(sizes):
        sizes = None if group_offsets is not None else [int(v) for v in sizes.tolist()]
    elif sizes is not None:
        sizes = [int(v) for v in sizes]
    if tables_ready is None:
        tables_ready = group_offsets is None and ids_t is None
    return torch.ops.gnf4b.grouped_gemm(x, W, S, group_offsets, ids_t, sizes, ids_l, fmt, op, n_out,
                                        int(max_rows) if max_rows else 0, int(path), int(split_k) if split_k else 0,
                                        bool(tables_ready))


def _require_cuda(t, fn_name: str, hint: str):
    if t.device.type != "cuda":
        raise RuntimeError(
            f"{fn_name} runs the fused sm_100a CUDA kernel and requires CUDA tensors "
            f"(got device '{t.device.type}'). {hint}")


# --------------------------------------------------------------------------- #
# public entry points
# --------------------------------------------------------------------------- #
def gemm_4bit_grouped(a_cat, B, absmax, sizes, expert_ids, block_m: int | None = None,
                      decode_config: tuple | None = None, split_k: int | None = None,
                      prefill_config: tuple | None = None, prefill_variant: int | None = None,
                      prefill_groups: int = 1, *, group_offsets=None, max_rows=None, path: int = 0,
                      tables_ready: bool | None = None):
    """Single-launch grouped NF4 GEMM (ref :697-907).

    ``a_cat [T,K]`` bf16/fp16 rows sorted by group, ``B [E,N,K//2]`` uint8 (any expert / row
    stride, last dimension contiguous), ``absmax [E,N,K//64]`` fp32 or bf16, ``sizes`` the
    per-group row counts (host sequence, CPU or CUDA tensor; zero-size groups produce no
    rows), ``expert_ids [G]`` indices into the stack handed in (list, CPU or CUDA tensor).
    Returns ``[T,N]`` bf16 in the same row order.

    ``split_k`` forces the streaming kernel's split-K factor (None = planner, 1 = off).
    ``block_m``, ``decode_config``, ``prefill_config``, ``prefill_variant`` and
    ``prefill_groups`` are Triton launch knobs of the reference; they are accepted and
    ignored -- results do not depend on them.

    Additions (keyword only): ``group_offsets`` -- a CUDA int32 ``[G+1]`` exclusive prefix sum
    of the group sizes; when given, ``sizes`` is not read at all, nothing is copied to the
    device and the call never synchronises (routing can change under CUDA-graph replay).
    ``max_rows`` -- the largest group size if the caller knows it (a path hint only).
    ``path`` -- 0 planner, 1 streaming kernel, 2 tensor-core kernel (ablation).
    ``tables_ready`` -- True promises that device-side ``group_offsets`` / ``expert_ids`` / ``sizes`` were NOT
    written by the kernel launched just before this call on the stream; the decode kernel then starts
    streaming weights while that kernel still runs.  Default: true for host lists (they are uploaded by a
    stream-ordered copy), false for device tensors.
    """
    E, N, _ = B.shape
    T, K = a_cat.shape
    _require_cuda(a_cat, "gemm_4bit_grouped",
                  "For a CPU-checkable decode of the same NF4 bytes, use dequant_ref(packed, absmax, N, K) "
                  "-- the pure-torch reference the kernel is pinned against.")
    if B.shape[2] * 2 != K:
        raise ValueError(f"a_cat has K={K} but B packs K={B.shape[2] * 2}")
    if tuple(absmax.shape) != (E, N, K // BLOCKSIZE):
        raise ValueError(f"absmax shape {tuple(absmax.shape)} != {(E, N, K // BLOCKSIZE)}")
    return _dispatch(_gnf4b.FMT_NF4, _gnf4b.OP_FWD, a_cat, B, absmax, sizes, expert_ids, N, split_k=split_k,
                     group_offsets=group_offsets, max_rows=max_rows, path=path, tables_ready=tables_ready)


def dgrad_eligible(grad_out, B, absmax, block_k: int = 64):
    """None if ``dgrad_4bit_grouped`` can take this problem, else the reason (ref :1034-1053; restated
    from there, message strings included, plus one rule of this kernel: N % 8 == 0)."""
    if grad_out.dtype != torch.bfloat16:
        return f"grad_out dtype {grad_out.dtype} is not bfloat16"
    if BLOCKSIZE % block_k:
        return f"BLOCK_K {block_k} does not divide the quant blocksize {BLOCKSIZE}"
    K = B.shape[2] * 2
    if K % block_k:
        return f"K {K} not divisible by BLOCK_K {block_k}"
    if absmax.shape[2] * BLOCKSIZE != K:
        return f"absmax blocks {absmax.shape[2]} do not tile K {K} at blocksize {BLOCKSIZE}"
    if B.numel() == 0:
        return "packed storage is empty (evicted?)"
    if B.shape[1] % 8:
        # not a rule of the reference: the sm_100a kernel fetches grad_out [T, N] by TMA, whose row
        # pitch (2 N bytes) must be a multiple of 16 bytes
        return f"N {B.shape[1]} is not a multiple of 8 (grad_out rows are fetched by TMA: 16-byte row pitch)"
    return None


def dgrad_4bit_grouped(grad_out, B, absmax, sizes, expert_ids, config=None, *, group_offsets=None,
                       max_rows=None):
    """``grad_a[t,:] = grad_out[t,:] @ dequant_nf4(B[e(t)])`` in one launch (ref :1056-1121).

    ``grad_out [T,N]`` bf16, same stack and grouping as the forward; returns ``[T,K]`` bf16.
    ``config`` (a Triton tile tuple in the reference) only takes part in the eligibility
    check; the result does not depend on it."""
    E, N, half = B.shape
    K = half * 2
    T = grad_out.shape[0]
    _require_cuda(grad_out, "dgrad_4bit_grouped",
                  "The CPU-checkable equivalent is grad_out @ dequant_ref(packed, absmax, N, K) per group.")
    block_k = (config or _DGRAD_DEFAULT)[2]
    why = dgrad_eligible(grad_out, B, absmax, block_k)
    if why is not None:
        raise ValueError(
            f"dgrad_4bit_grouped cannot run this problem: {why}. Callers that can fall back should "
            "check dgrad_eligible() first rather than catching this.")
    if grad_out.shape[1] != N:
        raise ValueError(f"grad_out has {grad_out.shape[1]} columns but the stack has N={N}")
    return _dispatch(_gnf4b.FMT_NF4, _gnf4b.OP_DGRAD, grad_out, B, absmax, sizes, expert_ids, K,
                     group_offsets=group_offsets, max_rows=max_rows)


# --------------------------------------------------------------------------- #
# expert FFN on CUDA tensors: gate_up GEMM -> activation -> down GEMM
# --------------------------------------------------------------------------- #
_FFN_WS = {}          # (device index, stream) -> zero-initialised uint8 workspace, grown on demand


def _launch_ffn(fmt, act, x, W_gu, S_gu, W_dn, S_dn, sizes, expert_ids, *, bias_gu=None, group_offsets=None,
                max_rows=None, tables_ready=None, fused=True):
    """One expert FFN per row, ``gnf4b_ffn_grouped``: a single fused launch for one-row groups, three launches
    otherwise.  ``x [T, K]`` bf16 -> bf16 ``[T, N_dn]``."""
    dev = x.device
    if x.dtype != torch.bfloat16:
        raise TypeError(f"activations must be bfloat16, got {x.dtype}")
    E, N_gu, half = W_gu.shape
    K_gu = half * 2
    N_dn = W_dn.shape[1]
    T = x.shape[0]
    if x.shape[1] != K_gu:
        raise ValueError(f"activations have {x.shape[1]} columns, the gate_up stack contracts over {K_gu}")
    if W_dn.shape[0] != E or N_gu % 2 or W_dn.shape[2] * 2 != N_gu // 2:
        raise ValueError(f"down stack {tuple(W_dn.shape)} does not follow gate_up {tuple(W_gu.shape)}")
    for t in (W_gu, S_gu, W_dn, S_dn):
        if t.device != dev:
            raise ValueError("activations, packed weights and scales must live on the same device")
    if not x.is_contiguous() or x.data_ptr() % 16:
        x = x.contiguous().clone() if x.data_ptr() % 16 else x.contiguous()
    if W_gu.stride(2) != 1:
        W_gu = W_gu.contiguous()
    if W_dn.stride(2) != 1:
        W_dn = W_dn.contiguous()
    if fmt == _gnf4b.FMT_NF4:
        if S_gu.dtype != S_dn.dtype or S_gu.dtype not in (torch.float32, torch.bfloat16):
            S_gu, S_dn = S_gu.to(torch.float32), S_dn.to(torch.float32)
        sdt = _gnf4b.S_F32 if S_gu.dtype == torch.float32 else _gnf4b.S_BF16
    else:
        sdt = _gnf4b.S_E8M0
    if S_gu.stride(2) != 1:
        S_gu = S_gu.contiguous()
    if S_dn.stride(2) != 1:
        S_dn = S_dn.contiguous()
    if bias_gu is not None:
        if bias_gu.dtype != torch.bfloat16 or tuple(bias_gu.shape) != (E, N_gu) or bias_gu.device != dev:
            raise ValueError(f"bias_gu must be a bfloat16 tensor of shape ({E}, {N_gu}) on {dev}")
        bias_gu = bias_gu.contiguous()
    out = torch.empty(T, N_dn, dtype=torch.bfloat16, device=dev)
    if T == 0:
        return out
    lib = _gnf4b.load()
    prev = -1
    if dev.index is not None and dev.index != torch.cuda.current_device():
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        stream_ptr = _raw_stream(dev)
        off_t, ids_t, G, max_rows = _group_tables(sizes, expert_ids, T, E, dev, group_offsets, max_rows, stream_ptr)
        if G == 0:
            return out
        off_p = off_t if isinstance(off_t, int) else off_t.data_ptr()
        ids_p = ids_t if isinstance(ids_t, int) else ids_t.data_ptr()
        flags = 0 if fused else _gnf4b.FLAG_FFN_UNFUSED
        if tables_ready is None:
            tables_ready = group_offsets is None and not (torch.is_tensor(sizes) and sizes.is_cuda) \
                and not (torch.is_tensor(expert_ids) and expert_ids.is_cuda)
        if tables_ready:
            flags |= _gnf4b.FLAG_TABLES_READY
        need = lib.gnf4b_ffn_workspace_bytes(fmt, T, G, N_gu, K_gu, N_dn, max_rows, flags)
        key = (dev.index, stream_ptr)
        ws = _FFN_WS.get(key)
        if ws is None or ws.numel() < need:
            # zero-filled once: the kernels leave the counters in it zeroed after every call
            ws = _FFN_WS[key] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        rc = lib.gnf4b_ffn_grouped(
            fmt, act, x.data_ptr(), _gnf4b.X_BF16, T, W_gu.data_ptr(), W_gu.stride(0), W_gu.stride(1),
            S_gu.data_ptr(), S_gu.stride(0), S_gu.stride(1), W_dn.data_ptr(), W_dn.stride(0), W_dn.stride(1),
            S_dn.data_ptr(), S_dn.stride(0), S_dn.stride(1), sdt, bias_gu.data_ptr() if bias_gu is not None else None,
            off_p, ids_p, G, E, N_gu, K_gu, N_dn, max_rows, out.data_ptr(), ws.data_ptr(), ws.numel(),
            _status_ptr(dev), flags, stream_ptr)
    finally:
        if prev >= 0:
            torch.cuda.set_device(prev)
    if rc:
        _gnf4b.check(rc, "gnf4b_ffn_grouped")
    return out


def ffn_4bit_grouped(a_cat, B_gu, absmax_gu, B_dn, absmax_dn, sizes, expert_ids, *, group_offsets=None, max_rows=None,
                     tables_ready: bool | None = None, fused: bool = True):
    """One NF4 expert FFN per row on CUDA tensors: ``(silu(gate) * up) @ W_dn[e].T`` with ``[gate | up] = a @ W_gu[e].T``
    -- the GPU counterpart of the reference's fused CPU FFN (``gnf4_native/cpu_kernels.c:763-986``).  For batch-1
    decode (every group one row) it is ONE kernel launch; larger groups run as gate_up GEMM, GLU kernel, down GEMM.
    Bit for bit ``gemm_4bit_grouped -> silu_glu -> gemm_4bit_grouped``.  ``fused=False`` forces the three launches."""
    _require_cuda(a_cat, "ffn_4bit_grouped", "The CPU-checkable equivalent composes dequant_ref per expert.")
    return _launch_ffn(_gnf4b.FMT_NF4, _gnf4b.ACT_SILU_GLU, a_cat, B_gu, absmax_gu, B_dn, absmax_dn, sizes, expert_ids,
                       group_offsets=group_offsets, max_rows=max_rows, tables_ready=tables_ready, fused=fused)


# --------------------------------------------------------------------------- #
# host-buffer entry points (activations, group tables and result in host memory)
# --------------------------------------------------------------------------- #
_HOST_STAGING = {}    # (device index, thread id) -> uint8 CUDA tensor, grown on demand (a call blocks, so one
                      # block per calling thread is enough and two threads never share one)
_HOST_NEED = {}       # (device, fmt, op, T, G, N, K, flags) -> staging bytes


def _host_i32(v, what):
    """-> (address, count, keep-alive) of a host int32 array."""
    if torch.is_tensor(v):
        if v.is_cuda:
            raise ValueError(f"{what} must live in host memory for the host-buffer entry points")
        if v.dtype != torch.int32 or not v.is_contiguous():
            v = v.to(torch.int32).contiguous()
        return v.data_ptr(), int(v.numel()), v
    arr = (ctypes.c_int32 * len(v))(*[int(i) for i in v])
    return ctypes.addressof(arr), len(v), arr


def _launch_host(fmt, op, x, W, S, sizes, expert_ids, n_out, out=None, *, split_k=None, path=_gnf4b.PATH_AUTO,
                 return_status=False):
    """One blocking grouped GEMM with host ``x`` / ``sizes`` / ``expert_ids`` / result and a device-resident
    stack: the library call ``gnf4b_gemm_grouped_host`` (tables and small ``x`` in one copy, launch, result
    copy, stream synchronise)."""
    if x.is_cuda:
        raise ValueError("the host-buffer entry points take host activations; use the plain entry points for CUDA tensors")
    dev = W.device
    if dev.type != "cuda" or S.device != dev:
        raise ValueError("the packed stack and its scales must be CUDA tensors on one device")
    if x.dtype == torch.bfloat16:
        xdt = _gnf4b.X_BF16
    elif x.dtype == torch.float16:
        xdt = _gnf4b.X_FP16
    else:
        raise TypeError(f"activations must be bfloat16 or float16, got {x.dtype}")
    if W.dtype != torch.uint8:
        raise TypeError(f"packed weights must be uint8, got {W.dtype}")
    E, N, half = W.shape
    K = half * 2
    T = x.shape[0]
    if x.shape[1] != (K if op == _gnf4b.OP_FWD else N):
        raise ValueError(f"activations have {x.shape[1]} columns, the stack wants {K if op == _gnf4b.OP_FWD else N}")
    if not x.is_contiguous():
        x = x.contiguous()
    if W.stride(2) != 1:
        W = W.contiguous()
    if fmt == _gnf4b.FMT_NF4:
        if S.dtype == torch.float32:
            sdt = _gnf4b.S_F32
        elif S.dtype == torch.bfloat16:
            sdt = _gnf4b.S_BF16
        else:
            S, sdt = S.to(torch.float32), _gnf4b.S_F32
    else:
        sdt = _gnf4b.S_E8M0
    if S.stride(2) != 1:
        S = S.contiguous()
    if out is None:
        out = torch.empty(T, n_out, dtype=torch.bfloat16, pin_memory=True)
    elif out.is_cuda or out.dtype != torch.bfloat16 or tuple(out.shape) != (T, n_out) or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous host bfloat16 tensor of shape ({T}, {n_out})")
    sz_p, G, sz_keep = _host_i32(sizes, "sizes")
    id_p, n_ids, id_keep = _host_i32(expert_ids, "expert_ids")
    if n_ids != G:
        raise ValueError(f"sizes has {G} groups but expert_ids has {n_ids}")
    if T == 0 or G == 0:
        if T:
            raise ValueError("rows without groups")
        return (out, 0) if return_status else out
    flags = path
    if split_k is not None:
        flags |= max(1, int(split_k)) << _gnf4b.SPLITK_SHIFT
    lib = _gnf4b.load()
    prev = -1
    if dev.index is not None and dev.index != torch.cuda.current_device():
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        key = (dev.index, fmt, op, T, G, N, K, flags)
        need = _HOST_NEED.get(key)
        if need is None:
            need = lib.gnf4b_host_staging_bytes(*key[1:])
            if len(_HOST_NEED) < 4096:
                _HOST_NEED[key] = need
        stage = _HOST_STAGING.get((dev.index, threading.get_ident()))
        if stage is None or stage.numel() < need:
            stage = _HOST_STAGING[(dev.index, threading.get_ident())] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        status = ctypes.c_int32(0) if return_status else None
        rc = lib.gnf4b_gemm_grouped_host(
            fmt, op, x.data_ptr(), xdt, T, W.data_ptr(), W.stride(0), W.stride(1),
            S.data_ptr(), sdt, S.stride(0), S.stride(1), sz_p, id_p, G, E, N, K,
            out.data_ptr(), stage.data_ptr(), stage.numel(),
            ctypes.addressof(status) if return_status else None, flags, _raw_stream(dev))
    finally:
        if prev >= 0:
            torch.cuda.set_device(prev)
    if rc == -1:      # GNF4B_EINVAL
        raise ValueError("gnf4b_gemm_grouped_host rejected the group tables: sizes must be >= 0 and sum to the "
                         f"number of rows ({T}), expert ids must lie in [0, {E}) or be PAD_EXPERT")
    if rc:
        _gnf4b.check(rc, "gnf4b_gemm_grouped_host")
    del sz_keep, id_keep
    return (out, int(status.value)) if return_status else out


class HostGroupedGemm:
    """The host-buffer grouped GEMM bound to one device-resident stack, for a loop that calls it every step:
    the stack is checked and its addresses and strides are read once, a call checks only what changes
    (activations, group tables, result buffer).

        run = HostGroupedGemm(B, absmax)                     # NF4 forward; fmt="mxfp4", op="dgrad" select the others
        out = run(a_host, sizes_i32, expert_ids_i32, out_host)

    ``a_host`` contiguous host bf16/fp16 ``[T, K]``; ``sizes_i32`` / ``expert_ids_i32`` contiguous host int32
    tensors of the same length; ``out_host`` contiguous host bf16 ``[T, N]``.  Same results as
    ``gemm_4bit_grouped_host`` (it is the same library call)."""

    def __init__(self, packed, scales, fmt: str = "nf4", op: str = "fwd", path: int = 0):
        if fmt not in ("nf4", "mxfp4") or op not in ("fwd", "dgrad"):
            raise ValueError("fmt is 'nf4' or 'mxfp4', op is 'fwd' or 'dgrad'")
        dev = packed.device
        if dev.type != "cuda" or scales.device != dev:
            raise ValueError("the packed stack and its scales must be CUDA tensors on one device")
        if packed.dtype != torch.uint8:
            raise TypeError(f"packed weights must be uint8, got {packed.dtype}")
        if packed.stride(2) != 1:
            packed = packed.contiguous()
        self.fmt = _gnf4b.FMT_NF4 if fmt == "nf4" else _gnf4b.FMT_MXFP4
        self.op = _gnf4b.OP_FWD if op == "fwd" else _gnf4b.OP_DGRAD
        if fmt == "nf4":
            if scales.dtype not in (torch.float32, torch.bfloat16):
                scales = scales.to(torch.float32)
            self.sdt = _gnf4b.S_F32 if scales.dtype == torch.float32 else _gnf4b.S_BF16
        else:
            if scales.dtype != torch.uint8:
                raise TypeError("MXFP4 scales are e8m0 bytes (uint8)")
            self.sdt = _gnf4b.S_E8M0
        if scales.stride(2) != 1:
            scales = scales.contiguous()
        self.W, self.S, self.dev, self.flags = packed, scales, dev, int(path)      # keeps the stack alive
        self.E, self.N, self.K = packed.shape[0], packed.shape[1], packed.shape[2] * 2
        self.cols_in = self.K if op == "fwd" else self.N
        self.cols_out = self.N if op == "fwd" else self.K
        self._w = (packed.data_ptr(), packed.stride(0), packed.stride(1))
        self._s = (scales.data_ptr(), self.sdt, scales.stride(0), scales.stride(1))
        self._lib = _gnf4b.load()
        self._need = {}

    def __call__(self, x, sizes_i32, ids_i32, out):
        T = x.shape[0]
        G = sizes_i32.numel()
        if (x.dtype is not torch.bfloat16 and x.dtype is not torch.float16) or x.shape[1] != self.cols_in \
                or x.is_cuda or not x.is_contiguous():
            raise ValueError(f"activations must be a contiguous host bf16/fp16 tensor with {self.cols_in} columns")
        if sizes_i32.dtype is not torch.int32 or ids_i32.dtype is not torch.int32 or ids_i32.numel() != G \
                or sizes_i32.is_cuda or ids_i32.is_cuda:
            raise ValueError("sizes and expert ids must be host int32 tensors of the same length")
        if out.dtype is not torch.bfloat16 or out.shape[0] != T or out.shape[1] != self.cols_out or out.is_cuda \
                or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous host bfloat16 tensor of shape ({T}, {self.cols_out})")
        if T == 0 or G == 0:
            return out
        dev = self.dev
        if dev.index != torch.cuda.current_device():
            with torch.cuda.device(dev):
                return self(x, sizes_i32, ids_i32, out)
        need = self._need.get((T, G))
        if need is None:
            need = self._lib.gnf4b_host_staging_bytes(self.fmt, self.op, T, G, self.N, self.K, self.flags)
            if len(self._need) < 4096:
                self._need[(T, G)] = need
        stage = _HOST_STAGING.get((dev.index, threading.get_ident()))
        if stage is None or stage.numel() < need:
            stage = _HOST_STAGING[(dev.index, threading.get_ident())] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        rc = self._lib.gnf4b_gemm_grouped_host(
            self.fmt, self.op, x.data_ptr(), _gnf4b.X_BF16 if x.dtype is torch.bfloat16 else _gnf4b.X_FP16, T,
            *self._w, *self._s, sizes_i32.data_ptr(), ids_i32.data_ptr(), G, self.E, self.N, self.K,
            out.data_ptr(), stage.data_ptr(), stage.numel(), None, self.flags, _raw_stream(dev))
        if rc == -1:      # GNF4B_EINVAL
            raise ValueError("gnf4b_gemm_grouped_host rejected the group tables: sizes must be >= 0 and sum to the "
                             f"number of rows ({T}), expert ids must lie in [0, {self.E}) or be PAD_EXPERT")
        if rc:
            _gnf4b.check(rc, "gnf4b_gemm_grouped_host")
        return out


class HostGroupedFfn:
    """One expert FFN per row with host buffers, bound to a device-resident gate_up / down pair:
    ``out = (silu(gate) * up) @ W_dn[e].T`` with ``[gate | up] = x @ W_gu[e].T`` -- the GPU counterpart of the
    reference's fused CPU entry point (``gnf4_native/cpu_kernels.c:947-986``).  One upload, gate_up GEMM,
    SiLU-GLU kernel, down GEMM, one download, one synchronise (``gnf4b_ffn_grouped_host``); the ``[T, 2H]``
    intermediate stays on the device.  Bit for bit what ``gemm -> ep_moe.silu_glu -> gemm`` gives.

        ffn = HostGroupedFfn(B_gu, absmax_gu, B_dn, absmax_dn)            # fmt="mxfp4" for MXFP4 stacks
        out = ffn(a_host, sizes_i32, expert_ids_i32, out_host)            # bf16 [T, N_dn]
    """

    def __init__(self, packed_gu, scales_gu, packed_dn, scales_dn, fmt: str = "nf4", path: int = 0):
        gu = HostGroupedGemm(packed_gu, scales_gu, fmt=fmt, path=path)
        dn = HostGroupedGemm(packed_dn, scales_dn, fmt=fmt, path=path)
        if gu.dev != dn.dev or gu.E != dn.E or gu.sdt != dn.sdt:
            raise ValueError("gate_up and down stacks must share device, expert count and scale dtype")
        if gu.N % 2 or dn.K != gu.N // 2:
            raise ValueError(f"down contracts over {dn.K} columns but gate_up yields 2 x {gu.N // 2}")
        self.gu, self.dn, self.dev, self.flags = gu, dn, gu.dev, int(path)
        self._lib = gu._lib
        self._need = {}

    def __call__(self, x, sizes_i32, ids_i32, out):
        gu, dn = self.gu, self.dn
        T, G = x.shape[0], sizes_i32.numel()
        if x.dtype is not torch.bfloat16 or x.shape[1] != gu.K or x.is_cuda or not x.is_contiguous():
            raise ValueError(f"activations must be a contiguous host bfloat16 tensor with {gu.K} columns")
        if sizes_i32.dtype is not torch.int32 or ids_i32.dtype is not torch.int32 or ids_i32.numel() != G \
                or sizes_i32.is_cuda or ids_i32.is_cuda:
            raise ValueError("sizes and expert ids must be host int32 tensors of the same length")
        if out.dtype is not torch.bfloat16 or out.shape[0] != T or out.shape[1] != dn.N or out.is_cuda \
                or not out.is_contiguous():
            raise ValueError(f"out must be a contiguous host bfloat16 tensor of shape ({T}, {dn.N})")
        if T == 0 or G == 0:
            return out
        dev = self.dev
        if dev.index != torch.cuda.current_device():
            with torch.cuda.device(dev):
                return self(x, sizes_i32, ids_i32, out)
        need = self._need.get((T, G))
        if need is None:
            need = self._lib.gnf4b_ffn_host_staging_bytes(gu.fmt, T, G, gu.N, gu.K, dn.N, self.flags)
            if len(self._need) < 4096:
                self._need[(T, G)] = need
        stage = _HOST_STAGING.get((dev.index, threading.get_ident()))
        if stage is None or stage.numel() < need:
            stage = _HOST_STAGING[(dev.index, threading.get_ident())] = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
        rc = self._lib.gnf4b_ffn_grouped_host(
            gu.fmt, x.data_ptr(), _gnf4b.X_BF16, T, *gu._w, gu._s[0], gu._s[2], gu._s[3],
            *dn._w, dn._s[0], dn._s[2], dn._s[3], gu.sdt, sizes_i32.data_ptr(), ids_i32.data_ptr(), G, gu.E,
            gu.N, gu.K, dn.N, out.data_ptr(), stage.data_ptr(), stage.numel(), None, self.flags, _raw_stream(dev))
        if rc == -1:      # GNF4B_EINVAL
            raise ValueError("gnf4b_ffn_grouped_host rejected the group tables: sizes must be >= 0 and sum to the "
                             f"number of rows ({T}), expert ids must lie in [0, {gu.E}) or be PAD_EXPERT")
        if rc:
            _gnf4b.check(rc, "gnf4b_ffn_grouped_host")
        return out


def ffn_4bit_grouped_host(a_host, B_gu, absmax_gu, B_dn, absmax_dn, sizes, expert_ids, out=None):
    """One-shot form of ``HostGroupedFfn`` for NF4 stacks: ``sizes`` / ``expert_ids`` may be sequences, ``out``
    is allocated (pinned) when absent."""
    ffn = HostGroupedFfn(B_gu, absmax_gu, B_dn, absmax_dn)
    sizes = torch.as_tensor(sizes, dtype=torch.int32).contiguous()
    expert_ids = torch.as_tensor(expert_ids, dtype=torch.int32).contiguous()
    if out is None:
        out = torch.empty(a_host.shape[0], ffn.dn.N, dtype=torch.bfloat16, pin_memory=True)
    return ffn(a_host.contiguous(), sizes, expert_ids, out)


def gemm_4bit_grouped_host(a_host, B, absmax, sizes, expert_ids, out=None, *, split_k=None, path: int = 0,
                           return_status: bool = False):
    """``gemm_4bit_grouped`` for a caller that holds activations and routing in HOST memory and wants the
    result there -- the calling convention of the reference's native CPU kernels
    (``gnf4_native/cpu_kernels.c:751``, driven from ``kernel/cpu_grouped.py:272``), with the packed stack
    ``B [E,N,K//2]`` / ``absmax`` resident on the GPU.  ``a_host [T,K]`` bf16/fp16 (pinned memory avoids a
    staging copy), ``sizes`` / ``expert_ids`` host int32 tensors or sequences, ``out`` an optional host bf16
    ``[T,N]`` to fill (a pinned tensor is allocated when absent: reuse one across calls).  Blocks until the
    result is in ``out``.  ``return_status=True`` also returns this call's ``GNF4B_ST_*`` bits."""
    return _launch_host(_gnf4b.FMT_NF4, _gnf4b.OP_FWD, a_host, B, absmax, sizes, expert_ids, B.shape[1], out,
                        split_k=split_k, path=path, return_status=return_status)


def dgrad_4bit_grouped_host(grad_host, B, absmax, sizes, expert_ids, out=None, *, return_status: bool = False):
    """``dgrad_4bit_grouped`` with host gradients in, host input-gradients out
    (``gnf4_native/cpu_kernels.c:1374``)."""
    return _launch_host(_gnf4b.FMT_NF4, _gnf4b.OP_DGRAD, grad_host, B, absmax, sizes, expert_ids, B.shape[2] * 2,
                        out, return_status=return_status)


def dequant_stack_cuda(B, absmax):
    """Element decode of a whole stack by the CUDA library's own decode routines ->
    ``[E,N,K]`` fp32.  Exists so the kernels' decode can be compared bit for bit with
    ``dequant_ref``."""
    _require_cuda(B, "dequant_stack_cuda", "Use dequant_ref on CPU tensors.")
    E, N, half = B.shape
    if B.stride(2) != 1:
        B = B.contiguous()
    if absmax.dtype not in (torch.float32, torch.bfloat16):
        absmax = absmax.to(torch.float32)
    if absmax.stride(2) != 1:
        absmax = absmax.contiguous()
    sdt = _gnf4b.S_F32 if absmax.dtype == torch.float32 else _gnf4b.S_BF16
    out = torch.empty(E, N, half * 2, dtype=torch.float32, device=B.device)
    lib = _gnf4b.load()
    with torch.cuda.device(B.device):
        rc = lib.gnf4b_dequant(_gnf4b.FMT_NF4, B.data_ptr(), B.stride(0), B.stride(1), absmax.data_ptr(), sdt,
                               absmax.stride(0), absmax.stride(1), E, N, half * 2, out.data_ptr(),
                               torch.cuda.current_stream(B.device).cuda_stream)
    _gnf4b.check(rc, "gnf4b_dequant")
    return out
