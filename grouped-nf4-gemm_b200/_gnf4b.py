"""Loader for libgnf4b.so, the C-ABI CUDA library behind nf4_grouped / mxfp4_grouped.

This module replaces the reference project's ``kernel/_triton_shim.py`` and its
``backends/`` detect layer on the grouped-GEMM path: there is exactly one backend
(hand-written sm_100a CUDA), it is loaded lazily at the first launch, and a missing
library is a loud ``RuntimeError`` -- there is no CPU or eager fallback.

Importing this module needs neither a GPU nor the built library (the reference's
modules are importable on a CPU-only box too, ``kernel/_triton_shim.py:18-25``).
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess
import threading
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_PATH = HERE / "libgnf4b.so"
INCLUDE = HERE.parent / "include"

FMT_NF4, FMT_MXFP4 = 0, 1
OP_FWD, OP_DGRAD = 0, 1
X_BF16, X_FP16 = 0, 1
S_F32, S_BF16, S_E8M0 = 0, 1, 2
PATH_AUTO, PATH_STREAM, PATH_TENSOR = 0, 1, 2
SPLITK_SHIFT = 8
FLAG_CTA_PAIR = 0x20000           # forward tensor kernel as CTA pairs (cta_group::2) instead of single CTAs
FLAG_SMEM_OPERANDS = 0x10000      # ablation: forward on the kernel with both MMA operands in shared memory
FLAG_TABLES_READY = 0x40000       # the group tables were not written by the kernel launched just before
FLAG_X_SILU_GLU, FLAG_X_GPT_OSS_GLU = 0x200000, 0x400000   # x is the gate_up output; the GLU is applied on load
FLAG_SPARSE_GROUPS = 0x1000000    # most groups of the list are empty: deal out only the ones that exist
FLAG_HOST_COPIES = 0x800000       # ablation: host-buffer entries move small calls with the copy engines
FLAG_FFN_UNFUSED = 0x100000       # ablation: gnf4b_ffn_grouped as three launches even where it would fuse
ACT_SILU_GLU, ACT_GPT_OSS_GLU = 0, 1
FLAG_DECODE_ONE_ROW = 0x80000     # ablation: decode kernel with one weight row per warp in flight, not two
FLAG_DECODE_BF16_ROWS = 0x2000000  # ablation: decode kernel with two activation rows as bf16 pairs, not fp32
ST_BAD_EXPERT, ST_BAD_OFFSETS, ST_TIMEOUT = 1, 2, 4
EUNSUPPORTED, ETOOBIG = -5, -6
NOALLOC_SCRATCH_BYTES = 8 << 20

_lib = None
_lock = threading.Lock()

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile csrc/*.cu into libgnf4b.so next to this file (nvcc cross-compiles
    sm_100a without a GPU).  Rebuilds when any source is newer than the library."""
    newest = max(p.stat().st_mtime for p in sources())
    if not force and LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= newest:
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIB_PATH)] + [str(p) for p in sorted(CSRC.glob("*.cu"))]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    env = dict(os.environ)
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout[-3000:] + r.stderr[-3000:])
    if verbose:
        print(r.stderr)
    return LIB_PATH


def _declare(lib):
    i32, i64, u32, vp, sz = C.c_int32, C.c_int64, C.c_uint32, C.c_void_p, C.c_size_t
    lib.gnf4b_abi_version.restype = C.c_int
    lib.gnf4b_abi_version.argtypes = []
    lib.gnf4b_strerror.restype = C.c_char_p
    lib.gnf4b_strerror.argtypes = [C.c_int]
    lib.gnf4b_last_cuda_error.restype = C.c_char_p
    lib.gnf4b_last_cuda_error.argtypes = []
    lib.gnf4b_gemm_grouped.restype = C.c_int
    lib.gnf4b_gemm_grouped.argtypes = [
        C.c_int, C.c_int, vp, C.c_int, i64, vp, i64, i64, vp, C.c_int, i64, i64,
        vp, vp, i32, i32, i64, i64, i32, vp, vp, sz, vp, u32, vp]
    lib.gnf4b_gemm_grouped_noalloc.restype = C.c_int
    lib.gnf4b_gemm_grouped_noalloc.argtypes = [
        C.c_int, C.c_int, vp, C.c_int, i64, vp, i64, i64, vp, C.c_int, i64, i64,
        vp, vp, i32, i32, i64, i64, i32, vp, vp, u32, vp]
    lib.gnf4b_gemm_grouped_host.restype = C.c_int
    lib.gnf4b_gemm_grouped_host.argtypes = [
        C.c_int, C.c_int, vp, C.c_int, i64, vp, i64, i64, vp, C.c_int, i64, i64,
        vp, vp, i32, i32, i64, i64, vp, vp, sz, vp, u32, vp]
    lib.gnf4b_ffn_grouped_host.restype = C.c_int
    lib.gnf4b_ffn_grouped_host.argtypes = [
        C.c_int, vp, C.c_int, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64, C.c_int,
        vp, vp, i32, i32, i64, i64, i64, vp, vp, sz, vp, u32, vp]
    lib.gnf4b_ffn_grouped.restype = C.c_int
    lib.gnf4b_ffn_grouped.argtypes = [
        C.c_int, C.c_int, vp, C.c_int, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64, C.c_int,
        vp, vp, vp, i32, i32, i64, i64, i64, i32, vp, vp, sz, vp, u32, vp]
    lib.gnf4b_ffn_workspace_bytes.restype = sz
    lib.gnf4b_ffn_workspace_bytes.argtypes = [C.c_int, i64, i32, i64, i64, i64, i32, u32]
    lib.gnf4b_glu_gpt_oss.restype = C.c_int
    lib.gnf4b_glu_gpt_oss.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    lib.gnf4b_ffn_host_staging_bytes.restype = sz
    lib.gnf4b_ffn_host_staging_bytes.argtypes = [C.c_int, i64, i32, i64, i64, i64, u32]
    lib.gnf4b_host_staging_bytes.restype = sz
    lib.gnf4b_host_staging_bytes.argtypes = [C.c_int, C.c_int, i64, i32, i64, i64, u32]
    lib.gnf4b_workspace_bytes.restype = sz
    lib.gnf4b_workspace_bytes.argtypes = [C.c_int, C.c_int, i64, i32, i64, i64, i32, u32]
    lib.gnf4b_plan_split_k.restype = C.c_int
    lib.gnf4b_plan_split_k.argtypes = [C.c_int, C.c_int, i64, i32, i64, i64, i32, u32]
    lib.gnf4b_build_offsets.restype = C.c_int
    lib.gnf4b_build_offsets.argtypes = [vp, i32, vp, vp]
    lib.gnf4b_upload_i32.restype = C.c_int
    lib.gnf4b_upload_i32.argtypes = [vp, vp, i64, vp]
    lib.gnf4b_dequant.restype = C.c_int
    lib.gnf4b_dequant.argtypes = [C.c_int, vp, i64, i64, vp, C.c_int, i64, i64, i32, i64, i64, vp, vp]
    lib.gnf4b_silu_glu.restype = C.c_int
    lib.gnf4b_silu_glu.argtypes = [vp, i64, i64, vp, vp]
    lib.gnf4b_combine_rows.restype = C.c_int
    lib.gnf4b_combine_rows.argtypes = [vp, i64, vp, vp, i32, i64, i64, vp, vp, vp]
    lib.gnf4b_route_topk.restype = C.c_int
    lib.gnf4b_route_topk.argtypes = [vp, i64, i32, i32, i32, i32, vp, vp, vp]
    lib.gnf4b_ep_plan.restype = C.c_int
    lib.gnf4b_ep_plan.argtypes = [vp, i32, i32, i32, i32, i32, vp, i64, vp, vp, vp, vp, vp]
    lib.gnf4b_ep_offsets.restype = C.c_int
    lib.gnf4b_ep_offsets.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    lib.gnf4b_ep_peer_layout.restype = C.c_int
    lib.gnf4b_ep_peer_layout.argtypes = [i32, i32, i32, i64, vp]
    lib.gnf4b_ep_peer_dispatch.restype = C.c_int
    lib.gnf4b_ep_peer_dispatch.argtypes = [vp, vp, i32, i32, i32, i32, vp, vp, i32, vp, vp, vp, vp]
    lib.gnf4b_ep_peer_combine.restype = C.c_int
    lib.gnf4b_ep_peer_combine.argtypes = [vp, i32, vp, vp, vp, i32, i64, vp, vp, vp]
    lib.gnf4b_ep_plan_large_scratch_bytes.restype = sz
    lib.gnf4b_ep_plan_large_scratch_bytes.argtypes = [i64, i32]
    lib.gnf4b_ep_plan_large.restype = C.c_int
    lib.gnf4b_ep_plan_large.argtypes = [vp, i64, i32, i32, i32, i32, vp, i64, vp, vp, vp, vp, sz, vp, vp]
    lib.gnf4b_ep_push_blocks.restype = C.c_int
    lib.gnf4b_ep_push_blocks.argtypes = [i32, vp, vp, vp, vp, i32, i32, vp, vp]
    lib.gnf4b_ep_wait_flags.restype = C.c_int
    lib.gnf4b_ep_wait_flags.argtypes = [vp, i32, i32, i32, vp, vp]
    lib.gnf4b_gather_rows_by_id.restype = C.c_int
    lib.gnf4b_gather_rows_by_id.argtypes = [vp, i64, i32, vp, i32, vp, vp, vp, vp]
    lib.gnf4b_gather_rows_addr.restype = C.c_int
    lib.gnf4b_gather_rows_addr.argtypes = [vp, i64, i32, vp, vp, vp, i32, i64, vp]
    lib.gnf4b_device_info.restype = C.c_int
    lib.gnf4b_device_info.argtypes = [vp, vp]
    return lib


EP_MAX_WORLD = 16


class EpPeerCtx(C.Structure):
    """gnf4b_ep_peer_ctx of include/gnf4b.h."""
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("e_local", C.c_int32), ("cap_max", C.c_int32),
                ("H", C.c_int64), ("peers", C.c_void_p * EP_MAX_WORLD)]


#: every symbol include/gnf4b.h declares
EXPORTS = ("gnf4b_abi_version", "gnf4b_strerror", "gnf4b_last_cuda_error", "gnf4b_gemm_grouped",
           "gnf4b_gemm_grouped_noalloc", "gnf4b_gemm_grouped_host", "gnf4b_host_staging_bytes",
           "gnf4b_ffn_grouped_host", "gnf4b_ffn_host_staging_bytes", "gnf4b_ffn_grouped", "gnf4b_ffn_workspace_bytes",
           "gnf4b_glu_gpt_oss",
           "gnf4b_workspace_bytes", "gnf4b_plan_split_k", "gnf4b_build_offsets", "gnf4b_upload_i32", "gnf4b_dequant", "gnf4b_silu_glu", "gnf4b_combine_rows", "gnf4b_ep_plan", "gnf4b_ep_offsets", "gnf4b_route_topk",
           "gnf4b_ep_peer_layout", "gnf4b_ep_peer_dispatch", "gnf4b_ep_peer_combine",
           "gnf4b_gather_rows_by_id", "gnf4b_gather_rows_addr", "gnf4b_ep_plan_large", "gnf4b_ep_plan_large_scratch_bytes",
           "gnf4b_ep_push_blocks", "gnf4b_ep_wait_flags",
           "gnf4b_device_info")


def load():
    """The library handle.  Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not LIB_PATH.exists():
                    raise RuntimeError(
                        f"libgnf4b.so is not built ({LIB_PATH}). This package has a single backend, "
                        "hand-written sm_100a CUDA, and no CPU or eager fallback: run "
                        "`python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc) first.")
                _lib = _declare(C.CDLL(str(LIB_PATH)))
                if _lib.gnf4b_abi_version() != 1:
                    raise RuntimeError("libgnf4b.so ABI version mismatch; rebuild it")
    return _lib


def check(rc: int, what: str):
    if rc == 0:
        return
    lib = load()
    msg = lib.gnf4b_strerror(rc).decode()
    if rc == -4:
        msg += " -- " + lib.gnf4b_last_cuda_error().decode()
    if rc in (-1, -2, -6):
        raise ValueError(f"{what}: {msg} (rc={rc})")
    raise RuntimeError(f"{what}: {msg} (rc={rc})")
