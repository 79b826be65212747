"""Build recipe for the test oracle (TEST INFRASTRUCTURE, never the product).

Two artefacts:

* ``oracle/libgnf4_oracle.so`` -- the C restatement in ``gnf4_oracle.c``.
* ``oracle/_ref/cpu_kernels-<isa>.so`` -- the REFERENCE project's own CPU
  kernels, compiled from its source file where it lies (``gnf4_native/cpu_kernels.c``
  in the reference checkout, one self-contained C11 file, flags as in its
  ``gnf4_native/build.py:71-73`` except that ``-march=native`` is replaced by three
  fixed ISA levels so the binaries can run on a different host than the one that
  built them).  The reference picks its AVX-512 path at COMPILE time
  (``cpu_kernels.c:120-122, 759``), so one binary per ISA level is built and the
  loader picks by the running CPU's flags.  No reference source is copied into
  this repository; when the checkout is absent only the prebuilt files are used.

Run:  python oracle/build.py [--ref-root /path/to/reference]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
ORACLE_SO = HERE / "libgnf4_oracle.so"
# the reference checkout: GNF4_REFERENCE_ROOT, else a directory named `reference` beside this repository
DEFAULT_REF_ROOT = Path(os.environ.get("GNF4_REFERENCE_ROOT") or HERE.parent.parent / "reference")

# name -> -march level; the loader tries them best-first
REF_VARIANTS = (("avx512", "x86-64-v4"), ("avx2", "x86-64-v3"), ("base", "x86-64"))


def _cc() -> str:
    # The image's default CC lacks libgomp.spec; the system gcc has OpenMP.
    for cand in ("/usr/bin/gcc", os.environ.get("CC"), "gcc", "cc"):
        if cand and shutil.which(cand):
            return cand
    raise RuntimeError("no C compiler found")


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(map(str, cmd)), r.stderr[-2000:]))


def _stale(out: Path, src: Path) -> bool:
    return (not out.exists()) or out.stat().st_mtime < src.stat().st_mtime


def build_oracle(force: bool = False) -> Path:
    src = HERE / "gnf4_oracle.c"
    if force or _stale(ORACLE_SO, src):
        _run([_cc(), "-O2", "-ffp-contract=off", "-shared", "-fPIC",
              "-o", str(ORACLE_SO), str(src), "-lm"])
    return ORACLE_SO


def build_ref(ref_root: Path = DEFAULT_REF_ROOT, force: bool = False):
    """Compile the reference's cpu_kernels.c into oracle/_ref/.  Returns the list
    of built files, or [] when the reference checkout is not present."""
    src = ref_root / "gnf4_native" / "cpu_kernels.c"
    if not src.exists():
        return sorted(REF_DIR.glob("cpu_kernels-*.so"))
    REF_DIR.mkdir(exist_ok=True)
    built = []
    for name, march in REF_VARIANTS:
        out = REF_DIR / f"cpu_kernels-{name}.so"
        if force or _stale(out, src):
            _run([_cc(), "-O3", f"-march={march}", "-ffp-contract=off", "-shared",
                  "-fPIC", "-fopenmp", "-o", str(out), str(src), "-lm", "-lpthread"])
        built.append(out)
    return built


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=str(DEFAULT_REF_ROOT))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print("oracle:", build_oracle(a.force))
    refs = build_ref(Path(a.ref_root), a.force)
    print("reference CPU kernels:", [str(p) for p in refs] or "not built (no checkout)")


if __name__ == "__main__":
    sys.exit(main())
