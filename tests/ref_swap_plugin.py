"""pytest plugin for running the reference project's own test files against this package: loaded with
``-p ref_swap_plugin``, it imports this repository's modules under the names the reference's tests import
(``nf4_grouped``, ``mxfp4_grouped``, ``nf4_qlora``, ``nf4_pack_ref``, ``mxfp4_pack_ref``) before any test module
is collected, so that those imports resolve to the sm_100a implementation whatever the reference's conftest does to
``sys.path`` afterwards."""
import importlib
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parents[1] / "grouped-nf4-gemm_b200"
if str(PKG) not in sys.path:
    sys.path.insert(0, str(PKG))
SWAPPED = {}
for name in ("_gnf4b", "nf4_grouped", "mxfp4_grouped", "nf4_qlora", "nf4_pack_ref", "mxfp4_pack_ref"):
    SWAPPED[name] = importlib.import_module(name)


def pytest_report_header(config):
    return ["grouped-nf4-gemm_b200 swapped in for: " + ", ".join(f"{k} <- {Path(m.__file__).name}" for k, m in SWAPPED.items())]


def pytest_collection_finish(session):
    # the swap must have held: every module of those names still comes from this package
    for name, mod in SWAPPED.items():
        now = sys.modules.get(name)
        assert now is mod and str(PKG) in str(Path(now.__file__).resolve()), f"{name} was replaced by {now}"
