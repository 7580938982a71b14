"""Source-level rules: every CTA loads its own tiles, sm_100a-only build,
and the library builds and loads without a GPU."""
import re
import shutil
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
CSRC = ROOT / "kernel_b200" / "csrc"


def _sources():
    return [p for p in CSRC.rglob("*") if p.suffix in {".cu", ".cuh", ".cpp", ".h"}]


def test_no_banned_load_qualifier_in_native_sources():
    # The qualifier that makes a TMA load deliver one tile to several CTAs must
    # not appear in any native source; it is spelled from pieces here so that
    # this file does not contain it either.
    needle = "." + "multi" + "cast" + "::" + "cluster"
    hits = [str(p) for p in _sources() if needle in p.read_text()]
    assert not hits, f"banned load qualifier named in {hits}"


def test_no_legacy_tensor_core_paths():
    pat = re.compile(r"wgmma|mma\.sync|wmma::")
    hits = [str(p) for p in _sources() if pat.search(p.read_text())]
    assert not hits


def test_gemm_kernel_uses_tcgen05_and_tma():
    text = (CSRC / "common" / "ptx.cuh").read_text()
    for token in ("tcgen05.mma", "tcgen05.alloc", "tcgen05.ld", "tcgen05.commit", "cp.async.bulk.tensor.2d"):
        assert token in text


def test_every_wait_is_bounded():
    text = (CSRC / "common" / "ptx.cuh").read_text()
    # the only spin loops live in the three bounded helpers (mbarrier, mbarrier with
    # cluster-scope acquire, flag), each of which takes a time limit
    assert text.count("while (") + text.count("for (;;)") == 3
    for helper in ("mbar_wait_bounded(", "mbar_wait_bounded_cluster(", "wait_flag_ge("):
        head = text[text.index("bool " + helper):]
        assert "limit_ns" in head[:head.index(")")]


@pytest.mark.skipif(shutil.which("nvcc") is None and not Path("/usr/local/cuda/bin/nvcc").exists(), reason="no nvcc")
def test_kernel_attributes_and_occupancy_are_cached_per_device():
    """A function attribute (dynamic shared memory above 48 KB) and an occupancy
    figure belong to a device's context.  A process may use several devices in its
    life, so a launcher that remembers them must remember them per device: no
    scalar "done once" flag next to ``cudaFuncSetAttribute`` or an occupancy query."""
    for p in _sources():
        text = p.read_text()
        if "cudaFuncSetAttribute" not in text and "cudaOccupancyMaxActiveBlocksPerMultiprocessor" not in text:
            continue
        scalars = re.findall(r"static\s+(?:bool|int|size_t)\s+(?:attr_set|cached_\w+|per_sm)\s*(?:=[^;\[]*)?;", text)
        assert not scalars, f"{p.name}: per-process cache of a per-device property: {scalars}"


def test_build_for_sm100a_and_load():
    from kernel_b200 import _native
    from kernel_b200.csrc import build

    assert "arch=compute_100a,code=sm_100a" in build.ARCH_FLAGS
    path = build.build()
    assert path.exists()
    lib = _native.lib()
    assert lib.kb_gemm_rs_data_bytes(8192, 8192, 8) == 2 * 8192 * 8192 * 2
    assert lib.kb_a2a_rows_bytes(8, 256, 8, 7168, 2) == 8 * 2048 * 7168 * 2
