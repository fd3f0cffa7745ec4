"""Rules the kernel sources keep, checked as text (no GPU needed).

* No source names a batched-memcpy runtime call or a cluster-wide TMA load: neither is safe to run on
  sm_100a with the driver generation this library targets, so the tree stays free of both, comments
  included.  (The words are assembled here so that this file does not name them.)
* Every kernel file that both receives shared-memory tiles from TMA and reads shared memory with ordinary
  loads carries the proxy fence that must precede the hand-back of such a tile."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
SOURCES = [p for pattern in ("*.cu", "*.cuh", "*.cpp", "*.h", "*.py") for p in ROOT.rglob(pattern)
           if not any(part in {"baseline", "build"} or part.endswith("_out") or part.startswith((".", "_"))
                      for part in p.relative_to(ROOT).parts[:-1])]

FORBIDDEN = ["multi" + "cast", "Memcpy" + "Batch", "Memcpy3D" + "Batch"]


def test_sources_were_found():
    assert any(p.suffix == ".cu" for p in SOURCES)


def test_no_source_names_a_closed_call():
    hits = [(str(p.relative_to(ROOT)), word) for p in SOURCES for word in FORBIDDEN
            if word.lower() in p.read_text(errors="replace").lower()]
    assert not hits, hits


def test_tma_fed_kernels_with_ordinary_readers_fence_before_release():
    csrc = ROOT / "katsu_b200" / "csrc"
    for path in sorted(csrc.glob("*.cu")):
        text = path.read_text()
        if re.search(r"\btma_load_\dd\(", text) and re.search(r"\bld_shared_(f32|v4)\(", text):
            assert "fence_proxy_async_smem();" in text, path.name
