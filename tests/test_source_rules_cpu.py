"""Textual checks of the CUDA sources against the rules of ``docs/contributing.md`` that a compiler does not enforce:
no TMA or bulk load with cluster multicast, no device trap, no unbounded spin on an mbarrier or a peer flag, a register
budget assertion next to every ``setmaxnreg`` layout, and none of the batched copy calls that fault on this driver."""
import re
from pathlib import Path

CSRC = Path(__file__).resolve().parents[1] / "pithtrain_b200" / "csrc"
SOURCES = sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def _code(path: Path) -> str:
    """Source text without // and /* */ comments."""
    text = path.read_text()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def test_sources_exist():
    assert len(SOURCES) > 15


def test_no_load_with_cluster_multicast():
    for p in SOURCES:
        for m in re.finditer(r"multicast::cluster", p.read_text()):
            line = p.read_text()[:m.start()].count("\n") + 1
            stmt = p.read_text().splitlines()[line - 1]
            # the only form in use: tcgen05.commit arriving on barriers of both CTAs of a pair
            assert "tcgen05.commit" in stmt, f"{p.name}:{line}: {stmt.strip()}"


def test_no_device_trap_and_no_failing_device_assert():
    for p in SOURCES:
        code = _code(p)
        assert "__trap" not in code and "trap;" not in code, p.name
        assert not re.search(r"\bassert\s*\(", code), f"{p.name}: device-side assert"


def test_every_mbarrier_poll_is_bounded():
    """``mbar_try_wait`` may be called directly only by the bounded wait itself and by the drain loops, which carry
    their own ``globaltimer_ns`` limit within a few lines."""
    for p in SOURCES:
        lines = p.read_text().splitlines()
        for i, ln in enumerate(lines):
            if "mbar_try_wait(" not in ln or "__device__" in ln:
                continue
            if p.name == "ptx.cuh":
                continue  # definition and mbar_wait_bounded
            window = "\n".join(lines[max(0, i - 8):i + 6])
            assert "globaltimer_ns()" in window, f"{p.name}:{i + 1}: mbarrier poll without a time limit nearby"


def test_no_unbounded_spin_on_global_flags():
    """Loops that wait on memory another GPU writes go through the bounded helpers (``wait_ge_bounded`` and friends):
    a bare ``while (ld_acquire(...) < x);`` style spin must not appear."""
    pat = re.compile(r"while\s*\(\s*[^;{}]*(ld_acquire|ld_volatile|\*\s*\(?\s*volatile)[^;{}]*\)\s*(;|\{\s*\})")
    for p in SOURCES:
        assert not pat.search(_code(p)), p.name


def test_register_budget_assertion_next_to_setmaxnreg():
    for p in SOURCES:
        code = p.read_text()
        if p.name == "ptx.cuh" or "setmaxnreg_inc<" not in code:
            continue
        assert "setmaxnreg budget exceeds the launch allocation" in code, f"{p.name}: setmaxnreg without a budget static_assert"


def test_closed_batched_copy_calls_are_not_named():
    names = ["cuda" + "Memcpy" + "Batch" + "Async", "cuda" + "Memcpy3D" + "Batch" + "Async", "cu" + "Memcpy" + "Batch" + "Async",
             "cu" + "Memcpy3D" + "Batch" + "Async"]
    root = CSRC.parents[1]
    for p in list(root.rglob("*.py")) + list(root.rglob("*.cu")) + list(root.rglob("*.cuh")) + list(root.rglob("*.h")):
        if any(part in ("_work", "gpurun_out", "baseline", ".git") for part in p.parts):
            continue
        text = p.read_text(errors="ignore")
        for n in names:
            assert n not in text, f"{p}: names {n}"
