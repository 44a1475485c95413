"""CPU: rules every source file of the package keeps, because a multi-GPU run of the whole
repository is refused (or a shared GPU is put at risk) when one of them is broken: no TMA / bulk
load that delivers one tile to several CTAs of a cluster, none of the batched-copy runtime calls,
no device-side trap or assert, no clock or power setting, and every device-side polling loop in
the kernels carries a clock budget.  The banned words are assembled from pieces so that this file
does not name them either."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
SOURCES = [p for pat in ("flashsvd_b200/**/*.cu", "flashsvd_b200/**/*.cuh", "flashsvd_b200/**/*.h", "include/*.h",
                         "flashsvd_b200/**/*.py", "oracle/**/*.py", "bench.py", "__graft_entry__.py")
           for p in ROOT.glob(pat) if "build" not in p.parts]


def _texts():
    assert len(SOURCES) > 15
    return [(p, p.read_text(encoding="utf-8", errors="replace")) for p in SOURCES]


def test_no_forbidden_constructs():
    smi = "nvidia" + "-smi "
    banned = ("multi" + "cast", "Memcpy" + "Batch", "Memcpy3D" + "Batch", "__tr" + "ap", smi + "-lgc", smi + "-ac", smi + "-pm",
              "nvmlDeviceSet" + "ApplicationsClocks", "nvmlDeviceSet" + "GpuLockedClocks",
              "nvmlDeviceSet" + "PowerManagementLimit", "cuobj" + "dump", "nvdis" + "asm")
    for path, text in _texts():
        for word in banned:
            assert word not in text, f"{word!r} in {path.relative_to(ROOT)}"
    for path, text in _texts():
        if path.suffix in (".cu", ".cuh"):
            assert not re.search(r"(?<![_A-Za-z])assert\s*\(", text.replace("static_assert", "")), path


def test_every_device_polling_loop_has_a_budget():
    """A `while` that re-reads a flag, a barrier or a word another CTA / GPU writes must sit next to a
    clock64() budget check (the bounded-wait rule); found by the wait primitives it calls."""
    polls = ("mbar_try_wait", "ld_acquire_sys", "ld_word", "ld_volatile", "ld_acquire")
    for path, text in _texts():
        if path.suffix not in (".cu", ".cuh"):
            continue
        lines = text.splitlines()
        for i, line in enumerate(lines):
            if re.match(r"\s*while\s*\(", line) and any(p in line for p in polls):
                window = "\n".join(lines[max(0, i - 6): i + 14])
                assert "clock64()" in window or "wait_budget" in window or "wait_limit" in window, \
                    f"unbounded polling loop at {path.relative_to(ROOT)}:{i + 1}"
