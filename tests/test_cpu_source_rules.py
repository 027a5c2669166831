"""Source-tree invariants of the device code, checked as text.

* No bulk-copy load that fans one tile out to several CTAs of a cluster, anywhere: every source file travels to
  multi-GPU jobs, where such a load from a peer's memory is not allowed; remote tiles are staged in
  local memory or fetched per CTA with plain peer loads instead.
* None of the batched-memcpy driver / runtime entry points is named.
* Every spin-wait wrapper in the device headers is bounded (takes a limit and reports a status).

The patterns are assembled from pieces so that this file does not contain them itself.
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE_ROOTS = ("csrc", "rumus_b200", "tests", "bench", "examples")
EXTS = (".cu", ".cuh", ".cpp", ".h", ".hpp", ".py", ".cc")


def _sources():
    for f in sorted(os.listdir(ROOT)):
        if f.endswith(EXTS) and os.path.isfile(os.path.join(ROOT, f)):
            yield os.path.join(ROOT, f)
    for root in SOURCE_ROOTS:
        for d, dirs, files in os.walk(os.path.join(ROOT, root)):
            dirs[:] = [x for x in dirs if x != "__pycache__"]
            for f in files:
                if f.endswith(EXTS):
                    yield os.path.join(d, f)


def _scan(patterns):
    hits = []
    for path in _sources():
        with open(path, errors="replace") as fh:
            for n, line in enumerate(fh, 1):
                if any(p.search(line) for p in patterns):
                    hits.append(f"{os.path.relpath(path, ROOT)}:{n}: {line.strip()[:120]}")
    return hits


def test_no_fan_out_bulk_loads_anywhere():
    q = "multi" + "cast" + "::" + "cluster"
    pats = [re.compile(re.escape(q)),
            re.compile("SM90_TMA_LOAD_" + "MULTI" + "CAST"),
            re.compile("SM100_TMA_2SM_LOAD_" + "MULTI" + "CAST")]
    assert _scan(pats) == []


def test_batched_memcpy_entry_points_are_not_named():
    names = ["cu" + "da" + "Memcpy" + "Batch" + "Async", "cu" + "da" + "Memcpy3D" + "Batch" + "Async",
             "cu" + "Memcpy" + "Batch" + "Async", "cu" + "Memcpy3D" + "Batch" + "Async"]
    assert _scan([re.compile(n) for n in names]) == []


def test_device_waits_are_bounded():
    """Every open-ended loop in device code is one of the wait wrappers: within a few lines it
    checks the global timer against a budget and records an error code before giving up.  The raw
    polling primitives are used nowhere else in a loop condition."""
    open_loop = re.compile(r"while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\)")
    bad, seen = [], 0
    for path in _sources():
        if not path.endswith((".cu", ".cuh")):
            continue
        lines = open(path, errors="replace").read().splitlines()
        for n, line in enumerate(lines):
            if open_loop.search(line):
                seen += 1
                body = "\n".join(lines[n:n + 12])
                if "globaltimer_ns()" not in body or "record_error" not in body:
                    bad.append(f"{os.path.relpath(path, ROOT)}:{n + 1}")
            if re.search(r"while\s*\(\s*!\s*(mbar_try_wait|ld_acquire)", line):
                bad.append(f"{os.path.relpath(path, ROOT)}:{n + 1} (raw poll loop)")
    assert seen >= 3 and bad == []
