"""In-tree build of the native libraries (``python -m rumus_b200.build``).

* every ``csrc/kernels/*.cu`` and ``csrc/comm/*.cu`` is compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``) and linked into
  ``rumus_b200/lib/librumus_b200_cuda.so``;
* every ``csrc/{cpu_oracle,serve,runtime}/*.cpp`` is compiled with g++ into
  ``rumus_b200/lib/librumus_b200_host.so``.

Objects are cached under ``build/obj`` keyed by source + header mtimes, and
translation units compile in parallel.  nvcc cross-compiles, so this runs on a
machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")
LIB = os.path.join(ROOT, "rumus_b200", "lib")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_stamp(dirs) -> str:
    h = hashlib.sha1()
    for d in dirs:
        for f in sorted(glob.glob(os.path.join(d, "*.cuh")) + glob.glob(os.path.join(d, "*.h"))
                        + glob.glob(os.path.join(d, "*.hpp"))):
            h.update(f.encode())
            h.update(str(os.path.getmtime(f)).encode())
    return h.hexdigest()[:12]


def _compile(cmd, out, stamp_file, stamp):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    with open(stamp_file, "w") as f:
        f.write(stamp)
    return out, r.stderr


def build(verbose: bool = False, jobs: int | None = None) -> dict:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    nvcc = _nvcc()
    cu_dirs = [os.path.join(CSRC, "kernels"), os.path.join(CSRC, "comm")]
    cpp_dirs = [os.path.join(CSRC, d) for d in ("cpu_oracle", "serve", "runtime")]
    cu_srcs = sorted(sum((glob.glob(os.path.join(d, "*.cu")) for d in cu_dirs), []))
    cpp_srcs = sorted(sum((glob.glob(os.path.join(d, "*.cpp")) for d in cpp_dirs), []))
    hstamp_cu = _headers_stamp(cu_dirs)
    hstamp_cpp = _headers_stamp(cpp_dirs)
    inc = sum((["-I", d] for d in cu_dirs + cpp_dirs), [])
    extra = ["-Xptxas", "-v"] if verbose else []

    tasks = []
    cu_objs, cpp_objs = [], []
    for src in cu_srcs:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        cu_objs.append(obj)
        stamp = f"{os.path.getmtime(src)}:{hstamp_cu}:{' '.join(NVCC_FLAGS)}"
        sf = obj + ".stamp"
        if os.path.exists(obj) and os.path.exists(sf) and open(sf).read() == stamp:
            continue
        tasks.append(([nvcc] + NVCC_FLAGS + extra + inc + ["-c", src, "-o", obj], obj, sf, stamp))
    for src in cpp_srcs:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        cpp_objs.append(obj)
        stamp = f"{os.path.getmtime(src)}:{hstamp_cpp}:{' '.join(CXX_FLAGS)}"
        sf = obj + ".stamp"
        if os.path.exists(obj) and os.path.exists(sf) and open(sf).read() == stamp:
            continue
        tasks.append((["g++"] + CXX_FLAGS + inc + ["-c", src, "-o", obj], obj, sf, stamp))

    jobs = jobs or max(1, (os.cpu_count() or 4))
    logs = []
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        futs = [ex.submit(_compile, *t) for t in tasks]
        for f in futs:
            out, log = f.result()
            if verbose and log:
                logs.append(log)
    cuda_so = os.path.join(LIB, "librumus_b200_cuda.so")
    host_so = os.path.join(LIB, "librumus_b200_host.so")
    relink_cuda = bool(cu_objs) and (not os.path.exists(cuda_so) or any(
        os.path.getmtime(o) > os.path.getmtime(cuda_so) for o in cu_objs))
    if relink_cuda:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", cuda_so] + cu_objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    relink_host = bool(cpp_objs) and (not os.path.exists(host_so) or any(
        os.path.getmtime(o) > os.path.getmtime(host_so) for o in cpp_objs))
    if relink_host:
        cmd = ["g++", "-shared", "-o", host_so] + cpp_objs + ["-pthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    if verbose:
        for l in logs:
            sys.stderr.write(l)
    return {"compiled": len(tasks), "cuda_so": cuda_so, "host_so": host_so,
            "cu_sources": len(cu_srcs), "cpp_sources": len(cpp_srcs)}


if __name__ == "__main__":
    info = build(verbose="-v" in sys.argv)
    print(info)
