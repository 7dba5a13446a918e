"""Ahead-of-time build of the sm_100a extension.

Every ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -rdc=true`` and linked
into ``tilerl_b200/_C.so`` (plain C ABI, loaded with ctypes; no torch headers, so
a full rebuild takes well under a minute).  The host-side C++ runtime
(``csrc/runtime.cpp``: paged allocator, block-table builder) is linked into the
same library.  The library is built in-tree so a source snapshot of the
repository carries it to the GPU machine.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
OUT = os.path.join(ROOT, "tilerl_b200", "_C.so")
OBJ = os.path.join(ROOT, "build", "obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-rdc=true", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    # global loads bypass L1: see "global loads and programmatic dependent launch" in csrc/common.cuh
    "-Xptxas", "-dlcm=cg",
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.sep not in c or os.path.exists(c)):
            return c
    return "nvcc"


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _stamp(path: str) -> str:
    h = hashlib.sha1()
    with open(path, "rb") as f:
        h.update(f.read())
    for hdr in sorted(os.listdir(CSRC)):
        if hdr.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC, hdr), "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, extra_flags=(), trace: bool = False, bounds: bool = False) -> str:
    """``trace=True`` builds ``tilerl_b200/_C_trace.so`` with ``-DTRL_TRACE`` (per-launch timestamps of a
    tick, read by ``tilerl_b200.utils.tick_trace``) next to the normal library.  ``bounds=True`` builds
    ``tilerl_b200/_C_bounds.so`` with ``-DTRL_DEBUG_BOUNDS``: the indices the kernels take from tables
    (KV slot of a token, block-table entries) are checked against the pool size; one out of range records
    an error word {bounds, site, index, limit} and is clamped, so the access stays inside the buffer."""
    assert not (trace and bounds)
    variant = "_trace" if trace else ("_bounds" if bounds else "")
    obj_dir = OBJ + variant
    out_path = OUT.replace("_C.so", f"_C{variant}.so")
    if trace:
        extra_flags = tuple(extra_flags) + ("-DTRL_TRACE",)
    if bounds:
        extra_flags = tuple(extra_flags) + ("-DTRL_DEBUG_BOUNDS",)
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in _sources():
        sp = os.path.join(CSRC, src)
        op = os.path.join(obj_dir, src + ".o")
        st = op + ".stamp"
        objs.append(op)
        stamp = _stamp(sp)
        if not force and os.path.exists(op) and os.path.exists(st) and open(st).read() == stamp:
            continue
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-x", "cu", "-c", sp, "-o", op]
        jobs.append((cmd, st, stamp))

    def run(job):
        cmd, st, stamp = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        if verbose and (r.stdout or r.stderr):
            print(r.stdout, r.stderr, file=sys.stderr)
        with open(st, "w") as f:
            f.write(stamp)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(out_path):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true",
               "-Xcompiler", "-fPIC", *objs, "-o", out_path]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return out_path


def build_tests(force: bool = False) -> list:
    """Standalone device checks under ``csrc/tests`` -> ``build/bin/<name>`` (run them on a GPU)."""
    tdir = os.path.join(CSRC, "tests")
    bdir = os.path.join(ROOT, "build", "bin")
    os.makedirs(bdir, exist_ok=True)
    outs = []
    for src in sorted(f for f in os.listdir(tdir) if f.endswith(".cu")):
        out = os.path.join(bdir, src[:-3])
        sp = os.path.join(tdir, src)
        if force or not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(sp):
            cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17",
                   "-o", out, sp]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        outs.append(out)
    return outs


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, trace="--trace" in sys.argv, bounds="--bounds" in sys.argv))
    if "--tests" in sys.argv:
        print("\n".join(build_tests(force="--force" in sys.argv)))
