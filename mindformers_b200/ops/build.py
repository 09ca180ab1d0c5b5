"""Build the sm_100a kernel library in-tree.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a`` and
linked into ``lib/libmfb200.so`` next to this file; ``csrc/data_helpers.cpp`` (CPU-only dataset
index builders) becomes ``lib/libmfb200_data.so``. The build is incremental: an object is rebuilt
only when its source, a header or the flags changed. Run ``python -m mindformers_b200.ops.build``.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
KERNEL_LIB = os.path.join(LIB_DIR, "libmfb200.so")
DATA_LIB = os.path.join(LIB_DIR, "libmfb200_data.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-pthread"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the sm_100a kernel library cannot be built")
    return exe


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    return h.hexdigest()


def _compile_one(src: str, headers, log) -> str:
    name = os.path.splitext(os.path.basename(src))[0]
    obj = os.path.join(OBJ_DIR, name + ".o")
    stamp = obj + ".sha"
    want = _digest([src] + headers, " ".join(NVCC_FLAGS))
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == want:
        return obj
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log[name] = res.stderr[-20000:]
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr[-4000:]}")
    with open(stamp, "w") as f:
        f.write(want)
    return obj


def build(verbose: bool = False, jobs: int | None = None) -> dict:
    """Compile and link everything; returns {"kernel_lib": path, "data_lib": path}."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    cu = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    log: dict = {}
    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, headers, log), cu))
    link_stamp = KERNEL_LIB + ".sha"
    want = _digest(objs)
    if not (os.path.exists(KERNEL_LIB) and os.path.exists(link_stamp) and open(link_stamp).read() == want):
        cmd = [_nvcc(), "-shared", "-o", KERNEL_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
        with open(link_stamp, "w") as f:
            f.write(want)
    # CPU-side native helpers
    cpp = os.path.join(CSRC, "data_helpers.cpp")
    if os.path.exists(cpp):
        stamp = DATA_LIB + ".sha"
        want = _digest([cpp], " ".join(CXX_FLAGS))
        if not (os.path.exists(DATA_LIB) and os.path.exists(stamp) and open(stamp).read() == want):
            cxx = shutil.which("g++") or "g++"
            res = subprocess.run([cxx] + CXX_FLAGS + [cpp, "-o", DATA_LIB], capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"g++ failed for {cpp}:\n{res.stderr[-4000:]}")
            with open(stamp, "w") as f:
                f.write(want)
    with open(os.path.join(LIB_DIR, "ptxas_log.json"), "w") as f:
        json.dump(log, f, indent=1)
    if verbose:
        for k, v in log.items():
            print(f"== {k}\n{v}")
    return {"kernel_lib": KERNEL_LIB, "data_lib": DATA_LIB if os.path.exists(DATA_LIB) else None}


if __name__ == "__main__":
    out = build(verbose="-v" in sys.argv)
    print(json.dumps(out))
