"""In-tree build of the sm_100a extension.

``build()`` compiles every ``csrc/*.cu`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (no torch
headers in the kernels, so each file takes seconds), ``csrc/bindings.cpp`` with the host compiler against
the torch headers, and links them into ``nmtgminor_b200/ops/_nmtg_b200_C.so`` next to this file.  nvcc
cross-compiles, so the build works on a machine without a GPU.  Objects are rebuilt only when their source
(or a header) is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_obj")
EXT_NAME = "_nmtg_b200_C"
SO_PATH = os.path.join(HERE, EXT_NAME + ".so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _extra_flags():
    """``NMTG_DEBUG_BOUNDS=1`` compiles the index checks that record status 6 (bad argument) instead of clamping."""
    return ["-DNMTG_DEBUG_BOUNDS"] if os.environ.get("NMTG_DEBUG_BOUNDS", "0") not in ("", "0") else []


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the sm_100a extension cannot be built")
    return cand


def sources():
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    return cu, cpp


def _newest_header_mtime() -> float:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return max([os.path.getmtime(h) for h in hs] + [0.0])


def _stale(src: str, obj: str, hdr_mtime: float) -> bool:
    if not os.path.exists(obj):
        return True
    m = os.path.getmtime(obj)
    return os.path.getmtime(src) > m or hdr_mtime > m


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout)
    return r.stdout


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile and link the extension; returns the path of the shared object."""
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OBJ_DIR, exist_ok=True)
    cu, cpp = sources()
    hdr = _newest_header_mtime()
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    inc = ["-I" + CSRC, "-I" + os.path.join(cuda_home, "include")]
    log: list = []
    jobs = []
    objs = []
    for f in cu:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ_DIR, f + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hdr):
            jobs.append([nvcc] + NVCC_FLAGS + _extra_flags() + inc + ["-c", src, "-o", obj])
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    host_inc = ["-I" + p for p in ce.include_paths("cuda")] + ["-I" + sysconfig.get_paths()["include"]]
    for f in cpp:
        src, obj = os.path.join(CSRC, f), os.path.join(OBJ_DIR, f + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hdr):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=" + EXT_NAME,
                         "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi] + inc + host_inc +
                        ["-c", src, "-o", obj])
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda c: _run(c, log), jobs))
    need_link = force or bool(jobs) or not os.path.exists(SO_PATH)
    if need_link:
        libdirs = ce.library_paths("cuda")
        link = ["g++", "-shared", "-o", SO_PATH] + objs
        for d in libdirs:
            link += ["-L" + d, "-Wl,-rpath," + d]
        link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        _run(link, log)
    if verbose:
        sys.stdout.write("\n".join(log) + "\n")
    with open(os.path.join(OBJ_DIR, "build.log"), "a") as fh:
        fh.write("\n".join(log) + "\n")
    return SO_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
