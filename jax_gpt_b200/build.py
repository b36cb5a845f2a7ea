"""In-tree build of the sm_100a extension.

Every ``.cu`` under ``csrc/`` is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
into an object file, ``bindings.cpp`` is compiled with the host compiler against the torch
headers, and everything is linked into ``jax_gpt_b200/_C.so`` next to this file. Objects are
rebuilt only when a source or header is newer. nvcc cross-compiles without a GPU.

Run ``python -m jax_gpt_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "_C.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-cudart", "shared",
]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newest_header_mtime() -> float:
    m = 0.0
    for f in os.listdir(CSRC):
        if f.endswith((".cuh", ".h", ".inc")):
            m = max(m, os.path.getmtime(os.path.join(CSRC, f)))
    return m


def _stale(src: str, obj: str, hdr_m: float) -> bool:
    if not os.path.exists(obj):
        return True
    om = os.path.getmtime(obj)
    return om < os.path.getmtime(src) or om < hdr_m


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def build(verbose: bool = False, force: bool = False, debug: bool = False) -> str:
    """Builds ``_C.so`` if needed and returns its path. ``debug`` builds ``_C_debug.so`` instead: the same
    sources with ``-DB200_DEBUG`` (data-dependent indices are range-checked, violations land in the status
    word and the access is skipped); load it with ``B200_DEBUG=1`` in the environment."""
    import torch
    from torch.utils import cpp_extension as ce

    OBJ = os.path.join(HERE, "build", "debug") if debug else globals()["OBJ"]
    LIB = os.path.join(HERE, "_C_debug.so") if debug else globals()["LIB"]
    NVCC_FLAGS = globals()["NVCC_FLAGS"] + (["-DB200_DEBUG"] if debug else [])
    os.makedirs(OBJ, exist_ok=True)
    hdr_m = _newest_header_mtime()
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    cu_files = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    objs = []
    for f in cu_files:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OBJ, f[:-3] + ".o")
        objs.append(obj)
        if force or _stale(src, obj, hdr_m):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj])
    # host-side bindings
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", os.path.join(_cuda_home(), "include"), "-isystem", sysconfig.get_paths()["include"]]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    for f in sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp")):
        bsrc = os.path.join(CSRC, f)
        bobj = os.path.join(OBJ, f[:-4] + ".o")
        objs.append(bobj)
        if force or _stale(bsrc, bobj, hdr_m):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-I", CSRC, *inc, f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                         "-DTORCH_EXTENSION_NAME=_C", "-c", bsrc, "-o", bobj])
    if jobs:
        if verbose:
            print(f"[b200 build] compiling {len(jobs)} translation unit(s)", file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if jobs or not os.path.exists(LIB):
        torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["g++", "-shared", "-o", LIB, *objs, f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
               "-ltorch_cuda", "-ltorch", f"-L{os.path.join(_cuda_home(), 'lib64')}", "-lcudart", "-lpthread",
               f"-Wl,-rpath,{torch_lib}"]
        _run(cmd)
        if verbose:
            print(f"[b200 build] linked {LIB}", file=sys.stderr)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, debug="--debug" in sys.argv))
