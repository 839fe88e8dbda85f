"""In-tree build of the sm_100a extension: ``python -m vllm_kunlun_b200.build``.

Kernel sources (``csrc/**/*.cu``) include no libtorch headers and are compiled straight with nvcc
for ``sm_100a``; only ``csrc/bindings.cpp`` sees torch.  Objects land in ``build/`` and the shared
object in ``vllm_kunlun_b200/_C.so`` so it travels with the source tree.  (The reference builds one
``CppExtension`` with ``-O3`` and no arch flags, ``setup.py:13-24``.)
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shlex
import subprocess
import sys
import sysconfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(ROOT, "build")
OUT = os.path.join(ROOT, "vllm_kunlun_b200", "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
              "-DNDEBUG"]


def _nvcc() -> str:
    for c in (os.environ.get("CUDA_HOME", ""), "/usr/local/cuda"):
        p = os.path.join(c, "bin", "nvcc")
        if c and os.path.exists(p):
            return p
    return "nvcc"


def _sources():
    cu, cpp = [], []
    for d, _, files in os.walk(CSRC):
        for f in sorted(files):
            p = os.path.join(d, f)
            if f.endswith(".cu"):
                cu.append(p)
            elif f.endswith(".cpp"):
                cpp.append(p)
    return sorted(cu), sorted(cpp)


def _headers_digest() -> str:
    h = hashlib.sha1()
    for d, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".h", ".cuh", ".hpp")):
                with open(os.path.join(d, f), "rb") as fh:
                    h.update(fh.read())
    return h.hexdigest()


def _stamp(src: str, cmd: list, hdr: str) -> str:
    h = hashlib.sha1()
    with open(src, "rb") as fh:
        h.update(fh.read())
    h.update(" ".join(cmd).encode())
    h.update(hdr.encode())
    return h.hexdigest()


def _compile(src: str, cmd: list, obj: str, hdr: str, verbose: bool):
    stamp_file = obj + ".stamp"
    stamp = _stamp(src, cmd, hdr)
    if os.path.exists(obj) and os.path.exists(stamp_file) and open(stamp_file).read() == stamp:
        return src, "", False
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {shlex.join(cmd)}\n{r.stdout}\n{r.stderr}")
    with open(stamp_file, "w") as fh:
        fh.write(stamp)
    return src, r.stderr, True


def build(verbose: bool = False, force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(BUILD, exist_ok=True)
    cu, cpp = _sources()
    hdr = _headers_digest()
    jobs = []
    objs = []
    nvcc = _nvcc()
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(nvcc)), "include") if os.sep in nvcc else "/usr/local/cuda/include"
    for s in cu:
        obj = os.path.join(BUILD, os.path.relpath(s, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        jobs.append((s, [nvcc, *NVCC_FLAGS, "-c", s, "-o", obj], obj))
    torch_inc = [f"-I{p}" for p in ce.include_paths()]
    py_inc = f"-I{sysconfig.get_paths()['include']}"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for s in cpp:
        obj = os.path.join(BUILD, os.path.relpath(s, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        jobs.append((s, ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C",
                         "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                         *torch_inc, py_inc, f"-I{cuda_inc}", "-c", s, "-o", obj], obj))
    if force:
        for _, _, obj in jobs:
            if os.path.exists(obj + ".stamp"):
                os.remove(obj + ".stamp")
    changed = False
    logs = {}
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        futs = [ex.submit(_compile, s, cmd, obj, hdr, verbose) for s, cmd, obj in jobs]
        for f in futs:
            src, log, did = f.result()
            changed |= did
            logs[src] = log
            if verbose and log:
                print(f"== {os.path.relpath(src, ROOT)}\n{log}")
    if changed or not os.path.exists(OUT):
        lib_dirs = ce.library_paths()
        cuda_lib = os.path.join(os.path.dirname(cuda_inc), "lib64")
        cmd = ["g++", "-shared", "-o", OUT, *objs, *[f"-L{d}" for d in lib_dirs], f"-L{cuda_lib}",
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
               *[f"-Wl,-rpath,{d}" for d in lib_dirs]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {shlex.join(cmd)}\n{r.stderr}")
    with open(os.path.join(BUILD, "ptxas.log"), "w") as fh:
        for s, log in logs.items():
            if log:
                fh.write(f"== {os.path.relpath(s, ROOT)}\n{log}\n")
    return OUT


def write_egg_info() -> str:
    """Entry-point metadata beside the sources, so that the installed vLLM finds the plugin from a checkout."""
    from ._entry_points import write_egg_info as _w
    return _w(ROOT)


if __name__ == "__main__":
    write_egg_info()
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
