"""Build the sm_100a extension in-tree: ``python -m uttt_b200.ops.build``.

Compiles ``csrc/*.cu`` with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (works without a
GPU) and links ``uttt_b200/ops/_C.so`` next to the sources, so the binary travels with the tree.
Object files are cached under ``uttt_b200/ops/csrc/build`` and rebuilt only when a source or
header is newer.
"""
from __future__ import annotations

import glob
import os
import subprocess
import time
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(CSRC, "build")
TARGET = os.path.join(HERE, "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xptxas", "-v",
              "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1"]


def _include_flags():
    import torch
    from torch.utils.cpp_extension import include_paths
    flags = []
    for p in include_paths("cuda"):
        flags += ["-isystem", p]
    flags += ["-isystem", sysconfig.get_paths()["include"]]
    return flags, os.path.join(os.path.dirname(torch.__file__), "lib")


def _stale(out: str, deps) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    import torch
    os.makedirs(BUILD, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    inc, torch_lib = _include_flags()
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    flags = [f for f in NVCC_FLAGS if not f.startswith("-D_GLIBCXX")] + [abi]
    build_dir = BUILD
    if os.environ.get("UTTT_B200_BOUNDS_CHECK", "0") == "1":
        # checked build: index tables are validated against buffer extents, violations go to the status word
        flags.append("-DUTTT_BOUNDS_CHECK")
        build_dir = BUILD + "_checked"
        os.makedirs(build_dir, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + [__file__]
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(build_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, "-c", src, "-o", obj] + flags + inc
            if src.endswith(".cpp"):
                cmd = [nvcc, "-x", "cu", "-c", src, "-o", obj] + flags + inc
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        started = time.time()
        res = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(build_dir, os.path.basename(src) + ".log")
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stderr[-6000:]}")
        if verbose:
            print(res.stderr)
        # date the object at the start of its compilation: a source edited while nvcc ran stays newer than it
        obj = cmd[cmd.index("-o") + 1]
        os.utime(obj, (started, started))
        return src

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    # the shared object remembers which flavour it was linked from, so switching flavours relinks
    marker = TARGET + ".flavour"
    flavour = "checked" if build_dir != BUILD else "regular"
    try:
        with open(marker) as fh:
            linked = fh.read().strip()
    except OSError:
        linked = "regular"
    if jobs or force or linked != flavour or _stale(TARGET, objs):
        cmd = [nvcc, "-shared", "-o", TARGET] + objs + [
            "-L" + torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-lcudart", "-Xlinker", "-rpath", "-Xlinker", torch_lib]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
        with open(marker, "w") as fh:
            fh.write(flavour)
        _check_symbols(TARGET)
    return TARGET


def _check_symbols(path: str) -> None:
    """Load the shared object with immediate binding: a declaration in the bindings that no object defines
    (a stale object, a changed signature) fails here instead of at the first import on a GPU machine."""
    import ctypes
    import torch  # noqa: F401  (the extension links against torch's libraries)
    try:
        ctypes.CDLL(path, mode=os.RTLD_NOW)
    except OSError as exc:
        raise RuntimeError(f"{path} does not load: {exc}") from exc


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="--force" in sys.argv)
    print(path)
