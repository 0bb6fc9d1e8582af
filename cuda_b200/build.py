"""In-tree build of libcuda_llm_b200.so for sm_100a.

``python -m cuda_b200.build`` compiles every ``csrc/*.cu`` unit with nvcc (in parallel) and
links them into ``cuda_b200/lib/libcuda_llm_b200.so``.  The reference builds one extension
through ``setup.py`` with a kernel registry and an arch list (``setup.py:40-52,70-76`` in the
reference project); this build has one target architecture and no registry.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libcuda_llm_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-diag-suppress", "177",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    units = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    hdr_digest = _digest(headers)
    nvcc = _nvcc()
    jobs = []
    for u in units:
        src = os.path.join(CSRC, u)
        obj = os.path.join(OBJ, u[:-3] + ".o")
        stamp = obj + ".stamp"
        want = _digest([src]) + hdr_digest
        have = open(stamp).read() if os.path.exists(stamp) else ""
        if force or have != want or not os.path.exists(obj):
            jobs.append((src, obj, stamp, want))

    def run(job):
        src, obj, stamp, want = job
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        with open(stamp, "w") as f:
            f.write(want)
        return src, r.stderr

    if jobs:
        workers = int(os.environ.get("MAX_JOBS", str(min(len(jobs), os.cpu_count() or 4))))
        with ThreadPoolExecutor(max_workers=workers) as ex:
            for src, log in ex.map(run, jobs):
                if verbose or ptxas_info:
                    print(f"[build] {os.path.basename(src)}\n{log}" if ptxas_info else
                          f"[build] {os.path.basename(src)}", flush=True)
    objs = [os.path.join(OBJ, u[:-3] + ".o") for u in units]
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                     "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


EXT_SRC = os.path.join(HERE, "ext", "fused_online_softmax_cuda.cpp")
EXT_DIR = os.path.join(HERE, "compat")


def extension_path() -> str:
    import sysconfig
    return os.path.join(EXT_DIR, "fused_online_softmax_cuda" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_extension(verbose: bool = False, force: bool = False) -> str:
    """Compile the PyTorch extension ``fused_online_softmax_cuda`` (the reference's module name,
    ``setup.py:128`` in the reference project) from ``ext/fused_online_softmax_cuda.cpp`` with the host
    compiler and link it against ``libcuda_llm_b200.so`` (found at run time through an ``$ORIGIN``
    rpath).  The product lands in ``cuda_b200/compat``, the directory a caller puts on ``sys.path``."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as C
    lib = build(verbose=verbose)
    out = extension_path()
    stamp = out + ".stamp"
    want = _digest([EXT_SRC, os.path.join(ROOT, "include", "cuda_llm_b200.h")]) + torch.__version__
    if not force and os.path.exists(out) and os.path.exists(stamp) and open(stamp).read() == want:
        return out
    try:
        inc = C.include_paths(device_type="cuda")
        libdirs = C.library_paths(device_type="cuda")
    except TypeError:                              # older signature
        inc, libdirs = C.include_paths(cuda=True), C.library_paths(cuda=True)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-DTORCH_EXTENSION_NAME=fused_online_softmax_cuda", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-I", os.path.join(ROOT, "include"), "-I", sysconfig.get_paths()["include"]]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [EXT_SRC, "-o", out, "-L", LIBDIR, "-lcuda_llm_b200", "-Wl,-rpath,$ORIGIN/../lib"]
    for d in libdirs:
        cmd += ["-L", d]
    cmd += ["-Wl,-rpath," + libdirs[0], "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-lcudart"]
    if verbose:
        print("[build] fused_online_softmax_cuda extension", flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"extension build failed:\n{r.stdout}\n{r.stderr[-4000:]}")
    with open(stamp, "w") as f:
        f.write(want)
    return out


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
    if "--no-extension" not in sys.argv:
        print(build_extension(verbose=True, force="--force" in sys.argv))
