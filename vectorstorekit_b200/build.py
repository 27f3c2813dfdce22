"""Builds ``libvsk_cuda.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m vectorstorekit_b200.build            # build if sources are newer than the library
    python -m vectorstorekit_b200.build --force

nvcc cross-compiles without a GPU.  Object files go to ``vectorstorekit_b200/_build``.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libvsk_cuda.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime() -> float:
    files = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(f) for f in files)


def up_to_date() -> bool:
    return os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime()


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    hdr_mtime = max(os.path.getmtime(f) for f in glob.glob(os.path.join(CSRC, "*.cuh")) +
                    glob.glob(os.path.join(HERE, "..", "include", "*.h")))

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        if (not force and os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src)
                and os.path.getmtime(obj) >= hdr_mtime):
            return obj, ""
        cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(compile_one, sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    # NCCL is looked up with dlopen when a communicator is first asked for: no -lnccl here
    cmd = [nvcc, "-shared", "-cudart", "static", "-o", LIB] + objs + ["-lpthread", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


# ---- the checked variant ---------------------------------------------------------------------------------------
LIB_CHECKED = os.path.join(HERE, "libvsk_cuda_checked.so")
OBJ_CHECKED = os.path.join(HERE, "_build_checked")


def _compile_checked(nvcc: str, src: str, obj: str) -> str:
    """nvcc's own steps for one source (as `nvcc --dryrun` lists them), with the PTX pass of ``ptx_check.py`` between
    the front end and ptxas.  Returns the pass's report line."""
    stem = os.path.basename(src)[:-3]
    keep = os.path.join(OBJ_CHECKED, stem + ".steps")
    os.makedirs(keep, exist_ok=True)
    cmd = [nvcc] + NVCC_FLAGS + ["-DVSK_CHECKED", "--dryrun", "--keep", "--keep-dir", keep, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc --dryrun failed for {src}:\n{r.stderr}")
    steps = [ln[3:] for ln in r.stderr.splitlines() if ln.startswith("#$ ")]
    ptx = os.path.join(keep, stem + ".ptx")
    script = ["set -e"]
    for st in steps:
        first = st.split()[0] if st.split() else ""
        if first == "ptxas" or first.endswith("/ptxas"):
            script.append(f"{sys.executable} {os.path.join(HERE, 'ptx_check.py')} {ptx}")
        # `NAME=value` lines set nvcc's internal variables; the commands below only use the simple ones ($CICC_PATH,
        # PATH, LD_LIBRARY_PATH): lists with quotes and spaces are already expanded inside the commands
        if "=" in first and not first.startswith('"'):
            name, _, value = st.partition("=")
            if name.isidentifier() and value.strip() and " " not in value.strip() and '"' not in value:
                script.append(f"export {name}={value.strip()}")
            continue
        script.append(st)
    r = subprocess.run(["bash", "-c", "\n".join(script)], capture_output=True, text=True, cwd=keep)
    if r.returncode != 0:
        raise RuntimeError(f"checked build failed for {src}:\n{r.stdout}\n{r.stderr}")
    shutil.rmtree(keep, ignore_errors=True)     # hundreds of MB of preprocessed sources and PTX
    return r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""


def build_checked(force: bool = False, verbose: bool = False) -> str:
    """``libvsk_cuda_checked.so``: the same sources with -DVSK_CHECKED and every global access of every kernel routed
    through a range test (``ptx_check.py``, ``csrc/checked.cuh``).  A testing aid; loaded with VSK_CHECKED=1."""
    deps = _deps_mtime()
    deps = max(deps, os.path.getmtime(os.path.join(HERE, "ptx_check.py")))
    if not force and os.path.exists(LIB_CHECKED) and os.path.getmtime(LIB_CHECKED) >= deps:
        return LIB_CHECKED
    os.makedirs(OBJ_CHECKED, exist_ok=True)
    nvcc = _nvcc()

    def one(src):
        obj = os.path.join(OBJ_CHECKED, os.path.basename(src)[:-3] + ".o")
        return obj, _compile_checked(nvcc, src, obj)

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(one, sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log + "\n")
    cmd = [nvcc, "-shared", "-cudart", "static", "-o", LIB_CHECKED] + [o for o, _ in results] + ["-lpthread", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_CHECKED


if __name__ == "__main__":
    if "--checked" in sys.argv:
        print(build_checked(force="--force" in sys.argv, verbose="-v" in sys.argv))
    else:
        print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
