"""In-tree build of libdeltacnn_b200.so (sm_100a only).

Each translation unit under csrc/ is compiled to an object file in parallel and
relinked only when a source or header is newer than its object. The shared library
lands next to this file so that it travels with the package.

Usage: python deltacnn_b200/build.py [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libdeltacnn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, verbose):
    obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
    extra = os.environ.get("DC_NVCC_EXTRA", "").split()          # e.g. -DDC_IRB_STAMPS for a development build
    cmd = ["nvcc"] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force=False, verbose=False):
    """Compile what is out of date and link the shared library; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    # objects compiled with other extra flags are stale whatever their age
    flags_file = os.path.join(OBJ_DIR, "flags.txt")
    flags = os.environ.get("DC_NVCC_EXTRA", "")
    try:
        with open(flags_file) as f:
            same = f.read() == flags
    except OSError:
        same = flags == ""
    if not same:
        force = True
    with open(flags_file, "w") as f:
        f.write(flags)
    hdr_time = _newest_header()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(CSRC, src)), hdr_time)
        if stale:
            todo.append(src)
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as pool:
            list(pool.map(lambda s: _compile(s, verbose), todo))
    if todo or not os.path.exists(LIB_PATH):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs + ["-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
