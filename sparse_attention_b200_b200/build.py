"""Builds libsparse_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every csrc/*.cu is compiled to an object file of its own (in parallel, only when it or a
header is newer than its object) and the objects are linked into the shared library."""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libsparse_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")))


def headers():
    return glob.glob(os.path.join(HERE, "csrc", "*.h")) + glob.glob(os.path.join(HERE, "csrc", "*.cuh")) \
        + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def _obj(src):
    return os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")


def stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in sources() + headers())


def _compile(nvcc, src, verbose):
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", "-o", _obj(src), src]
    return src, subprocess.run(cmd, capture_output=True, text=True)


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    newest_header = max([os.path.getmtime(h) for h in headers()] + [0.0])
    todo = [s for s in sources()
            if force or not os.path.exists(_obj(s))
            or os.path.getmtime(_obj(s)) < max(os.path.getmtime(s), newest_header)]
    failed = False
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        for src, res in pool.map(lambda s: _compile(nvcc, s, verbose), todo):
            if verbose or res.returncode:
                sys.stderr.write(f"== {os.path.basename(src)}\n" + res.stdout + res.stderr)
            failed = failed or res.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libsparse_b200.so")
    # objects of sources that no longer exist must not be linked
    keep = {_obj(s) for s in sources()}
    res = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + sorted(keep),
                         capture_output=True, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libsparse_b200.so failed")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
