"""Builds the sm_100a CUDA sources in ``csrc/`` into ``libgemlite_b200.so`` next to this file.

nvcc cross-compiles for sm_100a without a GPU; the library is linked against the static CUDA
runtime so that it only needs the driver at run time.  Run ``python -m gemlite_b200.build``.
"""
import os
import subprocess
import sys
import hashlib
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libgemlite_b200.so")
OBJ_DIR = os.path.join(HERE, "csrc", "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _digest(path, extra):
    h = hashlib.sha256()
    h.update(" ".join(extra).encode())
    for p in [path] + sorted(
        os.path.join(d, f) for d in (CSRC, os.path.join(HERE, "..", "include")) for f in os.listdir(d)
        if f.endswith((".cuh", ".h"))
    ):
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _compile_one(src, verbose):
    os.makedirs(OBJ_DIR, exist_ok=True)
    obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
    stamp = obj + ".sha"
    flags = list(NVCC_FLAGS)
    if verbose:
        flags += ["-Xptxas", "-v"]
    dig = _digest(src, flags)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig and not verbose:
        return obj, ""
    cmd = [_nvcc()] + flags + ["-x", "cu", "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
    with open(stamp, "w") as fh:
        fh.write(dig)
    return obj, res.stderr


def build(verbose=False, force=False):
    """Compile every source for sm_100a and link the shared library. Returns its path."""
    srcs = sources()
    if force and os.path.isdir(OBJ_DIR):
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    objs = [r[0] for r in results]
    if verbose:
        for (_, log), s in zip(results, srcs):
            sys.stderr.write("==== %s\n%s\n" % (os.path.basename(s), log))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static", "-Xlinker", "--exclude-libs=ALL"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
