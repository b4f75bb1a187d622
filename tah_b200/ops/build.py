"""Build the CUDA library in-tree with nvcc for sm_100a.

``python -m tah_b200.ops.build`` compiles every ``csrc/*.cu`` into
``tah_b200/lib/libtahb200.so`` (a plain C ABI shared library, loaded with ctypes by
:mod:`tah_b200.ops.cuda`).  Object files are cached by source hash, so a rebuild only
recompiles what changed.  nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC = os.path.join(ROOT, "csrc")
LIB_DIR = os.path.join(ROOT, "tah_b200", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtahb200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v"]
# --use_fast_math would flush denormals and use approximate div/sqrt; the kernels call the precise
# forms where rounding matters, so drop it from the list above if bit-parity work needs it
FLAGS.remove("--use_fast_math")


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _hash(path: str) -> str:
    h = hashlib.sha256()
    for p in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(p, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()[:16]


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    jobs = []
    for src in _sources():
        obj = os.path.join(obj_dir, f"{os.path.basename(src)[:-3]}.{_hash(src)}.o")
        jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        if os.path.exists(obj) and not force:
            return obj, ""
        for old in os.listdir(obj_dir):
            if old.startswith(os.path.basename(src)[:-3] + ".") and old.endswith(".o"):
                os.remove(os.path.join(obj_dir, old))
        cmd = [NVCC, *FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        results = list(pool.map(compile_one, jobs))
    objs = [o for o, _ in results]
    logs = "".join(l for _, l in results)
    if logs:
        with open(os.path.join(LIB_DIR, "ptxas.log"), "a") as fh:
            fh.write(logs)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < newest:
        cmd = [NVCC, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose and logs:
        print(logs)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
