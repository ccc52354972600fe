"""Build libb200lmk.so in-tree with nvcc for sm_100a (no torch involved: the library has a plain C ABI).

Each source is compiled to an object file (in parallel, only when it or a header changed) and the objects are linked
into landmark_attention_b200/lib/libb200lmk.so.
"""
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "_obj")
LIB_PATH = os.path.join(LIB_DIR, "libb200lmk.so")
SOURCES = ["api.cu", "attn_general.cu", "attn_sm100.cu", "attn_mask_sm100.cu", "grouped_softmax.cu", "retrieval.cu",
           "scores_sm100.cu", "cache_store.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return hs + [os.path.join(HERE, "..", "include", "b200lmk.h")]


def _newer(path, deps):
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into landmark_attention_b200/lib/libb200lmk.so; returns the path."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = _headers()
    jobs = []
    for s in SOURCES:
        src, obj = os.path.join(CSRC, s), os.path.join(OBJ_DIR, s[:-3] + ".o")
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in SOURCES]

    def run(cmd):
        return cmd, subprocess.run(cmd, capture_output=True, text=True)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, res in pool.map(run, jobs):
            if res.returncode != 0:
                raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + res.stdout + res.stderr)
            if verbose:
                print(res.stderr)
    if jobs or _newer(LIB_PATH, objs):
        res = subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *objs], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
