"""Builds libi_core.so (the C++ core plus the sm_100a kernels) in-tree.

Every translation unit is compiled with
`nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3` and linked with the
static CUDA runtime, so the library loads on a machine without a GPU or driver
(calls that need a device then fail with an error message).  Run as
`python -m i_b200.build` or through `__graft_entry__.build()`.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(ROOT)
CSRC = os.path.join(ROOT, "csrc")
OUT_DIR = os.path.join(ROOT, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libi_core.so")

SOURCES = [
    "core/parser.cc",
    "core/validate.cc",
    "core/lower.cc",
    "core/plan.cc",
    "core/schedule.cc",
    "core/runtime.cc",
    "kernels/map.cu",
    "kernels/reduce.cu",
    "kernels/softmax.cu",
    "kernels/contract_simt.cu",
    "kernels/device_util.cu",
    "kernels/gemm_tcgen05.cu",
    "kernels/attention_tcgen05.cu",
    "kernels/dispatch.cu",
    "kernels/attention_static.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "-Xptxas", "-v",
    "-cudart", "static",
    "-I", os.path.join(REPO, "include"),
    "-I", os.path.join(CSRC, "core"),
    "-I", os.path.join(CSRC, "kernels"),
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _headers():
    out = []
    for base in (os.path.join(REPO, "include"), CSRC):
        for d, _, files in os.walk(base):
            out += [os.path.join(d, f) for f in files if f.endswith((".h", ".cuh"))]
    return out


def _compile(src, headers, verbose, obj_dir=None, extra=()):
    obj = os.path.join(obj_dir or OBJ_DIR, src.replace("/", "_") + ".o")
    path = os.path.join(CSRC, src)
    if _newer(obj, [path] + headers):
        return obj, ""
    cmd = [_nvcc()] + NVCC_FLAGS + list(extra) + ["-x", "cu", "-c", path, "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, proc.stdout, proc.stderr))
    return obj, proc.stderr if verbose else ""


def build(verbose=False, force=False, out_dir=None, extra_flags=()):
    """Compile what changed and link libi_core.so; returns its path.

    `out_dir` and `extra_flags` build a variant beside the shipped library, e.g. one with the
    attention kernels' cycle counters compiled in (`extra_flags=["-DIB_ATTN_PROFILE=1"]`).
    """
    out_dir = out_dir or OUT_DIR
    obj_dir = os.path.join(out_dir, "obj")
    lib = os.path.join(out_dir, "libi_core.so")
    os.makedirs(obj_dir, exist_ok=True)
    headers = _headers()
    if force:
        for f in os.listdir(obj_dir):
            os.remove(os.path.join(obj_dir, f))
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(lambda s: _compile(s, headers, verbose, obj_dir, extra_flags), SOURCES))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    if not _newer(lib, objs):
        cmd = [_nvcc(), "-shared", "-cudart", "static", "-o", lib] + objs + ["-lpthread", "-ldl", "-lrt"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (proc.stdout, proc.stderr))
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
