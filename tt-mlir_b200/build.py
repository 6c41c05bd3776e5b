"""Builds libttb200.so: the sm_100a kernels, the C++ runtime target and both C ABIs.

Usage: python build.py [--force] [--jobs N].  nvcc cross-compiles for sm_100a without a
GPU.  Objects land in tt-mlir_b200/build/, the library in tt-mlir_b200/lib/ (both ignored by
git; the library travels with the source tree to the machine that runs it).  The flatbuffer
accessor header is regenerated from schema/ttnn_schema.py first.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libttb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-I" + os.path.join(HERE, "runtime"), "-I" + os.path.join(HERE, "runtime", "include"),
    "-I" + os.path.join(ROOT, "include"),
]
CUDA_INCLUDE = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")  # nvtx3 (header-only) for the C++ files
CXX_FLAGS = [
    "-std=c++17", "-O2", "-g", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-I" + CUDA_INCLUDE,
    "-I" + os.path.join(HERE, "runtime"), "-I" + os.path.join(HERE, "runtime", "include"),
    "-I" + os.path.join(ROOT, "include"),
]


def _sources():
    cu = sorted(f for f in os.listdir(os.path.join(HERE, "csrc")) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(os.path.join(HERE, "runtime")) if f.endswith(".cpp"))
    return [os.path.join(HERE, "csrc", f) for f in cu], [os.path.join(HERE, "runtime", f) for f in cpp]


def _headers_digest():
    h = hashlib.sha256()
    for base in ("csrc", "runtime", os.path.join("runtime", "include", "tt", "runtime"),
                 os.path.join("runtime", "generated")):
        d = os.path.join(HERE, base)
        for f in sorted(os.listdir(d)):
            if f.endswith((".h", ".cuh")):
                h.update(open(os.path.join(d, f), "rb").read())
    for f in sorted(os.listdir(os.path.join(ROOT, "include"))):
        h.update(open(os.path.join(ROOT, "include", f), "rb").read())
    return h.hexdigest()


def generate_schema_header():
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from ttmlir_b200.schema import gen_cpp
    from ttmlir_b200.schema.ttnn_schema import S
    text = gen_cpp.gen(S)
    path = os.path.join(HERE, "runtime", "generated", "ttnn_schema.h")
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)


def _compile(src, obj, cmd, stamp):
    key = hashlib.sha256((open(src, "rb").read().hex() + stamp + " ".join(cmd)).encode()).hexdigest()
    keyfile = obj + ".key"
    if os.path.exists(obj) and os.path.exists(keyfile) and open(keyfile).read() == key:
        return obj, False
    r = subprocess.run(cmd + ["-c", src, "-o", obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{r.stdout}\n{r.stderr}")
    if r.stderr.strip():
        sys.stderr.write(r.stderr)
    with open(keyfile, "w") as f:
        f.write(key)
    return obj, True


def build(force: bool = False, jobs: int | None = None, verbose: bool = True) -> str:
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    generate_schema_header()
    cu, cpp = _sources()
    stamp = _headers_digest() + ("force" + str(os.getpid()) if force else "")
    tasks = []
    for s in cu:
        tasks.append((s, os.path.join(BUILD, os.path.basename(s) + ".o"), ["nvcc"] + NVCC_FLAGS))
    for s in cpp:
        tasks.append((s, os.path.join(BUILD, os.path.basename(s) + ".o"), ["g++"] + CXX_FLAGS))
    changed = False
    objs = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        futs = [ex.submit(_compile, s, o, c, stamp) for s, o, c in tasks]
        for f in futs:
            obj, did = f.result()
            objs.append(obj)
            changed = changed or did
    if changed or not os.path.exists(LIB):
        cmd = ["nvcc", "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                       "-cudart", "static", "-ldl", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking failed:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(f"built {LIB}")
    elif verbose:
        print(f"up to date: {LIB}")
    return LIB


if __name__ == "__main__":
    j = None
    if "--jobs" in sys.argv:
        j = int(sys.argv[sys.argv.index("--jobs") + 1])
    build(force="--force" in sys.argv, jobs=j)
