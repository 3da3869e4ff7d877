"""Builds the native libraries in-tree (``oneflow_b200/lib``).

``python -m oneflow_b200.build`` compiles every CUDA source for sm_100a with nvcc and the
C++ runtime with g++. Objects are cached by source mtime so rebuilds are incremental.
The libraries are plain shared objects with a C ABI bound through ctypes, so no PyTorch
headers are needed and a full build takes about a minute.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
LIB = os.path.join(ROOT, "lib")
OBJ = os.path.join(ROOT, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _newer(src, obj, deps):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in [src] + deps)


def _run(cmd, log):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{p.stdout[-4000:]}")
    return p.stdout


def build_kernels(verbose=False, jobs=None):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) + glob.glob(os.path.join(CSRC, "comm", "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True) + glob.glob(
        os.path.join(CSRC, "**", "*.cuh"), recursive=True)
    nvcc = _nvcc()
    objs, todo = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.relpath(s, CSRC).replace(os.sep, "_") + ".o")
        objs.append(o)
        if _newer(s, o, headers):
            todo.append((s, o))
    def compile_one(so):
        s, o = so
        out = _run([nvcc] + NVCC_FLAGS + ["-I", CSRC, "-c", s, "-o", o], o + ".log")
        if verbose:
            print(out)
        return s
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 4)) as ex:
        for s in ex.map(compile_one, todo):
            print(f"[build] compiled {os.path.relpath(s, ROOT)}", flush=True)
    lib = os.path.join(LIB, "libofb_kernels.so")
    if todo or not os.path.exists(lib):
        _run([nvcc, "-shared", "-o", lib] + objs + ["-lcudart"], os.path.join(OBJ, "link_kernels.log"))
        print(f"[build] linked {os.path.relpath(lib, ROOT)}", flush=True)
    return lib


def build_core(verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "core", "*.cpp")))
    if not srcs:
        return None
    headers = glob.glob(os.path.join(CSRC, "core", "*.h"))
    lib = os.path.join(LIB, "libofb_core.so")
    if os.path.exists(lib) and not any(_newer(s, lib, headers) for s in srcs):
        return lib
    cxx = shutil.which("g++") or "g++"
    _run([cxx] + CXX_FLAGS + ["-shared", "-o", lib] + srcs + ["-lrt", "-ldl"], os.path.join(OBJ, "core.log"))
    print(f"[build] built {os.path.relpath(lib, ROOT)}", flush=True)
    return lib


def build_api(verbose=False):
    """C++ inference API (csrc/api): graph compiler and executor on top of libofb_kernels.so and libofb_core.so."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "api", "*.cpp")))
    if not srcs:
        return None
    headers = glob.glob(os.path.join(CSRC, "api", "*.h")) + [os.path.join(CSRC, "kernels", "ofb_kernels.h"),
                                                              os.path.join(CSRC, "core", "ofc_core.h")]
    lib = os.path.join(LIB, "libofb_api.so")
    kern = os.path.join(LIB, "libofb_kernels.so")
    core = os.path.join(LIB, "libofb_core.so")
    if os.path.exists(lib) and not any(_newer(s, lib, headers + [kern, core]) for s in srcs):
        return lib
    _run([_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", lib] + srcs +
         ["-L", LIB, "-lofb_kernels", "-lofb_core", "-lcudart", "-Xlinker", "-rpath=$ORIGIN"], os.path.join(OBJ, "api.log"))
    print(f"[build] built {os.path.relpath(lib, ROOT)}", flush=True)
    return lib


def build_sanitizers(verbose=False):
    """The host runtime's multi-threaded self-test (csrc/core/selftest) linked with the runtime's sources under ThreadSanitizer
    and under AddressSanitizer + UBSan: lib/ofb_core_selftest_tsan, lib/ofb_core_selftest_asan."""
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "core", "*.cpp"))) + [os.path.join(CSRC, "core", "selftest", "core_selftest.cpp")]
    headers = glob.glob(os.path.join(CSRC, "core", "*.h"))
    cxx = shutil.which("g++") or "g++"
    outs = []
    for tag, flags in (("tsan", ["-fsanitize=thread"]), ("asan", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"])):
        exe = os.path.join(LIB, f"ofb_core_selftest_{tag}")
        if not os.path.exists(exe) or any(_newer(s, exe, headers) for s in srcs):
            _run([cxx, "-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", "-pthread"] + flags + ["-o", exe] + srcs + ["-lrt", "-ldl"],
                 os.path.join(OBJ, f"selftest_{tag}.log"))
            print(f"[build] built {os.path.relpath(exe, ROOT)}", flush=True)
        outs.append(exe)
    return outs


def build_api_sanitized(verbose=False):
    """The graph API's sources (parser, plan compiler, autodiff, passes, host operators) compiled with the C++ training example
    under AddressSanitizer + UBSan: lib/ofb_api_train_asan. It links the regular kernel and runtime libraries; on the host
    device (-1) no CUDA code runs."""
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "api", "*.cpp"))) + [os.path.join(CSRC, "api", "examples", "train_graph.cpp")]
    headers = glob.glob(os.path.join(CSRC, "api", "*.h")) + glob.glob(os.path.join(CSRC, "common", "*.h"))
    exe = os.path.join(LIB, "ofb_api_train_asan")
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    if not os.path.exists(exe) or any(_newer(s, exe, headers) for s in srcs):
        cxx = shutil.which("g++") or "g++"
        _run([cxx, "-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", "-pthread", "-fsanitize=address,undefined",
              "-fno-sanitize-recover=undefined", "-I", os.path.join(cuda, "include"), "-I", os.path.join(CSRC, "api"), "-o", exe] + srcs +
             ["-L", LIB, "-lofb_kernels", "-lofb_core", "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{LIB}"],
             os.path.join(OBJ, "api_asan.log"))
        print(f"[build] built {os.path.relpath(exe, ROOT)}", flush=True)
    return exe


def build_api_thread_sanitized(verbose=False):
    """The same program under ThreadSanitizer, with the host runtime's sources compiled in (the scheduler's worker threads are
    what runs the operators of a plan): lib/ofb_api_train_tsan."""
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "api", "*.cpp"))) + [os.path.join(CSRC, "api", "examples", "train_graph.cpp")] + \
        sorted(glob.glob(os.path.join(CSRC, "core", "*.cpp")))
    headers = glob.glob(os.path.join(CSRC, "api", "*.h")) + glob.glob(os.path.join(CSRC, "common", "*.h")) + glob.glob(os.path.join(CSRC, "core", "*.h"))
    exe = os.path.join(LIB, "ofb_api_train_tsan")
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    if not os.path.exists(exe) or any(_newer(s, exe, headers) for s in srcs):
        cxx = shutil.which("g++") or "g++"
        _run([cxx, "-O1", "-g", "-std=c++17", "-fno-omit-frame-pointer", "-pthread", "-fsanitize=thread", "-I", os.path.join(cuda, "include"),
              "-I", os.path.join(CSRC, "api"), "-o", exe] + srcs +
             ["-L", LIB, "-lofb_kernels", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lrt", "-ldl", f"-Wl,-rpath,{LIB}"],
             os.path.join(OBJ, "api_tsan.log"))
        print(f"[build] built {os.path.relpath(exe, ROOT)}", flush=True)
    return exe


def build_all(verbose=False):
    return [build_kernels(verbose), build_core(verbose), build_api(verbose)]


if __name__ == "__main__":
    if "--sanitizers" in sys.argv:
        build_sanitizers(verbose="-v" in sys.argv)
        build_api_sanitized(verbose="-v" in sys.argv)
        build_api_thread_sanitized(verbose="-v" in sys.argv)
    else:
        build_all(verbose="-v" in sys.argv)
