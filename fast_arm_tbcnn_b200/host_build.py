"""Builds the C++ host layer (the tbn:: API mirror) and its test driver with g++.

    python -m fast_arm_tbcnn_b200.host_build [--force]

Produces host/lib/libtbn_host.so (links against lib/libtbn_cuda.so), host/bin/run_graph and the Python
module host/lib/_tbn<ext suffix> (pybind11; `sys.path.insert(0, "host/lib"); import _tbn`).
"""
import glob
import os
import subprocess
import sys
import sysconfig

from . import build as _cuda_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "host")
LIB = os.path.join(HOST, "lib", "libtbn_host.so")
RUN_GRAPH = os.path.join(HOST, "bin", "run_graph")
SHARDED_GEMM = os.path.join(HOST, "bin", "sharded_gemm")
PY_MODULE = os.path.join(HOST, "lib", "_tbn" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))


def _stale(target, deps):
    return not os.path.exists(target) or any(os.path.getmtime(d) > os.path.getmtime(target) for d in deps)


def build(force=False):
    cuda_lib = _cuda_build.build()
    srcs = sorted(glob.glob(os.path.join(HOST, "src", "*.cpp")))
    hdrs = glob.glob(os.path.join(HOST, "include", "tbn", "**", "*.hpp"), recursive=True) + [
        os.path.join(ROOT, "include", "tbn_cuda.h")]
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    os.makedirs(os.path.dirname(RUN_GRAPH), exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    inc = ["-I", os.path.join(HOST, "include"), "-I", os.path.join(ROOT, "include")]
    cuda_dir = os.path.dirname(cuda_lib)
    if force or _stale(LIB, srcs + hdrs + [cuda_lib]):
        cmd = [cxx, "-std=c++20", "-O2", "-fPIC", "-shared", "-Wall", "-o", LIB] + inc + srcs + [
            "-L", cuda_dir, "-ltbn_cuda", "-Wl,-rpath,$ORIGIN/../../fast_arm_tbcnn_b200/lib"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("g++ failed building " + LIB)
    driver = os.path.join(HOST, "tests", "run_graph.cpp")
    if force or _stale(RUN_GRAPH, [driver, LIB] + hdrs):
        cmd = [cxx, "-std=c++20", "-O2", "-Wall", "-o", RUN_GRAPH] + inc + [driver, "-L", os.path.dirname(LIB), "-ltbn_host",
               "-L", cuda_dir, "-ltbn_cuda", "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN/../../fast_arm_tbcnn_b200/lib"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("g++ failed building " + RUN_GRAPH)
    driver2 = os.path.join(HOST, "tests", "sharded_gemm.cpp")
    if force or _stale(SHARDED_GEMM, [driver2, LIB] + hdrs):
        cmd = [cxx, "-std=c++20", "-O2", "-Wall", "-o", SHARDED_GEMM] + inc + [driver2, "-L", os.path.dirname(LIB), "-ltbn_host",
               "-L", cuda_dir, "-ltbn_cuda", "-Wl,-rpath,$ORIGIN/../lib", "-Wl,-rpath,$ORIGIN/../../fast_arm_tbcnn_b200/lib"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("g++ failed building " + SHARDED_GEMM)
    build_python_module(force, cxx, inc, cuda_dir, hdrs)
    return LIB, RUN_GRAPH


def build_python_module(force=False, cxx="g++", inc=(), cuda_dir="", hdrs=()):
    """The `_tbn` extension module (same Python API as the reference's pybind module)."""
    import pybind11
    src = os.path.join(HOST, "python", "bindings.cpp")
    if force or _stale(PY_MODULE, [src, LIB] + list(hdrs)):
        cmd = [cxx, "-std=c++20", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-o", PY_MODULE,
               "-I", sysconfig.get_paths()["include"], "-I", pybind11.get_include()] + list(inc) + [
               src, "-L", os.path.dirname(LIB), "-ltbn_host", "-L", cuda_dir, "-ltbn_cuda", "-Wl,-rpath,$ORIGIN",
               "-Wl,-rpath,$ORIGIN/../../fast_arm_tbcnn_b200/lib"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("g++ failed building " + PY_MODULE)
    return PY_MODULE


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
