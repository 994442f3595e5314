"""Build recipe for the CUDA library: one nvcc invocation, sm_100a only, output in-tree next to the sources.

`build()` is idempotent: it recompiles only when a source file is newer than the shared object.
"""
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "libofa_b200.so")
CLI = os.path.join(CSRC, "ofa_cli")              # the command-line host (csrc/ofa_cli.cpp), linked against LIB
SOURCES = ["runtime.cu", "noalloc.cu"]
HEADERS = ["common.cuh", "task_api.h", "elementwise.cuh", "gemm_tc.cuh", "attn_common.cuh", "attn_tc.cuh", "dp_nccl.inc", "simt_f32.cuh", "decode.cuh",
           "megakernel.cuh", os.path.join("..", "..", "include", "ofa_b200.h")]


def nvcc_path():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return p


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    """Compile csrc/ into csrc/libofa_b200.so for sm_100a. Returns the path of the library."""
    if not force and not needs_build():
        return LIB
    cmd = [nvcc_path(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--shared",
           "-Xcompiler", "-fPIC", "-o", LIB, "-ldl"] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))


def build_cli(force=False):
    """Compile csrc/ofa_cli.cpp (plain C++ over the C ABI) next to the library. Returns the path of the binary."""
    src = os.path.join(CSRC, "ofa_cli.cpp")
    hdr = os.path.join(CSRC, "..", "..", "include", "ofa_b200.h")
    if not force and os.path.exists(CLI) and os.path.getmtime(CLI) >= max(os.path.getmtime(src), os.path.getmtime(hdr)):
        return CLI
    build()
    cxx = shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise RuntimeError("no C++ compiler for ofa_cli")
    r = subprocess.run([cxx, "-O2", "-std=c++17", "-o", CLI, src, "-L" + CSRC, "-lofa_b200", "-Wl,-rpath,$ORIGIN"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building ofa_cli failed:\n" + r.stdout + r.stderr)
    return CLI
