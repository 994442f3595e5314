"""TEST / MEASUREMENT INFRASTRUCTURE - not product code; nothing in the package imports this.

Builds the reference project's own sm_100a programs, unmodified, from the sources where they lie in a checkout of
Bobliuuu/open-flapping-airplanes, into oracle/_ref/ (git-ignored). They are the "kernel to beat" timed beside this
library on the same GPU:

  oracle/_ref/ofa_tc3           llm/b200/megakernel/ofa.cu with the tcgen05 GEMM backend and three pipeline stages, built as
                                llm/b200/megakernel/build.sh does with NODOOM=1 (b200-run/modal_app.py:75 names the flags);
                                fixed at the reference's shapes V=100352 tied, T=512, B=8 (ofa.cu:71)
  oracle/_ref/test_gemm_sm100   llm/b200/gemm_tcgen05/test_gemm_sm100.cu (README.md:65-71), the 15-shape GEMM table

Nothing is copied into the repository: nvcc reads the reference tree in place, and the Doom link stubs are extracted at
build time from the here-document inside the reference's build.sh into oracle/_ref/. Without a reference checkout the
function reports that and builds nothing (the GPU box only uses the prebuilt files).

  python oracle/build_ref_cuda.py [/path/to/reference]
"""
import os
import re
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REF = os.environ.get("OFA_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))   # a checkout of the reference project


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build(ref=DEFAULT_REF, force=False, verbose=False):
    """Returns dict name -> path of what exists afterwards; {} when there is no reference checkout or no nvcc."""
    mk = os.path.join(ref, "llm", "b200", "megakernel")
    gm = os.path.join(ref, "llm", "b200", "gemm_tcgen05")
    have = {n: os.path.join(OUT, n) for n in ("ofa_tc3", "test_gemm_sm100") if os.path.exists(os.path.join(OUT, n))}
    if not os.path.isdir(mk) or not os.path.exists(_nvcc()):
        return have
    os.makedirs(OUT, exist_ok=True)
    log = []
    # the five extern "C" Doom symbols ofa.cu links against, as the reference's own NODOOM build stubs them
    stub = os.path.join(OUT, "doom_stub.cu")
    text = open(os.path.join(mk, "build.sh")).read()
    m = re.search(r"<<'STUB'\n(.*?)\nSTUB\n", text, re.S)
    if not m:
        raise RuntimeError("the reference's build.sh no longer carries the NODOOM stub")
    if not os.path.exists(stub) or open(stub).read() != m.group(1) + "\n":
        open(stub, "w").write(m.group(1) + "\n")
    jobs = [
        ("ofa_tc3", [os.path.join(mk, "ofa.cu"), stub],
         ["-arch=sm_100a", "-O3", "-std=c++17", "--extended-lambda", "-rdc=true", "-maxrregcount=128", "-DOFA_GEMM_BACKEND=1", "-DGEMM100_STAGES=3"], ["-lpthread"]),
        ("test_gemm_sm100", [os.path.join(gm, "test_gemm_sm100.cu")],
         ["-arch=sm_100a", "-O3", "-std=c++17", "-DOFA_GEMM_BACKEND=1"], ["-lcublas"]),
    ]
    for name, srcs, flags, libs in jobs:
        out = os.path.join(OUT, name)
        if not force and not _newer(out, srcs):
            have[name] = out
            continue
        cmd = [_nvcc()] + flags + srcs + ["-o", out] + libs
        r = subprocess.run(cmd, capture_output=True, text=True, cwd=OUT)
        log.append(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"building the reference's {name} failed:\n{r.stdout}{r.stderr}")
        have[name] = out
    if verbose and log:
        print("\n".join(log))
    return have


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REF, force="--force" in sys.argv, verbose=True))
