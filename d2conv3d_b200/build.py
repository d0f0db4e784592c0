"""Builds libd2conv3d.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m d2conv3d_b200.build [--force] [--verbose] [--microbench]

--microbench also builds the stand-alone programs of csrc/microbench into build/: l2_rates (the L2 scatter-add and
gather rates that bound the sampling kernels) and mma_rate (clocks per tcgen05.mma of the kernels' shape).  They run
on the GPU and are not part of the library.

The library links only the CUDA runtime (statically); it has no dependency on
torch or Python.  A GPU is not needed to build.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libd2conv3d.so")
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = ["d2c_api.cu", "depthwise.cu", "deform_sm100_fwd.cu", "deform_sm100_bwd.cu", "deform_sm100_dw.cu",
           "act_norm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", INCLUDE,
]


def _nvcc():
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def _deps():
    out = [os.path.join(INCLUDE, "d2conv3d.h")]
    for f in os.listdir(CSRC):
        if os.path.isfile(os.path.join(CSRC, f)):
            out.append(os.path.join(CSRC, f))
    return out


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force=False, verbose=False, unit_trace=False):
    """unit_trace: compile the forward kernel's per-unit timeline instrumentation in (-DD2C_UNIT_TRACE, see
    csrc/deform_sm100_fwd_kernel.cuh and unit_trace.py); always rebuilds.  Build again without it afterwards: the
    instrumented library is for measurements only."""
    if not force and not unit_trace and not needs_build():
        return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DD2C_UNIT_TRACE"] if unit_trace else [])
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [_nvcc()] + NVCC_FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed building libd2conv3d.so")
    cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static", "-Xlinker", "-soname=libd2conv3d.so"]
    subprocess.run(cmd, check=True)
    return LIB


def build_microbench():
    os.makedirs(OBJ_DIR, exist_ok=True)
    outs = []
    for name in ("l2_rates", "mma_rate"):
        out = os.path.join(OBJ_DIR, name)
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-o", out,
               os.path.join(CSRC, "microbench", name + ".cu")]
        subprocess.run(cmd, check=True)
        outs.append(out)
    return outs


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, unit_trace="--unit-trace" in sys.argv))
    if "--microbench" in sys.argv:
        print(build_microbench())
