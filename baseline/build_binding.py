"""Builds the C++ drop-in binding: the reference's UNMODIFIED pybind / autograd layer (csrc/ops/dconv.cpp with
dconv3d.h and dconv1d.h, read where they lie in the reference checkout) linked against libd2conv3d.so through
baseline/binding/d2c_dconv_binding.cpp, which supplies the four `*_cuda` functions that the reference implements
in its two .cu files.  Output: baseline/_ref/_binding/dconv_d2c_ops.so (git-ignored; travels to the GPU box).

    python baseline/build_binding.py <path of the reference checkout>

Needs no GPU.  Used only by tests/test_gpu_cpp_binding.py.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref", "_binding")
NAME = "dconv_d2c_ops"


def build(ref, verbose=False):
    from torch.utils import cpp_extension
    csrc = os.path.join(ref, "ops", "dconv-native", "csrc", "ops")
    libdir = os.path.join(ROOT, "d2conv3d_b200")
    if not os.path.exists(os.path.join(libdir, "libd2conv3d.so")):
        raise RuntimeError("build libd2conv3d.so first (python -m d2conv3d_b200.build)")
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "8")
    cpp_extension.load(
        name=NAME,
        sources=[os.path.join(csrc, "dconv.cpp"), os.path.join(HERE, "binding", "d2c_dconv_binding.cpp")],
        extra_include_paths=[csrc, os.path.join(ROOT, "include"), os.path.join(cpp_extension.CUDA_HOME, "include")],
        extra_cflags=["-O2"],
        extra_ldflags=[f"-L{libdir}", "-l:libd2conv3d.so", "'-Wl,-rpath,$$ORIGIN/../../../d2conv3d_b200'"],
        build_directory=OUT, with_cuda=True, is_python_module=False, verbose=verbose)
    return os.path.join(OUT, NAME + ".so")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    print(build(sys.argv[1], verbose="--verbose" in sys.argv))
