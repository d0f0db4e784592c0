"""Runs the reference's OWN unit-test files, unmodified, against this repository's drop-in packages:

    ops/dconv-native/test/test_deform_conv.py          DeformConv1dTester, DeformConv3dTester
    ops/dconv-native/test/test_modules.py              DeformConvTester
    ops/fast-depthwise-conv3d/test/test_conv3d_depthwise.py   DepthwiseConv3dTester

The files are not part of this repository: baseline/install_ref.sh puts them beside the reference's compiled
extension in baseline/_ref/_reference_tests (git-ignored), from where they are loaded by path.  Each file runs in
an interpreter of its own in which d2conv3d_b200.install_as_dropin() has registered this package's mirrors under
the names `dconv_native` and `fast_depthwise_conv3d`, so `from dconv_native import deform_conv3d` in the test
file resolves to the C-ABI-backed implementation here.  Two things are set up around the unmodified files: a stub
for the `expecttest` module (a test helper that torch.testing's TestCase imports and this image does not ship), and
TF32 switched off for cuDNN / cuBLAS, because the suites compare against PyTorch's own convolutions at 1e-5 .. 1e-7
and were written when those ran in plain fp32.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SUITES = os.path.join(ROOT, "baseline", "_ref", "_reference_tests")

RUNNER = r"""
import importlib.util, os, sys, types, unittest
sys.path.insert(0, %(root)r)
try:
    import expecttest  # noqa: F401
except ImportError:
    stub = types.ModuleType("expecttest")
    stub.TestCase = unittest.TestCase
    sys.modules["expecttest"] = stub
import torch
# the suites compare with cuDNN / cuBLAS results at 1e-5 .. 1e-7: those must be evaluated in plain fp32, not TF32
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False
import d2conv3d_b200
d2conv3d_b200.install_as_dropin()
import dconv_native, fast_depthwise_conv3d
assert dconv_native.__file__.startswith(%(root)r + os.sep + "d2conv3d_b200"), dconv_native.__file__
assert fast_depthwise_conv3d.__file__.startswith(%(root)r + os.sep + "d2conv3d_b200"), fast_depthwise_conv3d.__file__
n0 = d2conv3d_b200._lib.launch_count()
spec = importlib.util.spec_from_file_location("_reference_suite", %(path)r)
mod = importlib.util.module_from_spec(spec)
spec.loader.exec_module(mod)
suite = unittest.defaultTestLoader.loadTestsFromModule(mod)
result = unittest.TextTestRunner(verbosity=2, stream=sys.stdout).run(suite)
d2conv3d_b200._lib.device_status()
print("TESTS_RUN", result.testsRun, "FAILURES", len(result.failures), "ERRORS", len(result.errors),
      "SKIPPED", len(result.skipped), "LAUNCHES", d2conv3d_b200._lib.launch_count() - n0)
sys.exit(0 if result.wasSuccessful() and result.testsRun > 0 else 1)
"""

FILES = [("dconv_native", "test_deform_conv.py", 20), ("dconv_native", "test_modules.py", 4),
         ("fast_depthwise_conv3d", "test_conv3d_depthwise.py", 2)]


@pytest.mark.parametrize("pkg,fname,min_tests", FILES)
def test_reference_suite_passes_on_the_dropin(pkg, fname, min_tests):
    path = os.path.join(SUITES, pkg, fname)
    if not os.path.exists(path):
        pytest.skip("the reference's test files are not installed (baseline/install_ref.sh)")
    r = subprocess.run([sys.executable, "-c", RUNNER % dict(root=ROOT, path=path)], capture_output=True, text=True,
                       timeout=1500)
    tail = (r.stdout[-6000:] + "\n" + r.stderr[-3000:])
    assert r.returncode == 0, tail
    summary = [ln for ln in r.stdout.splitlines() if ln.startswith("TESTS_RUN")][-1].split()
    assert int(summary[1]) >= min_tests, tail
    assert int(summary[9]) > 0, "no kernel of this library was launched"
