#!/bin/bash
# Builds the UNMODIFIED reference extensions (dconv_native, fast_depthwise_conv3d) for sm_100 and installs
# them into baseline/_ref (git-ignored; it travels to the GPU box with the repo snapshot).  They are used
# only as a GPU-side parity oracle and as the "kernel to beat" timing -- never on the product path.
# The reference checkout is read-only, so the build runs from a copy under /tmp.
set -euo pipefail
REF=${1:?usage: install_ref.sh <path of the reference checkout>}
HERE=$(cd "$(dirname "$0")" && pwd)
WORK=$(mktemp -d /tmp/refbuild.XXXXXX)
export TORCH_CUDA_ARCH_LIST=10.0 MAX_JOBS=8 CC=/usr/bin/gcc CXX=/usr/bin/g++
for pkg in dconv-native fast-depthwise-conv3d; do
  cp -r "$REF/ops/$pkg" "$WORK/$pkg"
  python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
      --target "$HERE/_ref" --upgrade "$WORK/$pkg"
done
# the reference's own unit tests travel with the install (same git-ignored folder), so that they can be run
# unmodified against this repository's drop-in on a GPU box where the reference checkout is not mounted
mkdir -p "$HERE/_ref/_reference_tests/dconv_native" "$HERE/_ref/_reference_tests/fast_depthwise_conv3d"
cp "$REF"/ops/dconv-native/test/*.py "$HERE/_ref/_reference_tests/dconv_native/"
cp "$REF"/ops/fast-depthwise-conv3d/test/*.py "$HERE/_ref/_reference_tests/fast_depthwise_conv3d/"
rm -rf "$WORK"
echo "installed into $HERE/_ref"
