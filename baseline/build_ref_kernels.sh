#!/bin/bash
# Builds the reference's own CUDA extensions (kairos_cuda_accel, awq_backend) for sm_100a, unmodified, from
# a scratch copy of its sources, and leaves ONLY the two built .so files in baseline/_ref/ (git-ignored).
# They are the same-box GPU baseline that baseline/time_ref_kernels.py times beside this library's kernels.
#   usage: baseline/build_ref_kernels.sh <root of the reference source tree>
set -e
REF="$1"
[ -d "$REF/kernels" ] || { echo "usage: $0 <root of the reference source tree>"; exit 2; }
HERE="$(cd "$(dirname "$0")" && pwd)"
WORK="$(mktemp -d /tmp/kairos_ref_build.XXXXXX)"
cp -r "$REF/kernels" "$WORK/kairos_kernels"
cp -r "$REF/thirdparty/AWQ/kernels" "$WORK/awq_kernels"
export TORCH_CUDA_ARCH_LIST="10.0a"
export MAX_JOBS="${MAX_JOBS:-4}"
for d in kairos_kernels awq_kernels; do
  (cd "$WORK/$d" && python setup.py build_ext --inplace > "$WORK/$d.log" 2>&1) || { tail -30 "$WORK/$d.log"; echo "build of $d failed (log: $WORK/$d.log)"; exit 1; }
done
mkdir -p "$HERE/_ref"
cp "$WORK"/kairos_kernels/kairos_cuda_accel*.so "$WORK"/awq_kernels/awq_backend*.so "$HERE/_ref/"
ls -la "$HERE/_ref"
