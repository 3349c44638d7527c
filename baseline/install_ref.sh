#!/usr/bin/env bash
# Puts an UNMODIFIED copy of the parts of the reference's Python kernel package that this
# repository's CUDA kernels replace (vibe_kernels: its package file, common/, and the Triton
# softmax / RMSNorm / gather / scatter_add sub-packages -- the other kernel families are not on
# this path and are left out) under baseline/_ref/, which is git-ignored and travels to the GPU
# machine with the working tree on single-GPU runs.
# It is used for two things only: generating golden vectors from the reference's own kernels
# (tests/golden/make_golden_gpu.py) and timing them beside ours (bench.py's per-op table).
# The package is pure Python; its compiled companion (vibetensor._C) cannot be built here and
# is not needed for torch tensors (baseline/ref_kernels.py explains the stand-in).
# Usage: install_ref.sh <reference checkout>   (or VBT_REFERENCE_DIR in the environment)
set -euo pipefail
REF="${1:-${VBT_REFERENCE_DIR:-}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
if [ -z "$REF" ] || [ ! -d "$REF/vibe_kernels" ]; then
  echo "install_ref: no reference checkout (argument 1 or VBT_REFERENCE_DIR)" >&2
  exit 3
fi
rm -rf "$HERE/_ref/vibe_kernels"
mkdir -p "$HERE/_ref"
mkdir -p "$HERE/_ref/vibe_kernels"
cp "$REF/vibe_kernels/__init__.py" "$HERE/_ref/vibe_kernels/"
for sub in common softmax rmsnorm indexing; do
  cp -r "$REF/vibe_kernels/$sub" "$HERE/_ref/vibe_kernels/$sub"
done
find "$HERE/_ref/vibe_kernels" -name "__pycache__" -type d -prune -exec rm -rf {} +
echo "installed $HERE/_ref/vibe_kernels"
