#!/usr/bin/env bash
# TEST INFRASTRUCTURE ONLY.  Compiles VibeTensor's own CPU implementation of the
# vt:: op path from the sources where they lie (argument 1, or VBT_REFERENCE_DIR: the
# reference checkout) plus oracle/ref_shim.cpp into oracle/_ref/libvbt_ref_cpu.so.
# Reference sources are never copied into this repository; only the built .so
# (git-ignored) lands in oracle/_ref/.  The reference's own CMake build is not
# used: its third-party submodules are empty, so only the CPU files that compile
# on their own are listed here.
set -euo pipefail
REF="${1:-${VBT_REFERENCE_DIR:-}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
OBJ="$OUT/obj"
mkdir -p "$OBJ/shim/absl/log" "$OBJ/shim/dlpack"

if [ -z "$REF" ] || [ ! -d "$REF/src/vbt" ]; then
  echo "build_ref: no reference checkout (argument 1 or VBT_REFERENCE_DIR)" >&2
  exit 3
fi

# <absl/log/log.h>: the reference only uses LOG(level) << ... and CHECK(cond).
cat > "$OBJ/shim/absl/log/log.h" <<'EOF'
#pragma once
#include <cstdlib>
#include <iostream>
struct VbtNullLog { template <class T> VbtNullLog& operator<<(const T&) { return *this; } };
#define LOG(level) VbtNullLog()
#define CHECK(cond) do { if (!(cond)) std::abort(); } while (0)
EOF

# DLPack header: any copy shipped with an installed Python package will do.
DLPACK="$(python - <<'EOF'
import glob, sys, sysconfig
site = sysconfig.get_paths()["purelib"]
hits = sorted(glob.glob(site + "/**/dlpack/dlpack.h", recursive=True))
print(hits[0] if hits else "")
EOF
)"
if [ -z "$DLPACK" ]; then echo "build_ref: no dlpack.h found" >&2; exit 4; fi
cp "$DLPACK" "$OBJ/shim/dlpack/dlpack.h"

SRCS=(
  src/vbt/core/tensor.cc src/vbt/core/storage.cc src/vbt/core/broadcast.cc
  src/vbt/core/overlap.cc src/vbt/core/strided_loop.cc src/vbt/core/write_guard.cc
  src/vbt/core/contiguity.cc src/vbt/core/view_ops.cc src/vbt/core/tensor_ops.cc
  src/vbt/core/tensor_iter.cc src/vbt/core/indexing_basic.cc
  src/vbt/core/indexing_advanced.cc src/vbt/core/indexing_advanced_stats.cc
  src/vbt/core/tensor_iterator/core.cc
  src/vbt/cpu/storage.cc src/vbt/cpu/allocator.cc src/vbt/cpu/pinned_allocator.cc
  src/vbt/cpu/tensor_iterator/reduction.cc src/vbt/cpu/tensor_iterator/for_each_cpu.cc
  src/vbt/ops/default_kernels.cc src/vbt/ops/embedding_dispatch.cc
  src/vbt/ops/indexing_dispatch.cc src/vbt/ops/reduction_dim_dispatch.cc
  src/vbt/dispatch/dispatcher.cc src/vbt/dispatch/kernel_function.cc
  src/vbt/dispatch/dispatch_key_set.cc
  src/vbt/cuda/device_count.cc
)
FLAGS=(-std=c++20 -O2 -fPIC -w
  -DVBT_WITH_CUDA=0 -DVBT_INTERNAL_TESTS=0 -DVBT_WITH_AUTOGRAD=0
  -DVBT_WITH_DISPATCH_V2=1 -DVBT_HAS_DLPACK_BF16=1
  -I"$OBJ/shim" -I"$REF/include" -I"$REF/src")

pids=()
objs=()
for s in "${SRCS[@]}"; do
  o="$OBJ/$(echo "$s" | tr '/' '_').o"
  objs+=("$o")
  if [ ! -f "$o" ] || [ "$REF/$s" -nt "$o" ]; then
    g++ "${FLAGS[@]}" -c "$REF/$s" -o "$o" &
    pids+=($!)
  fi
done
g++ "${FLAGS[@]}" -c "$HERE/ref_shim.cpp" -o "$OBJ/ref_shim.o" &
pids+=($!)
for p in "${pids[@]}"; do wait "$p"; done

g++ -shared -o "$OUT/libvbt_ref_cpu.so" "$OBJ/ref_shim.o" "${objs[@]}" -lpthread
echo "built $OUT/libvbt_ref_cpu.so"
