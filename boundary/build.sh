#!/usr/bin/env bash
# Builds the reference-facing artefacts of libvbt_b200.so against a VibeTensor checkout:
#   _build/libvbt_b200_plugin.so   vbt_b200_plugin.c  -- a plugin for the stable plugin C ABI
#   _build/vbt_b200_glue.o         vbt_b200_glue.cc   -- the in-tree binding, compiled (not
#                                  linked: the rest of the core is not built here) so that every
#                                  use of the reference's types is checked by the compiler
#   _build/libvbt_test_host.so     test_host.c        -- the plugin-host test double
# Usage: build.sh <reference checkout>   (or VBT_REFERENCE_DIR in the environment).
# Only headers are read from the checkout; nothing is copied from it.
set -euo pipefail
REF="${1:-${VBT_REFERENCE_DIR:-}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(dirname "$HERE")"
OUT="$HERE/_build"
if [ -z "$REF" ] || [ ! -f "$REF/include/vbt/plugin/vbt_plugin.h" ]; then
  echo "boundary/build.sh: no reference checkout (argument 1 or VBT_REFERENCE_DIR)" >&2
  exit 3
fi
LIBDIR="$ROOT/vibetensor_b200/lib"
if [ ! -f "$LIBDIR/libvbt_b200.so" ]; then
  echo "boundary/build.sh: build libvbt_b200.so first (python -m vibetensor_b200.build)" >&2
  exit 4
fi
mkdir -p "$OUT/shim/dlpack" "$OUT/shim/absl/log"
# DLPack header: any copy shipped with an installed Python package will do.
DLPACK="$(python - <<'PY'
import glob, sysconfig
site = sysconfig.get_paths()["purelib"]
hits = sorted(glob.glob(site + "/**/dlpack/dlpack.h", recursive=True))
print(hits[0] if hits else "")
PY
)"
if [ -z "$DLPACK" ]; then echo "boundary/build.sh: no dlpack.h found" >&2; exit 5; fi
cp "$DLPACK" "$OUT/shim/dlpack/dlpack.h"
# <absl/log/log.h>: the reference's headers only use LOG(level) << ... and CHECK(cond).
cat > "$OUT/shim/absl/log/log.h" <<'H'
#pragma once
#include <cstdlib>
#include <iostream>
struct VbtNullLog { template <class T> VbtNullLog& operator<<(const T&) { return *this; } };
#define LOG(level) VbtNullLog()
#define CHECK(cond) do { if (!(cond)) std::abort(); } while (0)
H
INC=(-I"$OUT/shim" -I"$REF/include" -I"$ROOT/include")
CUDA_HOME="${CUDA_HOME:-/usr/local/cuda}"

gcc -std=c11 -O2 -fPIC -fvisibility=hidden -Wall -Wextra -Wno-unused-parameter "${INC[@]}" \
    -shared -o "$OUT/libvbt_b200_plugin.so" "$HERE/vbt_b200_plugin.c" \
    -L"$LIBDIR" -lvbt_b200 -Wl,-rpath,'$ORIGIN/../../vibetensor_b200/lib'

g++ -std=c++20 -O2 -fPIC -Wall -Wno-unused-function -Wno-switch "${INC[@]}" -I"$REF/src" -I"$CUDA_HOME/include" \
    -DVBT_WITH_CUDA=1 -DVBT_INTERNAL_TESTS=0 -DVBT_WITH_AUTOGRAD=0 -DVBT_WITH_DISPATCH_V2=1 -DVBT_HAS_DLPACK_BF16=1 \
    -c "$HERE/vbt_b200_glue.cc" -o "$OUT/vbt_b200_glue.o"

gcc -std=c11 -O2 -fPIC -fvisibility=hidden -Wall -Wextra "${INC[@]}" \
    -shared -o "$OUT/libvbt_test_host.so" "$HERE/test_host.c" -ldl
echo "built $OUT/libvbt_b200_plugin.so $OUT/vbt_b200_glue.o $OUT/libvbt_test_host.so"
