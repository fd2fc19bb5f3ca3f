#!/usr/bin/env bash
# TEST INFRASTRUCTURE — builds the real reference (CTensor src tree) as a shared library.
#
#   oracle/build_ref.sh REFERENCE_ROOT      (the reference checkout; or set CTENSOR_REFERENCE)
#
# Output: oracle/_ref/libctensor_ref.so, oracle/_ref/libctensor_ref_as_shipped.so (+ oracle/_ref/BUILD_INFO.txt).  Nothing else is
# written; no reference source is copied into the repository.
#
# The reference's HEAD does not compile (an unfinished CUDA allocator stub).  Two spots are
# removed on the fly, into a throw-away directory that is deleted on exit:
#   1. src/core/tensor.h   : the `//Memory pool` / `struct Block` / `class CudaMemoryPool` block
#   2. src/core/tensor.cpp : `#include <cuda>` and the `else if (dev.type == DeviceType::CUDA)`
#                            branch of Storage::allocate
# Every other file is compiled from where it lies under REFERENCE_ROOT, reached through a
# farm of symbolic links in the same throw-away directory (a quoted #include looks beside the
# including file first, so the two patched files must sit beside links to their neighbours).
#
# Flags: the two SIMD targets use exactly the reference's own per-target flags
# (CMakeLists.txt:63,71; GCC's default -ffp-contract=fast is part of what is being pinned).
# The scalar/OpenMP core is built -O2 -fopenmp ("tuned": the shipped CMake build gives it
# neither -O nor -fopenmp), which changes speed but not results (its arithmetic is plain
# double-precision + - * / and libm calls).
set -euo pipefail
REF="${1:-${CTENSOR_REFERENCE:-}}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
[ -n "$REF" ] || { echo "usage: build_ref.sh REFERENCE_ROOT (or set CTENSOR_REFERENCE)" >&2; exit 2; }
[ -d "$REF/src/core" ] || { echo "build_ref: no reference at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d /tmp/ctref.XXXXXX)"
trap 'rm -rf "$TMP"' EXIT
. "$HERE/ref_farm.sh"
make_ref_farm "$REF" "$TMP"

S="$TMP/src"
# the reference tree itself comes last: it only supplies header-only callers (the optimizers of
# src/neuralnet/train_utils.h); "core/tensor.h" still resolves to the patched copy above
INC="-I$S -I$S/core -I$S/cpu/AVX2 -I$S/cpu/AVX512 -I$REF/src"
CXX="${REF_CXX:-g++}"   # the g++ on PATH, not $CXX
STD="-std=gnu++20 -fPIC -w"
CORE_FLAGS="-O2 -fopenmp"
AVX2_FLAGS="-O3 -mavx2 -mfma -fopenmp"       # CMakeLists.txt:63
AVX512_FLAGS="-O3 -mavx512f -mavx512dq"      # CMakeLists.txt:71 (no OpenMP: single-threaded)

# Two builds of the same sources: the checker (scalar core -O2 -fopenmp) and, for the benchmark's
# baseline table only, the scalar core as the reference's CMake build ships it (no -O, no -fopenmp:
# CMakeLists.txt:28-61 gives those targets no per-target flags).
build_variant() { # object dir, core flags, output name
  local OBJ="$1" CORE="$2" LIBNAME="$3"
  mkdir -p "$OBJ"
  pids=()
  cc() { # name flags source
    $CXX $STD $2 $INC -c "$3" -o "$OBJ/$1.o" & pids+=($!)
  }
  cc tensor        "$CORE"         "$TMP/src/core/tensor.cpp"
  cc opsmp         "$CORE"         "$S/core/opsmp.cpp"
  cc ops_dispatch  "$CORE"         "$S/core/ops_dispatch.cpp"
  cc autograd      "$CORE"         "$S/core/autograd.cpp"
  cc avx2_f32      "$AVX2_FLAGS"   "$S/cpu/AVX2/ops_avx2_f32.cpp"
  cc avx2_d64      "$AVX2_FLAGS"   "$S/cpu/AVX2/ops_avx2_d64.cpp"
  cc avx512_f32    "$AVX512_FLAGS" "$S/cpu/AVX512/ops_avx512_f32.cpp"
  cc avx512_d64    "$AVX512_FLAGS" "$S/cpu/AVX512/ops_avx512_d64.cpp"
  cc loss          "$CORE"         "$REF/src/neuralnet/loss.cpp"      # GradCrossEntropy for the shim
  cc ref_shim      "$CORE_FLAGS"   "$HERE/ref_shim.cpp"
  for p in "${pids[@]}"; do wait "$p"; done
  $CXX -shared -o "$OUT/$LIBNAME" "$OBJ"/*.o -fopenmp
}
build_variant "$TMP/obj" "$CORE_FLAGS" libctensor_ref.so
build_variant "$TMP/obj_shipped" "" libctensor_ref_as_shipped.so
{
  echo "reference: $REF"
  echo "compiler: $($CXX --version | head -1)"
  echo "core flags: $CORE_FLAGS"
  echo "avx2 flags: $AVX2_FLAGS"
  echo "avx512 flags: $AVX512_FLAGS"
  echo "patched: tensor.h (CudaMemoryPool block removed), tensor.cpp (<cuda> include + CUDA allocate branch removed)"
} > "$OUT/BUILD_INFO.txt"
echo "built $OUT/libctensor_ref.so $OUT/libctensor_ref_as_shipped.so"
