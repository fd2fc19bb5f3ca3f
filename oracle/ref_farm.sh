# TEST INFRASTRUCTURE — sourced by build_ref.sh and build_callers_ref.sh.
#
# make_ref_farm REFERENCE_ROOT TMPDIR: a compilable view of the reference's second-generation
# tree under TMPDIR/src.  The reference's HEAD does not compile (an unfinished CUDA allocator
# stub); two spots are removed on the fly:
#   1. src/core/tensor.h   : the `//Memory pool` / `struct Block` / `class CudaMemoryPool` block
#   2. src/core/tensor.cpp : `#include <cuda>` and the `else if (dev.type == DeviceType::CUDA)`
#                            branch of Storage::allocate
# Every other file is reached through symbolic links (a quoted #include looks beside the
# including file first, so the two patched files must sit beside links to their neighbours).
# Nothing is copied into the repository; the caller deletes TMPDIR.
make_ref_farm() {
  local REF="$1" TMP="$2" d f
  for d in core cpu/AVX2 cpu/AVX512; do
    mkdir -p "$TMP/src/$d"
    for f in "$REF/src/$d"/*.h "$REF/src/$d"/*.cpp; do
      case "$(basename "$f")" in tensor.h|tensor.cpp) [ "$d" = core ] && continue ;; esac
      ln -s "$f" "$TMP/src/$d/$(basename "$f")"
    done
  done
  # spot 1: drop the CUDA pool block (from the "//Memory pool" marker up to the line before
  # "// STORAGE & INTERNAL IMPLEMENTATION")
  awk '
    /^\/\/Memory pool/ {skip=1}
    /^\/\/ STORAGE & INTERNAL IMPLEMENTATION/ {skip=0}
    !skip {print}
  ' "$REF/src/core/tensor.h" > "$TMP/src/core/tensor.h"
  # spot 2: drop "#include <cuda>" and the CUDA branch of Storage::allocate
  awk '
    /^#include <cuda>/ {next}
    /else if\(dev\.type == DeviceType::CUDA\)/ {print "    }"; skip=1; next}
    skip && /^    }$/ {skip=0; next}
    !skip {print}
  ' "$REF/src/core/tensor.cpp" > "$TMP/src/core/tensor.cpp"
}
