#!/usr/bin/env bash
# TEST INFRASTRUCTURE — builds tests/cpp/callers_program.cpp against the REFERENCE ITSELF, both
# generations, as the CPU twins the GPU builds of the same program are compared with.
#
#   oracle/build_callers_ref.sh REFERENCE_ROOT      (or set CTENSOR_REFERENCE)
#
# Outputs (only into oracle/_ref/): callers_gen2_ref, callers_gen2_ref_scalar, callers_gen1_ref,
# train_step_gen2_ref_scalar, time_avx_gen2_ref, verify_gen1_ref.
#   gen 2: the reference's src/core (tensor, opsmp, ops_dispatch, autograd, both SIMD back-ends,
#          shipped per-target flags) + src/neuralnet/layer.cpp, loss.cpp, Relu.cpp, batchnorm/batchnorm.cpp,
#          dropout/dropout.cpp, norm/norm.cpp
#   gen 1: the reference's root tensor1.cpp, opsmp.cpp, autograd.cpp, layer.cpp, loss.cpp, data.cpp,
#          batchnorm.cpp, Relu.cpp, dropout.cpp
# All sources are compiled where they lie (the second generation through the patched symlink
# farm of ref_farm.sh); nothing is copied into the repository.
set -euo pipefail
REF="${1:-${CTENSOR_REFERENCE:-}}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
PROGRAM="$HERE/../tests/cpp/callers_program.cpp"
[ -n "$REF" ] || { echo "usage: build_callers_ref.sh REFERENCE_ROOT (or set CTENSOR_REFERENCE)" >&2; exit 2; }
[ -d "$REF/src/core" ] || { echo "build_callers_ref: no reference at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d /tmp/ctcallers.XXXXXX)"
trap 'rm -rf "$TMP"' EXIT
. "$HERE/ref_farm.sh"
make_ref_farm "$REF" "$TMP"
CXX="${REF_CXX:-g++}"
STD="-std=gnu++20 -w"
mkdir -p "$TMP/obj2" "$TMP/obj1"
# The callers' side of the tree — src/neuralnet, src/dashboard, the umbrella headers core.h and
# neuralnet.h — file by file as symbolic links, so that every "core/tensor.h" they ask for is the
# farm's patched one (a link to a whole directory would lead back into the real tree).
(cd "$REF/src" && find neuralnet dashboard -type f \( -name '*.h' -o -name '*.cpp' \)) | while read -r f; do
  mkdir -p "$TMP/src/$(dirname "$f")"
  ln -s "$REF/src/$f" "$TMP/src/$f"
done
for f in core.h neuralnet.h; do ln -s "$REF/src/$f" "$TMP/src/$f"; done

# ---- second generation ------------------------------------------------------------------------
S="$TMP/src"
INC2="-I$S -I$S/core -I$S/cpu/AVX2 -I$S/cpu/AVX512 -I$S/neuralnet"
pids=()
cc2() { $CXX $STD $2 $INC2 -c "$3" -o "$TMP/obj2/$1.o" & pids+=($!); }
cc2 tensor       "-O2 -fopenmp"                 "$S/core/tensor.cpp"
cc2 opsmp        "-O2 -fopenmp"                 "$S/core/opsmp.cpp"
cc2 ops_dispatch "-O2 -fopenmp"                 "$S/core/ops_dispatch.cpp"
cc2 autograd     "-O2 -fopenmp"                 "$S/core/autograd.cpp"
cc2 avx2_f32     "-O3 -mavx2 -mfma -fopenmp"    "$S/cpu/AVX2/ops_avx2_f32.cpp"
cc2 avx2_d64     "-O3 -mavx2 -mfma -fopenmp"    "$S/cpu/AVX2/ops_avx2_d64.cpp"
cc2 avx512_f32   "-O3 -mavx512f -mavx512dq"     "$S/cpu/AVX512/ops_avx512_f32.cpp"
cc2 avx512_d64   "-O3 -mavx512f -mavx512dq"     "$S/cpu/AVX512/ops_avx512_d64.cpp"
cc2 layer        "-O2 -fopenmp"                 "$S/neuralnet/layer.cpp"
cc2 loss         "-O2 -fopenmp"                 "$S/neuralnet/loss.cpp"
cc2 batchnorm    "-O2 -fopenmp"                 "$S/neuralnet/batchnorm/batchnorm.cpp"
cc2 relu         "-O2 -fopenmp"                 "$S/neuralnet/Relu.cpp"
cc2 dropout      "-O2 -fopenmp"                 "$S/neuralnet/dropout/dropout.cpp"
cc2 norm         "-O2 -fopenmp"                 "$S/neuralnet/norm/norm.cpp"
$CXX $STD -O1 $INC2 -c "$PROGRAM" -o "$TMP/obj2/program.o" & pids+=($!)
for p in "${pids[@]}"; do wait "$p"; done
$CXX -o "$OUT/callers_gen2_ref" "$TMP"/obj2/*.o -fopenmp
# The same program with the dispatcher's CPU feature probes answering "no" (a command-line macro
# over __builtin_cpu_supports; the source is untouched): what the reference does on a host
# without AVX2 / AVX-512, its scalar+OpenMP back-end everywhere.  On an AVX host the SIMD entries
# throw for dim-wise reductions ("sum_avx512: only dim=-1", also inside accumulate_grad) and
# multiply permuted matrices as if they were contiguous, so Linear and most backward passes
# cannot run there; the scalar back-end honours strides and dims.
$CXX $STD -O2 -fopenmp '-D__builtin_cpu_supports(x)=0' $INC2 -c "$S/core/ops_dispatch.cpp" -o "$TMP/obj2/ops_dispatch.o"
$CXX -o "$OUT/callers_gen2_ref_scalar" "$TMP"/obj2/*.o -fopenmp
# the reference's own timing program (test/time_avx.cpp) as shipped: SIMD dispatcher against add_mp
$CXX $STD -O2 -fopenmp $INC2 -c "$REF/test/time_avx.cpp" -o "$TMP/time_avx.o"
$CXX $STD -O2 -fopenmp $INC2 -c "$S/core/ops_dispatch.cpp" -o "$TMP/ops_dispatch_simd.o"
$CXX -o "$OUT/time_avx_gen2_ref" $(ls "$TMP"/obj2/*.o | grep -v -e program.o -e ops_dispatch.o) "$TMP/ops_dispatch_simd.o" "$TMP/time_avx.o" -fopenmp
# the timed training step (tests/cpp/train_step_program.cpp) on the same scalar back-end
$CXX $STD -O1 $INC2 -c "$HERE/../tests/cpp/train_step_program.cpp" -o "$TMP/train_step.o"
rm -f "$TMP/obj2/program.o"
$CXX -o "$OUT/train_step_gen2_ref_scalar" "$TMP"/obj2/*.o "$TMP/train_step.o" -fopenmp

# ---- first generation (root of the reference tree) -----------------------------------------------
pids=()
cc1() { $CXX $STD -O2 -fopenmp -DCTB_GEN1 -I"$REF" -c "$2" -o "$TMP/obj1/$1.o" & pids+=($!); }
for f in tensor1 opsmp autograd layer loss data batchnorm Relu dropout; do cc1 "$f" "$REF/$f.cpp"; done
cc1 program "$PROGRAM"
$CXX $STD -O2 -fopenmp -I"$REF" -c "$REF/ops1.cpp" -o "$TMP/ops1.o" & pids+=($!)
$CXX $STD -O1 -fopenmp -I"$REF" -c "$REF/verify.cpp" -o "$TMP/verify.o" & pids+=($!)
for p in "${pids[@]}"; do wait "$p"; done
$CXX -o "$OUT/callers_gen1_ref" "$TMP"/obj1/*.o -fopenmp
# the reference's own gradient checks of the first generation (root verify.cpp: losses and one backward
# pass per operator, printed), linked with the reference's tensor1 / opsmp / ops1 / autograd / loss
rm -f "$TMP/obj1/program.o"
$CXX -o "$OUT/verify_gen1_ref" "$TMP"/obj1/*.o "$TMP/ops1.o" "$TMP/verify.o" -fopenmp
echo "built $OUT/callers_gen2_ref $OUT/callers_gen1_ref"
