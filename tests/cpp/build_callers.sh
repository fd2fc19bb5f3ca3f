#!/usr/bin/env bash
# Builds tests/cpp/callers_program.cpp against the B200 host layers together with the
# reference's own callers of the operator path — autograd.cpp, layer.cpp, loss.cpp, batchnorm.cpp,
# Relu.cpp — UNCHANGED:
# the proof that the host layers are drop-in replacements for the reference's tensor/operator files.
#
#   tests/cpp/build_callers.sh REFERENCE_ROOT      (or set CTENSOR_REFERENCE)
#
# Outputs: tests/cpp/_built/callers_gen2_b200, tests/cpp/_built/callers_gen1_b200.
#
# What a maintainer of the reference does is: replace tensor.h / device.h / ops_dispatch.h /
# opsmp.h (second generation) or tensor1.h / opsmp.h / ops1.h (first generation) by the headers
# of ctensor_b200/host, drop tensor.cpp / ops_dispatch.cpp / opsmp.cpp and the cpu/ back-ends,
# add the glue translation unit, and link libctensor_host.so (or libctensor_gen1.so) + libctb200.so.
# This script does exactly that without touching the reference: a throw-away directory of
# symbolic links stands for the edited tree (a quoted #include looks beside the including file
# first, so the callers must sit beside links to the replaced headers).
set -euo pipefail
REF="${1:-${CTENSOR_REFERENCE:-}}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
PKG="$ROOT/ctensor_b200"
OUT="$HERE/_built"
[ -n "$REF" ] || { echo "usage: build_callers.sh REFERENCE_ROOT (or set CTENSOR_REFERENCE)" >&2; exit 2; }
[ -d "$REF/src/core" ] || { echo "build_callers: no reference at $REF" >&2; exit 3; }
mkdir -p "$OUT"
TMP="$(mktemp -d /tmp/ctdropin.XXXXXX)"
trap 'rm -rf "$TMP"' EXIT
CXX="${HOST_CXX:-g++}"          # the g++ on PATH
FLAGS="-std=gnu++20 -O2 -fopenmp -w"
LINK="-L$PKG -lctb200 -Wl,-rpath,\$ORIGIN/../../../ctensor_b200"

# ---- second generation: src/core + src/neuralnet --------------------------------------------------
G2="$TMP/gen2/src"
mkdir -p "$G2/core" "$G2/neuralnet"
for f in tensor.h device.h ops_dispatch.h opsmp.h ctb_host.h ctb_optimizer.h optimizer_classes.h; do ln -s "$PKG/host/include/$f" "$G2/core/$f"; done
ln -s "$PKG/host/include/train_utils.h" "$G2/neuralnet/train_utils.h"      # replaces the reference's (optimizers, StepLR)
for f in autograd.h autograd.cpp; do ln -s "$REF/src/core/$f" "$G2/core/$f"; done                        # unchanged
for f in layer.h layer.cpp loss.h loss.cpp module.h Relu.h Relu.cpp; do ln -s "$REF/src/neuralnet/$f" "$G2/neuralnet/$f"; done   # unchanged
mkdir -p "$G2/neuralnet/batchnorm"
for f in batchnorm.h batchnorm.cpp; do ln -s "$REF/src/neuralnet/batchnorm/$f" "$G2/neuralnet/batchnorm/$f"; done      # unchanged
ln -s "$PKG/host/glue/autograd_glue.cpp" "$G2/core/autograd_glue.cpp"
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -o "$OUT/callers_gen2_b200" \
    "$HERE/callers_program.cpp" "$G2/core/autograd.cpp" "$G2/core/autograd_glue.cpp" \
    "$G2/neuralnet/layer.cpp" "$G2/neuralnet/loss.cpp" "$G2/neuralnet/batchnorm/batchnorm.cpp" "$G2/neuralnet/Relu.cpp" -lctensor_host $LINK

# The convolution and pooling modules are not part of the operator path (their loops run on the
# host, over the managed storage); they must still COMPILE against the replaced headers.
mkdir -p "$G2/neuralnet/conv" "$G2/neuralnet/pooling"
for d in conv pooling; do for f in $d.h $d.cpp; do ln -s "$REF/src/neuralnet/$d/$f" "$G2/neuralnet/$d/$f"; done; done
for d in conv pooling; do
  $CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -c "$G2/neuralnet/$d/$d.cpp" -o "$TMP/$d.o"
done

# ---- first generation: the root of the reference tree ----------------------------------------------
if [ -f "$PKG/libctensor_gen1.so" ]; then
  G1="$TMP/gen1"
  mkdir -p "$G1"
  for f in tensor1.h opsmp.h ops1.h ctb_gen1.h train_utils.h; do ln -s "$PKG/host/gen1/include/$f" "$G1/$f"; done
  for f in ctb_optimizer.h optimizer_classes.h; do ln -s "$PKG/host/include/$f" "$G1/$f"; done
  for f in autograd.h autograd.cpp layer.h layer.cpp loss.h loss.cpp module.h batchnorm.h batchnorm.cpp Relu.h Relu.cpp; do ln -s "$REF/$f" "$G1/$f"; done   # unchanged
  ln -s "$PKG/host/gen1/autograd_glue_gen1.cpp" "$G1/autograd_glue_gen1.cpp"
  $CXX $FLAGS -DCTB_GEN1 -I"$G1" -o "$OUT/callers_gen1_b200" \
      "$HERE/callers_program.cpp" "$G1/autograd.cpp" "$G1/autograd_glue_gen1.cpp" "$G1/layer.cpp" "$G1/loss.cpp" \
      "$G1/batchnorm.cpp" "$G1/Relu.cpp" -lctensor_gen1 $LINK
fi
echo "built $(ls "$OUT" | tr '\n' ' ')"
