#!/usr/bin/env bash
# Builds tests/cpp/callers_program.cpp against the B200 host layers together with the
# reference's own callers of the operator path — autograd.cpp, layer.cpp, loss.cpp, batchnorm.cpp,
# Relu.cpp, dropout.cpp, norm.cpp, metrics.h (with the umbrella headers core.h / neuralnet.h) — UNCHANGED:
# the proof that the host layers are drop-in replacements for the reference's tensor/operator files.
#
#   tests/cpp/build_callers.sh REFERENCE_ROOT      (or set CTENSOR_REFERENCE)
#
# Outputs: tests/cpp/_built/callers_gen2_b200, callers_gen1_b200, train_step_gen2_b200(_edited, _edited4),
# reference_test_tensor_b200, reference_test_ops_b200, reference_time_avx_b200, reference_verify_gen1_b200.
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
mkdir -p "$G2/core"
for f in tensor.h device.h ops_dispatch.h opsmp.h ctb_host.h ctb_optimizer.h optimizer_classes.h; do ln -s "$PKG/host/include/$f" "$G2/core/$f"; done
# the callers' side, unchanged: autograd, the headers of src/core that only build on tensor.h (the
# Ops:: declarations, the dtype switch macro, the image readers' declarations), the umbrella headers,
# and src/neuralnet + src/dashboard file by file (a link to a whole directory would lead a quoted
# #include back into the real tree, to the reference's own tensor.h)
for f in autograd.h autograd.cpp ops.h dispatch.h data.h; do ln -s "$REF/src/core/$f" "$G2/core/$f"; done
for f in core.h neuralnet.h; do ln -s "$REF/src/$f" "$G2/$f"; done
(cd "$REF/src" && find neuralnet dashboard -type f \( -name '*.h' -o -name '*.cpp' \)) | while read -r f; do
  mkdir -p "$G2/$(dirname "$f")"
  [ "$f" = neuralnet/train_utils.h ] || ln -s "$REF/src/$f" "$G2/$f"
done
ln -s "$PKG/host/include/train_utils.h" "$G2/neuralnet/train_utils.h"      # replaces the reference's (optimizers, StepLR)
ln -s "$PKG/host/glue/autograd_glue.cpp" "$G2/core/autograd_glue.cpp"
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -o "$OUT/callers_gen2_b200" \
    "$HERE/callers_program.cpp" "$G2/core/autograd.cpp" "$G2/core/autograd_glue.cpp" \
    "$G2/neuralnet/layer.cpp" "$G2/neuralnet/loss.cpp" "$G2/neuralnet/batchnorm/batchnorm.cpp" "$G2/neuralnet/Relu.cpp" \
    "$G2/neuralnet/dropout/dropout.cpp" "$G2/neuralnet/norm/norm.cpp" -lctensor_host $LINK

# the timed training step (bench.py runs it for its `host_layer.train_step` key)
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -o "$OUT/train_step_gen2_b200" \
    "$HERE/train_step_program.cpp" "$G2/core/autograd.cpp" "$G2/core/autograd_glue.cpp" \
    "$G2/neuralnet/layer.cpp" "$G2/neuralnet/loss.cpp" -lctensor_host $LINK

# The same step with the edits the integration notes ask of autograd.cpp applied: accumulate_grad
# (src/core/autograd.cpp:64-156: host loops over the storage) becomes a call of the host layer's
# GPU version, and ensure_grad_buffer (:15-40) stops clearing gradient buffers with a host memset
# (fresh storage comes zeroed; an existing buffer is cleared on the GPU).  Both touch managed
# memory from the CPU, which drags every gradient buffer across PCIe and back in each step.  The
# edits are made on the fly on a copy in the scratch directory (the old bodies are kept under
# other names); nothing of it enters the repository.
sed -e 's/^void accumulate_grad(Tensor& target, const Tensor& grad_src) {/static void accumulate_grad_host_loops(Tensor\& target, const Tensor\& grad_src) {/' \
    -e 's/^void ensure_grad_buffer(Tensor &t, bool zero_existing) {/static void ensure_grad_buffer_host_memset(Tensor \&t, bool zero_existing) {/' \
    "$REF/src/core/autograd.cpp" > "$G2/core/autograd_edited.cpp"
cat >> "$G2/core/autograd_edited.cpp" <<'EOF'

#include "ctb_host.h"
void accumulate_grad(Tensor& target, const Tensor& grad_src) {
    if (!target.impl) return;
    ensure_grad_buffer(target, false);
    Tensor g = tensor_from_grad(target);
    ctb_host::accumulate_grad(g, grad_src);
}
void ensure_grad_buffer(Tensor& t, bool zero_existing) {
    if (!t.impl) throw std::runtime_error("ensure_grad_buffer: undefined tensor");
    if (!t.impl->grad)
        t.impl->grad = intrusive_ptr<Tensorimpl>(new Tensorimpl(t.shape(), t._dtype(), false, t.device()));   // zeroed storage
    else if (zero_existing)
        ctb_host::zero_grad(t);
}
EOF
grep -q "accumulate_grad_host_loops" "$G2/core/autograd_edited.cpp" || { echo "build_callers: accumulate_grad not found in autograd.cpp" >&2; exit 4; }
grep -q "ensure_grad_buffer_host_memset" "$G2/core/autograd_edited.cpp" || { echo "build_callers: ensure_grad_buffer not found in autograd.cpp" >&2; exit 4; }
# Third edit, in loss.cpp: the body of GradCrossEntropy::backward (src/neuralnet/loss.cpp:319-370,
# host loops over the logits) becomes one call of the host layer (its old body is commented out on
# the copy: from the definition line to the first closing brace in column 0).
awk '/^void GradCrossEntropy::backward\(const Tensor& self\) \{/ { skip = 1 } { if (skip) print "// " $0; else print } skip && /^}/ { skip = 0 }' \
    "$REF/src/neuralnet/loss.cpp" > "$G2/neuralnet/loss_edited.cpp"
cat >> "$G2/neuralnet/loss_edited.cpp" <<'EOF'

#include "ctb_host.h"
void GradCrossEntropy::backward(const Tensor& self) {
    if (!self.impl->grad) throw std::runtime_error("GradCrossEntropy: missing self grad");
    if (!pred.requires_grad()) return;
    double grad_out = read_scalar_at(self.impl->grad->data->data.get(), 0, self._dtype());
    if (reduction == "mean") grad_out /= static_cast<double>(pred.shape()[0]);
    accumulate_grad(pred, ctb_host::cross_entropy_backward(pred, target, (double)(float)grad_out));
}
EOF
grep -q "^// void GradCrossEntropy::backward" "$G2/neuralnet/loss_edited.cpp" || { echo "build_callers: GradCrossEntropy::backward not found in loss.cpp" >&2; exit 4; }
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -o "$OUT/train_step_gen2_b200_edited" \
    "$HERE/train_step_program.cpp" "$G2/core/autograd_edited.cpp" "$G2/core/autograd_glue.cpp" \
    "$G2/neuralnet/layer.cpp" "$G2/neuralnet/loss_edited.cpp" -lctensor_host $LINK

# A fourth edit, optional: the body of Loss::CrossEntropy (src/neuralnet/loss.cpp:90-118, eleven operators
# and a host read of the reduced value) becomes one call of the host layer, the backward node attached as
# the reference attaches it.
awk '/^Tensor Loss::CrossEntropy\(const Tensor& pred_, const Tensor& target_, std::string reduction\) \{/ { skip = 1 } { if (skip) print "// " $0; else print } skip && /^}/ { skip = 0 }' \
    "$G2/neuralnet/loss_edited.cpp" > "$G2/neuralnet/loss_edited4.cpp"
cat >> "$G2/neuralnet/loss_edited4.cpp" <<'EOF'

Tensor Loss::CrossEntropy(const Tensor& pred_, const Tensor& target_, std::string reduction) {
    if (!pred_.impl || !target_.impl) throw std::runtime_error("Loss::CrossEntropy: null tensor");
    if (pred_.impl->ndim != 2) throw std::runtime_error("CrossEntropy: Pred must be 2D [Batch, Classes]");
    Tensor result = ctb_host::cross_entropy(pred_, target_, reduction == "mean");
    if (pred_.requires_grad()) {
        result.impl->requires_grad = true;
        result.impl->grad_fn = std::make_shared<GradCrossEntropy>(pred_, target_, reduction);
    }
    return result;
}
EOF
grep -q "^// Tensor Loss::CrossEntropy" "$G2/neuralnet/loss_edited4.cpp" || { echo "build_callers: Loss::CrossEntropy not found in loss.cpp" >&2; exit 4; }
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -o "$OUT/train_step_gen2_b200_edited4" \
    "$HERE/train_step_program.cpp" "$G2/core/autograd_edited.cpp" "$G2/core/autograd_glue.cpp" \
    "$G2/neuralnet/layer.cpp" "$G2/neuralnet/loss_edited4.cpp" -lctensor_host $LINK

# The reference's own unit tests of the tensor type and the operator dispatcher (test/test.cpp,
# test/test_ops.cpp: known answers for creation, indexing, views, gather, arithmetic, matmul, reductions,
# broadcasting, astype, a backward pass), unchanged: they exit non-zero on the first failed assertion.
$CXX $FLAGS -I"$G2" -I"$G2/core" -o "$OUT/reference_test_tensor_b200" "$REF/test/test.cpp" -lctensor_host $LINK
$CXX $FLAGS -I"$G2" -I"$G2/core" -o "$OUT/reference_test_ops_b200" "$REF/test/test_ops.cpp" \
    "$G2/core/autograd.cpp" "$G2/core/autograd_glue.cpp" -lctensor_host $LINK

# The reference's own timing program (test/time_avx.cpp: 100 x add_mp and 100 x add of two 1000 x 1000
# tensors), unchanged; bench.py runs it beside the same file linked with the reference.
$CXX $FLAGS -I"$G2" -I"$G2/core" -o "$OUT/reference_time_avx_b200" "$REF/test/time_avx.cpp" -lctensor_host $LINK

# The convolution and pooling modules and the checkpoint reader/writer are not part of the operator
# path (their loops run on the host, over the managed storage); they must still COMPILE against the
# replaced headers, and so must a unit that includes the whole of nn.h (every header of the tree).
for f in conv/conv pooling/pooling check; do
  $CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -c "$G2/neuralnet/$f.cpp" -o "$TMP/$(basename $f).o"
done
printf '#include <iomanip>\n#include "neuralnet/nn.h"\nint main() { return 0; }\n' > "$TMP/everything.cpp"
$CXX $FLAGS -I"$G2" -I"$G2/core" -I"$G2/neuralnet" -c "$TMP/everything.cpp" -o "$TMP/everything.o"

# ---- first generation: the root of the reference tree ----------------------------------------------
if [ -f "$PKG/libctensor_gen1.so" ]; then
  G1="$TMP/gen1"
  mkdir -p "$G1"
  for f in tensor1.h opsmp.h ops1.h ctb_gen1.h train_utils.h; do ln -s "$PKG/host/gen1/include/$f" "$G1/$f"; done
  for f in ctb_optimizer.h optimizer_classes.h; do ln -s "$PKG/host/include/$f" "$G1/$f"; done
  for f in autograd.h autograd.cpp layer.h layer.cpp loss.h loss.cpp module.h batchnorm.h batchnorm.cpp Relu.h Relu.cpp \
           dropout.h dropout.cpp pooling.h pooling.cpp check.h check.cpp; do ln -s "$REF/$f" "$G1/$f"; done   # unchanged
  ln -s "$PKG/host/gen1/autograd_glue_gen1.cpp" "$G1/autograd_glue_gen1.cpp"
  $CXX $FLAGS -DCTB_GEN1 -I"$G1" -o "$OUT/callers_gen1_b200" \
      "$HERE/callers_program.cpp" "$G1/autograd.cpp" "$G1/autograd_glue_gen1.cpp" "$G1/layer.cpp" "$G1/loss.cpp" \
      "$G1/batchnorm.cpp" "$G1/Relu.cpp" "$G1/dropout.cpp" -lctensor_gen1 $LINK
  # the reference's own gradient checks of this generation (root verify.cpp), unchanged; its printed
  # output is compared with what the same file prints when linked with the reference
  ln -s "$REF/verify.cpp" "$G1/verify.cpp"
  $CXX $FLAGS -DCTB_GEN1 -I"$G1" -o "$OUT/reference_verify_gen1_b200" "$G1/verify.cpp" "$G1/autograd.cpp" \
      "$G1/autograd_glue_gen1.cpp" "$G1/loss.cpp" -lctensor_gen1 $LINK
  for f in pooling check; do $CXX $FLAGS -DCTB_GEN1 -I"$G1" -c "$G1/$f.cpp" -o "$TMP/gen1_$f.o"; done      # compile only
fi
echo "built $(ls "$OUT" | tr '\n' ' ')"
