// Glue between the host layer (libctensor_host.so) and the caller's autograd library.
//
// The reference creates a result's backward node inside each operator
// (src/core/ops_dispatch.cpp:159-167,247-286,312-315,378-381; src/core/tensor.cpp:192,228,424)
// and Tensor::backward() calls backward(root) (src/core/tensor.cpp:142-147,
// src/core/autograd.cpp:500-535).  The node classes (GradAdd, GradMulScalar, ...) are defined by
// the autograd library itself (src/core/autograd.h/.cpp), which the host layer does not
// contain.  This translation unit is compiled BESIDE the caller's unchanged autograd.cpp — it
// includes the caller's own autograd.h — and, in a static initialiser, hands the host layer a
// factory that builds the same node the reference's operator would have built, plus the
// entry point behind Tensor::backward().  Nothing in autograd.cpp, layer.cpp or loss.cpp is
// edited:
//
//   g++ -std=c++17 -fopenmp -I <dir with tensor.h ops_dispatch.h opsmp.h device.h ctb_host.h> \
//       autograd.cpp layer.cpp loss.cpp autograd_glue.cpp main.cpp -lctensor_host -lctb200
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "autograd.h"      // the caller's
#include "ctb_host.h"

namespace {

using Inputs = std::vector<Tensor>;
using Maker = std::shared_ptr<GradFn> (*)(const Inputs&, double);

template <typename Node> std::shared_ptr<GradFn> binary_node(const Inputs& in, double) {
    return std::make_shared<Node>(in[0], in[1]);
}
template <typename Node> std::shared_ptr<GradFn> unary_node(const Inputs& in, double) {
    return std::make_shared<Node>(in[0]);
}
template <typename Node> std::shared_ptr<GradFn> scalar_node(const Inputs& in, double s) {
    return std::make_shared<Node>(in[0], s);
}

const std::unordered_map<std::string, Maker>& makers() {
    static const std::unordered_map<std::string, Maker> table = {
        {"add", binary_node<GradAdd>}, {"sub", binary_node<GradSub>}, {"mul", binary_node<GradMul>},
        {"div", binary_node<GradDiv>}, {"pow", binary_node<GradPow>}, {"matmul", binary_node<GradMatMul>},
        {"add_scalar", scalar_node<GradAddScalar>}, {"sub_scalar", scalar_node<GradSubScalar>},
        {"sub_scalar_rev", scalar_node<GradSubAfterScalar>}, {"mul_scalar", scalar_node<GradMulScalar>},
        {"div_scalar", scalar_node<GradDivScalar>}, {"div_scalar_rev", scalar_node<GradScalarDiv>},
        {"pow_scalar", scalar_node<GradPowScalar>}, {"pow_scalar_rev", scalar_node<GradScalarPow>},
        {"abs", unary_node<GradAbs>}, {"log", unary_node<GradLn>}, {"ln", unary_node<GradLn>},
        {"exp", unary_node<GradExp>}, {"sqrt", unary_node<GradSqrt>}, {"sin", unary_node<GradSin>},
        {"asin", unary_node<GradASin>}, {"cos", unary_node<GradCos>}, {"acos", unary_node<GradACos>},
        {"tan", unary_node<GradTan>}, {"atan", unary_node<GradATan>}, {"tanh", unary_node<GradTanh>},
        {"sinh", unary_node<GradSinh>}, {"cosh", unary_node<GradCosh>}, {"sigmoid", unary_node<GradSigmoid>},
        {"relu", unary_node<GradRelu>}, {"softplus", unary_node<GradSoftplus>},
        {"sum", [](const Inputs& in, double dim) -> std::shared_ptr<GradFn> { return std::make_shared<GradSum>(in[0], (int)dim); }},
        {"gather", [](const Inputs& in, double dim) -> std::shared_ptr<GradFn> {
             return std::make_shared<GradGather>(in[0], in[1], (size_t)dim);
         }},
        {"reshape", [](const Inputs& in, double) -> std::shared_ptr<GradFn> {
             return std::make_shared<GradReshape>(in[0], in[0].shape());
         }},
    };
    return table;
}

std::shared_ptr<GradFn> make_node(const std::string& op, const Inputs& in, double scalar) {
    if (op == "permute") {       // inputs: the source; the permutation travels in ctb_host::last_permutation()
        return std::make_shared<GradPermute>(in[0], ctb_host::last_permutation());
    }
    const auto it = makers().find(op);
    return it == makers().end() ? nullptr : it->second(in, scalar);
}

const bool registered = [] {
    ctb_host::set_grad_factory(make_node);
    ctb_host::set_backward_entry([](Tensor& root) { backward(root); });
    return true;
}();

}  // namespace
