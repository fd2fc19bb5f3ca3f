// Glue between the first-generation host layer (libctensor_gen1.so) and the caller's autograd
// library.  The reference's opsmp.cpp and tensor1.cpp create a result's backward node themselves
// (root opsmp.cpp:178-245,292,364-391,443-448; tensor1.cpp:361,405) and Tensor::backward() calls the
// free function backward(Tensor&) of autograd.cpp (tensor1.cpp:471-475).  The node classes are
// defined by the caller's autograd.h, which the host layer does not contain; this translation
// unit is compiled BESIDE the caller's unchanged autograd.cpp, layer.cpp and loss.cpp and, in a
// static initialiser, registers a factory that builds the node the reference's operator would
// have built, and the backward entry point:
//
//   g++ -std=c++17 -fopenmp -I <dir with tensor1.h opsmp.h ops1.h ctb_gen1.h> \
//       autograd.cpp layer.cpp loss.cpp autograd_glue_gen1.cpp main.cpp -lctensor_gen1 -lctb200
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "autograd.h"      // the caller's
#include "ctb_gen1.h"

namespace {

using Inputs = std::vector<Tensor>;
using Maker = std::shared_ptr<GradFn> (*)(const Inputs&, double, const std::vector<size_t>&);

template <typename Node> std::shared_ptr<GradFn> binary_node(const Inputs& in, double, const std::vector<size_t>&) {
    return std::make_shared<Node>(in[0], in[1]);
}
template <typename Node> std::shared_ptr<GradFn> unary_node(const Inputs& in, double, const std::vector<size_t>&) {
    return std::make_shared<Node>(in[0]);
}
template <typename Node> std::shared_ptr<GradFn> scalar_node(const Inputs& in, double s, const std::vector<size_t>&) {
    return std::make_shared<Node>(in[0], s);
}

std::shared_ptr<GradFn> make_node(const std::string& op, const Inputs& in, double scalar, const std::vector<size_t>& dims) {
    static const std::unordered_map<std::string, Maker> table = {
        {"add", binary_node<GradAdd>}, {"diff", binary_node<GradSub>}, {"mult", binary_node<GradMul>},
        {"div", binary_node<GradDiv>}, {"pow", binary_node<GradPow>}, {"matmul", binary_node<GradMatMul>},
        {"add_scalar", scalar_node<GradAddScalar>}, {"sub_scalar", scalar_node<GradSubScalar>},
        {"sub_afterscalar", scalar_node<GradSubAfterScalar>}, {"mult_scalar", scalar_node<GradMulScalar>},
        {"div_scalar", scalar_node<GradDivScalar>}, {"scalar_div", scalar_node<GradScalarDiv>},
        {"pow_scalar", scalar_node<GradPowScalar>}, {"scalar_pow", scalar_node<GradScalarPow>},
        {"abs", unary_node<GradAbs>}, {"ln", unary_node<GradLn>}, {"exp", unary_node<GradExp>},
        {"sqrt", unary_node<GradSqrt>}, {"sin", unary_node<GradSin>}, {"asin", unary_node<GradASin>},
        {"cos", unary_node<GradCos>}, {"acos", unary_node<GradACos>}, {"tan", unary_node<GradTan>},
        {"atan", unary_node<GradATan>}, {"tanh", unary_node<GradTanH>}, {"sinh", unary_node<GradSinH>},
        {"cosh", unary_node<GradCosH>}, {"sigmoid", unary_node<GradSigmoid>}, {"Relu", unary_node<GradRelu>},
        {"softplus", unary_node<GradSoftPlus>},
        {"sum", [](const Inputs& i, double dim, const std::vector<size_t>&) -> std::shared_ptr<GradFn> {
             return std::make_shared<GradSum>(i[0], (int)dim);
         }},
        {"permute", [](const Inputs& i, double, const std::vector<size_t>& d) -> std::shared_ptr<GradFn> {
             return std::make_shared<GradPermute>(i[0], d);
         }},
        {"reshape", [](const Inputs& i, double, const std::vector<size_t>& old_shape) -> std::shared_ptr<GradFn> {
             return std::make_shared<GradReshape>(i[0], old_shape);
         }},
    };
    const auto it = table.find(op);
    return it == table.end() ? nullptr : it->second(in, scalar, dims);
}

const bool registered = [] {
    ctb_gen1::set_grad_factory(make_node);
    ctb_gen1::set_backward_entry([](Tensor& root) { backward(root); });
    return true;
}();

}  // namespace
