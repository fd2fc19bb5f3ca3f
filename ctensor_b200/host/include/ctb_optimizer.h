// Optimizer vocabulary shared by both host layers (second generation: ctb_host, first: ctb_gen1)
// and by the optimizer classes of optimizer_classes.h.
#pragma once

namespace ctb_opt {
// The optimizers of the reference's train_utils.h, in the order of the C ABI's ctb_optimizer codes.
enum class Kind : int { SGD = 0, Adam, AdamW, Adamax, NAdam, RAdam, RMSprop, Adagrad, Lion };
struct Hyper {
    double lr = 0.0, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, weight_decay = 0.0, alpha = 0.99;
};
}  // namespace ctb_opt
