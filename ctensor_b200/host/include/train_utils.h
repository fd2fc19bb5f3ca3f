// Drop-in for the reference's src/neuralnet/train_utils.h (optimizers and StepLR) on the second-
// generation host layer; the classes are in optimizer_classes.h.
#pragma once
#include "ctb_host.h"
#include "tensor.h"
#define CTB_OPT_NS ctb_host
#include "optimizer_classes.h"
