// Drop-in for the reference's root train_utils.h (optimizers :26-540 and StepLR :542-560) on the
// first-generation host layer; the classes are in optimizer_classes.h of the second-generation
// include directory, which must be on the include path (or copied beside this file).
#pragma once
#include "ctb_gen1.h"
#include "tensor1.h"
#define CTB_OPT_NS ctb_gen1
#include "optimizer_classes.h"
