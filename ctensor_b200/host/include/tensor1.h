// Legacy spelling of the tensor header (tensor1.h of the reference's root tree).  The types are
// the ones of tensor.h; the legacy tree has no Device, which is why every tensor of this
// library lives in host-dereferenceable managed memory whatever its Device tag says.
// One documented difference between the two generations of the reference is NOT reproduced:
// the legacy tree rounds integer stores with lrint (tensor1.h:36), the current tree and this
// library truncate (src/core/tensor.h:77).
#pragma once
#include "tensor.h"
