// TEST INFRASTRUCTURE: see ../framework/op_kernel.h.  The Padding enum lives there.
#pragma once
#include "tensorflow/core/framework/op_kernel.h"
