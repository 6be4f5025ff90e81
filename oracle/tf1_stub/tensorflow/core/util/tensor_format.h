// TEST INFRASTRUCTURE. Stand-in header: everything lives in op_kernel.h of this directory tree.
#pragma once
#include <tensorflow/core/framework/op_kernel.h>
