// Test double, NOT TensorFlow (see op_kernel.h beside this file): intentionally empty.
#ifndef ORACLE_TF_STUB_COMMON_SHAPE_FNS_H
#define ORACLE_TF_STUB_COMMON_SHAPE_FNS_H
#include "tensorflow/core/framework/shape_inference.h"
#endif
