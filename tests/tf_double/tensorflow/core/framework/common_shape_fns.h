// Test double, NOT TensorFlow (see op_kernel.h beside this file): intentionally empty.
#ifndef TF_DOUBLE_COMMON_SHAPE_FNS_H
#define TF_DOUBLE_COMMON_SHAPE_FNS_H
#include "tensorflow/core/framework/shape_inference.h"
#endif
