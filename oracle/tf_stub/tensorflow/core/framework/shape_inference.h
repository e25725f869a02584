// Test double, NOT TensorFlow: the few names that the reference's TF-free math headers
// (include/utils/im2col.hpp, include/kernels/mex_kernel_common.hpp) mention, so that the
// reference sources can be compiled in place by oracle/Makefile without TensorFlow.
// Nothing here is executed by the oracle except Status and errors::InvalidArgument.
#ifndef ORACLE_TF_STUB_SHAPE_INFERENCE_H
#define ORACLE_TF_STUB_SHAPE_INFERENCE_H
#include <cstdint>
#include <string>
#include <vector>
namespace tensorflow {
typedef long long int64;
typedef int int32;
class Status {
public:
    Status() : ok_(true) {}
    explicit Status(const std::string& m) : ok_(false), msg_(m) {}
    static Status OK() { return Status(); }
    bool ok() const { return ok_; }
    const std::string& message() const { return msg_; }
private:
    bool ok_; std::string msg_;
};
namespace errors {
template <typename... A> Status InvalidArgument(const A&...) { return Status("invalid argument"); }
}
namespace shape_inference {
struct DimensionHandle {};
struct DimensionOrConstant { DimensionOrConstant(DimensionHandle) {} DimensionOrConstant(int64) {} };
class InferenceContext {
public:
    Status Add(DimensionHandle, DimensionOrConstant, DimensionHandle*) { return Status::OK(); }
    Status Subtract(DimensionHandle, DimensionOrConstant, DimensionHandle*) { return Status::OK(); }
    Status Divide(DimensionHandle, DimensionOrConstant, bool, DimensionHandle*) { return Status::OK(); }
};
}  // namespace shape_inference
}  // namespace tensorflow
#define TF_RETURN_IF_ERROR(expr) do { ::tensorflow::Status _s = (expr); if (!_s.ok()) return _s; } while (0)
#endif
