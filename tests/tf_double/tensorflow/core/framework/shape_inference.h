// Test double, NOT TensorFlow (see op_kernel.h beside this file): Status, errors and the few shape-inference names
// that the reference's TF-free math headers mention.
#ifndef TF_DOUBLE_SHAPE_INFERENCE_H
#define TF_DOUBLE_SHAPE_INFERENCE_H
#include <cstdint>
#include <sstream>
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
    const std::string& error_message() const { return msg_; }
private:
    bool ok_; std::string msg_;
};
namespace errors {
inline void AppendAll(std::ostringstream&) {}
template <typename A, typename... R> void AppendAll(std::ostringstream& o, const A& a, const R&... r) { o << a; AppendAll(o, r...); }
template <typename... A> Status InvalidArgument(const A&... a) { std::ostringstream o; o << "InvalidArgument: "; AppendAll(o, a...); return Status(o.str()); }
template <typename... A> Status Internal(const A&... a) { std::ostringstream o; o << "Internal: "; AppendAll(o, a...); return Status(o.str()); }
template <typename... A> Status Unimplemented(const A&... a) { std::ostringstream o; o << "Unimplemented: "; AppendAll(o, a...); return Status(o.str()); }
}  // namespace errors
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
