// Test double, NOT TensorFlow (see op_kernel.h beside this file): Status, errors and the few shape-inference names
// that the reference's TF-free math headers mention.
#ifndef TF_DOUBLE_SHAPE_INFERENCE_H
#define TF_DOUBLE_SHAPE_INFERENCE_H
#include <cstdint>
#include <cstdlib>
#include <utility>
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
// Functional stand-ins: a dimension is a known int64 (-1 = unknown), a shape a vector of them.
struct DimensionHandle { int64 v; DimensionHandle() : v(-1) {} explicit DimensionHandle(int64 x) : v(x) {} };
struct DimensionOrConstant { int64 v; DimensionOrConstant(DimensionHandle d) : v(d.v) {} DimensionOrConstant(int64 x) : v(x) {} DimensionOrConstant(int x) : v(x) {} };
struct ShapeHandle { std::vector<int64> dims; bool known; ShapeHandle() : known(false) {} };

// Attribute values arrive as text ("3,3", "true", "0.5", "L2"), typed on request as the OpKernel double does.
class InferenceContext {
public:
    std::vector<ShapeHandle> inputs, outputs;
    std::vector<std::pair<std::string, std::string>> attrs;

    ShapeHandle input(int i) const { return inputs[size_t(i)]; }
    void set_output(int i, const ShapeHandle& s) { if (outputs.size() <= size_t(i)) outputs.resize(size_t(i) + 1); outputs[size_t(i)] = s; }
    Status WithRank(const ShapeHandle& s, int rank, ShapeHandle* out) {
        if (int(s.dims.size()) != rank) return errors::InvalidArgument("Shape must be rank ", rank, " but is rank ", s.dims.size());
        *out = s; return Status::OK();
    }
    DimensionHandle Dim(const ShapeHandle& s, int i) const { return DimensionHandle(s.dims[size_t(i)]); }
    Status Merge(DimensionHandle a, DimensionHandle b, DimensionHandle* out) {
        if (a.v >= 0 && b.v >= 0 && a.v != b.v) return errors::InvalidArgument("Dimensions must be equal, but are ", a.v, " and ", b.v);
        *out = a.v >= 0 ? a : b; return Status::OK();
    }
    ShapeHandle MakeShape(const std::vector<DimensionHandle>& d) { ShapeHandle s; s.known = true; for (auto& x : d) s.dims.push_back(x.v); return s; }
    Status Add(DimensionHandle a, DimensionOrConstant b, DimensionHandle* out) { *out = DimensionHandle((a.v < 0 || b.v < 0) ? -1 : a.v + b.v); return Status::OK(); }
    Status Subtract(DimensionHandle a, DimensionOrConstant b, DimensionHandle* out) {
        if (a.v >= 0 && b.v >= 0 && a.v < b.v) return errors::InvalidArgument("Negative dimension size caused by subtracting ", b.v, " from ", a.v);
        *out = DimensionHandle(a.v < 0 ? -1 : a.v - b.v); return Status::OK();
    }
    Status Divide(DimensionHandle a, DimensionOrConstant b, bool evenly, DimensionHandle* out) {
        if (b.v <= 0) return errors::InvalidArgument("Divisor must be positive but is ", b.v);
        if (evenly && a.v >= 0 && a.v % b.v) return errors::InvalidArgument("Dimension size must be evenly divisible by ", b.v, " but is ", a.v);
        *out = DimensionHandle(a.v < 0 ? -1 : a.v / b.v); return Status::OK();
    }
    Status Multiply(DimensionHandle a, DimensionOrConstant b, DimensionHandle* out) { *out = DimensionHandle(a.v < 0 ? -1 : a.v * b.v); return Status::OK(); }

    const std::string* Find(const std::string& name) const { for (auto& kv : attrs) if (kv.first == name) return &kv.second; return nullptr; }
    Status GetAttr(const std::string& name, std::vector<int32>* out) const {
        const std::string* t = Find(name); if (!t) return errors::InvalidArgument("No attr named '", name, "'");
        out->clear(); std::stringstream ss(*t); std::string item;
        while (std::getline(ss, item, ',')) if (!item.empty()) out->push_back(std::atoi(item.c_str()));
        return Status::OK();
    }
    Status GetAttr(const std::string& name, int* out) const { const std::string* t = Find(name); if (!t) return errors::InvalidArgument("No attr named '", name, "'"); *out = std::atoi(t->c_str()); return Status::OK(); }
    Status GetAttr(const std::string& name, bool* out) const { const std::string* t = Find(name); if (!t) return errors::InvalidArgument("No attr named '", name, "'"); *out = (*t == "true" || *t == "1" || *t == "True"); return Status::OK(); }
    Status GetAttr(const std::string& name, float* out) const { const std::string* t = Find(name); if (!t) return errors::InvalidArgument("No attr named '", name, "'"); *out = float(std::atof(t->c_str())); return Status::OK(); }
    Status GetAttr(const std::string& name, std::string* out) const { const std::string* t = Find(name); if (!t) return errors::InvalidArgument("No attr named '", name, "'"); *out = *t; return Status::OK(); }
};
inline Status UnchangedShape(InferenceContext* c) { c->set_output(0, c->input(0)); return Status::OK(); }
}  // namespace shape_inference
}  // namespace tensorflow
#define TF_RETURN_IF_ERROR(expr) do { ::tensorflow::Status _s = (expr); if (!_s.ok()) return _s; } while (0)
#endif
