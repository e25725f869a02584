// Test double, NOT TensorFlow: a small functional stand-in for the part of the OpKernel API that the reference's
// kernel classes (include/kernels/*_kernel_common.hpp, src/kernels/mex_kernel_common.cpp) and the B200 OpKernels in
// simnets_tf_b200/tf_opkernels use.  It lets those sources be compiled and RUN without TensorFlow: attrs come from a
// string map, tensors wrap caller-owned device pointers, allocate_output hands out caller-provided buffers,
// allocate_temp carves a caller-provided scratch block, kernels register in a process-wide table.
#ifndef TF_DOUBLE_OP_KERNEL_H
#define TF_DOUBLE_OP_KERNEL_H
#include <cassert>
#include <cstdlib>
#include <functional>
#include <initializer_list>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>
#include "tensorflow/core/framework/shape_inference.h"

namespace Eigen {
struct GpuDevice {
    void* stream_ = nullptr;
    void* stream() const { return stream_; }
};
}  // namespace Eigen

namespace tensorflow {
typedef unsigned char uint8;
enum DataType { DT_INVALID = 0, DT_FLOAT = 1, DT_DOUBLE = 2, DT_UINT8 = 4 };
template <typename T> struct DataTypeToEnum;
template <> struct DataTypeToEnum<float> { static const DataType value = DT_FLOAT; };
template <> struct DataTypeToEnum<double> { static const DataType value = DT_DOUBLE; };
template <> struct DataTypeToEnum<uint8> { static const DataType value = DT_UINT8; };
inline size_t DataTypeSize(DataType d) { return d == DT_DOUBLE ? 8 : (d == DT_FLOAT ? 4 : 1); }

class TensorShape {
public:
    TensorShape() {}
    TensorShape(std::initializer_list<int64> d) : d_(d) {}
    explicit TensorShape(const std::vector<int64>& d) : d_(d) {}
    void AddDim(int64 v) { d_.push_back(v); }
    int dims() const { return int(d_.size()); }
    int64 dim_size(int i) const { return d_[size_t(i)]; }
    int64 num_elements() const { int64 n = 1; for (int64 v : d_) n *= v; return n; }
    const std::vector<int64>& dim_sizes() const { return d_; }
private:
    std::vector<int64> d_;
};

template <typename T> struct FlatView {
    T* p; int64 n;
    T* data() const { return p; }
    int64 size() const { return n; }
};
template <typename T, int N> struct TensorView {
    T* p; int64 d[N];
    T* data() const { return p; }
    int64 dimension(int i) const { return d[i]; }
};

class Tensor {
public:
    Tensor() {}
    Tensor(DataType dt, const TensorShape& s, void* p) : dt_(dt), s_(s), p_(p) {}
    const TensorShape& shape() const { return s_; }
    int dims() const { return s_.dims(); }
    int64 dim_size(int i) const { return s_.dim_size(i); }
    int64 NumElements() const { return s_.num_elements(); }
    DataType dtype() const { return dt_; }
    void* raw() const { return p_; }
    template <typename T> FlatView<T> flat() const { return FlatView<T>{static_cast<T*>(p_), s_.num_elements()}; }
    template <typename T, int N> TensorView<T, N> tensor() const {
        TensorView<T, N> v; v.p = static_cast<T*>(p_);
        for (int i = 0; i < N; ++i) v.d[i] = i < s_.dims() ? s_.dim_size(i) : 1;
        return v;
    }
private:
    DataType dt_ = DT_INVALID; TensorShape s_; void* p_ = nullptr;
};

// attrs as text: ints / floats / bools as printed numbers ("1", "0.5", "inf"), lists comma separated, strings verbatim
class OpKernelConstruction {
public:
    explicit OpKernelConstruction(const std::map<std::string, std::string>& attrs) : attrs_(attrs) {}
    Status GetAttr(const char* name, int* v) const { std::string s; Status st = Find(name, &s); if (st.ok()) *v = std::atoi(s.c_str()); return st; }
    Status GetAttr(const char* name, float* v) const { std::string s; Status st = Find(name, &s); if (st.ok()) *v = std::strtof(s.c_str(), nullptr); return st; }
    Status GetAttr(const char* name, bool* v) const { std::string s; Status st = Find(name, &s); if (st.ok()) *v = std::atoi(s.c_str()) != 0; return st; }
    Status GetAttr(const char* name, std::string* v) const { return Find(name, v); }
    Status GetAttr(const char* name, std::vector<int>* v) const {
        std::string s; Status st = Find(name, &s); if (!st.ok()) return st;
        v->clear(); std::stringstream ss(s); std::string item;
        while (std::getline(ss, item, ',')) if (!item.empty()) v->push_back(std::atoi(item.c_str()));
        return st;
    }
    void SetStatus(const Status& s) { if (status_.ok()) status_ = s; }
    const Status& status() const { return status_; }
private:
    Status Find(const char* name, std::string* out) const {
        auto it = attrs_.find(name);
        if (it == attrs_.end()) return Status(std::string("attr not found: ") + name);
        *out = it->second; return Status::OK();
    }
    std::map<std::string, std::string> attrs_;
    Status status_;
};

class OpKernelContext {
public:
    std::vector<Tensor> inputs;            // set by the caller
    std::vector<void*> output_buffers;     // caller-owned memory for output i
    std::vector<Tensor> outputs;           // filled by allocate_output
    char* scratch = nullptr;               // caller-owned block for allocate_temp
    size_t scratch_bytes = 0, scratch_used = 0;
    Eigen::GpuDevice device;

    const Tensor& input(int i) const { return inputs[size_t(i)]; }
    Status allocate_output(int i, const TensorShape& shape, Tensor** out) {
        if (i < 0 || size_t(i) >= output_buffers.size()) return Status("no buffer for this output");
        if (outputs.size() < output_buffers.size()) outputs.resize(output_buffers.size());   // once: later calls must not move earlier outputs
        outputs[size_t(i)] = Tensor(inputs.empty() ? DT_FLOAT : inputs[0].dtype(), shape, output_buffers[size_t(i)]);
        *out = &outputs[size_t(i)];
        return Status::OK();
    }
    Status allocate_temp(DataType dt, const TensorShape& shape, Tensor* out) {
        const size_t bytes = (size_t(shape.num_elements()) * DataTypeSize(dt) + 255) & ~size_t(255);
        if (scratch_used + bytes > scratch_bytes) return Status("scratch block too small");
        *out = Tensor(dt, shape, scratch + scratch_used);
        scratch_used += bytes;
        return Status::OK();
    }
    template <typename D> const D& eigen_device() const { return device; }
    void SetStatus(const Status& s) { if (status_.ok()) status_ = s; }
    const Status& status() const { return status_; }
private:
    Status status_;
};

class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction*) {}
    virtual ~OpKernel() {}
    virtual void Compute(OpKernelContext*) {}
};

// ---- registration -------------------------------------------------------------------------------------------------
static const char* const DEVICE_GPU = "GPU";
static const char* const DEVICE_CPU = "CPU";
struct KernelDef { std::string name, device; DataType dtype = DT_INVALID; };
class Name {
public:
    explicit Name(const char* n) { def_.name = n; }
    Name& Device(const char* d) { def_.device = d; return *this; }
    template <typename T> Name& TypeConstraint(const char*) { def_.dtype = DataTypeToEnum<T>::value; return *this; }
    const KernelDef& def() const { return def_; }
private:
    KernelDef def_;
};
typedef std::function<OpKernel*(OpKernelConstruction*)> KernelFactory;
inline std::map<std::string, KernelFactory>& KernelRegistry() { static std::map<std::string, KernelFactory> r; return r; }
inline std::string KernelKey(const std::string& name, const std::string& device, DataType dt) {
    return name + "/" + device + "/" + (dt == DT_DOUBLE ? "double" : "float");
}
struct KernelRegistrar {
    KernelRegistrar(const Name& n, KernelFactory f) { KernelRegistry()[KernelKey(n.def().name, n.def().device, n.def().dtype)] = f; }
};
}  // namespace tensorflow

#define TF_DOUBLE_CAT2(a, b) a##b
#define TF_DOUBLE_CAT(a, b) TF_DOUBLE_CAT2(a, b)
#define REGISTER_KERNEL_BUILDER(builder, ...)                                                              \
    static ::tensorflow::KernelRegistrar TF_DOUBLE_CAT(tf_double_registrar_, __COUNTER__)(                 \
        ::tensorflow::builder, [](::tensorflow::OpKernelConstruction* c) -> ::tensorflow::OpKernel* { return new __VA_ARGS__(c); });
#define OP_REQUIRES_OK(ctx, expr) do { ::tensorflow::Status _s = (expr); if (!_s.ok()) { (ctx)->SetStatus(_s); return; } } while (0)
#define OP_REQUIRES(ctx, cond, status) do { if (!(cond)) { (ctx)->SetStatus(status); return; } } while (0)
#endif
