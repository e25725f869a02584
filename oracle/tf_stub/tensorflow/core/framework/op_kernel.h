// Test double, NOT TensorFlow: just enough of OpKernel / OpKernelConstruction / OpKernelContext
// for the reference's src/kernels/mex_kernel_common.cpp to compile in place.  Only
// MexDimensionsData::CalculateDimensions() from that file is ever executed by the oracle.
#ifndef ORACLE_TF_STUB_OP_KERNEL_H
#define ORACLE_TF_STUB_OP_KERNEL_H
#include "tensorflow/core/framework/shape_inference.h"
namespace tensorflow {
class TensorShape { public: int64 dim_size(int) const { return 0; } };
class Tensor { public: const TensorShape& shape() const { return s_; } private: TensorShape s_; };
class OpKernelConstruction {
public:
    template <typename T> Status GetAttr(const char*, T*) const { return Status::OK(); }
    void SetStatus(const Status&) {}
};
class OpKernelContext {
public:
    const Tensor& input(int) const { return t_; }
    void SetStatus(const Status&) {}
private:
    Tensor t_;
};
class OpKernel {
public:
    explicit OpKernel(OpKernelConstruction*) {}
    virtual ~OpKernel() {}
};
}  // namespace tensorflow
#define OP_REQUIRES_OK(ctx, expr) do { ::tensorflow::Status _s = (expr); if (!_s.ok()) { (ctx)->SetStatus(_s); return; } } while (0)
#define OP_REQUIRES(ctx, cond, status) do { if (!(cond)) { (ctx)->SetStatus(status); return; } } while (0)
#endif
