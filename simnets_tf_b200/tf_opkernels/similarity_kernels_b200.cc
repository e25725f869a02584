// TensorFlow GPU OpKernels of the Similarity op family on top of libsimnets_b200.
//
// These classes take the place of SimilarityKernelGPU / SimilarityInputGradKernelGPU /
// SimilarityParametersGradKernelGPU of the reference (src/kernels/similarity_kernel_gpu.cu:24-147,
// similarity_grad_kernel_gpu.cu:24-292).  Op registrations, attrs, shape functions and the Python wrappers of the
// reference stay as they are; attr parsing and validation stay in the reference's SimilarityKernelCommon
// (include/kernels/similarity_kernel_common.hpp), which this file includes from the reference checkout and derives
// from.  Only Compute() changes: no im2col buffer, no interlaced parameter buffer, one library call per op.
// The library never allocates: scratch comes from allocate_temp, launches go to TensorFlow's compute stream.
#include <cstdlib>
#include <type_traits>

#include "kernels/similarity_kernel_common.hpp"
#include "simnets_b200.h"

using namespace tensorflow;

namespace {

#define B200_REQUIRES_OK(ctx, rc) \
    OP_REQUIRES(ctx, (rc) == SIMNETS_OK, errors::Internal("simnets_b200: ", simnets_status_string(rc)))

// L2 with normalization_term and without ignore_nan_input: the reference's fast op adds the -0.5*K*log(2*pi) constant
// (batch - n) times to sample n (src/kernels/similarity_kernel_cpu.cpp:118-120), its SimilarityRef op once.  Default:
// once.  Set the environment variable SIMNETS_B200_LEGACY_BATCH_CONSTANT=1 before the kernels are constructed to
// reproduce the fast op bit for bit.
inline bool LegacyBatchConstant() {
    static const bool on = [] { const char* v = std::getenv("SIMNETS_B200_LEGACY_BATCH_CONSTANT"); return v && v[0] == '1'; }();
    return on;
}

class SimilarityB200Base : public SimilarityKernelCommon {
protected:
    explicit SimilarityB200Base(OpKernelConstruction* c) : SimilarityKernelCommon(c) {}

    template <typename T>
    simnets_sim_desc Describe(const Tensor& x, const Tensor& templates) const {
        simnets_sim_desc d = {};
        d.dtype = std::is_same<T, double>::value ? SIMNETS_F64 : SIMNETS_F32;
        d.batch = int32_t(x.dim_size(0)); d.channels = int32_t(x.dim_size(1));
        d.height = int32_t(x.dim_size(2)); d.width = int32_t(x.dim_size(3));
        d.num_instances = int32_t(templates.dim_size(0));
        d.block_h = blocks_[0]; d.block_w = blocks_[1];
        d.stride_h = stride_[0]; d.stride_w = stride_[1];
        d.pad_h = padding_[0]; d.pad_w = padding_[1];
        d.similarity_function = similarity_function_ == SIM_FUNC_L1 ? SIMNETS_SIM_L1 : SIMNETS_SIM_L2;
        d.normalization_term = normalization_term_; d.ignore_nan_input = ignore_nan_input_;
        d.normalization_term_fudge = normalization_term_fudge_; d.out_of_bounds_value = out_of_bounds_value_;
        d.flags = LegacyBatchConstant() ? SIMNETS_FLAG_SIM_BATCH_CONST_QUIRK : 0u;
        return d;
    }

    // shape checks the reference performs in CalculateDimensions (similarity_kernel_common.hpp:158-161)
    // plus the block extents: templates and weights are [num_instances, channels, block_h, block_w] with the attr's blocks
    bool ShapesAgree(const Tensor& x, const Tensor& t, const Tensor& w) const {
        return x.dims() == 4 && t.dims() == 4 && w.dims() == 4 && x.dim_size(1) == t.dim_size(1) && x.dim_size(1) == w.dim_size(1) &&
               t.dim_size(0) == w.dim_size(0) && t.dim_size(2) == blocks_[0] && t.dim_size(3) == blocks_[1] &&
               w.dim_size(2) == blocks_[0] && w.dim_size(3) == blocks_[1];
    }

    // output_grad: [batch, num_instances, height_out, width_out]
    static bool OutputGradAgrees(const Tensor& dy, const simnets_sim_desc& d) {
        int32_t oh = 0, ow = 0;
        if (simnets_similarity_output_dims(&d, &oh, &ow) != SIMNETS_OK) return false;
        return dy.dims() == 4 && dy.dim_size(0) == d.batch && dy.dim_size(1) == d.num_instances && dy.dim_size(2) == oh && dy.dim_size(3) == ow;
    }

    // scratch for one call, from TensorFlow's allocator
    static Status Workspace(OpKernelContext* ctx, const simnets_sim_desc& d, Tensor* ws, size_t* bytes) {
        *bytes = simnets_similarity_workspace_bytes(&d);
        return ctx->allocate_temp(DT_UINT8, TensorShape({int64(*bytes ? *bytes : 1)}), ws);
    }
};

template <typename T>
class SimilarityKernelB200 : public SimilarityB200Base {
public:
    explicit SimilarityKernelB200(OpKernelConstruction* c) : SimilarityB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &t = ctx->input(1), &w = ctx->input(2);
        OP_REQUIRES(ctx, ShapesAgree(x, t, w), errors::InvalidArgument("Number of channels mismatch between input and templates / weights"));
        const simnets_sim_desc d = Describe<T>(x, t);
        int32_t oh = 0, ow = 0;
        B200_REQUIRES_OK(ctx, simnets_similarity_output_dims(&d, &oh, &ow));
        Tensor* y = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({int64(d.batch), int64(d.num_instances), int64(oh), int64(ow)}), &y));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_similarity_forward(&d, x.flat<T>().data(), t.flat<T>().data(), w.flat<T>().data(),
                                                         y->flat<T>().data(), ws.flat<uint8>().data(), n, stream));
    }
};

template <typename T>
class SimilarityInputGradKernelB200 : public SimilarityB200Base {
public:
    explicit SimilarityInputGradKernelB200(OpKernelConstruction* c) : SimilarityB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &t = ctx->input(1), &w = ctx->input(2), &dy = ctx->input(3);
        OP_REQUIRES(ctx, ShapesAgree(x, t, w), errors::InvalidArgument("Number of channels mismatch between input and templates / weights"));
        const simnets_sim_desc d = Describe<T>(x, t);
        OP_REQUIRES(ctx, OutputGradAgrees(dy, d), errors::InvalidArgument("output_grad must have the shape of the op's output"));
        Tensor* dx = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &dx));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_similarity_input_grad(&d, x.flat<T>().data(), t.flat<T>().data(), w.flat<T>().data(),
                                                            dy.flat<T>().data(), dx->flat<T>().data(), ws.flat<uint8>().data(), n, stream));
    }
};

template <typename T>
class SimilarityParametersGradKernelB200 : public SimilarityB200Base {
public:
    explicit SimilarityParametersGradKernelB200(OpKernelConstruction* c) : SimilarityB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &t = ctx->input(1), &w = ctx->input(2), &dy = ctx->input(3);
        OP_REQUIRES(ctx, ShapesAgree(x, t, w), errors::InvalidArgument("Number of channels mismatch between input and templates / weights"));
        const simnets_sim_desc d = Describe<T>(x, t);
        OP_REQUIRES(ctx, OutputGradAgrees(dy, d), errors::InvalidArgument("output_grad must have the shape of the op's output"));
        Tensor *dt = nullptr, *dw = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, t.shape(), &dt));
        OP_REQUIRES_OK(ctx, ctx->allocate_output(1, w.shape(), &dw));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_similarity_params_grad(&d, x.flat<T>().data(), t.flat<T>().data(), w.flat<T>().data(),
                                                             dy.flat<T>().data(), dt->flat<T>().data(), dw->flat<T>().data(),
                                                             ws.flat<uint8>().data(), n, stream));
    }
};

}  // namespace

REGISTER_KERNEL_BUILDER(Name("Similarity").Device(DEVICE_GPU).TypeConstraint<float>("T"), SimilarityKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("Similarity").Device(DEVICE_GPU).TypeConstraint<double>("T"), SimilarityKernelB200<double>);
REGISTER_KERNEL_BUILDER(Name("SimilarityInputGrad").Device(DEVICE_GPU).TypeConstraint<float>("T"), SimilarityInputGradKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("SimilarityInputGrad").Device(DEVICE_GPU).TypeConstraint<double>("T"), SimilarityInputGradKernelB200<double>);
REGISTER_KERNEL_BUILDER(Name("SimilarityParametersGrad").Device(DEVICE_GPU).TypeConstraint<float>("T"), SimilarityParametersGradKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("SimilarityParametersGrad").Device(DEVICE_GPU).TypeConstraint<double>("T"), SimilarityParametersGradKernelB200<double>);
