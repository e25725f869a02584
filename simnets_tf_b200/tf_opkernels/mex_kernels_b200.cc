// TensorFlow GPU OpKernels of the Mex op family on top of libsimnets_b200.
//
// These classes take the place of MEXKernelGPU / MEXGradInputKernelGPU / MEXGradOffsetsKernelGPU of the reference
// (src/kernels/mex_kernel_gpu.cu:60-171, mex_grad_kernel_gpu.cu:23-395).  Attr parsing and validation stay in the
// reference's MEXKernelCommon (include/kernels/mex_kernel_common.hpp, src/kernels/mex_kernel_common.cpp:29-58), which
// this file derives from; the library resolves -1 in padding / strides and derives the region geometry itself
// (simnets_mex_dims), exactly as MexDimensionsData::CalculateDimensions does, so no patch, split-patch or padded
// offsets buffer is allocated: one scratch block from allocate_temp, one library call per op.
#include <type_traits>

#include "kernels/mex_kernel_common.hpp"
#include "simnets_b200.h"

using namespace tensorflow;

namespace {

#define B200_REQUIRES_OK(ctx, rc) \
    OP_REQUIRES(ctx, (rc) == SIMNETS_OK, errors::Internal("simnets_b200: ", simnets_status_string(rc)))

class MexB200Base : public MEXKernelCommon {
protected:
    explicit MexB200Base(OpKernelConstruction* c) : MEXKernelCommon(c) {}

    template <typename T>
    simnets_mex_desc Describe(const Tensor& x) const {
        simnets_mex_desc d = {};
        d.dtype = std::is_same<T, double>::value ? SIMNETS_F64 : SIMNETS_F32;
        d.batch = int32_t(x.dim_size(0)); d.channels = int32_t(x.dim_size(1));
        d.height = int32_t(x.dim_size(2)); d.width = int32_t(x.dim_size(3));
        d.num_instances = num_instances_;
        // padding: three entries; a pair [h, w] means [-1, h, w], as the reference's ExpandDimSpec turns it
        // (src/kernels/mex_kernel_common.cpp:8-27); -1 is resolved by the library to the image extent.  Other lengths
        // index past the end in the reference; here Compute() rejects them (PaddingOk) before this function runs.
        int32_t pad3[3] = {0, 0, 0};
        if (padding_.size() == 3) { pad3[0] = padding_[0]; pad3[1] = padding_[1]; pad3[2] = padding_[2]; }
        else if (padding_.size() == 2) { pad3[0] = -1; pad3[1] = padding_[0]; pad3[2] = padding_[1]; }
        for (int a = 0; a < 3; ++a) {
            d.blocks[a] = blocks_[size_t(a)];
            d.strides[a] = strides_[size_t(a)];
            d.padding[a] = pad3[a];
        }
        d.epsilon = epsilon_; d.softmax_mode = softmax_mode_;
        d.blocks_out_of_bounds_value = blocks_out_of_bounds_value_;
        d.blocks_round_down = blocks_round_down_; d.use_unshared_regions = use_unshared_regions_;
        d.n_shared_offset_region = int32_t(shared_offset_region_.size());
        for (size_t a = 0; a < shared_offset_region_.size() && a < 3; ++a) d.shared_offset_region[a] = shared_offset_region_[a];
        d.n_unshared_offset_region = int32_t(unshared_offset_region_.size());
        for (size_t a = 0; a < unshared_offset_region_.size() && a < 3; ++a) d.unshared_offset_region[a] = unshared_offset_region_[a];
        return d;
    }

    bool PaddingOk() const { return padding_.size() == 2 || padding_.size() == 3; }

    // offsets: [num_regions, num_instances, block_c, block_h, block_w] (mex_kernel_common.cpp:60-61)
    static bool OffsetsAgree(const Tensor& offsets, const simnets_mex_geometry& g, int num_instances) {
        return offsets.dims() == 5 && offsets.dim_size(0) == g.num_regions && offsets.dim_size(1) == num_instances &&
               offsets.dim_size(2) == g.block_c && offsets.dim_size(3) == g.block_h && offsets.dim_size(4) == g.block_w;
    }

    // orig_output and output_grad: [batch, num_instances * channels_out, height_out, width_out]; a wrong shape must be an
    // InvalidArgument, not an out-of-bounds device read
    static bool OutputAgrees(const Tensor& t, const simnets_mex_desc& d, const simnets_mex_geometry& g) {
        return t.dims() == 4 && t.dim_size(0) == d.batch && t.dim_size(1) == g.channels_out_total && t.dim_size(2) == g.height_out &&
               t.dim_size(3) == g.width_out;
    }

    static Status Workspace(OpKernelContext* ctx, const simnets_mex_desc& d, Tensor* ws, size_t* bytes) {
        *bytes = simnets_mex_workspace_bytes(&d);
        return ctx->allocate_temp(DT_UINT8, TensorShape({int64(*bytes ? *bytes : 1)}), ws);
    }
};

template <typename T>
class MexKernelB200 : public MexB200Base {
public:
    explicit MexKernelB200(OpKernelConstruction* c) : MexB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &offsets = ctx->input(1);
        OP_REQUIRES(ctx, x.dims() == 4, errors::InvalidArgument("input must be 4-dimensional"));
        OP_REQUIRES(ctx, PaddingOk(), errors::InvalidArgument("padding should be a list with 2 or 3 elements"));
        const simnets_mex_desc d = Describe<T>(x);
        simnets_mex_geometry g;
        B200_REQUIRES_OK(ctx, simnets_mex_dims(&d, &g));
        OP_REQUIRES(ctx, OffsetsAgree(offsets, g, num_instances_), errors::InvalidArgument("offsets must be [num_regions, num_instances, block_c, block_h, block_w]"));
        Tensor* y = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, TensorShape({int64(d.batch), int64(g.channels_out_total), int64(g.height_out), int64(g.width_out)}), &y));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_mex_forward(&d, x.flat<T>().data(), offsets.flat<T>().data(), y->flat<T>().data(),
                                                  ws.flat<uint8>().data(), n, stream));
    }
};

template <typename T>
class MexInputGradKernelB200 : public MexB200Base {
public:
    explicit MexInputGradKernelB200(OpKernelConstruction* c) : MexB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &offsets = ctx->input(1), &y = ctx->input(2), &dy = ctx->input(3);
        OP_REQUIRES(ctx, x.dims() == 4, errors::InvalidArgument("input must be 4-dimensional"));
        OP_REQUIRES(ctx, PaddingOk(), errors::InvalidArgument("padding should be a list with 2 or 3 elements"));
        const simnets_mex_desc d = Describe<T>(x);
        simnets_mex_geometry g;
        B200_REQUIRES_OK(ctx, simnets_mex_dims(&d, &g));
        OP_REQUIRES(ctx, OffsetsAgree(offsets, g, num_instances_), errors::InvalidArgument("offsets must be [num_regions, num_instances, block_c, block_h, block_w]"));
        OP_REQUIRES(ctx, OutputAgrees(y, d, g), errors::InvalidArgument("orig_output must have the shape of the op's output"));
        OP_REQUIRES(ctx, OutputAgrees(dy, d, g), errors::InvalidArgument("output_grad must have the shape of the op's output"));
        Tensor* dx = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, x.shape(), &dx));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_mex_input_grad(&d, x.flat<T>().data(), offsets.flat<T>().data(), y.flat<T>().data(), dy.flat<T>().data(),
                                                     dx->flat<T>().data(), ws.flat<uint8>().data(), n, stream));
    }
};

template <typename T>
class MexOffsetsGradKernelB200 : public MexB200Base {
public:
    explicit MexOffsetsGradKernelB200(OpKernelConstruction* c) : MexB200Base(c) {}
    void Compute(OpKernelContext* ctx) override {
        const Tensor &x = ctx->input(0), &offsets = ctx->input(1), &y = ctx->input(2), &dy = ctx->input(3);
        OP_REQUIRES(ctx, x.dims() == 4, errors::InvalidArgument("input must be 4-dimensional"));
        OP_REQUIRES(ctx, PaddingOk(), errors::InvalidArgument("padding should be a list with 2 or 3 elements"));
        const simnets_mex_desc d = Describe<T>(x);
        simnets_mex_geometry g;
        B200_REQUIRES_OK(ctx, simnets_mex_dims(&d, &g));
        OP_REQUIRES(ctx, OffsetsAgree(offsets, g, num_instances_), errors::InvalidArgument("offsets must be [num_regions, num_instances, block_c, block_h, block_w]"));
        OP_REQUIRES(ctx, OutputAgrees(y, d, g), errors::InvalidArgument("orig_output must have the shape of the op's output"));
        OP_REQUIRES(ctx, OutputAgrees(dy, d, g), errors::InvalidArgument("output_grad must have the shape of the op's output"));
        Tensor* doff = nullptr;
        OP_REQUIRES_OK(ctx, ctx->allocate_output(0, offsets.shape(), &doff));
        Tensor ws; size_t n = 0;
        OP_REQUIRES_OK(ctx, Workspace(ctx, d, &ws, &n));
        void* stream = (void*)ctx->template eigen_device<Eigen::GpuDevice>().stream();
        B200_REQUIRES_OK(ctx, simnets_mex_offsets_grad(&d, x.flat<T>().data(), offsets.flat<T>().data(), y.flat<T>().data(), dy.flat<T>().data(),
                                                       doff->flat<T>().data(), ws.flat<uint8>().data(), n, stream));
    }
};

}  // namespace

REGISTER_KERNEL_BUILDER(Name("Mex").Device(DEVICE_GPU).TypeConstraint<float>("T"), MexKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("Mex").Device(DEVICE_GPU).TypeConstraint<double>("T"), MexKernelB200<double>);
REGISTER_KERNEL_BUILDER(Name("MexInputGrad").Device(DEVICE_GPU).TypeConstraint<float>("T"), MexInputGradKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("MexInputGrad").Device(DEVICE_GPU).TypeConstraint<double>("T"), MexInputGradKernelB200<double>);
REGISTER_KERNEL_BUILDER(Name("MexOffsetsGrad").Device(DEVICE_GPU).TypeConstraint<float>("T"), MexOffsetsGradKernelB200<float>);
REGISTER_KERNEL_BUILDER(Name("MexOffsetsGrad").Device(DEVICE_GPU).TypeConstraint<double>("T"), MexOffsetsGradKernelB200<double>);
