// Drives the B200 OpKernels (simnets_tf_b200/tf_opkernels/*.cc) through the TensorFlow test double in this folder:
// looks a kernel up in the double's registry, constructs it from textual attrs (the reference's own constructors parse
// and validate them), wraps caller-owned device buffers as tensors and calls Compute().  Host code only.
#include <cstring>
#include <map>
#include <memory>
#include <sstream>
#include <string>

#include "tensorflow/core/framework/op_kernel.h"

using namespace tensorflow;

namespace {
std::map<std::string, std::string> ParseAttrs(const char* text) {
    std::map<std::string, std::string> out;
    std::stringstream ss(text ? text : "");
    std::string item;
    while (std::getline(ss, item, ';')) {
        const size_t eq = item.find('=');
        if (eq != std::string::npos) out[item.substr(0, eq)] = item.substr(eq + 1);
    }
    return out;
}
void CopyMessage(const std::string& m, char* err, int errn) {
    if (!err || errn <= 0) return;
    std::strncpy(err, m.c_str(), size_t(errn - 1));
    err[errn - 1] = 0;
}
}  // namespace

extern "C" {

int tfk_count() { return int(KernelRegistry().size()); }

int tfk_has(const char* op, const char* device, int is_double) {
    return KernelRegistry().count(KernelKey(op, device, is_double ? DT_DOUBLE : DT_FLOAT)) ? 1 : 0;
}

// 0 = ran; 1 = the kernel's constructor rejected the attrs; 2 = Compute reported an error; 3 = no such kernel.
// in_dims / out_dims hold 5 entries per tensor (unused ones ignored / zeroed).
int tfk_run(const char* op, int is_double, const char* attrs, int n_in, void* const* in_ptrs, const int* in_ranks,
            const long long* in_dims, int n_out, void* const* out_ptrs, int* out_ranks, long long* out_dims, void* scratch,
            unsigned long long scratch_bytes, void* stream, char* err, int errn) {
    const DataType dt = is_double ? DT_DOUBLE : DT_FLOAT;
    auto it = KernelRegistry().find(KernelKey(op, DEVICE_GPU, dt));
    if (it == KernelRegistry().end()) { CopyMessage("kernel not registered", err, errn); return 3; }
    OpKernelConstruction construction(ParseAttrs(attrs));
    std::unique_ptr<OpKernel> kernel(it->second(&construction));
    if (!construction.status().ok()) { CopyMessage(construction.status().message(), err, errn); return 1; }
    OpKernelContext ctx;
    for (int i = 0; i < n_in; ++i) {
        std::vector<int64> dims(in_dims + 5 * i, in_dims + 5 * i + in_ranks[i]);
        ctx.inputs.push_back(Tensor(dt, TensorShape(dims), in_ptrs[i]));
    }
    ctx.output_buffers.assign(out_ptrs, out_ptrs + n_out);
    ctx.scratch = static_cast<char*>(scratch);
    ctx.scratch_bytes = size_t(scratch_bytes);
    ctx.device.stream_ = stream;
    kernel->Compute(&ctx);
    if (!ctx.status().ok()) { CopyMessage(ctx.status().message(), err, errn); return 2; }
    for (int i = 0; i < n_out; ++i) {
        out_ranks[i] = size_t(i) < ctx.outputs.size() ? ctx.outputs[size_t(i)].dims() : 0;
        for (int a = 0; a < 5; ++a) out_dims[5 * i + a] = a < out_ranks[i] ? ctx.outputs[size_t(i)].dim_size(a) : 0;
    }
    return 0;
}

}  // extern "C"
