// Reads the op registry of the TensorFlow test double after the reference's src/ops/*.cpp have registered their ops in it
// (compiled unchanged from a checkout), and runs their shape functions.  Host code only, no CUDA.
#include <cstring>
#include <sstream>
#include <string>

#include "tensorflow/core/framework/op.h"

using namespace tensorflow;

namespace {
void Copy(const std::string& m, char* out, int n) {
    if (!out || n <= 0) return;
    std::strncpy(out, m.c_str(), size_t(n - 1));
    out[n - 1] = 0;
}
const OpDefDouble* Find(const char* name) {
    for (auto& d : OpRegistryDouble()) if (d.name == name) return &d;
    return nullptr;
}
}  // namespace

extern "C" {

int tfop_count() { return int(OpRegistryDouble().size()); }

// One op as text: "name|in1;in2|out1|attr:type=default;attr:type|has_shape_fn"
int tfop_describe(int index, char* out, int n) {
    if (index < 0 || index >= tfop_count()) return 1;
    const OpDefDouble& d = OpRegistryDouble()[size_t(index)];
    std::ostringstream o;
    o << d.name << "|";
    for (size_t i = 0; i < d.inputs.size(); ++i) o << (i ? ";" : "") << d.inputs[i];
    o << "|";
    for (size_t i = 0; i < d.outputs.size(); ++i) o << (i ? ";" : "") << d.outputs[i];
    o << "|";
    for (size_t i = 0; i < d.attrs.size(); ++i) {
        o << (i ? ";" : "") << d.attrs[i].name << ":" << d.attrs[i].type;
        if (d.attrs[i].has_default) o << "=" << d.attrs[i].default_value;
    }
    o << "|" << (d.shape_fn ? 1 : 0);
    Copy(o.str(), out, n);
    return 0;
}

// Runs the op's shape function.  attrs: "name=value;..." (lists comma separated); shapes: 5 dims per tensor.
// 0 = ok, 1 = the shape function returned an error (message in err), 2 = no such op / no shape function.
int tfop_shape(const char* op, const char* attrs, int n_in, const int* in_ranks, const long long* in_dims,
               int max_out, int* n_out, int* out_ranks, long long* out_dims, char* err, int errn) {
    const OpDefDouble* d = Find(op);
    if (!d || !d->shape_fn) { Copy("no such op or no shape function", err, errn); return 2; }
    shape_inference::InferenceContext c;
    for (int i = 0; i < n_in; ++i) {
        shape_inference::ShapeHandle s;
        s.known = true;
        s.dims.assign(in_dims + 5 * i, in_dims + 5 * i + in_ranks[i]);
        c.inputs.push_back(s);
    }
    // defaults of the registration first, then the caller's values
    for (auto& a : d->attrs) {
        if (!a.has_default) continue;
        std::string v = a.default_value;
        std::string clean;
        for (char ch : v) if (ch != '[' && ch != ']' && ch != '\'' && ch != ' ') clean += ch;
        c.attrs.push_back(std::make_pair(a.name, clean));
    }
    std::stringstream ss(attrs ? attrs : "");
    std::string item;
    while (std::getline(ss, item, ';')) {
        const size_t eq = item.find('=');
        if (eq == std::string::npos) continue;
        const std::string k = item.substr(0, eq), v = item.substr(eq + 1);
        bool found = false;
        for (auto& kv : c.attrs) if (kv.first == k) { kv.second = v; found = true; }
        if (!found) c.attrs.push_back(std::make_pair(k, v));
    }
    const Status st = d->shape_fn(&c);
    if (!st.ok()) { Copy(st.message(), err, errn); return 1; }
    *n_out = int(c.outputs.size());
    for (int i = 0; i < *n_out && i < max_out; ++i) {
        out_ranks[i] = int(c.outputs[size_t(i)].dims.size());
        for (int j = 0; j < out_ranks[i] && j < 5; ++j) out_dims[5 * i + j] = c.outputs[size_t(i)].dims[size_t(j)];
    }
    return 0;
}

}  // extern "C"
