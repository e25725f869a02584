// Test double, NOT TensorFlow (see op_kernel.h beside this file): REGISTER_OP and a registry of what was registered
// (name, inputs, outputs, attrs with their type text and default, shape function), enough to compile the reference's
// src/ops/*.cpp unchanged and to check their registrations and shape functions.
#ifndef TF_DOUBLE_OP_H
#define TF_DOUBLE_OP_H
#include <string>
#include <vector>
#include "tensorflow/core/framework/shape_inference.h"
namespace tensorflow {
struct OpAttrDef { std::string name, type, default_value; bool has_default; };
struct OpDefDouble {
    std::string name, doc;
    std::vector<std::string> inputs, outputs;
    std::vector<OpAttrDef> attrs;
    Status (*shape_fn)(shape_inference::InferenceContext*);
    OpDefDouble() : shape_fn(nullptr) {}
};
inline std::vector<OpDefDouble>& OpRegistryDouble() { static std::vector<OpDefDouble> r; return r; }
inline std::string TrimDouble(const std::string& s) {
    size_t a = s.find_first_not_of(" \t\n"), b = s.find_last_not_of(" \t\n");
    return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}
class OpDefBuilderWrapper {
public:
    explicit OpDefBuilderWrapper(const char* name) { def_.name = name; }
    OpDefBuilderWrapper& Input(const std::string& spec) { def_.inputs.push_back(spec); return *this; }
    OpDefBuilderWrapper& Output(const std::string& spec) { def_.outputs.push_back(spec); return *this; }
    OpDefBuilderWrapper& Attr(const std::string& spec) {        // "name: type" or "name: type = default"
        OpAttrDef a;
        const size_t colon = spec.find(':');
        a.name = TrimDouble(spec.substr(0, colon));
        std::string rest = spec.substr(colon + 1);
        // the default follows the last '=' that is outside braces ({'L1', 'L2'} = 'L2')
        int depth = 0; size_t eq = std::string::npos;
        for (size_t i = 0; i < rest.size(); ++i) { if (rest[i] == '{') ++depth; else if (rest[i] == '}') --depth; else if (rest[i] == '=' && depth == 0) eq = i; }
        a.has_default = eq != std::string::npos;
        a.type = TrimDouble(a.has_default ? rest.substr(0, eq) : rest);
        a.default_value = a.has_default ? TrimDouble(rest.substr(eq + 1)) : std::string();
        def_.attrs.push_back(a);
        return *this;
    }
    OpDefBuilderWrapper& SetShapeFn(Status (*fn)(shape_inference::InferenceContext*)) { def_.shape_fn = fn; return *this; }
    OpDefBuilderWrapper& Doc(const std::string& d) { def_.doc = d; return *this; }
    const OpDefDouble& def() const { return def_; }
private:
    OpDefDouble def_;
};
struct OpRegistrarDouble { OpRegistrarDouble(const OpDefBuilderWrapper& b) { OpRegistryDouble().push_back(b.def()); } };
}  // namespace tensorflow
#define TF_DOUBLE_CAT2(a, b) a##b
#define TF_DOUBLE_CAT(a, b) TF_DOUBLE_CAT2(a, b)
#define REGISTER_OP(name) static ::tensorflow::OpRegistrarDouble TF_DOUBLE_CAT(op_registrar_, __COUNTER__) = ::tensorflow::OpDefBuilderWrapper(name)
#endif
