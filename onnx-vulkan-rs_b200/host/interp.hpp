// Node-level host layer above the C ABI: the counterpart of the reference's
// operator functions in crates/onnx-vulkan-core/src/interp.rs for the
// quantized matrix-product path.  It mirrors their interface - a node with
// named inputs/outputs and attributes, an environment mapping names to
// tensors, weights prepared once per session and cached by initializer name -
// and calls nothing but the functions declared in ovk_cuda.h.
//
//   reference                                   here
//   NodeIr / AttrValue   (src/graph.rs:149,197) ovk::host::NodeIr / AttrValue
//   ExecutionEnv         (src/execution.rs:15)  ovk::host::Env
//   KernelCache::packed_weight (src/cache.rs:231) Env's weight caches
//   is_implemented_node  (src/interp.rs:338)    is_implemented_node
//   unsupported_quantization (src/interp.rs:781) unsupported_quantization
//   exec_dispatch        (src/interp.rs:1071)   exec_dispatch
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "ovk_cuda.h"

namespace ovk {
namespace host {

struct AttrValue {
    enum Kind { Int, Ints, Str } kind = Int;
    int64_t i = 0;
    std::vector<int64_t> ints;
    std::string s;
};

struct NodeIr {
    std::string domain, op, name;
    std::vector<std::string> inputs, outputs;
    std::map<std::string, AttrValue> attrs;
    int64_t int_attr(const std::string &key, int64_t fallback) const;
    std::vector<int64_t> ints_attr(const std::string &key) const;
    std::string str_attr(const std::string &key, const std::string &fallback) const;
    bool present(size_t index) const { return index < inputs.size() && !inputs[index].empty(); }
};

// A tensor of the environment: always resident on the device; constants
// (initializers) also keep their host bytes, which is what lets quantization
// parameters be read without a device round trip, as the reference reads them
// from the graph's initializers.
struct Tensor {
    int32_t dtype = 0;  // ElementType code (src/graph.rs:13-41)
    std::vector<int64_t> shape;
    void *dev = nullptr;
    size_t bytes = 0;
    bool initializer = false;
    bool spent = false;  // a folded range that its one DynamicQuantizeLinear has consumed
    std::vector<uint8_t> host;
    int64_t elem_count() const;
};

// core::Error (src/error.rs:6-14) flattened to a status + message, nothing throws.
struct Result {
    int32_t status = OVK_OK;
    std::string message;
    bool ok() const { return status == OVK_OK; }
};

class Env {
public:
    explicit Env(ovk_ctx *ctx) : ctx_(ctx) {}
    ~Env();
    Env(const Env &) = delete;
    Env &operator=(const Env &) = delete;

    ovk_ctx *context() const { return ctx_; }
    // env.set with a host tensor: uploaded at once (ExecutionEnv::ensure_device_dtype, execution.rs:391)
    Result set(const std::string &name, int32_t dtype, const std::vector<int64_t> &shape, const void *data,
               size_t bytes, bool initializer);
    // a fresh device tensor owned by the environment
    Result alloc(const std::string &name, int32_t dtype, const std::vector<int64_t> &shape, Tensor **out);
    const Tensor *find(const std::string &name) const;
    // env.host(name): download (flushes, like stream_download)
    Result host(const std::string &name, std::vector<uint8_t> *out, int32_t *dtype, std::vector<int64_t> *shape);
    void release(const std::string &name);
    // which kernel the last dispatched node selected (the role of KernelCache::pipeline_keys)
    std::string last_kernel() const;

    // weights prepared once per session, keyed by initializer name (cache.rs:231)
    std::map<std::string, ovk_nbits_weight *> nbits_weights;
    std::map<std::string, ovk_mmi_weight *> mmi_weights;
    std::map<std::string, ovk_qconv_weight *> qconv_weights;
    // MatMulNBits weight name -> the scale and zero-point tensors its object points into
    std::map<std::string, std::pair<std::string, std::string>> nbits_deps;

private:
    ovk_ctx *ctx_;
    std::map<std::string, Tensor> tensors_;
};

size_t dtype_size(int32_t dtype);

// The claim predicate: which nodes of the path this layer takes (interp.rs:338, :452-464, :560-572).
bool is_implemented_node(const NodeIr &node);
// Load-time refusal of quantization forms the kernels do not cover, with the
// reference's wording (interp.rs:781-847).  Empty string = supported.
std::string unsupported_quantization(const NodeIr &node, const Env &env);
// Runs one node: reads its inputs from the environment, enqueues, sets its
// outputs.  No host synchronisation inside (interp.rs:1071-1196).
Result exec_dispatch(Env &env, const NodeIr &node);

}  // namespace host
}  // namespace ovk
