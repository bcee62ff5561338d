// Node-level host layer above the C ABI (see interp.hpp).  Every function
// names the reference function it mirrors (crates/onnx-vulkan-core/src/).
#include "interp.hpp"

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace ovk {
namespace host {

namespace {

Result fail(int32_t status, const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return Result{status, buf};
}

Result from_abi(ovk_ctx *ctx, int32_t rc)
{
    if (rc == OVK_OK)
        return Result{};
    return Result{rc, ovk_last_error(ctx)};
}

#define OVKH_TRY(expr)       \
    do {                     \
        Result r_ = (expr);  \
        if (!r_.ok())        \
            return r_;       \
    } while (0)

#define OVKH_ENSURE(cond, ...)                            \
    do {                                                  \
        if (!(cond))                                      \
            return fail(OVK_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

int64_t product(const std::vector<int64_t> &shape, size_t begin, size_t end)
{
    int64_t p = 1;
    for (size_t i = begin; i < end; i++)
        p *= shape[i];
    return p < 0 ? 0 : p;
}

// one scalar of a constant, sign handled by dtype (zp_value, interp.rs:4697-4705)
Result scalar_i32(const Env &env, const std::string &name, const char *what, int32_t *out)
{
    const Tensor *t = env.find(name);
    OVKH_ENSURE(t, "%s: %s is not in the environment", what, name.c_str());
    OVKH_ENSURE(t->elem_count() == 1, "QLinear: zero point of %s is not per-tensor (%lld values)", name.c_str(),
                (long long)t->elem_count());
    OVKH_ENSURE(!t->host.empty(), "%s: %s is not a constant", what, name.c_str());
    if (t->dtype == OVK_INT8)
        *out = int8_t(t->host[0]);
    else if (t->dtype == OVK_UINT8)
        *out = t->host[0];
    else if (t->dtype == OVK_INT32)
        memcpy(out, t->host.data(), 4);
    else
        return fail(OVK_INVALID_ARGUMENT, "%s: %s has dtype %d", what, name.c_str(), t->dtype);
    return Result{};
}

Result floats_of(const Env &env, const std::string &name, const char *what, std::vector<float> *out)
{
    const Tensor *t = env.find(name);
    OVKH_ENSURE(t, "%s: %s is not in the environment", what, name.c_str());
    OVKH_ENSURE(t->dtype == OVK_FLOAT && !t->host.empty(), "%s: %s is not a float32 constant", what, name.c_str());
    out->resize(size_t(t->elem_count()));
    memcpy(out->data(), t->host.data(), out->size() * 4);
    return Result{};
}

// requantize_ratio (interp.rs:4682-4694): x_scale * w_scale[c] / y_scale in f32, left to right
Result requantize_ratio(const Env &env, const std::string &x_scale, const std::string &w_scale,
                        const std::string &y_scale, std::vector<float> *ratio)
{
    std::vector<float> x, w, y;
    OVKH_TRY(floats_of(env, x_scale, "QLinear", &x));
    OVKH_TRY(floats_of(env, w_scale, "QLinear", &w));
    OVKH_TRY(floats_of(env, y_scale, "QLinear", &y));
    OVKH_ENSURE(x.size() == 1 && y.size() == 1, "QLinear: activation scales must be per-tensor (x %zu, y %zu)", x.size(),
                y.size());
    OVKH_ENSURE(y[0] != 0.0f, "QLinear: y_scale is zero");
    ratio->clear();
    for (float ws : w) {
        volatile float p = x[0] * ws;
        ratio->push_back(p / y[0]);
    }
    return Result{};
}

// column_step (interp.rs:2600-2610): 0 one value, 1 one per column, -1 anything else
int column_step(const std::vector<int64_t> &shape, int64_t n, size_t rank)
{
    if (shape.size() > rank)
        return -1;
    for (size_t i = 0; i + 1 < shape.size(); i++)
        if (shape[i] != 1)
            return -1;
    if (shape.empty() || shape.back() == 1)
        return 0;
    return shape.back() == n ? 1 : -1;
}

// How an operand of shape `shape` broadcasts over an output [.., rows, n] whose leading dimensions are
// folded into `rows`: (row stride, column stride) in elements, or false when it does neither of one
// value / one per column / one per row / a full matrix.
bool broadcast_strides(const std::vector<int64_t> &shape, const std::vector<int64_t> &out_shape, int64_t *rs, int64_t *cs)
{
    if (shape.size() > out_shape.size())
        return false;
    const int64_t n = out_shape.back();
    const int64_t last = shape.empty() ? 1 : shape.back();
    if (last != 1 && last != n)
        return false;
    *cs = last == n && n != 1 ? 1 : 0;
    bool all_one = true, all_equal = true;
    const size_t lead = out_shape.size() - 1, have = shape.empty() ? 0 : shape.size() - 1;
    for (size_t i = 0; i < lead; i++) {  // leading dimensions, right-aligned
        const int64_t od = out_shape[lead - 1 - i];
        const int64_t sd = i < have ? shape[have - 1 - i] : 1;
        all_one = all_one && sd == 1;
        all_equal = all_equal && sd == od;
    }
    if (all_one) {
        *rs = 0;
        return true;
    }
    if (!all_equal)
        return false;
    *rs = *cs ? n : 1;
    return true;
}

// ------------------------------------------------------------------ MatMulNBits
// interp::matmul_nbits (interp.rs:6429-6561)
Result matmul_nbits(Env &env, const NodeIr &node)
{
    const int64_t k = node.int_attr("K", 0), n = node.int_attr("N", 0), bs = node.int_attr("block_size", 0);
    const Tensor *a = env.find(node.inputs[0]);
    const Tensor *quant = env.find(node.inputs[1]);
    const Tensor *scales = env.find(node.inputs[2]);
    const Tensor *zp = node.present(3) ? env.find(node.inputs[3]) : nullptr;
    OVKH_ENSURE(a && quant && scales && (zp || !node.present(3)), "MatMulNBits: an input is missing");
    OVKH_ENSURE(!a->shape.empty(), "MatMulNBits: A is a scalar");
    OVKH_ENSURE(a->shape.back() == k, "MatMulNBits: A's last dimension Some(%lld) disagrees with K=%lld",
                (long long)a->shape.back(), (long long)k);
    OVKH_ENSURE(quant->dtype == OVK_UINT8 && (!zp || zp->dtype == OVK_UINT8) &&
                    (scales->dtype == OVK_FLOAT || scales->dtype == OVK_FLOAT16),
                "MatMulNBits: expected u8 weight and zero point with f32 scales, got %d/%d/%d", quant->dtype,
                zp ? zp->dtype : OVK_UINT8, scales->dtype);
    const int64_t n_blocks = (k + bs - 1) / bs;
    OVKH_ENSURE(quant->elem_count() >= n * n_blocks * (bs / 8) * 4 && scales->elem_count() >= n * n_blocks &&
                    (!zp || zp->elem_count() >= n * ((n_blocks + 1) / 2)),
                "MatMulNBits: packed weight is short for K=%lld N=%lld block_size=%lld", (long long)k, (long long)n,
                (long long)bs);
    const int64_t rows = product(a->shape, 0, a->shape.size() - 1);
    auto it = env.nbits_weights.find(node.inputs[1]);
    if (it == env.nbits_weights.end()) {
        ovk_nbits_weight *w = nullptr;
        OVKH_TRY(from_abi(env.context(), ovk_nbits_prepack(env.context(), quant->dev, scales->dev, scales->dtype,
                                                            zp ? zp->dev : nullptr, n, k, node.int_attr("bits", 0), bs,
                                                            OVK_NBITS_DEFAULT, &w)));
        it = env.nbits_weights.emplace(node.inputs[1], w).first;
        // the weight object points into the scale and zero-point tensors too
        env.nbits_deps[node.inputs[1]] = {node.inputs[2], zp ? node.inputs[3] : std::string()};
    }
    std::vector<int64_t> out_shape(a->shape.begin(), a->shape.end() - 1);
    out_shape.push_back(n);
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], a->dtype, out_shape, &out));
    a = env.find(node.inputs[0]);  // alloc may have rehashed nothing, but keep the pointer fresh
    return from_abi(env.context(), ovk_matmul_nbits(env.context(), it->second, a->dev, a->dtype, rows, out->dev, a->dtype));
}

// ------------------------------------------------------- DynamicQuantizeLinear
// interp::dynamic_quantize (interp.rs:1945-1970)
Result dynamic_quantize(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    OVKH_ENSURE(x && x->dtype == OVK_FLOAT, "DynamicQuantizeLinear: x must be float32");
    const std::vector<int64_t> shape = x->shape;
    const int64_t count = x->elem_count();
    Tensor *y = nullptr, *scale = nullptr, *zp = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_UINT8, shape, &y));
    OVKH_TRY(env.alloc(node.outputs[1], OVK_FLOAT, {}, &scale));
    OVKH_TRY(env.alloc(node.outputs[2], OVK_UINT8, {}, &zp));
    x = env.find(node.inputs[0]);
    // the producer of x may have folded its range into a slot (ExecutionEnv::computed_range,
    // execution.rs:112): the range pass is then skipped (interp.rs:1979-1983)
    const Tensor *folded = env.find(node.inputs[0] + "/range");
    if (folded && !folded->spent && count > 0) {
        Result r = from_abi(env.context(),
                            ovk_dynamic_quantize_folded(env.context(), static_cast<const float *>(x->dev), count,
                                                        static_cast<uint32_t *>(folded->dev), static_cast<uint8_t *>(y->dev),
                                                        static_cast<float *>(scale->dev), static_cast<uint8_t *>(zp->dev)));
        // the quantize pass leaves the slot zero: a second quantization of the same tensor finds its range itself
        const_cast<Tensor *>(folded)->spent = true;
        return r;
    }
    return from_abi(env.context(),
                    ovk_dynamic_quantize(env.context(), static_cast<const float *>(x->dev), count,
                                         static_cast<uint8_t *>(y->dev), static_cast<float *>(scale->dev),
                                         static_cast<uint8_t *>(zp->dev)));
}

// ---------------------------------------------- DecomposedGelu, DecomposedGeluQuantize
Result scalar_f32(const Env &env, const std::string &name, const char *what, float *out);

// interp::gelu_push (interp.rs:9094-9116): the three constants of the GELU, each one f32 value read
// on the host; anything else is the form the reference replays as five elementwise nodes, which are
// outside this layer.
Result gelu_constants(const Env &env, const NodeIr &node, float (&c)[3])
{
    const Tensor *x = env.find(node.inputs[0]);
    OVKH_ENSURE(x, "%s: x is missing", node.op.c_str());
    bool fusable = x->dtype == OVK_FLOAT;
    for (int i = 0; i < 3 && fusable; i++) {
        const Tensor *t = env.find(node.inputs[1 + i]);
        OVKH_ENSURE(t, "%s: input %d is missing", node.op.c_str(), 1 + i);
        fusable = t->dtype == OVK_FLOAT && t->elem_count() == 1 && !t->host.empty();
    }
    if (!fusable)
        return fail(OVK_UNSUPPORTED,
                    "%s: not one pass (a non-f32 operand, or a constant that is not one value known on the host): the "
                    "reference replays Div, Erf, Add, Mul, Mul here",
                    node.op.c_str());
    for (int i = 0; i < 3; i++)
        OVKH_TRY(scalar_f32(env, node.inputs[1 + i], node.op.c_str(), &c[i]));
    return Result{};
}

// interp::decomposed_gelu (interp.rs:9039-9084)
Result decomposed_gelu(Env &env, const NodeIr &node)
{
    float c[3];
    OVKH_TRY(gelu_constants(env, node, c));
    const Tensor *x = env.find(node.inputs[0]);
    const std::vector<int64_t> shape = x->shape;
    const int64_t count = x->elem_count();
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, shape, &out));
    x = env.find(node.inputs[0]);
    return from_abi(env.context(),
                    ovk_decomposed_gelu(env.context(), static_cast<const float *>(x->dev), count, c[0], c[1], c[2],
                                        node.int_attr("factor_first", 0) == 1, static_cast<float *>(out->dev)));
}

// interp::decomposed_gelu_quantize (interp.rs:9125-9150): the GELU's inputs and attributes, the
// quantization's three outputs
Result decomposed_gelu_quantize(Env &env, const NodeIr &node)
{
    float c[3];
    OVKH_TRY(gelu_constants(env, node, c));
    const Tensor *x = env.find(node.inputs[0]);
    const std::vector<int64_t> shape = x->shape;
    const int64_t count = x->elem_count();
    Tensor *y = nullptr, *scale = nullptr, *zp = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_UINT8, shape, &y));
    OVKH_TRY(env.alloc(node.outputs[1], OVK_FLOAT, {}, &scale));
    OVKH_TRY(env.alloc(node.outputs[2], OVK_UINT8, {}, &zp));
    x = env.find(node.inputs[0]);
    return from_abi(env.context(),
                    ovk_decomposed_gelu_quantize(env.context(), static_cast<const float *>(x->dev), count, c[0], c[1], c[2],
                                                 node.int_attr("factor_first", 0) == 1, static_cast<uint8_t *>(y->dev),
                                                 static_cast<float *>(scale->dev), static_cast<uint8_t *>(zp->dev)));
}

// --------------------------------------------------------------- MatMulInteger
Result mmi_weight(Env &env, const std::string &b_name, int64_t k, ovk_mmi_weight **out, int64_t *n)
{
    const Tensor *b = env.find(b_name);
    OVKH_ENSURE(b, "MatMulInteger: B is missing");
    OVKH_ENSURE(b->shape.size() == 2, "MatMulInteger: B rank %zu != 2", b->shape.size());
    OVKH_ENSURE(b->shape[0] == k, "MatMulInteger: K mismatch (A %lld, B %lld)", (long long)k, (long long)b->shape[0]);
    OVKH_ENSURE(b->dtype == OVK_UINT8 || b->dtype == OVK_INT8, "MatMulInteger: B has dtype %d", b->dtype);
    *n = b->shape[1];
    auto it = env.mmi_weights.find(b_name);  // packed_b: once per weight name (interp.rs:2712-2768)
    if (it == env.mmi_weights.end()) {
        ovk_mmi_weight *w = nullptr;
        OVKH_TRY(from_abi(env.context(), ovk_mmi_prepack(env.context(), b->dev, b->dtype == OVK_INT8, k, *n, &w)));
        it = env.mmi_weights.emplace(b_name, w).first;
    }
    *out = it->second;
    return Result{};
}

Result scalar_zp_dev(const Env &env, const NodeIr &node, size_t index, const void **dev)
{
    *dev = nullptr;
    if (!node.present(index))
        return Result{};
    const Tensor *t = env.find(node.inputs[index]);
    OVKH_ENSURE(t, "MatMulInteger: zero point %s is missing", node.inputs[index].c_str());
    OVKH_ENSURE(t->elem_count() == 1, "MatMulInteger: only per-tensor zero points");
    *dev = t->dev;
    return Result{};
}

// interp::matmul_integer (interp.rs:2090-2183)
Result matmul_integer(Env &env, const NodeIr &node)
{
    const Tensor *a = env.find(node.inputs[0]);
    OVKH_ENSURE(a, "MatMulInteger: A is missing");
    OVKH_ENSURE(a->shape.size() >= 2, "MatMulInteger: A rank %zu < 2", a->shape.size());
    OVKH_ENSURE(a->dtype == OVK_UINT8 || a->dtype == OVK_INT8, "MatMulInteger: A has dtype %d", a->dtype);
    const int64_t k = a->shape.back(), m = product(a->shape, 0, a->shape.size() - 1);
    ovk_mmi_weight *w = nullptr;
    int64_t n = 0;
    OVKH_TRY(mmi_weight(env, node.inputs[1], k, &w, &n));
    const void *a_zp, *b_zp;
    OVKH_TRY(scalar_zp_dev(env, node, 2, &a_zp));
    OVKH_TRY(scalar_zp_dev(env, node, 3, &b_zp));
    std::vector<int64_t> out_shape(a->shape.begin(), a->shape.end() - 1);
    out_shape.push_back(n);
    const int a_signed = a->dtype == OVK_INT8;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_INT32, out_shape, &out));
    a = env.find(node.inputs[0]);
    return from_abi(env.context(), ovk_matmul_integer(env.context(), w, a->dev, a_signed, m, a_zp, b_zp,
                                                      static_cast<int32_t *>(out->dev)));
}

// interp::matmul_integer_scale_bias (interp.rs:2405-2572)
Result matmul_integer_scale_bias(Env &env, const NodeIr &node)
{
    OVKH_ENSURE(node.inputs.size() >= 6, "MatMulIntegerScaleBias: %zu inputs", node.inputs.size());
    const Tensor *a = env.find(node.inputs[0]);
    const Tensor *scale = env.find(node.inputs[4]);
    const Tensor *bias = env.find(node.inputs[5]);
    const Tensor *prod = node.present(6) ? env.find(node.inputs[6]) : nullptr;
    OVKH_ENSURE(a && scale && bias && (prod || !node.present(6)), "MatMulIntegerScaleBias: an input is missing");
    OVKH_ENSURE(a->shape.size() >= 2, "MatMulInteger: A rank %zu < 2", a->shape.size());
    const int64_t k = a->shape.back(), m = product(a->shape, 0, a->shape.size() - 1);
    ovk_mmi_weight *w = nullptr;
    int64_t n = 0;
    OVKH_TRY(mmi_weight(env, node.inputs[1], k, &w, &n));
    const size_t rank = a->shape.size();
    const int ss = column_step(scale->shape, n, rank), bs = column_step(bias->shape, n, rank);
    const int ps = prod ? column_step(prod->shape, n, rank) : 0;
    if (scale->dtype != OVK_FLOAT || bias->dtype != OVK_FLOAT || (prod && prod->dtype != OVK_FLOAT))
        return fail(OVK_UNSUPPORTED, "MatMulIntegerScaleBias: scale, product and bias must be float32");
    if (ss < 0 || bs < 0 || ps < 0 || a->dtype != OVK_UINT8) {
        // interp::integer_scale_bias_unfused (interp.rs:2630-2665): a scale, product or bias that broadcasts over
        // rows (or a signed A) is not fused; MatMulInteger runs, then Cast, Mul, Add [, Relu] in one pass with
        // general broadcasting.  No range is folded: the quantization that follows makes its own pass.
        std::vector<int64_t> out_shape(a->shape.begin(), a->shape.end() - 1);
        out_shape.push_back(n);
        int64_t srs, scs, brs, bcs, prs = 0, pcs = 0;
        if (!broadcast_strides(scale->shape, out_shape, &srs, &scs) || !broadcast_strides(bias->shape, out_shape, &brs, &bcs) ||
            (prod && !broadcast_strides(prod->shape, out_shape, &prs, &pcs)))
            return fail(OVK_UNSUPPORTED, "MatMulIntegerScaleBias: a scale, product or bias that broadcasts neither over "
                                         "rows nor over columns");
        const void *a_zp, *b_zp;
        OVKH_TRY(scalar_zp_dev(env, node, 2, &a_zp));
        OVKH_TRY(scalar_zp_dev(env, node, 3, &b_zp));
        const std::string acc_name = node.outputs[0] + "/acc";
        Tensor *acc = nullptr, *out = nullptr;
        OVKH_TRY(env.alloc(acc_name, OVK_INT32, out_shape, &acc));
        OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, out_shape, &out));
        acc = const_cast<Tensor *>(env.find(acc_name));
        a = env.find(node.inputs[0]);
        scale = env.find(node.inputs[4]);
        bias = env.find(node.inputs[5]);
        prod = node.present(6) ? env.find(node.inputs[6]) : nullptr;
        OVKH_TRY(from_abi(env.context(), ovk_matmul_integer(env.context(), w, a->dev, a->dtype == OVK_INT8, m, a_zp, b_zp,
                                                            static_cast<int32_t *>(acc->dev))));
        return from_abi(env.context(),
                        ovk_integer_scale_bias_unfused(env.context(), static_cast<const int32_t *>(acc->dev), m, n,
                                                       static_cast<const float *>(scale->dev), srs, scs,
                                                       prod ? static_cast<const float *>(prod->dev) : nullptr, prs, pcs,
                                                       static_cast<const float *>(bias->dev), brs, bcs,
                                                       node.int_attr("relu", 0) == 1 ? OVK_EPILOGUE_RELU : 0u,
                                                       static_cast<float *>(out->dev)));
    }
    const void *a_zp, *b_zp;
    OVKH_TRY(scalar_zp_dev(env, node, 2, &a_zp));
    OVKH_TRY(scalar_zp_dev(env, node, 3, &b_zp));
    uint32_t flags = 0;
    if (node.int_attr("relu", 0) == 1)
        flags |= OVK_EPILOGUE_RELU;
    Tensor *range = nullptr;
    if (node.int_attr("range", 0) == 1) {  // fused_range: the slot the following DynamicQuantizeLinear reads
        flags |= OVK_EPILOGUE_RANGE;
        OVKH_TRY(env.alloc(node.outputs[0] + "/range", OVK_INT32, {4}, &range));
        OVKH_TRY(from_abi(env.context(), ovk_fill(env.context(), range->dev, 0, 16, 0)));
    }
    std::vector<int64_t> out_shape(a->shape.begin(), a->shape.end() - 1);
    out_shape.push_back(n);
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, out_shape, &out));
    a = env.find(node.inputs[0]);
    scale = env.find(node.inputs[4]);
    bias = env.find(node.inputs[5]);
    prod = node.present(6) ? env.find(node.inputs[6]) : nullptr;
    range = range ? const_cast<Tensor *>(env.find(node.outputs[0] + "/range")) : nullptr;
    return from_abi(env.context(),
                    ovk_matmul_integer_scale_bias(env.context(), w, a->dev, 0, m, a_zp, b_zp,
                                                  static_cast<const float *>(scale->dev), ss,
                                                  prod ? static_cast<const float *>(prod->dev) : nullptr, ps,
                                                  static_cast<const float *>(bias->dev), bs, flags,
                                                  range ? static_cast<uint32_t *>(range->dev) : nullptr,
                                                  static_cast<float *>(out->dev)));
}

// interp::qlinear_matmul (interp.rs:4845-4875)
Result qlinear_matmul(Env &env, const NodeIr &node)
{
    const Tensor *a = env.find(node.inputs[0]);
    OVKH_ENSURE(a && a->shape.size() >= 2, "QLinearMatMul: A is missing or has rank < 2");
    const int64_t k = a->shape.back(), m = product(a->shape, 0, a->shape.size() - 1);
    ovk_mmi_weight *w = nullptr;
    int64_t n = 0;
    OVKH_TRY(mmi_weight(env, node.inputs[3], k, &w, &n));
    std::vector<float> ratio;
    OVKH_TRY(requantize_ratio(env, node.inputs[1], node.inputs[4], node.inputs[6], &ratio));
    OVKH_ENSURE(ratio.size() == 1 || int64_t(ratio.size()) == n, "QLinearMatMul: %zu scales for %lld columns", ratio.size(),
                (long long)n);
    int32_t y_zp = 0;
    OVKH_TRY(scalar_i32(env, node.inputs[7], "QLinearMatMul", &y_zp));
    const Tensor *yz = env.find(node.inputs[7]);
    const int32_t out_dtype = yz->dtype;
    const Tensor *azp = env.find(node.inputs[2]);
    const Tensor *bzp = env.find(node.inputs[5]);
    OVKH_ENSURE(azp && bzp, "QLinearMatMul: a zero point is missing");
    Tensor *ratio_dev = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0] + "/ratio", OVK_FLOAT, {int64_t(ratio.size())}, &ratio_dev));
    OVKH_TRY(from_abi(env.context(), ovk_upload(env.context(), ratio_dev->dev, 0, ratio.data(), ratio.size() * 4)));
    // the weight zero point must be one value; a per-column one must be all zero (interp.rs:826-833)
    const void *bzp_dev = bzp->elem_count() == 1 ? bzp->dev : nullptr;
    std::vector<int64_t> out_shape(a->shape.begin(), a->shape.end() - 1);
    out_shape.push_back(n);
    const int a_signed = a->dtype == OVK_INT8;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], out_dtype, out_shape, &out));
    a = env.find(node.inputs[0]);
    azp = env.find(node.inputs[2]);
    ratio_dev = const_cast<Tensor *>(env.find(node.outputs[0] + "/ratio"));
    Result r = from_abi(env.context(),
                        ovk_qlinear_matmul(env.context(), w, a->dev, a_signed, m, azp->dev, bzp_dev,
                                           static_cast<const float *>(ratio_dev->dev), int64_t(ratio.size()), y_zp,
                                           out_dtype == OVK_INT8, out->dev));
    return r;
}

// ------------------------------------------------------ ConvInteger / QLinearConv
// same_pads (interp.rs:3425-3437)
void same_pads(bool upper, int64_t in_dim, int64_t k, int64_t stride, int64_t dil, int64_t *begin, int64_t *end)
{
    const int64_t out = (in_dim + stride - 1) / stride;
    const int64_t needed = std::max<int64_t>((out - 1) * stride + (k - 1) * dil + 1 - in_dim, 0);
    const int64_t half = needed / 2;
    *begin = upper ? half : needed - half;
    *end = upper ? needed - half : half;
}

struct ConvCall {
    ovk_conv_params p;
    ovk_qconv_weight *w;
    int64_t c_out, h_out, w_out;
    bool one_d;
};

// conv_geometry (interp.rs:3439-3536) + the once-per-session filter bank
Result conv_setup(Env &env, const NodeIr &node, const std::string &x_name, const std::string &w_name, ConvCall *c)
{
    const char *op = node.op.c_str();
    const Tensor *x = env.find(x_name);
    const Tensor *wt = env.find(w_name);
    OVKH_ENSURE(x && wt, "%s: x or w is missing", op);
    const size_t spatial = x->shape.size() >= 2 ? x->shape.size() - 2 : 0;
    OVKH_ENSURE(spatial == 1 || spatial == 2, "%s: only 1D/2D (rank %zu)", op, x->shape.size());
    OVKH_ENSURE(wt->shape.size() == spatial + 2, "%s: weight rank %zu", op, wt->shape.size());
    std::vector<int64_t> ks = node.ints_attr("kernel_shape"), strides = node.ints_attr("strides"),
                         dils = node.ints_attr("dilations"), pads = node.ints_attr("pads");
    if (ks.empty())
        ks.assign(wt->shape.begin() + 2, wt->shape.end());
    if (strides.empty())
        strides.assign(spatial, 1);
    if (dils.empty())
        dils.assign(spatial, 1);
    if (pads.empty())
        pads.assign(2 * spatial, 0);
    OVKH_ENSURE(ks.size() == spatial && strides.size() == spatial && dils.size() == spatial,
                "%s: kernel_shape/strides/dilations do not match the spatial rank %zu", op, spatial);
    OVKH_ENSURE(pads.size() == 2 * spatial, "%s: pads of wrong length", op);
    const std::string auto_pad = node.str_attr("auto_pad", "NOTSET");
    if (auto_pad == "VALID") {
        pads.assign(2 * spatial, 0);
    } else if (auto_pad == "SAME_UPPER" || auto_pad == "SAME_LOWER") {
        for (size_t d = 0; d < spatial; d++)
            same_pads(auto_pad == "SAME_UPPER", x->shape[2 + d], ks[d], strides[d], dils[d], &pads[d], &pads[spatial + d]);
    } else if (auto_pad != "NOTSET") {
        return fail(OVK_UNSUPPORTED, "%s: auto_pad '%s' not supported", op, auto_pad.c_str());
    }
    c->one_d = spatial == 1;
    ovk_conv_params &p = c->p;
    p.n = x->shape[0];
    p.c_in = x->shape[1];
    p.h = x->shape[2];
    p.w = c->one_d ? 1 : x->shape[3];
    p.strides[0] = strides[0];
    p.strides[1] = c->one_d ? 1 : strides[1];
    p.dilations[0] = dils[0];
    p.dilations[1] = c->one_d ? 1 : dils[1];
    p.pads[0] = pads[0];
    p.pads[1] = c->one_d ? 0 : pads[1];
    p.pads[2] = c->one_d ? pads[1] : pads[2];
    p.pads[3] = c->one_d ? 0 : pads[3];
    const int64_t group = node.int_attr("group", 1);
    OVKH_ENSURE(wt->dtype == OVK_UINT8 || wt->dtype == OVK_INT8, "%s: weight dtype %d", op, wt->dtype);
    auto it = env.qconv_weights.find(w_name);
    if (it == env.qconv_weights.end()) {
        ovk_qconv_weight *w = nullptr;
        OVKH_TRY(from_abi(env.context(), ovk_qconv_prepack(env.context(), wt->dev, wt->dtype == OVK_INT8, wt->shape[0],
                                                            wt->shape[1], ks[0], c->one_d ? 1 : ks[1], group, &w)));
        it = env.qconv_weights.emplace(w_name, w).first;
    }
    c->w = it->second;
    c->c_out = wt->shape[0];
    if (ovk_conv_output_shape(c->w, &p, &c->h_out, &c->w_out) != OVK_OK)
        return fail(OVK_INVALID_ARGUMENT, "%s: degenerate output shape", op);
    return Result{};
}

std::vector<int64_t> conv_out_shape(const ConvCall &c)
{
    if (c.one_d)
        return {c.p.n, c.c_out, c.h_out};
    return {c.p.n, c.c_out, c.h_out, c.w_out};
}

// interp::conv_integer_with (interp.rs:4421-4651)
Result conv_integer(Env &env, const NodeIr &node)
{
    ConvCall c;
    OVKH_TRY(conv_setup(env, node, node.inputs[0], node.inputs[1], &c));
    int32_t x_zp = 0, w_zp = 0;
    if (node.present(2))
        OVKH_TRY(scalar_i32(env, node.inputs[2], "ConvInteger", &x_zp));
    if (node.present(3))
        OVKH_TRY(scalar_i32(env, node.inputs[3], "ConvInteger", &w_zp));
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_INT32, conv_out_shape(c), &out));
    const Tensor *x = env.find(node.inputs[0]);
    return from_abi(env.context(), ovk_conv_integer(env.context(), c.w, x->dev, x->dtype == OVK_INT8, &c.p, x_zp, w_zp,
                                                    static_cast<int32_t *>(out->dev)));
}

// channel_step (interp.rs:4404-4417): how an operand broadcasts against an [N, C_out, ..] output of
// this rank: 0 one value, 1 one per channel, -1 anything else
int channel_step(const std::vector<int64_t> &shape, int64_t c_out, size_t rank)
{
    if (shape.size() > rank)
        return -1;
    bool ones = true;
    for (int64_t d : shape)
        ones = ones && d == 1;
    if (ones)
        return 0;
    if (rank < 2 || shape.size() < rank - 1)  // the channel axis, counted from the right
        return -1;
    const size_t channel = shape.size() - (rank - 1);
    for (size_t i = 0; i < shape.size(); i++)
        if (i != channel && shape[i] != 1)
            return -1;
    return shape[channel] == c_out ? 1 : -1;
}

// interp::conv_integer_scale_bias (interp.rs:4359-4371): ConvInteger with the Cast, Mul, Add [, Relu]
// that follow it applied to each accumulator
Result conv_integer_scale_bias(Env &env, const NodeIr &node)
{
    const Tensor *scale = env.find(node.inputs[4]);
    const Tensor *bias = env.find(node.inputs[5]);
    const Tensor *prod = node.present(6) ? env.find(node.inputs[6]) : nullptr;
    OVKH_ENSURE(scale && bias && (prod || !node.present(6)), "ConvIntegerScaleBias: an input is missing");
    ConvCall c;
    OVKH_TRY(conv_setup(env, node, node.inputs[0], node.inputs[1], &c));
    const std::vector<int64_t> out_shape = conv_out_shape(c);
    const int ss = channel_step(scale->shape, c.c_out, out_shape.size());
    const int bs = channel_step(bias->shape, c.c_out, out_shape.size());
    const int ps = prod ? channel_step(prod->shape, c.c_out, out_shape.size()) : 0;
    if (ss < 0 || bs < 0 || ps < 0 || scale->dtype != OVK_FLOAT || bias->dtype != OVK_FLOAT ||
        (prod && prod->dtype != OVK_FLOAT))
        return fail(OVK_UNSUPPORTED,
                    "ConvIntegerScaleBias: not fused (a scale, product or bias that is not f32 or broadcasts other "
                    "than per tensor or per channel): the reference runs ConvInteger, Cast, Mul, Add as separate "
                    "nodes here");
    int32_t x_zp = 0, w_zp = 0;
    if (node.present(2))
        OVKH_TRY(scalar_i32(env, node.inputs[2], "ConvInteger", &x_zp));
    if (node.present(3))
        OVKH_TRY(scalar_i32(env, node.inputs[3], "ConvInteger", &w_zp));
    uint32_t flags = node.int_attr("relu", 0) == 1 ? OVK_EPILOGUE_RELU : 0;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, out_shape, &out));
    const Tensor *x = env.find(node.inputs[0]);
    scale = env.find(node.inputs[4]);
    bias = env.find(node.inputs[5]);
    prod = node.present(6) ? env.find(node.inputs[6]) : nullptr;
    return from_abi(env.context(),
                    ovk_conv_integer_scale_bias(env.context(), c.w, x->dev, x->dtype == OVK_INT8, &c.p, x_zp, w_zp,
                                                static_cast<const float *>(scale->dev), ss,
                                                prod ? static_cast<const float *>(prod->dev) : nullptr, ps,
                                                static_cast<const float *>(bias->dev), bs, flags, nullptr,
                                                static_cast<float *>(out->dev)));
}

// interp::qlinear_conv (interp.rs:4796-4837)
Result qlinear_conv(Env &env, const NodeIr &node)
{
    const std::string refusal = unsupported_quantization(node, env);
    if (!refusal.empty())
        return fail(OVK_UNSUPPORTED, "%s", refusal.c_str());
    ConvCall c;
    OVKH_TRY(conv_setup(env, node, node.inputs[0], node.inputs[3], &c));
    std::vector<float> ratio;
    OVKH_TRY(requantize_ratio(env, node.inputs[1], node.inputs[4], node.inputs[6], &ratio));
    // a per-tensor weight scale is broadcast so that bias[c] still has its own channel (interp.rs:4817-4824)
    if (ratio.size() == 1)
        ratio.assign(size_t(c.c_out), ratio[0]);
    OVKH_ENSURE(int64_t(ratio.size()) == c.c_out, "QLinearConv: %zu scales for %lld channels", ratio.size(),
                (long long)c.c_out);
    int32_t x_zp = 0, w_zp = 0, y_zp = 0;
    OVKH_TRY(scalar_i32(env, node.inputs[2], "QLinearConv", &x_zp));
    OVKH_TRY(scalar_i32(env, node.inputs[7], "QLinearConv", &y_zp));
    const Tensor *wz = env.find(node.inputs[5]);
    if (wz && wz->elem_count() == 1)
        OVKH_TRY(scalar_i32(env, node.inputs[5], "QLinearConv", &w_zp));
    const int32_t out_dtype = env.find(node.inputs[7])->dtype;
    const Tensor *bias = node.present(8) ? env.find(node.inputs[8]) : nullptr;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], out_dtype, conv_out_shape(c), &out));
    const Tensor *x = env.find(node.inputs[0]);
    bias = node.present(8) ? env.find(node.inputs[8]) : nullptr;
    return from_abi(env.context(),
                    ovk_qlinear_conv(env.context(), c.w, x->dev, x->dtype == OVK_INT8, &c.p, x_zp, w_zp, ratio.data(),
                                     bias ? static_cast<const int32_t *>(bias->dev) : nullptr, y_zp,
                                     out_dtype == OVK_INT8, out->dev));
}

// ---------------------------------------------------- GatherBlockQuantized / ArgMax
// interp::gather_block_quantized (interp.rs:2874-2990)
Result gather_block_quantized(Env &env, const NodeIr &node)
{
    const int64_t block_size = node.int_attr("block_size", 0);
    const Tensor *table = env.find(node.inputs[0]);
    const Tensor *indices = env.find(node.inputs[1]);
    const Tensor *scales = env.find(node.inputs[2]);
    const Tensor *zp = env.find(node.inputs[3]);
    OVKH_ENSURE(table && indices && scales && zp, "GatherBlockQuantized: an input is missing");
    OVKH_ENSURE(table->shape.size() == 2, "GatherBlockQuantized: expected a 2-D table, got rank %zu", table->shape.size());
    const int64_t rows = std::max<int64_t>(table->shape[0], 0), cols = std::max<int64_t>(table->shape[1], 0) * 2;
    OVKH_ENSURE(cols > 0 && cols % block_size == 0, "GatherBlockQuantized: %lld columns is not a multiple of block_size %lld",
                (long long)cols, (long long)block_size);
    const int64_t n_blocks = cols / block_size;
    OVKH_ENSURE(table->dtype == OVK_UINT8 && zp->dtype == OVK_UINT8 &&
                    (scales->dtype == OVK_FLOAT || scales->dtype == OVK_FLOAT16),
                "GatherBlockQuantized: expected a u8 table and zero point with f32 scales, got %d/%d/%d", table->dtype,
                zp->dtype, scales->dtype);
    OVKH_ENSURE(scales->elem_count() >= rows * n_blocks && zp->elem_count() >= rows * ((n_blocks + 1) / 2),
                "GatherBlockQuantized: scales or zero points are short for %lldx%lld blocks", (long long)rows,
                (long long)n_blocks);
    OVKH_ENSURE(indices->dtype == OVK_INT64 || indices->dtype == OVK_INT32, "GatherBlockQuantized: indices have dtype %d",
                indices->dtype);
    std::vector<int64_t> out_shape = indices->shape;
    out_shape.push_back(cols);
    const int64_t count = indices->elem_count();
    // indices that came from the host are checked there, as the reference does; a
    // device-only tensor (the token an ArgMax node produced) is read in place
    const bool on_host = !indices->host.empty() || count == 0;
    const int32_t idx_dtype = indices->dtype;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, out_shape, &out));
    indices = env.find(node.inputs[1]);
    return from_abi(env.context(),
                    ovk_gather_block_quantized(env.context(), table->dev, scales->dev, scales->dtype, zp->dev, rows, cols, 4,
                                               block_size, on_host ? static_cast<const void *>(indices->host.data())
                                                                   : indices->dev,
                                               idx_dtype, on_host ? 1 : 0, count, out->dev, OVK_FLOAT));
}

// interp::argmax (interp.rs:8493-8527) over arg_extreme_axis (:8552)
Result argmax(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    OVKH_ENSURE(x, "ArgMax: x is missing");
    const int64_t rank = int64_t(x->shape.size());
    OVKH_ENSURE(rank > 0, "ArgMax: x is a scalar: it has no axis");
    int64_t axis = node.int_attr("axis", 0);
    if (axis < 0)
        axis += rank;
    OVKH_ENSURE(axis >= 0 && axis < rank, "ArgMax: axis %lld of a rank-%lld tensor", (long long)node.int_attr("axis", 0),
                (long long)rank);
    if (x->dtype != OVK_FLOAT && x->dtype != OVK_FLOAT16)
        return fail(OVK_UNSUPPORTED, "ArgMax: dtype %d is reduced on the host by the reference, not by this layer", x->dtype);
    const bool keepdims = node.int_attr("keepdims", 1) == 1;
    std::vector<int64_t> out_shape = x->shape;
    if (keepdims)
        out_shape[size_t(axis)] = 1;
    else
        out_shape.erase(out_shape.begin() + axis);
    const int64_t outer = product(x->shape, 0, size_t(axis)), c = x->shape[size_t(axis)],
                  inner = product(x->shape, size_t(axis) + 1, x->shape.size());
    const int32_t dtype = x->dtype;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_INT64, out_shape, &out));
    x = env.find(node.inputs[0]);
    return from_abi(env.context(), ovk_argmax(env.context(), x->dev, dtype, outer, c, std::max<int64_t>(inner, 1),
                                              static_cast<int64_t *>(out->dev)));
}

// ------------------------------------------ the QOperator chain around QLinearConv
Result scalar_f32(const Env &env, const std::string &name, const char *what, float *out)
{
    std::vector<float> v;
    OVKH_TRY(floats_of(env, name, what, &v));
    OVKH_ENSURE(v.size() == 1, "%s: %s is not per-tensor", what, name.c_str());
    *out = v[0];
    return Result{};
}

// interp::qlinear_add (interp.rs:4878-4962)
Result qlinear_add(Env &env, const NodeIr &node)
{
    const Tensor *a = env.find(node.inputs[0]);
    const Tensor *b = env.find(node.inputs[3]);
    OVKH_ENSURE(a && b, "QLinearAdd: an operand is missing");
    float a_scale, b_scale, c_scale;
    int32_t a_zp, b_zp, c_zp;
    OVKH_TRY(scalar_f32(env, node.inputs[1], "QLinearAdd", &a_scale));
    OVKH_TRY(scalar_f32(env, node.inputs[4], "QLinearAdd", &b_scale));
    OVKH_TRY(scalar_f32(env, node.inputs[6], "QLinearAdd", &c_scale));
    OVKH_ENSURE(c_scale != 0.0f, "QLinearAdd: C_scale is zero");
    OVKH_TRY(scalar_i32(env, node.inputs[2], "QLinearAdd", &a_zp));
    OVKH_TRY(scalar_i32(env, node.inputs[5], "QLinearAdd", &b_zp));
    OVKH_TRY(scalar_i32(env, node.inputs[7], "QLinearAdd", &c_zp));
    const int32_t out_dtype = env.find(node.inputs[7])->dtype;
    OVKH_ENSURE((a->dtype == OVK_UINT8 || a->dtype == OVK_INT8) && a->dtype == b->dtype && a->dtype == out_dtype,
                "QLinearAdd: operand dtypes %d/%d/%d", a->dtype, b->dtype, out_dtype);
    OVKH_ENSURE(a->shape.size() <= 8 && b->shape.size() <= 8, "QLinearAdd: rank %zu > 8",
                std::max(a->shape.size(), b->shape.size()));
    // the broadcast shape first (the entry point computes it again and checks it)
    const size_t rank = std::max(a->shape.size(), b->shape.size());
    std::vector<int64_t> out_shape(rank);
    for (size_t d = 0; d < rank; d++) {
        const int64_t ea = d + a->shape.size() >= rank ? a->shape[d + a->shape.size() - rank] : 1;
        const int64_t eb = d + b->shape.size() >= rank ? b->shape[d + b->shape.size() - rank] : 1;
        OVKH_ENSURE(ea == eb || ea == 1 || eb == 1, "QLinearAdd: shapes do not broadcast");
        out_shape[d] = ea == 1 ? eb : ea;
    }
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], out_dtype, out_shape, &out));
    a = env.find(node.inputs[0]);
    b = env.find(node.inputs[3]);
    return from_abi(env.context(),
                    ovk_qlinear_add(env.context(), a->dev, a->shape.data(), int32_t(a->shape.size()), a_scale, a_zp, b->dev,
                                    b->shape.data(), int32_t(b->shape.size()), b_scale, b_zp, c_scale, c_zp,
                                    out_dtype == OVK_INT8, out->dev, nullptr, nullptr));
}

// MaxPool on a quantized tensor (interp.rs: pool() takes the MAXPOOL_Q kernel for u8 / i8 input)
Result maxpool_q(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    OVKH_ENSURE(x, "MaxPool: x is missing");
    if (x->dtype != OVK_UINT8 && x->dtype != OVK_INT8)
        return fail(OVK_UNSUPPORTED, "MaxPool: dtype %d is pooled by the host runtime's float kernel, not by this layer", x->dtype);
    OVKH_ENSURE(x->shape.size() == 4, "MaxPool: only NCHW (rank %zu)", x->shape.size());
    std::vector<int64_t> ks = node.ints_attr("kernel_shape"), st = node.ints_attr("strides"), dl = node.ints_attr("dilations"),
                         pd = node.ints_attr("pads");
    OVKH_ENSURE(ks.size() == 2, "MaxPool: kernel_shape must have two entries");
    if (st.empty())
        st.assign(2, 1);
    if (dl.empty())
        dl.assign(2, 1);
    if (pd.empty())
        pd.assign(4, 0);
    OVKH_ENSURE(st.size() == 2 && dl.size() == 2 && pd.size() == 4, "MaxPool: strides/dilations/pads of wrong length");
    const std::string auto_pad = node.str_attr("auto_pad", "NOTSET");
    if (auto_pad == "VALID") {
        pd.assign(4, 0);
    } else if (auto_pad == "SAME_UPPER" || auto_pad == "SAME_LOWER") {
        for (size_t d = 0; d < 2; d++)
            same_pads(auto_pad == "SAME_UPPER", x->shape[2 + d], ks[d], st[d], dl[d], &pd[d], &pd[2 + d]);
    } else if (auto_pad != "NOTSET") {
        return fail(OVK_UNSUPPORTED, "MaxPool: auto_pad '%s' not supported", auto_pad.c_str());
    }
    const int64_t ho = (x->shape[2] + pd[0] + pd[2] - (dl[0] * (ks[0] - 1) + 1)) / st[0] + 1;
    const int64_t wo = (x->shape[3] + pd[1] + pd[3] - (dl[1] * (ks[1] - 1) + 1)) / st[1] + 1;
    OVKH_ENSURE(ho > 0 && wo > 0, "MaxPool: degenerate output shape");
    const int32_t dtype = x->dtype;
    const std::vector<int64_t> shape = x->shape;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], dtype, {shape[0], shape[1], ho, wo}, &out));
    x = env.find(node.inputs[0]);
    return from_abi(env.context(), ovk_maxpool_q(env.context(), x->dev, dtype == OVK_INT8, shape[0], shape[1], shape[2],
                                                 shape[3], ks.data(), st.data(), pd.data(), dl.data(), out->dev, nullptr,
                                                 nullptr));
}

// qdq_layout (interp.rs:5006-5035)
Result qdq_layout(const NodeIr &node, const std::vector<int64_t> &x_shape, const Tensor &scale, int64_t *inner, int64_t *axis_len)
{
    const int64_t len = std::max<int64_t>(scale.elem_count(), 1);
    *inner = 1;
    *axis_len = 1;
    if (scale.shape.empty() || len == 1)
        return Result{};
    OVKH_ENSURE(scale.shape.size() == 1, "%s: per-axis scale must be 1-D", node.op.c_str());
    const int64_t rank = int64_t(x_shape.size());
    int64_t axis = node.int_attr("axis", 1);
    if (axis < 0)
        axis += rank;
    OVKH_ENSURE(axis >= 0 && axis < rank, "%s: axis %lld out of rank %lld", node.op.c_str(), (long long)axis, (long long)rank);
    OVKH_ENSURE(x_shape[size_t(axis)] == len, "%s: scale of length %lld, axis %lld of dimension %lld", node.op.c_str(),
                (long long)len, (long long)axis, (long long)x_shape[size_t(axis)]);
    *inner = std::max<int64_t>(product(x_shape, size_t(axis) + 1, x_shape.size()), 1);
    *axis_len = len;
    return Result{};
}

// interp::quantize_linear (interp.rs:5117-5177)
Result quantize_linear(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    const Tensor *scale = env.find(node.inputs[1]);
    const Tensor *zp = node.present(2) ? env.find(node.inputs[2]) : nullptr;
    OVKH_ENSURE(x && scale && (zp || !node.present(2)), "QuantizeLinear: an input is missing");
    OVKH_ENSURE(x->dtype == OVK_FLOAT && scale->dtype == OVK_FLOAT, "QuantizeLinear: x and scale must be float32");
    const int32_t out_dtype = zp ? zp->dtype : int32_t(node.int_attr("output_dtype", OVK_UINT8));
    OVKH_ENSURE(out_dtype == OVK_UINT8 || out_dtype == OVK_INT8,
                "QuantizeLinear: output dtype %d not supported (only uint8/int8)", out_dtype);
    int64_t inner, axis_len;
    OVKH_TRY(qdq_layout(node, x->shape, *scale, &inner, &axis_len));
    const std::vector<int64_t> shape = x->shape;
    const int64_t n = x->elem_count();
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], out_dtype, shape, &out));
    x = env.find(node.inputs[0]);
    scale = env.find(node.inputs[1]);
    zp = node.present(2) ? env.find(node.inputs[2]) : nullptr;
    return from_abi(env.context(), ovk_quantize_linear(env.context(), static_cast<const float *>(x->dev), n, inner, axis_len,
                                                       static_cast<const float *>(scale->dev), zp ? zp->dev : nullptr,
                                                       out_dtype == OVK_INT8, out->dev));
}

// interp::dequantize_linear (interp.rs:5055-5115)
Result dequantize_linear(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    const Tensor *scale = env.find(node.inputs[1]);
    const Tensor *zp = node.present(2) ? env.find(node.inputs[2]) : nullptr;
    OVKH_ENSURE(x && scale && (zp || !node.present(2)), "DequantizeLinear: an input is missing");
    OVKH_ENSURE(x->dtype == OVK_UINT8 || x->dtype == OVK_INT8 || x->dtype == OVK_INT32,
                "DequantizeLinear: dtype %d not supported (only uint8/int8/int32)", x->dtype);
    OVKH_ENSURE(scale->dtype == OVK_FLOAT && (!zp || zp->dtype == x->dtype), "DequantizeLinear: scale or zero point dtype");
    int64_t inner, axis_len;
    OVKH_TRY(qdq_layout(node, x->shape, *scale, &inner, &axis_len));
    const std::vector<int64_t> shape = x->shape;
    const int64_t n = x->elem_count();
    const int32_t dtype = x->dtype;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], OVK_FLOAT, shape, &out));
    x = env.find(node.inputs[0]);
    scale = env.find(node.inputs[1]);
    zp = node.present(2) ? env.find(node.inputs[2]) : nullptr;
    return from_abi(env.context(), ovk_dequantize_linear(env.context(), x->dev, dtype, n, inner, axis_len,
                                                         static_cast<const float *>(scale->dev), zp ? zp->dev : nullptr,
                                                         static_cast<float *>(out->dev)));
}

// interp::qlinear_global_average_pool (interp.rs:4975-5000)
Result qlinear_global_average_pool(Env &env, const NodeIr &node)
{
    const Tensor *x = env.find(node.inputs[0]);
    OVKH_ENSURE(x && x->shape.size() >= 2, "QLinearGlobalAveragePool: x is missing or has rank < 2");
    OVKH_ENSURE(node.int_attr("channels_last", 0) == 0, "QLinearGlobalAveragePool: channels_last is not supported");
    float x_scale, y_scale;
    int32_t x_zp, y_zp;
    OVKH_TRY(scalar_f32(env, node.inputs[1], "QLinearGlobalAveragePool", &x_scale));
    OVKH_TRY(scalar_i32(env, node.inputs[2], "QLinearGlobalAveragePool", &x_zp));
    OVKH_TRY(scalar_f32(env, node.inputs[3], "QLinearGlobalAveragePool", &y_scale));
    OVKH_TRY(scalar_i32(env, node.inputs[4], "QLinearGlobalAveragePool", &y_zp));
    OVKH_ENSURE(x->dtype == OVK_UINT8 || x->dtype == OVK_INT8, "QLinearGlobalAveragePool: x has dtype %d", x->dtype);
    std::vector<int64_t> out_shape = x->shape;
    for (size_t d = 2; d < out_shape.size(); d++)
        out_shape[d] = 1;
    const int64_t n = x->shape[0], c = x->shape[1], hw = product(x->shape, 2, x->shape.size());
    const int32_t dtype = x->dtype;
    Tensor *out = nullptr;
    OVKH_TRY(env.alloc(node.outputs[0], dtype, out_shape, &out));
    x = env.find(node.inputs[0]);
    return from_abi(env.context(), ovk_qlinear_global_average_pool(env.context(), x->dev, dtype == OVK_INT8, n, c, hw, x_scale,
                                                                   x_zp, y_scale, y_zp, out->dev));
}

}  // namespace

// ----------------------------------------------------------------------- types
int64_t NodeIr::int_attr(const std::string &key, int64_t fallback) const
{
    auto it = attrs.find(key);
    return it != attrs.end() && it->second.kind == AttrValue::Int ? it->second.i : fallback;
}
std::vector<int64_t> NodeIr::ints_attr(const std::string &key) const
{
    auto it = attrs.find(key);
    return it != attrs.end() && it->second.kind == AttrValue::Ints ? it->second.ints : std::vector<int64_t>();
}
std::string NodeIr::str_attr(const std::string &key, const std::string &fallback) const
{
    auto it = attrs.find(key);
    return it != attrs.end() && it->second.kind == AttrValue::Str ? it->second.s : fallback;
}

int64_t Tensor::elem_count() const
{
    int64_t p = 1;
    for (int64_t d : shape)
        p *= d;
    return p < 0 ? 0 : p;
}

size_t dtype_size(int32_t dtype)
{
    switch (dtype) {
    case OVK_INT64:
        return 8;
    case OVK_FLOAT:
    case OVK_INT32:
        return 4;
    case OVK_FLOAT16:
        return 2;
    case OVK_UINT8:
    case OVK_INT8:
        return 1;
    default:
        return 0;
    }
}

Env::~Env()
{
    for (auto &kv : nbits_weights)
        ovk_nbits_weight_destroy(ctx_, kv.second);
    for (auto &kv : mmi_weights)
        ovk_mmi_weight_destroy(ctx_, kv.second);
    for (auto &kv : qconv_weights)
        ovk_qconv_weight_destroy(ctx_, kv.second);
    for (auto &kv : tensors_)
        ovk_free(ctx_, kv.second.dev);
}

Result Env::alloc(const std::string &name, int32_t dtype, const std::vector<int64_t> &shape, Tensor **out)
{
    const size_t es = dtype_size(dtype);
    if (es == 0)
        return fail(OVK_INVALID_ARGUMENT, "dtype %d with unknown size", dtype);
    release(name);
    Tensor t;
    t.dtype = dtype;
    t.shape = shape;
    t.bytes = size_t(t.elem_count()) * es;
    Result r = from_abi(ctx_, ovk_alloc(ctx_, std::max<size_t>(t.bytes, 4), &t.dev));
    if (!r.ok())
        return r;
    auto ins = tensors_.emplace(name, std::move(t));
    *out = &ins.first->second;
    return Result{};
}

Result Env::set(const std::string &name, int32_t dtype, const std::vector<int64_t> &shape, const void *data, size_t bytes,
                bool initializer)
{
    Tensor *t = nullptr;
    Result r = alloc(name, dtype, shape, &t);
    if (!r.ok())
        return r;
    if (bytes != t->bytes)
        return fail(OVK_INVALID_ARGUMENT, "%s: %zu bytes given for a tensor of %zu", name.c_str(), bytes, t->bytes);
    t->initializer = initializer;
    if (initializer || bytes <= 4096)
        t->host.assign(static_cast<const uint8_t *>(data), static_cast<const uint8_t *>(data) + bytes);
    return from_abi(ctx_, ovk_upload(ctx_, t->dev, 0, data, bytes));
}

const Tensor *Env::find(const std::string &name) const
{
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

Result Env::host(const std::string &name, std::vector<uint8_t> *out, int32_t *dtype, std::vector<int64_t> *shape)
{
    const Tensor *t = find(name);
    if (!t)
        return fail(OVK_INVALID_ARGUMENT, "%s is not in the environment", name.c_str());
    out->resize(t->bytes);
    *dtype = t->dtype;
    *shape = t->shape;
    return from_abi(ctx_, ovk_download(ctx_, t->dev, 0, out->data(), t->bytes));
}

// A weight prepared from this name holds pointers into the tensor's device
// buffer (MatMulNBits) or a packed copy of its bytes (MatMulInteger, the
// convolutions): both die with the tensor, and the next node that names it
// prepares the weight again from the new contents.  The destroy calls wait for
// the stream, so no kernel still reads what is freed here.
void Env::release(const std::string &name)
{
    for (auto dep = nbits_deps.begin(); dep != nbits_deps.end();) {
        const bool hit = dep->first == name || dep->second.first == name || dep->second.second == name;
        if (hit) {
            auto nb = nbits_weights.find(dep->first);
            if (nb != nbits_weights.end()) {
                ovk_nbits_weight_destroy(ctx_, nb->second);
                nbits_weights.erase(nb);
            }
            dep = nbits_deps.erase(dep);
        } else {
            ++dep;
        }
    }
    auto mm = mmi_weights.find(name);
    if (mm != mmi_weights.end()) {
        ovk_mmi_weight_destroy(ctx_, mm->second);
        mmi_weights.erase(mm);
    }
    auto qc = qconv_weights.find(name);
    if (qc != qconv_weights.end()) {
        ovk_qconv_weight_destroy(ctx_, qc->second);
        qconv_weights.erase(qc);
    }
    auto it = tensors_.find(name);
    if (it == tensors_.end())
        return;
    ovk_free(ctx_, it->second.dev);
    tensors_.erase(it);
}

std::string Env::last_kernel() const { return ovk_last_kernel(ctx_); }

// --------------------------------------------------------------------- predicates
// interp::is_implemented_node for the operators of this path (interp.rs:338, :452-464, :560-572)
bool is_implemented_node(const NodeIr &node)
{
    const std::string &op = node.op;
    if (op == "MatMulNBits") {
        const int64_t bs = node.int_attr("block_size", 0);
        // an absent zero point (implicit 8) is accepted here; the reference refuses it (:447-463)
        return node.int_attr("bits", 0) == 4 && bs > 0 && bs % 8 == 0 && node.int_attr("K", 0) > 0 &&
               node.int_attr("N", 0) > 0 && node.present(2) && !node.present(4) && !node.present(5) &&
               node.outputs.size() == 1;
    }
    if (op == "GatherBlockQuantized") {  // interp.rs:470-480
        const int64_t bs = node.int_attr("block_size", 0);
        return node.int_attr("bits", 4) == 4 && bs > 0 && bs % 2 == 0 && node.int_attr("gather_axis", 0) == 0 &&
               node.int_attr("quantize_axis", 1) == 1 && node.present(0) && node.present(1) && node.present(2) &&
               node.present(3) && node.outputs.size() == 1;
    }
    if (op == "ArgMax")  // the reversed tie-break is refused (tests/argmax.rs:192)
        return node.inputs.size() == 1 && node.outputs.size() == 1 && node.int_attr("select_last_index", 0) == 0 &&
               (node.int_attr("keepdims", 1) == 0 || node.int_attr("keepdims", 1) == 1);
    if (op == "QLinearAdd" || op == "QLinearGlobalAveragePool") {
        const size_t want = op == "QLinearAdd" ? 8 : 5;
        bool all = node.inputs.size() == want;
        for (size_t i = 0; all && i < want; i++)
            all = node.present(i);
        return all && node.outputs.size() == 1;
    }
    if (op == "QuantizeLinear" || op == "DequantizeLinear")
        return node.inputs.size() >= 2 && node.inputs.size() <= 3 && node.present(0) && node.present(1) &&
               node.outputs.size() == 1 && node.int_attr("block_size", 0) == 0;
    if (op == "MaxPool")  // the quantized-domain pooling; a float input is refused at dispatch
        return node.inputs.size() == 1 && node.outputs.size() == 1 && node.int_attr("ceil_mode", 0) == 0 &&
               node.int_attr("storage_order", 0) == 0;
    if (op == "DynamicQuantizeLinear")
        return node.inputs.size() == 1 && node.outputs.size() == 3;
    if (op == "DecomposedGelu")  // x, divisor, offset, factor (rewrite.rs:600-697)
        return node.inputs.size() == 4 && node.outputs.size() == 1;
    if (op == "DecomposedGeluQuantize")  // rewrite.rs:699-735
        return node.inputs.size() == 4 && node.outputs.size() == 3;
    if (op == "MatMulInteger")
        return node.inputs.size() >= 2 && node.inputs.size() <= 4 && node.outputs.size() == 1;
    if (op == "MatMulIntegerScaleBias")
        return node.inputs.size() >= 6 && node.inputs.size() <= 7 && node.outputs.size() == 1;
    if (op == "ConvInteger")
        return node.inputs.size() >= 2 && node.inputs.size() <= 4 && node.outputs.size() == 1;
    if (op == "ConvIntegerScaleBias")
        return node.inputs.size() >= 6 && node.inputs.size() <= 7 && node.present(4) && node.present(5) &&
               node.outputs.size() == 1;
    if (op == "QLinearConv") {
        const std::string ap = node.str_attr("auto_pad", "NOTSET");
        bool all = node.inputs.size() >= 8 && node.inputs.size() <= 9;
        for (size_t i = 0; all && i < 8; i++)
            all = node.present(i);
        return all && (ap == "NOTSET" || ap == "VALID" || ap == "SAME_UPPER" || ap == "SAME_LOWER") &&
               node.outputs.size() == 1;
    }
    if (op == "QLinearMatMul") {
        bool all = node.inputs.size() == 8;
        for (size_t i = 0; all && i < 8; i++)
            all = node.present(i);
        return all && node.outputs.size() == 1;
    }
    return false;
}

// interp::unsupported_quantization (interp.rs:781-847), same wording
std::string unsupported_quantization(const NodeIr &node, const Env &env)
{
    struct Pair {
        size_t scale, zero;
        const char *slot;
    };
    auto constant = [&](size_t index) -> const Tensor * {
        if (!node.present(index))
            return nullptr;
        const Tensor *t = env.find(node.inputs[index]);
        return t && t->initializer ? t : nullptr;
    };
    auto refuse = [&](const char *slot, const char *why) { return node.op + ": " + slot + " " + why; };
    auto check_scalar = [&](const Pair &p) -> std::string {
        const Tensor *scale = constant(p.scale), *zero = constant(p.zero);
        if (!scale || !zero)
            return refuse(p.slot, "scale or zero point is not a constant");
        if (scale->dtype != OVK_FLOAT)
            return refuse(p.slot, "scale is not float32");
        if (std::max<int64_t>(scale->elem_count(), 1) != 1 || std::max<int64_t>(zero->elem_count(), 1) != 1)
            return refuse(p.slot, "scale or zero point is not per-tensor");
        return "";
    };
    if (node.op == "QLinearAdd" || node.op == "QLinearGlobalAveragePool") {
        const Pair add_pairs[3] = {{1, 2, "A"}, {4, 5, "B"}, {6, 7, "C"}};
        const Pair gap_pairs[2] = {{1, 2, "x"}, {3, 4, "y"}};
        const Pair *pairs = node.op == "QLinearAdd" ? add_pairs : gap_pairs;
        const int count = node.op == "QLinearAdd" ? 3 : 2;
        for (int i = 0; i < count; i++) {
            const std::string why = check_scalar(pairs[i]);
            if (!why.empty())
                return why;
        }
        return "";
    }
    if (node.op != "QLinearConv" && node.op != "QLinearMatMul")
        return "";
    const bool conv = node.op == "QLinearConv";
    const Pair scalar_pairs[2] = {{1, 2, conv ? "x" : "a"}, {6, 7, "y"}};
    for (const Pair &p : scalar_pairs) {
        const std::string why = check_scalar(p);
        if (!why.empty())
            return why;
    }
    const char *slot = conv ? "w" : "b";
    const Tensor *scale = constant(4), *zero = constant(5);
    if (!scale || !zero)
        return refuse(slot, "scale or zero point is not a constant");
    if (scale->dtype != OVK_FLOAT)
        return refuse(slot, "scale is not float32");
    if (std::max<int64_t>(scale->elem_count(), 1) != std::max<int64_t>(zero->elem_count(), 1))
        return refuse(slot, "scale and zero point have different lengths");
    if (zero->elem_count() > 1 && std::any_of(zero->host.begin(), zero->host.end(), [](uint8_t b) { return b != 0; }))
        return refuse(slot, "per-channel zero point is not zero (asymmetric weights)");
    if (conv && node.present(8)) {
        const Tensor *bias = constant(8);
        if (bias && bias->dtype != OVK_INT32)
            return refuse("B", "bias is not int32");
    }
    return "";
}

// interp::exec_dispatch (interp.rs:1071-1196), the operators of the path and its two decode-step neighbours
Result exec_dispatch(Env &env, const NodeIr &node)
{
    if (!is_implemented_node(node))
        return fail(OVK_UNSUPPORTED, "%s: this form of the node is not implemented", node.op.c_str());
    if (node.op == "MatMulNBits")
        return matmul_nbits(env, node);
    if (node.op == "DynamicQuantizeLinear")
        return dynamic_quantize(env, node);
    if (node.op == "DecomposedGelu")
        return decomposed_gelu(env, node);
    if (node.op == "DecomposedGeluQuantize")
        return decomposed_gelu_quantize(env, node);
    if (node.op == "MatMulInteger")
        return matmul_integer(env, node);
    if (node.op == "MatMulIntegerScaleBias")
        return matmul_integer_scale_bias(env, node);
    if (node.op == "QLinearMatMul") {
        const std::string refusal = unsupported_quantization(node, env);
        if (!refusal.empty())
            return fail(OVK_UNSUPPORTED, "%s", refusal.c_str());
        return qlinear_matmul(env, node);
    }
    if (node.op == "ConvInteger")
        return conv_integer(env, node);
    if (node.op == "ConvIntegerScaleBias")
        return conv_integer_scale_bias(env, node);
    if (node.op == "GatherBlockQuantized")
        return gather_block_quantized(env, node);
    if (node.op == "ArgMax")
        return argmax(env, node);
    if (node.op == "QLinearAdd" || node.op == "QLinearGlobalAveragePool") {
        const std::string refusal = unsupported_quantization(node, env);
        if (!refusal.empty())
            return fail(OVK_UNSUPPORTED, "%s", refusal.c_str());
        return node.op == "QLinearAdd" ? qlinear_add(env, node) : qlinear_global_average_pool(env, node);
    }
    if (node.op == "MaxPool")
        return maxpool_q(env, node);
    if (node.op == "QuantizeLinear")
        return quantize_linear(env, node);
    if (node.op == "DequantizeLinear")
        return dequantize_linear(env, node);
    return qlinear_conv(env, node);
}

}  // namespace host
}  // namespace ovk

// ---------------------------------------------------------------------------
// A small C surface over the classes above, so that the node-level layer can be
// driven from tests written in any language (used by tests/test_gpu_host_layer.py).
using namespace ovk::host;

struct ovkh_env {
    ovk_ctx *ctx = nullptr;
    Env *env = nullptr;
    std::string err;
};

#define OVKH_API extern "C" __attribute__((visibility("default")))

OVKH_API int32_t ovkh_env_create(int32_t device, ovkh_env **out)
{
    ovk_ctx *ctx = nullptr;
    const int32_t rc = ovk_ctx_create(device, nullptr, &ctx);
    if (rc != OVK_OK)
        return rc;
    ovkh_env *e = new ovkh_env();
    e->ctx = ctx;
    e->env = new Env(ctx);
    *out = e;
    return OVK_OK;
}

OVKH_API void ovkh_env_destroy(ovkh_env *e)
{
    if (!e)
        return;
    delete e->env;
    ovk_ctx_destroy(e->ctx);
    delete e;
}

OVKH_API const char *ovkh_last_error(const ovkh_env *e) { return e ? e->err.c_str() : ""; }

OVKH_API int32_t ovkh_set(ovkh_env *e, const char *name, int32_t dtype, const int64_t *shape, int32_t ndim,
                          const void *data, size_t bytes, int32_t initializer)
{
    Result r = e->env->set(name, dtype, std::vector<int64_t>(shape, shape + ndim), data, bytes, initializer != 0);
    e->err = r.message;
    return r.status;
}

OVKH_API NodeIr *ovkh_node_create(const char *op, const char *domain, const char *name)
{
    NodeIr *n = new NodeIr();
    n->op = op;
    n->domain = domain;
    n->name = name;
    return n;
}
OVKH_API void ovkh_node_destroy(NodeIr *n) { delete n; }
OVKH_API void ovkh_node_input(NodeIr *n, const char *name) { n->inputs.push_back(name); }
OVKH_API void ovkh_node_output(NodeIr *n, const char *name) { n->outputs.push_back(name); }
OVKH_API void ovkh_node_attr_int(NodeIr *n, const char *key, int64_t v)
{
    AttrValue a;
    a.kind = AttrValue::Int;
    a.i = v;
    n->attrs[key] = a;
}
OVKH_API void ovkh_node_attr_ints(NodeIr *n, const char *key, const int64_t *v, int32_t count)
{
    AttrValue a;
    a.kind = AttrValue::Ints;
    a.ints.assign(v, v + count);
    n->attrs[key] = a;
}
OVKH_API void ovkh_node_attr_str(NodeIr *n, const char *key, const char *v)
{
    AttrValue a;
    a.kind = AttrValue::Str;
    a.s = v;
    n->attrs[key] = a;
}
OVKH_API int32_t ovkh_is_implemented(const NodeIr *n) { return is_implemented_node(*n) ? 1 : 0; }
OVKH_API int32_t ovkh_unsupported_quantization(ovkh_env *e, const NodeIr *n)
{
    e->err = unsupported_quantization(*n, *e->env);
    return e->err.empty() ? 0 : 1;
}
OVKH_API int32_t ovkh_execute(ovkh_env *e, const NodeIr *n)
{
    Result r = exec_dispatch(*e->env, *n);
    e->err = r.message;
    return r.status;
}
OVKH_API const char *ovkh_last_kernel(ovkh_env *e) { return ovk_last_kernel(e->ctx); }
OVKH_API int32_t ovkh_info(ovkh_env *e, const char *name, int32_t *dtype, int32_t *ndim, int64_t *shape8, size_t *bytes)
{
    const Tensor *t = e->env->find(name);
    if (!t) {
        e->err = std::string(name) + " is not in the environment";
        return OVK_INVALID_ARGUMENT;
    }
    *dtype = t->dtype;
    *ndim = int32_t(t->shape.size());
    for (size_t i = 0; i < t->shape.size() && i < 8; i++)
        shape8[i] = t->shape[i];
    *bytes = t->bytes;
    return OVK_OK;
}
OVKH_API int32_t ovkh_get(ovkh_env *e, const char *name, void *dst, size_t bytes)
{
    std::vector<uint8_t> data;
    int32_t dtype;
    std::vector<int64_t> shape;
    Result r = e->env->host(name, &data, &dtype, &shape);
    e->err = r.message;
    if (!r.ok())
        return r.status;
    if (bytes < data.size()) {
        e->err = "destination too small";
        return OVK_INVALID_ARGUMENT;
    }
    memcpy(dst, data.data(), data.size());
    return OVK_OK;
}
