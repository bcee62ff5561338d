// The rest of the QOperator chain around QLinearConv, so that a quantized
// residual block stays int8 on the device: QLinearAdd, MaxPool on quantized
// codes, QLinearGlobalAveragePool, QuantizeLinear and DequantizeLinear.
// All are one pass over their tensors (HBM-bound, one byte or word per element).
//
// Reference: crates/onnx-vulkan-core/src/shaders/qlinear.rs:69-211,
// src/shaders/quantize_linear.rs:16-121, src/shaders/pooling.rs:15-66 and the
// host functions interp::qlinear_add (src/interp.rs:4878-4962),
// qlinear_global_average_pool (:4975-5000), quantize_linear (:5117-5177),
// dequantize_linear (:5055-5115).
#include "ovk_internal.h"

#include <cmath>

namespace {

constexpr int MAX_RANK = 8;

struct Strides {
    uint32_t out[MAX_RANK], a[MAX_RANK], b[MAX_RANK];
    int rank;
};

__device__ __forceinline__ int32_t code_of(const uint8_t *p, int64_t i, int is_signed)
{
    return is_signed ? int32_t(static_cast<const int8_t *>(static_cast<const void *>(p))[i]) : int32_t(p[i]);
}

// C = saturate(round(fma(A, ra, fma(B, rb, fixed)))): MLAS's kernel operation for operation
// (shaders/qlinear.rs:69-83)
__device__ __forceinline__ uint32_t add_code(int32_t av, int32_t bv, float ra, float rb, float fixed, int is_signed)
{
    const float y = rintf(fmaf(float(av), ra, fmaf(float(bv), rb, fixed)));
    const float c = is_signed ? fminf(fmaxf(y, -128.0f), 127.0f) : fminf(fmaxf(y, 0.0f), 255.0f);
    return uint32_t(int32_t(c)) & 0xffu;
}

// Byte -> float and float -> byte without the quarter-rate conversion instructions: a byte put into
// the low mantissa bits of 2^23 is the float 2^23 + b, and adding 1.5 * 2^23 to a value already clamped to
// the byte range rounds it to nearest-even with the result in the low byte.  Clamping before rounding gives
// the same code as rounding before clamping because the bounds are integers.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
template <int J>
__device__ __forceinline__ float byte_to_float(uint32_t word, float bias)
{
    // byte J of `word` under the exponent of 2^23; `word` already has its sign bits flipped for int8
    return __fsub_rn(__uint_as_float(prmt(word, 0x4B000000u, 0x7650u | J)), bias);
}
__device__ __forceinline__ uint32_t add_word(uint32_t aw, uint32_t bw, float ra, float rb, float fixed, float bias, float lo,
                                             float hi)
{
    uint32_t r[4];
#define OVK_ADD_ONE(J)                                                                                        \
    {                                                                                                         \
        const float y = fmaf(byte_to_float<J>(aw, bias), ra, fmaf(byte_to_float<J>(bw, bias), rb, fixed));    \
        r[J] = __float_as_uint(__fadd_rn(fminf(fmaxf(y, lo), hi), 12582912.0f));                              \
    }
    OVK_ADD_ONE(0) OVK_ADD_ONE(1) OVK_ADD_ONE(2) OVK_ADD_ONE(3)
#undef OVK_ADD_ONE
    return prmt(prmt(r[0], r[1], 0x0040u), prmt(r[2], r[3], 0x0040u), 0x5410u);  // the four low bytes
}

// same shape on both sides: sixteen elements per thread, 128 bits in from each side, 128 bits out
__global__ void __launch_bounds__(256)
qlinear_add_flat_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ b, uint4 *__restrict__ out,
                        int64_t vecs, float ra, float rb, float fixed, int is_signed)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= vecs)
        return;
    uint4 av = __ldcs(a + i), bv = __ldcs(b + i);
    // int8: b ^ 0x80 is the byte b + 128, so the bias grows by 128
    const uint32_t flip = is_signed ? 0x80808080u : 0u;
    const float bias = is_signed ? 8388736.0f : 8388608.0f;
    const float lo = is_signed ? -128.0f : 0.0f, hi = is_signed ? 127.0f : 255.0f;
    uint4 o;
    o.x = add_word(av.x ^ flip, bv.x ^ flip, ra, rb, fixed, bias, lo, hi);
    o.y = add_word(av.y ^ flip, bv.y ^ flip, ra, rb, fixed, bias, lo, hi);
    o.z = add_word(av.z ^ flip, bv.z ^ flip, ra, rb, fixed, bias, lo, hi);
    o.w = add_word(av.w ^ flip, bv.w ^ flip, ra, rb, fixed, bias, lo, hi);
    __stcs(out + i, o);
}

// general ONNX broadcasting, one element per thread
__global__ void __launch_bounds__(256)
qlinear_add_bcast_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ b, uint8_t *__restrict__ out,
                         int64_t n, Strides st, float ra, float rb, float fixed, int is_signed)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    uint32_t rem = uint32_t(i), off_a = 0, off_b = 0;
    for (int d = 0; d < st.rank; d++) {
        const uint32_t c = rem / st.out[d];
        rem -= c * st.out[d];
        off_a += c * st.a[d];
        off_b += c * st.b[d];
    }
    out[i] = uint8_t(add_code(code_of(a, off_a, is_signed), code_of(b, off_b, is_signed), ra, rb, fixed, is_signed));
}

// MaxPool on codes: out-of-bound taps are skipped (shaders/qlinear.rs:160-211)
__global__ void __launch_bounds__(256)
maxpool_q_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ out, int64_t total, int c, int h_in, int w_in,
                 int h_out, int w_out, int kh, int kw, int sh, int sw, int phb, int pwb, int dh, int dw, int is_signed)
{
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (o >= total)
        return;
    const int ow = int(o % w_out);
    const int64_t t1 = o / w_out;
    const int oh = int(t1 % h_out);
    const int64_t plane = (t1 / h_out) * int64_t(h_in) * w_in;  // (n * C + ch) planes
    (void)c;
    int32_t acc = INT32_MIN;
    for (int r = 0; r < kh; r++) {
        const int ih = oh * sh - phb + r * dh;
        if (ih < 0 || ih >= h_in)
            continue;
        for (int s = 0; s < kw; s++) {
            const int iw = ow * sw - pwb + s * dw;
            if (iw < 0 || iw >= w_in)
                continue;
            acc = max(acc, code_of(x, plane + int64_t(ih) * w_in + iw, is_signed));
        }
    }
    out[o] = uint8_t(uint32_t(acc) & 0xffu);
}

// QuantizeLinear: saturate(rne(x / scale) + zero_point), c = (i / inner) % axis_len
// (shaders/quantize_linear.rs:72-121; the division is IEEE here, which is what div_rn emulates there)
__global__ void __launch_bounds__(256)
quantize_linear_kernel(const float *__restrict__ x, const float *__restrict__ scale, const uint8_t *__restrict__ zp,
                       uint8_t *__restrict__ out, int64_t n, int64_t inner, int64_t axis_len, int is_signed)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int64_t c = (i / inner) % axis_len;
    const int32_t zero = zp ? code_of(zp, c, is_signed) : 0;
    const float r = rintf(__fdiv_rn(x[i], scale[c]));
    // float -> int as the reference's i32(): saturating, NaN to 0
    int32_t q = (r >= 2147483648.0f) ? INT32_MAX : (r <= -2147483648.0f ? INT32_MIN : (r != r ? 0 : int32_t(r)));
    q = int32_t(uint32_t(q) + uint32_t(zero));
    q = is_signed ? max(-128, min(127, q)) : max(0, min(255, q));
    out[i] = uint8_t(uint32_t(q) & 0xffu);
}

// DequantizeLinear: (x - zero_point) * scale for u8 / i8 / i32 input (quantize_linear.rs:16-70)
template <int KIND>  // 0 u8, 1 i8, 2 i32
__global__ void __launch_bounds__(256)
dequantize_linear_kernel(const void *__restrict__ x, const float *__restrict__ scale, const void *__restrict__ zp,
                         float *__restrict__ out, int64_t n, int64_t inner, int64_t axis_len)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int64_t c = (i / inner) % axis_len;
    int32_t q, zero = 0;
    if (KIND == 2) {
        q = static_cast<const int32_t *>(x)[i];
        if (zp)
            zero = static_cast<const int32_t *>(zp)[c];
    } else {
        q = code_of(static_cast<const uint8_t *>(x), i, KIND);
        if (zp)
            zero = code_of(static_cast<const uint8_t *>(zp), c, KIND);
    }
    out[i] = __fmul_rn(float(int32_t(uint32_t(q) - uint32_t(zero))), scale[c]);
}

// QLinearGlobalAveragePool = dequantize, average pool over the whole plane, quantize, with the
// reference's arithmetic: one thread per (n, c), a sequential f32 sum in row-major order divided by
// the count (shaders/pooling.rs:38-54), then QuantizeLinear.
__global__ void __launch_bounds__(128)
qlinear_gap_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ out, int64_t planes, int64_t hw, float x_scale,
                   int32_t x_zp, float y_scale, int32_t y_zp, int is_signed)
{
    const int64_t p = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (p >= planes)
        return;
    float acc = 0.0f;
    for (int64_t i = 0; i < hw; i++)
        acc = __fadd_rn(acc, __fmul_rn(float(code_of(x, p * hw + i, is_signed) - x_zp), x_scale));
    const float mean = __fdiv_rn(acc, float(uint32_t(hw > 0 ? hw : 1)));
    const float r = rintf(__fdiv_rn(mean, y_scale));
    int32_t q = (r >= 2147483648.0f) ? INT32_MAX : (r <= -2147483648.0f ? INT32_MIN : (r != r ? 0 : int32_t(r)));
    q = int32_t(uint32_t(q) + uint32_t(y_zp));
    q = is_signed ? max(-128, min(127, q)) : max(0, min(255, q));
    out[p] = uint8_t(uint32_t(q) & 0xffu);
}

unsigned blocks_for(int64_t n, int threads) { return unsigned(ceil_div64(n, threads)); }

}  // namespace

extern "C" int32_t ovk_qlinear_add(ovk_ctx *ctx, const void *a, const int64_t *a_shape, int32_t a_rank, float a_scale,
                                   int32_t a_zp, const void *b, const int64_t *b_shape, int32_t b_rank, float b_scale,
                                   int32_t b_zp, float c_scale, int32_t c_zp, int32_t is_signed, void *out,
                                   int64_t *out_shape, int32_t *out_rank)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, a_rank >= 0 && b_rank >= 0 && a_rank <= MAX_RANK && b_rank <= MAX_RANK, "QLinearAdd: rank %d > %d",
                std::max(a_rank, b_rank), MAX_RANK);
    OVK_REQUIRE(ctx, c_scale != 0.0f, "QLinearAdd: C_scale is zero");
    // numpy-style broadcast, aligned at the last dimension
    const int rank = std::max(a_rank, b_rank);
    int64_t shape[MAX_RANK], sa[MAX_RANK], sb[MAX_RANK];
    int64_t run_a = 1, run_b = 1, n = 1;
    for (int d = rank - 1; d >= 0; d--) {
        const int da = d - (rank - a_rank), db = d - (rank - b_rank);
        const int64_t ea = da >= 0 ? a_shape[da] : 1, eb = db >= 0 ? b_shape[db] : 1;
        OVK_REQUIRE(ctx, ea == eb || ea == 1 || eb == 1, "QLinearAdd: shapes do not broadcast (%lld vs %lld)", (long long)ea,
                    (long long)eb);
        shape[d] = ea == 1 ? eb : ea;
        sa[d] = ea == 1 ? 0 : run_a;
        sb[d] = eb == 1 ? 0 : run_b;
        run_a *= ea;
        run_b *= eb;
        n *= shape[d];
    }
    if (out_rank)
        *out_rank = rank;
    if (out_shape)
        for (int d = 0; d < rank; d++)
            out_shape[d] = shape[d];
    if (n <= 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, a && b && out, "QLinearAdd: null pointer");
    OVK_REQUIRE(ctx, n < (int64_t(1) << 32), "QLinearAdd: %lld elements", (long long)n);
    float ra = a_scale / c_scale, rb = b_scale / c_scale;
    // the operands are exchanged where ORT exchanges them before MLAS: when A is constant along the
    // innermost span that is broadcast over (or the output is one element); the kernel's rounding is
    // not symmetric in A and B (interp.rs:4906-4916)
    int inner = -1;
    for (int d = rank - 1; d >= 0; d--)
        if (shape[d] > 1) {
            inner = d;
            break;
        }
    if (inner < 0 || sa[inner] == 0) {
        std::swap(a, b);
        for (int d = 0; d < rank; d++)
            std::swap(sa[d], sb[d]);
        std::swap(ra, rb);
        std::swap(a_zp, b_zp);
        std::swap(run_a, run_b);
    }
    // MLAS folds the zero points into one addend, with this contraction (interp.rs:4918)
    volatile float rbz = rb * float(b_zp);
    const float fixed = float(c_zp) - std::fmaf(ra, float(a_zp), rbz);
    const bool flat = run_a == n && run_b == n && (n % 16) == 0 && aligned_to(a, 16) && aligned_to(b, 16) && aligned_to(out, 16);
    if (flat) {
        qlinear_add_flat_kernel<<<blocks_for(n / 16, 256), 256, 0, ctx->stream>>>(
            static_cast<const uint4 *>(a), static_cast<const uint4 *>(b), static_cast<uint4 *>(out), n / 16, ra, rb,
            fixed, is_signed ? 1 : 0);
        OVK_LAUNCHED(ctx, "qlinear_add");
    } else {
        Strides st = {};
        st.rank = rank;
        int64_t run = 1;
        for (int d = rank - 1; d >= 0; d--) {
            st.out[d] = uint32_t(run);
            st.a[d] = uint32_t(sa[d]);
            st.b[d] = uint32_t(sb[d]);
            run *= shape[d];
        }
        qlinear_add_bcast_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(a), static_cast<const uint8_t *>(b), static_cast<uint8_t *>(out), n, st, ra, rb,
            fixed, is_signed ? 1 : 0);
        OVK_LAUNCHED(ctx, "qlinear_add_broadcast");
    }
    return OVK_OK;
}

extern "C" int32_t ovk_maxpool_q(ovk_ctx *ctx, const void *x, int32_t is_signed, int64_t n, int64_t c, int64_t h,
                                 int64_t w, const int64_t *kernel, const int64_t *strides, const int64_t *pads,
                                 const int64_t *dilations, void *out, int64_t *h_out, int64_t *w_out)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, kernel && strides && pads && dilations, "MaxPool: null geometry");
    const int64_t kh = kernel[0], kw = kernel[1], sh = strides[0], sw = strides[1], dh = dilations[0], dw = dilations[1];
    OVK_REQUIRE(ctx, kh > 0 && kw > 0 && sh > 0 && sw > 0 && dh > 0 && dw > 0, "MaxPool: bad kernel, stride or dilation");
    // floor mode, pads = {h_begin, w_begin, h_end, w_end}
    const int64_t ho = (h + pads[0] + pads[2] - (dh * (kh - 1) + 1)) / sh + 1;
    const int64_t wo = (w + pads[1] + pads[3] - (dw * (kw - 1) + 1)) / sw + 1;
    OVK_REQUIRE(ctx, ho > 0 && wo > 0 && h < (1 << 30) && w < (1 << 30), "MaxPool: degenerate output shape");
    if (h_out)
        *h_out = ho;
    if (w_out)
        *w_out = wo;
    const int64_t total = n * c * ho * wo;
    if (total <= 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && out, "MaxPool: null pointer");
    maxpool_q_kernel<<<blocks_for(total, 256), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t *>(x), static_cast<uint8_t *>(out), total, int(c), int(h), int(w), int(ho), int(wo),
        int(kh), int(kw), int(sh), int(sw), int(pads[0]), int(pads[1]), int(dh), int(dw), is_signed ? 1 : 0);
    OVK_LAUNCHED(ctx, "maxpool_q");
    return OVK_OK;
}

extern "C" int32_t ovk_quantize_linear(ovk_ctx *ctx, const float *x, int64_t n, int64_t inner, int64_t axis_len,
                                       const float *scale, const void *zero_point, int32_t is_signed, void *out)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, n >= 0 && inner >= 1 && axis_len >= 1, "QuantizeLinear: layout %lld / %lld / %lld", (long long)n,
                (long long)inner, (long long)axis_len);
    if (n == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && scale && out, "QuantizeLinear: null pointer");
    quantize_linear_kernel<<<blocks_for(n, 256), 256, 0, ctx->stream>>>(x, scale, static_cast<const uint8_t *>(zero_point),
                                                                        static_cast<uint8_t *>(out), n, inner, axis_len,
                                                                        is_signed ? 1 : 0);
    OVK_LAUNCHED(ctx, "quantize_linear");
    return OVK_OK;
}

extern "C" int32_t ovk_dequantize_linear(ovk_ctx *ctx, const void *x, int32_t x_dtype, int64_t n, int64_t inner,
                                         int64_t axis_len, const float *scale, const void *zero_point, float *out)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, x_dtype == OVK_UINT8 || x_dtype == OVK_INT8 || x_dtype == OVK_INT32,
                "DequantizeLinear: dtype %d not supported (only uint8/int8/int32)", x_dtype);
    OVK_REQUIRE(ctx, n >= 0 && inner >= 1 && axis_len >= 1, "DequantizeLinear: layout %lld / %lld / %lld", (long long)n,
                (long long)inner, (long long)axis_len);
    if (n == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && scale && out, "DequantizeLinear: null pointer");
    const unsigned grid = blocks_for(n, 256);
    if (x_dtype == OVK_UINT8)
        dequantize_linear_kernel<0><<<grid, 256, 0, ctx->stream>>>(x, scale, zero_point, out, n, inner, axis_len);
    else if (x_dtype == OVK_INT8)
        dequantize_linear_kernel<1><<<grid, 256, 0, ctx->stream>>>(x, scale, zero_point, out, n, inner, axis_len);
    else
        dequantize_linear_kernel<2><<<grid, 256, 0, ctx->stream>>>(x, scale, zero_point, out, n, inner, axis_len);
    OVK_LAUNCHED(ctx, "dequantize_linear");
    return OVK_OK;
}

extern "C" int32_t ovk_qlinear_global_average_pool(ovk_ctx *ctx, const void *x, int32_t is_signed, int64_t n, int64_t c,
                                                   int64_t hw, float x_scale, int32_t x_zp, float y_scale, int32_t y_zp,
                                                   void *out)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, n >= 0 && c >= 0 && hw >= 0, "QLinearGlobalAveragePool: shape %lld x %lld x %lld", (long long)n,
                (long long)c, (long long)hw);
    if (n * c == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && out, "QLinearGlobalAveragePool: null pointer");
    qlinear_gap_kernel<<<blocks_for(n * c, 128), 128, 0, ctx->stream>>>(static_cast<const uint8_t *>(x),
                                                                         static_cast<uint8_t *>(out), n * c, hw, x_scale,
                                                                         x_zp, y_scale, y_zp, is_signed ? 1 : 0);
    OVK_LAUNCHED(ctx, "qlinear_global_average_pool");
    return OVK_OK;
}
