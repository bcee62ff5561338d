// DecomposedGelu: the exact GELU spelled as Div -> Erf -> Add -> Mul -> Mul, as the
// reference evaluates it in one pass (crates/onnx-vulkan-core/src/shaders/
// elementwise.rs:71-118): erf by the five-term rational approximation
// (Abramowitz & Stegun 7.1.26), every step rounded on its own as the five
// separate kernels round, and the two orders of the closing products.
//
// The reference's shader calls the device's exp(), whose last bits differ from
// device to device; here exp is spelled out in IEEE operations only (argument
// reduction by ln 2 in two parts, a degree-7 polynomial by fused multiply-adds,
// scaling by the exponent bits), so that the CPU port of this file's arithmetic
// and the kernels agree bit for bit.  Its error is about one ulp over the range
// erf needs (arguments -a*a <= 0).
#pragma once

#include <cstdint>

struct GeluParams {
    float divisor, offset, factor;
    int factor_first;
};

// exp(x) for x <= 0 (and small positive x); 0 below -104, where the result underflows.
__device__ __forceinline__ float ovk_exp_ieee(float x)
{
    if (!(x > -104.0f))
        return x != x ? x : 0.0f;
    // n = rint(x * log2 e) and its integer, without the quarter-rate rounding and conversion instructions: for
    // |t| < 2^22 the sum t + 1.5 * 2^23 is rounded to an integer (to nearest even, as rintf rounds), its low
    // mantissa bits are that integer, and subtracting the constant again is exact.
    const float shifted = __fadd_rn(__fmul_rn(x, 1.44269504088896341f), 12582912.0f);
    const float n = __fsub_rn(shifted, 12582912.0f);
    const int e = __float_as_int(shifted) - 0x4B400000;
    float r = fmaf(n, -0.693145751953125f, x);        // ln 2, high part (exact product for |n| < 2^11)
    r = fmaf(n, -1.42860682030941723e-6f, r);         // ln 2, low part
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    // p * 2^e.  p lies in [0.70, 1.42] (|r| <= 0.35), so while e >= -125 the product is a normal number and the
    // scaling is exact: the exponent field takes e.  Below that - arguments under -86.6, where the result is a
    // denormal - two exact-or-once-rounded steps, so that the result rounds once.
    if (e >= -125)
        return __int_as_float(__float_as_int(p) + e * 8388608);  // e * 2^23: into the exponent field
    const int e1 = e / 2, e2 = e - e1;
    union { uint32_t u; float f; } s1, s2;
    s1.u = uint32_t(e1 + 127) << 23;
    s2.u = uint32_t(e2 + 127) << 23;
    return __fmul_rn(__fmul_rn(p, s1.f), s2.f);
}

__device__ __forceinline__ float ovk_erf_approx(float x)
{
    const float s = x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);  // sign(): 0 for 0
    const float a = fabsf(x);
    // (the correctly rounded reciprocal is the correctly rounded quotient 1 / d: the same bits, half the instructions)
    const float t = __frcp_rn(__fadd_rn(1.0f, __fmul_rn(0.3275911f, a)));
    float poly = __fmul_rn(t, 1.061405429f);
    poly = __fmul_rn(t, __fadd_rn(-1.453152027f, poly));
    poly = __fmul_rn(t, __fadd_rn(1.421413741f, poly));
    poly = __fmul_rn(t, __fadd_rn(-0.284496736f, poly));
    poly = __fmul_rn(t, __fadd_rn(0.254829592f, poly));
    const float ex = ovk_exp_ieee(__fmul_rn(-a, a));
    return __fmul_rn(s, __fsub_rn(1.0f, __fmul_rn(poly, ex)));
}

__device__ __forceinline__ float ovk_decomposed_gelu(float v, const GeluParams &g)
{
    const float e = __fadd_rn(ovk_erf_approx(__fdiv_rn(v, g.divisor)), g.offset);
    return g.factor_first ? __fmul_rn(v, __fmul_rn(e, g.factor)) : __fmul_rn(__fmul_rn(v, e), g.factor);
}
