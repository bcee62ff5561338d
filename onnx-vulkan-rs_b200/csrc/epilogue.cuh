// What happens to an int32 accumulator after the K loop, shared by every
// integer kernel (small-shape, tensor-core GEMM, convolution).
//
//  1. zero-point correction, the algebra of the reference's cooperative kernel
//     (crates/onnx-vulkan-core/src/shaders/glsl/matmul_integer_coop.comp:22-33):
//       sum (a - za)(b - zb) = sum ab - za*sum_k b - zb*sum_k a + K*za*zb
//  2. one of three stores:
//       RAW      the int32 itself (MatMulInteger / ConvInteger)
//       SCALE    fl(fl(float(acc) * s) + bias), s = scale [* product], optional
//                Relu and range fold (matmul_integer_coop.comp:156-196): every
//                multiply and add separately rounded, never contracted
//       REQUANT  sat(rne(f32(acc + bias[c]) * ratio[c]) + y_zp)
//                (src/shaders/qlinear.rs:28-63)
#pragma once
#include <cstdint>

enum : int { EPI_RAW = 0, EPI_SCALE = 1, EPI_REQUANT = 2 };

struct EpiParams {
    int mode;
    // SCALE
    const float *scale;
    const float *product;
    const float *fbias;
    int scale_step, product_step, bias_step;
    unsigned flags;  // OVK_EPILOGUE_RELU | OVK_EPILOGUE_RANGE
    uint32_t *range;
    // REQUANT (channel index c = column for a matmul, filter for a convolution)
    const float *ratio;
    int ratio_step;
    const int32_t *ibias;
    int y_zp;
    int y_signed;
    // 1: the per-channel constants above belong to the ROWS of the product, not its columns (a pointwise
    // convolution computed as filters x pixels, whose rows are the output channels)
    int by_row;
};

__device__ __forceinline__ int32_t load_zp(const void *p, int is_signed)
{
    if (!p)
        return 0;
    const uint8_t b = *static_cast<const uint8_t *>(p);
    return is_signed ? int32_t(int8_t(b)) : int32_t(b);
}

__device__ __forceinline__ float epi_scale_value(const EpiParams &e, int64_t c, float x)
{
    float s = e.scale[c * e.scale_step];
    if (e.product)
        s = __fmul_rn(s, e.product[c * e.product_step]);
    const float y = __fmul_rn(x, s);
    const float z = __fadd_rn(y, e.fbias[c * e.bias_step]);
    return (e.flags & 1u) ? fmaxf(z, 0.0f) : z;
}

__device__ __forceinline__ int32_t epi_requant_value(const EpiParams &e, int64_t c, int32_t acc)
{
    if (e.ibias)
        acc = int32_t(uint32_t(acc) + uint32_t(e.ibias[c]));
    const float r = rintf(__fmul_rn(float(acc), e.ratio[c * e.ratio_step]));
    int32_t q = int32_t(uint32_t(__float2int_rn(r)) + uint32_t(e.y_zp));
    // __float2int_rn saturates like the reference's i32(); detect the wrap of "+ y_zp"
    if (e.y_signed)
        q = max(-128, min(127, q));
    else
        q = max(0, min(255, q));
    return q;
}

// Folds per-thread extrema into the shared range slot: one atomic pair per warp.
__device__ __forceinline__ void epi_fold_range(const EpiParams &e, float run_max, float run_neg)
{
    if (!(e.flags & 2u) || !e.range)
        return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        run_max = fmaxf(run_max, __shfl_xor_sync(0xffffffffu, run_max, o));
        run_neg = fmaxf(run_neg, __shfl_xor_sync(0xffffffffu, run_neg, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(e.range + 0, __float_as_uint(run_neg) & 0x7fffffffu);
        atomicMax(e.range + 1, __float_as_uint(run_max) & 0x7fffffffu);
    }
}
