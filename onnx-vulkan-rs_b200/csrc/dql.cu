// DynamicQuantizeLinear: range pass + quantize pass, both on the device.
//
// Follows interp::quantize_on_device (crates/onnx-vulkan-core/src/interp.rs
// :1977-2085) and the two shaders of src/shaders/dynamic_quantize.rs: PARTIAL
// (:106-152, min/max folded into an 8-byte slot by atomic max on the bit
// patterns of -min and max) and QUANTIZE (:160-222).  The reference needs a
// hand-made correctly rounded division (div_rn, :56-83) because Vulkan's
// OpFDiv may be 2.5 ULP off; CUDA's `/` without fast-math, spelled
// __fdiv_rn here, IS the IEEE division, so the results are bit-equal to the
// operator definition (tests/dynamic_quantize.rs:16-26) without it.
#include "ovk_internal.h"

namespace {

__device__ __forceinline__ void fold(float v, float &mn, float &mx)
{
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
}

// range[0] = bits of -min, range[1] = bits of max, both >= 0 so that unsigned
// order is float order; the slot is zero when the kernel starts (= range [0,0]): it is zeroed when
// the context is created and again by the last block of every quantize pass (range[2] counts them).
__global__ void __launch_bounds__(256)
dql_range_kernel(const float *__restrict__ x, int64_t n, uint32_t *__restrict__ range, int vec_ok)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    float mn = 0.0f, mx = 0.0f;  // 0 is always part of the range
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    if (vec_ok) {
        const int64_t n4 = n >> 2;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        // four independent 16-byte loads in flight per thread, and a quarter of the blocks: every
        // block ends with two atomics on the same two words, which is what a short input waits for
        int64_t i = tid;
        for (; i + 3 * stride < n4; i += 4 * stride) {
            const float4 v0 = __ldg(x4 + i), v1 = __ldg(x4 + i + stride), v2 = __ldg(x4 + i + 2 * stride),
                         v3 = __ldg(x4 + i + 3 * stride);
            fold(v0.x, mn, mx); fold(v0.y, mn, mx); fold(v0.z, mn, mx); fold(v0.w, mn, mx);
            fold(v1.x, mn, mx); fold(v1.y, mn, mx); fold(v1.z, mn, mx); fold(v1.w, mn, mx);
            fold(v2.x, mn, mx); fold(v2.y, mn, mx); fold(v2.z, mn, mx); fold(v2.w, mn, mx);
            fold(v3.x, mn, mx); fold(v3.y, mn, mx); fold(v3.z, mn, mx); fold(v3.w, mn, mx);
        }
        for (; i < n4; i += stride) {
            const float4 v = __ldg(x4 + i);
            fold(v.x, mn, mx);
            fold(v.y, mn, mx);
            fold(v.z, mn, mx);
            fold(v.w, mn, mx);
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
            fold(x[i], mn, mx);
    } else {
        for (int64_t i = tid; i < n; i += stride)
            fold(x[i], mn, mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float smn[8], smx[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        smn[warp] = mn;
        smx[warp] = mx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) {
            mn = fminf(mn, smn[w]);
            mx = fmaxf(mx, smx[w]);
        }
        // the mask turns a -0.0 into 0 (shader :143-145)
        atomicMax(range + 0, __float_as_uint(-mn) & 0x7fffffffu);
        atomicMax(range + 1, __float_as_uint(mx) & 0x7fffffffu);
    }
}

__device__ __forceinline__ void scale_zp_from_range(const uint32_t *range, float &scale, float &zp)
{
    const float mn = -__uint_as_float(range[0]);
    const float mx = __uint_as_float(range[1]);
    scale = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
    if (scale == 0.0f)
        scale = 1.0f;
    zp = rintf(fminf(fmaxf(__fdiv_rn(-mn, scale), 0.0f), 255.0f));
}

__device__ __forceinline__ uint32_t quant1(float v, float scale, float zp)
{
    const float q = __fadd_rn(rintf(__fdiv_rn(v, scale)), zp);
    return uint32_t(fminf(fmaxf(q, 0.0f), 255.0f));
}

__global__ void __launch_bounds__(256)
dql_quantize_kernel(const float *__restrict__ x, int64_t n, uint32_t *__restrict__ range,
                    float *__restrict__ scale_out, uint8_t *__restrict__ zp_out,
                    uint8_t *__restrict__ y, int vec_ok)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    __shared__ float s_scale, s_zp;
    if (threadIdx.x == 0) {
        float scale, zp;
        scale_zp_from_range(range, scale, zp);
        s_scale = scale;
        s_zp = zp;
        if (blockIdx.x == 0) {
            scale_out[0] = scale;
            zp_out[0] = uint8_t(zp);
        }
        // the block that reads the range last leaves the slot zeroed for the next call
        __threadfence();
        if (atomicAdd(range + 2, 1u) == gridDim.x - 1) {
            range[0] = 0u;
            range[1] = 0u;
            range[2] = 0u;
        }
    }
    __syncthreads();
    const float scale = s_scale, zp = s_zp;
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    if (vec_ok) {
        const int64_t n4 = n >> 2;
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        uint32_t *y4 = reinterpret_cast<uint32_t *>(y);
        auto pack = [&](const float4 &v) {
            return quant1(v.x, scale, zp) | (quant1(v.y, scale, zp) << 8) | (quant1(v.z, scale, zp) << 16) |
                   (quant1(v.w, scale, zp) << 24);
        };
        int64_t i = tid;
        for (; i + 3 * stride < n4; i += 4 * stride) {
            const float4 v0 = __ldg(x4 + i), v1 = __ldg(x4 + i + stride), v2 = __ldg(x4 + i + 2 * stride),
                         v3 = __ldg(x4 + i + 3 * stride);
            y4[i] = pack(v0);
            y4[i + stride] = pack(v1);
            y4[i + 2 * stride] = pack(v2);
            y4[i + 3 * stride] = pack(v3);
        }
        for (; i < n4; i += stride)
            y4[i] = pack(__ldg(x4 + i));
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
            y[i] = uint8_t(quant1(x[i], scale, zp));
    } else {
        for (int64_t i = tid; i < n; i += stride)
            y[i] = uint8_t(quant1(x[i], scale, zp));
    }
}

__global__ void dql_identity_kernel(float *scale_out, uint8_t *zp_out)
{
    scale_out[0] = 1.0f;
    zp_out[0] = 0;
}

}  // namespace

extern "C" int32_t ovk_dynamic_quantize(ovk_ctx *ctx, const float *x, int64_t n, uint8_t *y,
                                        float *y_scale, uint8_t *y_zero_point)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_dynamic_quantize: null context");
    OVK_REQUIRE(ctx, n >= 0, "DynamicQuantizeLinear: negative element count");
    OVK_REQUIRE(ctx, y_scale && y_zero_point, "DynamicQuantizeLinear: y_scale or y_zero_point is null");
    OVK_REQUIRE(ctx, aligned_to(y_scale, 4), "DynamicQuantizeLinear: y_scale is not 4-byte aligned");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n == 0) {  // empty input: scale 1, zero point 0 (interp.rs:1949-1966)
        dql_identity_kernel<<<1, 1, 0, ctx->stream>>>(y_scale, y_zero_point);
        OVK_LAUNCHED(ctx, "dql_identity");
        return OVK_OK;
    }
    OVK_REQUIRE(ctx, x && y, "DynamicQuantizeLinear: x or y is null");
    OVK_REQUIRE(ctx, aligned_to(x, 4), "DynamicQuantizeLinear: x is not 4-byte aligned");
    const int vec_ok = aligned_to(x, 16) && aligned_to(y, 4);
    const int64_t work = vec_ok ? (n + 3) / 4 : n;
    // both passes: grid-stride, four vectors per thread and trip, at most four blocks per SM
    unsigned blocks1 = unsigned(std::min<int64_t>(ceil_div64(work, 1024), int64_t(ctx->sm_count) * 4));
    OVK_CUDA(ctx, ovk_launch_pdl(dql_range_kernel, dim3(blocks1), dim3(256), 0, ctx->stream, x, n, ctx->range_slot, vec_ok));
    OVK_LAUNCHED(ctx, "dql_range");
    unsigned blocks2 = blocks1;
    OVK_CUDA(ctx, ovk_launch_pdl(dql_quantize_kernel, dim3(blocks2), dim3(256), 0, ctx->stream, x, n, ctx->range_slot, y_scale,
                                 y_zero_point, y, vec_ok));
    OVK_LAUNCHED(ctx, "dql_quantize");
    return OVK_OK;
}
