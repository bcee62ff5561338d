// DynamicQuantizeLinear: range pass + quantize pass, both on the device - as two launches, or, when
// the tensor fits in the registers of one block per SM, as ONE launch whose blocks meet at a counter.
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
#include "gelu.cuh"

namespace {

// What the passes read: x itself, or DecomposedGelu(x) computed on the fly (the
// reference's gelu_partial / gelu_quantize shaders, shaders/dynamic_quantize.rs:224-247,
// whose load() is the GELU: its f32 result is never stored).
struct LoadPlain {
    __device__ __forceinline__ float operator()(float v) const { return v; }
};
struct LoadGelu {
    GeluParams g;
    __device__ __forceinline__ float operator()(float v) const { return ovk_decomposed_gelu(v, g); }
};

__device__ __forceinline__ void fold(float v, float &mn, float &mx)
{
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
}

// range[0] = bits of -min, range[1] = bits of max, both >= 0 so that unsigned
// order is float order; the slot is zero when the kernel starts (= range [0,0]): it is zeroed when
// the context is created and again by the last block of every quantize pass (range[2] counts them).
template <typename Load>
__global__ void __launch_bounds__(256)
dql_range_kernel(const float *__restrict__ x, int64_t n, uint32_t *__restrict__ range, int vec_ok, Load load)
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
            fold(load(v0.x), mn, mx); fold(load(v0.y), mn, mx); fold(load(v0.z), mn, mx); fold(load(v0.w), mn, mx);
            fold(load(v1.x), mn, mx); fold(load(v1.y), mn, mx); fold(load(v1.z), mn, mx); fold(load(v1.w), mn, mx);
            fold(load(v2.x), mn, mx); fold(load(v2.y), mn, mx); fold(load(v2.z), mn, mx); fold(load(v2.w), mn, mx);
            fold(load(v3.x), mn, mx); fold(load(v3.y), mn, mx); fold(load(v3.z), mn, mx); fold(load(v3.w), mn, mx);
        }
        for (; i < n4; i += stride) {
            const float4 v = __ldg(x4 + i);
            fold(load(v.x), mn, mx);
            fold(load(v.y), mn, mx);
            fold(load(v.z), mn, mx);
            fold(load(v.w), mn, mx);
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
            fold(load(x[i]), mn, mx);
    } else {
        for (int64_t i = tid; i < n; i += stride)
            fold(load(x[i]), mn, mx);
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

template <typename Load>
__global__ void __launch_bounds__(256)
dql_quantize_kernel(const float *__restrict__ x, int64_t n, uint32_t *__restrict__ range,
                    float *__restrict__ scale_out, uint8_t *__restrict__ zp_out,
                    uint8_t *__restrict__ y, int vec_ok, Load load)
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
            return quant1(load(v.x), scale, zp) | (quant1(load(v.y), scale, zp) << 8) |
                   (quant1(load(v.z), scale, zp) << 16) | (quant1(load(v.w), scale, zp) << 24);
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
            y[i] = uint8_t(quant1(load(x[i]), scale, zp));
    } else {
        for (int64_t i = tid; i < n; i += stride)
            y[i] = uint8_t(quant1(load(x[i]), scale, zp));
    }
}

// Both passes in one launch.  Every thread keeps its (loaded, for the GELU form already transformed)
// values in registers: up to VPT vectors of four, so x is read once and the GELU is evaluated once.
// Between the passes the blocks meet at a counter: slot[0], slot[1] take the folded range, slot[2]
// counts arrivals, slot[3] departures; the block that leaves last zeroes all four for the next call.
// The launch has at most one block per SM and a block waits for nothing but its siblings, which wait
// for nothing but a free SM, so the meeting cannot deadlock; the wait is bounded all the same and a
// limit that runs out is reported through the status word (the bytes are then quantized with whatever
// range had arrived).
constexpr int ONE_PASS_THREADS = 1024;
constexpr int ONE_PASS_VPT_MAX = 8;

template <typename Load, int VPT>
__global__ void __launch_bounds__(ONE_PASS_THREADS, 1)
dql_one_pass_kernel(const float4 *__restrict__ x4, int64_t n4, uint32_t *__restrict__ slot, float *__restrict__ scale_out,
                    uint8_t *__restrict__ zp_out, uint32_t *__restrict__ y4, Load load, int *status, long long wait_cycles)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    const int64_t first = int64_t(blockIdx.x) * ONE_PASS_THREADS + threadIdx.x;
    const int64_t stride = int64_t(gridDim.x) * ONE_PASS_THREADS;
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {  // every load is issued before the first value is used
        const int64_t i = first + j * stride;
        v[j] = i < n4 ? __ldg(x4 + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float mn = 0.0f, mx = 0.0f;  // 0 is always part of the range
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        if (first + j * stride < n4) {
            v[j].x = load(v[j].x);
            v[j].y = load(v[j].y);
            v[j].z = load(v[j].z);
            v[j].w = load(v[j].w);
            fold(v[j].x, mn, mx);
            fold(v[j].y, mn, mx);
            fold(v[j].z, mn, mx);
            fold(v[j].w, mn, mx);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    __shared__ float smn[32], smx[32], s_scale, s_zp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        smn[warp] = mn;
        smx[warp] = mx;
    }
    __syncthreads();
    if (warp == 0) {
        mn = smn[lane];
        mx = smx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (lane == 0) {
            atomicMax(slot + 0, __float_as_uint(-mn) & 0x7fffffffu);
            atomicMax(slot + 1, __float_as_uint(mx) & 0x7fffffffu);
            __threadfence();
            atomicAdd(slot + 2, 1u);
            const long long t0 = clock64();
            while (comm::ld_acquire_gpu(slot + 2) < gridDim.x) {
                if (clock64() - t0 > wait_cycles) {
                    atomicExch(status, OVK_DEV_TIMEOUT_GRID);
                    break;
                }
                __nanosleep(32);
            }
            float scale, zp;
            const uint32_t folded[2] = {__ldcg(slot + 0), __ldcg(slot + 1)};
            scale_zp_from_range(folded, scale, zp);
            s_scale = scale;
            s_zp = zp;
            if (blockIdx.x == 0) {
                scale_out[0] = scale;
                zp_out[0] = uint8_t(zp);
            }
            if (atomicAdd(slot + 3, 1u) == gridDim.x - 1) {
                slot[0] = 0u;
                slot[1] = 0u;
                slot[2] = 0u;
                slot[3] = 0u;
            }
        }
    }
    __syncthreads();
    const float scale = s_scale, zp = s_zp;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int64_t i = first + j * stride;
        if (i < n4)
            y4[i] = quant1(v[j].x, scale, zp) | (quant1(v[j].y, scale, zp) << 8) | (quant1(v[j].z, scale, zp) << 16) |
                    (quant1(v[j].w, scale, zp) << 24);
    }
}

__global__ void dql_identity_kernel(float *scale_out, uint8_t *zp_out)
{
    scale_out[0] = 1.0f;
    zp_out[0] = 0;
}

__global__ void __launch_bounds__(256)
gelu_kernel(const float *__restrict__ x, int64_t n, float *__restrict__ out, GeluParams g)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        out[i] = ovk_decomposed_gelu(x[i], g);
}

// Both passes, or - when `folded` is a slot a producer has already folded the range of x into - only
// the second one (interp.rs:1979-1983).
template <typename Load>
int32_t quantize_passes(ovk_ctx *ctx, const char *what, const float *x, int64_t n, uint32_t *folded, uint8_t *y,
                        float *y_scale, uint8_t *y_zero_point, Load load)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "%s: null context", what);
    OVK_REQUIRE(ctx, n >= 0, "%s: negative element count", what);
    OVK_REQUIRE(ctx, y_scale && y_zero_point, "%s: y_scale or y_zero_point is null", what);
    OVK_REQUIRE(ctx, aligned_to(y_scale, 4), "%s: y_scale is not 4-byte aligned", what);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n == 0) {  // empty input: scale 1, zero point 0 (interp.rs:1949-1966)
        dql_identity_kernel<<<1, 1, 0, ctx->stream>>>(y_scale, y_zero_point);
        OVK_LAUNCHED(ctx, "dql_identity");
        return OVK_OK;
    }
    OVK_REQUIRE(ctx, x && y, "%s: x or y is null", what);
    OVK_REQUIRE(ctx, aligned_to(x, 4), "%s: x is not 4-byte aligned", what);
    OVK_REQUIRE(ctx, !folded || aligned_to(folded, 4), "%s: the range slot is not 4-byte aligned", what);
    const int vec_ok = aligned_to(x, 16) && aligned_to(y, 4);
    const int64_t work = vec_ok ? (n + 3) / 4 : n;
    // both passes: grid-stride, four vectors per thread and trip, at most four blocks per SM
    const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(work, 1024), int64_t(ctx->sm_count) * 4));
    uint32_t *range = folded ? folded : ctx->range_slot;
    if (!folded && vec_ok && n % 4 == 0) {
        const int64_t n4 = n / 4;
        const int64_t grid = std::min<int64_t>(ctx->sm_count, ceil_div64(n4, ONE_PASS_THREADS));
        const int64_t per_thread = ceil_div64(n4, grid * ONE_PASS_THREADS);
        if (per_thread <= ONE_PASS_VPT_MAX) {
            uint32_t *slot = ctx->range_slot + 4;  // four words of its own, zero between calls
            const float4 *x4 = reinterpret_cast<const float4 *>(x);
            uint32_t *y4 = reinterpret_cast<uint32_t *>(y);
            const long long limit = 2000000000ll;  // about a second
#define OVK_ONE_PASS(V)                                                                                               \
    OVK_CUDA(ctx, ovk_launch_pdl(dql_one_pass_kernel<Load, V>, dim3(unsigned(grid)), dim3(ONE_PASS_THREADS), 0, ctx->stream, \
                                 x4, n4, slot, y_scale, y_zero_point, y4, load, ctx->dev_status, limit))
            if (per_thread <= 1) OVK_ONE_PASS(1);
            else if (per_thread <= 2) OVK_ONE_PASS(2);
            else if (per_thread <= 4) OVK_ONE_PASS(4);
            else OVK_ONE_PASS(8);
#undef OVK_ONE_PASS
            OVK_LAUNCHED(ctx, "dql_one_pass");
            return OVK_OK;
        }
    }
    if (!folded) {
        OVK_CUDA(ctx, ovk_launch_pdl(dql_range_kernel<Load>, dim3(blocks), dim3(256), 0, ctx->stream, x, n, range, vec_ok, load));
        OVK_LAUNCHED(ctx, "dql_range");
    }
    OVK_CUDA(ctx, ovk_launch_pdl(dql_quantize_kernel<Load>, dim3(blocks), dim3(256), 0, ctx->stream, x, n, range, y_scale,
                                 y_zero_point, y, vec_ok, load));
    OVK_LAUNCHED(ctx, "dql_quantize");
    return OVK_OK;
}

}  // namespace

extern "C" int32_t ovk_dynamic_quantize(ovk_ctx *ctx, const float *x, int64_t n, uint8_t *y,
                                        float *y_scale, uint8_t *y_zero_point)
{
    return quantize_passes(ctx, "DynamicQuantizeLinear", x, n, nullptr, y, y_scale, y_zero_point, LoadPlain{});
}

extern "C" int32_t ovk_dynamic_quantize_folded(ovk_ctx *ctx, const float *x, int64_t n, uint32_t *range, uint8_t *y,
                                               float *y_scale, uint8_t *y_zero_point)
{
    if (ctx && !range)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "DynamicQuantizeLinear: the folded range is null");
    return quantize_passes(ctx, "DynamicQuantizeLinear", x, n, range, y, y_scale, y_zero_point, LoadPlain{});
}

extern "C" int32_t ovk_decomposed_gelu(ovk_ctx *ctx, const float *x, int64_t n, float divisor, float offset, float factor,
                                       int32_t factor_first, float *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "DecomposedGelu: null context");
    OVK_REQUIRE(ctx, n >= 0, "DecomposedGelu: negative element count");
    if (n == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && out, "DecomposedGelu: x or the output is null");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    const GeluParams g = {divisor, offset, factor, factor_first ? 1 : 0};
    const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(n, 256), int64_t(ctx->sm_count) * 8));
    OVK_CUDA(ctx, ovk_launch_pdl(gelu_kernel, dim3(blocks), dim3(256), 0, ctx->stream, x, n, out, g));
    OVK_LAUNCHED(ctx, "decomposed_gelu");
    return OVK_OK;
}

extern "C" int32_t ovk_decomposed_gelu_quantize(ovk_ctx *ctx, const float *x, int64_t n, float divisor, float offset,
                                                float factor, int32_t factor_first, uint8_t *y, float *y_scale,
                                                uint8_t *y_zero_point)
{
    LoadGelu load;
    load.g = {divisor, offset, factor, factor_first ? 1 : 0};
    return quantize_passes(ctx, "DecomposedGeluQuantize", x, n, nullptr, y, y_scale, y_zero_point, load);
}
