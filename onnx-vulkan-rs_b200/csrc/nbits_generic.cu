// MatMulNBits, general form: any M, any block_size that is a multiple of 8,
// ragged K, optional zero points, f32/f16 activations, scales and outputs,
// read straight from the operator's own layout.
//
// It keeps the arithmetic of the reference's correctness kernel
// (crates/onnx-vulkan-core/src/shaders/matmul_nbits.rs:316-374): per 32-bit
// word `part = fma(nibble - z, a, part)` over its eight weights, then
// `acc = fma(part, scale, acc)`; here one warp owns a column and keeps up to
// four rows of A in flight, and the K reduction is a warp shuffle.
#include "ovk_internal.h"

namespace {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

constexpr int ROWS = 4;

template <typename TA, typename TS, typename TY>
__global__ void __launch_bounds__(256)
nbits_rows_kernel(const TA *__restrict__ a, const uint32_t *__restrict__ quant,
                  const TS *__restrict__ scales, const uint8_t *__restrict__ zp, TY *__restrict__ y,
                  int64_t M, int K, int N, int n_blocks, int blob_words, int block_size,
                  int zp_row_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t col = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (col >= N)
        return;
    const int words = n_blocks * blob_words;
    const uint32_t *q = quant + col * words;
    for (int64_t m0 = 0; m0 < M; m0 += ROWS) {
        float acc[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; r++)
            acc[r] = 0.0f;
        for (int w = lane; w < words; w += 32) {
            const int block = w / blob_words;
            const int k0 = block * block_size + (w % blob_words) * 8;
            const uint32_t word = __ldg(q + w);
            float z = 8.0f;
            if (zp)
                z = float((zp[col * zp_row_bytes + block / 2] >> (4 * (block & 1))) & 15);
            const float s = to_f32<TS>(scales[col * n_blocks + block]);
            float part[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; r++)
                part[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int k = k0 + i;
                if (k < K) {
                    const float wv = float((word >> (4 * i)) & 15u) - z;
#pragma unroll
                    for (int r = 0; r < ROWS; r++)
                        if (m0 + r < M)
                            part[r] = fmaf(wv, to_f32<TA>(a[(m0 + r) * K + k]), part[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < ROWS; r++)
                acc[r] = fmaf(part[r], s, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < ROWS; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m0 + r < M)
                y[(m0 + r) * N + col] = from_f32<TY>(v);
        }
    }
}

template <typename TA, typename TS, typename TY>
int32_t launch_rows(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int64_t m, void *y)
{
    const int warps_per_block = 8;
    const int64_t blocks = ceil_div64(w->n, warps_per_block);
    nbits_rows_kernel<TA, TS, TY><<<static_cast<unsigned>(blocks), warps_per_block * 32, 0, ctx->stream>>>(
        static_cast<const TA *>(a), reinterpret_cast<const uint32_t *>(w->b),
        static_cast<const TS *>(w->scales), w->zp, static_cast<TY *>(y), m, int(w->k), int(w->n),
        int(w->n_blocks), int(w->block_size / 8), int(w->block_size), int((w->n_blocks + 1) / 2));
    OVK_LAUNCHED(ctx, "nbits_rows");
    return OVK_OK;
}

}  // namespace

// Dispatch over the three real types; used by ovk_matmul_nbits for every form
// the tuned kernels do not take.
int32_t ovk_nbits_rows(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                       int64_t m, void *y, int32_t y_dtype)
{
    OVK_REQUIRE(ctx, aligned_to(w->b, 4), "MatMulNBits: packed weight is not 4-byte aligned");
    const bool ah = a_dtype == OVK_FLOAT16, sh = w->scales_dtype == OVK_FLOAT16, yh = y_dtype == OVK_FLOAT16;
#define GO(TA, TS, TY) return launch_rows<TA, TS, TY>(ctx, w, a, m, y)
    if (!ah && !sh && !yh) GO(float, float, float);
    if (!ah && !sh && yh) GO(float, float, __half);
    if (!ah && sh && !yh) GO(float, __half, float);
    if (!ah && sh && yh) GO(float, __half, __half);
    if (ah && !sh && !yh) GO(__half, float, float);
    if (ah && !sh && yh) GO(__half, float, __half);
    if (ah && sh && !yh) GO(__half, __half, float);
    GO(__half, __half, __half);
#undef GO
}
