// MatMulNBits host side: validation, once-per-weight preparation and routing.
// Mirrors interp::matmul_nbits (crates/onnx-vulkan-core/src/interp.rs:6429-6561),
// its load-time predicate (:452-464) and shaders::matmul_nbits::route
// (src/shaders/matmul_nbits.rs:430-436).
#include "ovk_internal.h"

int32_t ovk_nbits_rows(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                       int64_t m, void *y, int32_t y_dtype);
int32_t ovk_nbits_decode_prepack(ovk_ctx *ctx, ovk_nbits_weight *w);
bool ovk_nbits_decode_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, int32_t a_dtype,
                              int32_t y_dtype);
int32_t ovk_nbits_decode(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                         int64_t m, void *y, int32_t y_dtype);
bool ovk_nbits_decode_group_compatible(const ovk_nbits_weight *a, const ovk_nbits_weight *b);
int32_t ovk_nbits_decode_group(ovk_ctx *ctx, int count, const ovk_nbits_weight *const *ws, const void *a, int32_t a_dtype,
                               int64_t m, void *const *ys, int32_t y_dtype);
bool ovk_nbits_gemm_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, int32_t a_dtype,
                            int32_t y_dtype, const void *a, const void *y);
int32_t ovk_nbits_gemm(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                       int64_t m, void *y, int32_t y_dtype);

extern "C" {

int32_t ovk_nbits_prepack(ovk_ctx *ctx, const void *b, const void *scales, int32_t scales_dtype,
                          const void *zero_points, int64_t n, int64_t k, int64_t bits,
                          int64_t block_size, uint32_t flags, ovk_nbits_weight **out)
{
    if (!ctx || !out)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_nbits_prepack: null argument");
    *out = nullptr;
    // the claim predicate of the reference (interp.rs:452-464)
    OVK_REFUSE(ctx, bits != 4, "MatMulNBits: bits=%lld is not supported (4 only)", (long long)bits);
    OVK_REFUSE(ctx, block_size <= 0 || block_size % 8 != 0,
               "MatMulNBits: block_size=%lld must be a positive multiple of 8", (long long)block_size);
    OVK_REQUIRE(ctx, k > 0 && n > 0, "MatMulNBits: K=%lld N=%lld must be positive", (long long)k, (long long)n);
    OVK_REQUIRE(ctx, b && scales, "MatMulNBits: packed weight or scales missing");
    OVK_REFUSE(ctx, scales_dtype != OVK_FLOAT && scales_dtype != OVK_FLOAT16,
               "MatMulNBits: expected u8 weight and zero point with f32 or f16 scales, got scales dtype %d",
               scales_dtype);
    OVK_REQUIRE(ctx, k < (int64_t(1) << 31) && n < (int64_t(1) << 31), "MatMulNBits: K or N too large");
    ovk_nbits_weight *w = new ovk_nbits_weight();
    w->b = static_cast<const uint8_t *>(b);
    w->scales = scales;
    w->zp = static_cast<const uint8_t *>(zero_points);
    w->scales_dtype = scales_dtype;
    w->n = n;
    w->k = k;
    w->block_size = block_size;
    w->n_blocks = ceil_div64(k, block_size);
    if (!(flags & OVK_NBITS_NO_DECODE_COPY)) {
        int32_t rc = ovk_nbits_decode_prepack(ctx, w);
        if (rc != OVK_OK) {
            delete w;
            return rc;
        }
        // a load-time call: wait for the copy, so that the decode kernel (which starts
        // streaming weights before its stream predecessors have finished) never sees it half written
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) {
            cudaFree(w->decode);
            delete w;
            return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: weight preparation: %s", cudaGetErrorString(e));
        }
    }
    *out = w;
    return OVK_OK;
}

void ovk_nbits_weight_destroy(ovk_ctx *ctx, ovk_nbits_weight *w)
{
    if (!w)
        return;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    cudaFree(w->decode);
    cudaFree(w->gemm_w);
    delete w;
}

int32_t ovk_matmul_nbits(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                         int64_t m, void *y, int32_t y_dtype)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_matmul_nbits: null argument");
    OVK_REQUIRE(ctx, m >= 0, "MatMulNBits: %lld rows of A", (long long)m);
    OVK_REFUSE(ctx, (a_dtype != OVK_FLOAT && a_dtype != OVK_FLOAT16) ||
                        (y_dtype != OVK_FLOAT && y_dtype != OVK_FLOAT16),
               "MatMulNBits: A and Y must be f32 or f16, got %d/%d", a_dtype, y_dtype);
    if (m == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, a && y, "MatMulNBits: A or Y is null");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (ovk_nbits_decode_applies(ctx, w, m, a_dtype, y_dtype))
        return ovk_nbits_decode(ctx, w, a, a_dtype, m, y, y_dtype);
    if (ovk_nbits_gemm_applies(ctx, w, m, a_dtype, y_dtype, a, y))
        return ovk_nbits_gemm(ctx, w, a, a_dtype, m, y, y_dtype);
    return ovk_nbits_rows(ctx, w, a, a_dtype, m, y, y_dtype);
}

// Several weights over the same activations in one launch where the decode kernel applies and the
// weights have the same tile shape; otherwise one call per weight.
int32_t ovk_matmul_nbits_group(ovk_ctx *ctx, int32_t count, const ovk_nbits_weight *const *weights, const void *a,
                               int32_t a_dtype, int64_t m, void *const *ys, int32_t y_dtype)
{
    if (!ctx || !weights || !ys)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_matmul_nbits_group: null argument");
    OVK_REQUIRE(ctx, count >= 1 && count <= 4, "MatMulNBits: a group of %d weights (1 to 4)", count);
    for (int j = 0; j < count; j++)
        OVK_REQUIRE(ctx, weights[j] && (ys[j] || m == 0), "MatMulNBits: member %d of the group is null", j);
    for (int j = 1; j < count; j++)
        OVK_REQUIRE(ctx, weights[j]->k == weights[0]->k, "MatMulNBits: member %d of the group has K=%lld, member 0 K=%lld", j,
                    (long long)weights[j]->k, (long long)weights[0]->k);
    bool together = count > 1 && m >= 1 && m <= 8 && a &&
                    (a_dtype == OVK_FLOAT || a_dtype == OVK_FLOAT16) && (y_dtype == OVK_FLOAT || y_dtype == OVK_FLOAT16);
    for (int j = 0; together && j < count; j++)
        together = ovk_nbits_decode_applies(ctx, weights[j], m, a_dtype, y_dtype) &&
                   ovk_nbits_decode_group_compatible(weights[0], weights[j]);
    if (together) {
        OVK_CUDA(ctx, cudaSetDevice(ctx->device));
        return ovk_nbits_decode_group(ctx, count, weights, a, a_dtype, m, ys, y_dtype);
    }
    for (int j = 0; j < count; j++) {
        const int32_t rc = ovk_matmul_nbits(ctx, weights[j], a, a_dtype, m, ys[j], y_dtype);
        if (rc != OVK_OK)
            return rc;
    }
    return OVK_OK;
}

}  // extern "C"
