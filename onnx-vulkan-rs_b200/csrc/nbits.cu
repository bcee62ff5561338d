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
bool ovk_nbits_gemm_f32_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, const void *a, const void *y);
int32_t ovk_nbits_gemm_f32(ovk_ctx *ctx, const ovk_nbits_weight *w, const float *a, int64_t m, void *y, int32_t y_dtype);
bool ovk_nbits_gemm_is_per_block(const ovk_ctx *ctx, const ovk_nbits_weight *w);
int32_t ovk_nbits_gemm_into(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int64_t m, void *const *y_dst,
                            int n_dst, int64_t ldy, int64_t col0, int32_t y_dtype, const OvkCommView *view, void *y_multicast);
int32_t ovk_comm_gather_cols(ovk_ctx *ctx, const OvkCommView &view, const void *src, size_t src_pitch, int elem_bytes,
                             int64_t m, int64_t n_shard, int64_t col0, int64_t n_total, void *const *y_peers,
                             bool skip_self, void *y_multicast);

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
    if (a_dtype == OVK_FLOAT && ovk_nbits_gemm_f32_applies(ctx, w, m, a, y))
        return ovk_nbits_gemm_f32(ctx, w, static_cast<const float *>(a), m, y, y_dtype);
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

#ifndef OVK_NSPLIT_FUSED_MAX_RANKS
#define OVK_NSPLIT_FUSED_MAX_RANKS 4
#endif

// One rank's share of a MatMulNBits split over weight columns, exchange included.
//
// The prefill kernel with per-block scaling stores every finished tile into every rank's matrix
// itself (the exchange rides on the product); the other kernels compute this rank's column block
// - in place inside its own matrix where they can take a row pitch, in a temporary otherwise - and
// the exchange kernel spreads it.  Either way the call returns with one wait enqueued behind it:
// until every peer's stores into this rank's matrix have been announced.
int32_t ovk_matmul_nbits_nsplit(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype, int64_t m,
                                int64_t col0, int64_t n_total, void *const *y_peers, int32_t y_dtype)
{
    return ovk_matmul_nbits_nsplit_multicast(ctx, w, a, a_dtype, m, col0, n_total, y_peers, nullptr, y_dtype);
}

int32_t ovk_matmul_nbits_nsplit_multicast(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype, int64_t m,
                                          int64_t col0, int64_t n_total, void *const *y_peers, void *y_multicast,
                                          int32_t y_dtype)
{
    if (!ctx || !w || !y_peers)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_matmul_nbits_nsplit: null argument");
    const int world = ctx->comm.world, rank = ctx->comm.rank;
    OVK_REQUIRE(ctx, world >= 1, "MatMulNBits (column split): ovk_comm_init has not been called");
    OVK_REQUIRE(ctx, m >= 0, "MatMulNBits: %lld rows of A", (long long)m);
    OVK_REFUSE(ctx, (a_dtype != OVK_FLOAT && a_dtype != OVK_FLOAT16) || (y_dtype != OVK_FLOAT && y_dtype != OVK_FLOAT16),
               "MatMulNBits: A and Y must be f32 or f16, got %d/%d", a_dtype, y_dtype);
    OVK_REQUIRE(ctx, col0 >= 0 && col0 + w->n <= n_total && n_total < (int64_t(1) << 31),
                "MatMulNBits (column split): columns [%lld, %lld) of %lld", (long long)col0, (long long)(col0 + w->n),
                (long long)n_total);
    for (int r = 0; r < world; r++)
        OVK_REQUIRE(ctx, y_peers[r], "MatMulNBits (column split): the matrix of rank %d is null", r);
    OVK_REQUIRE(ctx, m == 0 || a, "MatMulNBits: A is null");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int es = y_dtype == OVK_FLOAT16 ? 2 : 4;
    const OvkCommView view = ovk_comm_next(ctx);  // every rank counts the call, also one with no rows
    void *own = y_peers[rank];
    void *own_block = static_cast<uint8_t *>(own) + size_t(col0) * es;
    if (m == 0)
        return ovk_comm_gather_cols(ctx, view, own_block, size_t(n_total) * es, es, 0, w->n, col0, n_total, y_peers, true, y_multicast);
    const bool prefill = ovk_nbits_gemm_applies(ctx, w, m, a_dtype, y_dtype, a, own_block);
    // The exchange inside the product (every tile stored into every rank's Y as it is finished) up to four ranks;
    // beyond, the product into this rank's own Y and then the all-gather kernel: at eight ranks every CTA's store
    // warp has seven peers to write, the links carry 7/8 of Y per GPU against a product of an eighth the size,
    // and the step in two kernels measured faster (gate|up of a 7B model, M = 4096: 0.389 ms fused against
    // 0.093 + 0.255 ms; at four ranks 0.240 fused against 0.151 + 0.226).
    if (prefill && ovk_nbits_gemm_is_per_block(ctx, w) && y_dtype == OVK_FLOAT16 && world <= OVK_NSPLIT_FUSED_MAX_RANKS) {
        int32_t rc = ovk_nbits_gemm_into(ctx, w, a, m, y_peers, world, n_total, col0, y_dtype, &view, y_multicast);
        if (rc != OVK_OK)
            return rc;
        return world > 1 ? ovk_comm_wait_done(ctx, view) : OVK_OK;
    }
    if (prefill) {
        void *dst[1] = {own};
        int32_t rc = ovk_nbits_gemm_into(ctx, w, a, m, dst, 1, n_total, col0, y_dtype, nullptr, nullptr);
        if (rc != OVK_OK)
            return rc;
        return ovk_comm_gather_cols(ctx, view, own_block, size_t(n_total) * es, es, m, w->n, col0, n_total, y_peers, true, y_multicast);
    }
    // kernels that write a contiguous [m, N] result: through a temporary
    void *tmp = nullptr;
    OVK_CUDA(ctx, cudaMallocAsync(&tmp, size_t(m) * w->n * es + 256, ctx->stream));
    int32_t rc = ovk_matmul_nbits(ctx, w, a, a_dtype, m, tmp, y_dtype);
    if (rc == OVK_OK)
        rc = ovk_comm_gather_cols(ctx, view, tmp, size_t(w->n) * es, es, m, w->n, col0, n_total, y_peers, false, y_multicast);
    cudaFreeAsync(tmp, ctx->stream);
    return rc;
}

}  // extern "C"
