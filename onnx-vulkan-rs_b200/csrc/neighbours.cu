// The two launches either side of the lm_head product in a decode step:
// GatherBlockQuantized (the int4 embedding row of the token) and the greedy
// ArgMax over the logits.  Both are latency-sized; they exist so that a decode
// loop never leaves the device between the token index and the next one.
//
// Reference: crates/onnx-vulkan-core/src/shaders/gather_block_quantized.rs:26-57
// with interp::gather_block_quantized (src/interp.rs:2874-2990), and
// shaders/reduction.rs:76-190 with interp::arg_extreme_axis (src/interp.rs:8552-8690).
#include "ovk_internal.h"

namespace {

// ---------------------------------------------------------------- gather
// One thread per 32-bit word of the gathered rows: eight nibbles, one zero
// point, one scale, (q - z) * scale in f32 exactly as the reference's kernel.
template <bool SCALE_F32, bool OUT_F32, bool IDX64>
__global__ void __launch_bounds__(256)
gather_block_quantized_kernel(const uint32_t *__restrict__ table, const void *__restrict__ indices,
                              const void *__restrict__ scales, const uint8_t *__restrict__ zp, void *__restrict__ out,
                              int64_t count_words, int words_per_row, int64_t rows, int n_blocks, int block_size,
                              int zp_row_bytes, int *status)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count_words)
        return;
    const int64_t j = i / words_per_row;
    const int word = int(i - j * words_per_row);
    int64_t row = IDX64 ? static_cast<const int64_t *>(indices)[j] : int64_t(static_cast<const int32_t *>(indices)[j]);
    if (row < 0)
        row += rows;  // negative indices count from the end (interp.rs:2901-2906)
    const bool inside = row >= 0 && row < rows;
    if (!inside) {
        // indices that live on the device cannot be refused before the launch:
        // the row is written as zeros and the context reports it at the next flush
        atomicExch(status, OVK_DEV_BAD_INDEX);
    }
    float v[8];
    if (inside) {
        const uint32_t q = table[row * words_per_row + word];
        const int block = (word * 8) / block_size;  // block_size is a multiple of 8 here
        const float s = SCALE_F32 ? static_cast<const float *>(scales)[row * n_blocks + block]
                                  : __half2float(static_cast<const __half *>(scales)[row * n_blocks + block]);
        const float z = zp ? float((zp[row * zp_row_bytes + (block >> 1)] >> (4 * (block & 1))) & 15u) : 8.0f;
#pragma unroll
        for (int e = 0; e < 8; e++)
            v[e] = __fmul_rn(float((q >> (4 * e)) & 15u) - z, s);
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++)
            v[e] = 0.0f;
    }
    if constexpr (OUT_F32) {
        float4 *o = reinterpret_cast<float4 *>(static_cast<float *>(out) + i * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        __half2 h[4];
#pragma unroll
        for (int e = 0; e < 4; e++)
            h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__half *>(out) + i * 8) = *reinterpret_cast<uint4 *>(h);
    }
}

// The general form (block sizes that are not a multiple of 8, odd widths): one
// thread per element, the reference's own indexing.
template <bool SCALE_F32, bool OUT_F32, bool IDX64>
__global__ void __launch_bounds__(256)
gather_block_quantized_elem_kernel(const uint8_t *__restrict__ table, const void *__restrict__ indices,
                                   const void *__restrict__ scales, const uint8_t *__restrict__ zp,
                                   void *__restrict__ out, int64_t count, int cols, int row_bytes, int64_t rows,
                                   int n_blocks, int block_size, int zp_row_bytes, int *status)
{
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count)
        return;
    const int64_t j = i / cols;
    const int c = int(i - j * cols);
    int64_t row = IDX64 ? static_cast<const int64_t *>(indices)[j] : int64_t(static_cast<const int32_t *>(indices)[j]);
    if (row < 0)
        row += rows;
    float v = 0.0f;
    if (row >= 0 && row < rows) {
        const int block = c / block_size;
        const float q = float((table[row * row_bytes + (c >> 1)] >> (4 * (c & 1))) & 15u);
        const float z = zp ? float((zp[row * zp_row_bytes + (block >> 1)] >> (4 * (block & 1))) & 15u) : 8.0f;
        const float s = SCALE_F32 ? static_cast<const float *>(scales)[row * n_blocks + block]
                                  : __half2float(static_cast<const __half *>(scales)[row * n_blocks + block]);
        v = __fmul_rn(q - z, s);
    } else {
        atomicExch(status, OVK_DEV_BAD_INDEX);
    }
    if constexpr (OUT_F32)
        static_cast<float *>(out)[i] = v;
    else
        static_cast<__half *>(out)[i] = __float2half_rn(v);
}

// ---------------------------------------------------------------- argmax
// Candidate order of the reference: larger value wins, equal values go to the
// smaller index, a value that is not greater than -FLT_MAX (so also NaN and
// -inf) is never a candidate, and a row without candidates answers 0.
struct Best {
    float v;
    uint32_t i;
};
__device__ __forceinline__ Best better(Best a, Best b)
{
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best block_best(Best mine, Best *shared /* 32 entries */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, mine.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, mine.i, o);
        mine = better(mine, other);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
        shared[warp] = mine;
    __syncthreads();
    if (warp == 0) {
        Best b = lane < int(blockDim.x >> 5) ? shared[lane] : Best{-3.4028235e38f, 0xffffffffu};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            Best other;
            other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
            other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
            b = better(b, other);
        }
        mine = b;
    }
    return mine;  // valid in warp 0
}

// grid = rows * splits.  Each CTA scans its share of one row; with more than
// one split the partial results go to `partial` and the CTA that arrives last
// at the row's counter (which it resets for the next call) picks among them.
template <bool X_F32>
__global__ void __launch_bounds__(256)
argmax_kernel(const void *__restrict__ x, int64_t *__restrict__ out, int c, int inner, int splits, Best *partial,
              unsigned int *counters)
{
    __shared__ Best shared[32];
    __shared__ bool last;
    const int r = blockIdx.x / splits, split = blockIdx.x - r * splits;
    const int j = r % inner;
    const int64_t base = int64_t(r / inner) * c * inner + j;
    const int per = (c + splits - 1) / splits;
    const int start = split * per, end = min(start + per, c);
    Best b{-3.4028235e38f, 0xffffffffu};
    if (inner == 1 && X_F32 && ((base + start) & 3) == 0) {
        // contiguous row: 128-bit loads over the aligned middle, k ascending per thread
        const float4 *v4 = reinterpret_cast<const float4 *>(static_cast<const float *>(x) + base + start);
        const int n4 = (end - start) >> 2;
        for (int k = threadIdx.x; k < n4; k += blockDim.x) {
            const float4 q = v4[k];
            const uint32_t k0 = uint32_t(start + 4 * k);
            if (q.x > b.v) b = Best{q.x, k0};
            if (q.y > b.v) b = Best{q.y, k0 + 1};
            if (q.z > b.v) b = Best{q.z, k0 + 2};
            if (q.w > b.v) b = Best{q.w, k0 + 3};
        }
        for (int k = start + 4 * n4 + threadIdx.x; k < end; k += blockDim.x) {
            const float v = static_cast<const float *>(x)[base + k];
            if (v > b.v || (v == b.v && uint32_t(k) < b.i)) b = Best{v, uint32_t(k)};
        }
    } else if (inner == 1 && !X_F32 && ((base + start) & 7) == 0) {
        const uint4 *v8 = reinterpret_cast<const uint4 *>(static_cast<const __half *>(x) + base + start);
        const int n8 = (end - start) >> 3;
        for (int k = threadIdx.x; k < n8; k += blockDim.x) {
            const uint4 q = v8[k];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            const uint32_t k0 = uint32_t(start + 8 * k);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e]));
                if (f.x > b.v) b = Best{f.x, k0 + 2 * e};
                if (f.y > b.v) b = Best{f.y, k0 + 2 * e + 1};
            }
        }
        for (int k = start + 8 * n8 + threadIdx.x; k < end; k += blockDim.x) {
            const float v = __half2float(static_cast<const __half *>(x)[base + k]);
            if (v > b.v || (v == b.v && uint32_t(k) < b.i)) b = Best{v, uint32_t(k)};
        }
    } else {
        for (int k = start + threadIdx.x; k < end; k += blockDim.x) {
            const int64_t at = base + int64_t(k) * inner;
            const float v = X_F32 ? static_cast<const float *>(x)[at] : __half2float(static_cast<const __half *>(x)[at]);
            if (v > b.v) b = Best{v, uint32_t(k)};
        }
    }
    b = block_best(b, shared);
    if (splits == 1) {
        if (threadIdx.x == 0)
            out[r] = b.i == 0xffffffffu ? 0 : int64_t(b.i);
        return;
    }
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = b;
        __threadfence();
        const unsigned int seen = atomicAdd(&counters[r], 1u);
        last = seen == unsigned(splits - 1);
        if (last)
            counters[r] = 0;  // ready for the next call on this stream
    }
    __syncthreads();
    if (!last)
        return;
    __threadfence();
    Best f{-3.4028235e38f, 0xffffffffu};
    for (int s = threadIdx.x; s < splits; s += blockDim.x)
        f = better(f, partial[r * splits + s]);
    __syncthreads();
    f = block_best(f, shared);
    if (threadIdx.x == 0)
        out[r] = f.i == 0xffffffffu ? 0 : int64_t(f.i);
}

}  // namespace

extern "C" int32_t ovk_gather_block_quantized(ovk_ctx *ctx, const void *table, const void *scales, int32_t scales_dtype,
                                              const void *zero_points, int64_t rows, int64_t cols, int64_t bits,
                                              int64_t block_size, const void *indices, int32_t indices_dtype,
                                              int32_t indices_on_host, int64_t count, void *out, int32_t out_dtype)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REFUSE(ctx, bits != 4, "GatherBlockQuantized: only 4-bit tables (got %lld)", (long long)bits);
    OVK_REFUSE(ctx, block_size <= 0 || block_size % 2 != 0, "GatherBlockQuantized: block_size %lld is not a positive even number",
               (long long)block_size);
    OVK_REQUIRE(ctx, rows >= 0 && cols > 0 && cols % block_size == 0,
                "GatherBlockQuantized: %lld columns is not a multiple of block_size %lld", (long long)cols,
                (long long)block_size);
    OVK_REQUIRE(ctx, scales_dtype == OVK_FLOAT || scales_dtype == OVK_FLOAT16, "GatherBlockQuantized: scales dtype %d", scales_dtype);
    OVK_REQUIRE(ctx, out_dtype == OVK_FLOAT || out_dtype == OVK_FLOAT16, "GatherBlockQuantized: output dtype %d", out_dtype);
    OVK_REQUIRE(ctx, indices_dtype == OVK_INT32 || indices_dtype == OVK_INT64, "GatherBlockQuantized: index dtype %d", indices_dtype);
    OVK_REQUIRE(ctx, count >= 0 && count * cols < (int64_t(1) << 40), "GatherBlockQuantized: %lld indices", (long long)count);
    if (count == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, table && scales && indices && out, "GatherBlockQuantized: null pointer");
    const bool idx64 = indices_dtype == OVK_INT64;
    const void *idx_dev = indices;
    if (indices_on_host) {
        // the reference's check (interp.rs:2908-2911), before anything is enqueued
        for (int64_t j = 0; j < count; j++) {
            int64_t g = idx64 ? static_cast<const int64_t *>(indices)[j] : int64_t(static_cast<const int32_t *>(indices)[j]);
            if (g < 0)
                g += rows;
            OVK_REQUIRE(ctx, g >= 0 && g < rows, "GatherBlockQuantized: an index falls outside the %lld-row table",
                        (long long)rows);
        }
        const size_t bytes = size_t(count) * (idx64 ? 8 : 4);
        OVK_REQUIRE(ctx, bytes <= size_t(OVK_PARAM_FLOATS) * 4, "GatherBlockQuantized: %lld host indices exceed the parameter buffer",
                    (long long)count);
        OVK_CUDA(ctx, cudaMemcpyAsync(ctx->params, indices, bytes, cudaMemcpyHostToDevice, ctx->stream));
        idx_dev = ctx->params;
    }
    const int n_blocks = int(cols / block_size);
    const int zp_row_bytes = (n_blocks + 1) / 2;
    const bool sf = scales_dtype == OVK_FLOAT, of = out_dtype == OVK_FLOAT;
    const bool words = block_size % 8 == 0 && aligned_to(table, 4) && aligned_to(out, 16);
#define OVK_GBQ(KERNEL, ...)                                                                    \
    do {                                                                                        \
        if (sf && of && idx64) KERNEL<true, true, true> __VA_ARGS__;                             \
        else if (sf && of) KERNEL<true, true, false> __VA_ARGS__;                                \
        else if (sf && idx64) KERNEL<true, false, true> __VA_ARGS__;                             \
        else if (sf) KERNEL<true, false, false> __VA_ARGS__;                                     \
        else if (of && idx64) KERNEL<false, true, true> __VA_ARGS__;                             \
        else if (of) KERNEL<false, true, false> __VA_ARGS__;                                     \
        else if (idx64) KERNEL<false, false, true> __VA_ARGS__;                                  \
        else KERNEL<false, false, false> __VA_ARGS__;                                            \
    } while (0)
    if (words) {
        const int words_per_row = int(cols / 8);
        const int64_t total = count * words_per_row;
        const unsigned grid = unsigned(ceil_div64(total, 256));
        OVK_GBQ(gather_block_quantized_kernel,
                <<<grid, 256, 0, ctx->stream>>>(static_cast<const uint32_t *>(table), idx_dev, scales,
                                                static_cast<const uint8_t *>(zero_points), out, total, words_per_row,
                                                rows, n_blocks, int(block_size), zp_row_bytes, ctx->dev_status));
        OVK_LAUNCHED(ctx, "gather_block_quantized");
    } else {
        const int64_t total = count * cols;
        const unsigned grid = unsigned(ceil_div64(total, 256));
        OVK_GBQ(gather_block_quantized_elem_kernel,
                <<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t *>(table), idx_dev, scales,
                                                static_cast<const uint8_t *>(zero_points), out, total, int(cols),
                                                int(cols / 2), rows, n_blocks, int(block_size), zp_row_bytes,
                                                ctx->dev_status));
        OVK_LAUNCHED(ctx, "gather_block_quantized_elem");
    }
#undef OVK_GBQ
    return OVK_OK;
}

extern "C" int32_t ovk_argmax(ovk_ctx *ctx, const void *x, int32_t x_dtype, int64_t outer, int64_t c, int64_t inner,
                              int64_t *out)
{
    OVK_REQUIRE(ctx, ctx, "null context");
    OVK_REQUIRE(ctx, x_dtype == OVK_FLOAT || x_dtype == OVK_FLOAT16, "ArgMax: dtype %d (f32 or f16 on the device)", x_dtype);
    OVK_REQUIRE(ctx, outer >= 0 && inner >= 1 && c >= 0 && c < (int64_t(1) << 31) && inner < (int64_t(1) << 31),
                "ArgMax: shape %lld x %lld x %lld", (long long)outer, (long long)c, (long long)inner);
    const int64_t rows = outer * inner;
    if (rows == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && out, "ArgMax: null pointer");
    OVK_REQUIRE(ctx, c > 0, "ArgMax: the reduced axis is empty");
    // interp::argmax_splits (interp.rs): aim for about one CTA per SM, at least 1024 elements per split
    int64_t splits = 1;
    if (rows < ctx->sm_count)
        splits = std::max<int64_t>(1, std::min<int64_t>(ceil_div64(ctx->sm_count, rows), c / 1024));
    OVK_REQUIRE(ctx, rows * splits < (int64_t(1) << 31), "ArgMax: %lld rows", (long long)rows);
    void *scratch = nullptr;
    unsigned int *counters = nullptr;
    if (splits > 1) {
        // counters first: they must start at zero and are left at zero by every call
        const size_t counter_bytes = (size_t(rows) * 4 + 255) & ~size_t(255);
        const bool fresh = ctx->scratch_bytes < counter_bytes + size_t(rows * splits) * sizeof(Best);
        int32_t rc = ovk_scratch(ctx, counter_bytes + size_t(rows * splits) * sizeof(Best), &scratch);
        if (rc != OVK_OK)
            return rc;
        (void)fresh;
        counters = static_cast<unsigned int *>(scratch);
        // the workspace is shared with other operators, which may have left anything there
        OVK_CUDA(ctx, cudaMemsetAsync(counters, 0, counter_bytes, ctx->stream));
        scratch = static_cast<uint8_t *>(scratch) + counter_bytes;
    }
    const unsigned grid = unsigned(rows * splits);
    if (x_dtype == OVK_FLOAT)
        argmax_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, out, int(c), int(inner), int(splits),
                                                           static_cast<Best *>(scratch), counters);
    else
        argmax_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, out, int(c), int(inner), int(splits),
                                                            static_cast<Best *>(scratch), counters);
    OVK_LAUNCHED(ctx, "argmax");
    return OVK_OK;
}
