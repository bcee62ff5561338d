// MatMulNBits prefill (M > 8) with f32 activations.
//
// The tensor-core kernels multiply fp16 activations; the reference computes in f32 throughout
// (crates/onnx-vulkan-core/src/shaders/matmul_nbits.rs:340-372), and its models feed f32.  Rounding the
// activations to fp16 would cost 2^-11 per element and fail the f32 tolerance, so every row is split the
// way the decode kernel splits it: after an exact power-of-two normalisation of the row,
// x = hi + lo with hi = fl16(x) and lo = fl16(x - hi), about 22 bits of the activation.  The two parts go
// through the prefill kernel as two rows (the product is linear in the activations, every block's
// partial sum is still exact, accumulation is f32), and a last pass adds the two result rows and undoes
// the normalisation: y = (y_hi + y_lo) * 2^e.  Twice the tensor time of an fp16 call - and two orders of
// magnitude faster than the one-row-at-a-time kernel these calls took before (36 ms for 512 x 3584 x 18944).
#include "ovk_internal.h"

bool ovk_nbits_gemm_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, int32_t a_dtype,
                            int32_t y_dtype, const void *a, const void *y);
int32_t ovk_nbits_gemm(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype,
                       int64_t m, void *y, int32_t y_dtype);

namespace {

// The prefill kernel asks for the context's workspace itself (partial sums of K ranges shared between
// CTAs, below 30 MB on 148 SMs) and gets the START of the block: the buffers of this file lie behind that.
constexpr size_t INNER_WORKSPACE = size_t(32) << 20;
constexpr size_t CHUNK_BYTES = size_t(384) << 20;  // most workspace one chunk of rows may take

// One block per row: hi and lo parts of the normalised row as fp16 rows r and rows + r, 2^e to pow2[r].
__global__ void __launch_bounds__(256)
split_rows_kernel(const float *__restrict__ a, int rows, int K, __half *__restrict__ parts, float *__restrict__ pow2)
{
    const int r = blockIdx.x;
    const float *x = a + size_t(r) * K;
    float mx = 0.0f;
    for (int k = threadIdx.x; k < K; k += 256)
        mx = fmaxf(mx, fabsf(x[k]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __shared__ float wmax[8];
    __shared__ float s_scale;
    if ((threadIdx.x & 31) == 0)
        wmax[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            mx = fmaxf(mx, wmax[w]);
        int e = 0;
        if (mx > 0.0f && mx < 3.0e38f)
            frexpf(mx, &e);
        e = max(-100, min(100, e));
        s_scale = ldexpf(1.0f, e);
        pow2[r] = s_scale;
    }
    __syncthreads();
    const float inv = 1.0f / s_scale;  // an exact power of two
    __half *hi = parts + size_t(r) * K, *lo = parts + size_t(rows + r) * K;
    for (int k = threadIdx.x; k < K; k += 256) {
        const float v = x[k] * inv;
        const __half h = __float2half_rn(v);
        hi[k] = h;
        lo[k] = __float2half_rn(v - __half2float(h));
    }
}

template <typename T>
__device__ __forceinline__ T to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }

// y[r][n] = (y2[r][n] + y2[rows + r][n]) * pow2[r]
template <typename T>
__global__ void __launch_bounds__(256)
join_rows_kernel(const float *__restrict__ y2, const float *__restrict__ pow2, int rows, int64_t N, T *__restrict__ y)
{
    const int64_t total = int64_t(rows) * N;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int64_t r = i / N;
        y[i] = to_out<T>(__fmul_rn(__fadd_rn(y2[i], y2[total + i]), pow2[r]));
    }
}

}  // namespace

bool ovk_nbits_gemm_f32_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, const void *a, const void *y)
{
    // what the fp16 kernels need of the weight and of K, asked with stand-in pointers of the alignment the
    // workspace has
    alignas(16) static const char stand_in[16] = {};
    return m > 8 && aligned_to(a, 4) && aligned_to(y, 2) &&
           ovk_nbits_gemm_applies(ctx, w, 2 * m, OVK_FLOAT16, OVK_FLOAT, stand_in, stand_in);
}

int32_t ovk_nbits_gemm_f32(ovk_ctx *ctx, const ovk_nbits_weight *w, const float *a, int64_t m, void *y, int32_t y_dtype)
{
    const int64_t K = w->k, N = w->n;
    const size_t per_row = size_t(K) * 2 * 2 + size_t(N) * 4 * 2 + 4;
    const int64_t chunk = std::max<int64_t>(16, std::min<int64_t>(m, int64_t(CHUNK_BYTES / per_row)));
    const size_t parts_bytes = (size_t(2 * chunk) * K * 2 + 255) & ~size_t(255);
    const size_t y2_bytes = (size_t(2 * chunk) * N * 4 + 255) & ~size_t(255);
    void *ws = nullptr;
    int32_t rc = ovk_scratch(ctx, INNER_WORKSPACE + parts_bytes + y2_bytes + size_t(chunk) * 4 + 256, &ws);
    if (rc != OVK_OK)
        return rc;
    uint8_t *base = static_cast<uint8_t *>(ws) + INNER_WORKSPACE;
    __half *parts = reinterpret_cast<__half *>(base);
    float *y2 = reinterpret_cast<float *>(base + parts_bytes);
    float *pow2 = reinterpret_cast<float *>(base + parts_bytes + y2_bytes);
    for (int64_t r0 = 0; r0 < m; r0 += chunk) {
        const int rows = int(std::min<int64_t>(chunk, m - r0));
        split_rows_kernel<<<unsigned(rows), 256, 0, ctx->stream>>>(a + size_t(r0) * K, rows, int(K), parts, pow2);
        OVK_LAUNCHED(ctx, "nbits_split_rows");
        rc = ovk_nbits_gemm(ctx, w, parts, OVK_FLOAT16, 2 * int64_t(rows), y2, OVK_FLOAT);
        if (rc != OVK_OK)
            return rc;
        const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(int64_t(rows) * N, 256), int64_t(ctx->sm_count) * 16));
        if (y_dtype == OVK_FLOAT)
            join_rows_kernel<float><<<blocks, 256, 0, ctx->stream>>>(y2, pow2, rows, N, static_cast<float *>(y) + size_t(r0) * N);
        else
            join_rows_kernel<__half><<<blocks, 256, 0, ctx->stream>>>(y2, pow2, rows, N, static_cast<__half *>(y) + size_t(r0) * N);
        OVK_LAUNCHED(ctx, "nbits_join_rows");
    }
    return OVK_OK;
}
