// MatMulInteger and its fused forms: host logic, weight preparation, and the
// one-output-per-thread kernel for shapes the tensor-core tiles do not cover.
//
// Host side mirrors interp::matmul_integer (crates/onnx-vulkan-core/src/
// interp.rs:2090-2183), packed_b (:2712-2768), matmul_integer_scale_bias
// (:2405-2572) and qlinear_matmul (:4845-4875).  The small kernel has the role
// of glsl/matmul_integer_small.comp and the any-K kernel
// (src/shaders/matmul_integer.rs:52-85): any M, N, K and both operand signs.
#include "ovk_internal.h"
#include "epilogue.cuh"

bool ovk_mmi_tc_applies(const ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int64_t m);
int32_t ovk_mmi_tc_launch_group(ovk_ctx *ctx, int count, const ovk_mmi_weight *const *ws, const void *a, int32_t a_signed,
                                int64_t m, const void *a_zp, const void *b_zp, const EpiParams *epis, void *const *outs);
bool ovk_mmi_wants_large_tiles(const ovk_ctx *ctx, const ovk_mmi_weight *w, int64_t m);
int32_t ovk_mmi_tc_launch(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed,
                          int64_t m, const void *a_zp, const void *b_zp, const EpiParams &epi,
                          void *out);

namespace {

// B [K,N] -> bt [n_pad, k_pad] (K contiguous, zero padded) and colsum[n].
// One block per 32 columns; threads walk K.  Sign handling: bytes are copied
// as they are, the sum interprets them with the operand's sign.
__global__ void __launch_bounds__(256)
mmi_pack_b_kernel(const uint8_t *__restrict__ b, int K, int N, int k_pad, int b_signed,
                  uint8_t *__restrict__ bt, int32_t *__restrict__ colsum)
{
    __shared__ uint8_t tile[32][33];
    __shared__ int32_t sums[8][32];
    const int n0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    int32_t local = 0;  // thread (tx, ty) sums column n0+tx over its k rows
    for (int k0 = 0; k0 < k_pad; k0 += 32) {
        // load 32 (k) x 32 (n), coalesced along n
        for (int r = ty; r < 32; r += 8) {
            const int k = k0 + r, n = n0 + tx;
            uint8_t v = 0;
            if (k < K && n < N)
                v = b[int64_t(k) * N + n];
            tile[r][tx] = v;
            local += b_signed ? int32_t(int8_t(v)) : int32_t(v);
        }
        __syncthreads();
        // store transposed: row n, 32 consecutive k
        for (int r = ty; r < 32; r += 8) {
            const int n = n0 + r, k = k0 + tx;
            if (k < k_pad)
                bt[int64_t(n) * k_pad + k] = tile[tx][r];
        }
        __syncthreads();
    }
    sums[ty][tx] = local;
    __syncthreads();
    if (ty == 0) {
        int32_t s = 0;
        for (int i = 0; i < 8; i++)
            s += sums[i][tx];
        colsum[n0 + tx] = s;
    }
}

__device__ __forceinline__ int32_t sx(uint32_t byte, int is_signed)
{
    return is_signed ? int32_t(int8_t(byte)) : int32_t(byte);
}

// One output per thread; 16x16 threads per block.  Computes sum ab, sum a and
// applies the zero-point algebra, so it shares the epilogue with the tiled kernels.
__global__ void __launch_bounds__(256)
mmi_small_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ bt,
                 const int32_t *__restrict__ colsum, int64_t M, int K, int N, int k_pad,
                 int a_signed, int b_signed, const void *a_zp_p, const void *b_zp_p, EpiParams epi,
                 void *out, int words_ok)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    const int64_t row = int64_t(blockIdx.y) * 16 + (threadIdx.x >> 4);
    const int col = blockIdx.x * 16 + (threadIdx.x & 15);
    float run_max = 0.0f, run_neg = 0.0f;
    if (row < M && col < N) {
        const uint8_t *ar = a + row * K;
        const uint8_t *br = bt + int64_t(col) * k_pad;
        int32_t acc = 0, asum = 0;
        int k = 0;
        if (words_ok) {
            const uint32_t *aw = reinterpret_cast<const uint32_t *>(ar);
            const uint32_t *bw = reinterpret_cast<const uint32_t *>(br);
            for (; k + 4 <= K; k += 4) {
                const uint32_t x = aw[k >> 2], y = bw[k >> 2];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int32_t av = sx((x >> (8 * i)) & 0xff, a_signed);
                    acc += av * sx((y >> (8 * i)) & 0xff, b_signed);
                    asum += av;
                }
            }
        }
        for (; k < K; k++) {
            const int32_t av = sx(ar[k], a_signed);
            acc += av * sx(br[k], b_signed);
            asum += av;
        }
        const int32_t za = load_zp(a_zp_p, a_signed), zb = load_zp(b_zp_p, b_signed);
        const uint32_t corrected = uint32_t(acc) - uint32_t(za) * uint32_t(colsum[col]) -
                                   uint32_t(zb) * uint32_t(asum) + uint32_t(K) * uint32_t(za) * uint32_t(zb);
        const int32_t v = int32_t(corrected);
        const int64_t o = row * N + col;
        if (epi.mode == EPI_RAW) {
            static_cast<int32_t *>(out)[o] = v;
        } else if (epi.mode == EPI_SCALE) {
            const float f = epi_scale_value(epi, col, float(v));
            static_cast<float *>(out)[o] = f;
            run_max = fmaxf(run_max, f);
            run_neg = fmaxf(run_neg, -f);
        } else {
            static_cast<uint8_t *>(out)[o] = uint8_t(epi_requant_value(epi, col, v));
        }
    }
    if (epi.mode == EPI_SCALE)
        epi_fold_range(epi, run_max, run_neg);
}

// Cast, Mul, Add [, Relu] over an int32 matrix with operands that broadcast in any of the two
// directions: out[r][c] = fl(fl(float(acc[r][c]) * s) + bias), s = scale or fl(scale * product), each
// operand addressed by (row stride, column stride) in elements.  The nodes the reference runs when a
// scale or bias broadcasts over rows and the fused store does not apply (interp.rs:2630-2665).
__global__ void __launch_bounds__(256)
scale_bias_broadcast_kernel(const int32_t *__restrict__ acc, int64_t rows, int64_t cols, const float *__restrict__ scale,
                            int64_t srs, int64_t scs, const float *__restrict__ product, int64_t prs, int64_t pcs,
                            const float *__restrict__ bias, int64_t brs, int64_t bcs, int relu, float *__restrict__ out)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    const int64_t total = rows * cols;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t r = i / cols, c = i - r * cols;
        float s = scale[r * srs + c * scs];
        if (product)
            s = __fmul_rn(s, product[r * prs + c * pcs]);
        const float z = __fadd_rn(__fmul_rn(float(acc[i]), s), bias[r * brs + c * bcs]);
        out[i] = relu ? fmaxf(z, 0.0f) : z;
    }
}

int32_t run_mmi(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed, int64_t m,
                const void *a_zp, const void *b_zp, const EpiParams &epi, void *out,
                const char *op)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "%s: null argument", op);
    OVK_REQUIRE(ctx, m >= 0, "%s: %lld rows of A", op, (long long)m);
    if (m == 0 || w->n == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, a && out, "%s: A or the output is null", op);
    // |(a - za)(b - zb)| <= 255^2, so K terms fit i32 up to K = 33025 (interp.rs:2216-2218)
    OVK_REFUSE(ctx, w->k > 33025, "%s: K=%lld could overflow the int32 accumulator", op, (long long)w->k);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (ovk_mmi_tc_applies(ctx, w, a, m))
        return ovk_mmi_tc_launch(ctx, w, a, a_signed, m, a_zp, b_zp, epi, out);
    OVK_REQUIRE(ctx, ceil_div64(m, 16) <= 65535, "%s: %lld rows exceed the small-shape grid", op, (long long)m);
    dim3 grid(unsigned(ceil_div64(w->n, 16)), unsigned(ceil_div64(m, 16)));
    const int words_ok = aligned_to(a, 4) && (w->k % 4 == 0);
    OVK_CUDA(ctx, ovk_launch_pdl(mmi_small_kernel, grid, dim3(256), 0, ctx->stream, static_cast<const uint8_t *>(a),
                                 static_cast<const uint8_t *>(w->bt), static_cast<const int32_t *>(w->colsum), m, int(w->k),
                                 int(w->n), int(w->k_pad), int(a_signed), int(w->b_signed), a_zp, b_zp, epi, out, words_ok));
    OVK_LAUNCHED(ctx, "mmi_small");
    return OVK_OK;
}

}  // namespace

extern "C" {

int32_t ovk_mmi_prepack(ovk_ctx *ctx, const void *b, int32_t b_signed, int64_t k, int64_t n,
                        ovk_mmi_weight **out)
{
    if (!ctx || !out)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_mmi_prepack: null argument");
    *out = nullptr;
    OVK_REQUIRE(ctx, k >= 0 && n >= 0, "MatMulInteger: B is [%lld, %lld]", (long long)k, (long long)n);
    OVK_REQUIRE(ctx, b || k * n == 0, "MatMulInteger: B is null");
    OVK_REQUIRE(ctx, k < (1 << 30) && n < (1 << 30), "MatMulInteger: B is too large");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    ovk_mmi_weight *w = new ovk_mmi_weight();
    w->k = k;
    w->n = n;
    w->b_signed = b_signed ? 1 : 0;
    w->k_pad = std::max<int64_t>(128, ceil_div64(k, 128) * 128);  // whole 128-byte K slabs for the tensor path
    w->n_pad = std::max<int64_t>(32, ceil_div64(n, 32) * 32);
    cudaError_t e = cudaMalloc(&w->bt, size_t(w->n_pad) * size_t(w->k_pad));
    if (e == cudaSuccess)
        e = cudaMalloc(&w->colsum, size_t(w->n_pad) * sizeof(int32_t));
    if (e != cudaSuccess) {
        cudaFree(w->bt);
        delete w;
        return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger: packed weight allocation: %s", cudaGetErrorString(e));
    }
    mmi_pack_b_kernel<<<unsigned(w->n_pad / 32), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t *>(b), int(k), int(n), int(w->k_pad), w->b_signed, w->bt, w->colsum);
    ctx->last_kernel = "mmi_pack_b";
    ctx->launches++;
    e = cudaGetLastError();
    int32_t rc = OVK_OK;
    if (e != cudaSuccess)
        rc = ovk_fail(ctx, OVK_BACKEND, "mmi_pack_b: %s", cudaGetErrorString(e));
    if (rc != OVK_OK) {
        cudaFree(w->bt);
        cudaFree(w->colsum);
        delete w;
        return rc;
    }
    *out = w;
    return OVK_OK;
}

void ovk_mmi_weight_destroy(ovk_ctx *ctx, ovk_mmi_weight *w)
{
    if (!w)
        return;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    cudaFree(w->bt);
    cudaFree(w->colsum);
    free(w->tmap_b);
    delete w;
}

int32_t ovk_matmul_integer(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed,
                           int64_t m, const void *a_zp, const void *b_zp, int32_t *out)
{
    EpiParams epi = {};
    epi.mode = EPI_RAW;
    return run_mmi(ctx, w, a, a_signed, m, a_zp, b_zp, epi, out, "MatMulInteger");
}

int32_t ovk_matmul_integer_scale_bias(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a,
                                      int32_t a_signed, int64_t m, const void *a_zp,
                                      const void *b_zp, const float *scale, int32_t scale_step,
                                      const float *product, int32_t product_step,
                                      const float *bias, int32_t bias_step, uint32_t flags,
                                      uint32_t *range, float *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "MatMulIntegerScaleBias: null context");
    OVK_REQUIRE(ctx, scale && bias, "MatMulIntegerScaleBias: scale or bias is null");
    // interp::column_step (interp.rs:2600-2610): one value or one per column;
    // anything else is not fused by the reference either
    OVK_REFUSE(ctx, (scale_step | bias_step | product_step) & ~1,
               "MatMulIntegerScaleBias: a scale, product or bias that broadcasts over rows is not fused");
    OVK_REQUIRE(ctx, !(flags & OVK_EPILOGUE_RANGE) || range,
                "MatMulIntegerScaleBias: range folding requested without a range slot");
    EpiParams epi = {};
    epi.mode = EPI_SCALE;
    epi.scale = scale;
    epi.scale_step = scale_step;
    epi.product = product;
    epi.product_step = product ? product_step : 0;
    epi.fbias = bias;
    epi.bias_step = bias_step;
    epi.flags = flags;
    epi.range = range;
    return run_mmi(ctx, w, a, a_signed, m, a_zp, b_zp, epi, out, "MatMulIntegerScaleBias");
}

// Several weights over the same A (the q, k and v projections of an attention block).  One launch
// when every member takes the 128-row tensor-core tiles and the members agree on K and on the
// signedness of B; one call per member otherwise.  Results are those of separate calls.
static int32_t run_mmi_group(ovk_ctx *ctx, int32_t count, const ovk_mmi_weight *const *ws, const void *a, int32_t a_signed,
                             int64_t m, const void *a_zp, const void *b_zp, const EpiParams *epis, void *const *outs,
                             const char *op)
{
    if (!ctx || !ws || !outs)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "%s: null argument", op);
    OVK_REQUIRE(ctx, count >= 1 && count <= 4, "%s: a group of %d weights (1 to 4)", op, count);
    for (int j = 0; j < count; j++)
        OVK_REQUIRE(ctx, ws[j] && (outs[j] || m == 0), "%s: member %d of the group is null", op, j);
    for (int j = 1; j < count; j++)
        OVK_REQUIRE(ctx, ws[j]->k == ws[0]->k, "%s: member %d of the group has K=%lld, member 0 K=%lld", op, j,
                    (long long)ws[j]->k, (long long)ws[0]->k);
    bool together = count > 1 && m > 0 && a && ws[0]->k <= 33025 && !(epis[0].flags & OVK_EPILOGUE_RANGE);
    for (int j = 0; together && j < count; j++)
        together = ws[j]->n > 0 && ws[j]->b_signed == ws[0]->b_signed && ovk_mmi_tc_applies(ctx, ws[j], a, m) &&
                   !ovk_mmi_wants_large_tiles(ctx, ws[j], m);
    if (together) {
        OVK_CUDA(ctx, cudaSetDevice(ctx->device));
        return ovk_mmi_tc_launch_group(ctx, count, ws, a, a_signed, m, a_zp, b_zp, epis, outs);
    }
    for (int j = 0; j < count; j++) {
        const int32_t rc = run_mmi(ctx, ws[j], a, a_signed, m, a_zp, b_zp, epis[j], outs[j], op);
        if (rc != OVK_OK)
            return rc;
    }
    return OVK_OK;
}

int32_t ovk_matmul_integer_group(ovk_ctx *ctx, int32_t count, const ovk_mmi_weight *const *weights, const void *a,
                                 int32_t a_signed, int64_t m, const void *a_zp, const void *b_zp, int32_t *const *outs)
{
    EpiParams epis[4] = {};
    for (int j = 0; j < 4; j++)
        epis[j].mode = EPI_RAW;
    return run_mmi_group(ctx, count, weights, a, a_signed, m, a_zp, b_zp, epis, reinterpret_cast<void *const *>(outs),
                         "MatMulInteger");
}

int32_t ovk_matmul_integer_scale_bias_group(ovk_ctx *ctx, int32_t count, const ovk_mmi_weight *const *weights,
                                            const void *a, int32_t a_signed, int64_t m, const void *a_zp, const void *b_zp,
                                            const float *const *scales, int32_t scale_step, const float *product,
                                            int32_t product_step, const float *const *biases, int32_t bias_step,
                                            uint32_t flags, float *const *outs)
{
    if (!ctx || !scales || !biases)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "MatMulIntegerScaleBias: null argument");
    OVK_REQUIRE(ctx, count >= 1 && count <= 4, "MatMulIntegerScaleBias: a group of %d weights (1 to 4)", count);
    OVK_REFUSE(ctx, (scale_step | bias_step | product_step) & ~1,
               "MatMulIntegerScaleBias: a scale, product or bias that broadcasts over rows is not fused");
    OVK_REFUSE(ctx, flags & OVK_EPILOGUE_RANGE, "MatMulIntegerScaleBias: a group folds no range (its members are different tensors)");
    OVK_REFUSE(ctx, product && product_step != 0, "MatMulIntegerScaleBias: the second scale factor of a group is one value");
    EpiParams epis[4] = {};
    for (int j = 0; j < count; j++) {
        OVK_REQUIRE(ctx, scales[j] && biases[j], "MatMulIntegerScaleBias: scale or bias of member %d is null", j);
        epis[j].mode = EPI_SCALE;
        epis[j].scale = scales[j];
        epis[j].scale_step = scale_step;
        epis[j].product = product;
        epis[j].product_step = 0;
        epis[j].fbias = biases[j];
        epis[j].bias_step = bias_step;
        epis[j].flags = flags;
    }
    return run_mmi_group(ctx, count, weights, a, a_signed, m, a_zp, b_zp, epis, reinterpret_cast<void *const *>(outs),
                         "MatMulIntegerScaleBias");
}

int32_t ovk_integer_scale_bias_unfused(ovk_ctx *ctx, const int32_t *acc, int64_t rows, int64_t cols, const float *scale,
                                       int64_t scale_row_stride, int64_t scale_col_stride, const float *product,
                                       int64_t product_row_stride, int64_t product_col_stride, const float *bias,
                                       int64_t bias_row_stride, int64_t bias_col_stride, uint32_t flags, float *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_integer_scale_bias_unfused: null context");
    OVK_REQUIRE(ctx, rows >= 0 && cols >= 0, "Cast/Mul/Add: a negative shape");
    OVK_REFUSE(ctx, flags & OVK_EPILOGUE_RANGE, "Cast/Mul/Add: the unfused nodes fold no range (the quantization that follows makes its own pass)");
    if (rows == 0 || cols == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, acc && scale && bias && out, "Cast/Mul/Add: a tensor is null");
    OVK_REQUIRE(ctx, scale_row_stride >= 0 && scale_col_stride >= 0 && bias_row_stride >= 0 && bias_col_stride >= 0 &&
                         product_row_stride >= 0 && product_col_stride >= 0,
                "Cast/Mul/Add: a negative stride");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(rows * cols, 256), int64_t(ctx->sm_count) * 8));
    OVK_CUDA(ctx, ovk_launch_pdl(scale_bias_broadcast_kernel, dim3(blocks), dim3(256), 0, ctx->stream, acc, rows, cols, scale,
                                 scale_row_stride, scale_col_stride, product, product_row_stride, product_col_stride, bias,
                                 bias_row_stride, bias_col_stride, int(flags & OVK_EPILOGUE_RELU), out));
    OVK_LAUNCHED(ctx, "scale_bias_broadcast");
    return OVK_OK;
}

int32_t ovk_qlinear_matmul(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed,
                           int64_t m, const void *a_zp, const void *b_zp, const float *ratio,
                           int64_t ratio_len, int32_t y_zp, int32_t y_signed, void *out)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "QLinearMatMul: null argument");
    OVK_REQUIRE(ctx, ratio, "QLinearMatMul: ratio is null");
    OVK_REQUIRE(ctx, ratio_len == 1 || ratio_len == w->n, "QLinearMatMul: %lld scales for %lld columns",
                (long long)ratio_len, (long long)w->n);
    EpiParams epi = {};
    epi.mode = EPI_REQUANT;
    epi.ratio = ratio;
    epi.ratio_step = ratio_len == 1 ? 0 : 1;
    epi.y_zp = y_zp;
    epi.y_signed = y_signed;
    return run_mmi(ctx, w, a, a_signed, m, a_zp, b_zp, epi, out, "QLinearMatMul");
}

}  // extern "C"
