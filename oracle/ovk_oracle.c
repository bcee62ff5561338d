/*
 * CPU oracle for the quantized matrix-product path.  TEST INFRASTRUCTURE ONLY:
 * it is the checker for the CUDA kernels and the timed CPU baseline of the
 * benchmark; the shipped library never links, loads or calls it.
 *
 * Every function restates, on the host, the arithmetic of one step of the
 * reference (automataIA/onnx-vulkan-rs); the file:line each one follows is
 * given above it (paths inside crates/onnx-vulkan-core/ unless stated).
 *
 * Parity status: pinned against the reference's own known-answer tests (the
 * literal vectors of tests/qlinear.rs and the closed-form generators of
 * tests/matmul_nbits.rs, tests/dynamic_quantize.rs,
 * tests/matmul_integer_variants.rs, tests/conv_integer_im2col.rs), restated in
 * tests/test_oracle_golden.py.  The reference cannot be compiled here (Rust,
 * Vulkan), so no output of the reference itself backs these functions.
 *
 * Build: see oracle/Makefile (-O3 -march=x86-64-v3 -fopenmp -ffp-contract=off).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

/* dtype codes: ElementType of src/graph.rs:13-41 */
enum { ORC_FLOAT = 1, ORC_UINT8 = 2, ORC_INT8 = 3, ORC_INT32 = 6, ORC_FLOAT16 = 10 };

/* ------------------------------------------------------------------ fp16 */

static inline float f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* double -> binary16 with a single round-to-nearest-even */
static inline uint16_t f64_to_f16(double d)
{
    uint64_t b;
    memcpy(&b, &d, 8);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    int64_t exp = (int64_t)((b >> 52) & 0x7ff);
    uint64_t man = b & 0xfffffffffffffull;
    if (exp == 0x7ff)
        return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp == 0 && man == 0)
        return sign;
    int64_t e = exp - 1023; /* unbiased */
    uint64_t sig = man | (1ull << 52); /* 53-bit significand, value = sig * 2^(e-52) */
    if (exp == 0) {
        return sign; /* double subnormals are far below half's range */
    }
    if (e > 15)
        return (uint16_t)(sign | 0x7c00u);
    int shift; /* bits to drop from sig so that the result is in units of the target ulp */
    int64_t he;
    if (e >= -14) { /* normal half: keep 11 bits */
        shift = 42;
        he = e + 15;
    } else { /* subnormal half: ulp is 2^-24 */
        shift = (int)(42 + (-14 - e));
        he = 0;
        if (shift > 63)
            return sign;
    }
    uint64_t kept = sig >> shift;
    uint64_t rem = sig & ((1ull << shift) - 1);
    uint64_t half = 1ull << (shift - 1);
    if (rem > half || (rem == half && (kept & 1)))
        kept++;
    uint32_t out;
    if (he == 0) {
        out = (uint32_t)kept; /* may carry into the exponent field: correct */
    } else {
        out = (uint32_t)(((uint64_t)he << 10) + (kept - 0x400u)); /* carry propagates */
    }
    if (out >= 0x7c00u)
        out = 0x7c00u;
    return (uint16_t)(sign | out);
}

ORC_EXPORT void orc_f16_to_f32(const uint16_t *src, float *dst, size_t n)
{
    for (size_t i = 0; i < n; i++)
        dst[i] = f16_to_f32(src[i]);
}

ORC_EXPORT void orc_f64_to_f16(const double *src, uint16_t *dst, size_t n)
{
    for (size_t i = 0; i < n; i++)
        dst[i] = f64_to_f16(src[i]);
}

static inline double load_real(const void *p, int dtype, size_t i)
{
    if (dtype == ORC_FLOAT16)
        return (double)f16_to_f32(((const uint16_t *)p)[i]);
    return (double)((const float *)p)[i];
}

ORC_EXPORT int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_EXPORT void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : 1);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------ MatMulNBits */

/* nibble k of column n: element 2i sits in the LOW nibble of byte i
 * (src/shaders/matmul_nbits.rs:15-19, tests/matmul_nbits.rs:19-34). */
static inline int nib_at(const uint8_t *b, size_t row_bytes, size_t n, size_t k)
{
    uint8_t byte = b[n * row_bytes + k / 2];
    return (byte >> (4 * (k & 1))) & 15;
}

/* zero point of (column n, block blk): row stride ceil(n_blocks/2) bytes, low
 * nibble first (tests/matmul_nbits.rs:36-46); absent => 8 (operator spec). */
static inline int zp_at(const uint8_t *zp, size_t zp_row, size_t n, size_t blk)
{
    if (!zp)
        return 8;
    return (zp[n * zp_row + blk / 2] >> (4 * (blk & 1))) & 15;
}

/*
 * The operator's definition, y[m][n] = sum_k a[m][k] * (nib - zp) * scale, with
 * every product and the sum in f64 and ONE rounding to the output dtype
 * (scalar reference of tests/matmul_nbits.rs:79-91; layout
 * src/shaders/matmul_nbits.rs:1-25).  a/scales/y may be f32 or f16.
 */
ORC_EXPORT int orc_matmul_nbits(const void *a, int a_dtype, int64_t M, int64_t K, int64_t N,
                                int64_t block_size, const uint8_t *b, const void *scales,
                                int scales_dtype, const uint8_t *zp, void *y, int y_dtype)
{
    if (block_size <= 0 || (block_size % 8) != 0 || K <= 0 || N <= 0 || M < 0)
        return 1;
    size_t n_blocks = (size_t)((K + block_size - 1) / block_size);
    size_t row_bytes = n_blocks * (size_t)block_size / 2;
    size_t zp_row = (n_blocks + 1) / 2;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        for (int64_t m = 0; m < M; m++) {
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++) {
                size_t blk = (size_t)(k / block_size);
                double w = (double)(nib_at(b, row_bytes, (size_t)n, (size_t)k) -
                                    zp_at(zp, zp_row, (size_t)n, blk)) *
                           load_real(scales, scales_dtype, (size_t)n * n_blocks + blk);
                acc += load_real(a, a_dtype, (size_t)(m * K + k)) * w;
            }
            size_t o = (size_t)(m * N + n);
            if (y_dtype == ORC_FLOAT16)
                ((uint16_t *)y)[o] = f64_to_f16(acc);
            else
                ((float *)y)[o] = (float)acc;
        }
    }
    return 0;
}

/*
 * The same product in the reference shader's own f32 order
 * (src/shaders/matmul_nbits.rs:316-374): per 32-bit word `part = fma(nib - z,
 * a, part)` over its eight weights, then `acc = fma(part, scale, acc)`; 64
 * strided partial sums combined by a 6-level tree.  f32 in, f32 out (the only
 * form the reference runs, src/interp.rs:6460-6466); this is also the timed
 * CPU baseline of the decode path.
 */
ORC_EXPORT int orc_matmul_nbits_f32_shader_order(const float *a, int64_t M, int64_t K, int64_t N,
                                                 int64_t block_size, const uint8_t *b,
                                                 const float *scales, const uint8_t *zp, float *y)
{
    if (block_size <= 0 || (block_size % 8) != 0 || K <= 0 || N <= 0 || M < 0)
        return 1;
    size_t n_blocks = (size_t)((K + block_size - 1) / block_size);
    size_t blob_words = (size_t)block_size / 8;
    size_t words = n_blocks * blob_words;
    size_t zp_row = (n_blocks + 1) / 2;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        const uint8_t *col = b + (size_t)n * words * 4;
        for (int64_t m = 0; m < M; m++) {
            float red[64];
            for (int t = 0; t < 64; t++) {
                float acc = 0.0f;
                for (size_t w = (size_t)t; w < words; w += 64) {
                    size_t blk = w / blob_words;
                    size_t k0 = blk * (size_t)block_size + (w % blob_words) * 8;
                    uint32_t word;
                    memcpy(&word, col + 4 * w, 4);
                    float z = (float)zp_at(zp, zp_row, (size_t)n, blk);
                    float part = 0.0f;
                    for (int i = 0; i < 8; i++) {
                        size_t k = k0 + (size_t)i;
                        if ((int64_t)k >= K)
                            break;
                        part = fmaf((float)((word >> (4 * i)) & 15u) - z, a[m * K + (int64_t)k],
                                    part);
                    }
                    acc = fmaf(part, scales[(size_t)n * n_blocks + blk], acc);
                }
                red[t] = acc;
            }
            for (int s = 32; s > 0; s /= 2)
                for (int t = 0; t < s; t++)
                    red[t] = red[t] + red[t + s];
            y[m * N + n] = red[0];
        }
    }
    return 0;
}

/* ------------------------------------------------ DynamicQuantizeLinear */

/*
 * The ONNX definition with IEEE division and ties-to-even, the reference's
 * target (tests/dynamic_quantize.rs:16-26; shader
 * src/shaders/dynamic_quantize.rs:160-216): the range always includes 0, a
 * -0.0 counts as 0 (:143-145), scale 1 when the range is empty, empty input
 * gives scale 1 and zero point 0 (src/interp.rs:1949-1966).
 */
ORC_EXPORT void orc_dynamic_quantize(const float *x, size_t n, uint8_t *y, float *y_scale,
                                     uint8_t *y_zp)
{
    float mn = 0.0f, mx = 0.0f;
    for (size_t i = 0; i < n; i++) {
        float v = x[i];
        if (v < mn)
            mn = v;
        if (v > mx)
            mx = v;
    }
    float scale = (mx == mn) ? 1.0f : (mx - mn) / 255.0f;
    float q = -mn / scale;
    if (q < 0.0f)
        q = 0.0f;
    if (q > 255.0f)
        q = 255.0f;
    float zp = nearbyintf(q); /* default rounding mode: ties to even */
    *y_scale = scale;
    *y_zp = (uint8_t)zp;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        float v = nearbyintf(x[i] / scale) + zp;
        if (v < 0.0f)
            v = 0.0f;
        if (v > 255.0f)
            v = 255.0f;
        y[i] = (uint8_t)v;
    }
}

/* -------------------------------------------------------- DecomposedGelu */

/*
 * exp for the erf approximation below.  The reference's shader calls the
 * device's exp(), which no two devices round alike; this restatement and the
 * CUDA kernels spell it in IEEE operations only - reduction by ln 2 in two
 * parts, a degree-7 polynomial in fused multiply-adds, scaling by exponent
 * bits in two exact steps - so that both give the same bits.
 */
static inline float exp_ieee(float x)
{
    if (!(x > -104.0f))
        return x != x ? x : 0.0f;
    const float n = nearbyintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    const int e = (int)n;
    const int e1 = e / 2, e2 = e - e1;
    union { uint32_t u; float f; } s1, s2;
    s1.u = (uint32_t)(e1 + 127) << 23;
    s2.u = (uint32_t)(e2 + 127) << 23;
    return (p * s1.f) * s2.f;
}

/* erf_approx of src/shaders/elementwise.rs:71-80 (Abramowitz & Stegun 7.1.26), each operation rounded. */
static inline float erf_approx(float x)
{
    const float s = x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);
    const float a = fabsf(x);
    const float t = 1.0f / (1.0f + 0.3275911f * a);
    float poly = t * 1.061405429f;
    poly = t * (-1.453152027f + poly);
    poly = t * (1.421413741f + poly);
    poly = t * (-0.284496736f + poly);
    poly = t * (0.254829592f + poly);
    return s * (1.0f - poly * exp_ieee(-a * a));
}

/*
 * decomposed_gelu of src/shaders/elementwise.rs:110-118 (host side
 * src/interp.rs:9034-9084): e = erf(v / divisor) + offset, then the graph's
 * order of the two products.
 */
ORC_EXPORT void orc_decomposed_gelu(const float *x, size_t n, float divisor, float offset, float factor,
                                    int factor_first, float *out)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        const float v = x[i];
        const float e = erf_approx(v / divisor) + offset;
        out[i] = factor_first ? v * (e * factor) : (v * e) * factor;
    }
}

ORC_EXPORT float orc_erf_approx(float x) { return erf_approx(x); }
ORC_EXPORT float orc_exp_ieee(float x) { return exp_ieee(x); }

/* -------------------------------------------------------- MatMulInteger */

static inline int64_t byte_val(const uint8_t *p, size_t i, int is_signed)
{
    return is_signed ? (int64_t)(int8_t)p[i] : (int64_t)p[i];
}

/*
 * A [M,K] x B [K,N] -> i32 with per-tensor zero points, i64 accumulation and
 * an error on i32 overflow (src/host_ops.rs:1157-1199; sign handling
 * src/shaders/matmul_integer.rs:52-85).  Returns 2 on overflow.
 */
ORC_EXPORT int orc_matmul_integer(const uint8_t *a, int a_signed, const uint8_t *b, int b_signed,
                                  int64_t M, int64_t K, int64_t N, int32_t a_zp, int32_t b_zp,
                                  int32_t *out)
{
    int overflow = 0;
    /* transpose B once so the inner loop is contiguous */
    int16_t *bt = (int16_t *)__builtin_malloc((size_t)(N * K + 1) * sizeof(int16_t));
    if (!bt)
        return 3;
    for (int64_t k = 0; k < K; k++)
        for (int64_t n = 0; n < N; n++)
            bt[n * K + k] = (int16_t)(byte_val(b, (size_t)(k * N + n), b_signed) - b_zp);
#pragma omp parallel for schedule(static) reduction(| : overflow)
    for (int64_t m = 0; m < M; m++) {
        int16_t *ar = (int16_t *)__builtin_malloc((size_t)(K + 1) * sizeof(int16_t));
        for (int64_t k = 0; k < K; k++)
            ar[k] = (int16_t)(byte_val(a, (size_t)(m * K + k), a_signed) - a_zp);
        for (int64_t n = 0; n < N; n++) {
            const int16_t *bc = bt + n * K;
            int64_t sum = 0;
            for (int64_t k = 0; k < K; k++)
                sum += (int64_t)ar[k] * (int64_t)bc[k];
            if (sum > INT32_MAX || sum < INT32_MIN)
                overflow |= 1;
            out[m * N + n] = (int32_t)sum;
        }
        __builtin_free(ar);
    }
    __builtin_free(bt);
    return overflow ? 2 : 0;
}

/*
 * The fused MatMulInteger -> Cast -> Mul -> Add [-> Relu] epilogue, rounded as
 * the three separate kernels round (src/shaders/glsl/matmul_integer_coop.comp:
 * 156-196): x = float(acc); s = scale (* product: one rounding); y = fl(x*s);
 * z = fl(y + bias); relu = max(z, 0).  A step is 0 (one value), 1 (one per
 * column) or 2 (one per row), index = col*(step&1) + row*(step>>1)
 * (src/interp.rs:2600-2610).  `range` (may be NULL) receives {-min, max} of
 * the stored values, both starting from 0 (:178-196).
 */
ORC_EXPORT void orc_scale_bias_epilogue(const int32_t *acc, int64_t M, int64_t N,
                                        const float *scale, int scale_step, const float *product,
                                        int product_step, const float *bias, int bias_step,
                                        int relu, float *out, float *range)
{
    float run_max = 0.0f, run_neg = 0.0f;
    for (int64_t r = 0; r < M; r++) {
        for (int64_t c = 0; c < N; c++) {
            volatile float x = (float)acc[r * N + c];
            volatile float s = scale[c * (scale_step & 1) + r * (scale_step >> 1)];
            if (product) {
                volatile float p = product[c * (product_step & 1) + r * (product_step >> 1)];
                s = s * p;
            }
            volatile float yv = x * s;
            volatile float z = yv + bias[c * (bias_step & 1) + r * (bias_step >> 1)];
            float v = z;
            if (relu)
                v = (z > 0.0f) ? z : 0.0f; /* max(z, 0.0) */
            out[r * N + c] = v;
            if (v > run_max)
                run_max = v;
            if (-v > run_neg)
                run_neg = -v;
        }
    }
    if (range) {
        range[0] = run_neg;
        range[1] = run_max;
    }
}

/* ------------------------------------------- ConvInteger / QLinearConv */

typedef struct {
    int64_t n, c_in, c_out, group, gsi;
    int64_t h_in, w_in, h_out, w_out;
    int64_t kh, kw, sh, sw, dh, dw;
    int64_t phb, phe, pwb, pwe;
} orc_conv_geom;

/* SAME_UPPER / SAME_LOWER padding of one dimension (src/interp.rs:3425-3437) */
static void same_pads(int upper, int64_t in_dim, int64_t k, int64_t stride, int64_t dil,
                      int64_t *begin, int64_t *end)
{
    int64_t out = (in_dim + stride - 1) / stride;
    int64_t needed = (out - 1) * stride + (k - 1) * dil + 1 - in_dim;
    if (needed < 0)
        needed = 0;
    int64_t half = needed / 2;
    if (upper) {
        *begin = half;
        *end = needed - half;
    } else {
        *begin = needed - half;
        *end = half;
    }
}

/*
 * Output geometry of Conv/ConvInteger (src/interp.rs:3439-3536).  x_shape is
 * [N,C,H,W] (a 1-D conv is passed with W = 1, kw = 1).  auto_pad: 0 NOTSET,
 * 1 VALID, 2 SAME_UPPER, 3 SAME_LOWER.  pads = {h_begin, w_begin, h_end, w_end}.
 * Returns 1 for a degenerate output.
 */
ORC_EXPORT int orc_conv_geometry(const int64_t x_shape[4], const int64_t w_shape[4],
                                 const int64_t strides[2], const int64_t dilations[2],
                                 const int64_t pads[4], int auto_pad, int64_t group,
                                 orc_conv_geom *g)
{
    g->n = x_shape[0];
    g->c_in = x_shape[1];
    g->h_in = x_shape[2];
    g->w_in = x_shape[3];
    g->c_out = w_shape[0];
    g->gsi = w_shape[1];
    g->kh = w_shape[2];
    g->kw = w_shape[3];
    g->group = group;
    g->sh = strides[0];
    g->sw = strides[1];
    g->dh = dilations[0];
    g->dw = dilations[1];
    g->phb = pads[0];
    g->pwb = pads[1];
    g->phe = pads[2];
    g->pwe = pads[3];
    if (auto_pad == 1) {
        g->phb = g->pwb = g->phe = g->pwe = 0;
    } else if (auto_pad == 2 || auto_pad == 3) {
        same_pads(auto_pad == 2, g->h_in, g->kh, g->sh, g->dh, &g->phb, &g->phe);
        same_pads(auto_pad == 2, g->w_in, g->kw, g->sw, g->dw, &g->pwb, &g->pwe);
    }
    g->h_out = (g->h_in + g->phb + g->phe - (g->dh * (g->kh - 1) + 1)) / g->sh + 1;
    g->w_out = (g->w_in + g->pwb + g->pwe - (g->dw * (g->kw - 1) + 1)) / g->sw + 1;
    return (g->h_out > 0 && g->w_out > 0) ? 0 : 1;
}

/*
 * Direct integer convolution, one output at a time
 * (src/shaders/conv_integer.rs:73-110): NCHW x, [C_out, C_in/group, KH, KW] w,
 * per-tensor zero points, padding contributes exactly 0.  i32 accumulation
 * with wrap-around as on the device.
 */
ORC_EXPORT void orc_conv_integer(const uint8_t *x, int x_signed, const uint8_t *w, int w_signed,
                                 const orc_conv_geom *g, int32_t x_zp, int32_t w_zp, int32_t *out)
{
    int64_t gso = g->c_out / g->group;
    int64_t total_oc = g->n * g->c_out;
#pragma omp parallel for schedule(static)
    for (int64_t noc = 0; noc < total_oc; noc++) {
        int64_t bn = noc / g->c_out, m = noc % g->c_out;
        int64_t grp = m / gso;
        for (int64_t oh = 0; oh < g->h_out; oh++) {
            for (int64_t ow = 0; ow < g->w_out; ow++) {
                int32_t acc = 0;
                for (int64_t cg = 0; cg < g->gsi; cg++) {
                    int64_t ic = grp * g->gsi + cg;
                    for (int64_t r = 0; r < g->kh; r++) {
                        int64_t ih = oh * g->sh - g->phb + r * g->dh;
                        if (ih < 0 || ih >= g->h_in)
                            continue;
                        for (int64_t s = 0; s < g->kw; s++) {
                            int64_t iw = ow * g->sw - g->pwb + s * g->dw;
                            if (iw < 0 || iw >= g->w_in)
                                continue;
                            size_t xi = (size_t)(((bn * g->c_in + ic) * g->h_in + ih) * g->w_in + iw);
                            size_t wi = (size_t)(((m * g->gsi + cg) * g->kh + r) * g->kw + s);
                            acc += (int32_t)((byte_val(x, xi, x_signed) - x_zp) *
                                             (byte_val(w, wi, w_signed) - w_zp));
                        }
                    }
                }
                out[((bn * g->c_out + m) * g->h_out + oh) * g->w_out + ow] = acc;
            }
        }
    }
}

/* ratio[c] = x_scale * w_scale[c] / y_scale in f32, left to right
 * (src/interp.rs:4682-4694). */
ORC_EXPORT void orc_requantize_ratio(float x_scale, const float *w_scale, size_t n, float y_scale,
                                     float *ratio)
{
    for (size_t i = 0; i < n; i++) {
        volatile float p = x_scale * w_scale[i];
        ratio[i] = p / y_scale;
    }
}

/*
 * The epilogue of the QOperator family (src/shaders/qlinear.rs:28-63):
 * q = i32(rne(f32(acc + bias[c]) * ratio[c])) + y_zp, saturated to u8 or i8,
 * c = (i / inner) % axis_len.  bias may be NULL.
 */
ORC_EXPORT void orc_requantize(const int32_t *acc, size_t n, size_t inner, size_t axis_len,
                               const int32_t *bias, const float *ratio, int32_t y_zp,
                               int out_signed, uint8_t *out)
{
    if (inner == 0)
        inner = 1;
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        size_t c = (i / inner) % axis_len;
        int32_t a = acc[i];
        if (bias)
            a = (int32_t)((uint32_t)a + (uint32_t)bias[c]);
        volatile float prod = (float)a * ratio[c];
        float r = nearbyintf(prod);
        /* f32 -> i32 as the device converts it: saturating */
        int64_t qi;
        if (r >= 2147483648.0f)
            qi = INT32_MAX;
        else if (r <= -2147483648.0f)
            qi = INT32_MIN;
        else
            qi = (int64_t)r;
        int64_t q = (int64_t)(int32_t)((uint32_t)(int32_t)qi + (uint32_t)y_zp);
        if (out_signed) {
            if (q < -128)
                q = -128;
            if (q > 127)
                q = 127;
            out[i] = (uint8_t)(int8_t)q;
        } else {
            if (q < 0)
                q = 0;
            if (q > 255)
                q = 255;
            out[i] = (uint8_t)q;
        }
    }
}

/* ------------------------------------------------------------------------
 * GatherBlockQuantized: out[j, c] = (unpack(table[idx[j], c]) - zp) * scale in
 * f32 (crates/onnx-vulkan-core/src/shaders/gather_block_quantized.rs:40-57);
 * negative indices count from the end and an index outside the table is an
 * error (src/interp.rs:2896-2911).  table [rows, cols/2] u8 with element 2i in
 * the low nibble, scales [rows, cols/block_size] (f32 or f16), zero points
 * [rows, ceil(n_blocks/2)] u8 nibble packed or NULL (8).  out f32.
 * Returns 0, or 1 when an index is outside the table.
 */
ORC_EXPORT int orc_gather_block_quantized(const uint8_t *table, const int64_t *indices, size_t count,
                                          const void *scales, int scales_dtype, const uint8_t *zp,
                                          int64_t rows, int64_t cols, int64_t block_size, float *out)
{
    const size_t row_bytes = (size_t)cols / 2;
    const size_t n_blocks = (size_t)(cols / block_size);
    const size_t zp_row = (n_blocks + 1) / 2;
    for (size_t j = 0; j < count; j++) {
        int64_t r = indices[j];
        if (r < 0)
            r += rows;
        if (r < 0 || r >= rows)
            return 1;
    }
    for (size_t j = 0; j < count; j++) {
        int64_t r = indices[j] < 0 ? indices[j] + rows : indices[j];
        for (int64_t c = 0; c < cols; c++) {
            size_t block = (size_t)(c / block_size);
            float q = (float)nib_at(table, row_bytes, (size_t)r, (size_t)c);
            float z = zp ? (float)zp_at(zp, zp_row, (size_t)r, block) : 8.0f;
            float s = (float)load_real(scales, scales_dtype, (size_t)r * n_blocks + block);
            volatile float d = q - z;
            out[j * (size_t)cols + (size_t)c] = d * s;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------
 * ArgMax over one axis, first occurrence, as the device kernels decide it
 * (shaders/reduction.rs:97-131, :156-186): a value is a candidate only if it
 * is greater than -FLT_MAX (so NaN and -inf never are), larger wins, equal
 * values go to the smaller index, no candidate answers 0.  x is
 * [outer, c, inner] f32, out [outer*inner] int64.
 */
ORC_EXPORT void orc_argmax(const float *x, int64_t outer, int64_t c, int64_t inner, int64_t *out)
{
    for (int64_t r = 0; r < outer * inner; r++) {
        const int64_t base = (r / inner) * c * inner + r % inner;
        float best = -3.4028235e38f;
        int64_t at = 0;
        for (int64_t k = 0; k < c; k++) {
            float v = x[base + k * inner];
            if (v > best) {
                best = v;
                at = k;
            }
        }
        out[r] = at;
    }
}

/* ------------------------------------------------------------------------
 * QLinearAdd, MLAS's kernel operation for operation (shaders/qlinear.rs:69-143,
 * src/interp.rs:4878-4962, tests/qlinear.rs:317-322):
 *   ra = A_scale / C_scale, rb = B_scale / C_scale,
 *   fixed = c_zp - fma(ra, a_zp, rb * b_zp),
 *   C = saturate(rne(fma(A, ra, fma(B, rb, fixed)))),
 * the operands exchanged when A is constant along the innermost broadcast span
 * (or the output is one element).  Shapes broadcast numpy-style, rank <= 8.
 * out must hold the broadcast element count.  Returns 0, 1 on a shape error.
 */
ORC_EXPORT int orc_qlinear_add(const uint8_t *a, const int64_t *a_shape, int a_rank, float a_scale, int32_t a_zp,
                               const uint8_t *b, const int64_t *b_shape, int b_rank, float b_scale, int32_t b_zp,
                               float c_scale, int32_t c_zp, int is_signed, uint8_t *out)
{
    int rank = a_rank > b_rank ? a_rank : b_rank;
    int64_t shape[8], sa[8], sb[8], run_a = 1, run_b = 1, n = 1;
    if (rank > 8)
        return 1;
    for (int d = rank - 1; d >= 0; d--) {
        int da = d - (rank - a_rank), db = d - (rank - b_rank);
        int64_t ea = da >= 0 ? a_shape[da] : 1, eb = db >= 0 ? b_shape[db] : 1;
        if (ea != eb && ea != 1 && eb != 1)
            return 1;
        shape[d] = ea == 1 ? eb : ea;
        sa[d] = ea == 1 ? 0 : run_a;
        sb[d] = eb == 1 ? 0 : run_b;
        run_a *= ea;
        run_b *= eb;
        n *= shape[d];
    }
    float ra = a_scale / c_scale, rb = b_scale / c_scale;
    int inner = -1;
    for (int d = rank - 1; d >= 0; d--)
        if (shape[d] > 1) {
            inner = d;
            break;
        }
    if (inner < 0 || sa[inner] == 0) {
        const uint8_t *tp = a; a = b; b = tp;
        for (int d = 0; d < rank; d++) { int64_t t = sa[d]; sa[d] = sb[d]; sb[d] = t; }
        float tf = ra; ra = rb; rb = tf;
        int32_t tz = a_zp; a_zp = b_zp; b_zp = tz;
    }
    volatile float rbz = rb * (float)b_zp;
    float fixed = (float)c_zp - fmaf(ra, (float)a_zp, rbz);
    for (int64_t i = 0; i < n; i++) {
        int64_t rem = i, oa = 0, ob = 0, run = n;
        for (int d = 0; d < rank; d++) {
            run /= shape[d];
            int64_t c = rem / run;
            rem -= c * run;
            oa += c * sa[d];
            ob += c * sb[d];
        }
        int32_t av = is_signed ? (int8_t)a[oa] : a[oa], bv = is_signed ? (int8_t)b[ob] : b[ob];
        float y = nearbyintf(fmaf((float)av, ra, fmaf((float)bv, rb, fixed)));
        float lo = is_signed ? -128.0f : 0.0f, hi = is_signed ? 127.0f : 255.0f;
        y = y < lo ? lo : (y > hi ? hi : y);
        out[i] = (uint8_t)(int32_t)y;
    }
    return 0;
}

/* MaxPool on quantized codes (shaders/qlinear.rs:160-211): floor mode, padding taps skipped. */
ORC_EXPORT void orc_maxpool_q(const uint8_t *x, int is_signed, int64_t n, int64_t c, int64_t h, int64_t w,
                              const int64_t *kernel, const int64_t *strides, const int64_t *pads,
                              const int64_t *dilations, uint8_t *out)
{
    int64_t ho = (h + pads[0] + pads[2] - (dilations[0] * (kernel[0] - 1) + 1)) / strides[0] + 1;
    int64_t wo = (w + pads[1] + pads[3] - (dilations[1] * (kernel[1] - 1) + 1)) / strides[1] + 1;
    for (int64_t p = 0; p < n * c; p++)
        for (int64_t oh = 0; oh < ho; oh++)
            for (int64_t ow = 0; ow < wo; ow++) {
                int32_t acc = INT32_MIN;
                for (int64_t r = 0; r < kernel[0]; r++) {
                    int64_t ih = oh * strides[0] - pads[0] + r * dilations[0];
                    if (ih < 0 || ih >= h)
                        continue;
                    for (int64_t s = 0; s < kernel[1]; s++) {
                        int64_t iw = ow * strides[1] - pads[1] + s * dilations[1];
                        if (iw < 0 || iw >= w)
                            continue;
                        int32_t v = (int32_t)byte_val(x, (size_t)((p * h + ih) * w + iw), is_signed);
                        if (v > acc)
                            acc = v;
                    }
                }
                out[(p * ho + oh) * wo + ow] = (uint8_t)((uint32_t)acc & 0xffu);
            }
}

static inline int32_t sat_i32(float r)
{
    if (r != r)
        return 0;
    if (r >= 2147483648.0f)
        return INT32_MAX;
    if (r <= -2147483648.0f)
        return INT32_MIN;
    return (int32_t)r;
}

/* QuantizeLinear: saturate(rne(x / scale) + zero_point), channel (i / inner) % axis_len
 * (shaders/quantize_linear.rs:72-121).  zp may be NULL. */
ORC_EXPORT void orc_quantize_linear(const float *x, int64_t n, int64_t inner, int64_t axis_len, const float *scale,
                                    const uint8_t *zp, int is_signed, uint8_t *out)
{
    for (int64_t i = 0; i < n; i++) {
        int64_t c = (i / inner) % axis_len;
        int32_t zero = zp ? (int32_t)byte_val(zp, (size_t)c, is_signed) : 0;
        volatile float quot = x[i] / scale[c];
        int32_t q = (int32_t)((uint32_t)sat_i32(nearbyintf(quot)) + (uint32_t)zero);
        int32_t lo = is_signed ? -128 : 0, hi = is_signed ? 127 : 255;
        q = q < lo ? lo : (q > hi ? hi : q);
        out[i] = (uint8_t)((uint32_t)q & 0xffu);
    }
}

/* DequantizeLinear: (x - zero_point) * scale; kind 0 u8, 1 i8, 2 i32 (quantize_linear.rs:16-70). */
ORC_EXPORT void orc_dequantize_linear(const void *x, int kind, int64_t n, int64_t inner, int64_t axis_len,
                                      const float *scale, const void *zp, float *out)
{
    for (int64_t i = 0; i < n; i++) {
        int64_t c = (i / inner) % axis_len;
        int32_t q, zero = 0;
        if (kind == 2) {
            q = ((const int32_t *)x)[i];
            if (zp)
                zero = ((const int32_t *)zp)[c];
        } else {
            q = (int32_t)byte_val((const uint8_t *)x, (size_t)i, kind);
            if (zp)
                zero = (int32_t)byte_val((const uint8_t *)zp, (size_t)c, kind);
        }
        volatile float d = (float)(int32_t)((uint32_t)q - (uint32_t)zero);
        out[i] = d * scale[c];
    }
}

/* QLinearGlobalAveragePool = DequantizeLinear, GlobalAveragePool (a sequential f32 sum in
 * row-major order divided by the count, shaders/pooling.rs:38-54), QuantizeLinear
 * (src/interp.rs:4975-5000, tests/qlinear.rs:419-452). */
ORC_EXPORT void orc_qlinear_global_average_pool(const uint8_t *x, int is_signed, int64_t planes, int64_t hw,
                                                float x_scale, int32_t x_zp, float y_scale, int32_t y_zp,
                                                uint8_t *out)
{
    for (int64_t p = 0; p < planes; p++) {
        volatile float acc = 0.0f;
        for (int64_t i = 0; i < hw; i++) {
            volatile float v = (float)((int32_t)byte_val(x, (size_t)(p * hw + i), is_signed) - x_zp) * x_scale;
            acc = acc + v;
        }
        volatile float mean = acc / (float)(uint32_t)(hw > 0 ? hw : 1);
        volatile float quot = mean / y_scale;
        int32_t q = (int32_t)((uint32_t)sat_i32(nearbyintf(quot)) + (uint32_t)y_zp);
        int32_t lo = is_signed ? -128 : 0, hi = is_signed ? 127 : 255;
        q = q < lo ? lo : (q > hi ? hi : q);
        out[p] = (uint8_t)((uint32_t)q & 0xffu);
    }
}
