// ConvInteger / QLinearConv: host logic, the direct kernel that covers every
// geometry (groups, depthwise, 1-D, strides, dilations), and REQUANTIZE.
//
// Host side mirrors interp::conv_integer_with (crates/onnx-vulkan-core/src/
// interp.rs:4421-4651), conv_geometry (:3439-3536), qlinear_conv (:4796-4837)
// and requantize (:4714-4788).  The direct kernel follows
// src/shaders/conv_integer.rs:73-110 (one thread per output, padding
// contributes exactly 0) with the requantising epilogue of
// src/shaders/qlinear.rs:28-63 applied in the same pass instead of a second one.
#include "ovk_internal.h"
#include "epilogue.cuh"

#include <cstring>

bool ovk_qconv_tc_applies(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, const void *x);
int32_t ovk_qconv_tc_launch(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                            const ConvGeom &g, int32_t x_zp, int32_t w_zp, const EpiParams &epi,
                            void *out, const ConvLayout &lay);
int32_t ovk_qconv_pad_nhwc(ovk_ctx *ctx, const void *x, const ConvGeom &g, int32_t fill, uint8_t *xp);
int32_t ovk_qconv_tc_prepare_weight(ovk_ctx *ctx, ovk_qconv_weight *w);
int ovk_qconv_tc_launches(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, const void *x);
bool ovk_mmi_tc_applies(const ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int64_t m);
int32_t ovk_mmi_tc_launch_with_row_sums(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed, int64_t m,
                                        const void *a_zp, const void *b_zp, const EpiParams &epi, void *out,
                                        const int32_t *row_sums);

namespace {

__device__ __forceinline__ int32_t sx8(uint8_t b, int is_signed)
{
    return is_signed ? int32_t(int8_t(b)) : int32_t(b);
}

__device__ __forceinline__ int32_t conv_point(const uint8_t *__restrict__ x, const uint8_t *__restrict__ w,
                                              const ConvGeom &g, int x_signed, int w_signed, int32_t x_zp,
                                              int32_t w_zp, int64_t o, int *channel)
{
    const int ow = int(o % g.w_out);
    int64_t t1 = o / g.w_out;
    const int oh = int(t1 % g.h_out);
    t1 /= g.h_out;
    const int m = int(t1 % g.c_out);
    const int64_t bn = t1 / g.c_out;
    const int gso = g.c_out / g.group;
    const int grp = m / gso;
    int32_t acc = 0;
    for (int cg = 0; cg < g.cig; cg++) {
        const int ic = grp * g.cig + cg;
        for (int r = 0; r < g.kh; r++) {
            const int ih = oh * g.sh - g.phb + r * g.dh;
            if (ih < 0 || ih >= g.h_in)
                continue;
            for (int s = 0; s < g.kw; s++) {
                const int iw = ow * g.sw - g.pwb + s * g.dw;
                if (iw < 0 || iw >= g.w_in)
                    continue;
                const int64_t xi = ((bn * g.c_in + ic) * g.h_in + ih) * int64_t(g.w_in) + iw;
                const int64_t wi = ((int64_t(m) * g.cig + cg) * g.kh + r) * g.kw + s;
                acc += (sx8(x[xi], x_signed) - x_zp) * (sx8(w[wi], w_signed) - w_zp);
            }
        }
    }
    *channel = m;
    return acc;
}

__global__ void __launch_bounds__(256)
conv_direct_kernel(const uint8_t *__restrict__ x, const uint8_t *__restrict__ w, ConvGeom g,
                   int x_signed, int w_signed, int32_t x_zp, int32_t w_zp, EpiParams epi,
                   void *out, int64_t total)
{
    const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    float v = 0.0f;  // what a thread past the end contributes to the range fold
    if (o < total) {
        int m;
        const int32_t acc = conv_point(x, w, g, x_signed, w_signed, x_zp, w_zp, o, &m);
        if (epi.mode == EPI_RAW) {
            static_cast<int32_t *>(out)[o] = acc;
        } else if (epi.mode == EPI_SCALE) {
            v = epi_scale_value(epi, m, float(acc));
            static_cast<float *>(out)[o] = v;
        } else {
            static_cast<uint8_t *>(out)[o] = uint8_t(epi_requant_value(epi, m, acc));
        }
    }
    if (epi.mode == EPI_SCALE)  // uniform over the grid: the fold's warp exchange sees all 32 lanes
        epi_fold_range(epi, fmaxf(v, 0.0f), fmaxf(-v, 0.0f));
}

// Depthwise convolution (one filter per channel, group = C_in = C_out): a block takes 256 consecutive outputs
// of ONE plane, so the channel - and with it the filter, which goes to shared memory once, and all the
// per-channel constants - is the block's, a thread needs one division for its row, and neighbouring threads read
// neighbouring input bytes.  Same arithmetic and epilogue as the direct kernel.
constexpr int DW_MAX_TAPS = 128;
__global__ void __launch_bounds__(256)
conv_depthwise_kernel(const uint8_t *__restrict__ x, const uint8_t *__restrict__ w, ConvGeom g, int x_signed, int w_signed,
                      int32_t x_zp, int32_t w_zp, EpiParams epi, void *out)
{
    __shared__ int32_t taps[DW_MAX_TAPS];
    const int plane_out = g.h_out * g.w_out;
    const int pc = blockIdx.y;  // image * C + channel
    const int c = pc % g.c_out;
    const int ntaps = g.kh * g.kw;
    for (int i = threadIdx.x; i < ntaps; i += 256)
        taps[i] = sx8(w[size_t(c) * ntaps + i], w_signed) - w_zp;
    __syncthreads();
    const int pix = blockIdx.x * 256 + threadIdx.x;
    float v = 0.0f;
    if (pix < plane_out) {
        const int oh = pix / g.w_out, ow = pix - oh * g.w_out;
        const uint8_t *xp = x + size_t(pc) * g.h_in * g.w_in;
        int32_t acc = 0;
        for (int r = 0; r < g.kh; r++) {
            const int ih = oh * g.sh - g.phb + r * g.dh;
            if (ih < 0 || ih >= g.h_in)
                continue;
            for (int s2 = 0; s2 < g.kw; s2++) {
                const int iw = ow * g.sw - g.pwb + s2 * g.dw;
                if (iw < 0 || iw >= g.w_in)
                    continue;
                acc += (sx8(xp[size_t(ih) * g.w_in + iw], x_signed) - x_zp) * taps[r * g.kw + s2];
            }
        }
        const size_t o = size_t(pc) * plane_out + pix;
        if (epi.mode == EPI_RAW) {
            static_cast<int32_t *>(out)[o] = acc;
        } else if (epi.mode == EPI_SCALE) {
            v = epi_scale_value(epi, c, float(acc));
            static_cast<float *>(out)[o] = v;
        } else {
            static_cast<uint8_t *>(out)[o] = uint8_t(epi_requant_value(epi, c, acc));
        }
    }
    if (epi.mode == EPI_SCALE)
        epi_fold_range(epi, fmaxf(v, 0.0f), fmaxf(-v, 0.0f));
}

// REQUANTIZE on its own (shaders/qlinear.rs:28-63): four outputs per thread.
__global__ void __launch_bounds__(256)
requantize_kernel(const int32_t *__restrict__ acc, int64_t n, int64_t inner, int64_t axis_len,
                  EpiParams epi, uint8_t *__restrict__ out)
{
    const int64_t base = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (base >= n)
        return;
    uint32_t packed = 0;
    int j = 0;
    for (; j < 4 && base + j < n; j++) {
        const int64_t i = base + j;
        const int64_t c = (i / inner) % axis_len;
        packed |= (uint32_t(epi_requant_value(epi, c, acc[i])) & 0xffu) << (8 * j);
    }
    if (j == 4 && ((reinterpret_cast<uintptr_t>(out) & 3) == 0)) {
        *reinterpret_cast<uint32_t *>(out + base) = packed;
    } else {
        for (int t = 0; t < j; t++)
            out[base + t] = uint8_t(packed >> (8 * t));
    }
}

int32_t make_geom(ovk_ctx *ctx, const ovk_qconv_weight *w, const ovk_conv_params *p, ConvGeom *g,
                  const char *op)
{
    OVK_REQUIRE(ctx, p->n >= 0 && p->c_in > 0 && p->h > 0 && p->w > 0, "%s: bad input shape", op);
    OVK_REQUIRE(ctx, p->c_in == w->cig * w->group, "%s: input has %lld channels, the weight expects %lld x %lld groups",
                op, (long long)p->c_in, (long long)w->cig, (long long)w->group);
    OVK_REQUIRE(ctx, w->c_out % w->group == 0, "%s: C_out %lld is not a multiple of group %lld", op,
                (long long)w->c_out, (long long)w->group);
    OVK_REQUIRE(ctx, p->strides[0] > 0 && p->strides[1] > 0 && p->dilations[0] > 0 && p->dilations[1] > 0,
                "%s: strides and dilations must be positive", op);
    OVK_REQUIRE(ctx, p->pads[0] >= 0 && p->pads[1] >= 0 && p->pads[2] >= 0 && p->pads[3] >= 0,
                "%s: negative padding", op);
    const int64_t h_out = (p->h + p->pads[0] + p->pads[2] - (p->dilations[0] * (w->kh - 1) + 1)) / p->strides[0] + 1;
    const int64_t w_out = (p->w + p->pads[1] + p->pads[3] - (p->dilations[1] * (w->kw - 1) + 1)) / p->strides[1] + 1;
    OVK_REQUIRE(ctx, h_out > 0 && w_out > 0, "%s: degenerate output shape", op);
    OVK_REQUIRE(ctx, p->n * w->c_out * h_out * w_out < (int64_t(1) << 40) && p->h < (1 << 24) && p->w < (1 << 24),
                "%s: tensor too large", op);
    g->n = int(p->n);
    g->c_in = int(p->c_in);
    g->c_out = int(w->c_out);
    g->group = int(w->group);
    g->cig = int(w->cig);
    g->h_in = int(p->h);
    g->w_in = int(p->w);
    g->h_out = int(h_out);
    g->w_out = int(w_out);
    g->kh = int(w->kh);
    g->kw = int(w->kw);
    g->sh = int(p->strides[0]);
    g->sw = int(p->strides[1]);
    g->dh = int(p->dilations[0]);
    g->dw = int(p->dilations[1]);
    g->phb = int(p->pads[0]);
    g->pwb = int(p->pads[1]);
    g->phe = int(p->pads[2]);
    g->pwe = int(p->pads[3]);
    return OVK_OK;
}

// [n][h + frame][w + frame][c] -> NCHW: the end of a channels-last chain.  A block takes one image row:
// its pixels go through shared memory so that reads run along C and writes along W.
__global__ void __launch_bounds__(256)
unpad_nchw_kernel(const uint8_t *__restrict__ xp, uint8_t *__restrict__ out, int C, int H, int W, int HP, int WP, int pt,
                  int pl)
{
    extern __shared__ uint8_t row[];  // [W][C + 1]
    const int h = blockIdx.x, n = blockIdx.y;
    const uint8_t *src = xp + ((size_t(n) * HP + h + pt) * WP + pl) * size_t(C);
    for (int i = threadIdx.x; i < W * C; i += blockDim.x)
        row[(i / C) * (C + 1) + i % C] = src[i];
    __syncthreads();
    for (int i = threadIdx.x; i < W * C; i += blockDim.x) {
        const int c = i / W, w = i - c * W;
        out[((size_t(n) * C + c) * H + h) * W + w] = row[w * (C + 1) + c];
    }
}

// One image [C][P] of bytes -> [P][C] (pixels become rows with their channels contiguous): 64 x 64 tiles
// through shared memory, 32-bit accesses on both sides where the rows allow it.
__global__ void __launch_bounds__(256)
pixels_major_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ out, int C, int P, int words_ok)
{
    __shared__ uint8_t tile[64][68];  // [channel][pixel], rows padded against bank conflicts
    const int c0 = blockIdx.y * 64, p0 = blockIdx.x * 64;
    const int t = threadIdx.x;
    for (int i = 0; i < 4; i++) {
        const int c = c0 + (t >> 4) + 16 * i, pp = p0 + 4 * (t & 15);
        uint32_t v = 0;
        if (c < C) {
            if (words_ok && pp + 4 <= P) {
                v = *reinterpret_cast<const uint32_t *>(x + size_t(c) * P + pp);
            } else {
                for (int e = 0; e < 4; e++)
                    if (pp + e < P)
                        v |= uint32_t(x[size_t(c) * P + pp + e]) << (8 * e);
            }
        }
        *reinterpret_cast<uint32_t *>(&tile[(t >> 4) + 16 * i][4 * (t & 15)]) = v;
    }
    __syncthreads();
    for (int i = 0; i < 4; i++) {
        const int pp = (t >> 4) + 16 * i, cc = 4 * (t & 15);
        if (p0 + pp < P && c0 + cc < C) {  // C is a multiple of 16: a group of four channels exists whole
            const uint32_t v = uint32_t(tile[cc][pp]) | (uint32_t(tile[cc + 1][pp]) << 8) | (uint32_t(tile[cc + 2][pp]) << 16) |
                               (uint32_t(tile[cc + 3][pp]) << 24);
            *reinterpret_cast<uint32_t *>(out + size_t(p0 + pp) * C + c0 + cc) = v;
        }
    }
}

// sum of a filter's weights, one warp per filter (the zero-point term of the pointwise product)
__global__ void __launch_bounds__(256)
filter_sums_kernel(const uint8_t *__restrict__ w, int c_out, int k, int w_signed, int32_t *__restrict__ sums)
{
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= c_out)
        return;
    int32_t s = 0;
    for (int i = lane; i < k; i += 32)
        s += sx8(w[size_t(row) * k + i], w_signed);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        sums[row] = s;
}

// One image -> its patch matrix [output pixels][C_in * KH * KW], a patch in the order the operator lays a
// filter out (channel, then row, then column), positions in the padding holding the image's zero point so
// that they contribute (zp - zp) * w = 0.  One byte per thread: this route is for matrices of a few MB.
// (`pitch` >= K: rows padded to whole 16-byte units; the padding is written as 0 and meets zero filter bytes.)
// (`images`: that many consecutive images, their patch rows one image after the other.)
// A thread builds 16 consecutive bytes of a patch row and stores them at once, stepping (channel, row, column)
// from byte to byte instead of dividing for each.
__global__ void __launch_bounds__(256)
patches_kernel(const uint8_t *__restrict__ x0, uint8_t *__restrict__ out, ConvGeom g, int x_zp, int pitch, int images,
               uint32_t pad_byte)
{
    const int taps = g.kh * g.kw, K = g.c_in * taps;
    const int plane = g.h_out * g.w_out;
    const int chunks = pitch >> 4;  // pitch is a multiple of 16
    const int64_t total = int64_t(images) * plane * chunks;
    const size_t in_plane = size_t(g.h_in) * g.w_in;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int64_t row = i / chunks;
        const int kk0 = int(i - row * chunks) << 4;
        const int img = int(row / plane), pix = int(row - int64_t(img) * plane);
        const int oh = pix / g.w_out, ow = pix - oh * g.w_out;
        const int ih0 = oh * g.sh - g.phb, iw0 = ow * g.sw - g.pwb;
        int c = kk0 / taps, t = kk0 - c * taps;
        int r = t / g.kw, s2 = t - r * g.kw;
        const uint8_t *xc = x0 + (size_t(img) * g.c_in + c) * in_plane;
        uint32_t words[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int e = 0; e < 16; e++) {
            uint32_t byte = pad_byte;  // beyond K: 0, or the zero point where the filters' padding holds theirs
            if (kk0 + e < K) {
                const int ih = ih0 + r * g.dh, iw = iw0 + s2 * g.dw;
                byte = (ih >= 0 && ih < g.h_in && iw >= 0 && iw < g.w_in) ? xc[size_t(ih) * g.w_in + iw] : uint32_t(x_zp & 0xff);
                if (++s2 == g.kw) {
                    s2 = 0;
                    if (++r == g.kh) {
                        r = 0;
                        xc += in_plane;
                    }
                }
            }
            words[e >> 2] |= byte << (8 * (e & 3));
        }
        *reinterpret_cast<uint4 *>(out + size_t(row) * pitch + kk0) = make_uint4(words[0], words[1], words[2], words[3]);
    }
}

// The same matrix built a row of output pixels at a time: the input rows that row of patches looks at - all
// channels, with their frame of zero-point bytes - are laid down in shared memory once (coalesced reads, the
// bounds decided there), and the patch rows are assembled from shared memory (the 7 x 7 stem of a
// ResNet).  Taken when those rows are few and long and fit in 48 KB.
__global__ void __launch_bounds__(256)
patches_rows_kernel(const uint8_t *__restrict__ x0, uint8_t *__restrict__ out, ConvGeom g, int x_zp, int pitch, int wpad,
                    uint32_t pad_byte)
{
    extern __shared__ uint8_t rows[];  // [c_in][kh][wpad], column 0 = input column -pwb
    const int oh = blockIdx.x, img = blockIdx.y;
    const int taps = g.kh * g.kw, K = g.c_in * taps;
    const size_t in_plane = size_t(g.h_in) * g.w_in;
    const uint8_t *xi = x0 + size_t(img) * g.c_in * in_plane;
    const int ih0 = oh * g.sh - g.phb;
    const int lines = g.c_in * g.kh;
    const uint8_t zp = uint8_t(x_zp & 0xff);
    // a warp per line of the slab, its lanes along the line
    for (int line = threadIdx.x >> 5; line < lines; line += 8) {
        const int c = line / g.kh, r = line - c * g.kh;
        const int ih = ih0 + r * g.dh;
        const bool inside = ih >= 0 && ih < g.h_in;
        const uint8_t *src = xi + size_t(c) * in_plane + size_t(inside ? ih : 0) * g.w_in;
        uint8_t *dst = rows + size_t(line) * wpad;
        for (int i = threadIdx.x & 31; i < wpad; i += 32) {
            const int iw = i - g.pwb;
            dst[i] = (inside && iw >= 0 && iw < g.w_in) ? src[iw] : zp;
        }
    }
    __syncthreads();
    // A thread owns one 32-bit word of the patch row - its four positions in the slab are worked out once - and
    // walks along the output pixels with it; the threads of a patch row write its words side by side.
    // (Sixteen bytes per thread with (channel, row, column) stepped from byte to byte cost four times the
    // instructions, and the pass was bound by them.)
    const int words = pitch >> 2, per_pass = 256 / words;  // pitch <= 1024
    const int word = threadIdx.x % words, sub = threadIdx.x / words;
    if (sub >= per_pass)
        return;
    int off[4];
    uint32_t mask = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int kk = word * 4 + e;
        off[e] = 0;
        if (kk < K) {
            const int c = kk / taps, t = kk - c * taps;
            const int r = t / g.kw, s2 = t - r * g.kw;
            off[e] = (c * g.kh + r) * wpad + s2 * g.dw;
            mask |= 0xffu << (8 * e);
        }
    }
    uint32_t *out_row = reinterpret_cast<uint32_t *>(out + (size_t(img) * g.h_out + oh) * g.w_out * size_t(pitch));
    for (int ow = sub; ow < g.w_out; ow += per_pass) {
        const uint8_t *base = rows + ow * g.sw;
        const uint32_t v = uint32_t(base[off[0]]) | (uint32_t(base[off[1]]) << 8) | (uint32_t(base[off[2]]) << 16) |
                           (uint32_t(base[off[3]]) << 24);
        out_row[size_t(ow) * words + word] = (v & mask) | (~mask & (pad_byte * 0x01010101u));
    }
}

// sum of every patch row (the term the filters' zero point multiplies), one warp per row
__global__ void __launch_bounds__(256)
patch_sums_kernel(const uint8_t *__restrict__ patches, int64_t rows, int pitch, int x_signed, int32_t *__restrict__ sums)
{
    const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows)
        return;
    const uint32_t *w = reinterpret_cast<const uint32_t *>(patches + size_t(row) * pitch);  // pitch is a multiple of 16
    int32_t s = 0;
    for (int i = lane; i < pitch / 4; i += 32)
        s = x_signed ? __dp4a(int(w[i]), int(0x01010101), s) : int32_t(__dp4a(w[i], 0x01010101u, uint32_t(s)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        sums[row] = s;
}

// [C_out][images * plane] -> [images][C_out][plane]: the product over several images' patches back to NCHW
template <typename T>
__global__ void __launch_bounds__(256)
unbatch_kernel(const T *__restrict__ d, T *__restrict__ out, int c_out, int images, int plane)
{
    const int64_t total = int64_t(images) * c_out * plane;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int pix = int(i % plane);
        const int64_t t = i / plane;
        const int co = int(t % c_out), img = int(t / c_out);
        out[i] = d[(size_t(co) * images + img) * plane + pix];
    }
}

// ... and a warp per plane, for planes of any size (7 x 7): no division per byte
__global__ void __launch_bounds__(256)
unbatch_planes_kernel(const uint8_t *__restrict__ d, uint8_t *__restrict__ out, int c_out, int images, int plane_bytes)
{
    const int lane = threadIdx.x & 31;
    const int64_t planes = int64_t(images) * c_out;
    for (int64_t w = (int64_t(blockIdx.x) * 256 + threadIdx.x) >> 5; w < planes; w += int64_t(gridDim.x) * 8) {
        const int co = int(w % c_out), img = int(w / c_out);
        const uint8_t *src = d + (size_t(co) * images + img) * plane_bytes;
        uint8_t *dst = out + size_t(w) * plane_bytes;
        for (int i = lane; i < plane_bytes; i += 32)
            dst[i] = src[i];
    }
}

// the same in 16-byte pieces, for planes that are whole pieces (a byte at a time the pass ran at 0.5 TB/s)
__global__ void __launch_bounds__(256)
unbatch_pieces_kernel(const uint4 *__restrict__ d, uint4 *__restrict__ out, int c_out, int images, int pieces)
{
    const int64_t total = int64_t(images) * c_out * pieces;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int piece = int(i % pieces);
        const int64_t t = i / pieces;
        const int co = int(t % c_out), img = int(t / c_out);
        out[i] = d[(size_t(co) * images + img) * pieces + piece];
    }
}

// filters [C_out][K] -> [C_out][pitch], the tail of every row `fill` (K is no multiple of 16: 7 x 7 over 3 channels)
__global__ void __launch_bounds__(256)
pad_filter_rows_kernel(const uint8_t *__restrict__ w, uint8_t *__restrict__ out, int c_out, int K, int pitch, uint8_t fill)
{
    const int64_t total = int64_t(c_out) * pitch;
    for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x) * 256) {
        const int row = int(i / pitch), kk = int(i - int64_t(row) * pitch);
        out[i] = kk < K ? w[size_t(row) * K + kk] : fill;
    }
}

// A convolution as the product filters [C_out][K] x patches [K][pixels], K = C_in * KH * KW - the route the
// reference takes at batch 1 (to_hwc + im2col + its cooperative-matrix GEMM, src/shaders/conv_integer.rs:374-527).
// The filter bank in the operator's own layout is the row operand of the MatMulInteger tensor-core kernels;
// the patch matrix of one image, [pixels][K], takes the place of the packed weight (a view: no copy, no
// padding, the bulk loads zero-fill what lies outside); the result [C_out][pixels] is the NCHW output as it
// stands, and the per-channel constants of the epilogue belong to the rows (EpiParams::by_row).  For a 1 x 1,
// stride-1, unpadded layer the patch matrix is the image turned pixels-major.
// Taken when the convolution kernel would need three launches or more for the filter bank (one per 32-256
// filters that fit in shared memory) or does not take the geometry at all, for up to four images whose patch matrices stay small: the pointwise layers of
// the dynamic-int8 encoder (1024 -> 2048 over a thousand frames: 6.5 ms on the one-output-per-thread kernel
// they used to take) and the last stages of a ResNet at batch 1 (512 -> 512 3 x 3 on 7 x 7: 0.55 ms).
#ifndef OVK_GEMM_ROUTE_MAX_IMAGES
#define OVK_GEMM_ROUTE_MAX_IMAGES 4
#endif
#ifndef OVK_GEMM_ROUTE_FEW_PIXELS
#define OVK_GEMM_ROUTE_FEW_PIXELS 3200
#endif
constexpr int64_t GEMM_ROUTE_MAX_BYTES = int64_t(32) << 20;

bool gemm_route_applies(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, int32_t w_zp, const ConvLayout &lay,
                        const void *x)
{
    if (g.group != 1 || lay.x_cl || lay.y_cl)
        return false;
    // the convolution kernel in one launch - two for filters larger than 1 x 1 - is the faster way
    // (128 -> 128 3 x 3 on 28 x 28: 12 against 21 us; 1024 -> 256 1 x 1 on 14 x 14 in two launches: 33 against 15 us),
    // and so it is for more than a few images, one product per image being what this route costs; where the
    // convolution kernel does not take the geometry at all (the 7 x 7 stem over 3 channels) any batch comes here
    const int conv_launches = w_zp != 0 ? 0 : ovk_qconv_tc_launches(ctx, w, g, x);  // symmetric weights only, there
    // (measured at 8 and 64 images: this route wins while images x output pixels stay small - 7 x 7 planes at 64
    // images 340 -> 60 us, 14 x 14 at 8 images 56 -> 27 us - and loses beyond: 14 x 14 at 64 images 69 -> 92 us)
    // (a strided filter larger than 1 x 1 is computed at every position by the convolution kernel and kept
    // on the stride lattice only: against it this route holds on for stride x stride times as many pixels -
    // 256 -> 256 3 x 3 stride 2 on 28 x 28 at 64 images: 175 -> 85 us)
    const bool few_kept = g.kh * g.kw > 1 && g.sh * g.sw >= 4 && conv_launches >= 3 &&
                          int64_t(g.n) * g.h_out * g.w_out <= int64_t(OVK_GEMM_ROUTE_FEW_PIXELS) * g.sh * g.sw;
    const bool few = g.n <= OVK_GEMM_ROUTE_MAX_IMAGES || int64_t(g.n) * g.h_out * g.w_out <= OVK_GEMM_ROUTE_FEW_PIXELS;
    if (conv_launches == 1 || (conv_launches == 2 && g.kh * g.kw > 1) || (conv_launches > 0 && !few && !few_kept))
        return false;
    const int64_t K = (int64_t(g.c_in) * g.kh * g.kw + 15) / 16 * 16, pixels = int64_t(g.h_out) * g.w_out;
    if (pixels * K > GEMM_ROUTE_MAX_BYTES)
        return false;
    ovk_mmi_weight patches = {};
    patches.k = K;
    patches.n = pixels;
    return ovk_mmi_tc_applies(ctx, &patches, w->w, g.c_out);  // (a padded copy of the filters is as well aligned)
}

int32_t run_gemm_route(ovk_ctx *ctx, const ovk_qconv_weight *wc, const void *x, int32_t x_signed, const ConvGeom &g,
                       int32_t x_zp, int32_t w_zp, EpiParams epi, void *out, size_t out_elem)
{
    ovk_qconv_weight *w = const_cast<ovk_qconv_weight *>(wc);  // the filter sums are built at first use
    const int K_true = g.c_in * g.kh * g.kw;
    const int K = (K_true + 15) / 16 * 16;  // rows of both operands in whole 16-byte units
    const int64_t pixels = int64_t(g.h_out) * g.w_out;
    if (!w->wsum) {
        OVK_CUDA(ctx, cudaMalloc(&w->wsum, size_t(g.c_out) * sizeof(int32_t)));
        filter_sums_kernel<<<unsigned(ceil_div64(int64_t(g.c_out) * 32, 256)), 256, 0, ctx->stream>>>(w->w, g.c_out, K_true,
                                                                                                     w->w_signed, w->wsum);
        OVK_LAUNCHED(ctx, "conv_filter_sums");
    }
    const uint8_t *filters = w->w;
    // An asymmetric weight over rows padded to 16 bytes: with zero padding the terms of the zero points
    // (K * w_zp * x_zp, w_zp * sum of a patch, x_zp * sum of a filter) would count the padding.  The padding of
    // both operands holds the operand's own zero point instead - (x_zp - x_zp) * (w_zp - w_zp) = 0 - and the sums
    // are taken over the padded rows; that copy of the filters depends on the call's w_zp and lives in the
    // scratch buffer (C_out x K bytes: 10 KB for the 7 x 7 stem).
    const bool zp_padding = w_zp != 0 && K != K_true;
    if (K != K_true && !zp_padding) {
        if (!w->w_rows16) {
            OVK_CUDA(ctx, cudaMalloc(&w->w_rows16, size_t(g.c_out) * K));
            pad_filter_rows_kernel<<<unsigned(ceil_div64(int64_t(g.c_out) * K, 256)), 256, 0, ctx->stream>>>(w->w, w->w_rows16,
                                                                                                             g.c_out, K_true, K, uint8_t(0));
            OVK_LAUNCHED(ctx, "conv_pad_filter_rows");
        }
        filters = w->w_rows16;
    }
    // Images per product: as many as keep the patch matrix under its limit.  Several images' patches are one
    // matrix [images * pixels][K]; their product [C_out][images * pixels] is then put back image by image.
    const int group = int(std::max<int64_t>(1, std::min<int64_t>(g.n, GEMM_ROUTE_MAX_BYTES / (pixels * K))));
    const size_t patch_bytes = (size_t(group) * pixels * K + 255) & ~size_t(255);
    const size_t d_bytes = group > 1 ? (size_t(g.c_out) * group * pixels * out_elem + 255) & ~size_t(255) : 0;
    const size_t sums_bytes = w_zp != 0 ? (size_t(group) * pixels * sizeof(int32_t) + 255) & ~size_t(255) : 0;
    const size_t fpad_bytes = zp_padding ? (size_t(g.c_out) * K + 255) & ~size_t(255) : 0;
    const size_t fsum_bytes = zp_padding ? (size_t(g.c_out) * sizeof(int32_t) + 255) & ~size_t(255) : 0;
    void *ws = nullptr;
    int32_t rc = ovk_scratch(ctx, patch_bytes + d_bytes + sums_bytes + fpad_bytes + fsum_bytes + 256, &ws);
    if (rc != OVK_OK)
        return rc;
    uint8_t *patches_dev = static_cast<uint8_t *>(ws);
    uint8_t *d_dev = patches_dev + patch_bytes;
    int32_t *sums_dev = reinterpret_cast<int32_t *>(d_dev + d_bytes);
    const int32_t *filter_sums = w->wsum;
    if (zp_padding) {
        uint8_t *fpad = reinterpret_cast<uint8_t *>(sums_dev) + sums_bytes;
        int32_t *fsum = reinterpret_cast<int32_t *>(fpad + fpad_bytes);
        pad_filter_rows_kernel<<<unsigned(ceil_div64(int64_t(g.c_out) * K, 256)), 256, 0, ctx->stream>>>(w->w, fpad, g.c_out, K_true, K,
                                                                                                         uint8_t(w_zp & 0xff));
        OVK_LAUNCHED(ctx, "conv_pad_filter_rows");
        filter_sums_kernel<<<unsigned(ceil_div64(int64_t(g.c_out) * 32, 256)), 256, 0, ctx->stream>>>(fpad, g.c_out, K, w->w_signed, fsum);
        OVK_LAUNCHED(ctx, "conv_filter_sums");
        filters = fpad;
        filter_sums = fsum;
    }
    const uint32_t pad_byte = zp_padding ? uint32_t(x_zp) & 0xffu : 0u;
    // the zero points where the kernels read zero points: in device memory (the image's, then the filters')
    uint8_t *zp_dev = reinterpret_cast<uint8_t *>(ctx->range_slot + 40);
    if (x_zp != 0)
        OVK_CUDA(ctx, cudaMemsetAsync(zp_dev, x_zp & 0xff, 1, ctx->stream));
    if (w_zp != 0)
        OVK_CUDA(ctx, cudaMemsetAsync(zp_dev + 1, w_zp & 0xff, 1, ctx->stream));
    ovk_mmi_weight patches = {};
    patches.k = K;
    patches.k_pad = K;
    patches.b_signed = x_signed ? 1 : 0;
    patches.bt = patches_dev;
    // column sums enter only multiplied by the filters' zero point: when that is 0 any readable words do
    patches.colsum = w_zp != 0 ? sums_dev : reinterpret_cast<int32_t *>(patches_dev);
    epi.by_row = 1;
    const bool turn_only = K == K_true && g.kh == 1 && g.kw == 1 && g.sh == 1 && g.sw == 1 && !g.phb && !g.phe && !g.pwb && !g.pwe;
    const int64_t in_pixels = int64_t(g.h_in) * g.w_in;
    const int words_ok = (in_pixels % 4) == 0 && aligned_to(x, 4);
    for (int img = 0; img < g.n; img += group) {
        const int images = std::min(group, g.n - img);
        const uint8_t *xi = static_cast<const uint8_t *>(x) + size_t(img) * g.c_in * in_pixels;
        if (turn_only && images == 1) {
            pixels_major_kernel<<<dim3(unsigned(ceil_div64(pixels, 64)), unsigned(ceil_div64(g.c_in, 64))), 256, 0, ctx->stream>>>(
                xi, patches_dev, g.c_in, int(pixels), words_ok);
            OVK_LAUNCHED(ctx, "conv_pixels_major");
        } else {
            const int wpad = g.w_in + g.pwb + g.pwe;
            const size_t slab = size_t(g.c_in) * g.kh * wpad;
            // (few, long lines: with the 1536 lines of 9 bytes of a 512-channel 3 x 3 layer on 7 x 7 the fill
            // of the slab is a chain of short loads and the pass takes three times as long as the plain one)
            if (slab <= 48 * 1024 && g.c_in * g.kh <= 64 && wpad >= 64 && K <= 1024 && g.h_out <= 65535 && images <= 65535) {
                patches_rows_kernel<<<dim3(unsigned(g.h_out), unsigned(images)), 256, slab, ctx->stream>>>(xi, patches_dev, g, x_zp, K, wpad,
                                                                                                           pad_byte);
            } else {
                const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(int64_t(images) * pixels * K, 256), int64_t(ctx->sm_count) * 32));
                patches_kernel<<<blocks, 256, 0, ctx->stream>>>(xi, patches_dev, g, x_zp, K, images, pad_byte);
            }
            OVK_LAUNCHED(ctx, "conv_patches");
        }
        patches.n = int64_t(images) * pixels;
        patches.n_pad = patches.n;
        if (w_zp != 0) {
            patch_sums_kernel<<<unsigned(ceil_div64(patches.n * 32, 256)), 256, 0, ctx->stream>>>(patches_dev, patches.n, K, x_signed,
                                                                                                  sums_dev);
            OVK_LAUNCHED(ctx, "conv_patch_sums");
        }
        uint8_t *dst = static_cast<uint8_t *>(out) + size_t(img) * g.c_out * pixels * out_elem;
        rc = ovk_mmi_tc_launch_with_row_sums(ctx, &patches, filters, w->w_signed, g.c_out, w_zp != 0 ? zp_dev + 1 : nullptr,
                                             x_zp != 0 ? zp_dev : nullptr, epi, images > 1 ? d_dev : dst, filter_sums);
        if (rc != OVK_OK)
            return rc;
        if (images > 1) {
            const int64_t total = int64_t(images) * g.c_out * pixels;
            const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(total, 256), int64_t(ctx->sm_count) * 32));
            if ((pixels * int64_t(out_elem)) % 16 == 0 && aligned_to(dst, 16) && aligned_to(d_dev, 16)) {
                const int pieces = int(pixels * int64_t(out_elem) / 16);
                const unsigned vblocks = unsigned(std::min<int64_t>(ceil_div64(total * int64_t(out_elem) / 16, 256), int64_t(ctx->sm_count) * 32));
                unbatch_pieces_kernel<<<vblocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint4 *>(d_dev), reinterpret_cast<uint4 *>(dst),
                                                                       g.c_out, images, pieces);
            } else if (pixels * int64_t(out_elem) <= 1024) {
                const unsigned pblocks = unsigned(std::min<int64_t>(ceil_div64(int64_t(images) * g.c_out, 8), int64_t(ctx->sm_count) * 32));
                unbatch_planes_kernel<<<pblocks, 256, 0, ctx->stream>>>(d_dev, dst, g.c_out, images, int(pixels * int64_t(out_elem)));
            } else if (out_elem == 1)
                unbatch_kernel<uint8_t><<<blocks, 256, 0, ctx->stream>>>(d_dev, dst, g.c_out, images, int(pixels));
            else
                unbatch_kernel<uint32_t><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint32_t *>(d_dev),
                                                                        reinterpret_cast<uint32_t *>(dst), g.c_out, images, int(pixels));
            OVK_LAUNCHED(ctx, "conv_unbatch");
        }
    }
    return OVK_OK;
}

int32_t run_conv(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                 const ovk_conv_params *p, int32_t x_zp, int32_t w_zp, const EpiParams &epi,
                 void *out, const char *op, const ConvLayout &lay = ConvLayout())
{
    if (!ctx || !w || !p)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "%s: null argument", op);
    ConvGeom g;
    int32_t rc = make_geom(ctx, w, p, &g, op);
    if (rc != OVK_OK)
        return rc;
    const int64_t total = int64_t(g.n) * g.c_out * g.h_out * g.w_out;
    if (total == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, x && out, "%s: x or the output is null", op);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (gemm_route_applies(ctx, w, g, w_zp, lay, x))
        return run_gemm_route(ctx, w, x, x_signed, g, x_zp, w_zp, epi, out,
                              epi.mode == EPI_REQUANT ? sizeof(uint8_t) : sizeof(int32_t));
    if (ovk_qconv_tc_applies(ctx, w, g, x)) {
        const int32_t rc_tc = ovk_qconv_tc_launch(ctx, w, x, x_signed, g, x_zp, w_zp, epi, out, lay);
        if (rc_tc != OVK_UNSUPPORTED)  // an asymmetric weight or no room for the stages: the direct kernel runs
            return rc_tc;
    }
    // the direct kernel reads and writes the operator's layout only
    OVK_REFUSE(ctx, lay.x_cl || lay.y_cl,
               "%s: the channels-last layout is taken by the group-1, symmetric-weight tensor-core kernel (strides up to 4) only", op);
    if (g.group == g.c_in && g.c_out == g.c_in && g.kh * g.kw <= DW_MAX_TAPS && int64_t(g.n) * g.c_out < 65536) {
        conv_depthwise_kernel<<<dim3(unsigned(ceil_div64(int64_t(g.h_out) * g.w_out, 256)), unsigned(g.n * g.c_out)), 256, 0,
                                ctx->stream>>>(static_cast<const uint8_t *>(x), w->w, g, x_signed, w->w_signed, x_zp, w_zp, epi, out);
        OVK_LAUNCHED(ctx, "conv_depthwise");
        return OVK_OK;
    }
    conv_direct_kernel<<<unsigned(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(
        static_cast<const uint8_t *>(x), w->w, g, x_signed, w->w_signed, x_zp, w_zp, epi, out, total);
    OVK_LAUNCHED(ctx, "conv_direct");
    return OVK_OK;
}

}  // namespace

extern "C" {

int32_t ovk_qconv_prepack(ovk_ctx *ctx, const void *wt, int32_t w_signed, int64_t c_out,
                          int64_t c_in_per_group, int64_t kh, int64_t kw, int64_t group,
                          ovk_qconv_weight **out)
{
    if (!ctx || !out)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_qconv_prepack: null argument");
    *out = nullptr;
    OVK_REQUIRE(ctx, wt, "ConvInteger: weight is null");
    OVK_REQUIRE(ctx, c_out > 0 && c_in_per_group > 0 && kh > 0 && kw > 0 && group > 0,
                "ConvInteger: bad weight shape [%lld,%lld,%lld,%lld] group %lld", (long long)c_out,
                (long long)c_in_per_group, (long long)kh, (long long)kw, (long long)group);
    OVK_REQUIRE(ctx, c_out * c_in_per_group * kh * kw < (int64_t(1) << 31), "ConvInteger: weight too large");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    ovk_qconv_weight *w = new ovk_qconv_weight();
    w->c_out = c_out;
    w->cig = c_in_per_group;
    w->kh = kh;
    w->kw = kw;
    w->group = group;
    w->w_signed = w_signed ? 1 : 0;
    const size_t bytes = size_t(c_out * c_in_per_group * kh * kw);
    cudaError_t e = cudaMalloc(&w->w, (bytes + 255) & ~size_t(255));
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w->w, wt, bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    int32_t rc = OVK_OK;
    if (e != cudaSuccess)
        rc = ovk_fail(ctx, OVK_BACKEND, "ConvInteger: weight copy: %s", cudaGetErrorString(e));
    if (rc == OVK_OK)
        rc = ovk_qconv_tc_prepare_weight(ctx, w);
    if (rc != OVK_OK) {
        cudaFree(w->w);
        delete w;
        return rc;
    }
    *out = w;
    return OVK_OK;
}

void ovk_qconv_weight_destroy(ovk_ctx *ctx, ovk_qconv_weight *w)
{
    if (!w)
        return;
    if (ctx)
        cudaStreamSynchronize(ctx->stream);
    cudaFree(w->w);
    cudaFree(w->w_taps);
    cudaFree(w->wsum);
    cudaFree(w->w_rows16);
    cudaFree(w->ratio_dev);
    delete w;
}

int32_t ovk_conv_output_shape(const ovk_qconv_weight *w, const ovk_conv_params *p, int64_t *h_out,
                              int64_t *w_out)
{
    if (!w || !p || !h_out || !w_out)
        return OVK_INVALID_ARGUMENT;
    if (p->strides[0] <= 0 || p->strides[1] <= 0)
        return OVK_INVALID_ARGUMENT;
    *h_out = (p->h + p->pads[0] + p->pads[2] - (p->dilations[0] * (w->kh - 1) + 1)) / p->strides[0] + 1;
    *w_out = (p->w + p->pads[1] + p->pads[3] - (p->dilations[1] * (w->kw - 1) + 1)) / p->strides[1] + 1;
    return (*h_out > 0 && *w_out > 0) ? OVK_OK : OVK_INVALID_ARGUMENT;
}

int32_t ovk_conv_integer(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                         const ovk_conv_params *p, int32_t x_zp, int32_t w_zp, int32_t *out)
{
    EpiParams epi = {};
    epi.mode = EPI_RAW;
    return run_conv(ctx, w, x, x_signed, p, x_zp, w_zp, epi, out, "ConvInteger");
}

int32_t ovk_conv_integer_scale_bias(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x,
                                    int32_t x_signed, const ovk_conv_params *p, int32_t x_zp,
                                    int32_t w_zp, const float *scale, int32_t scale_step,
                                    const float *product, int32_t product_step, const float *bias,
                                    int32_t bias_step, uint32_t flags, uint32_t *range, float *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ConvIntegerScaleBias: null context");
    OVK_REQUIRE(ctx, scale && bias, "ConvIntegerScaleBias: scale or bias is null");
    OVK_REQUIRE(ctx, (scale_step | 1) == 1 && (bias_step | 1) == 1 && (product_step | 1) == 1,
                "ConvIntegerScaleBias: a step is 0 (per tensor) or 1 (per channel)");
    OVK_REQUIRE(ctx, !(flags & OVK_EPILOGUE_RANGE) || range, "ConvIntegerScaleBias: range requested without a slot");
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
    return run_conv(ctx, w, x, x_signed, p, x_zp, w_zp, epi, out, "ConvIntegerScaleBias");
}

static int32_t qlinear_conv_any(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                                const ovk_conv_params *p, int32_t x_zp, int32_t w_zp, const float *ratio_host,
                                const int32_t *bias, int32_t y_zp, int32_t y_signed, void *y, const ConvLayout &lay)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "QLinearConv: null argument");
    OVK_REQUIRE(ctx, ratio_host, "QLinearConv: ratio is null");
    // the per-channel ratio is a graph constant: uploaded when its content changes
    // (the reference keys its parameter cache by content, interp.rs:4751-4753)
    ovk_qconv_weight *wm = const_cast<ovk_qconv_weight *>(w);
    const size_t nratio = size_t(w->c_out);
    if (!wm->ratio_dev)
        OVK_CUDA(ctx, cudaMalloc(&wm->ratio_dev, nratio * sizeof(float)));
    if (wm->ratio_host.size() != nratio || memcmp(wm->ratio_host.data(), ratio_host, nratio * sizeof(float)) != 0) {
        wm->ratio_host.assign(ratio_host, ratio_host + nratio);
        // ordered after the kernels already enqueued, which may still read the old values
        OVK_CUDA(ctx, cudaMemcpyAsync(wm->ratio_dev, wm->ratio_host.data(), nratio * sizeof(float),
                                      cudaMemcpyHostToDevice, ctx->stream));
    }
    float *ratio_dev = wm->ratio_dev;
    EpiParams epi = {};
    epi.mode = EPI_REQUANT;
    epi.ratio = ratio_dev;
    epi.ratio_step = 1;
    epi.ibias = bias;
    epi.y_zp = y_zp;
    epi.y_signed = y_signed;
    return run_conv(ctx, w, x, x_signed, p, x_zp, w_zp, epi, y, "QLinearConv", lay);
}

int32_t ovk_qlinear_conv(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                         const ovk_conv_params *p, int32_t x_zp, int32_t w_zp,
                         const float *ratio_host, const int32_t *bias, int32_t y_zp,
                         int32_t y_signed, void *y)
{
    return qlinear_conv_any(ctx, w, x, x_signed, p, x_zp, w_zp, ratio_host, bias, y_zp, y_signed, y, ConvLayout());
}

int32_t ovk_qlinear_conv_layout(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed,
                                int32_t x_layout, const ovk_conv_params *p, int32_t x_zp, int32_t w_zp,
                                const float *ratio_host, const int32_t *bias, int32_t y_zp, int32_t y_signed,
                                void *y, int32_t y_layout, const int64_t *y_pads)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "QLinearConv: null argument");
    OVK_REQUIRE(ctx, (x_layout | 1) == 1 && (y_layout | 1) == 1, "QLinearConv: a layout is OVK_LAYOUT_NCHW or OVK_LAYOUT_PADDED_NHWC");
    ConvLayout lay;
    lay.x_cl = x_layout == OVK_LAYOUT_PADDED_NHWC;
    lay.y_cl = y_layout == OVK_LAYOUT_PADDED_NHWC;
    if (lay.y_cl) {
        OVK_REQUIRE(ctx, y_pads, "QLinearConv: a channels-last output needs its frame (y_pads)");
        for (int i = 0; i < 4; i++) {
            OVK_REQUIRE(ctx, y_pads[i] >= 0 && y_pads[i] < 65536, "QLinearConv: y_pads[%d] = %lld", i, (long long)y_pads[i]);
            lay.y_pads[i] = int(y_pads[i]);
        }
        OVK_REFUSE(ctx, w->c_out % 16 != 0, "QLinearConv: a channels-last output needs C_out = %lld to be a multiple of 16",
                   (long long)w->c_out);
        OVK_REQUIRE(ctx, aligned_to(y, 16), "QLinearConv: a channels-last output must be 16-byte aligned");
    }
    if (lay.x_cl)
        OVK_REQUIRE(ctx, aligned_to(x, 16), "QLinearConv: a channels-last input must be 16-byte aligned");
    return qlinear_conv_any(ctx, w, x, x_signed, p, x_zp, w_zp, ratio_host, bias, y_zp, y_signed, y, lay);
}

static int32_t layout_geom(ovk_ctx *ctx, const char *op, int64_t n, int64_t c, int64_t h, int64_t w, const int64_t *pads,
                           ConvGeom *g)
{
    OVK_REQUIRE(ctx, pads, "%s: pads is null", op);
    OVK_REQUIRE(ctx, n >= 0 && c > 0 && h > 0 && w > 0 && n < (1 << 24) && c < (1 << 16) && h < (1 << 20) && w < (1 << 20),
                "%s: bad shape [%lld,%lld,%lld,%lld]", op, (long long)n, (long long)c, (long long)h, (long long)w);
    for (int i = 0; i < 4; i++)
        OVK_REQUIRE(ctx, pads[i] >= 0 && pads[i] < 65536, "%s: pads[%d] = %lld", op, i, (long long)pads[i]);
    OVK_REFUSE(ctx, c % 4 != 0, "%s: %lld channels (a multiple of 4)", op, (long long)c);
    *g = ConvGeom{};
    g->n = int(n);
    g->c_in = int(c);
    g->h_in = int(h);
    g->w_in = int(w);
    g->phb = int(pads[0]);
    g->pwb = int(pads[1]);
    g->phe = int(pads[2]);
    g->pwe = int(pads[3]);
    return OVK_OK;
}

int32_t ovk_nchw_to_padded_nhwc(ovk_ctx *ctx, const void *x, int64_t n, int64_t c, int64_t h, int64_t w,
                                const int64_t *pads, int32_t fill, void *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_nchw_to_padded_nhwc: null context");
    ConvGeom g;
    int32_t rc = layout_geom(ctx, "ovk_nchw_to_padded_nhwc", n, c, h, w, pads, &g);
    if (rc != OVK_OK || n == 0)
        return rc;
    OVK_REQUIRE(ctx, x && out && aligned_to(out, 16), "ovk_nchw_to_padded_nhwc: x or out is null, or out is not 16-byte aligned");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    return ovk_qconv_pad_nhwc(ctx, x, g, fill, static_cast<uint8_t *>(out));
}

int32_t ovk_padded_nhwc_to_nchw(ovk_ctx *ctx, const void *x, int64_t n, int64_t c, int64_t h, int64_t w,
                                const int64_t *pads, void *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_padded_nhwc_to_nchw: null context");
    ConvGeom g;
    int32_t rc = layout_geom(ctx, "ovk_padded_nhwc_to_nchw", n, c, h, w, pads, &g);
    if (rc != OVK_OK || n == 0)
        return rc;
    OVK_REQUIRE(ctx, x && out, "ovk_padded_nhwc_to_nchw: x or out is null");
    const size_t sm = size_t(w) * (c + 1);
    OVK_REFUSE(ctx, sm > 48 * 1024, "ovk_padded_nhwc_to_nchw: rows of %lld pixels x %lld channels are too large", (long long)w,
               (long long)c);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    unpad_nchw_kernel<<<dim3(unsigned(h), unsigned(n)), 256, sm, ctx->stream>>>(
        static_cast<const uint8_t *>(x), static_cast<uint8_t *>(out), int(c), int(h), int(w), int(h + pads[0] + pads[2]),
        int(w + pads[1] + pads[3]), int(pads[0]), int(pads[1]));
    OVK_LAUNCHED(ctx, "unpad_nchw");
    return OVK_OK;
}

int32_t ovk_requantize(ovk_ctx *ctx, const int32_t *acc, int64_t count, int64_t inner,
                       int64_t axis_len, const int32_t *bias, const float *ratio, int32_t y_zp,
                       int32_t y_signed, void *out)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "Requantize: null context");
    OVK_REQUIRE(ctx, count >= 0 && axis_len > 0, "Requantize: empty scale");
    if (count == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, acc && ratio && out, "Requantize: null tensor");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    EpiParams epi = {};
    epi.mode = EPI_REQUANT;
    epi.ratio = ratio;
    epi.ratio_step = 1;
    epi.ibias = bias;
    epi.y_zp = y_zp;
    epi.y_signed = y_signed;
    requantize_kernel<<<unsigned(ceil_div64(ceil_div64(count, 4), 256)), 256, 0, ctx->stream>>>(
        acc, count, std::max<int64_t>(inner, 1), axis_len, epi, static_cast<uint8_t *>(out));
    OVK_LAUNCHED(ctx, "requantize");
    return OVK_OK;
}

}  // extern "C"
