// ConvInteger / QLinearConv on tcgen05 kind::i8: a stride-1, group-1
// convolution as a sum of SHIFTED GEMMs over a padded channels-last image.
//
// The reference takes this shape (batch > 1) through its blocked implicit-GEMM
// ladder with split-K and a separate REQUANTIZE pass
// (crates/onnx-vulkan-core/src/shaders/conv_integer.rs:188-344,
// src/interp.rs:4577-4585, src/shaders/qlinear.rs:28-63), and for batch 1
// through to_hwc + im2col + the cooperative-matrix GEMM
// (conv_integer.rs:374-527).  Here:
//
//  1. one pass rewrites NCHW x as Xp[n][h + pad][w + pad][c] with the PADDING
//     SET TO x_zero_point, so a padded tap contributes (zp - zp) * w = 0 and the
//     zero-point term is the same -zp * sum(w[co]) for every pixel;
//  2. with v = (n*HP + h)*WP + w numbering the pixels of the padded grid, tap
//     (kh, kw) of output v is row v + kh*dh*WP + kw*dw of Xp: the A operand of a
//     tap is a plain 2-D tile [128 pixels x C_in bytes] at a row offset, which
//     TMA loads directly (K-major, swizzled).  Outputs that fall on padding
//     columns/rows (7% for 56x56 + 1) are computed and dropped;
//  3. the filter bank (tap-major, K contiguous) stays resident in shared
//     memory; one thread issues the MMAs of all taps into a tensor-memory
//     accumulator (two of them, so the epilogue of one tile overlaps the MMAs
//     of the next);
//  4. four epilogue warps read the accumulator (one pixel per thread), apply
//     -zp * wsum, and either store int32 or requantise in the same pass, NCHW.
#include "ovk_internal.h"
#include "epilogue.cuh"
#include "umma.cuh"

#include <cstdlib>

namespace {

constexpr int BM = 128;  // pixels per tile
constexpr int THREADS = 192;
constexpr long long WAIT_CYCLES = 2000000000ll;
constexpr size_t W_SMEM_MAX = 112 * 1024;

struct ConvTcParams {
    int64_t v_total;   // N * HP * WP
    int hpwp, wp;      // padded plane and row
    int h_out, w_out, c_out, co_pad;
    int taps, kw, dh, dw;
    int kch;           // bytes of K per slice (min(C_in, 128))
    int chunks;        // C_in / kch
    int sw_layout;     // UMMA layout code of the swizzle
    int sbo;           // 8 * kch
    int halo;          // 1: one halo tile per pixel tile, taps addressed by descriptor offset
    int halo_rows;     // rows of a halo tile
    uint32_t a_stage, w_slice;  // bytes
    int stages;
    int x_signed, w_signed;
    int32_t x_zp;
    const int32_t *wsum;
    EpiParams epi;
    void *out;
    int *status;
    int m_tiles;
};

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity)
{
    if (umma::mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (uint32_t spins = 0;; spins++) {
        if (umma::mbar_try_wait(bar, parity))
            return true;
        if ((spins & 63u) == 63u && clock64() - t0 > WAIT_CYCLES)
            return false;
    }
}

constexpr int MAX_STAGES = 8;

__global__ void __launch_bounds__(THREADS, 1)
qconv_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvTcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int slices = p.taps * p.chunks;
    uint8_t *sWt = smem;                                   // slices x w_slice: resident filters
    uint8_t *sA = smem + size_t(slices) * p.w_slice;       // stages x a_stage: pixel tiles
    uint64_t *bars = reinterpret_cast<uint64_t *>(sA + size_t(p.stages) * p.a_stage);
    uint64_t *a_full = bars, *a_empty = bars + MAX_STAGES;
    uint64_t *acc_full = a_empty + MAX_STAGES, *acc_empty = acc_full + 2;
    uint64_t *w_full = acc_empty + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(w_full + 1);
    // per-channel constants of the epilogue, staged once: bias - zp * sum(w) and the requantisation ratio
    int32_t *s_corr = reinterpret_cast<int32_t *>(tmem_slot + 2);
    float *s_ratio = reinterpret_cast<float *>(s_corr + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int co = threadIdx.x; co < p.co_pad; co += THREADS) {
        int32_t corr = 0;
        float ratio = 0.0f;
        if (co < p.c_out) {
            corr = int32_t(0u - uint32_t(p.x_zp) * uint32_t(p.wsum[co]));
            if (p.epi.mode == EPI_REQUANT) {
                if (p.epi.ibias)
                    corr = int32_t(uint32_t(corr) + uint32_t(p.epi.ibias[co]));
                ratio = p.epi.ratio[co * p.epi.ratio_step];
            }
        }
        s_corr[co] = corr;
        s_ratio[co] = ratio;
    }
    uint32_t tmem_cols = 32;
    while (tmem_cols < uint32_t(2 * p.co_pad))
        tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            umma::mbar_init(&a_full[s], 1);
            umma::mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], 4);
        }
        umma::mbar_init(w_full, 1);
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, tmem_cols);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            umma::prefetch_tmap(&tmX);
            umma::prefetch_tmap(&tmW);
            // the whole filter bank, once
            umma::mbar_expect_tx(w_full, uint32_t(slices) * uint32_t(p.co_pad) * uint32_t(p.kch));
            for (int sl = 0; sl < slices; sl++) {
                const int tap = sl / p.chunks, ch = sl % p.chunks;
                umma::tma_load_2d(sWt + size_t(sl) * p.w_slice, &tmW, w_full, ch * p.kch, tap * p.co_pad);
            }
            int seq = 0;
            for (int tile = blockIdx.x; tile < p.m_tiles; tile += gridDim.x) {
                const int64_t v0 = int64_t(tile) * BM;
                const int loads = p.halo ? 1 : slices;
                for (int sl = 0; sl < loads; sl++, seq++) {
                    const int s = seq % p.stages;
                    if (!wait_bounded(&a_empty[s], ((seq / p.stages) & 1) ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = p.m_tiles;
                        break;
                    }
                    if (p.halo) {
                        umma::mbar_expect_tx(&a_full[s], uint32_t(p.halo_rows) * uint32_t(p.kch));
                        umma::tma_load_2d(sA + size_t(s) * p.a_stage, &tmX, &a_full[s], 0, int(v0));
                    } else {
                        const int tap = sl / p.chunks, ch = sl % p.chunks;
                        const int off = (tap / p.kw) * p.dh * p.wp + (tap % p.kw) * p.dw;
                        umma::mbar_expect_tx(&a_full[s], uint32_t(BM) * uint32_t(p.kch));
                        umma::tma_load_2d(sA + size_t(s) * p.a_stage, &tmX, &a_full[s], ch * p.kch, int(v0 + off));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma::instr_desc(2, p.x_signed ? 1 : 0, p.w_signed ? 1 : 0, BM, uint32_t(p.co_pad));
            bool ok = wait_bounded(w_full, 0);
            if (!ok)
                atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
            int seq = 0, tile_seq = 0;
            const int ksteps = p.kch / 32;
            for (int tile = blockIdx.x; tile < p.m_tiles && ok; tile += gridDim.x, tile_seq++) {
                const int b = tile_seq & 1;
                if (!wait_bounded(&acc_empty[b], ((tile_seq >> 1) & 1) ^ 1)) {
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                umma::tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(b * p.co_pad);
                if (p.halo) {
                    const int s = seq % p.stages;
                    if (!wait_bounded(&a_full[s], (seq / p.stages) & 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    umma::tc_fence_after();
                    const uint32_t a_base = umma::smem_u32(sA + size_t(s) * p.a_stage);
                    for (int tap = 0; tap < p.taps; tap++) {
                        const int off = (tap / p.kw) * p.dh * p.wp + (tap % p.kw) * p.dw;
                        const uint32_t a_addr = a_base + uint32_t(off) * uint32_t(p.kch);
                        const uint32_t w_addr = umma::smem_u32(sWt + size_t(tap) * p.w_slice);
                        for (int j = 0; j < ksteps; j++) {
                            // The tap's rows start `off` rows into the halo tile.  The swizzle is a function of
                            // the absolute shared-memory address (TMA wrote the tile with the same function),
                            // so the descriptor needs no base offset: measured bit-exact with 0, wrong otherwise.
                            const uint64_t da = umma::smem_desc(a_addr + j * 32, p.sbo, p.sw_layout);
                            const uint64_t dw = umma::smem_desc(w_addr + j * 32, p.sbo, p.sw_layout);
                            umma::mma_i8(d_tmem, da, dw, idesc, (tap | j) != 0);
                        }
                    }
                    umma::mma_commit(&a_empty[s]);
                    seq++;
                } else {
                    for (int sl = 0; sl < slices && ok; sl++, seq++) {
                        const int s = seq % p.stages;
                        if (!wait_bounded(&a_full[s], (seq / p.stages) & 1)) {
                            atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                            ok = false;
                            break;
                        }
                        umma::tc_fence_after();
                        const uint32_t a_addr = umma::smem_u32(sA + size_t(s) * p.a_stage);
                        const uint32_t w_addr = umma::smem_u32(sWt + size_t(sl) * p.w_slice);
                        for (int j = 0; j < ksteps; j++) {
                            const uint64_t da = umma::smem_desc(a_addr + j * 32, p.sbo, p.sw_layout);
                            const uint64_t dw = umma::smem_desc(w_addr + j * 32, p.sbo, p.sw_layout);
                            umma::mma_i8(d_tmem, da, dw, idesc, (sl | j) != 0);
                        }
                        umma::mma_commit(&a_empty[s]);
                    }
                }
                if (ok)
                    umma::mma_commit(&acc_full[b]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        int tile_seq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.m_tiles; tile += gridDim.x, tile_seq++) {
            const int b = tile_seq & 1;
            if (ok && !wait_bounded(&acc_full[b], (tile_seq >> 1) & 1)) {
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                ok = false;
            }
            umma::tc_fence_after();
            const int64_t v = int64_t(tile) * BM + q * 32 + lane;
            const int64_t img = v / p.hpwp;
            const int rem = int(v % p.hpwp);
            const int oh = rem / p.wp, ow = rem % p.wp;
            const bool valid = ok && v < p.v_total && oh < p.h_out && ow < p.w_out;
            const int64_t plane = int64_t(p.h_out) * p.w_out;
            const int64_t o_base = img * p.c_out * plane + int64_t(oh) * p.w_out + ow;
            for (int c0 = 0; c0 < p.co_pad; c0 += 32) {
                uint32_t r[32];
                umma::tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * p.co_pad + c0), r);
                umma::tmem_ld_wait();
                if (c0 + 32 >= p.co_pad) {  // last read of this accumulator: hand it back
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        umma::mbar_arrive(&acc_empty[b]);
                }
                if (!valid)
                    continue;
                if (p.epi.mode == EPI_RAW) {
                    int32_t *o = static_cast<int32_t *>(p.out) + o_base + int64_t(c0) * plane;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < p.c_out)
                            o[j * plane] = int32_t(r[j] + uint32_t(s_corr[c0 + j]));
                } else {
                    uint8_t *o = static_cast<uint8_t *>(p.out) + o_base + int64_t(c0) * plane;
                    const int lo = p.epi.y_signed ? -128 : 0, hi = p.epi.y_signed ? 127 : 255;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (c0 + j < p.c_out) {
                            // sat(rne(f32(acc + bias) * ratio) + y_zp), shaders/qlinear.rs:28-63
                            const int32_t acc = int32_t(r[j] + uint32_t(s_corr[c0 + j]));
                            const float f = rintf(__fmul_rn(float(acc), s_ratio[c0 + j]));
                            const int32_t qv = int32_t(uint32_t(__float2int_rn(f)) + uint32_t(p.epi.y_zp));
                            o[j * plane] = uint8_t(max(lo, min(hi, qv)));
                        }
                    }
                }
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, tmem_cols);
}

// NCHW -> padded NHWC with the padding set to the zero point.  One block per
// padded image row; channels go through shared memory in groups so that reads
// run along W and writes along C.
__global__ void __launch_bounds__(256)
conv_pad_nhwc_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ xp, int C, int H, int W, int HP, int WP,
                     int pt, int pl, uint32_t zp_byte, int cgroup)
{
    extern __shared__ uint8_t tile[];  // [W][cgroup + 4]
    const int hp = blockIdx.x, n = blockIdx.y;
    uint8_t *dst_row = xp + (size_t(n) * HP + hp) * size_t(WP) * C;
    const int h = hp - pt;
    if (h < 0 || h >= H) {
        const uint32_t w4 = zp_byte * 0x01010101u;
        for (int i = threadIdx.x; i < WP * C / 4; i += blockDim.x)
            reinterpret_cast<uint32_t *>(dst_row)[i] = w4;
        return;
    }
    const int pitch = cgroup + 4;
    for (int c0 = 0; c0 < C; c0 += cgroup) {
        const int cg = min(cgroup, C - c0);
        for (int i = threadIdx.x; i < cg * W; i += blockDim.x) {
            const int c = i / W, w = i % W;
            tile[w * pitch + c] = x[((size_t(n) * C + c0 + c) * H + h) * W + w];
        }
        __syncthreads();
        // cg is a multiple of 4: write words
        const int words = cg / 4;
        for (int i = threadIdx.x; i < WP * words; i += blockDim.x) {
            const int wpix = i / words, cw = i % words;
            const int w = wpix - pl;
            uint32_t v = zp_byte * 0x01010101u;
            if (w >= 0 && w < W) {
                const uint8_t *t = tile + w * pitch + cw * 4;
                v = uint32_t(t[0]) | (uint32_t(t[1]) << 8) | (uint32_t(t[2]) << 16) | (uint32_t(t[3]) << 24);
            }
            reinterpret_cast<uint32_t *>(dst_row + size_t(wpix) * C + c0)[cw] = v;
        }
        __syncthreads();
    }
}

// [C_out, C_in, KH, KW] -> [tap][co_pad][C_in] (zero padded rows) and wsum[co]
__global__ void __launch_bounds__(256)
conv_pack_w_kernel(const uint8_t *__restrict__ w, uint8_t *__restrict__ wt, int32_t *__restrict__ wsum, int c_out,
                   int co_pad, int c_in, int taps, int w_signed)
{
    const int co = blockIdx.x;
    int32_t local = 0;
    for (int i = threadIdx.x; i < taps * c_in; i += blockDim.x) {
        const int tap = i / c_in, c = i % c_in;
        uint8_t v = 0;
        if (co < c_out) {
            v = w[(size_t(co) * c_in + c) * taps + tap];
            local += w_signed ? int32_t(int8_t(v)) : int32_t(v);
        }
        wt[(size_t(tap) * co_pad + co) * c_in + c] = v;
    }
    __shared__ int32_t red[256];
    red[threadIdx.x] = local;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (int(threadIdx.x) < s)
            red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        wsum[co] = red[0];
}

int conv_mode()
{
    // OVK_CONV_TAPS=1 selects one TMA load per tap instead of one halo tile per pixel tile
    static int mode = -1;
    if (mode < 0) {
        const char *e = getenv("OVK_CONV_TAPS");
        mode = (e && e[0] == '1') ? 0 : 1;
    }
    return mode;
}

}  // namespace

int32_t ovk_qconv_tc_prepare_weight(ovk_ctx *ctx, ovk_qconv_weight *w)
{
    const int64_t c_in = w->cig, taps = w->kh * w->kw;
    if (w->group != 1 || (c_in != 32 && c_in != 64 && c_in % 128 != 0) || w->c_out > 256)
        return OVK_OK;  // the direct kernel takes these
    const int64_t co_pad = ceil_div64(w->c_out, 32) * 32;
    if (size_t(taps) * co_pad * c_in > W_SMEM_MAX)
        return OVK_OK;
    OVK_CUDA(ctx, cudaMalloc(&w->w_taps, size_t(taps) * co_pad * c_in));
    OVK_CUDA(ctx, cudaMalloc(&w->wsum, size_t(co_pad) * sizeof(int32_t)));
    conv_pack_w_kernel<<<unsigned(co_pad), 256, 0, ctx->stream>>>(w->w, w->w_taps, w->wsum, int(w->c_out), int(co_pad),
                                                                  int(c_in), int(taps), w->w_signed);
    w->c_out_pad = co_pad;
    OVK_LAUNCHED(ctx, "conv_pack_w");
    return OVK_OK;
}

// Stride 1, group 1, a filter bank that fits in shared memory, symmetric
// weights (w_zp = 0 is checked at launch); everything else takes the direct kernel.
bool ovk_qconv_tc_applies(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, const void *x)
{
    (void)ctx;
    (void)x;
    if (!w->w_taps || g.sh != 1 || g.sw != 1 || g.group != 1)
        return false;
    const int64_t hp = int64_t(g.h_in) + g.phb + g.phe, wp = int64_t(g.w_in) + g.pwb + g.pwe;
    const int64_t v_total = int64_t(g.n) * hp * wp;
    return v_total >= 4 * BM && v_total < (int64_t(1) << 31) - 65536 && (wp * g.c_in) % 4 == 0;
}

int32_t ovk_qconv_tc_launch(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed, const ConvGeom &g,
                            int32_t x_zp, int32_t w_zp, const EpiParams &epi, void *out)
{
    if (w_zp != 0)
        return OVK_UNSUPPORTED;  // caller falls back to the direct kernel
    const int C = g.c_in;
    const int HP = g.h_in + g.phb + g.phe, WP = g.w_in + g.pwb + g.pwe;
    const int64_t v_total = int64_t(g.n) * HP * WP;
    const size_t xp_bytes = size_t(v_total) * C;
    void *ws = nullptr;
    int32_t rc = ovk_scratch(ctx, xp_bytes + 1024, &ws);
    if (rc != OVK_OK)
        return rc;
    uint8_t *xp = static_cast<uint8_t *>(ws);
    {
        int cgroup = C;
        while (size_t(g.w_in) * (cgroup + 4) > 40 * 1024 && cgroup > 4)
            cgroup = ((cgroup / 2) + 3) & ~3;
        const size_t sm = size_t(g.w_in) * (cgroup + 4);
        OVK_REQUIRE(ctx, sm <= 48 * 1024, "ConvInteger: input rows of %d pixels are too wide for the layout pass", g.w_in);
        conv_pad_nhwc_kernel<<<dim3(unsigned(HP), unsigned(g.n)), 256, sm, ctx->stream>>>(
            static_cast<const uint8_t *>(x), xp, C, g.h_in, g.w_in, HP, WP, g.phb, g.pwb, uint32_t(x_zp) & 0xffu, cgroup);
        OVK_LAUNCHED(ctx, "conv_pad_nhwc");
    }
    ConvTcParams p = {};
    p.v_total = v_total;
    p.hpwp = HP * WP;
    p.wp = WP;
    p.h_out = g.h_out;
    p.w_out = g.w_out;
    p.c_out = g.c_out;
    p.co_pad = int(w->c_out_pad);
    p.taps = g.kh * g.kw;
    p.kw = g.kw;
    p.dh = g.dh;
    p.dw = g.dw;
    p.kch = std::min(C, 128);
    p.chunks = C / p.kch;
    p.sw_layout = p.kch == 128 ? umma::LAYOUT_SW128 : (p.kch == 64 ? umma::LAYOUT_SW64 : umma::LAYOUT_SW32);
    p.sbo = 8 * p.kch;
    const int max_off = (g.kh - 1) * g.dh * WP + (g.kw - 1) * g.dw;
    p.halo = conv_mode() == 1 && p.chunks == 1 && BM + max_off <= 256;
    p.halo_rows = p.halo ? BM + max_off : BM;
    p.a_stage = uint32_t((size_t(p.halo_rows) * p.kch + 1023) & ~size_t(1023));
    p.w_slice = uint32_t((size_t(p.co_pad) * p.kch + 1023) & ~size_t(1023));
    const size_t w_bytes = size_t(p.taps) * p.chunks * p.w_slice;
    const size_t avail = ctx->smem_optin - w_bytes - 1024 - 2048;
    p.stages = int(std::min<size_t>(MAX_STAGES, avail / p.a_stage));
    if (p.stages < 2)
        return OVK_UNSUPPORTED;
    p.x_signed = x_signed ? 1 : 0;
    p.w_signed = w->w_signed;
    p.x_zp = x_zp;
    p.wsum = w->wsum;
    p.epi = epi;
    p.out = out;
    p.status = ctx->dev_status;
    p.m_tiles = int(ceil_div64(v_total, BM));
    const CUtensorMapSwizzle swz = p.kch == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                : (p.kch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUtensorMap tmX, tmW;
    if (!ovk_make_tmap_2d(&tmX, xp, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(C), uint64_t(v_total), uint64_t(C),
                          uint32_t(p.kch), uint32_t(p.halo_rows), swz) ||
        !ovk_make_tmap_2d(&tmW, w->w_taps, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(C), uint64_t(p.taps) * p.co_pad,
                          uint64_t(C), uint32_t(p.kch), uint32_t(p.co_pad), swz))
        return ovk_fail(ctx, OVK_BACKEND, "ConvInteger: cuTensorMapEncodeTiled failed");
    const size_t smem = w_bytes + size_t(p.stages) * p.a_stage + 512 + 2048;
    OVK_CUDA(ctx, cudaFuncSetAttribute(qconv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const unsigned grid = unsigned(std::min<int>(p.m_tiles, ctx->sm_count));
    qconv_tc_kernel<<<grid, THREADS, smem, ctx->stream>>>(tmX, tmW, p);
    OVK_LAUNCHED(ctx, p.halo ? "qconv_tc_halo" : "qconv_tc_taps");
    return OVK_OK;
}
