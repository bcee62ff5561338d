// ConvInteger / QLinearConv on tcgen05 kind::i8: a group-1 convolution as a sum
// of SHIFTED GEMMs over a padded channels-last image.  Strides (up to 4) are taken
// by forming the products at every position and storing those on the stride
// lattice; a filter bank too large for shared memory by several launches of as
// many filters as fit.
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


namespace {

constexpr int BM = 128;  // pixels per tile
constexpr int EPI_WARPS = 16;            // four per tensor-memory lane quarter
constexpr int MMA_WARPS = 2;              // two issuing threads on different schedulers take alternate tiles
constexpr int THREADS = (2 + EPI_WARPS + (MMA_WARPS - 1)) * 32;  // TMA, issuer 0, epilogue warps, issuer 1
constexpr long long WAIT_CYCLES = 2000000000ll;
constexpr size_t W_SMEM_MAX = 112 * 1024;

struct ConvTcParams {
    int64_t v_total;   // N * HP * WP
    int hpwp, wp;      // padded plane and row
    int h_out, w_out, c_out, co_pad;  // c_out / co_pad: the filters of THIS launch (a bank too large for shared
                                      // memory is taken in several launches of as many filters as fit)
    int c_out_total;                  // channels of the output tensor
    int slice_filters;                // > 0: blockIdx.y numbers equal slices of that many filters, all in one launch
    int sh, sw;                       // strides: the products are computed at every position of the padded grid and
                                      // only the positions on the stride lattice are stored (2 x 2: a quarter)
    int w_tap_rows;                   // rows between two taps in the packed filter bank (all filters, padded)
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
    int nacc;
    int issuers;  // 1 or 2 MMA-issuing threads
    uint64_t magic_hpwp, magic_wp;  // ceil(2^64 / divisor), 0 for a divisor of 1
    // requantised bytes stored channels-last into a padded image [n][h_out + frame][w_out + frame][c_out]
    // (the input layout of the next convolution) instead of NCHW
    int out_cl;
    int y_wp;               // padded row of the output image, in pixels
    int64_t y_hpwp;         // padded plane of the output image, in pixels
    int y_pt, y_pl;         // frame above and to the left
};

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity)
{
    if (umma::mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (;;) {
        if (umma::mbar_try_wait_hint(bar, parity, 1000u))  // parked for up to a microsecond, not spinning
            return true;
        __nanosleep(64);  // and out of the issue slots of the thread that feeds the tensor core
        if (clock64() - t0 > WAIT_CYCLES)
            return false;
    }
}

constexpr int MAX_STAGES = 8;
constexpr int MAX_ACC = 8;  // tensor-memory accumulators in flight (512 columns / co_pad, at most 8)

__global__ void __launch_bounds__(THREADS, 1)
qconv_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvTcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int slices = p.taps * p.chunks;
    uint8_t *sWt = smem;                                   // slices x w_slice: resident filters
    uint8_t *sA = smem + size_t(slices) * p.w_slice;       // stages x a_stage: pixel tiles
    uint64_t *bars = reinterpret_cast<uint64_t *>(sA + size_t(p.stages) * p.a_stage);
    uint64_t *a_full = bars, *a_empty = bars + MAX_STAGES;
    uint64_t *acc_full = a_empty + MAX_STAGES, *acc_empty = acc_full + MAX_ACC;
    uint64_t *w_full = acc_empty + MAX_ACC;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(w_full + 1);
    // per-channel constants of the epilogue, staged once: bias - zp * sum(w) and the requantisation ratio
    int32_t *s_corr = reinterpret_cast<int32_t *>(tmem_slot + 2);
    float *s_ratio = reinterpret_cast<float *>(s_corr + 256);
    // per tap: offset of its first pixel row inside a halo tile and start of its filter slice, both in
    // 16-byte units (the unit of a descriptor's address field)
    uint32_t *s_tap_a = reinterpret_cast<uint32_t *>(s_ratio + 256);
    uint32_t *s_tap_w = s_tap_a + 64;
    float *s_fbias = reinterpret_cast<float *>(s_tap_w + 64);  // present only for the scale-and-bias store

    // The next kernel of the stream, if it was launched as a programmatic dependent (the next layer of a
    // channels-last chain is), may be scheduled as SMs fall free: its launch latency and its prologue -
    // barriers, tensor memory, its filter bank - then overlap this kernel's tail.  It reads what this
    // kernel writes only behind its own griddepcontrol.wait, which returns when this grid has finished.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // A bank cut into equal slices is one launch, a row of the grid per slice: the slices' CTAs fill the SMs
    // together (98 pixel tiles x 4 slices: 2.7 rounds of the GPU instead of 4 launches of 98 CTAs each).
    const int co0 = p.slice_filters > 0 ? int(blockIdx.y) * p.slice_filters : 0;
    for (int tap = threadIdx.x; tap < p.taps && tap < 64; tap += THREADS) {
        const int off = (tap / p.kw) * p.dh * p.wp + (tap % p.kw) * p.dw;
        s_tap_a[tap] = uint32_t(off) * uint32_t(p.kch) >> 4;
        s_tap_w[tap] = (umma::smem_u32(sWt) + uint32_t(tap) * p.w_slice) >> 4;
    }
    for (int co = threadIdx.x; co < p.co_pad; co += THREADS) {
        int32_t corr = 0;
        float ratio = 0.0f;
        if (co < p.c_out) {
            const int ch = co0 + co;  // the filter's number in the whole bank
            corr = int32_t(0u - uint32_t(p.x_zp) * uint32_t(p.wsum[ch]));
            if (p.epi.mode == EPI_REQUANT) {
                if (p.epi.ibias)
                    corr = int32_t(uint32_t(corr) + uint32_t(p.epi.ibias[ch]));
                ratio = p.epi.ratio[ch * p.epi.ratio_step];
            } else if (p.epi.mode == EPI_SCALE) {
                // s = scale or fl(scale * product), as epi_scale_value computes it per element
                ratio = p.epi.scale[ch * p.epi.scale_step];
                if (p.epi.product)
                    ratio = __fmul_rn(ratio, p.epi.product[ch * p.epi.product_step]);
            }
        }
        s_corr[co] = corr;
        s_ratio[co] = ratio;
        if (p.epi.mode == EPI_SCALE)
            s_fbias[co] = co < p.c_out ? p.epi.fbias[(co0 + co) * p.epi.bias_step] : 0.0f;
    }
    const int nacc = p.nacc;  // power of two
    uint32_t tmem_cols = 32;
    while (tmem_cols < uint32_t(nacc * p.co_pad))
        tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            umma::mbar_init(&a_full[s], 1);
            umma::mbar_init(&a_empty[s], 1);
        }
        for (int b = 0; b < nacc; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], EPI_WARPS / min(EPI_WARPS / 4, nacc));  // the warps of one tile group
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
                umma::tma_load_2d(sWt + size_t(sl) * p.w_slice, &tmW, w_full, ch * p.kch, tap * p.w_tap_rows + co0);
            }
            // launched with programmatic stream serialization: everything above ran while the layout
            // pass was still draining; its output is read from here on
            asm volatile("griddepcontrol.wait;" ::: "memory");
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
    } else if (warp == 1 || warp == 2 + EPI_WARPS) {
        // The issue of a tcgen05.mma blocks until the tensor core takes it, and between two of them this
        // thread competes with the epilogue warps of its scheduler for issue slots.  Two issuers on two
        // schedulers, each with its own tiles (and accumulators), keep the tensor core fed.
        if (lane == 0) {
            const int me = warp == 1 ? 0 : 1;
            const int issuers = p.issuers;
            const uint32_t idesc = umma::instr_desc(2, p.x_signed ? 1 : 0, p.w_signed ? 1 : 0, BM, uint32_t(p.co_pad));
            bool ok = wait_bounded(w_full, 0);
            if (!ok)
                atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
            const int loads_per_tile = p.halo ? 1 : slices;
            const int ksteps = p.kch / 32;
            // descriptor halves that never change: LBO = 1 (unused by swizzled K-major), version 1,
            // stride between 8-row groups, swizzle mode
            const uint32_t desc_lo_flags = 1u << 16;
            const uint32_t desc_hi = ((uint32_t(p.sbo) >> 4) & 0x3fffu) | (1u << 14) | (uint32_t(p.sw_layout) << 29);
            const uint32_t a_unit = uint32_t(p.kch) >> 4;  // 16-byte units per pixel row
            const uint32_t a_step_w = uint32_t(p.dw) * a_unit, a_step_h = uint32_t(p.dh * p.wp) * a_unit;
            const uint32_t w16 = umma::smem_u32(sWt) >> 4, w_step = p.w_slice >> 4;
            const int khn = p.taps / p.kw;
            int tile_seq = me;
            for (int tile = me < issuers ? int(blockIdx.x) + me * int(gridDim.x) : p.m_tiles; tile < p.m_tiles && ok;
                 tile += issuers * int(gridDim.x), tile_seq += issuers) {
                int seq = tile_seq * loads_per_tile;  // position of the tile's first load in the stage ring
                const int b = tile_seq & (nacc - 1);
                if (!wait_bounded(&acc_empty[b], ((tile_seq / nacc) & 1) ^ 1)) {
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
                    // The tap's rows start some rows into the halo tile.  The swizzle is a function of the
                    // absolute shared-memory address (TMA wrote the tile with the same function), so the
                    // descriptor needs no base offset: measured bit-exact with 0, wrong otherwise.
                    const uint32_t a16 = umma::smem_u32(sA + size_t(s) * p.a_stage) >> 4;
                    // tap (kh, kw) starts (kh*dh*WP + kw*dw) pixel rows into the halo tile and one filter
                    // slice further.  The issuing thread shares its scheduler with waiting warps, so the
                    // loop is kept to an add or two per MMA: shared-memory addresses are below 2^18, so
                    // (address >> 4) + offset never carries into the descriptor's flag bits, and the
                    // common 3x3 filter over 64 channels is unrolled completely.
                    const uint32_t a0 = a16 | desc_lo_flags, w0 = w16 | desc_lo_flags;
                    if (khn == 3 && p.kw == 3 && ksteps == 2) {
#pragma unroll
                        for (int kh = 0; kh < 3; kh++) {
#pragma unroll
                            for (int kw = 0; kw < 3; kw++) {
                                const uint32_t a_lo = a0 + uint32_t(kh) * a_step_h + uint32_t(kw) * a_step_w;
                                const uint32_t w_lo = w0 + uint32_t(kh * 3 + kw) * w_step;
                                umma::mma_i8_lohi(d_tmem, a_lo, desc_hi, w_lo, desc_hi, idesc, (kh | kw) ? 1u : 0u);
                                umma::mma_i8_lohi(d_tmem, a_lo + 2u, desc_hi, w_lo + 2u, desc_hi, idesc, 1u);
                            }
                        }
                    } else {
                        uint32_t accumulate = 0;
                        uint32_t a_h = a0, w_cur = w0;
                        for (int kh = 0; kh < khn; kh++, a_h += a_step_h) {
                            uint32_t a_t = a_h;
                            for (int kw = 0; kw < p.kw; kw++, a_t += a_step_w, w_cur += w_step) {
                                for (int j = 0; j < ksteps; j++) {
                                    umma::mma_i8_lohi(d_tmem, a_t + 2u * j, desc_hi, w_cur + 2u * j, desc_hi, idesc, accumulate);
                                    accumulate = 1;
                                }
                            }
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
    } else if (warp < 2 + EPI_WARPS) {
        // ---------------------------------------------------------------- epilogue
        // warp w reads lane quarter w % 4 (a hardware rule).  The four warps of a quarter work on
        // DIFFERENT tiles (tile sequence number mod 4, as far as there are accumulators in flight):
        // a tile's epilogue is a chain of long-latency steps (barrier poll, tcgen05.ld, wait,
        // arrive, stores) that took ~2000 clocks however little each warp had to do, and with all
        // sixteen warps on the same tile that chain was the kernel's pace.  What is left of the
        // four then shares a tile's 16-channel column groups round robin.
        const int q = warp & 3;
        const int sub = (warp - 2) >> 2;
        constexpr int SUBS = EPI_WARPS / 4;
        const int G = min(SUBS, nacc);  // tile groups (a power of two)
        const int CS = SUBS / G;        // warps of a quarter that share a tile
        const int tg = sub & (G - 1), cs = sub / G;
        int tile_seq = 0;
        bool ok = true;
        const int64_t plane = int64_t(p.h_out) * p.w_out;
        const int lo = p.epi.y_signed ? -128 : 0, hi = p.epi.y_signed ? 127 : 255;
        const float clamp_lo = float(lo - p.epi.y_zp), clamp_hi = float(hi - p.epi.y_zp);
        const int32_t round_fix = p.epi.y_zp - 0x4B400000;
        float run_max = 0.0f, run_neg = 0.0f;  // extrema of the scale-and-bias store, folded once at the end
        for (int tile = blockIdx.x; tile < p.m_tiles; tile += gridDim.x, tile_seq++) {
            if ((tile_seq & (G - 1)) != tg)
                continue;  // another group's tile
            const int b = tile_seq & (nacc - 1);
            if (ok && !wait_bounded(&acc_full[b], (tile_seq / nacc) & 1)) {
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                ok = false;
            }
            umma::tc_fence_after();
            // pixel coordinates without a division: the high half of n * ceil(2^64 / d) is floor(n / d)
            // for every 32-bit n (a divisor of 1 has no such constant and is passed as 0)
            const uint32_t v = uint32_t(tile) * BM + q * 32 + lane;
            const uint32_t img = p.magic_hpwp ? uint32_t(__umul64hi(uint64_t(v), p.magic_hpwp)) : v;
            const uint32_t rem = v - img * uint32_t(p.hpwp);
            uint32_t oh = p.magic_wp ? uint32_t(__umul64hi(uint64_t(rem), p.magic_wp)) : rem;
            uint32_t ow = rem - oh * uint32_t(p.wp);
            bool on_lattice = true;
            if (p.sh != 1 || p.sw != 1) {
                const uint32_t qh = oh / uint32_t(p.sh), qw = ow / uint32_t(p.sw);
                on_lattice = qh * uint32_t(p.sh) == oh && qw * uint32_t(p.sw) == ow;
                oh = qh;
                ow = qw;
            }
            const bool valid = ok && on_lattice && int64_t(v) < p.v_total && int(oh) < p.h_out && int(ow) < p.w_out;
            const int64_t o_base = (int64_t(img) * p.c_out_total + co0) * plane + int64_t(oh) * p.w_out + ow;
            // this warp's last column group: after reading it the accumulator is handed back
            int last_c0 = -1;
            for (int c0 = cs * 16; c0 < p.co_pad; c0 += CS * 16)
                last_c0 = c0;
            if (last_c0 < 0) {
                umma::tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    umma::mbar_arrive(&acc_empty[b]);
            }
            for (int c0 = cs * 16; c0 < p.co_pad; c0 += CS * 16) {
                uint32_t r[16];
                umma::tmem_ld_32x16(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * p.co_pad + c0), r);
                umma::tmem_ld_wait();
                if (c0 == last_c0) {
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        umma::mbar_arrive(&acc_empty[b]);
                }
                // lanes on padding positions store nothing; they skip the block below and meet the others at
                // the __syncwarp that closes it, so the warp is whole again before the next warp-wide tcgen05.ld
                if (valid) {
                // constants of the 16 channels: four 128-bit shared loads each
                int32_t corr[16];
                float ratio[16];
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const int4 cv = *reinterpret_cast<const int4 *>(s_corr + c0 + j);
                    const float4 rv = *reinterpret_cast<const float4 *>(s_ratio + c0 + j);
                    corr[j] = cv.x; corr[j + 1] = cv.y; corr[j + 2] = cv.z; corr[j + 3] = cv.w;
                    ratio[j] = rv.x; ratio[j + 1] = rv.y; ratio[j + 2] = rv.z; ratio[j + 3] = rv.w;
                }
                const int nch = min(16, p.c_out - c0);  // channels of this group that exist
                if (p.epi.mode == EPI_RAW) {
                    int32_t *o = static_cast<int32_t *>(p.out) + o_base + int64_t(c0) * plane;
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (j < nch)
                            o[int64_t(j) * plane] = int32_t(r[j] + uint32_t(corr[j]));
                } else if (p.epi.mode == EPI_SCALE) {
                    // fl(fl(float(acc) * s) + bias) [Relu], every step separately rounded
                    // (glsl/matmul_integer_coop.comp:156-196)
                    float *o = static_cast<float *>(p.out) + o_base + int64_t(c0) * plane;
                    const bool relu = p.epi.flags & 1u;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int32_t acc = int32_t(r[j] + uint32_t(corr[j]));
                        float z = __fadd_rn(__fmul_rn(float(acc), ratio[j]), s_fbias[c0 + j]);
                        if (relu)
                            z = fmaxf(z, 0.0f);
                        if (j < nch) {
                            o[int64_t(j) * plane] = z;
                            run_max = fmaxf(run_max, z);
                            run_neg = fmaxf(run_neg, -z);
                        }
                    }
                } else if (p.out_cl) {
                    // the same bytes, channels-last: this pixel's 16 channels are 16 contiguous bytes, one store
                    uint32_t packed[4];
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        uint32_t word = 0;
#pragma unroll
                        for (int t = 0; t < 4; t++) {
                            const int32_t acc = int32_t(r[j + t] + uint32_t(corr[j + t]));
                            const float x = __fmul_rn(float(acc), ratio[j + t]);
                            const float xc = fminf(fmaxf(x, clamp_lo), clamp_hi);
                            const int32_t qv = __float_as_int(__fadd_rn(xc, 12582912.0f)) + round_fix;
                            word |= (uint32_t(qv) & 0xffu) << (8 * t);
                        }
                        packed[j >> 2] = word;
                    }
                    uint8_t *o = static_cast<uint8_t *>(p.out) +
                                 ((int64_t(img) * p.y_hpwp + int64_t(int(oh) + p.y_pt) * p.y_wp + (int(ow) + p.y_pl)) *
                                      p.c_out_total + co0 + c0);
                    if (nch > 0)  // C_out is a multiple of 16 here: a group exists whole or not at all
                        *reinterpret_cast<uint4 *>(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                } else {
                    uint8_t *o = static_cast<uint8_t *>(p.out) + o_base + int64_t(c0) * plane;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        // sat(rne(f32(acc + bias) * ratio) + y_zp), shaders/qlinear.rs:28-63.  The bounds
                        // are integers, so clamping x to [lo - zp, hi - zp] first and rounding after gives
                        // the same byte; the rounding is the 1.5 * 2^23 trick (adds on the full-rate
                        // pipes instead of a quarter-rate conversion), exact for the clamped range.
                        const int32_t acc = int32_t(r[j] + uint32_t(corr[j]));
                        const float x = __fmul_rn(float(acc), ratio[j]);
                        const float xc = fminf(fmaxf(x, clamp_lo), clamp_hi);
                        const int32_t qv = __float_as_int(__fadd_rn(xc, 12582912.0f)) + round_fix;
                        if (j < nch)
                            o[0] = uint8_t(qv);
                        o += plane;
                    }
                }
                }
                __syncwarp();
            }
        }
        if (p.epi.mode == EPI_SCALE)
            epi_fold_range(p.epi, run_max, run_neg);
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, tmem_cols);
}

// NCHW -> padded NHWC with the padding set to the zero point.  One block per
// padded image row; channels go through shared memory in groups so that reads
// run along W (32-bit when the rows allow it) and writes along C (32-bit, 64+
// contiguous bytes per pixel).
__global__ void __launch_bounds__(256)
conv_pad_nhwc_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ xp, int C, int H, int W, int HP, int WP,
                     int pt, int pl, uint32_t zp_byte, int cgroup, int pitch, int words_ok)
{
    extern __shared__ __align__(16) uint8_t tile[];  // [cgroup][pitch]
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // see conv_pad_nhwc_fast_kernel
    const int hp = blockIdx.x, n = blockIdx.y;
    uint8_t *dst_row = xp + (size_t(n) * HP + hp) * size_t(WP) * C;
    const int h = hp - pt;
    const uint32_t zp4 = zp_byte * 0x01010101u;
    if (h < 0 || h >= H) {
        for (int i = threadIdx.x; i < WP * C / 4; i += blockDim.x)
            reinterpret_cast<uint32_t *>(dst_row)[i] = zp4;
        return;
    }
    for (int c0 = 0; c0 < C; c0 += cgroup) {
        const int cg = min(cgroup, C - c0);
        if (words_ok) {
            const int wpr = W >> 2;
            for (int i = threadIdx.x; i < cg * wpr; i += blockDim.x) {
                const int c = i / wpr, ww = i - c * wpr;
                const uint32_t *src = reinterpret_cast<const uint32_t *>(x + ((size_t(n) * C + c0 + c) * H + h) * W);
                reinterpret_cast<uint32_t *>(tile + c * pitch)[ww] = __ldg(src + ww);
            }
        } else {
            for (int i = threadIdx.x; i < cg * W; i += blockDim.x) {
                const int c = i / W, w = i - c * W;
                tile[c * pitch + w] = x[((size_t(n) * C + c0 + c) * H + h) * W + w];
            }
        }
        __syncthreads();
        const int words = cg >> 2;  // channel groups are multiples of 4
        for (int i = threadIdx.x; i < WP * words; i += blockDim.x) {
            const int wpix = i / words, cw = i - wpix * words;
            const int w = wpix - pl;
            uint32_t v = zp4;
            if (w >= 0 && w < W) {
                const uint8_t *t = tile + (cw * 4) * pitch + w;
                v = uint32_t(t[0]) | (uint32_t(t[pitch]) << 8) | (uint32_t(t[2 * pitch]) << 16) |
                    (uint32_t(t[3 * pitch]) << 24);
            }
            reinterpret_cast<uint32_t *>(dst_row + size_t(wpix) * C + c0)[cw] = v;
        }
        __syncthreads();
    }
}

// The same pass for the common aligned case (W a multiple of 4, C a multiple of
// 16, 4-byte aligned input): one block per image and group of R input rows.  A
// channel's R rows are one contiguous run of R*W bytes, read as 32-bit words
// into shared memory [C][R*W + 4]; then every thread takes four pixels x sixteen
// channels - sixteen words, four 4x4 byte transposes (byte permutes), four
// 128-bit stores of 16 channels each, the four threads of a pixel quad writing
// one pixel's 64 contiguous bytes.  About a twentieth of the instructions of the
// general kernel above.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// (a, b, c, d) = four channels x four pixels (pixel p in byte p)  ->  out[p] = the four channels of pixel p
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&out)[4])
{
    const uint32_t ab_lo = prmt(a, b, 0x5140), ab_hi = prmt(a, b, 0x7362);  // a0 b0 a1 b1 | a2 b2 a3 b3
    const uint32_t cd_lo = prmt(c, d, 0x5140), cd_hi = prmt(c, d, 0x7362);
    out[0] = prmt(ab_lo, cd_lo, 0x5410);  // a0 b0 c0 d0
    out[1] = prmt(ab_lo, cd_lo, 0x7632);  // a1 b1 c1 d1
    out[2] = prmt(ab_hi, cd_hi, 0x5410);
    out[3] = prmt(ab_hi, cd_hi, 0x7632);
}

// (Channels in groups of `cgroup` over blockIdx.z: a block's shared memory is then a few tens of KB whatever C
// is, several blocks share an SM, and their loads are in flight together - with all 512 channels of a 28 x 28
// image in one block the pass ran at a tenth of the memory's rate.  A group writes 128 contiguous bytes of
// every pixel.  The frame is written by the blocks of the first group.)
__global__ void __launch_bounds__(256)
conv_pad_nhwc_fast_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ xp, int C_all, int H, int W, int HP, int WP,
                          int pt, int pl, uint32_t zp_byte, int R, int pitch_words, int cgroup)
{
    extern __shared__ __align__(16) uint32_t slab[];  // [channels of the group][pitch_words]
    const int c_begin = blockIdx.z * cgroup;
    const int C = min(cgroup, C_all - c_begin);  // the channels this block turns
    // the convolution kernel may start its prologue (barriers, tensor memory, filter bank) now; it
    // reads this kernel's output only after griddepcontrol.wait
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int n = blockIdx.y, h0 = blockIdx.x * R;
    const int rows = min(R, H - h0);
    const int words_per_ch = rows * W / 4;
    const uint32_t zp4 = zp_byte * 0x01010101u;
    const uint4 zp16 = make_uint4(zp4, zp4, zp4, zp4);
    // ---- read: a warp per channel, its lanes over the words of the channel's run
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // (a run is at most 64 words; four channels are fetched before anything is stored, so that a
    // warp has eight loads in flight instead of one)
    const size_t ch_stride = size_t(H) * W / 4;  // words between channels
    const uint32_t *src0 = reinterpret_cast<const uint32_t *>(x + ((size_t(n) * C_all + c_begin) * H + h0) * W);
    // (rows wider than 256 pixels are a run of more than 64 words: taken 64 words at a time)
    for (int w0 = 0; w0 < words_per_ch; w0 += 64) {
        const bool has0 = w0 + lane < words_per_ch, has1 = w0 + lane + 32 < words_per_ch;
        for (int c = warp * 4; c < C; c += nwarps * 4) {
            uint32_t v[4][2];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint32_t *src = src0 + size_t(c + k) * ch_stride + w0;
                v[k][0] = (c + k < C && has0) ? __ldg(src + lane) : 0u;
                v[k][1] = (c + k < C && has1) ? __ldg(src + lane + 32) : 0u;
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (c + k < C && has0)
                    slab[(c + k) * pitch_words + w0 + lane] = v[k][0];
                if (c + k < C && has1)
                    slab[(c + k) * pitch_words + w0 + lane + 32] = v[k][1];
            }
        }
    }
    // ---- the padding this block owns: left/right columns of its rows (a warp per row), and the
    // rows above the first / below the last group
    uint8_t *img = xp + size_t(n) * HP * WP * C_all;
    const int c16 = C / 16;
    if (blockIdx.z == 0) {
        const int all16 = C_all / 16;
        const int pr = WP - pl - W;  // padding columns on the right
        for (int r = warp; r < rows; r += nwarps) {
            uint4 *row = reinterpret_cast<uint4 *>(img + size_t(pt + h0 + r) * WP * C_all);
            for (int i = lane; i < pl * all16; i += 32)
                row[i] = zp16;
            uint4 *right = row + size_t(pl + W) * all16;
            for (int i = lane; i < pr * all16; i += 32)
                right[i] = zp16;
        }
        if (blockIdx.x == 0)
            for (int i = threadIdx.x; i < pt * WP * all16; i += blockDim.x)
                reinterpret_cast<uint4 *>(img)[i] = zp16;
        if (h0 + rows == H) {
            const int below = HP - pt - H;
            uint4 *dst = reinterpret_cast<uint4 *>(img + size_t(pt + H) * WP * C_all);
            for (int i = threadIdx.x; i < below * WP * all16; i += blockDim.x)
                dst[i] = zp16;
        }
    }
    __syncthreads();
    // ---- transpose and write
    // one item = (pixel quad, group of 16 channels); the threads of a quad are neighbours so that
    // they write one pixel's contiguous bytes.  c16 is a power of two for the channel counts the
    // tensor path takes (32, 64, 128, 256, ...) or small; the row of a quad comes from one multiply.
    // (Rows that are no whole words - 14 pixels - are taken in groups whose run is: a quad of the run may then
    // straddle two rows, and every pixel of it finds its own row.)
    const int quads = rows * W / 4;
    const uint32_t inv_w = (65536u + uint32_t(W) - 1u) / uint32_t(W);  // pixels of a group < 2^10 + 2^8
    const bool c16_pow2 = (c16 & (c16 - 1)) == 0;
    const int c16_shift = 31 - __clz(c16);
    for (int i = threadIdx.x; i < quads * c16; i += blockDim.x) {
        const int quad = c16_pow2 ? i >> c16_shift : i / c16;
        const int cq = i - quad * c16;
        const uint32_t *src = slab + (cq * 16) * pitch_words + quad;
        uint32_t t[4][4];
#pragma unroll
        for (int g = 0; g < 4; g++)
            transpose4x4(src[(4 * g) * pitch_words], src[(4 * g + 1) * pitch_words], src[(4 * g + 2) * pitch_words],
                         src[(4 * g + 3) * pitch_words], t[g]);
        int r = int((uint32_t(quad * 4) * inv_w) >> 16);
        if (r * W > quad * 4)
            r--;  // the rounded-up reciprocal overshoots by at most one
        int w = quad * 4 - r * W;
#pragma unroll
        for (int px = 0; px < 4; px++) {
            uint8_t *dst = img + (size_t(pt + h0 + r) * WP + pl + w) * C_all + c_begin + cq * 16;
            *reinterpret_cast<uint4 *>(dst) = make_uint4(t[0][px], t[1][px], t[2][px], t[3][px]);
            if (++w == W) {
                w = 0;
                r++;
            }
        }
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

}  // namespace

int32_t ovk_qconv_tc_prepare_weight(ovk_ctx *ctx, ovk_qconv_weight *w)
{
    const int64_t c_in = w->cig, taps = w->kh * w->kw;
    if (w->group != 1 || (c_in != 32 && c_in != 64 && c_in % 128 != 0) || taps > 64)
        return OVK_OK;  // the direct kernel takes these
    const int64_t co_pad = ceil_div64(w->c_out, 32) * 32;
    // at least 32 filters at a time must fit beside two pixel stages (a launch takes as many as fit)
    if (size_t(taps) * 32 * c_in > W_SMEM_MAX + 48 * 1024)
        return OVK_OK;
    w->whole_bank = w->c_out <= 256 && size_t(taps) * co_pad * c_in <= W_SMEM_MAX;
    OVK_CUDA(ctx, cudaMalloc(&w->w_taps, size_t(taps) * co_pad * c_in));
    OVK_CUDA(ctx, cudaMalloc(&w->wsum, size_t(co_pad) * sizeof(int32_t)));
    conv_pack_w_kernel<<<unsigned(co_pad), 256, 0, ctx->stream>>>(w->w, w->w_taps, w->wsum, int(w->c_out), int(co_pad),
                                                                  int(c_in), int(taps), w->w_signed);
    w->c_out_pad = co_pad;
    OVK_LAUNCHED(ctx, "conv_pack_w");
    return OVK_OK;
}

// One group, channel counts the K slices take, strides up to 4 (computed at every position, stored on the
// stride lattice), symmetric weights (w_zp = 0 is checked at launch); everything else takes the direct kernel.
bool ovk_qconv_tc_applies(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, const void *x)
{
    (void)ctx;
    (void)x;
    if (!w->w_taps || g.group != 1 || g.sh > 4 || g.sw > 4)
        return false;
    const int64_t hp = int64_t(g.h_in) + g.phb + g.phe, wp = int64_t(g.w_in) + g.pwb + g.pwe;
    const int64_t v_total = int64_t(g.n) * hp * wp;
    // (small images too: a 7 x 7 plane is one tile, and even one launch per 32 filters beats one thread per output)
    return v_total >= 1 && v_total < (int64_t(1) << 31) - 65536 && (wp * g.c_in) % 4 == 0;
}

// How many launches ovk_qconv_tc_launch would need for this geometry (the filter bank taken in slices that fit
// in shared memory beside two pixel stages), 0 when the kernel does not take it at all.
int ovk_qconv_tc_launches(const ovk_ctx *ctx, const ovk_qconv_weight *w, const ConvGeom &g, const void *x)
{
    if (!ovk_qconv_tc_applies(ctx, w, g, x))
        return 0;
    const int C = g.c_in, kch = std::min(C, 128), chunks = C / kch, taps = g.kh * g.kw;
    const int WP = g.w_in + g.pwb + g.pwe;
    const int max_off = (g.kh - 1) * g.dh * WP + (g.kw - 1) * g.dw;
    const bool halo = chunks == 1 && BM + max_off <= 256;
    const size_t a_stage = (size_t(halo ? BM + max_off : BM) * kch + 1023) & ~size_t(1023);
    const size_t fixed = 1024 + 2048 + 512 + 1024;
    auto bank_bytes = [&](int filters) { return size_t(taps) * chunks * ((size_t(filters) * kch + 1023) & ~size_t(1023)); };
    int per_launch = std::min(256, int(w->c_out_pad));
    while (per_launch > 32 && bank_bytes(per_launch) + 2 * a_stage + fixed > ctx->smem_optin)
        per_launch -= 32;
    if (bank_bytes(per_launch) + 2 * a_stage + fixed > ctx->smem_optin)
        return 0;
    return int(ceil_div64(g.c_out, per_launch));
}

// NCHW x -> xp[n][h + frame][w + frame][c] with the frame set to `fill` (the layout pass of the
// convolution, also an entry point of its own).  g gives n, c_in, h_in, w_in and the four pads.
int32_t ovk_qconv_pad_nhwc(ovk_ctx *ctx, const void *x, const ConvGeom &g, int32_t fill, uint8_t *xp)
{
    const int C = g.c_in;
    const int HP = g.h_in + g.phb + g.phe, WP = g.w_in + g.pwb + g.pwe;
    const int32_t x_zp = fill;
    // Without a frame the image's pixels are one run per channel, and the rows need not be told apart: a
    // 14 x 14 plane, whose rows of 14 bytes are no whole words, is turned as one row of 196 pixels.
    int h_in = g.h_in, w_in = g.w_in;
    if (HP == g.h_in && WP == g.w_in && (g.w_in % 4) != 0 && (int64_t(g.h_in) * g.w_in) % 4 == 0 &&
        int64_t(g.h_in) * g.w_in <= 1024) {
        w_in = g.h_in * g.w_in;
        h_in = 1;
    }
    // rows per block: about 256 pixels, and a whole number of words (W = 14: an even number of rows)
    const int row_unit = (w_in % 4) == 0 ? 1 : ((w_in % 2) == 0 ? 2 : 4);
    const bool fast_layout = (int64_t(h_in) * w_in) % 4 == 0 && h_in % row_unit == 0 && (C % 16) == 0 && aligned_to(x, 4) &&
                             w_in <= (row_unit == 1 ? 1024 : 128) && g.n <= 65535;
    if (fast_layout) {
        const int R = std::max(row_unit, std::min(h_in, 256 / w_in) / row_unit * row_unit);
        const int pitch_words = R * w_in / 4 + 1;
        const int cgroup = std::min(C, 128);
        const size_t sm = size_t(cgroup) * pitch_words * 4;
        if (sm > 48 * 1024)
            OVK_CUDA(ctx, cudaFuncSetAttribute(conv_pad_nhwc_fast_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sm)));
        OVK_REQUIRE(ctx, sm <= ctx->smem_optin && ceil_div64(C, cgroup) <= 65535,
                    "ConvInteger: %d channels are too many for the layout pass", C);
        const bool flat = h_in != g.h_in;
        conv_pad_nhwc_fast_kernel<<<dim3(unsigned(ceil_div64(h_in, R)), unsigned(g.n), unsigned(ceil_div64(C, cgroup))), 256, sm,
                                    ctx->stream>>>(static_cast<const uint8_t *>(x), xp, C, h_in, w_in, flat ? h_in : HP,
                                                   flat ? w_in : WP, g.phb, g.pwb, uint32_t(x_zp) & 0xffu, R, pitch_words, cgroup);
        OVK_LAUNCHED(ctx, "conv_pad_nhwc_fast");
    } else {
        const int pitch = ((g.w_in + 3) & ~3) + 4;
        int cgroup = C;
        while (size_t(cgroup) * pitch > 40 * 1024 && cgroup > 4)
            cgroup = ((cgroup / 2) + 3) & ~3;
        const size_t sm = size_t(cgroup) * pitch;
        OVK_REQUIRE(ctx, sm <= 48 * 1024, "ConvInteger: input rows of %d pixels are too wide for the layout pass", g.w_in);
        const int words_ok = (g.w_in % 4) == 0 && aligned_to(x, 4);
        conv_pad_nhwc_kernel<<<dim3(unsigned(HP), unsigned(g.n)), 256, sm, ctx->stream>>>(
            static_cast<const uint8_t *>(x), xp, C, g.h_in, g.w_in, HP, WP, g.phb, g.pwb, uint32_t(x_zp) & 0xffu, cgroup,
            pitch, words_ok);
        OVK_LAUNCHED(ctx, "conv_pad_nhwc");
    }
    return OVK_OK;
}

int32_t ovk_qconv_tc_launch(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x, int32_t x_signed, const ConvGeom &g,
                            int32_t x_zp, int32_t w_zp, const EpiParams &epi, void *out, const ConvLayout &lay)
{
    if (w_zp != 0)
        return OVK_UNSUPPORTED;  // caller falls back to the direct kernel
    const int C = g.c_in;
    const int HP = g.h_in + g.phb + g.phe, WP = g.w_in + g.pwb + g.pwe;
    const int64_t v_total = int64_t(g.n) * HP * WP;
    const uint8_t *xp = static_cast<const uint8_t *>(x);
    if (!lay.x_cl) {
        // the operator's NCHW: one pass rewrites it; a channels-last caller has done that once, upstream
        const size_t xp_bytes = size_t(v_total) * C;
        void *ws = nullptr;
        int32_t rc = ovk_scratch(ctx, xp_bytes + 1024, &ws);
        if (rc != OVK_OK)
            return rc;
        rc = ovk_qconv_pad_nhwc(ctx, x, g, x_zp, static_cast<uint8_t *>(ws));
        if (rc != OVK_OK)
            return rc;
        xp = static_cast<const uint8_t *>(ws);
    }
    ConvTcParams p = {};
    p.out_cl = lay.y_cl;
    p.y_pt = lay.y_pads[0];
    p.y_pl = lay.y_pads[1];
    p.y_wp = g.w_out + lay.y_pads[1] + lay.y_pads[3];
    p.y_hpwp = int64_t(g.h_out + lay.y_pads[0] + lay.y_pads[2]) * p.y_wp;
    p.v_total = v_total;
    p.hpwp = HP * WP;
    p.wp = WP;
    p.h_out = g.h_out;
    p.w_out = g.w_out;
    p.c_out_total = g.c_out;
    p.sh = g.sh;
    p.sw = g.sw;
    p.w_tap_rows = int(w->c_out_pad);
    p.taps = g.kh * g.kw;
    p.kw = g.kw;
    p.dh = g.dh;
    p.dw = g.dw;
    p.kch = std::min(C, 128);
    p.chunks = C / p.kch;
    p.sw_layout = p.kch == 128 ? umma::LAYOUT_SW128 : (p.kch == 64 ? umma::LAYOUT_SW64 : umma::LAYOUT_SW32);
    p.sbo = 8 * p.kch;
    const int max_off = (g.kh - 1) * g.dh * WP + (g.kw - 1) * g.dw;
    // one halo tile per pixel tile when all taps of a tile fit one TMA box (256 rows); one load per tap otherwise
    p.halo = p.chunks == 1 && BM + max_off <= 256;
    p.halo_rows = p.halo ? BM + max_off : BM;
    p.a_stage = uint32_t((size_t(p.halo_rows) * p.kch + 1023) & ~size_t(1023));
    const size_t epi_extra = epi.mode == EPI_SCALE ? 1024 : 0;  // the per-channel float bias
    const size_t fixed = 1024 + 2048 + 512 + epi_extra;
    auto bank_bytes = [&](int filters) {
        return size_t(p.taps) * p.chunks * ((size_t(filters) * p.kch + 1023) & ~size_t(1023));
    };
    // Filters per launch: the whole bank when it fits beside two pixel stages (four where that costs no extra
    // launch), else as many multiples of 32 (at most 256, the widest MMA) as do; the launches differ only in the
    // filters, constants and output channels they address.
    int per_launch = std::min(256, int(w->c_out_pad));
    while (per_launch > 32 && bank_bytes(per_launch) + 2 * p.a_stage + fixed > ctx->smem_optin)
        per_launch -= 32;
    if (bank_bytes(per_launch) + 2 * p.a_stage + fixed > ctx->smem_optin)
        return OVK_UNSUPPORTED;
    p.x_signed = x_signed ? 1 : 0;
    p.w_signed = w->w_signed;
    p.x_zp = x_zp;
    p.status = ctx->dev_status;
    p.m_tiles = int(ceil_div64(v_total, BM));
    p.magic_hpwp = p.hpwp > 1 ? ~uint64_t(0) / uint64_t(p.hpwp) + 1 : 0;
    p.magic_wp = p.wp > 1 ? ~uint64_t(0) / uint64_t(p.wp) + 1 : 0;
    const CUtensorMapSwizzle swz = p.kch == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                                : (p.kch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUtensorMap tmX;
    if (!ovk_make_tmap_2d(&tmX, xp, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(C), uint64_t(v_total), uint64_t(C),
                          uint32_t(p.kch), uint32_t(p.halo_rows), swz))
        return ovk_fail(ctx, OVK_BACKEND, "ConvInteger: cuTensorMapEncodeTiled failed");
    const size_t out_elem = epi.mode == EPI_REQUANT ? 1 : 4;
    const int64_t plane = int64_t(g.h_out) * g.w_out;
    // (a slightly narrower slice that divides the bank - 512 filters as 4 x 128 rather than 160 + 160 + 160 + 32 - keeps
    // the slices equal, which is what the single launch below needs)
    if (g.c_out > per_launch)
        for (int f = per_launch; f >= 32 && 2 * f > per_launch; f -= 32)
            if (g.c_out % f == 0) {
                per_launch = f;
                break;
            }
    // equal slices go as one launch, a row of the grid each; a bank with a narrower last slice as one launch per slice
    const bool merged = g.c_out > per_launch && g.c_out % per_launch == 0 && g.c_out / per_launch <= 65535;
    p.slice_filters = merged ? per_launch : 0;
    for (int co0 = 0; co0 < g.c_out; co0 += merged ? g.c_out : per_launch) {
        p.c_out = std::min(per_launch, g.c_out - co0);
        p.co_pad = (p.c_out + 31) / 32 * 32;
        p.w_slice = uint32_t((size_t(p.co_pad) * p.kch + 1023) & ~size_t(1023));
        const size_t w_bytes = size_t(p.taps) * p.chunks * p.w_slice;
        const size_t avail = ctx->smem_optin - w_bytes - fixed;
        p.stages = int(std::min<size_t>(MAX_STAGES, avail / p.a_stage));
        if (p.stages < 2)
            return OVK_UNSUPPORTED;
        // With two issuers taking alternate tiles every stage and accumulator must always come back to
        // the same issuer (a waiter may be at most one phase behind its barrier): an even ring, one load
        // per tile.  Otherwise one thread issues everything.
        p.issuers = 1;
        if (p.halo) {
            p.stages &= ~1;
            p.issuers = MMA_WARPS;
        }
        // this launch's filters: their sums, constants and output channels
        p.wsum = w->wsum + co0;
        p.epi = epi;
        if (epi.ibias)
            p.epi.ibias = epi.ibias + co0;
        if (epi.ratio)
            p.epi.ratio = epi.ratio + size_t(co0) * epi.ratio_step;
        if (epi.scale)
            p.epi.scale = epi.scale + size_t(co0) * epi.scale_step;
        if (epi.product)
            p.epi.product = epi.product + size_t(co0) * epi.product_step;
        if (epi.fbias)
            p.epi.fbias = epi.fbias + size_t(co0) * epi.bias_step;
        p.out = static_cast<uint8_t *>(out) + (lay.y_cl ? size_t(co0) : size_t(co0) * plane * out_elem);
        p.nacc = 2;
        while (p.nacc * 2 <= MAX_ACC && p.nacc * 2 * p.co_pad <= 512)
            p.nacc *= 2;
        CUtensorMap tmW;
        if (!ovk_make_tmap_2d(&tmW, w->w_taps + size_t(co0) * C, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(C),
                              uint64_t(p.taps) * w->c_out_pad - co0, uint64_t(C), uint32_t(p.kch), uint32_t(p.co_pad), swz))
            return ovk_fail(ctx, OVK_BACKEND, "ConvInteger: cuTensorMapEncodeTiled failed");
        const size_t smem = w_bytes + size_t(p.stages) * p.a_stage + 512 + 2048 + 512 + epi_extra;
        OVK_CUDA(ctx, cudaFuncSetAttribute(qconv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        const unsigned grid = unsigned(std::min<int>(p.m_tiles, ctx->sm_count));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid, merged ? unsigned(g.c_out / per_launch) : 1u);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        OVK_CUDA(ctx, cudaLaunchKernelEx(&cfg, qconv_tc_kernel, tmX, tmW, p));
        OVK_LAUNCHED(ctx, p.halo ? "qconv_tc_halo" : "qconv_tc_taps");
    }
    return OVK_OK;
}
