// Internal declarations shared by the translation units of libovk_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <utility>
#include <vector>

#include "ovk_cuda.h"
#include "comm.cuh"

// Device-side error codes written to ovk_ctx::dev_status by bounded waits.
enum : int {
    OVK_DEV_OK = 0,
    OVK_DEV_TIMEOUT_TMA = 1,   // a consumer gave up waiting for a bulk copy
    OVK_DEV_TIMEOUT_MMA = 2,   // the epilogue gave up waiting for the tensor core
    OVK_DEV_TIMEOUT_SLOT = 3,  // a producer gave up waiting for a free stage
    OVK_DEV_BAD_INDEX = 4,     // a gather index read on the device fell outside the table
    OVK_DEV_TIMEOUT_PEER = 5,  // a flag another GPU writes never reached the expected value
    OVK_DEV_TIMEOUT_SELFTEST = 6,  // ovk_selftest_device_timeout: the wait that is meant to run out
    OVK_DEV_TIMEOUT_GRID = 7,      // a block gave up waiting for the other blocks of its own launch
};

struct ovk_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = 0;
    size_t smem_optin = 0;
    std::string err;
    const char *last_kernel = "";
    uint64_t launches = 0;
    // device scratch owned by the context
    uint32_t *range_slot = nullptr;  // 64 x u32, zero between calls: folded range and block counters of DynamicQuantizeLinear
    int *dev_status = nullptr;       // sticky error word written by bounded waits
    int *host_status = nullptr;      // pinned mirror read by ovk_flush
    float *params = nullptr;         // OVK_PARAM_FLOATS floats: per-call constants (requantize ratios)
    void *scratch = nullptr;         // grow-on-demand workspace (row sums, NHWC staging, ...)
    size_t scratch_bytes = 0;
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    int clock_khz = 0;
    // the GPUs of one box this context exchanges results with (ovk_comm_init); world == 0: none
    struct {
        int rank = 0, world = 0;
        uint32_t epoch = 0;  // number of collective calls made so far; the same on every rank
        OvkCommFlags *flags[OVK_MAX_RANKS] = {};
        long long wait_cycles = 2000000000ll;  // about a second
    } comm;
    // MatMulNBits prefill with K ranges shared between CTAs: one arrival counter per output tile,
    // zero between launches (the CTA that arrives last at a tile resets it)
    uint32_t *tile_counters = nullptr;
    int mmi_pairs = -1;    // the same for the 256-row MatMulInteger kernel
    int nbits_pairs = -1;  // pairs of CTAs the MatMulNBits prefill kernel can run at once (-1: not asked yet)
};
constexpr int OVK_TILE_COUNTERS = 65536;

constexpr int OVK_PARAM_FLOATS = 16384;

// Sets the context's (or, without a context, the thread's) error message and returns `code`.
int32_t ovk_fail(ovk_ctx *ctx, int32_t code, const char *fmt, ...);

// Grows the context workspace to at least `bytes` (stream-ordered: the old
// block is released only after work already enqueued has finished).
int32_t ovk_scratch(ovk_ctx *ctx, size_t bytes, void **out);

#define OVK_CUDA(ctx, expr)                                                               \
    do {                                                                                  \
        cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return ovk_fail((ctx), OVK_BACKEND, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

#define OVK_REQUIRE(ctx, cond, ...)                                \
    do {                                                           \
        if (!(cond))                                               \
            return ovk_fail((ctx), OVK_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

#define OVK_REFUSE(ctx, cond, ...)                            \
    do {                                                      \
        if (cond)                                             \
            return ovk_fail((ctx), OVK_UNSUPPORTED, __VA_ARGS__); \
    } while (0)

// Records a kernel launch (name for ovk_last_kernel, count for ovk_launch_count)
// and turns a launch error into a status.
#define OVK_LAUNCHED(ctx, name)                                                        \
    do {                                                                               \
        (ctx)->last_kernel = (name);                                                   \
        (ctx)->launches++;                                                             \
        cudaError_t e_ = cudaGetLastError();                                           \
        if (e_ != cudaSuccess)                                                         \
            return ovk_fail((ctx), OVK_BACKEND, "%s: %s", (name), cudaGetErrorString(e_)); \
    } while (0)

// Starts the next collective call on this context: bumps the call number and describes the peers to a kernel.
OvkCommView ovk_comm_next(ovk_ctx *ctx);
// Enqueues the wait for every peer's `done` announcement of call `view.epoch`.
int32_t ovk_comm_wait_done(ovk_ctx *ctx, const OvkCommView &view);

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// A launch that may begin while the previous kernel of the stream is still draining (programmatic
// dependent launch).  Kernels launched this way call griddepcontrol.launch_dependents early and touch
// nothing another kernel produces, and write nothing, before griddepcontrol.wait: only their prologue
// (barriers, tensor memory, index arithmetic) and the launch latency overlap the predecessor.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
static inline cudaError_t ovk_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         Args &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define OVK_PDL_LAUNCH_DEPENDENTS() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define OVK_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
#endif
static inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---------------------------------------------------------------- weights

struct ovk_nbits_weight {
    const uint8_t *b = nullptr;       // operator layout [N, n_blocks, bs/2]
    const void *scales = nullptr;     // [N, n_blocks] f32 / f16
    const uint8_t *zp = nullptr;      // [N, ceil(n_blocks/2)] or null (implicit 8)
    int32_t scales_dtype = OVK_FLOAT;
    int64_t n = 0, k = 0, block_size = 0, n_blocks = 0;
    // decode copy (built by prepack when block_size is a multiple of 32): tiles of
    // dec_p 16-column panels x dec_kc quantization blocks, each tile contiguous
    void *decode = nullptr;
    size_t decode_bytes = 0;
    int dec_p = 0, dec_kc = 0, dec_gb = 0, dec_nkc = 0, dec_ntiles = 0;
    uint32_t dec_s_off = 0, dec_z_off = 0, dec_tile_bytes = 0;
    // prefill copy (built on the first prefill call): nibble-permuted rows, f32 scales [block, n_pad],
    // one zero-point byte per block [n_pad, zp_pitch]
    void *gemm_w = nullptr;
    float *gemm_scales_t = nullptr;
    uint8_t *gemm_zp_t = nullptr;
    int64_t gemm_k_pad = 0, gemm_n_pad = 0, gemm_zp_pitch = 0;
};

struct ovk_mmi_weight {
    int64_t k = 0, n = 0;
    int64_t k_pad = 0;         // row pitch of bt in bytes (multiple of 16)
    int64_t n_pad = 0;
    int32_t b_signed = 0;
    uint8_t *bt = nullptr;     // [n_pad, k_pad] B transposed, K contiguous, zero padded
    int32_t *colsum = nullptr; // [n_pad] sum over k of b[k][n] (signed interpretation applied)
    void *tmap_b = nullptr;    // host copy of the CUtensorMap describing bt (128 bytes), or null
};

// Resolved geometry of one convolution call (interp::ConvGeom, src/interp.rs:3361-3384).
struct ConvGeom {
    int n, c_in, c_out, group, cig;
    int h_in, w_in, h_out, w_out;
    int kh, kw, sh, sw, dh, dw, phb, pwb, phe, pwe;
};

// Which of the two tensor layouts a convolution call reads and writes: the operator's NCHW, or
// channels-last inside a frame, [n][h + top + bottom][w + left + right][c], the frame holding the
// tensor's zero point (the layout the tensor-core kernel computes from).
struct ConvLayout {
    int x_cl = 0, y_cl = 0;
    int y_pads[4] = {0, 0, 0, 0};  // top, left, bottom, right frame of the output
};

struct ovk_qconv_weight {
    int64_t c_out = 0, cig = 0, kh = 0, kw = 0, group = 1;
    int32_t w_signed = 0;
    uint8_t *w = nullptr;       // copy in the operator layout [C_out, C_in/g, KH, KW]
    uint8_t *w_taps = nullptr;  // [KH*KW, C_out_pad, C_in] tap-major copy for the tensor path (group 1)
    int32_t *wsum = nullptr;    // [C_out_pad] sum of all weights of a filter (group 1)
    int64_t c_out_pad = 0;
    uint8_t *w_rows16 = nullptr;  // [C_out][K rounded up to 16] zero-padded rows, built when K is no multiple of 16
    bool whole_bank = false;    // the tensor-core convolution kernel holds all filters in shared memory at once
    // the last requantisation ratios uploaded for this filter bank (a content-keyed
    // parameter cache, as interp::param_buffer in the reference): constants of the
    // graph are uploaded once, not per call
    std::vector<float> ratio_host;
    float *ratio_dev = nullptr;
};
