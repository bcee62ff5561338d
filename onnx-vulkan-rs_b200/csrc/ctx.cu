// Context, buffers and timing: the CUDA counterpart of the verbs the
// reference's operators use from crates/vk-compute (context.rs, buffer.rs,
// stream.rs, pipeline.rs:246).
#include "ovk_internal.h"
#include "umma.cuh"

#include <algorithm>
#include <cstring>

static thread_local std::string g_tls_error;

int32_t ovk_fill_u32(ovk_ctx *ctx, void *dst, size_t words, uint32_t value);

int32_t ovk_fail(ovk_ctx *ctx, int32_t code, const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->err = buf;
    else
        g_tls_error = buf;
    return code;
}

int32_t ovk_scratch(ovk_ctx *ctx, size_t bytes, void **out)
{
    if (bytes > ctx->scratch_bytes) {
        // The old block may still be read by kernels already enqueued:
        // cudaFreeAsync orders the release after them.
        if (ctx->scratch)
            OVK_CUDA(ctx, cudaFreeAsync(ctx->scratch, ctx->stream));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
        size_t want = (bytes + 255) & ~size_t(255);
        OVK_CUDA(ctx, cudaMallocAsync(&ctx->scratch, want, ctx->stream));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return OVK_OK;
}

extern "C" {

int32_t ovk_ctx_create(int32_t device, void *stream, ovk_ctx **out)
{
    if (!out)
        return ovk_fail(nullptr, OVK_INVALID_ARGUMENT, "ovk_ctx_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return ovk_fail(nullptr, OVK_BACKEND, "ovk_ctx_create: no CUDA device (%s)",
                        cudaGetErrorString(e));
    if (device < 0 || device >= count)
        return ovk_fail(nullptr, OVK_INVALID_ARGUMENT, "ovk_ctx_create: device %d of %d", device, count);
    ovk_ctx *ctx = new ovk_ctx();
    ctx->device = device;
#define CTX_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t e_ = (expr);                                                           \
        if (e_ != cudaSuccess) {                                                           \
            int32_t rc = ovk_fail(nullptr, OVK_BACKEND, "%s: %s", #expr, cudaGetErrorString(e_)); \
            delete ctx;                                                                    \
            return rc;                                                                     \
        }                                                                                  \
    } while (0)
    CTX_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    CTX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        fprintf(stderr, "ovk: device %d is sm_%d%d; this library is built for sm_100a only\n",
                device, prop.major, prop.minor);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    ctx->clock_khz = prop.clockRate;
    if (stream) {
        ctx->stream = static_cast<cudaStream_t>(stream);
    } else {
        CTX_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        ctx->own_stream = true;
    }
    CTX_CUDA(cudaMalloc(&ctx->range_slot, 256));
    CTX_CUDA(cudaMalloc(&ctx->dev_status, 256));
    CTX_CUDA(cudaMalloc(&ctx->params, OVK_PARAM_FLOATS * sizeof(float)));
    CTX_CUDA(cudaMemset(ctx->dev_status, 0, 256));
    CTX_CUDA(cudaMemset(ctx->range_slot, 0, 256));  // DynamicQuantizeLinear leaves it zeroed after every call
    CTX_CUDA(cudaMallocHost(&ctx->host_status, 64));
    ctx->host_status[0] = 0;
    CTX_CUDA(cudaEventCreate(&ctx->t0));
    CTX_CUDA(cudaEventCreate(&ctx->t1));
#undef CTX_CUDA
    *out = ctx;
    return OVK_OK;
}

void ovk_ctx_destroy(ovk_ctx *ctx)
{
    if (!ctx)
        return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch)
        cudaFree(ctx->scratch);
    cudaFree(ctx->range_slot);
    cudaFree(ctx->dev_status);
    cudaFree(ctx->params);
    cudaFree(ctx->tile_counters);
    cudaFreeHost(ctx->host_status);
    cudaEventDestroy(ctx->t0);
    cudaEventDestroy(ctx->t1);
    if (ctx->own_stream)
        cudaStreamDestroy(ctx->stream);
    delete ctx;
}

const char *ovk_last_error(const ovk_ctx *ctx) { return ctx ? ctx->err.c_str() : g_tls_error.c_str(); }
const char *ovk_last_kernel(const ovk_ctx *ctx) { return ctx ? ctx->last_kernel : ""; }
uint64_t ovk_launch_count(const ovk_ctx *ctx) { return ctx ? ctx->launches : 0; }
void *ovk_stream(const ovk_ctx *ctx) { return ctx ? ctx->stream : nullptr; }
size_t ovk_workspace_bytes(const ovk_ctx *ctx) { return ctx ? ctx->scratch_bytes : 0; }

int32_t ovk_flush(ovk_ctx *ctx)
{
    if (!ctx)
        return ovk_fail(nullptr, OVK_INVALID_ARGUMENT, "ovk_flush: null context");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    OVK_CUDA(ctx, cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int),
                                  cudaMemcpyDeviceToHost, ctx->stream));
    OVK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int st = ctx->host_status[0];
    if (st != OVK_DEV_OK) {
        OVK_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), ctx->stream));
        OVK_CUDA(ctx, cudaMemsetAsync(ctx->range_slot, 0, 256, ctx->stream));  // a launch that gave up may have left counts
        if (st == OVK_DEV_BAD_INDEX)
            return ovk_fail(ctx, OVK_INVALID_ARGUMENT,
                            "GatherBlockQuantized: an index read on the device fell outside the table "
                            "(its row was written as zeros)");
        return ovk_fail(ctx, OVK_TIMEOUT, "a device-side wait gave up (code %d: %s)", st,
                        st == OVK_DEV_TIMEOUT_TMA    ? "bulk copy never arrived"
                        : st == OVK_DEV_TIMEOUT_MMA  ? "tensor core never signalled"
                        : st == OVK_DEV_TIMEOUT_SLOT ? "pipeline stage never freed"
                        : st == OVK_DEV_TIMEOUT_PEER ? "a peer GPU never signalled"
                        : st == OVK_DEV_TIMEOUT_GRID ? "a block of the same launch never arrived"
                                                     : "self-test wait on a barrier nothing arrives at");
    }
    return OVK_OK;
}

int32_t ovk_alloc(ovk_ctx *ctx, size_t bytes, void **dptr)
{
    if (!ctx || !dptr)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_alloc: null argument");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    *dptr = nullptr;
    // sizes are rounded up so that vector loads of the last elements stay inside
    OVK_CUDA(ctx, cudaMalloc(dptr, ((bytes ? bytes : 1) + 255) & ~size_t(255)));
    return OVK_OK;
}

int32_t ovk_free(ovk_ctx *ctx, void *dptr)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_free: null context");
    if (!dptr)
        return OVK_OK;
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    OVK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    OVK_CUDA(ctx, cudaFree(dptr));
    return OVK_OK;
}

int32_t ovk_upload(ovk_ctx *ctx, void *dst, size_t offset, const void *src, size_t bytes)
{
    if (!ctx || (!dst && bytes) || (!src && bytes))
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_upload: null argument");
    if (!bytes)
        return OVK_OK;
    OVK_CUDA(ctx, cudaMemcpyAsync(static_cast<char *>(dst) + offset, src, bytes,
                                  cudaMemcpyHostToDevice, ctx->stream));
    return OVK_OK;
}

int32_t ovk_download(ovk_ctx *ctx, const void *src, size_t offset, void *dst, size_t bytes)
{
    if (!ctx || (!dst && bytes) || (!src && bytes))
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_download: null argument");
    if (bytes)
        OVK_CUDA(ctx, cudaMemcpyAsync(dst, static_cast<const char *>(src) + offset, bytes,
                                      cudaMemcpyDeviceToHost, ctx->stream));
    return ovk_flush(ctx);
}

int32_t ovk_fill(ovk_ctx *ctx, void *dst, size_t offset, size_t bytes, uint32_t value)
{
    if (!ctx || (!dst && bytes))
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_fill: null argument");
    OVK_REQUIRE(ctx, (offset % 4) == 0 && (bytes % 4) == 0,
                "ovk_fill: offset %zu and size %zu must be multiples of 4", offset, bytes);
    if (!bytes)
        return OVK_OK;
    char *p = static_cast<char *>(dst) + offset;
    uint8_t b0 = value & 0xff;
    if (((value >> 8) & 0xff) == b0 && ((value >> 16) & 0xff) == b0 && (value >> 24) == b0) {
        OVK_CUDA(ctx, cudaMemsetAsync(p, b0, bytes, ctx->stream));
    } else {
        return ovk_fill_u32(ctx, p, bytes / 4, value);
    }
    return OVK_OK;
}

int32_t ovk_timer_start(ovk_ctx *ctx)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_timer_start: null context");
    OVK_CUDA(ctx, cudaEventRecord(ctx->t0, ctx->stream));
    return OVK_OK;
}

int32_t ovk_timer_stop(ovk_ctx *ctx, float *ms)
{
    if (!ctx || !ms)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_timer_stop: null argument");
    OVK_CUDA(ctx, cudaEventRecord(ctx->t1, ctx->stream));
    OVK_CUDA(ctx, cudaEventSynchronize(ctx->t1));
    OVK_CUDA(ctx, cudaEventElapsedTime(ms, ctx->t0, ctx->t1));
    return OVK_OK;
}

}  // extern "C"

// One thread waits, through the same bounded-wait helper the tensor-core
// kernels use, on a barrier nothing ever arrives at; after `polls` attempts it
// records the code in the status word and the kernel ends.  No copy and no
// tensor memory is in flight, nothing faults, nothing spins for long.
__global__ void selftest_timeout_kernel(int *status, uint32_t polls)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        umma::mbar_init(&bar, 1);
        umma::fence_barrier_init();
        if (!umma::mbar_wait_limit(&bar, 0, polls))
            atomicExch(status, OVK_DEV_TIMEOUT_SELFTEST);
    }
}

extern "C" int32_t ovk_selftest_device_timeout(ovk_ctx *ctx)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_selftest_device_timeout: null context");
    selftest_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, 1000u);
    OVK_LAUNCHED(ctx, "selftest_timeout");
    return OVK_OK;
}

__global__ void fill_u32_kernel(uint32_t *dst, size_t words, uint32_t value)
{
    size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x;
    size_t stride = size_t(gridDim.x) * blockDim.x;
    for (; i < words; i += stride)
        dst[i] = value;
}

int32_t ovk_fill_u32(ovk_ctx *ctx, void *dst, size_t words, uint32_t value)
{
    unsigned blocks = static_cast<unsigned>(std::min<size_t>((words + 255) / 256, 148 * 8));
    fill_u32_kernel<<<blocks, 256, 0, ctx->stream>>>(static_cast<uint32_t *>(dst), words, value);
    OVK_LAUNCHED(ctx, "fill_u32");
    return OVK_OK;
}
