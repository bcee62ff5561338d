// Exchange between the GPUs of one box, through peer memory.
//
// The reference runs on one device per process (crates/vk-compute/src/
// context.rs:685-711) and has nothing here.  The partitioned operators - the
// MatMulNBits prefill split over weight columns - end in an all-gather of the
// column blocks; this file holds its plumbing (shareable allocations and their
// handles, the flag blocks, the wait) and the exchange as a kernel of its own.
// The prefill kernel performs the same exchange from its epilogue
// (nbits_gemm.cu); this kernel serves the other MatMulNBits kernels and callers
// that already hold a finished column block.
//
// One process per GPU.  A buffer that peers write into is allocated with
// cudaMalloc (ovk_comm_alloc), exported as a 64-byte handle
// (cudaIpcGetMemHandle) that the host carries to the other processes by any
// channel it has, and mapped there (cudaIpcOpenMemHandle, which also enables
// peer access).  Kernels then use ordinary loads and stores on the mapped
// addresses: no library kernel is ever given a peer's memory, and no bulk-copy
// or multicast instruction touches it.
#include "ovk_internal.h"

#include <cstring>

namespace {

constexpr int COPY_THREADS = 256;
// CTAs of the exchange kernel, at most: measured at 2 ranks (77.6 MB to the one peer) 64 CTAs deliver 310 GB/s,
// 148 467 GB/s, 296 520 GB/s, 592 and 1184 534 GB/s - the stores in flight, not the links, set the rate below two
// CTAs per SM.
#ifndef OVK_GATHER_MAX_CTAS
#define OVK_GATHER_MAX_CTAS 296
#endif

struct GatherParams {
    const uint8_t *src;      // this rank's column block
    size_t src_pitch;        // bytes between its rows
    uint8_t *dst[OVK_MAX_RANKS];  // every rank's full matrix
    size_t dst_pitch;        // bytes between rows of the full matrix
    size_t dst_col;          // byte offset of the block inside a row
    int64_t rows;
    int64_t row_bytes;       // bytes of one row of the block
    int elem_bytes;
    int vec16;               // every address involved is a multiple of 16
    int skip_self;           // the block already sits in this rank's full matrix
    uint8_t *mc;             // multicast mapping of every rank's full matrix, or null
    int *status;
};

__global__ void __launch_bounds__(COPY_THREADS)
allgather_cols_kernel(OvkCommView c, GatherParams p)
{
    __shared__ int s_go, s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        if (blockIdx.x == 0)
            comm::announce(c, false, lane);  // this rank's earlier work on the stream is complete
        const bool go = comm::wait_all(c, false, lane);  // and so is every peer's: their buffers may be written
        if (lane == 0) {
            s_go = go;
            if (!go)
                atomicExch(p.status, OVK_DEV_TIMEOUT_PEER);
        }
    }
    __syncthreads();
    if (s_go) {
        if (p.vec16) {
            const int64_t per_row = p.row_bytes >> 4;
            const int64_t total = p.rows * per_row;
            for (int64_t i = int64_t(blockIdx.x) * COPY_THREADS + threadIdx.x; i < total;
                 i += int64_t(gridDim.x) * COPY_THREADS) {
                const int64_t r = i / per_row, ch = i - r * per_row;
                const uint4 v = *reinterpret_cast<const uint4 *>(p.src + r * p.src_pitch + (ch << 4));
                const size_t off = size_t(r) * p.dst_pitch + p.dst_col + (size_t(ch) << 4);
                if (p.mc) {  // one store, delivered to every rank by the switch
                    comm::st_multicast16(p.mc + off, v);
                    continue;
                }
                // ranks run in step: each starts behind itself, so that no rank's links take everybody's stores at once
                for (int j = 0; j < c.world; j++) {
                    const int d = c.rank + 1 + j < c.world ? c.rank + 1 + j : c.rank + 1 + j - c.world;
                    if (!(p.skip_self && d == c.rank))
                        *reinterpret_cast<uint4 *>(p.dst[d] + off) = v;
                }
            }
        } else {
            // ragged or unaligned blocks: element by element (2 or 4 bytes)
            const int64_t per_row = p.row_bytes / p.elem_bytes;
            const int64_t total = p.rows * per_row;
            for (int64_t i = int64_t(blockIdx.x) * COPY_THREADS + threadIdx.x; i < total;
                 i += int64_t(gridDim.x) * COPY_THREADS) {
                const int64_t r = i / per_row, e = i - r * per_row;
                const uint8_t *s = p.src + r * p.src_pitch + e * p.elem_bytes;
                const size_t off = size_t(r) * p.dst_pitch + p.dst_col + size_t(e) * p.elem_bytes;
                for (int d = 0; d < c.world; d++) {
                    if (p.skip_self && d == c.rank)
                        continue;
                    if (p.elem_bytes == 2)
                        *reinterpret_cast<uint16_t *>(p.dst[d] + off) = *reinterpret_cast<const uint16_t *>(s);
                    else
                        *reinterpret_cast<uint32_t *>(p.dst[d] + off) = *reinterpret_cast<const uint32_t *>(s);
                }
            }
        }
    }
    // every thread's stores are visible everywhere before this CTA is counted; the CTA counted last
    // announces the whole kernel's stores
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        OvkCommFlags *own = c.flags[c.rank];
        const uint32_t before = atomicAdd(&own->cta_done, 1u);
        s_last = before + 1u == gridDim.x;
        if (s_last)
            own->cta_done = 0;
        __threadfence_system();
    }
    __syncthreads();
    if (warp == 0 && s_last && s_go)
        comm::announce(c, true, lane);
}

__global__ void comm_wait_kernel(OvkCommView c, int *status)
{
    if (!comm::wait_all(c, true, int(threadIdx.x)) && threadIdx.x == 0)
        atomicExch(status, OVK_DEV_TIMEOUT_PEER);
}

__global__ void comm_barrier_kernel(OvkCommView c, int *status)
{
    __threadfence_system();
    comm::announce(c, true, int(threadIdx.x));
    if (!comm::wait_all(c, true, int(threadIdx.x)) && threadIdx.x == 0)
        atomicExch(status, OVK_DEV_TIMEOUT_PEER);
}

}  // namespace

OvkCommView ovk_comm_next(ovk_ctx *ctx)
{
    OvkCommView v = {};
    ctx->comm.epoch++;
    for (int r = 0; r < OVK_MAX_RANKS; r++)
        v.flags[r] = ctx->comm.flags[r];
    v.rank = ctx->comm.rank;
    v.world = ctx->comm.world;
    v.epoch = ctx->comm.epoch;
    v.wait_cycles = ctx->comm.wait_cycles;
    return v;
}

int32_t ovk_comm_wait_done(ovk_ctx *ctx, const OvkCommView &view)
{
    comm_wait_kernel<<<1, 32, 0, ctx->stream>>>(view, ctx->dev_status);
    OVK_LAUNCHED(ctx, "comm_wait");
    return OVK_OK;
}

// The exchange on prepared arguments; `view` is this call's epoch (already taken).
int32_t ovk_comm_gather_cols(ovk_ctx *ctx, const OvkCommView &view, const void *src, size_t src_pitch, int elem_bytes,
                             int64_t m, int64_t n_shard, int64_t col0, int64_t n_total, void *const *y_peers,
                             bool skip_self, void *y_multicast)
{
    GatherParams p = {};
    p.src = static_cast<const uint8_t *>(src);
    p.src_pitch = src_pitch;
    p.dst_pitch = size_t(n_total) * elem_bytes;
    p.dst_col = size_t(col0) * elem_bytes;
    p.rows = m;
    p.row_bytes = n_shard * elem_bytes;
    p.elem_bytes = elem_bytes;
    p.skip_self = skip_self;
    p.status = ctx->dev_status;
    bool vec = aligned_to(src, 16) && src_pitch % 16 == 0 && p.dst_pitch % 16 == 0 && p.dst_col % 16 == 0 &&
               p.row_bytes % 16 == 0;
    for (int r = 0; r < view.world; r++) {
        p.dst[r] = static_cast<uint8_t *>(y_peers[r]);
        vec = vec && aligned_to(y_peers[r], 16);
    }
    p.vec16 = vec;
    p.mc = vec && aligned_to(y_multicast, 16) ? static_cast<uint8_t *>(y_multicast) : nullptr;
    const int64_t chunks = m * (vec ? p.row_bytes / 16 : n_shard);
    const unsigned grid = unsigned(std::max<int64_t>(1, std::min<int64_t>(ceil_div64(chunks, COPY_THREADS * 4), OVK_GATHER_MAX_CTAS)));
    allgather_cols_kernel<<<grid, COPY_THREADS, 0, ctx->stream>>>(view, p);
    OVK_LAUNCHED(ctx, "allgather_cols");
    return ovk_comm_wait_done(ctx, view);
}

extern "C" {

size_t ovk_comm_flag_bytes(void) { return sizeof(OvkCommFlags); }

int32_t ovk_comm_alloc(ovk_ctx *ctx, size_t bytes, void **dptr)
{
    if (!ctx || !dptr)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_alloc: null argument");
    *dptr = nullptr;
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    void *p = nullptr;
    const size_t size = ((bytes ? bytes : 1) + 255) & ~size_t(255);
    OVK_CUDA(ctx, cudaMalloc(&p, size));
    cudaError_t e = cudaMemset(p, 0, size);
    if (e != cudaSuccess) {
        cudaFree(p);
        return ovk_fail(ctx, OVK_BACKEND, "ovk_comm_alloc: %s", cudaGetErrorString(e));
    }
    *dptr = p;
    return OVK_OK;
}

int32_t ovk_comm_export(ovk_ctx *ctx, void *dptr, void *handle_out)
{
    if (!ctx || !dptr || !handle_out)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == OVK_COMM_HANDLE_BYTES, "handle size");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    OVK_CUDA(ctx, cudaIpcGetMemHandle(&h, dptr));
    memcpy(handle_out, &h, sizeof h);
    return OVK_OK;
}

int32_t ovk_comm_import(ovk_ctx *ctx, const void *handle, void **peer_ptr)
{
    if (!ctx || !handle || !peer_ptr)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_import: null argument");
    *peer_ptr = nullptr;
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    OVK_CUDA(ctx, cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return OVK_OK;
}

int32_t ovk_comm_release(ovk_ctx *ctx, void *peer_ptr)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_release: null context");
    if (!peer_ptr)
        return OVK_OK;
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    OVK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    OVK_CUDA(ctx, cudaIpcCloseMemHandle(peer_ptr));
    return OVK_OK;
}

int32_t ovk_comm_init(ovk_ctx *ctx, int32_t rank, int32_t world, void *const *flag_blocks)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_init: null context");
    OVK_REQUIRE(ctx, world >= 1 && world <= OVK_MAX_RANKS, "ovk_comm_init: %d ranks (1 to %d)", world, OVK_MAX_RANKS);
    OVK_REQUIRE(ctx, rank >= 0 && rank < world, "ovk_comm_init: rank %d of %d", rank, world);
    OVK_REQUIRE(ctx, flag_blocks, "ovk_comm_init: the flag blocks are missing");
    for (int r = 0; r < world; r++)
        OVK_REQUIRE(ctx, flag_blocks[r] && aligned_to(flag_blocks[r], 256),
                    "ovk_comm_init: flag block of rank %d is null or not 256-byte aligned", r);
    ctx->comm.rank = rank;
    ctx->comm.world = world;
    ctx->comm.epoch = 0;
    for (int r = 0; r < OVK_MAX_RANKS; r++)
        ctx->comm.flags[r] = r < world ? static_cast<OvkCommFlags *>(flag_blocks[r]) : nullptr;
    return OVK_OK;
}

int32_t ovk_comm_set_timeout_ms(ovk_ctx *ctx, int32_t ms)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_set_timeout_ms: null context");
    OVK_REQUIRE(ctx, ms >= 1 && ms <= 60000, "ovk_comm_set_timeout_ms: %d ms (1 to 60000)", ms);
    ctx->comm.wait_cycles = (long long)ms * std::max(ctx->clock_khz, 1000);
    return OVK_OK;
}

int32_t ovk_comm_barrier(ovk_ctx *ctx)
{
    if (!ctx)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_comm_barrier: null context");
    OVK_REQUIRE(ctx, ctx->comm.world >= 1, "ovk_comm_barrier: ovk_comm_init has not been called");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    const OvkCommView v = ovk_comm_next(ctx);
    comm_barrier_kernel<<<1, 32, 0, ctx->stream>>>(v, ctx->dev_status);
    OVK_LAUNCHED(ctx, "comm_barrier");
    return OVK_OK;
}

int32_t ovk_allgather_cols(ovk_ctx *ctx, const void *y_shard, int32_t dtype, int64_t m, int64_t n_shard, int64_t col0,
                           int64_t n_total, void *const *y_peers)
{
    return ovk_allgather_cols_multicast(ctx, y_shard, dtype, m, n_shard, col0, n_total, y_peers, nullptr);
}

int32_t ovk_allgather_cols_multicast(ovk_ctx *ctx, const void *y_shard, int32_t dtype, int64_t m, int64_t n_shard,
                                     int64_t col0, int64_t n_total, void *const *y_peers, void *y_multicast)
{
    if (!ctx || !y_peers)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_allgather_cols: null argument");
    OVK_REQUIRE(ctx, ctx->comm.world >= 1, "ovk_allgather_cols: ovk_comm_init has not been called");
    OVK_REFUSE(ctx, dtype != OVK_FLOAT && dtype != OVK_FLOAT16 && dtype != OVK_INT32,
               "ovk_allgather_cols: dtype %d (f32, f16 or i32)", dtype);
    OVK_REQUIRE(ctx, m >= 0 && n_shard >= 0 && col0 >= 0 && col0 + n_shard <= n_total,
                "ovk_allgather_cols: columns [%lld, %lld) of %lld", (long long)col0, (long long)(col0 + n_shard),
                (long long)n_total);
    for (int r = 0; r < ctx->comm.world; r++)
        OVK_REQUIRE(ctx, y_peers[r], "ovk_allgather_cols: the matrix of rank %d is null", r);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    const int es = dtype == OVK_FLOAT16 ? 2 : 4;
    const OvkCommView v = ovk_comm_next(ctx);  // every rank counts this call, also one with nothing to send
    const bool in_place = y_shard == nullptr;
    const void *src = in_place ? static_cast<const uint8_t *>(y_peers[ctx->comm.rank]) + size_t(col0) * es : y_shard;
    const size_t pitch = size_t(in_place ? n_total : n_shard) * es;
    // a multicast store also writes this rank's own copy, so an in-place block is simply written again
    return ovk_comm_gather_cols(ctx, v, src, pitch, es, m, n_shard, col0, n_total, y_peers, in_place, y_multicast);
}

}  // extern "C"
