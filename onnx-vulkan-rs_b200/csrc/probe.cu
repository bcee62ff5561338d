// The tensor core's issue rate, measured: the denominator for the int8 kernels.
//
// No published or driver-measured dense int8 figure exists for this part, so the
// library measures what tcgen05.mma can deliver: one CTA per SM, one thread
// issuing a long unrolled run of 128 x 256 MMAs (K = 32 bytes for kind::i8, 16
// fp16 for kind::f16) over operands that sit in shared memory (their values do
// not matter), two accumulators alternating, timed with clock64 from the first
// issue to the completion of the last.  The result is multiply-accumulates per
// clock per SM - 8163 for kind::i8 and 4081 for kind::f16 on a B200, against
// the nominal 8192 and 4096 - which the caller scales by the SM count and the
// clock it samples while its own kernels run.
#include "ovk_internal.h"
#include "umma.cuh"

namespace {

constexpr int PROBE_N = 256, PROBE_KCH = 128, PROBE_ACC = 2, PROBE_ITERS = 200;
constexpr size_t PROBE_SMEM = 200 * 1024;

template <int F16>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(long long *out, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < int(PROBE_SMEM / 4); i += blockDim.x)
        reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u * (i & 3);
    if (threadIdx.x == 0) {
        umma::mbar_init(&bar, 1);
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        umma::tmem_alloc(&tmem_slot, 512);
        umma::tmem_relinquish();
    }
    umma::fence_proxy_async();
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (warp == 0 && lane == 0) {
        const uint32_t idesc = F16 ? umma::instr_desc(1, 0, 0, 128, PROBE_N) : umma::instr_desc(2, 0, 1, 128, PROBE_N);
        constexpr uint32_t sbo = 8 * PROBE_KCH;
        constexpr uint32_t desc_hi = ((sbo >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
        const uint32_t a_lo = ((umma::smem_u32(smem) >> 4) & 0x3fffu) | (1u << 16);
        const uint32_t b_lo = ((umma::smem_u32(smem + 96 * 1024) >> 4) & 0x3fffu) | (1u << 16);
        const long long t0 = clock64();
        for (int it = 0; it < PROBE_ITERS; it++) {
#pragma unroll
            for (int acc = 0; acc < PROBE_ACC; acc++) {
#pragma unroll
                for (int j = 0; j < PROBE_KCH / 32; j++) {
                    if (F16)
                        umma::mma_f16_lohi(tmem_base + acc * PROBE_N, a_lo + 2u * j, desc_hi, b_lo + 2u * j, desc_hi, idesc, 1u);
                    else
                        umma::mma_i8_lohi(tmem_base + acc * PROBE_N, a_lo + 2u * j, desc_hi, b_lo + 2u * j, desc_hi, idesc, 1u);
                }
            }
        }
        umma::mma_commit(&bar);
        const bool ok = umma::mbar_wait(&bar, 0);  // bounded
        const long long t1 = clock64();
        if (!ok)
            atomicExch(status, OVK_DEV_TIMEOUT_MMA);
        if (blockIdx.x == 0)
            out[0] = t1 - t0;
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, 512);
}

}  // namespace

extern "C" int32_t ovk_probe_mma_rate(ovk_ctx *ctx, int32_t dtype, double *mac_per_clk_per_sm)
{
    if (!ctx || !mac_per_clk_per_sm)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "ovk_probe_mma_rate: null argument");
    OVK_REFUSE(ctx, dtype != OVK_INT8 && dtype != OVK_FLOAT16, "ovk_probe_mma_rate: dtype %d (int8 or f16)", dtype);
    OVK_REQUIRE(ctx, PROBE_SMEM <= ctx->smem_optin, "ovk_probe_mma_rate: the device has too little shared memory");
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    long long *cycles = reinterpret_cast<long long *>(ctx->params);  // 8 bytes of the per-call parameter block
    const bool f16 = dtype == OVK_FLOAT16;
    if (f16) {
        OVK_CUDA(ctx, cudaFuncSetAttribute(mma_rate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PROBE_SMEM)));
        mma_rate_kernel<1><<<ctx->sm_count, 128, PROBE_SMEM, ctx->stream>>>(cycles, ctx->dev_status);
    } else {
        OVK_CUDA(ctx, cudaFuncSetAttribute(mma_rate_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PROBE_SMEM)));
        mma_rate_kernel<0><<<ctx->sm_count, 128, PROBE_SMEM, ctx->stream>>>(cycles, ctx->dev_status);
    }
    OVK_LAUNCHED(ctx, "mma_rate_probe");
    long long host_cycles = 0;
    OVK_CUDA(ctx, cudaMemcpyAsync(&host_cycles, cycles, sizeof host_cycles, cudaMemcpyDeviceToHost, ctx->stream));
    int32_t rc = ovk_flush(ctx);
    if (rc != OVK_OK)
        return rc;
    OVK_REQUIRE(ctx, host_cycles > 0, "ovk_probe_mma_rate: the probe reported no time");
    const double macs = double(PROBE_ITERS) * PROBE_ACC * (PROBE_KCH / 32) * 128.0 * PROBE_N * (f16 ? 16 : 32);
    *mac_per_clk_per_sm = macs / double(host_cycles);
    return OVK_OK;
}
