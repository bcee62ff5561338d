// Micro-benchmark: what one thread can get out of tcgen05.mma (cta_group::1).
//
// A single CTA per SM issues a long run of MMAs from one thread over operands
// that sit in shared memory (their values do not matter), with an unrolled,
// division-free loop, and reports cycles per MMA and MACs per clock per SM by
// shape, operand type and swizzle mode.  It answers the design questions of
// the tensor-core kernels in this directory: one issuing thread saturates the
// tensor core for N >= 128; an MMA costs max(48, N/2) cycles at M = 128 whatever
// the swizzle; the issue itself blocks until the tensor core accepts the MMA, so
// every instruction the issuing thread spends between two MMAs is lost.
//
// Build and run (not part of the library):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I .. -I ../../../include \
//        mma_rates.cu -o mma_rates -lcuda && ./mma_rates
#include <cstdio>
#include <cuda_runtime.h>
#include "umma.cuh"

template <int F16, int N, int KCH, int LAYOUT, int NACC, int M>
__global__ void __launch_bounds__(128, 1) bench_kernel(int iters, long long *out, int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x)
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
        const uint32_t idesc = F16 ? umma::instr_desc(1, 0, 0, M, N) : umma::instr_desc(2, 0, 1, M, N);
        constexpr uint32_t sbo = 8 * KCH;
        constexpr uint32_t desc_hi = ((sbo >> 4) & 0x3fffu) | (1u << 14) | (uint32_t(LAYOUT) << 29);
        const uint32_t a_lo = ((umma::smem_u32(smem) >> 4) & 0x3fffu) | (1u << 16);
        const uint32_t b_lo = ((umma::smem_u32(smem + 96 * 1024) >> 4) & 0x3fffu) | (1u << 16);
        constexpr int KSTEPS = KCH / 32;
        const long long t0 = clock64();
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int acc = 0; acc < NACC; acc++) {
#pragma unroll
                for (int j = 0; j < KSTEPS; j++) {
                    if (F16)
                        umma::mma_f16_lohi(tmem_base + acc * N, a_lo + 2u * j, desc_hi, b_lo + 2u * j, desc_hi, idesc, 1u);
                    else
                        umma::mma_i8_lohi(tmem_base + acc * N, a_lo + 2u * j, desc_hi, b_lo + 2u * j, desc_hi, idesc, 1u);
                }
            }
        }
        const long long t1 = clock64();
        umma::mma_commit(&bar);
        bool ok = false;
        for (int i = 0; i < 4000000 && !ok; i++)
            ok = umma::mbar_try_wait(&bar, 0);
        const long long t2 = clock64();
        if (!ok)
            atomicExch(status, 1);
        if (blockIdx.x == 0) {
            out[0] = t1 - t0;
            out[1] = t2 - t0;
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, 512);
}

long long *out;
int *status;

template <int F16, int N, int KCH, int LAYOUT, int NACC, int M>
void run(int grid)
{
    auto k = bench_kernel<F16, N, KCH, LAYOUT, NACC, M>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const int iters = 200;
    k<<<grid, 128, 200 * 1024>>>(iters, out, status);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        printf("error: %s\n", cudaGetErrorString(e));
        exit(1);
    }
    const int count = iters * NACC * (KCH / 32);
    const double macs = double(M) * N * 32 / (F16 ? 2 : 1);
    printf("grid %3d %s M=%3d N=%3d kch=%3d layout=%d nacc=%d: issue %6.1f cyc/MMA, done %6.1f cyc/MMA (%5.0f MAC/clk/SM) status %d\n", grid,
           F16 ? "f16" : "i8 ", M, N, KCH, LAYOUT, NACC, double(out[0]) / count, double(out[1]) / count,
           macs * count / double(out[1]), *status);
}

int main()
{
    cudaMallocManaged(&out, 256);
    cudaMallocManaged(&status, 4);
    *status = 0;
    for (int grid : {1, 148}) {
        run<1, 256, 128, 2, 1, 128>(grid);
        run<1, 256, 128, 2, 2, 128>(grid);
        run<1, 128, 128, 2, 1, 128>(grid);
        run<1, 128, 128, 2, 4, 128>(grid);
        run<1, 64, 128, 2, 1, 128>(grid);
        run<1, 64, 128, 2, 8, 128>(grid);
        run<1, 256, 128, 2, 1, 64>(grid);
        run<0, 256, 128, 2, 1, 128>(grid);
        run<0, 256, 128, 2, 2, 128>(grid);
        run<0, 128, 128, 2, 1, 128>(grid);
        run<0, 64, 128, 2, 1, 128>(grid);
        run<0, 64, 128, 2, 8, 128>(grid);
        run<0, 64, 64, 4, 1, 128>(grid);
        run<0, 64, 64, 4, 8, 128>(grid);
        run<0, 128, 64, 4, 4, 128>(grid);
        run<0, 256, 64, 4, 2, 128>(grid);
        run<0, 64, 32, 6, 8, 128>(grid);
    }
    return 0;
}
