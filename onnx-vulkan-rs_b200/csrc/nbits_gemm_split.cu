// MatMulNBits prefill for SMALL quantization blocks (32, 64) with fp16 scales:
// the dequantised weight enters the tensor core exactly, as TWO fp16 numbers.
//
// The general prefill kernel keeps integers (nibble - zero point) in the MMA and
// applies each block's scale to the block's partial sums on the CUDA cores; with
// 32-wide blocks that is one f32 multiply-add per 32 MACs, which the f32 pipes
// cannot deliver at the tensor core's rate.  Here the scale is applied to the
// WEIGHT instead, without rounding it: with t = nibble - zero point (an integer of
// at most 5 bits) and s an fp16 scale,
//     hi = fl16(t * s),   lo = fma16(t, s, -hi)        =>   hi + lo == t * s  exactly
// (the residual of an fp16 product is itself an fp16 number).  Both halves are
// written to shared memory as operand tiles and the token tile is multiplied by
// each: twice the MMAs, no work per block, one accumulator for the whole of K,
// read once per tile.  Products are exact, accumulation is the tensor core's f32.
// (The reference's rounding structure differs - it rounds each block's partial
// sum, shaders/matmul_nbits.rs:359-361 - both are within 1e-6 of the exact value.)
//
// One CTA computes 128 weight columns (UMMA M) x 256 tokens (UMMA N):
//   warp 0       TMA: token tiles [256 x 64 k] fp16 (128B swizzle) and the packed
//                nibbles of the slab [128 rows x 32 bytes], three stages
//   warp 1       tensor memory, MMA issue: eight K=16 MMAs per 64-k slab
//   warps 4-11   unpack: two threads per weight row, 32 k each
//   warps 12-15  epilogue: the tile's accumulator (two in flight), fp16 / f32 store
#include "ovk_internal.h"
#include "umma.cuh"

int32_t ovk_nbits_gemm_prepack(ovk_ctx *ctx, ovk_nbits_weight *w);

namespace {

constexpr int BW = 128, BT = 256, SLAB = 64, STAGES = 3, ACC_RING = 2;
constexpr int W_BYTES = BW * 128, X_BYTES = BT * 128, RAW_BYTES = BW * 32;
constexpr int THREADS = 16 * 32;
constexpr int UNPACK_THREADS = 256;
constexpr long long WAIT_CYCLES = 2000000000ll;

struct SplitParams {
    const float *scales_t;  // [nb_pad, n_pad] (fp16 values held as f32)
    const uint8_t *zp_t;    // [n_pad, zp_pitch] one byte per block
    void *y;
    int M, N;
    int ldy, col0;          // row pitch of y in elements and the column this product's results start at
    int n_pad, zp_pitch;
    int slabs;              // k_pad / 64
    int bs;                 // a power of two, 32 ... 256
    int m_tiles, n_tiles;
    int y_f32;
    int *status;
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
// for warps that wait on someone else's progress: parked, then out of the issue slots for a moment
__device__ __forceinline__ bool wait_parked(uint64_t *bar, uint32_t parity)
{
    if (umma::mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (;;) {
        if (umma::mbar_try_wait_hint(bar, parity, 1000u))
            return true;
        __nanosleep(64);
        if (clock64() - t0 > WAIT_CYCLES)
            return false;
    }
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }

struct UnpackConsts {
    uint32_t m_lo, m_hi, k_lo, k_hi;  // 0x000F000F, 0x00F000F0, 0x64006400, 0x54005400 held in registers
};

// eight nibbles of a permuted word (k ascending in pairs) -> the exact products (n - z) * s as hi + lo
__device__ __forceinline__ void unpack8_split(uint32_t w, uint32_t c_lo, uint32_t c_hi, __half2 s2, const UnpackConsts &u,
                                              uint4 &hi, uint4 &lo)
{
    const uint32_t w8 = w >> 8;
    const __half2 t0 = __hsub2(as_h2(and_or(w, u.m_lo, u.k_lo)), as_h2(c_lo));
    const __half2 t1 = __hsub2(as_h2(and_or(w, u.m_hi, u.k_hi)), as_h2(c_hi));
    const __half2 t2 = __hsub2(as_h2(and_or(w8, u.m_lo, u.k_lo)), as_h2(c_lo));
    const __half2 t3 = __hsub2(as_h2(and_or(w8, u.m_hi, u.k_hi)), as_h2(c_hi));
    const __half2 h0 = __hmul2(t0, s2), h1 = __hmul2(t1, s2), h2 = __hmul2(t2, s2), h3 = __hmul2(t3, s2);
    hi = make_uint4(as_u32(h0), as_u32(h1), as_u32(h2), as_u32(h3));
    lo = make_uint4(as_u32(__hfma2(t0, s2, __hneg2(h0))), as_u32(__hfma2(t1, s2, __hneg2(h1))),
                    as_u32(__hfma2(t2, s2, __hneg2(h2))), as_u32(__hfma2(t3, s2, __hneg2(h3))));
}

__global__ void __launch_bounds__(THREADS, 1)
nbits_gemm_split_kernel(const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmRaw, SplitParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sWh = smem;                       // STAGES x 16 KB: high halves of the weights (UMMA A operand)
    uint8_t *sWl = sWh + STAGES * W_BYTES;     // STAGES x 16 KB: low halves
    uint8_t *sX = sWl + STAGES * W_BYTES;      // STAGES x 32 KB: tokens (UMMA B operand)
    uint8_t *sR = sX + STAGES * X_BYTES;       // STAGES x 4 KB: packed nibbles as loaded
    uint64_t *bars = reinterpret_cast<uint64_t *>(sR + STAGES * RAW_BYTES);
    uint64_t *full_x = bars;                   // TMA landed
    uint64_t *full_w = full_x + STAGES;        // the unpack threads arrived
    uint64_t *empty = full_w + STAGES;         // MMAs of the stage finished
    uint64_t *acc_full = empty + STAGES;       // a tile's sums are complete
    uint64_t *acc_empty = acc_full + ACC_RING; // the four epilogue warps have read them
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + ACC_RING);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            umma::mbar_init(&full_x[s], 1);
            umma::mbar_init(&full_w[s], UNPACK_THREADS / 32);  // one arrival per unpack warp
            umma::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < ACC_RING; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], 4);
        }
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, ACC_RING * BT);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            umma::prefetch_tmap(&tmAct);
            umma::prefetch_tmap(&tmRaw);
            int s = 0;
            uint32_t ph = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * BT, n0 = (tile / p.m_tiles) * BW;
                for (int sl = 0; sl < p.slabs; sl++) {
                    if (!wait_parked(&empty[s], ph ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = total_tiles;
                        break;
                    }
                    umma::mbar_expect_tx(&full_x[s], X_BYTES + RAW_BYTES);
                    umma::tma_load_2d(sX + s * X_BYTES, &tmAct, &full_x[s], sl * SLAB, m0);
                    umma::tma_load_2d(sR + s * RAW_BYTES, &tmRaw, &full_x[s], sl * 32, n0);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // the whole warp runs the loop and stays converged (loop state and descriptors are then
        // warp-uniform values); one elected lane issues the tcgen05 instructions
        {
            const bool leader = umma::elect_one();
            const uint32_t idesc = umma::instr_desc(1 /*f32*/, 0 /*f16*/, 0 /*f16*/, BW, BT);
            const uint32_t desc_hi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
            const uint32_t wh16 = (umma::smem_u32(sWh) >> 4) | (1u << 16), wl16 = (umma::smem_u32(sWl) >> 4) | (1u << 16);
            const uint32_t x16 = (umma::smem_u32(sX) >> 4) | (1u << 16);
            int s = 0, b = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!wait_bounded(&acc_empty[b], acc_ph ^ 1)) {
                    if (leader)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    break;
                }
                umma::tc_fence_after();
                const uint32_t d = tmem_base + uint32_t(b * BT);
                for (int sl = 0; sl < p.slabs; sl++) {
                    // the unpack warps arrive on full_w after they have seen the slab's TMA land
                    // (tokens and nibbles complete the same barrier): one wait covers both operands
                    if (!wait_bounded(&full_w[s], ph)) {
                        if (leader)
                            atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    umma::tc_fence_after();
                    const uint32_t h_lo = wh16 + uint32_t(s) * (W_BYTES >> 4), l_lo = wl16 + uint32_t(s) * (W_BYTES >> 4);
                    const uint32_t x_lo = x16 + uint32_t(s) * (X_BYTES >> 4);
                    if (leader) {
                        umma::mma_f16_lohi(d, h_lo, desc_hi, x_lo, desc_hi, idesc, sl != 0);
                        umma::mma_f16_lohi(d, l_lo, desc_hi, x_lo, desc_hi, idesc, 1u);
#pragma unroll
                        for (int j = 1; j < 4; j++) {
                            umma::mma_f16_lohi(d, h_lo + 2u * j, desc_hi, x_lo + 2u * j, desc_hi, idesc, 1u);
                            umma::mma_f16_lohi(d, l_lo + 2u * j, desc_hi, x_lo + 2u * j, desc_hi, idesc, 1u);
                        }
                        umma::mma_commit(&empty[s]);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok && leader)
                    umma::mma_commit(&acc_full[b]);
                if (++b == ACC_RING) {
                    b = 0;
                    acc_ph ^= 1;
                }
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ------------------------------------------------------------------- unpack
        const int ut = threadIdx.x - 128;
        const int r = ut & 127, half = ut >> 7;  // weight row of the tile, which 32 of the slab's 64 k
        const uint32_t row_off = uint32_t(r) * 128u;
        const uint32_t swz = uint32_t(r & 7);
        UnpackConsts uc;
        asm volatile("mov.u32 %0, 0x000F000F;\n\tmov.u32 %1, 0x00F000F0;\n\tmov.u32 %2, 0x64006400;\n\tmov.u32 %3, 0x54005400;"
                     : "=r"(uc.m_lo), "=r"(uc.m_hi), "=r"(uc.k_lo), "=r"(uc.k_hi));
        const int bs_shift = 31 - __clz(p.bs);  // block sizes are powers of two here
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * BW + r;
            const uint8_t *zrow = p.zp_t + size_t(n) * p.zp_pitch;
            const float *scol = p.scales_t + n;
            // this thread's 32 k of a slab lie in one block; its scale and zero point are fetched one slab ahead
            int blk = (half * 32) >> bs_shift;
            float s_next = scol[size_t(blk) * p.n_pad];
            uint32_t z_next = zrow[blk];
            for (int sl = 0; sl < p.slabs; sl++) {
                const float sc = s_next;
                const uint32_t z = z_next;
                if (sl + 1 < p.slabs) {
                    const int nb = ((sl + 1) * SLAB + half * 32) >> bs_shift;
                    if (nb != blk) {
                        blk = nb;
                        s_next = scol[size_t(blk) * p.n_pad];
                        z_next = zrow[blk];
                    }
                }
                const __half2 s2 = __float2half2_rn(sc);  // the scale IS an fp16 number
                const uint32_t c_lo = z * 0x00010001u + 0x64006400u, c_hi = z * 0x00100010u + 0x54005400u;
                if (!wait_parked(&full_x[s], ph)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                    ok = false;
                    break;
                }
                const uint4 raw = *reinterpret_cast<const uint4 *>(sR + s * RAW_BYTES + r * 32 + half * 16);
                const uint32_t base_h = umma::smem_u32(sWh + s * W_BYTES) + row_off;
                const uint32_t base_l = umma::smem_u32(sWl + s * W_BYTES) + row_off;
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint4 hi, lo;
                    unpack8_split(words[i], c_lo, c_hi, s2, uc, hi, lo);
                    // chunk c (8 k) lands at 16-byte slot c ^ (row & 7): the 128B swizzle
                    const uint32_t slot = ((uint32_t(half * 4 + i)) ^ swz) << 4;
                    sts128(base_h + slot, hi);
                    sts128(base_l + slot, lo);
                }
                umma::fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
                // one arrival per warp: 32 lanes arriving on one barrier word are 32 serialised atomics
                __syncwarp();
                if (lane == 0)
                    umma::mbar_arrive(&full_w[s]);
                if (++s == STAGES) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
    } else if (warp >= 12) {
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;  // tensor-memory lane quarter this warp may read
        int b = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * BW + q * 32 + lane;
            const int m0 = (tile % p.m_tiles) * BT;
            if (ok && !wait_parked(&acc_full[b], acc_ph)) {
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                ok = false;
            }
            umma::tc_fence_after();
            const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * BT);
#pragma unroll 1
            for (int c = 0; c < BT / 32; c++) {
                uint32_t d[32];
                umma::tmem_ld_32x32(taddr + c * 32, d);
                umma::tmem_ld_wait();
                if (c == BT / 32 - 1) {  // everything of this accumulator has been read: hand it back
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        umma::mbar_arrive(&acc_empty[b]);
                }
                // lanes whose column does not exist skip the stores and meet the others at the __syncwarp
                // below: the next tcgen05.ld is warp-wide
                if (ok && n < p.N) {
                    const int mc = m0 + c * 32;
                    if (p.y_f32) {
                        float *y = static_cast<float *>(p.y) + p.col0;
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (mc + j < p.M)
                                y[size_t(mc + j) * p.ldy + n] = __uint_as_float(d[j]);
                    } else {
                        __half *y = static_cast<__half *>(p.y) + p.col0;
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (mc + j < p.M)
                                y[size_t(mc + j) * p.ldy + n] = __float2half_rn(__uint_as_float(d[j]));
                    }
                }
                __syncwarp();
            }
            if (++b == ACC_RING) {
                b = 0;
                acc_ph ^= 1;
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, ACC_RING * BT);
}

size_t split_smem() { return size_t(STAGES) * (2 * W_BYTES + X_BYTES + RAW_BYTES) + 512; }

}  // namespace

// Block sizes 32 and 64 with fp16 scales (an f32 scale would need more than two fp16 terms).
bool ovk_nbits_gemm_split_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w)
{
    const int64_t bs = w->block_size;
    const bool small = bs == 32 || bs == 64;
    return small && w->scales_dtype == OVK_FLOAT16 && split_smem() <= ctx->smem_optin;
}

int32_t ovk_nbits_gemm_split(ovk_ctx *ctx, const ovk_nbits_weight *wc, const void *a, int64_t m, void *y, int32_t y_dtype,
                             int64_t ldy, int64_t col0)
{
    ovk_nbits_weight *w = const_cast<ovk_nbits_weight *>(wc);  // the prefill copy is built lazily
    int32_t rc = ovk_nbits_gemm_prepack(ctx, w);
    if (rc != OVK_OK)
        return rc;
    CUtensorMap tmAct, tmRaw;
    if (!ovk_make_tmap_2d(&tmAct, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, uint64_t(w->k), uint64_t(m), uint64_t(w->k) * 2,
                          SLAB, BT, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !ovk_make_tmap_2d(&tmRaw, w->gemm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->gemm_k_pad / 2),
                          uint64_t(w->gemm_n_pad), uint64_t(w->gemm_k_pad / 2), 32, BW, CU_TENSOR_MAP_SWIZZLE_NONE))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: cuTensorMapEncodeTiled failed");
    SplitParams p = {};
    p.scales_t = w->gemm_scales_t;
    p.zp_t = w->gemm_zp_t;
    p.y = y;
    p.M = int(m);
    p.N = int(w->n);
    p.ldy = int(ldy);
    p.col0 = int(col0);
    p.n_pad = int(w->gemm_n_pad);
    p.zp_pitch = int(w->gemm_zp_pitch);
    p.slabs = int(w->gemm_k_pad / SLAB);
    p.bs = int(w->block_size);
    p.m_tiles = int(ceil_div64(m, BT));
    p.n_tiles = int(w->gemm_n_pad / BW);
    p.y_f32 = y_dtype == OVK_FLOAT;
    p.status = ctx->dev_status;
    OVK_CUDA(ctx, cudaFuncSetAttribute(nbits_gemm_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(split_smem())));
    const int64_t tiles = int64_t(p.m_tiles) * p.n_tiles;
    const unsigned grid = unsigned(std::min<int64_t>(tiles, ctx->sm_count));
    nbits_gemm_split_kernel<<<grid, THREADS, split_smem(), ctx->stream>>>(tmAct, tmRaw, p);
    OVK_LAUNCHED(ctx, "nbits_gemm_tc_split");
    return OVK_OK;
}
