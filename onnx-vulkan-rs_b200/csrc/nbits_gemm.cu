// MatMulNBits prefill (M > 8): dequant-GEMM on tcgen05 with per-block scaling.
//
// The reference has no tiled prefill kernel: its row kernel re-reads the whole
// weight once per row of A (crates/onnx-vulkan-core/src/shaders/
// matmul_nbits.rs:21-25, src/interp.rs:6499-6501).  Here the weight is read
// once per 128-token tile and the products run on the 5th-generation tensor
// cores, while the reference's rounding structure is kept: within a
// quantization block the sum of (nibble - zero point) * a is exact (the
// weights enter the MMA as small integers in fp16, products are exact, f32
// accumulation), and the block's scale multiplies that partial sum in f32 on
// the CUDA cores (matmul_nbits.rs:359-361).  Dequantising to scaled fp16
// weights instead would round every weight and fail the 1e-3 tolerance at
// large K.
//
// One CTA computes 128 weight columns (UMMA M) x 256 tokens (UMMA N), so every
// unpacked weight tile is used by 256 tokens:
//   warp 0      TMA: token tiles [256 x 64 k] fp16 into a 128B-swizzled ring,
//               plus the packed nibbles of the same slab [128 rows x 32 bytes]
//   warp 1      tcgen05.mma kind::f16, four K=16 steps per 64-k slab, one
//               tensor-memory accumulator (256 columns) per quantization block,
//               two in flight
//   warps 4-7   unpack: thread r owns weight row r of the tile; 32 bytes of
//               nibbles per slab -> 64 fp16 integers -> the swizzled operand stage
//   warps 8-15  promotion: tcgen05.ld a block's partial sums (one weight column
//               per thread, 128 tokens per warp), acc += partial * scale[n, block]
//               in registers, final store of Y
// Weight columns sit on tensor-memory LANES so the scale is one scalar per thread.
// The promotion warps hold 128 accumulators each: the register file is
// re-divided between the warpgroups with setmaxnreg.
#include <cstdlib>

#include "ovk_internal.h"
#include "umma.cuh"

namespace {

constexpr int BW = 128;    // weight columns per tile (UMMA M)
constexpr int BT = 256;    // tokens per tile (UMMA N)
constexpr int SLAB = 64;   // k per stage: 128 bytes of fp16
constexpr int STAGES = 4;
constexpr int ACC_RING = 2;
constexpr int A_BYTES = BW * 128, B_BYTES = BT * 128;
constexpr int RAW_BYTES = BW * 32;  // packed nibbles of one slab: 32 bytes per weight row
constexpr int THREADS = 16 * 32;  // four warpgroups: control, unpack, promotion x2
constexpr long long WAIT_CYCLES = 2000000000ll;

struct GemmParams {
    const uint8_t *wq;     // [n_pad, k_pad/2] nibble-permuted copy
    const float *scales_t; // [nb_pad, n_pad]
    const uint8_t *zp_t;   // [n_pad, zp_pitch] one byte per block, rows padded to 8
    void *y;
    int M, N, K;
    int k_pad, n_pad, n_blocks;
    int zp_pitch;
    int slabs;             // k_pad / 64
    int bs;                // block size (32, 64, 128, 256)
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

// For warps that wait on someone else's progress: the hardware parks the
// thread (up to a microsecond per attempt) instead of letting it spin in the
// issue slots of the warp that feeds the tensor core.
__device__ __forceinline__ bool wait_parked(uint64_t *bar, uint32_t parity)
{
    if (umma::mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (;;) {
        if (umma::mbar_try_wait_hint(bar, parity, 1000u))
            return true;
        __nanosleep(64);  // out of the issue slots of the thread that feeds the tensor core
        if (clock64() - t0 > WAIT_CYCLES)
            return false;
    }
}

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b)
{
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ uint4 ldg_nc16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// eight nibbles of a permuted word -> 8 fp16 integers (nibble - z), k ascending
struct UnpackConsts {
    uint32_t m_lo, m_hi, k_lo, k_hi;  // 0x000F000F, 0x00F000F0, 0x64006400, 0x54005400 held in registers
};
// (a & b) | c with all operands in registers: one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint4 unpack8(uint32_t w, uint32_t c_lo, uint32_t c_hi, const UnpackConsts &u)
{
    const uint32_t w8 = w >> 8;
    uint4 o;
    o.x = h2_sub(and_or(w, u.m_lo, u.k_lo), c_lo);
    o.y = h2_sub(and_or(w, u.m_hi, u.k_hi), c_hi);
    o.z = h2_sub(and_or(w8, u.m_lo, u.k_lo), c_lo);
    o.w = h2_sub(and_or(w8, u.m_hi, u.k_hi), c_hi);
    return o;
}

__global__ void __launch_bounds__(THREADS, 1)
nbits_gemm_kernel(const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmRaw, GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sW = smem;                       // STAGES x 16 KB: unpacked weights (UMMA A operand)
    uint8_t *sX = smem + STAGES * A_BYTES;    // STAGES x 16 KB: tokens (UMMA B operand)
    uint8_t *sR = sX + STAGES * B_BYTES;      // STAGES x 4 KB: packed nibbles as loaded
    uint64_t *bars = reinterpret_cast<uint64_t *>(sR + STAGES * RAW_BYTES);
    uint64_t *full_x = bars;                  // TMA landed
    uint64_t *full_w = full_x + STAGES;       // 128 unpack threads arrived
    uint64_t *empty = full_w + STAGES;        // MMAs of the stage finished
    uint64_t *acc_full = empty + STAGES;      // a block's partial sums are complete
    uint64_t *acc_empty = acc_full + ACC_RING;// all 8 promotion warps have read them
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + ACC_RING);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            umma::mbar_init(&full_x[s], 1);
            umma::mbar_init(&full_w[s], 128);
            umma::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < ACC_RING; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], 8);
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
    const int blocks_per_slab = p.bs >= SLAB ? 1 : SLAB / p.bs;  // 2 when block_size is 32
    const int slabs_per_block = p.bs >= SLAB ? p.bs / SLAB : 1;

    // 512 threads x 128 registers fill the register file; control and unpack warps give
    // registers back, the promotion warps take them (40*128 + 56*128 + 208*256 = 65536)
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ------------------------------------------------------------ tokens by TMA
        if (lane == 0) {
            umma::prefetch_tmap(&tmAct);
            umma::prefetch_tmap(&tmRaw);
            int seq = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * BT;
                const int n0 = (tile / p.m_tiles) * BW;
                for (int sl = 0; sl < p.slabs; sl++, seq++) {
                    const int s = seq % STAGES;
                    if (!wait_parked(&empty[s], ((seq / STAGES) & 1) ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = total_tiles;
                        break;
                    }
                    umma::mbar_expect_tx(&full_x[s], B_BYTES + RAW_BYTES);
                    umma::tma_load_2d(sX + s * B_BYTES, &tmAct, &full_x[s], sl * SLAB, m0);
                    umma::tma_load_2d(sR + s * RAW_BYTES, &tmRaw, &full_x[s], sl * 32, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issue
        // One thread feeds the tensor core, so its loop is kept to a few instructions per
        // MMA: descriptor high words are constants, low words advance by additions, block
        // boundaries are tracked with counters instead of divisions.
        if (lane == 0) {
            const uint32_t idesc = umma::instr_desc(1 /*f32*/, 0 /*f16*/, 0 /*f16*/, BW, BT);
            const uint32_t desc_hi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
            const uint32_t w16 = umma::smem_u32(sW) >> 4, x16 = umma::smem_u32(sX) >> 4;
            int s = 0, b = 0, slab_in_block = 0;
            uint32_t ph = 0, acc_ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int sl = 0; sl < p.slabs && ok; sl++) {
                    if (!wait_bounded(&full_x[s], ph) || !wait_bounded(&full_w[s], ph)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                        ok = false;
                        break;
                    }
                    umma::tc_fence_after();
                    const uint32_t w_lo = ((w16 + uint32_t(s) * (A_BYTES >> 4)) & 0x3fffu) | (1u << 16);
                    const uint32_t x_lo = ((x16 + uint32_t(s) * (B_BYTES >> 4)) & 0x3fffu) | (1u << 16);
                    if (p.bs >= SLAB) {
                        const bool first = slab_in_block == 0;
                        if (first) {  // the promotion warps must have drained this accumulator
                            if (!wait_bounded(&acc_empty[b], acc_ph ^ 1)) {
                                atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            umma::tc_fence_after();
                        }
                        const uint32_t d = tmem_base + uint32_t(b * BT);
                        umma::mma_f16_lohi(d, w_lo, desc_hi, x_lo, desc_hi, idesc, first ? 0u : 1u);
                        umma::mma_f16_lohi(d, w_lo + 2, desc_hi, x_lo + 2, desc_hi, idesc, 1u);
                        umma::mma_f16_lohi(d, w_lo + 4, desc_hi, x_lo + 4, desc_hi, idesc, 1u);
                        umma::mma_f16_lohi(d, w_lo + 6, desc_hi, x_lo + 6, desc_hi, idesc, 1u);
                        umma::mma_commit(&empty[s]);
                        if (++slab_in_block == slabs_per_block) {
                            umma::mma_commit(&acc_full[b]);
                            slab_in_block = 0;
                            if (++b == ACC_RING) {
                                b = 0;
                                acc_ph ^= 1;
                            }
                        }
                    } else {
                        // block_size 32: two blocks per slab, two K=16 steps each
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (!wait_bounded(&acc_empty[b], acc_ph ^ 1)) {
                                atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            umma::tc_fence_after();
                            const uint32_t d = tmem_base + uint32_t(b * BT);
                            umma::mma_f16_lohi(d, w_lo + 4 * h, desc_hi, x_lo + 4 * h, desc_hi, idesc, 0u);
                            umma::mma_f16_lohi(d, w_lo + 4 * h + 2, desc_hi, x_lo + 4 * h + 2, desc_hi, idesc, 1u);
                            umma::mma_commit(&acc_full[b]);
                            if (++b == ACC_RING) {
                                b = 0;
                                acc_ph ^= 1;
                            }
                        }
                        umma::mma_commit(&empty[s]);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    }
    } else if (warp < 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        // ------------------------------------------------------------------- unpack
        const int r = (warp - 4) * 32 + lane;  // weight row of the tile
        const uint32_t row_off = uint32_t(r) * 128u;
        const uint32_t swz = uint32_t(r & 7);
        UnpackConsts uc;
        asm volatile("mov.u32 %0, 0x000F000F;\n\tmov.u32 %1, 0x00F000F0;\n\tmov.u32 %2, 0x64006400;\n\tmov.u32 %3, 0x54005400;"
                     : "=r"(uc.m_lo), "=r"(uc.m_hi), "=r"(uc.k_lo), "=r"(uc.k_hi));
        int seq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * BW + r;
            // zero points: 8 blocks per 64-bit load, fetched one group ahead
            const uint2 *zrow = reinterpret_cast<const uint2 *>(p.zp_t + size_t(n) * p.zp_pitch);
            uint2 zcur = zrow[0], znext = zcur;
            int zgroup = 0;
            for (int sl = 0; sl < p.slabs; sl++, seq++) {
                const int blk0 = (sl * SLAB) / p.bs;
                if ((blk0 >> 3) != zgroup) {
                    zgroup = blk0 >> 3;
                    zcur = znext;
                }
                if ((blk0 & 7) == 0 && (zgroup + 1) * 8 < p.zp_pitch && (sl * SLAB) % p.bs == 0)
                    znext = zrow[zgroup + 1];
                const uint64_t zbits = (uint64_t(zcur.y) << 32) | zcur.x;
                const uint32_t z0 = uint32_t(zbits >> (8 * (blk0 & 7))) & 0xffu;
                const uint32_t z1 = blocks_per_slab == 2 ? uint32_t(zbits >> (8 * ((blk0 + 1) & 7))) & 0xffu : z0;
                const uint32_t lo0 = z0 * 0x00010001u + 0x64006400u, hi0 = z0 * 0x00100010u + 0x54005400u;
                const uint32_t lo1 = z1 * 0x00010001u + 0x64006400u, hi1 = z1 * 0x00100010u + 0x54005400u;
                const int s = seq % STAGES;
                // the nibbles have landed; the producer waited for the stage to be free before loading them
                if (!wait_parked(&full_x[s], (seq / STAGES) & 1)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                    ok = false;
                    break;
                }
                const uint4 *raw = reinterpret_cast<const uint4 *>(sR + s * RAW_BYTES + r * 32);
                const uint4 c0 = raw[0], c1 = raw[1];
                const uint32_t base = umma::smem_u32(sW + s * A_BYTES) + row_off;
                // chunk c (8 k) lands at 16-byte slot c ^ (row & 7): the 128B swizzle
                sts128(base + ((0u ^ swz) << 4), unpack8(c0.x, lo0, hi0, uc));
                sts128(base + ((1u ^ swz) << 4), unpack8(c0.y, lo0, hi0, uc));
                sts128(base + ((2u ^ swz) << 4), unpack8(c0.z, lo0, hi0, uc));
                sts128(base + ((3u ^ swz) << 4), unpack8(c0.w, lo0, hi0, uc));
                sts128(base + ((4u ^ swz) << 4), unpack8(c1.x, lo1, hi1, uc));
                sts128(base + ((5u ^ swz) << 4), unpack8(c1.y, lo1, hi1, uc));
                sts128(base + ((6u ^ swz) << 4), unpack8(c1.z, lo1, hi1, uc));
                sts128(base + ((7u ^ swz) << 4), unpack8(c1.w, lo1, hi1, uc));
                umma::fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
                umma::mbar_arrive(&full_w[s]);
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ---------------------------------------------------------------- promotion
        const int q = warp & 3;            // tensor-memory lane quarter this warp may read
        const int half = (warp - 8) >> 2;  // which 128 of the 256 tokens
        int acc_seq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * BW + q * 32 + lane;
            const int m0 = (tile % p.m_tiles) * BT + half * 128;
            float acc[128];
#pragma unroll
            for (int j = 0; j < 128; j++)
                acc[j] = 0.0f;
            float scale = p.scales_t[n];
            for (int blk = 0; blk < p.n_blocks; blk++, acc_seq++) {
                const float scale_next = blk + 1 < p.n_blocks ? p.scales_t[size_t(blk + 1) * p.n_pad + n] : 0.0f;
                const int b = acc_seq % ACC_RING;
                if (ok && !wait_parked(&acc_full[b], (acc_seq / ACC_RING) & 1)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    ok = false;
                }
                umma::tc_fence_after();
                const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * BT + half * 128);
                // two reads of 64 columns: both loads of a pair are in flight together, and the
                // accumulator goes back to the tensor core after two load latencies instead of four
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t d0[32], d1[32];
                    umma::tmem_ld_32x32(taddr + c * 64, d0);
                    umma::tmem_ld_32x32(taddr + c * 64 + 32, d1);
                    umma::tmem_ld_wait();
                    if (c == 1) {  // everything of this accumulator has been read: hand it back
                        umma::tc_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            umma::mbar_arrive(&acc_empty[b]);
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        acc[c * 64 + j] = fmaf(__uint_as_float(d0[j]), scale, acc[c * 64 + j]);
                        acc[c * 64 + 32 + j] = fmaf(__uint_as_float(d1[j]), scale, acc[c * 64 + 32 + j]);
                    }
                }
                scale = scale_next;
            }
            if (ok && n < p.N) {
                // the MMA thread can run only two blocks ahead while this store lasts: a row
                // pointer stepped by N and no bound test when all 128 token rows exist
                const bool whole = m0 + 128 <= p.M;
                if (p.y_f32) {
                    float *y = static_cast<float *>(p.y) + size_t(m0) * p.N + n;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 128; j++, y += p.N)
                            *y = acc[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 128; j++, y += p.N)
                            if (m0 + j < p.M)
                                *y = acc[j];
                    }
                } else {
                    __half *y = static_cast<__half *>(p.y) + size_t(m0) * p.N + n;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < 128; j++, y += p.N)
                            *y = __float2half_rn(acc[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 128; j++, y += p.N)
                            if (m0 + j < p.M)
                                *y = __float2half_rn(acc[j]);
                    }
                }
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, ACC_RING * BT);
}

// ------------------------------------------------------------------- prepack
// nibble k of a word moves to position {0,4,1,5,2,6,3,7}[k & 7] so that the
// two-mask unpack yields k-ascending pairs; rows and K are zero padded.
__global__ void __launch_bounds__(256)
nbits_gemm_pack_kernel(const uint32_t *__restrict__ src_w, const void *__restrict__ src_s, int scale_f32,
                       const uint8_t *__restrict__ src_z, uint32_t *__restrict__ dst_w, float *__restrict__ dst_s,
                       uint8_t *__restrict__ dst_z, int N, int n_pad, int n_blocks, int nb_pad, int zp_pitch,
                       int words_src, int words_dst)
{
    const int64_t total_w = int64_t(n_pad) * words_dst;
    const int64_t total_s = int64_t(nb_pad) * n_pad;
    const int zp_row = (n_blocks + 1) / 2;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total_w + total_s;
         i += int64_t(gridDim.x) * blockDim.x) {
        if (i < total_w) {
            const int n = int(i / words_dst), w = int(i % words_dst);
            uint32_t v = 0;
            if (n < N && w < words_src)
                v = src_w[int64_t(n) * words_src + w];
            uint32_t o = 0;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int pos = (k >> 1) + 4 * (k & 1);
                o |= ((v >> (4 * k)) & 15u) << (4 * pos);
            }
            dst_w[i] = o;
        } else {
            const int64_t j = i - total_w;
            const int blk = int(j / n_pad), n = int(j % n_pad);
            float s = 0.0f;
            uint32_t z = 0;
            if (n < N && blk < n_blocks) {
                s = scale_f32 ? static_cast<const float *>(src_s)[int64_t(n) * n_blocks + blk]
                              : __half2float(static_cast<const __half *>(src_s)[int64_t(n) * n_blocks + blk]);
                z = src_z ? (src_z[int64_t(n) * zp_row + blk / 2] >> (4 * (blk & 1))) & 15u : 8u;
            }
            dst_s[j] = s;
            dst_z[size_t(n) * zp_pitch + blk] = uint8_t(z);
        }
    }
}

size_t gemm_smem() { return size_t(STAGES) * (A_BYTES + B_BYTES + RAW_BYTES) + 512; }

}  // namespace

// The prefill copy: nibble-permuted [n_pad, k_pad/2] weights, f32 scales and
// (transposed to [block, n_pad]) and one zero-point byte per block, row major.  Built on the first prefill
// call (as the reference builds packed weights at first use, src/cache.rs:231).
int32_t ovk_nbits_gemm_prepack(ovk_ctx *ctx, ovk_nbits_weight *w)
{
    if (w->gemm_w)
        return OVK_OK;
    const int64_t n_pad = ceil_div64(w->n, BW) * BW;
    const int64_t k_src = w->n_blocks * w->block_size;  // the operator layout pads K to whole blocks
    const int64_t k_pad = ceil_div64(k_src, SLAB) * SLAB;
    const int64_t nb_pad = ceil_div64(k_pad, w->block_size);
    const size_t wbytes = size_t(n_pad) * size_t(k_pad / 2);
    const size_t sbytes = size_t(nb_pad) * n_pad * sizeof(float);
    const int64_t zp_pitch = ceil_div64(nb_pad, 8) * 8 + 8;  // one spare group so the look-ahead load stays inside
    const size_t zbytes = size_t(n_pad) * zp_pitch;
    uint8_t *blob = nullptr;
    OVK_CUDA(ctx, cudaMalloc(&blob, wbytes + sbytes + zbytes + 256));
    OVK_CUDA(ctx, cudaMemsetAsync(blob + wbytes + sbytes, 0, zbytes, ctx->stream));
    uint32_t *dw = reinterpret_cast<uint32_t *>(blob);
    float *ds = reinterpret_cast<float *>(blob + wbytes);
    uint8_t *dz = blob + wbytes + sbytes;
    const int64_t total = n_pad * (k_pad / 8) + nb_pad * n_pad;
    const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(total, 256), int64_t(ctx->sm_count) * 16));
    nbits_gemm_pack_kernel<<<blocks, 256, 0, ctx->stream>>>(
        reinterpret_cast<const uint32_t *>(w->b), w->scales, w->scales_dtype == OVK_FLOAT, w->zp, dw, ds, dz,
        int(w->n), int(n_pad), int(w->n_blocks), int(nb_pad), int(zp_pitch), int(k_src / 8), int(k_pad / 8));
    ctx->last_kernel = "nbits_gemm_pack";
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(blob);
        return ovk_fail(ctx, OVK_BACKEND, "nbits_gemm_pack: %s", cudaGetErrorString(e));
    }
    w->gemm_w = blob;
    w->gemm_scales_t = ds;
    w->gemm_zp_t = dz;
    w->gemm_k_pad = k_pad;
    w->gemm_n_pad = n_pad;
    w->gemm_zp_pitch = zp_pitch;
    return OVK_OK;
}

// fp16 activations with 16-byte aligned rows (TMA), block sizes that are whole
// MMA steps, more rows than the decode kernel takes.
bool ovk_nbits_gemm_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, int32_t a_dtype,
                            int32_t y_dtype, const void *a, const void *y)
{
    (void)y_dtype;
    const int64_t bs = w->block_size;
    return m > 8 && a_dtype == OVK_FLOAT16 && (bs == 32 || bs == 64 || bs == 128 || bs == 256) &&
           (w->k % 8) == 0 && aligned_to(a, 16) && aligned_to(y, 4) && aligned_to(w->b, 4) &&
           m < (int64_t(1) << 31) && gemm_smem() <= ctx->smem_optin &&
           aligned_to(w->scales, w->scales_dtype == OVK_FLOAT ? 4 : 2);
}

bool ovk_nbits_gemm_split_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w);
int32_t ovk_nbits_gemm_split(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int64_t m, void *y, int32_t y_dtype);

int32_t ovk_nbits_gemm(ovk_ctx *ctx, const ovk_nbits_weight *wc, const void *a, int32_t a_dtype, int64_t m,
                       void *y, int32_t y_dtype)
{
    (void)a_dtype;
    // small blocks with fp16 scales: the scale goes into the weight (exactly, as two fp16 terms)
    static const char *pin = getenv("OVK_NBITS_GEMM");  // "blocks" pins the per-block kernel (for comparisons)
    if (!(pin && pin[0] == 'b') && ovk_nbits_gemm_split_applies(ctx, wc))
        return ovk_nbits_gemm_split(ctx, wc, a, m, y, y_dtype);
    ovk_nbits_weight *w = const_cast<ovk_nbits_weight *>(wc);  // the prefill copy is built lazily
    int32_t rc = ovk_nbits_gemm_prepack(ctx, w);
    if (rc != OVK_OK)
        return rc;
    CUtensorMap tmAct;
    if (!ovk_make_tmap_2d(&tmAct, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, uint64_t(w->k), uint64_t(m), uint64_t(w->k) * 2,
                          SLAB, BT, CU_TENSOR_MAP_SWIZZLE_128B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: cuTensorMapEncodeTiled failed for A");
    CUtensorMap tmRaw;
    if (!ovk_make_tmap_2d(&tmRaw, w->gemm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->gemm_k_pad / 2),
                          uint64_t(w->gemm_n_pad), uint64_t(w->gemm_k_pad / 2), 32, BW, CU_TENSOR_MAP_SWIZZLE_NONE))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: cuTensorMapEncodeTiled failed for the packed weight");
    GemmParams p = {};
    p.wq = static_cast<const uint8_t *>(w->gemm_w);
    p.scales_t = w->gemm_scales_t;
    p.zp_t = w->gemm_zp_t;
    p.y = y;
    p.M = int(m);
    p.N = int(w->n);
    p.K = int(w->k);
    p.k_pad = int(w->gemm_k_pad);
    p.n_pad = int(w->gemm_n_pad);
    p.n_blocks = int(w->gemm_k_pad / w->block_size);
    p.zp_pitch = int(w->gemm_zp_pitch);
    p.slabs = int(w->gemm_k_pad / SLAB);
    p.bs = int(w->block_size);
    p.m_tiles = int(ceil_div64(m, BT));
    p.n_tiles = int(w->gemm_n_pad / BW);
    p.y_f32 = y_dtype == OVK_FLOAT;
    p.status = ctx->dev_status;
    OVK_CUDA(ctx, cudaFuncSetAttribute(nbits_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem())));
    const int64_t tiles = int64_t(p.m_tiles) * p.n_tiles;
    const unsigned grid = unsigned(std::min<int64_t>(tiles, ctx->sm_count));
    nbits_gemm_kernel<<<grid, THREADS, gemm_smem(), ctx->stream>>>(tmAct, tmRaw, p);
    OVK_LAUNCHED(ctx, "nbits_gemm_tc");
    return OVK_OK;
}
