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
// One CTA computes 128 weight columns (UMMA M) x up to 192 tokens (UMMA N):
//   warp 0      TMA: token tiles [192 x 64 k] fp16 into a 128B-swizzled ring of
//               eight stages, plus the packed nibbles of the same slab
//               [128 rows x 32 bytes]
//   warps 1-2   tcgen05.mma kind::f16, four K=16 steps per 64-k slab, the A
//               operand read from tensor memory; one accumulator (192 columns)
//               per quantization block, two to four in flight, blocks alternate
//               between the two issuing warps
//   warps 4-11  unpack, two groups of four warps on alternate slabs: thread r
//               owns weight row r of the tile; 32 bytes of nibbles per slab ->
//               64 fp16 integers -> one tcgen05.st of 32 columns into the
//               tensor-memory ring of four A stages
//   warps 12-19 promotion: tcgen05.ld a block's partial sums (one weight column
//               per thread, 96 tokens per warp), acc += partial * scale[n, block]
//               in registers, final store of Y
// The unpacked weights never touch shared memory: they go from registers to
// tensor memory and the MMA takes its A operand from there.  At equal token
// width that was 18 % faster than writing them to a swizzled shared-memory stage
// (which the MMA then reads back at 32 bytes per clock next to 64 for the
// tokens); the price is the tile width, since the A stages share the 512 columns
// with the accumulators: 384 + 4 x 32 (two accumulators of 192 tokens, three of
// 128 or four of 96, by the tile width of the launch).
// What sets the pace is not the tensor core (384 clocks per slab at 192 tokens)
// but the chains of long-latency steps each role runs per slab - barrier polls of
// ~100 clocks, tcgen05.st, fences, commits: ~700 clocks for an unpack warp, ~800
// for an issuing warp, measured with clock64 stamps.  Hence two issuing warps,
// two unpack groups, a store that is announced one slab late, and one barrier
// arrival per warp.  TMA itself needs ~500 clocks for the 28 KB of a slab
// (57 bytes per clock per SM, 14 TB/s over the GPU), the next ceiling.
// Weight columns sit on tensor-memory LANES so the scale is one scalar per thread.
// The promotion warps hold 96 accumulators each: the register file is
// re-divided between the warpgroups with setmaxnreg.
#include <cstdlib>

#include "ovk_internal.h"
#include "umma.cuh"

namespace {

constexpr int BW = 128;    // weight columns per tile (UMMA M)
constexpr int BT = 192;    // most tokens per tile (UMMA N)
constexpr int HALF = BT / 2;  // token rows per promotion warp
constexpr int SLAB = 64;   // k per stage: 128 bytes of fp16
constexpr int STAGES = 8;    // shared-memory ring: tokens + packed nibbles of a slab (TMA)
constexpr int A_STAGES = 4;  // tensor-memory ring: unpacked weights of a slab
constexpr int ACC_RING = 4;   // most accumulators in flight: 2 x 192, 3 x 128 or 4 x 96 columns
constexpr int B_BYTES = BT * 128;
constexpr int A_COLS = 32;                        // tensor-memory columns of one A stage: 64 k as fp16 pairs
constexpr int A_BASE = 2 * BT;                    // the A stages follow the accumulators
constexpr int TMEM_COLS = 512;
static_assert(A_BASE + A_STAGES * A_COLS <= TMEM_COLS, "tensor memory: accumulators + A stages");
constexpr int RAW_BYTES = BW * 32;  // packed nibbles of one slab: 32 bytes per weight row
constexpr int THREADS = 20 * 32;  // five warpgroups: control, unpack x2, promotion x2
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
    int bt;                // tokens per tile: a multiple of 32 up to BT, chosen per launch
    int ring, acc_stride;  // accumulators in flight and their distance in tensor-memory columns
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
    uint8_t *sX = smem;                       // STAGES x 24 KB: tokens (UMMA B operand)
    uint8_t *sR = sX + STAGES * B_BYTES;      // STAGES x 4 KB: packed nibbles as loaded
    uint64_t *bars = reinterpret_cast<uint64_t *>(sR + STAGES * RAW_BYTES);
    uint64_t *full_x = bars;                  // TMA landed
    uint64_t *full_w = full_x + STAGES;       // [A_STAGES] the four unpack warps arrived
    uint64_t *empty = full_w + A_STAGES;      // [STAGES] MMAs of the slab finished: its shared-memory AND its A stage are free
    uint64_t *acc_full = empty + STAGES;      // a block's partial sums are complete
    uint64_t *acc_empty = acc_full + ACC_RING;// all 8 promotion warps have read them
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + ACC_RING);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            umma::mbar_init(&full_x[s], 1);
            umma::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < A_STAGES; s++)
            umma::mbar_init(&full_w[s], 4);  // one arrival per unpack warp
        for (int b = 0; b < ACC_RING; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], 8);
        }
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, TMEM_COLS);
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.m_tiles * p.n_tiles;
    const int blocks_per_slab = p.bs >= SLAB ? 1 : SLAB / p.bs;  // 2 when block_size is 32
    const int slabs_per_block = p.bs >= SLAB ? p.bs / SLAB : 1;

    // 640 threads start with 96 registers each; control and unpack warps give registers back,
    // the promotion warps take them (40*128 + 64*256 + 152*256 = 60416 of the 61440)
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
        // ------------------------------------------------------------ tokens by TMA
        if (lane == 0) {
            umma::prefetch_tmap(&tmAct);
            umma::prefetch_tmap(&tmRaw);
            int seq = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile % p.m_tiles) * p.bt;
                const int n0 = (tile / p.m_tiles) * BW;
                for (int sl = 0; sl < p.slabs; sl++, seq++) {
                    const int s = seq % STAGES;
                    if (!wait_parked(&empty[s], ((seq / STAGES) & 1) ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = total_tiles;
                        break;
                    }
                    umma::mbar_expect_tx(&full_x[s], uint32_t(p.bt) * 128u + RAW_BYTES);
                    umma::tma_load_2d(sX + s * B_BYTES, &tmAct, &full_x[s], sl * SLAB, m0);
                    umma::tma_load_2d(sR + s * RAW_BYTES, &tmRaw, &full_x[s], sl * 32, n0);
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------------------------------------------ MMA issue
        // A timeline of this loop showed ~800 clocks of its own instructions per slab (barrier
        // polls, fences, commits: a chain of shared-memory and uniform-datapath latencies), of
        // which the four MMAs are 80 - the tensor core, which needs 384, was waiting for its
        // issuer.  So two warps issue, on two schedulers: warp 1 takes the even quantization
        // blocks, warp 2 the odd ones.  Each commit covers the MMAs of its own thread, a block's
        // accumulator has one writer, and the sums do not depend on how the two streams
        // interleave.
        // The whole warp runs the loop and stays converged; one elected lane issues the
        // tcgen05 instructions, so loop state and descriptors are warp-uniform values.
        const int me = warp - 1;
        const int issuers = p.bs >= SLAB ? 2 : 1;  // smaller blocks: two per slab, one issuer
        if (me < issuers) {
            const bool leader = umma::elect_one();
            const uint32_t idesc = umma::instr_desc(1 /*f32*/, 0 /*f16*/, 0 /*f16*/, BW, p.bt);
            const uint32_t desc_hi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
            const uint32_t x16 = umma::smem_u32(sX) >> 4;
            int s = 0, a = 0, b = 0, slab_in_block = 0, owner = 0;
            uint32_t a_ph = 0, acc_ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                for (int sl = 0; sl < p.slabs && ok; sl++) {
                    const uint32_t a_t = tmem_base + uint32_t(A_BASE + a * A_COLS);  // 8 columns per K=16 step
                    const uint32_t x_lo = ((x16 + uint32_t(s) * (B_BYTES >> 4)) & 0x3fffu) | (1u << 16);
                    if (p.bs >= SLAB) {
                        const bool first = slab_in_block == 0;
                        const bool last = ++slab_in_block == slabs_per_block;
                        // The unpack warps arrive on full_w after they have seen the slab's TMA land
                        // (tokens and nibbles complete the same barrier), so this one wait covers both
                        // operands.  Both issuers wait for every slab, also the other one's: a parity
                        // wait is only meaningful one phase behind its barrier, and a warp that ran
                        // ahead over the slabs it skips could fall two behind.
                        if (!wait_bounded(&full_w[a], a_ph)) {
                            if (leader)
                                atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                            ok = false;
                            break;
                        }
                        if (owner == me) {
                            if (first && !wait_bounded(&acc_empty[b], acc_ph ^ 1)) {  // drained by the promotion warps
                                if (leader)
                                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            umma::tc_fence_after();
                            const uint32_t d = tmem_base + uint32_t(b * p.acc_stride);
                            if (leader) {
                                umma::mma_f16_ts(d, a_t, x_lo, desc_hi, idesc, first ? 0u : 1u);
                                umma::mma_f16_ts(d, a_t + 8, x_lo + 2, desc_hi, idesc, 1u);
                                umma::mma_f16_ts(d, a_t + 16, x_lo + 4, desc_hi, idesc, 1u);
                                umma::mma_f16_ts(d, a_t + 24, x_lo + 6, desc_hi, idesc, 1u);
                                umma::mma_commit(&empty[s]);
                                if (last)
                                    umma::mma_commit(&acc_full[b]);
                            }
                        }
                        if (last) {
                            slab_in_block = 0;
                            owner ^= issuers - 1;  // blocks alternate between the issuing warps
                            if (++b == p.ring) {
                                b = 0;
                                acc_ph ^= 1;
                            }
                        }
                    } else {
                        // block_size 32: two blocks per slab, two K=16 steps each
                        if (!wait_bounded(&full_w[a], a_ph)) {
                            if (leader)
                                atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                            ok = false;
                            break;
                        }
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (!wait_bounded(&acc_empty[b], acc_ph ^ 1)) {
                                if (leader)
                                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                                ok = false;
                                break;
                            }
                            umma::tc_fence_after();
                            const uint32_t d = tmem_base + uint32_t(b * p.acc_stride);
                            if (leader) {
                                umma::mma_f16_ts(d, a_t + 16 * h, x_lo + 4 * h, desc_hi, idesc, 0u);
                                umma::mma_f16_ts(d, a_t + 16 * h + 8, x_lo + 4 * h + 2, desc_hi, idesc, 1u);
                                umma::mma_commit(&acc_full[b]);
                            }
                            if (++b == p.ring) {
                                b = 0;
                                acc_ph ^= 1;
                            }
                        }
                        if (leader)
                            umma::mma_commit(&empty[s]);
                    }
                    if (++s == STAGES)
                        s = 0;
                    if (++a == A_STAGES) {
                        a = 0;
                        a_ph ^= 1;
                    }
                }
            }
        }
    }
    } else if (warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
        // ------------------------------------------------------------------- unpack
        // two groups of four warps take alternate slabs (warps 4-7 the even ones, 8-11 the odd ones);
        // within a group, warp w owns the 32 weight rows of tensor-memory lane quarter w % 4
        const int group = (warp - 4) >> 2;
        const int r = (warp & 3) * 32 + lane;  // weight row of the tile = tensor-memory lane
        const uint32_t a_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16) + uint32_t(A_BASE);
        UnpackConsts uc;
        asm volatile("mov.u32 %0, 0x000F000F;\n\tmov.u32 %1, 0x00F000F0;\n\tmov.u32 %2, 0x64006400;\n\tmov.u32 %3, 0x54005400;"
                     : "=r"(uc.m_lo), "=r"(uc.m_hi), "=r"(uc.k_lo), "=r"(uc.k_hi));
        // One slab is ~120 instructions per thread, but as a chain (barrier poll, shared-memory
        // load, unpack, tensor-memory store, wait for the store, arrive) it took ~650 clocks, and
        // all four warps work on the same slab: that, not the tensor core, set the pace.  So the
        // store of slab j is announced only after slab j + 1 has been unpacked - by then it has
        // completed and the wait costs nothing - and block indices are shifts, not divisions.
        const int bs_shift = 31 - __clz(p.bs);  // block sizes are powers of two
        int seq = 0;       // global index of the current tile's first slab
        int pending = -1;  // A stage stored to but not yet announced
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, seq += p.slabs) {
            const int n = (tile / p.m_tiles) * BW + r;
            // zero points: one byte per block, fetched one slab of this group ahead
            const uint8_t *zrow = p.zp_t + size_t(n) * p.zp_pitch;
            auto zero_points = [&](int sl) -> uint32_t {
                const int blk = (sl * SLAB) >> bs_shift;
                const uint32_t z0 = zrow[blk];
                return z0 | (blocks_per_slab == 2 ? uint32_t(zrow[blk + 1]) << 8 : z0 << 8);
            };
            int sl = (seq ^ group) & 1;  // the first slab of this tile that this group takes
            uint32_t z_next = sl < p.slabs ? zero_points(sl) : 0u;
            for (; sl < p.slabs; sl += 2) {
                const int g = seq + sl;
                const uint32_t z0 = z_next & 0xffu, z1 = z_next >> 8;
                if (sl + 2 < p.slabs)
                    z_next = zero_points(sl + 2);
                const uint32_t lo0 = z0 * 0x00010001u + 0x64006400u, hi0 = z0 * 0x00100010u + 0x54005400u;
                const uint32_t lo1 = z1 * 0x00010001u + 0x64006400u, hi1 = z1 * 0x00100010u + 0x54005400u;
                const int s = g % STAGES;
                // the nibbles have landed
                if (!wait_parked(&full_x[s], (g / STAGES) & 1)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                    ok = false;
                    break;
                }
                // announce this group's previous slab: its store was issued a barrier wait ago
                if (pending >= 0) {
                    umma::tmem_st_wait();
                    umma::tc_fence_before();  // the store is ordered before the MMA warp's wait on full_w
                    // one arrival per warp: 32 lanes arriving on the same barrier word are 32 serialised
                    // shared-memory atomics
                    __syncwarp();
                    if (lane == 0)
                        umma::mbar_arrive(&full_w[pending]);
                }
                const uint4 *raw = reinterpret_cast<const uint4 *>(sR + s * RAW_BYTES + r * 32);
                const uint4 c0 = raw[0], c1 = raw[1];
                // 64 k of this row as 32 fp16 pairs, k ascending: the 32 columns of the A stage
                uint32_t wv[32];
                const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const uint4 o = c < 4 ? unpack8(words[c], lo0, hi0, uc) : unpack8(words[c], lo1, hi1, uc);
                    wv[4 * c] = o.x;
                    wv[4 * c + 1] = o.y;
                    wv[4 * c + 2] = o.z;
                    wv[4 * c + 3] = o.w;
                }
                // the A stage this slab goes into was read by the MMAs of the slab A_STAGES earlier,
                // whose completion is the `empty` barrier of that slab's shared-memory stage
                if (g >= A_STAGES && !wait_parked(&empty[(g - A_STAGES) % STAGES], ((g - A_STAGES) / STAGES) & 1)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                    ok = false;
                    break;
                }
                umma::tc_fence_after();
                pending = g % A_STAGES;
                umma::tmem_st_32x32(a_lane + uint32_t(pending * A_COLS), wv);
            }
        }
        if (pending >= 0) {
            umma::tmem_st_wait();
            umma::tc_fence_before();
            __syncwarp();
            if (lane == 0)
                umma::mbar_arrive(&full_w[pending]);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
        // ---------------------------------------------------------------- promotion
        const int q = warp & 3;            // tensor-memory lane quarter this warp may read
        const int half = (warp - 12) >> 2;  // which half of the tile's tokens
        // the tile's tokens are split between the two halves in whole 32-column chunks, and a warp
        // reads only the chunks that hold tokens
        const int hw = ((p.bt / 2 + 31) / 32) * 32;
        const int nchunks = (min(hw, p.bt - half * hw) + 31) / 32;
        int b = 0;
        uint32_t acc_ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * BW + q * 32 + lane;
            const int m0 = (tile % p.m_tiles) * p.bt + half * hw;
            // token rows of this warp that exist (may be <= 0): its share of the tile, cut at the end of M
            const int rows = min(p.M - m0, min(hw, p.bt - half * hw));
            float acc[HALF];
#pragma unroll
            for (int j = 0; j < HALF; j++)
                acc[j] = 0.0f;
            float scale = p.scales_t[n];
            for (int blk = 0; blk < p.n_blocks; blk++) {
                const float scale_next = blk + 1 < p.n_blocks ? p.scales_t[size_t(blk + 1) * p.n_pad + n] : 0.0f;
                if (ok && !wait_parked(&acc_full[b], acc_ph)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    ok = false;
                }
                umma::tc_fence_after();
                const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * p.acc_stride + half * hw);
#pragma unroll
                for (int c = 0; c < HALF / 32; c++) {
                    if (c >= nchunks)
                        break;
                    uint32_t d[32];
                    umma::tmem_ld_32x32(taddr + c * 32, d);
                    umma::tmem_ld_wait();
                    if (c == nchunks - 1) {  // everything of this accumulator has been read: hand it back
                        umma::tc_fence_before();
                        __syncwarp();
                        if (lane == 0)
                            umma::mbar_arrive(&acc_empty[b]);
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        acc[c * 32 + j] = fmaf(__uint_as_float(d[j]), scale, acc[c * 32 + j]);
                }
                scale = scale_next;
                if (++b == p.ring) {
                    b = 0;
                    acc_ph ^= 1;
                }
            }
            if (ok && n < p.N) {
                // the MMA thread can run only two blocks ahead while this store lasts: a row
                // pointer stepped by N and no bound test when all token rows of this warp exist
                const bool whole = rows >= HALF;
                if (p.y_f32) {
                    float *y = static_cast<float *>(p.y) + size_t(m0) * p.N + n;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.N)
                            *y = acc[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.N)
                            if (j < rows)
                                *y = acc[j];
                    }
                } else {
                    __half *y = static_cast<__half *>(p.y) + size_t(m0) * p.N + n;
                    if (whole) {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.N)
                            *y = __float2half_rn(acc[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.N)
                            if (j < rows)
                                *y = __float2half_rn(acc[j]);
                    }
                }
            }
        }
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, TMEM_COLS);
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

size_t gemm_smem() { return size_t(STAGES) * (B_BYTES + RAW_BYTES) + 512; }

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

// Tokens per tile.  A slab of a tile costs about 285 + (tokens) in units of 1.4 clocks
// (measured: 670, 575 and 535 clocks for 192, 128 and 96 tokens), the grid runs
// ceil(tiles / SMs) rounds and the last round is as long as a full one: a narrower tile that
// fills the last round better wins when the product is smaller.
int token_tile(int64_t m, int n_tiles, int sm_count)
{
    static const char *pin = getenv("OVK_NBITS_BT");
    if (pin && atoi(pin) >= 96 && atoi(pin) <= BT && atoi(pin) % 32 == 0)
        return atoi(pin);
    int best = BT;
    double best_cost = 0;
    for (int bt = BT; bt >= 96; bt -= 32) {
        const int64_t tiles = ceil_div64(m, bt) * n_tiles;
        const double cost = double(ceil_div64(tiles, sm_count)) * (285 + bt);
        if (bt == BT || cost < 0.97 * best_cost) {
            best = bt;
            best_cost = cost;
        }
    }
    return best;
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
    const int n_tiles = int(w->gemm_n_pad / BW);
    const int bt = token_tile(m, n_tiles, ctx->sm_count);
    CUtensorMap tmAct;
    if (!ovk_make_tmap_2d(&tmAct, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, uint64_t(w->k), uint64_t(m), uint64_t(w->k) * 2,
                          SLAB, uint32_t(bt), CU_TENSOR_MAP_SWIZZLE_128B))
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
    p.bt = bt;
    p.ring = bt > 128 ? 2 : (bt > 96 ? 3 : 4);
    p.acc_stride = bt > 128 ? BT : (bt > 96 ? 128 : 96);
    p.m_tiles = int(ceil_div64(m, bt));
    p.n_tiles = n_tiles;
    p.y_f32 = y_dtype == OVK_FLOAT;
    p.status = ctx->dev_status;
    OVK_CUDA(ctx, cudaFuncSetAttribute(nbits_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem())));
    const int64_t tiles = int64_t(p.m_tiles) * p.n_tiles;
    const unsigned grid = unsigned(std::min<int64_t>(tiles, ctx->sm_count));
    nbits_gemm_kernel<<<grid, THREADS, gemm_smem(), ctx->stream>>>(tmAct, tmRaw, p);
    OVK_LAUNCHED(ctx, "nbits_gemm_tc");
    return OVK_OK;
}
