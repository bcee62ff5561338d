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
//
// Work is handed out in UNITS of one quantization block (one 64-k slab for the
// blocks smaller than a slab) of one tile.  A launch either gives every CTA a
// run of whole tiles, or - when whole tiles would leave SMs idle in the last
// round - cuts the line of all units into one contiguous run per CTA, so that a
// tile's K range may be shared by several CTAs.  A CTA that holds only part of
// a tile's K writes its f32 partial sums to the workspace and counts itself at
// the tile's counter; the CTA that arrives last adds the parts in K order
// (always the same order, so results do not depend on who was last) and stores
// the tile.  Nobody waits for anybody.
//
//   warp 3      store: fp16 results go through a small shared-memory buffer so
//               that rows leave as 16-byte stores in 256-byte segments, and this
//               warp - not the promotion warps, which go straight on to the next
//               tile - issues them.  In a launch that is one rank of a column
//               split over several GPUs it stores every segment into EVERY
//               rank's copy of Y (plain stores through peer mappings): the
//               all-gather happens tile by tile while the tensor core works on
//               the next tile, and ends with one flag per peer.
#include "ovk_internal.h"
#include "umma.cuh"

namespace {

constexpr int BW = 128;    // weight columns per tile (UMMA M)
constexpr int BT = 192;    // most tokens per tile (UMMA N)
constexpr int HALF = BT / 2;  // token rows per promotion warp
constexpr int SLAB = 64;   // k per stage: 128 bytes of fp16
constexpr int STAGES = 6;    // shared-memory ring: tokens + packed nibbles of a slab (TMA); eight measured the same
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
constexpr int Y_ROWS = HALF;               // token rows of a promotion half's store buffer
constexpr int Y_BYTES = Y_ROWS * BW * 2;   // one half's buffer: 96 rows x 128 fp16
constexpr int PART_FLOATS = HALF * BW;     // f32 partial sums one promotion half holds for a tile

struct GemmParams {
    const uint8_t *wq;     // [n_pad, k_pad/2] nibble-permuted copy
    const float *scales_t; // [nb_pad, n_pad]
    const uint8_t *zp_t;   // [n_pad, zp_pitch] one byte per block, rows padded to 8
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
    // where results go: n_dst matrices of row pitch ldy elements, this launch's columns starting at col0
    void *y_dst[OVK_MAX_RANKS];
    void *y_mc;            // multicast mapping of all n_dst matrices (one store reaches every rank), or null
    int n_dst, ldy, col0;
    int vec_ok;            // every destination takes 16-byte stores at multiples of 8 columns
    OvkCommView comm;      // used when n_dst > 1
    // work units
    int units;             // per tile
    int unit_slabs;        // slabs of one unit (1, 2 or 4)
    int unit_blocks;       // quantization blocks of one unit (2 for blocks of 32, else 1)
    int shared_k;          // 1: contiguous runs of units, tiles may be shared between CTAs
    float *partials;       // [gridDim.x][2 items][2 halves][HALF][BW] f32
    uint32_t *counters;    // one per tile, zero between launches
};

// The run of units of this CTA and its walk, tile by tile.
struct Run {
    uint32_t u, end;  // the host keeps tiles x units below 2^31
};
// `cta` of `grid`: the CTA's number and the grid's size - or, when two CTAs work as a pair on tiles of
// twice the width, the pair's number and the number of pairs.
__device__ __forceinline__ uint32_t run_start(const GemmParams &p, uint32_t cta, uint32_t grid)
{
    const unsigned long long tiles = (unsigned long long)p.m_tiles * p.n_tiles;
    if (p.shared_k)
        return uint32_t(tiles * p.units * cta / grid);
    return uint32_t(tiles * cta / grid) * uint32_t(p.units);
}
__device__ __forceinline__ Run cta_run(const GemmParams &p, uint32_t cta, uint32_t grid)
{
    Run r;
    r.u = run_start(p, cta, grid);
    r.end = run_start(p, cta + 1, grid);
    return r;
}
// A CTA's tiles are consecutive numbers: one weight tile, the token tiles one after the other.
// (Measured: it makes no difference whether the CTAs running together share a weight tile or a
// token tile - both operands of these shapes stay in the L2.)
__device__ __forceinline__ void tile_origin(const GemmParams &p, int tile, int &m_index, int &n_index)
{
    n_index = tile / p.m_tiles;
    m_index = tile - n_index * p.m_tiles;
}
// Next item of the run: units [ub, ue) of `tile`.  Returns false at the end.
__device__ __forceinline__ bool next_item(const GemmParams &p, Run &r, int &tile, int &ub, int &ue)
{
    if (r.u >= r.end)
        return false;
    tile = int(r.u / uint32_t(p.units));
    ub = int(r.u - uint32_t(tile) * uint32_t(p.units));
    ue = int(min(uint32_t(p.units), uint32_t(ub) + (r.end - r.u)));
    r.u += uint32_t(ue - ub);
    return true;
}

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

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// What the store warp is told about the tile in a half's buffer.
struct PassDesc {
    int m_base;  // token row of the buffer's first row
    int rows;    // rows of the buffer that hold results (<= 0: none); -1000000: the CTA has no more tiles
    int n0;      // first weight column of the tile
    int pad;
};
constexpr int PASS_STOP = -1000000;

// PAIR: launched in clusters of two.  The pair computes tiles of 256 weight columns - CTA `crank` owns
// columns crank * 128 .. + 127 of the tile, in its own tensor memory, exactly as a single CTA owns its
// 128 - by tcgen05.mma.cta_group::2, which reads the token operand half from each CTA's shared memory:
// each CTA loads only half of the token rows of a slab, which halves what the L2 has to deliver per
// MMA.  One thread of CTA 0 issues; the unpack and promotion warps of both CTAs announce themselves at
// CTA 0's barriers, and the completion of the MMAs is signalled to the barriers of both.
template <bool PAIR>
__global__ void __launch_bounds__(THREADS, 1)
nbits_gemm_kernel(const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmRaw,
                  const __grid_constant__ GemmParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sX = smem;                       // STAGES x 24 KB: tokens (UMMA B operand)
    uint8_t *sR = sX + STAGES * B_BYTES;      // STAGES x 4 KB: packed nibbles as loaded
    uint8_t *sY = sR + STAGES * RAW_BYTES;    // 2 x 24 KB: results on their way out, one buffer per promotion half
    uint64_t *bars = reinterpret_cast<uint64_t *>(sY + 2 * Y_BYTES);
    uint64_t *full_x = bars;                  // TMA landed
    uint64_t *full_w = full_x + STAGES;       // [A_STAGES] the four unpack warps arrived
    uint64_t *empty = full_w + A_STAGES;      // [STAGES] MMAs of the slab finished: its shared-memory AND its A stage are free
    uint64_t *acc_full = empty + STAGES;      // a block's partial sums are complete
    uint64_t *acc_empty = acc_full + ACC_RING;// all 8 promotion warps have read them
    uint64_t *y_full = acc_empty + ACC_RING;  // [2] a half's buffer holds a pass (its four warps arrived)
    uint64_t *y_empty = y_full + 2;           // [2] the store warp has read it
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(y_empty + 2);
    uint32_t *s_count = tmem_slot + 1;        // the tile counter's value, for all promotion warps
    PassDesc *s_desc = reinterpret_cast<PassDesc *>(tmem_slot + 4);  // [2]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = PAIR ? umma::cluster_rank() : 0u;
    const uint32_t vcta = PAIR ? blockIdx.x >> 1 : blockIdx.x, vgrid = PAIR ? gridDim.x >> 1 : gridDim.x;
    constexpr int WIDE = PAIR ? 2 : 1;  // 128-column tiles per tile number

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            umma::mbar_init(&full_x[s], 1);
            umma::mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < A_STAGES; s++)
            umma::mbar_init(&full_w[s], PAIR ? 8 : 4);  // one arrival per unpack warp (of both CTAs)
        for (int b = 0; b < ACC_RING; b++) {
            umma::mbar_init(&acc_full[b], 1);
            umma::mbar_init(&acc_empty[b], PAIR ? 16 : 8);
        }
        for (int h = 0; h < 2; h++) {
            umma::mbar_init(&y_full[h], 4);  // one arrival per promotion warp of the half
            umma::mbar_init(&y_empty[h], 1);
        }
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            umma::tmem_alloc_pair(tmem_slot, TMEM_COLS);
            umma::tmem_relinquish_pair();
        } else {
            umma::tmem_alloc(tmem_slot, TMEM_COLS);
            umma::tmem_relinquish();
        }
    }
    umma::tc_fence_before();
    if constexpr (PAIR)
        umma::cluster_sync_all();  // the other CTA's barriers are initialised before anything arrives there
    else
        __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int blocks_per_slab = p.bs >= SLAB ? 1 : SLAB / p.bs;  // 2 when block_size is 32
    const int slabs_per_block = p.bs >= SLAB ? p.bs / SLAB : 1;

    // 640 threads start with 96 registers each; control and unpack warps give registers back,
    // the promotion warps take them (48*128 + 64*256 + 152*256 = 61440, all there are)
    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
    if (warp == 0) {
        // ------------------------------------------------------------ tokens by TMA
        if (lane == 0) {
            umma::prefetch_tmap(&tmAct);
            umma::prefetch_tmap(&tmRaw);
            int s = 0;
            uint32_t ph = 0;
            Run run = cta_run(p, vcta, vgrid);
            int tile, ub, ue;
            bool ok = true;
            while (ok && next_item(p, run, tile, ub, ue)) {
                int mi, ni;
                tile_origin(p, tile, mi, ni);
                // a pair: this CTA's half of the tile's token rows, and its own 128 weight rows
                const int tok_rows = PAIR ? p.bt / 2 : p.bt;
                const int m0 = mi * p.bt + int(crank) * (PAIR ? tok_rows : 0), n0 = (ni * WIDE + int(crank)) * BW;
                for (int sl = ub * p.unit_slabs; sl < ue * p.unit_slabs; sl++) {
                    if (!wait_parked(&empty[s], ph ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        ok = false;
                        break;
                    }
                    umma::mbar_expect_tx(&full_x[s], uint32_t(tok_rows) * 128u + RAW_BYTES);
                    umma::tma_load_2d(sX + s * B_BYTES, &tmAct, &full_x[s], sl * SLAB, m0);
                    umma::tma_load_2d(sR + s * RAW_BYTES, &tmRaw, &full_x[s], sl * 32, n0);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
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
        // Runs begin and end on block boundaries, so the per-block state carries over from one
        // item to the next exactly as it does from tile to tile.
        const int me = warp - 1;
        const int issuers = p.bs >= SLAB ? 2 : 1;  // smaller blocks: two per slab, one issuer
        if (me < issuers && crank == 0) {
            const bool leader = umma::elect_one();
            const uint32_t idesc = umma::instr_desc(1 /*f32*/, 0 /*f16*/, 0 /*f16*/, BW * WIDE, p.bt);
            const uint32_t desc_hi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
            const uint32_t x16 = umma::smem_u32(sX) >> 4;
            int s = 0, a = 0, b = 0, slab_in_block = 0, owner = 0;
            uint32_t a_ph = 0, acc_ph = 0;
            bool ok = true;
            Run run = cta_run(p, vcta, vgrid);
            int tile, ub, ue;
            while (ok && next_item(p, run, tile, ub, ue)) {
                for (int sl = ub * p.unit_slabs; sl < ue * p.unit_slabs && ok; sl++) {
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
                                if constexpr (PAIR) {
                                    umma::mma_f16_ts_pair(d, a_t, x_lo, desc_hi, idesc, first ? 0u : 1u);
                                    umma::mma_f16_ts_pair(d, a_t + 8, x_lo + 2, desc_hi, idesc, 1u);
                                    umma::mma_f16_ts_pair(d, a_t + 16, x_lo + 4, desc_hi, idesc, 1u);
                                    umma::mma_f16_ts_pair(d, a_t + 24, x_lo + 6, desc_hi, idesc, 1u);
                                    umma::mma_commit_pair(&empty[s]);
                                    if (last)
                                        umma::mma_commit_pair(&acc_full[b]);
                                } else {
                                    umma::mma_f16_ts(d, a_t, x_lo, desc_hi, idesc, first ? 0u : 1u);
                                    umma::mma_f16_ts(d, a_t + 8, x_lo + 2, desc_hi, idesc, 1u);
                                    umma::mma_f16_ts(d, a_t + 16, x_lo + 4, desc_hi, idesc, 1u);
                                    umma::mma_f16_ts(d, a_t + 24, x_lo + 6, desc_hi, idesc, 1u);
                                    umma::mma_commit(&empty[s]);
                                    if (last)
                                        umma::mma_commit(&acc_full[b]);
                                }
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
    } else if (warp == 3) {
        // -------------------------------------------------------------------- store
        // Takes the tiles the promotion halves leave in their buffers (half 0, half 1, half 0,
        // ...) and writes them out: a row of the buffer is 256 contiguous bytes of a row of Y, a
        // lane moves 16 of them, and in a column split over several GPUs every 16 bytes go to
        // every rank's Y.  The stores are not waited for here; the promotion warps have long gone
        // on to the next tile.
        const bool exchange = p.n_dst > 1;
        bool peers_ready = !exchange;
        bool ok = true;
        if (exchange && blockIdx.x == 0)
            comm::announce(p.comm, false, lane);  // this rank's earlier work on the stream is complete
        uint32_t seq = 0;
        for (bool running = !p.y_f32; running;) {  // f32 results are stored by the promotion warps themselves
#pragma unroll 1
            for (int h = 0; h < 2 && running; h++) {
                if (!wait_parked(&y_full[h], seq & 1)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    ok = false;
                    running = false;
                    break;
                }
                const PassDesc d = s_desc[h];
                if (d.rows == PASS_STOP) {
                    if (h == 1)
                        running = false;
                    continue;  // (the stop arrives on both halves in the same pass)
                }
                if (!peers_ready && d.rows > 0) {
                    // before the first store into a peer: its stream has reached this call too, so
                    // nothing there still reads what is about to be overwritten
                    peers_ready = true;
                    if (!comm::wait_all(p.comm, false, lane)) {
                        if (lane == 0)
                            atomicExch(p.status, OVK_DEV_TIMEOUT_PEER);
                        ok = false;
                    }
                }
                const uint8_t *buf = sY + h * Y_BYTES;
                // A lane keeps one 16-byte column chunk (lane & 15) and walks down the rows two at a
                // time, so a chunk costs a shared-memory load, a store and two additions; the ranks
                // are taken one after the other, each from the same buffer.
                const int cc = lane & 15, r0 = lane >> 4;
                const int n = d.n0 + cc * 8;
                const uint8_t *src0 = buf + r0 * (BW * 2) + cc * 16;
                const size_t off0 = (size_t(d.m_base + r0) * size_t(p.ldy) + size_t(p.col0 + n)) * 2;
                const size_t step = size_t(p.ldy) * 4;  // two rows of Y
                // The ranks are taken in an order that starts behind this rank and differs from CTA to CTA, so
                // that the ranks, which run in step, do not all store into the same peer at once.  (Measured at
                // 4 ranks it made no difference - the switch spreads the load - but it costs nothing.)
                const int first = exchange ? (p.comm.rank + 1 + int(blockIdx.x)) % p.n_dst : 0;
                if (p.y_mc && p.vec_ok && d.n0 + BW <= p.N) {
                    // one multicast store per chunk: it leaves over this GPU's links once and the switch
                    // delivers it to every rank, this one included
                    uint8_t *dst = static_cast<uint8_t *>(p.y_mc) + off0;
                    const uint8_t *src = src0;
#pragma unroll 4
                    for (int row = r0; row < Y_ROWS; row += 2, src += 2 * BW * 2, dst += step) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(src);
                        if (ok && row < d.rows)
                            comm::st_multicast16(dst, v);
                    }
                } else if (p.vec_ok && d.n0 + BW <= p.N) {
                    for (int j = 0; j < p.n_dst; j++) {
                        const int r = first + j < p.n_dst ? first + j : first + j - p.n_dst;
                        uint8_t *dst = static_cast<uint8_t *>(p.y_dst[r]) + off0;
                        const uint8_t *src = src0;
#pragma unroll 4
                        for (int row = r0; row < Y_ROWS; row += 2, src += 2 * BW * 2, dst += step) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(src);
                            if (ok && row < d.rows)
                                *reinterpret_cast<uint4 *>(dst) = v;
                        }
                    }
                } else {
                    // a tile at the ragged edge of N, or destinations that do not take 16-byte stores
                    for (int j = 0; j < p.n_dst; j++) {
                        const int r = first + j < p.n_dst ? first + j : first + j - p.n_dst;
                        uint8_t *dst = static_cast<uint8_t *>(p.y_dst[r]) + off0;
                        const uint8_t *src = src0;
                        for (int row = r0; row < Y_ROWS; row += 2, src += 2 * BW * 2, dst += step) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(src);
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                            if (ok && row < d.rows) {
#pragma unroll
                                for (int e = 0; e < 8; e++)
                                    if (n + e < p.N)
                                        reinterpret_cast<uint16_t *>(dst)[e] = uint16_t(w[e >> 1] >> (16 * (e & 1)));
                            }
                        }
                    }
                }
                // everything of the buffer has been read (the stores may still be on their way): hand it back
                __syncwarp();
                if (lane == 0)
                    umma::mbar_arrive(&y_empty[h]);
            }
            seq++;
        }
        if (exchange) {
            // every store of this CTA is visible everywhere before the CTA is counted; the CTA
            // counted last announces the kernel's stores to every rank
            __threadfence_system();
            __syncwarp();
            OvkCommFlags *own = p.comm.flags[p.comm.rank];
            uint32_t last = 0;
            if (lane == 0) {
                last = atomicAdd(&own->cta_done, 1u) + 1u == gridDim.x;
                if (last)
                    own->cta_done = 0;
                __threadfence_system();
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last && ok)
                comm::announce(p.comm, true, lane);
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
        // where this warp announces an A stage: the issuing CTA's barrier
        const uint32_t full_w_at = PAIR ? umma::mbar_in_cta(&full_w[0], 0) : 0u;
        auto announce = [&](int stage) {
            if constexpr (PAIR)
                umma::mbar_arrive_cluster(full_w_at + uint32_t(stage) * 8u);
            else
                umma::mbar_arrive(&full_w[stage]);
        };
        int seq = 0;       // number of slabs before the current item's first one
        int pending = -1;  // A stage stored to but not yet announced
        // This loop is the kernel's pace-setter, so ring positions are stepped by two inside an item (six
        // stages: no power of two) and divided out only once per item: slab g sits in stage s_g on the
        // ring's lap of parity ph_g, and the slab A_STAGES before it likewise in s_b / ph_b.
        bool ok = true;
        Run run = cta_run(p, vcta, vgrid);
        int tile, ub, ue;
        while (ok && next_item(p, run, tile, ub, ue)) {
            int mi, ni;
            tile_origin(p, tile, mi, ni);
            const int n = (ni * WIDE + int(crank)) * BW + r;
            const int sl0 = ub * p.unit_slabs, len = (ue - ub) * p.unit_slabs;
            // zero points: one byte per block, fetched one slab of this group ahead
            const uint8_t *zrow = p.zp_t + size_t(n) * p.zp_pitch;
            auto zero_points = [&](int sl) -> uint32_t {
                const int blk = (sl * SLAB) >> bs_shift;
                const uint32_t z0 = zrow[blk];
                return z0 | (blocks_per_slab == 2 ? uint32_t(zrow[blk + 1]) << 8 : z0 << 8);
            };
            int i = (seq ^ group) & 1;  // the first slab of this item that this group takes
            uint32_t z_next = i < len ? zero_points(sl0 + i) : 0u;
            int s_g = (seq + i) % STAGES, s_b = (seq + i + STAGES - A_STAGES) % STAGES;
            uint32_t ph_g = uint32_t((seq + i) / STAGES) & 1u;
            uint32_t ph_b = uint32_t((seq + i + STAGES - A_STAGES) / STAGES + 1) & 1u;
            for (; i < len; i += 2) {
                const int g = seq + i;
                const uint32_t z0 = z_next & 0xffu, z1 = z_next >> 8;
                if (i + 2 < len)
                    z_next = zero_points(sl0 + i + 2);
                const uint32_t lo0 = z0 * 0x00010001u + 0x64006400u, hi0 = z0 * 0x00100010u + 0x54005400u;
                const uint32_t lo1 = z1 * 0x00010001u + 0x64006400u, hi1 = z1 * 0x00100010u + 0x54005400u;
                const int s = s_g;
                // the nibbles have landed
                if (!wait_parked(&full_x[s], ph_g)) {
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
                        announce(pending);
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
                if (g >= A_STAGES && !wait_parked(&empty[s_b], ph_b)) {
                    if (lane == 0)
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                    ok = false;
                    break;
                }
                umma::tc_fence_after();
                pending = g & (A_STAGES - 1);
                umma::tmem_st_32x32(a_lane + uint32_t(pending * A_COLS), wv);
                if constexpr (PAIR) {
                    // across the pair an announcement takes longer to arrive, so it leaves at once (measured:
                    // 4 % faster than announcing a slab late, which is the faster way within one CTA)
                    umma::tmem_st_wait();
                    umma::tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        announce(pending);
                    pending = -1;
                }
                s_g += 2;
                if (s_g >= STAGES) {
                    s_g -= STAGES;
                    ph_g ^= 1u;
                }
                s_b += 2;
                if (s_b >= STAGES) {
                    s_b -= STAGES;
                    ph_b ^= 1u;
                }
            }
            seq += len;
        }
        if (pending >= 0) {
            umma::tmem_st_wait();
            umma::tc_fence_before();
            __syncwarp();
            if (lane == 0)
                announce(pending);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
        // ---------------------------------------------------------------- promotion
        const int q = warp & 3;            // tensor-memory lane quarter this warp may read
        const int half = (warp - 12) >> 2;  // which half of the tile's tokens
        // the tile's tokens are split between the two halves in whole 32-column chunks, and a warp
        // reads only the chunks that hold tokens
        const int hw = ((p.bt / 2 + 31) / 32) * 32;
        const int half_rows = min(hw, p.bt - half * hw);
        const int nchunks = (half_rows + 31) / 32;
        int b = 0;
        uint32_t acc_ph = 0;
        const uint32_t acc_empty_at = PAIR ? umma::mbar_in_cta(&acc_empty[0], 0) : 0u;  // the issuing CTA's barrier
        uint32_t yseq = 0;  // tiles this half has put into its buffer
        bool first_item = true;
        bool ok = true;
        Run run = cta_run(p, vcta, vgrid);
        int tile, ub, ue;
        // this thread's column of the half's token rows into the half's buffer, then the warp's arrival.
        // The buffer was handed back when the store warp had read the previous tile out of it, a tile's
        // time ago, so this wait is normally over before it starts.
        auto put_tile = [&](const float (&acc)[HALF], int m_base, int rows, int n0) {
            if (ok && !wait_parked(&y_empty[half], (yseq & 1) ^ 1)) {
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                ok = false;
            }
            if (rows != PASS_STOP) {
                const uint32_t ybuf = umma::smem_u32(sY) + uint32_t(half * Y_BYTES + (q * 32 + lane) * 2);
#pragma unroll
                for (int j = 0; j < HALF; j++)
                    asm volatile("st.shared.b16 [%0], %1;" ::"r"(ybuf + j * (BW * 2)), "h"(__half_as_ushort(__float2half_rn(acc[j])))
                                 : "memory");
            }
            if (q == 0 && lane == 0) {
                PassDesc d;
                d.m_base = m_base;
                d.rows = ok ? rows : (rows == PASS_STOP ? PASS_STOP : 0);
                d.n0 = n0;
                d.pad = 0;
                s_desc[half] = d;
            }
            __syncwarp();
            if (lane == 0)
                umma::mbar_arrive(&y_full[half]);  // release: the buffer and the descriptor are written
            yseq++;
        };
        while (next_item(p, run, tile, ub, ue)) {
            int mi, ni;
            tile_origin(p, tile, mi, ni);
            const int n0 = (ni * WIDE + int(crank)) * BW;
            const int n = n0 + q * 32 + lane;
            float acc[HALF];
#pragma unroll
            for (int j = 0; j < HALF; j++)
                acc[j] = 0.0f;
            const int blk0 = ub * p.unit_blocks, blk1 = ue * p.unit_blocks;
            float scale = p.scales_t[size_t(blk0) * p.n_pad + n];
            for (int blk = blk0; blk < blk1; blk++) {
                const float scale_next = blk + 1 < blk1 ? p.scales_t[size_t(blk + 1) * p.n_pad + n] : 0.0f;
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
                        if (lane == 0) {
                            if constexpr (PAIR)
                                umma::mbar_arrive_cluster(acc_empty_at + uint32_t(b) * 8u);
                            else
                                umma::mbar_arrive(&acc_empty[b]);
                        }
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
            bool store = true;
            if (ub != 0 || ue != p.units) {
                // Part of the tile's K: leave the partial sums in this CTA's slot (0 for the item its
                // run begins with, 1 for any later one - a run has at most two partial items) and
                // count this part at the tile.  The part counted last adds all parts in K order,
                // its own read back like the others so that the order of the additions is fixed.
                float *mine = p.partials + ((size_t(blockIdx.x) * 2 + (first_item ? 0 : 1)) * 2 + half) * PART_FLOATS +
                              q * 32 + lane;
#pragma unroll
                for (int j = 0; j < HALF; j++)
                    __stcg(mine + j * BW, acc[j]);
                __threadfence();
                named_bar_sync(1, 256);
                if (warp == 12 && lane == 0) {
                    // CTAs whose runs reach into this tile: from the one holding its first unit to the
                    // one holding its last
                    const long long total = (long long)p.m_tiles * p.n_tiles * p.units;
                    const long long x0 = (long long)tile * p.units, x1 = x0 + p.units - 1;
                    const long long c_first = ((x0 + 1) * vgrid + total - 1) / total - 1;
                    const long long c_last = ((x1 + 1) * vgrid + total - 1) / total - 1;
                    const uint32_t parts = uint32_t(c_last - c_first + 1);
                    uint32_t *counter = p.counters + size_t(tile) * WIDE + crank;  // each 128-column tile has its own
                    const uint32_t before = atomicAdd(counter, 1u);
                    const bool last = before + 1u == parts;
                    if (last)
                        *counter = 0;  // zero again for the next launch
                    __threadfence();
                    s_count[0] = last ? uint32_t(c_first) : 0xffffffffu;
                    s_count[1] = uint32_t(c_last);
                }
                named_bar_sync(1, 256);
                const uint32_t c_first = s_count[0], c_last = s_count[1];
                named_bar_sync(1, 256);  // s_count may be rewritten for the next partial item
                store = c_first != 0xffffffffu;
                if (store) {
#pragma unroll
                    for (int j = 0; j < HALF; j++)
                        acc[j] = 0.0f;
                    for (uint32_t c = c_first; c <= c_last; c++) {
                        // the part of CTA c is the item its run begins with, unless the run began in
                        // an earlier tile (only the first of the CTAs can)
                        const bool begins_here = run_start(p, c, vgrid) >= uint32_t(tile) * uint32_t(p.units);
                        const size_t holder = size_t(c) * WIDE + crank;  // the CTA of pair c with this CTA's columns
                        const float *part = p.partials + ((holder * 2 + (begins_here ? 0 : 1)) * 2 + half) * PART_FLOATS +
                                            q * 32 + lane;
#pragma unroll
                        for (int j = 0; j < HALF; j++)
                            acc[j] += __ldcg(part + j * BW);
                    }
                }
            }
            first_item = false;
            if (!store)
                continue;
            const int m0 = mi * p.bt + half * hw;
            // token rows of this warp that exist (may be <= 0): its share of the tile, cut at the end of M
            const int rows = min(p.M - m0, half_rows);
            if (p.y_f32) {
                if (ok && n < p.N) {
                    // the MMA thread can run only two blocks ahead while this store lasts: a row
                    // pointer stepped by the pitch and no bound test when all token rows of this warp exist
                    float *y = static_cast<float *>(p.y_dst[0]) + size_t(m0) * p.ldy + p.col0 + n;
                    if (rows >= HALF) {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.ldy)
                            *y = acc[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < HALF; j++, y += p.ldy)
                            if (j < rows)
                                *y = acc[j];
                    }
                }
            } else {
                put_tile(acc, m0, rows, n0);
            }
        }
        if (!p.y_f32) {
            float none[HALF];
            none[0] = 0.0f;
            put_tile(none, 0, PASS_STOP, 0);  // tells the store warp that this CTA has no more tiles
        }
    }
    umma::tc_fence_before();
    if constexpr (PAIR) {
        umma::cluster_sync_all();  // the other CTA's MMAs write this CTA's tensor memory too
        if (warp == 1)
            umma::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    } else {
        __syncthreads();
        if (warp == 1)
            umma::tmem_dealloc(tmem_base, TMEM_COLS);
    }
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

size_t gemm_smem() { return size_t(STAGES) * (B_BYTES + RAW_BYTES) + 2 * Y_BYTES + 512; }

}  // namespace

// The prefill copy: nibble-permuted [n_pad, k_pad/2] weights, f32 scales and
// (transposed to [block, n_pad]) and one zero-point byte per block, row major.  Built on the first prefill
// call (as the reference builds packed weights at first use, src/cache.rs:231).
int32_t ovk_nbits_gemm_prepack(ovk_ctx *ctx, ovk_nbits_weight *w)
{
    if (w->gemm_w)
        return OVK_OK;
    const int64_t n_pad = ceil_div64(w->n, 2 * BW) * (2 * BW);  // whole tiles of a pair of CTAs
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

// The shape of a launch: tokens per tile, and whether CTAs get whole tiles or runs of units.
// A slab of a tile costs about 285 + (tokens) in units of 1.4 clocks (measured: 670, 575 and 535
// clocks for 192, 128 and 96 tokens).  With whole tiles the grid runs ceil(tiles / SMs) rounds and
// the last round is as long as a full one; with runs of units every SM gets the same share of the
// slabs, at the price of the partial sums the shared tiles go through (taken as eight slabs' time
// per CTA).  The cheaper plan wins; whole tiles also win a near tie, since they need no workspace.
struct Plan {
    int bt;
    bool shared_k;
    unsigned grid;
    double cost;
};
// `sms`: how many CTAs (or pairs of CTAs) run at once; `slab_fixed`: the part of a slab's time that
// does not grow with the tile's tokens.
Plan plan_launch(int sms, double slab_fixed, int64_t m, int n_tiles, int units, int unit_slabs, int counters_per_tile)
{
    Plan best = {BT, false, 1, 0.0};
    double best_cost = 0;
    bool have = false;
    for (int bt = BT; bt >= 96; bt -= 32) {
        const int64_t tiles = ceil_div64(m, bt) * n_tiles;
        const double slab = slab_fixed + bt;
        const double whole = double(ceil_div64(tiles, sms)) * units * unit_slabs * slab;
        if (!have || whole < 0.97 * best_cost) {
            best = {bt, false, unsigned(std::min<int64_t>(tiles, sms)), whole};
            best_cost = whole;
            have = true;
        }
        const int64_t total_units = tiles * units;
        const int64_t grid = std::min<int64_t>(sms, total_units);
        if (tiles * counters_per_tile <= OVK_TILE_COUNTERS && units > 1 && grid > 0) {
            const double shared = (double(ceil_div64(total_units, grid)) * unit_slabs + 8.0) * slab;
            if (shared < 0.95 * best_cost) {
                best = {bt, true, unsigned(grid), shared};
                best_cost = shared;
            }
        }
    }
    return best;
}

#ifndef OVK_NBITS_PAIRS
#define OVK_NBITS_PAIRS 1
#endif
// How many pairs of CTAs of the pair kernel the GPU runs at once (0: none - clusters unavailable).
int pair_capacity(ovk_ctx *ctx)
{
    if (ctx->nbits_pairs >= 0)
        return ctx->nbits_pairs;
    ctx->nbits_pairs = 0;
    if (cudaFuncSetAttribute(nbits_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem())) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(ctx->sm_count & ~1));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = gemm_smem();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, nbits_gemm_kernel<true>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    ctx->nbits_pairs = clusters;
    return clusters;
}

bool ovk_nbits_gemm_split_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w);
int32_t ovk_nbits_gemm_split(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int64_t m, void *y, int32_t y_dtype,
                             int64_t ldy, int64_t col0);

// True when the prefill product of this weight would run the kernel of this file (the one that
// can store into several ranks' matrices) rather than the two-term-scale kernel.
bool ovk_nbits_gemm_is_per_block(const ovk_ctx *ctx, const ovk_nbits_weight *w)
{
    return !ovk_nbits_gemm_split_applies(ctx, w);
}

// Y[:, col0 : col0 + N] = A x dequant(B) in each of the n_dst matrices of row pitch ldy
// (n_dst > 1: fp16 only, `view` describes the ranks and the call's epoch).
int32_t ovk_nbits_gemm_into(ovk_ctx *ctx, const ovk_nbits_weight *wc, const void *a, int64_t m, void *const *y_dst,
                            int n_dst, int64_t ldy, int64_t col0, int32_t y_dtype, const OvkCommView *view, void *y_multicast)
{
    // small blocks with fp16 scales: the scale goes into the weight (exactly, as two fp16 terms)
    if (ovk_nbits_gemm_split_applies(ctx, wc)) {
        if (n_dst != 1)
            return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: the two-term-scale kernel stores into one matrix");
        return ovk_nbits_gemm_split(ctx, wc, a, m, y_dst[0], y_dtype, ldy, col0);
    }
    ovk_nbits_weight *w = const_cast<ovk_nbits_weight *>(wc);  // the prefill copy is built lazily
    int32_t rc = ovk_nbits_gemm_prepack(ctx, w);
    if (rc != OVK_OK)
        return rc;
    int n_tiles = int(ceil_div64(w->n, BW));
    const int bs = int(w->block_size);
    const int unit_slabs = bs >= SLAB ? bs / SLAB : 1;
    const int units = int(w->gemm_k_pad / SLAB) / unit_slabs;
    Plan plan = plan_launch(ctx->sm_count, 285.0, m, n_tiles, units, unit_slabs, 1);
    // Pairs of CTAs on tiles of 256 columns: every CTA loads half the token rows of a slab.
    bool pair = false;
    // A launch that stores into three or more ranks is bound by the exchange, and there pairs lose: at 4 ranks
    // the fused gate/up shard took 0.351 ms on pairs against 0.235 ms on single CTAs (at 2 ranks 0.260 against
    // 0.276 ms).
    if (OVK_NBITS_PAIRS && bs >= SLAB && n_dst <= 2 && pair_capacity(ctx) > 0) {
        const int pairs = pair_capacity(ctx);
        const int wide_tiles = int(ceil_div64(w->n, 2 * BW));
        // Measured on 4096 tokens, blocks of 128: 464 against 488 us at K=3584 N=18944, 553 against 606 us at
        // K=18944 N=3584, equal at N=2368; blocks of 64 and 256 gain 18-21 %.  Only a weight whose last
        // wide tile would be mostly padding stays with single CTAs.
        if (2 * wide_tiles == n_tiles || n_tiles >= 15) {
            plan = plan_launch(pairs, 285.0, m, wide_tiles, units, unit_slabs, 2);
            plan.grid *= 2;
            n_tiles = wide_tiles;
            pair = true;
        }
    }
    const int bt = plan.bt;
    CUtensorMap tmAct;
    if (!ovk_make_tmap_2d(&tmAct, a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, uint64_t(w->k), uint64_t(m), uint64_t(w->k) * 2,
                          SLAB, uint32_t(pair ? bt / 2 : bt), CU_TENSOR_MAP_SWIZZLE_128B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: cuTensorMapEncodeTiled failed for A");
    CUtensorMap tmRaw;
    if (!ovk_make_tmap_2d(&tmRaw, w->gemm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->gemm_k_pad / 2),
                          uint64_t(w->gemm_n_pad), uint64_t(w->gemm_k_pad / 2), 32, BW, CU_TENSOR_MAP_SWIZZLE_NONE))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulNBits: cuTensorMapEncodeTiled failed for the packed weight");
    GemmParams p = {};
    p.wq = static_cast<const uint8_t *>(w->gemm_w);
    p.scales_t = w->gemm_scales_t;
    p.zp_t = w->gemm_zp_t;
    p.M = int(m);
    p.N = int(w->n);
    p.K = int(w->k);
    p.k_pad = int(w->gemm_k_pad);
    p.n_pad = int(w->gemm_n_pad);
    p.n_blocks = int(w->gemm_k_pad / w->block_size);
    p.zp_pitch = int(w->gemm_zp_pitch);
    p.slabs = int(w->gemm_k_pad / SLAB);
    p.bs = bs;
    p.bt = bt;
    p.ring = bt > 128 ? 2 : (bt > 96 ? 3 : 4);
    p.acc_stride = bt > 128 ? BT : (bt > 96 ? 128 : 96);
    p.m_tiles = int(ceil_div64(m, bt));
    p.n_tiles = n_tiles;
    p.y_f32 = y_dtype == OVK_FLOAT;
    p.status = ctx->dev_status;
    p.n_dst = n_dst;
    p.ldy = int(ldy);
    p.col0 = int(col0);
    p.vec_ok = (ldy % 8) == 0 && (col0 % 8) == 0;
    for (int r = 0; r < n_dst; r++) {
        p.y_dst[r] = y_dst[r];
        p.vec_ok = p.vec_ok && aligned_to(y_dst[r], 16);
    }
    if (view)
        p.comm = *view;
    p.y_mc = n_dst > 1 && aligned_to(y_multicast, 16) ? y_multicast : nullptr;
    p.units = units;
    p.unit_slabs = unit_slabs;
    p.unit_blocks = bs >= SLAB ? 1 : SLAB / bs;
    p.shared_k = plan.shared_k ? 1 : 0;
    if (plan.shared_k) {
        if (!ctx->tile_counters) {
            OVK_CUDA(ctx, cudaMalloc(&ctx->tile_counters, OVK_TILE_COUNTERS * sizeof(uint32_t)));
            OVK_CUDA(ctx, cudaMemsetAsync(ctx->tile_counters, 0, OVK_TILE_COUNTERS * sizeof(uint32_t), ctx->stream));
        }
        void *ws = nullptr;
        rc = ovk_scratch(ctx, size_t(plan.grid) * 2 * 2 * PART_FLOATS * sizeof(float), &ws);
        if (rc != OVK_OK)
            return rc;
        p.partials = static_cast<float *>(ws);
        p.counters = ctx->tile_counters;
    }
    if (pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(plan.grid);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = gemm_smem();
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        OVK_CUDA(ctx, cudaLaunchKernelEx(&cfg, nbits_gemm_kernel<true>, tmAct, tmRaw, p));
        OVK_LAUNCHED(ctx, plan.shared_k ? "nbits_gemm_tc_pair_shared_k" : "nbits_gemm_tc_pair");
        return OVK_OK;
    }
    OVK_CUDA(ctx, cudaFuncSetAttribute(nbits_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem())));
    nbits_gemm_kernel<false><<<plan.grid, THREADS, gemm_smem(), ctx->stream>>>(tmAct, tmRaw, p);
    OVK_LAUNCHED(ctx, plan.shared_k ? "nbits_gemm_tc_shared_k" : "nbits_gemm_tc");
    return OVK_OK;
}

int32_t ovk_nbits_gemm(ovk_ctx *ctx, const ovk_nbits_weight *wc, const void *a, int32_t a_dtype, int64_t m,
                       void *y, int32_t y_dtype)
{
    (void)a_dtype;
    void *dst[1] = {y};
    return ovk_nbits_gemm_into(ctx, wc, a, m, dst, 1, wc->n, 0, y_dtype, nullptr, nullptr);
}
