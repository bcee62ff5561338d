// MatMulInteger on the 5th-generation tensor cores: tcgen05.mma kind::i8 with
// int32 accumulators in tensor memory, operands staged by TMA, fused epilogue.
//
// This is the successor of the reference's production int8 GEMM
// (crates/onnx-vulkan-core/src/shaders/glsl/matmul_integer_coop_smem.comp:
// a 128x128 shared-memory block of 16x16x32 cooperative-matrix tiles with the
// zero-point algebra applied at the store, :306-345) and of its epilogue
// (matmul_integer_coop.comp:156-196).
//
// A persistent CTA per SM computes 128 x BN tiles of A[M,K] (u8/i8, row major)
// times Bt[N,K] (the packed weight, K contiguous), two tensor-memory
// accumulators so that a tile's epilogue overlaps the next tile's MMAs:
//   warp 0    TMA producer: 128-byte K slabs of A and Bt into a ring of
//             128B-swizzled stages, completion on an mbarrier per stage
//   warp 1    allocates tensor memory, issues four K=32 MMAs per stage from one
//             thread, frees the stage with tcgen05.commit
//   warps 2-5 epilogue: tcgen05.ld the accumulator (one row per thread),
//             sum ab - za*sum_k b - zb*sum_k a + K*za*zb, then the store
//             selected by EpiParams (int32 / dequantised f32 / requantised u8)
// kind::i8 takes signed and unsigned bytes per operand, so nothing is flipped
// (the reference's FLIP_BYTES pass, shaders/matmul_integer.rs:25-38, is not needed).
// Ragged M, N and K are handled by TMA zero fill plus store predicates.
#include "ovk_internal.h"
#include "epilogue.cuh"
#include "umma.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes of K per stage = one 128-byte swizzle row
constexpr int A_BYTES = BM * BK;
constexpr int THREADS = 352;  // TMA, issuer 0, four epilogue warps, issuer 1, four more epilogue warps
constexpr long long WAIT_CYCLES = 2000000000ll;  // about a second

// Several weights over the same A in one launch (q, k and v of an attention block): the tiles of all
// members form one list, a tile looks up its member, and only the columns' constants, the packed
// weight and the output differ.
constexpr int MAX_GROUP = 4;
struct TcMember {
    const int32_t *colsum;
    const float *scale, *product, *fbias;
    void *out;
    int N;
    int tile_end;  // number of column tiles of this member and those before it
};
struct TmGroup {
    CUtensorMap m[MAX_GROUP];
};
// What the epilogue needs to know about the columns it stores.
struct ColView {
    const int32_t *colsum;
    const float *scale, *product, *fbias;
    void *out;
    int N;
};

struct TcParams {
    int64_t M;
    int N, K, num_kb;
    const int32_t *colsum;
    const int32_t *rowsum;  // valid when b_zp may be non-zero
    const void *a_zp, *b_zp;
    int a_signed, b_signed;
    EpiParams epi;
    void *out;
    int vec_ok;  // output rows may be written with 16-byte (int32/f32) or 4-byte (u8) stores
    int tma_out; // 32-bit results leave through shared memory and bulk tensor stores (whole 128-byte lines)
    int *status;
    int members;  // 0: one weight (the fields above); else the group below
    TcMember mem[MAX_GROUP];
};

// Accesses to the member table use constant indices (unrolled loops, a switch), so that the parameter block
// is read where it lies and no copy of it is made.
__device__ __forceinline__ int column_tiles(const TcParams &p, int bn)
{
    if (!p.members)
        return (p.N + bn - 1) / bn;
    int t = p.mem[0].tile_end;
#pragma unroll
    for (int i = 1; i < MAX_GROUP; i++)
        if (i < p.members)
            t = p.mem[i].tile_end;
    return t;
}
// Column tile `nt` of the launch: which member it belongs to and where its columns start there.
__device__ __forceinline__ int member_of(const TcParams &p, int nt, int bn, int &n0)
{
    int j = 0, first = 0;
#pragma unroll
    for (int i = 0; i + 1 < MAX_GROUP; i++)
        if (i + 1 < p.members && nt >= p.mem[i].tile_end) {
            first = p.mem[i].tile_end;
            j = i + 1;
        }
    n0 = (nt - first) * bn;
    return j;
}
__device__ __forceinline__ ColView view_of(const TcMember &m)
{
    ColView v;
    v.colsum = m.colsum;
    v.scale = m.scale;
    v.product = m.product;
    v.fbias = m.fbias;
    v.out = m.out;
    v.N = m.N;
    return v;
}
__device__ __forceinline__ ColView columns_of(const TcParams &p, int j)
{
    if (p.members) {
        switch (j) {
        case 1:
            return view_of(p.mem[1]);
        case 2:
            return view_of(p.mem[2]);
        case 3:
            return view_of(p.mem[3]);
        default:
            return view_of(p.mem[0]);
        }
    }
    ColView v;
    v.colsum = p.colsum;
    v.scale = p.epi.scale;
    v.product = p.epi.product;
    v.fbias = p.epi.fbias;
    v.out = p.out;
    v.N = p.N;
    return v;
}
__device__ __forceinline__ const CUtensorMap *map_of(const TmGroup &g, int j)
{
    switch (j) {
    case 1:
        return &g.m[1];
    case 2:
        return &g.m[2];
    case 3:
        return &g.m[3];
    default:
        return &g.m[0];
    }
}

__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity)
{
    const long long t0 = clock64();
    while (!umma::mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > WAIT_CYCLES)
            return false;
    }
    return true;
}

// For warps that wait on someone else's progress: parked by the hardware (up to a
// microsecond per attempt) instead of spinning in the issue slots of the MMA warp.
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

// 32-bit results on their way out.  A thread holds one row of 32 columns; stored from registers that is one
// 16-byte piece per row and instruction, 32 rows apart in memory - measured ~2.3 TB/s over the whole GPU, which
// is what paced the products of a few GOP.  Instead the warp lays its 32 x 32 block down in shared memory (rows of
// 128 bytes, 16-byte pieces XOR-swizzled by the row so that the 32 lanes spread over all banks) and one lane
// hands it to the bulk tensor store, which writes whole lines and clips the block at the ends of M and N.
struct OutStage {
    uint8_t *buf;            // this warp's `depth` buffers of 4 KB, 1024-byte aligned; null: stores from registers
    const CUtensorMap *map;  // the output as a [M][N] tensor of 32-bit elements, box 32 x 32, 128-byte swizzle
    int depth;               // 1 or 2 buffers
    int seq;                 // blocks stored so far
};
__device__ __forceinline__ void stage_out_block(OutStage &st, const uint32_t (&v)[32], int lane, int col0, int row0, bool live)
{
    // the buffer about to be written has been read by the store that used it last
    if (st.seq >= st.depth && lane == 0) {
        if (st.depth == 2)
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        else
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    __syncwarp();
    uint8_t *buf = st.buf + (st.depth == 2 ? (st.seq & 1) * 4096 : 0);
    const uint32_t row = umma::smem_u32(buf) + uint32_t(lane) * 128u;
#pragma unroll
    for (int j = 0; j < 8; j++)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row + uint32_t((j ^ (lane & 7)) << 4)), "r"(v[4 * j]),
                     "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                     : "memory");
    umma::fence_proxy_async();  // the bulk store reads through the async proxy
    __syncwarp();
    if (lane == 0 && live) {
        umma::tma_store_2d(st.map, buf, col0, row0);
        umma::tma_store_commit();
    }
    st.seq++;
}
// before the warp leaves: its stores have completed
__device__ __forceinline__ void stage_out_drain(const OutStage &st, int lane)
{
    if (st.buf && lane == 0)
        umma::tma_store_wait_all();
}

// What the epilogue fetches from global memory for one block of 32 columns - lane l those of column col0 + l.
// None of it depends on the accumulator, so it is requested a block ahead (the first block's before the wait for
// the accumulator): fetched where it is used, each block of every tile exposed a full memory latency to the one
// warp of its scheduler, and a product with the Cast-Mul-Add epilogue took twice the time of the plain one.
struct ColConsts {
    int32_t cs;  // column sum of B (only read where A has a zero point)
    float s, b;  // EPI_SCALE: scale [* product], bias;  EPI_REQUANT: s = ratio
    int32_t ib;  // EPI_REQUANT: integer bias
};
__device__ __forceinline__ ColConsts col_consts(const TcParams &p, const ColView &v, int col_l, int32_t za)
{
    ColConsts c = {0, 0.0f, 0.0f, 0};
    if (col_l >= v.N)
        return c;
    if (za != 0)
        c.cs = v.colsum[col_l];
    if (p.epi.by_row) {
        // the constants belong to the rows
    } else if (p.epi.mode == EPI_SCALE) {
        c.s = v.scale[col_l * p.epi.scale_step];
        if (v.product)
            c.s = __fmul_rn(c.s, v.product[col_l * p.epi.product_step]);
        c.b = v.fbias[col_l * p.epi.bias_step];
    } else if (p.epi.mode == EPI_REQUANT) {
        c.s = p.epi.ratio[col_l * p.epi.ratio_step];
        c.ib = p.epi.ibias ? p.epi.ibias[col_l] : 0;
    }
    return c;
}
// ... and for the thread's row: the term of B's zero point and the constants of EpiParams::by_row
struct RowConsts {
    uint32_t row_term;
    float s, b;
    int32_t ib;
};
__device__ __forceinline__ RowConsts row_consts(const TcParams &p, const ColView &v, int64_t row, int32_t za, int32_t zb)
{
    RowConsts c = {uint32_t(p.K) * uint32_t(za) * uint32_t(zb), 0.0f, 0.0f, 0};
    if (row >= p.M)
        return c;
    if (zb != 0 && p.rowsum)
        c.row_term -= uint32_t(zb) * uint32_t(p.rowsum[row]);
    if (p.epi.by_row) {
        if (p.epi.mode == EPI_SCALE) {
            c.s = v.scale[row * p.epi.scale_step];
            if (v.product)
                c.s = __fmul_rn(c.s, v.product[row * p.epi.product_step]);
            c.b = v.fbias[row * p.epi.bias_step];
        } else if (p.epi.mode == EPI_REQUANT) {
            c.s = p.epi.ratio[row * p.epi.ratio_step];
            c.ib = p.epi.ibias ? p.epi.ibias[row] : 0;
        }
    }
    return c;
}

// The columns of one accumulator row block: tcgen05.ld 32 columns at a time (one row per thread),
// the zero-point terms, then the store selected by EpiParams.  `hand_back` gets this warp's arrival
// as soon as the last columns have been read, before they are processed.
// (`hand_back_at`: the same barrier by its address in the cluster's window, when it lives in the other CTA of a pair.)
template <int BN>
__device__ __forceinline__ void epilogue_columns(const TcParams &p, const ColView &v, uint32_t taddr, uint64_t *hand_back,
                                                 int lane, int64_t row, bool row_ok, int n0, const RowConsts &rc, ColConsts cur,
                                                 int32_t za, float &run_max, float &run_neg, OutStage &st, bool live,
                                                 uint32_t hand_back_at = 0, int c_first = 0, int c_step = 32)
{
    // (`c_first`, `c_step`: the blocks of 32 columns this warp takes - all of them, or every other one where two
    // warps share a lane quarter)
    const uint32_t row_term = rc.row_term;
    // (The ragged-edge store loops below are unrolled by pragma: left to itself the compiler indexed the
    // 32 accumulators at run time there, which put all of them in local memory - every int8 kernel ran
    // 8-28 % slower.)
    const bool vec4 = p.vec_ok != 0;
    // constants that belong to this thread's row rather than to the columns (EpiParams::by_row)
    const bool by_row = p.epi.by_row != 0;
    const float s_row = rc.s, b_row = rc.b;
    const int32_t ib_row = rc.ib;
#pragma unroll 1
    for (int c0 = c_first; c0 < BN; c0 += c_step) {
        uint32_t r[32];
        umma::tmem_ld_32x32(taddr + uint32_t(c0), r);
        // the next block's constants travel while this one is worked on
        const ColConsts here = cur;
        if (c0 + c_step < BN)
            cur = col_consts(p, v, n0 + c0 + c_step + lane, za);
        umma::tmem_ld_wait();
        if (c0 + c_step >= BN) {  // this warp has read its part of the accumulator: hand it back
            umma::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (hand_back_at)
                    umma::mbar_arrive_cluster(hand_back_at);
                else
                    umma::mbar_arrive(hand_back);
            }
        }
        if (n0 + c0 >= v.N)  // the same for every lane of the warp
            continue;
        const int col0 = n0 + c0;
        // Every thread of the warp needs the constants of the same 32 columns (a thread is a row).
        // Lane l fetches those of column col0 + l - coalesced loads, all in flight together - and the
        // loop below takes them by shuffle; a load per element from every thread made the
        // dequantising store several times as long as the int32 one.  All lanes take part, rows past
        // M included; only the stores are predicated.
        const int32_t cs_l = here.cs, ib_l = here.ib;
        const float s_l = here.s, b_l = here.b;
        if (za != 0) {
#pragma unroll
            for (int j = 0; j < 32; j++)
                r[j] = r[j] - uint32_t(za) * uint32_t(__shfl_sync(0xffffffffu, cs_l, j)) + row_term;
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                r[j] += row_term;
        }
        if (p.epi.mode == EPI_RAW) {
            int32_t *o = static_cast<int32_t *>(v.out) + row * v.N + col0;
            if (st.buf) {
                stage_out_block(st, r, lane, col0, int(row) - lane, live);
            } else if (!row_ok) {
                // a row past M: nothing to store (no divergent `continue`: the next tcgen05.ld is warp-wide)
            } else if (vec4 && col0 + 32 <= v.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<int4 *>(o + j) = make_int4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < v.N)
                        o[j] = int32_t(r[j]);
            }
        } else if (p.epi.mode == EPI_SCALE) {
            // fl(fl(float(acc) * s) + bias) [Relu], as epi_scale_value computes it
            const bool relu = p.epi.flags & 1u;
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float sj = by_row ? s_row : __shfl_sync(0xffffffffu, s_l, j);
                const float bj = by_row ? b_row : __shfl_sync(0xffffffffu, b_l, j);
                const float z = __fadd_rn(__fmul_rn(float(int32_t(r[j])), sj), bj);
                f[j] = relu ? fmaxf(z, 0.0f) : z;
                if (row_ok && col0 + j < v.N) {
                    run_max = fmaxf(run_max, f[j]);
                    run_neg = fmaxf(run_neg, -f[j]);
                }
            }
            float *o = static_cast<float *>(v.out) + row * v.N + col0;
            if (st.buf) {
                uint32_t bits[32];
#pragma unroll
                for (int j = 0; j < 32; j++)
                    bits[j] = __float_as_uint(f[j]);
                stage_out_block(st, bits, lane, col0, int(row) - lane, live);
            } else if (!row_ok) {
            } else if (vec4 && col0 + 32 <= v.N) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(o + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < v.N)
                        o[j] = f[j];
            }
        } else {
            // sat(rne(f32(acc + bias) * ratio) + y_zp), as epi_requant_value computes it
            uint32_t q8[32];
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float ratio = by_row ? s_row : __shfl_sync(0xffffffffu, s_l, j);
                const int32_t acc = int32_t(r[j] + uint32_t(by_row ? ib_row : __shfl_sync(0xffffffffu, ib_l, j)));
                // (the conversion rounds to nearest even itself: the same value as converting rintf of it)
                int32_t qv = int32_t(uint32_t(__float2int_rn(__fmul_rn(float(acc), ratio))) + uint32_t(p.epi.y_zp));
                qv = p.epi.y_signed ? max(-128, min(127, qv)) : max(0, min(255, qv));
                q8[j] = uint32_t(qv) & 0xffu;
            }
            uint8_t *o = static_cast<uint8_t *>(v.out) + row * v.N + col0;
            if (!row_ok) {
            } else if (vec4 && col0 + 32 <= v.N) {
                uint32_t w8[8];
#pragma unroll
                for (int j = 0; j < 8; j++)
                    w8[j] = q8[4 * j] | (q8[4 * j + 1] << 8) | (q8[4 * j + 2] << 16) | (q8[4 * j + 3] << 24);
                // a thread's 32 bytes are one sector of its row: as two 16-byte stores where the row allows it
                // (as eight 4-byte ones the same product took 1.6 times as long as with its 32-bit results)
                if ((reinterpret_cast<uintptr_t>(o) & 15u) == 0) {
                    *reinterpret_cast<uint4 *>(o) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
                    *reinterpret_cast<uint4 *>(o + 16) = make_uint4(w8[4], w8[5], w8[6], w8[7]);
                } else {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        *reinterpret_cast<uint32_t *>(o + 4 * j) = w8[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (col0 + j < v.N)
                        o[j] = uint8_t(q8[j]);
            }
        }
    }
}

template <int BN> constexpr int stages_for() { return BN == 256 ? 4 : (BN == 128 ? 6 : 8); }
constexpr int OUT_STAGE_BYTES = 8 * 4096;  // eight epilogue warps, a 32 x 32 block of 32-bit results each (the pair kernel: its own split)
template <int BN> constexpr size_t smem_for()
{
    return size_t(stages_for<BN>()) * (A_BYTES + BN * BK) + 1024 /*alignment slack*/ + 256 /*barriers*/ + OUT_STAGE_BYTES +
           1024 /*its alignment*/;
}

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
mmi_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ TmGroup tmBs, const __grid_constant__ TmGroup tmYs,
              const __grid_constant__ TcParams p)
{
    constexpr int STAGES = stages_for<BN>();
    constexpr int B_BYTES = BN * BK;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA = smem;
    uint8_t *sB = smem + STAGES * A_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(sB + STAGES * B_BYTES);
    uint64_t *empty = full + STAGES;
    uint64_t *acc_full = empty + STAGES;   // [2] a tile's accumulator is complete
    uint64_t *acc_empty = acc_full + 2;    // [2] the eight epilogue warps have read it
    uint64_t *started = acc_empty + 2;     // [2] the tile's first (overwriting) MMA has been issued
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(started + 2);
    uint8_t *out_stage = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 1023) & ~uintptr_t(1023));

    OVK_PDL_LAUNCH_DEPENDENTS();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // persistent: tiles are taken round robin, N fastest so that CTAs running together share rows of A
    const int n_tiles = column_tiles(p, BN);
    const int total_tiles = n_tiles * int((p.M + BM - 1) / BM);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            umma::mbar_init(&full[s], 1);
            umma::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            umma::mbar_init(&acc_full[b], 2);  // one arrival per issuing thread
            umma::mbar_init(&acc_empty[b], 8);
            umma::mbar_init(&started[b], 1);
        }
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        umma::tmem_alloc(tmem_slot, 2 * BN);  // two accumulators: the epilogue of a tile overlaps the next tile's MMAs
        umma::tmem_relinquish();
    }
    umma::tc_fence_before();
    __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    OVK_PDL_WAIT();  // barriers and tensor memory were set up while the previous kernel drained

    if (warp == 0) {
        if (lane == 0) {
            umma::prefetch_tmap(&tmA);
#pragma unroll
            for (int j = 0; j < MAX_GROUP; j++)
                if (j < max(p.members, 1))
                    umma::prefetch_tmap(&tmBs.m[j]);
            int s = 0;
            uint32_t ph = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int m0 = (tile / n_tiles) * BM;
                int n0;
                const CUtensorMap *tmB = map_of(tmBs, member_of(p, tile % n_tiles, BN, n0));
                for (int kb = 0; kb < p.num_kb; kb++) {
                    if (!wait_parked(&empty[s], ph ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = total_tiles;
                        break;
                    }
                    umma::mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    umma::tma_load_2d(sA + s * A_BYTES, &tmA, &full[s], kb * BK, m0);
                    umma::tma_load_2d(sB + s * B_BYTES, tmB, &full[s], kb * BK, n0);
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 6) {
        // Two issuing threads, on two schedulers, take alternate K stages of every tile.  One
        // thread's round per stage (barrier poll, fence, four MMAs, commit) is a chain of several
        // hundred clocks; with narrow tiles (four 48- or 64-clock MMAs per stage) that chain is
        // longer than the MMAs, and a single issuer set the pace of the short-K products (T=1000,
        // K=4096, N=1024: 12.9 -> 10.9 us).  The 256-wide tiles, whose MMAs outlast the chain,
        // measure the same with one issuer or two.  Integer accumulation is exact and commutative, so the order in
        // which the two streams reach the tensor core does not change a bit of the result; the
        // one MMA that must come first is the tile's overwriting one, and the other thread waits
        // for `started` before its first MMA of the tile.
        if (lane == 0) {
            const int me = warp == 1 ? 0 : 1;
            const uint32_t idesc = umma::instr_desc(2, p.a_signed ? 1 : 0, p.b_signed ? 1 : 0, BM, BN);
            // descriptor high words are constants and low words advance by additions, so
            // an issuing thread spends a few instructions per MMA
            const uint32_t desc_hi = ((1024u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW128 << 29);
            const uint32_t a16 = umma::smem_u32(sA) >> 4, b16 = umma::smem_u32(sB) >> 4;
            bool ok = true;
            int s = 0, b = 0;
            uint32_t ph = 0, acc_ph = 0, turn = 0;  // turn: whose stage the next one is
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (!wait_bounded(&acc_empty[b], acc_ph ^ 1)) {
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    break;
                }
                umma::tc_fence_after();
                const uint32_t d = tmem_base + uint32_t(b * BN);
                bool issued = false;
                for (int kb = 0; kb < p.num_kb; kb++, turn ^= 1) {
                    if (turn == uint32_t(me)) {
                        if (!wait_bounded(&full[s], ph)) {
                            atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                            ok = false;
                            break;
                        }
                        if (kb != 0 && !issued && !wait_bounded(&started[b], acc_ph)) {
                            atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                            ok = false;
                            break;
                        }
                        umma::tc_fence_after();
                        const uint32_t a_lo = ((a16 + uint32_t(s) * (A_BYTES >> 4)) & 0x3fffu) | (1u << 16);
                        const uint32_t b_lo = ((b16 + uint32_t(s) * (B_BYTES >> 4)) & 0x3fffu) | (1u << 16);
                        umma::mma_i8_lohi(d, a_lo, desc_hi, b_lo, desc_hi, idesc, kb != 0);
                        if (kb == 0) {
                            // The other thread's first MMA of this tile must reach the tensor core after this
                            // overwriting one.  The order comes from the fence pair - before_thread_sync here,
                            // after_thread_sync behind the other thread's wait on `started` - together with the
                            // tensor core running the MMAs on one accumulator in the order it was given them.
                            umma::tc_fence_before();
                            umma::mbar_arrive(&started[b]);
                        }
                        umma::mma_i8_lohi(d, a_lo + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                        umma::mma_i8_lohi(d, a_lo + 4, desc_hi, b_lo + 4, desc_hi, idesc, 1u);
                        umma::mma_i8_lohi(d, a_lo + 6, desc_hi, b_lo + 6, desc_hi, idesc, 1u);
                        umma::mma_commit(&empty[s]);
                        issued = true;
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) {
                    if (issued)
                        umma::mma_commit(&acc_full[b]);  // arrives when this thread's MMAs have finished
                    else
                        umma::mbar_arrive(&acc_full[b]);  // a tile of one stage: nothing of this thread's to wait for
                }
                if (++b == 2) {
                    b = 0;
                    acc_ph ^= 1;
                }
            }
        }
    } else {
        // Epilogue: warp w may read tensor-memory lanes 32*(w % 4) .. +31.  Two warps per lane quarter (2-5 and
        // 7-10), one on the even and one on the odd blocks of 32 columns: the products of a few GOP are paced
        // by this part (conversions, shuffles, stores; the MMAs of a short K are over long before), and one
        // warp per scheduler left most of its issue slots to dependency stalls.
        const int q = warp & 3;
        const int ew = warp < 6 ? warp - 2 : warp - 3;  // 0..7
        const int c_first = (ew >> 2) * 32;
        const int32_t za = load_zp(p.a_zp, p.a_signed), zb = load_zp(p.b_zp, p.b_signed);
        float run_max = 0.0f, run_neg = 0.0f;
        OutStage st = {p.tma_out ? out_stage + ew * 4096 : nullptr, nullptr, 1, 0};
        bool ready = true;
        int b = 0;
        uint32_t acc_ph = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int64_t m0 = int64_t(tile / n_tiles) * BM;
            int n0;
            const int member = member_of(p, tile % n_tiles, BN, n0);
            const ColView cols = columns_of(p, member);
            st.map = map_of(tmYs, member);
            // what the epilogue reads from memory is asked for before the accumulator is waited for
            const int64_t row = m0 + q * 32 + lane;
            const RowConsts rc = row_consts(p, cols, row, za, zb);
            const ColConsts first = col_consts(p, cols, n0 + c_first + lane, za);
            if (ready && !wait_parked(&acc_full[b], acc_ph)) {
                ready = false;
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
            }
            umma::tc_fence_after();
            const bool row_ok = ready && row < p.M;
            epilogue_columns<BN>(p, cols, tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b * BN), &acc_empty[b], lane, row,
                                 row_ok, n0, rc, first, za, run_max, run_neg, st, ready, 0, c_first, 64);
            if (++b == 2) {
                b = 0;
                acc_ph ^= 1;
            }
        }
        stage_out_drain(st, lane);
        if (p.epi.mode == EPI_SCALE)
            epi_fold_range(p.epi, run_max, run_neg);
    }
    umma::tc_fence_before();
    __syncthreads();
    if (warp == 1)
        umma::tmem_dealloc(tmem_base, 2 * BN);
}

// ---------------------------------------------------------------------------
// 256 x 256 tiles for large products.  A 128 x 256 tile takes 12 KB of operands
// per K = 32 step, which at the tensor core's rate is more than the shared-memory
// ring can keep in flight over the latency of the L2; a 256 x 256 tile (two
// M = 128 MMAs per step sharing the B stage, the two accumulators filling all 512
// tensor-memory columns) takes 16 KB per TWO steps' worth of MACs.  With no
// spare accumulator a tile's epilogue does not overlap the next tile's MMAs,
// which is cheap for the long K this kernel is chosen for.  Stages are 64 bytes
// of K (six of 32 KB, 64B swizzle) so that five can be in flight.
//   warp 0      TMA producer
//   warp 1      tensor-memory allocation, MMA issue
//   warps 2-9   epilogue: warps 2-5 the upper 128 rows, 6-9 the lower
constexpr int BM2 = 256, BN2 = 256, BK2 = 64, STAGES2 = 6;
constexpr int A2_BYTES = BM2 * BK2, B2_BYTES = BN2 * BK2;
constexpr int THREADS2 = 11 * 32;  // TMA, issuer 0, eight epilogue warps, issuer 1
constexpr size_t SMEM2 = size_t(STAGES2) * (A2_BYTES + B2_BYTES) + 1024 + 256 + 8 * 4096 /*one block per epilogue warp*/ + 1024;

// PAIR: clusters of two CTAs on tiles of 512 x 256.  CTA `crank` owns rows crank * 256 .. + 255 of the tile (its A
// stage, its accumulators, its epilogue, exactly as a single CTA owns its 256) but loads only HALF of the
// B stage: tcgen05.mma.cta_group::2 (M = 256: 128 rows from each CTA) reads B half from each CTA's shared
// memory, so a CTA pulls 24 KB instead of 32 KB out of the L2 per K step - the L2, not the tensor core,
// paces this kernel.  Both CTAs' loads are counted at CTA 0's `full` barrier, one thread pair of CTA 0
// issues, completions are signalled to the barriers of both CTAs.
template <bool PAIR>
__global__ void __launch_bounds__(THREADS2, 1)
mmi_tc256_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmY, const __grid_constant__ TcParams p)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sA = smem;
    // a CTA of a pair holds half of a B stage, which leaves room for a second staging block per epilogue warp
    constexpr int B_STAGE = PAIR ? B2_BYTES / 2 : B2_BYTES;
    constexpr int OUT_DEPTH = PAIR ? 2 : 1;
    uint8_t *sB = smem + STAGES2 * A2_BYTES;
    uint64_t *full = reinterpret_cast<uint64_t *>(sB + STAGES2 * B_STAGE);
    uint64_t *empty = full + STAGES2;
    uint64_t *acc_full = empty + STAGES2;  // the tile's accumulators are complete
    uint64_t *acc_empty = acc_full + 1;    // the eight epilogue warps have read them
    uint64_t *started = acc_empty + 1;     // the tile's first (overwriting) MMAs have been issued
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(started + 1);
    uint8_t *out_stage = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(tmem_slot + 2) + 1023) & ~uintptr_t(1023));

    OVK_PDL_LAUNCH_DEPENDENTS();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = PAIR ? umma::cluster_rank() : 0u;
    const int vcta = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x), vgrid = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
    constexpr int TM = PAIR ? 2 * BM2 : BM2;  // rows of a tile number
    const int n_tiles = (p.N + BN2 - 1) / BN2;
    const int total_tiles = n_tiles * int((p.M + TM - 1) / TM);
    const int num_kb = (p.K + BK2 - 1) / BK2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES2; s++) {
            umma::mbar_init(&full[s], 1);
            umma::mbar_init(&empty[s], 1);
        }
        umma::mbar_init(acc_full, 2);  // one arrival per issuing thread
        umma::mbar_init(acc_empty, PAIR ? 16 : 8);
        umma::mbar_init(started, 1);
        umma::fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            umma::tmem_alloc_pair(tmem_slot, 512);
            umma::tmem_relinquish_pair();
        } else {
            umma::tmem_alloc(tmem_slot, 512);
            umma::tmem_relinquish();
        }
    }
    umma::tc_fence_before();
    if constexpr (PAIR)
        umma::cluster_sync_all();  // the other CTA's barriers are initialised before anything is counted there
    else
        __syncthreads();
    umma::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    OVK_PDL_WAIT();  // barriers and tensor memory were set up while the previous kernel drained

    if (warp == 0) {
        if (lane == 0) {
            umma::prefetch_tmap(&tmA);
            umma::prefetch_tmap(&tmB);
            int s = 0;
            uint32_t ph = 0;
            const uint32_t full_at = PAIR ? umma::mbar_in_cta(&full[0], 0) : 0u;  // CTA 0 counts both CTAs' bytes
            for (int tile = vcta; tile < total_tiles; tile += vgrid) {
                const int m0 = (tile / n_tiles) * TM + int(crank) * BM2;
                const int n0 = (tile % n_tiles) * BN2 + (PAIR ? int(crank) * (BN2 / 2) : 0);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!wait_parked(&empty[s], ph ^ 1)) {
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                        tile = total_tiles;
                        break;
                    }
                    if constexpr (PAIR) {
                        if (crank == 0)
                            umma::mbar_expect_tx(&full[s], 2 * (A2_BYTES + B2_BYTES / 2));
                        umma::tma_load_2d_pair(sA + s * A2_BYTES, &tmA, full_at + uint32_t(s) * 8u, kb * BK2, m0);
                        umma::tma_load_2d_pair(sB + s * B_STAGE, &tmB, full_at + uint32_t(s) * 8u, kb * BK2, n0);
                        if (++s == STAGES2) {
                            s = 0;
                            ph ^= 1;
                        }
                        continue;
                    }
                    umma::mbar_expect_tx(&full[s], A2_BYTES + B2_BYTES);
                    umma::tma_load_2d(sA + s * A2_BYTES, &tmA, &full[s], kb * BK2, m0);
                    umma::tma_load_2d(sB + s * B_STAGE, &tmB, &full[s], kb * BK2, n0);
                    if (++s == STAGES2) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 10) {
        // two issuing threads on alternate K stages, as in mmi_tc_kernel
        if (lane == 0 && crank == 0) {
            const int me = warp == 1 ? 0 : 1;
            const uint32_t idesc = umma::instr_desc(2, p.a_signed ? 1 : 0, p.b_signed ? 1 : 0, PAIR ? 256 : 128, BN2);
            // 64-byte rows, 64B swizzle: 512 bytes between 8-row groups
            const uint32_t desc_hi = ((512u >> 4) & 0x3fffu) | (1u << 14) | (umma::LAYOUT_SW64 << 29);
            const uint32_t a16 = (umma::smem_u32(sA) >> 4) | (1u << 16), b16 = (umma::smem_u32(sB) >> 4) | (1u << 16);
            constexpr uint32_t HALF = (128 * BK2) >> 4;  // the lower 128 rows of a stage of A
            bool ok = true;
            int s = 0;
            uint32_t ph = 0, acc_ph = 0, turn = 0;
            for (int tile = vcta; tile < total_tiles && ok; tile += vgrid) {
                if (!wait_bounded(acc_empty, acc_ph ^ 1)) {
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                    break;
                }
                umma::tc_fence_after();
                bool issued = false;
                for (int kb = 0; kb < num_kb; kb++, turn ^= 1) {
                    if (turn == uint32_t(me)) {
                        if (!wait_bounded(&full[s], ph)) {
                            atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
                            ok = false;
                            break;
                        }
                        if (kb != 0 && !issued && !wait_bounded(started, acc_ph)) {
                            atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
                            ok = false;
                            break;
                        }
                        umma::tc_fence_after();
                        const uint32_t a_lo = a16 + uint32_t(s) * (A2_BYTES >> 4);
                        const uint32_t b_lo = b16 + uint32_t(s) * (B_STAGE >> 4);
                        const uint32_t acc = kb != 0;
                        if constexpr (PAIR) {
                            umma::mma_i8_lohi_pair(tmem_base, a_lo, desc_hi, b_lo, desc_hi, idesc, acc);
                            umma::mma_i8_lohi_pair(tmem_base + BN2, a_lo + HALF, desc_hi, b_lo, desc_hi, idesc, acc);
                        } else {
                            umma::mma_i8_lohi(tmem_base, a_lo, desc_hi, b_lo, desc_hi, idesc, acc);
                            umma::mma_i8_lohi(tmem_base + BN2, a_lo + HALF, desc_hi, b_lo, desc_hi, idesc, acc);
                        }
                        if (kb == 0) {
                            umma::tc_fence_before();  // orders both overwriting MMAs before the other thread's (see mmi_tc_kernel)
                            umma::mbar_arrive(started);
                        }
                        if constexpr (PAIR) {
                            umma::mma_i8_lohi_pair(tmem_base, a_lo + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                            umma::mma_i8_lohi_pair(tmem_base + BN2, a_lo + HALF + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                            umma::mma_commit_pair(&empty[s]);
                        } else {
                            umma::mma_i8_lohi(tmem_base, a_lo + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                            umma::mma_i8_lohi(tmem_base + BN2, a_lo + HALF + 2, desc_hi, b_lo + 2, desc_hi, idesc, 1u);
                            umma::mma_commit(&empty[s]);
                        }
                        issued = true;
                    }
                    if (++s == STAGES2) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (ok) {
                    if constexpr (PAIR) {
                        if (issued) {
                            umma::mma_commit_pair(acc_full);
                        } else {
                            umma::mbar_arrive(acc_full);
                            umma::mbar_arrive_cluster(umma::mbar_in_cta(acc_full, 1));
                        }
                    } else {
                        if (issued)
                            umma::mma_commit(acc_full);
                        else
                            umma::mbar_arrive(acc_full);
                    }
                }
                acc_ph ^= 1;
            }
        }
    } else if (warp >= 2 && warp < 10) {
        const int q = warp & 3;           // tensor-memory lane quarter this warp may read
        const int half = (warp - 2) >> 2;  // upper or lower 128 rows of this CTA's rows of the tile
        const uint32_t acc_empty_at = PAIR ? umma::mbar_in_cta(acc_empty, 0) : 0u;
        const int32_t za = load_zp(p.a_zp, p.a_signed), zb = load_zp(p.b_zp, p.b_signed);
        float run_max = 0.0f, run_neg = 0.0f;
        OutStage st = {p.tma_out ? out_stage + (warp - 2) * OUT_DEPTH * 4096 : nullptr, &tmY, OUT_DEPTH, 0};
        bool ready = true;
        uint32_t acc_ph = 0;
        for (int tile = vcta; tile < total_tiles; tile += vgrid) {
            const int64_t m0 = int64_t(tile / n_tiles) * TM + int64_t(crank) * BM2 + half * 128;
            const int n0 = (tile % n_tiles) * BN2;
            const int64_t row = m0 + q * 32 + lane;
            const ColView cols = columns_of(p, 0);
            const RowConsts rc = row_consts(p, cols, row, za, zb);
            const ColConsts first = col_consts(p, cols, n0 + lane, za);
            if (ready && !wait_parked(acc_full, acc_ph)) {
                ready = false;
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_MMA);
            }
            umma::tc_fence_after();
            const bool row_ok = ready && row < p.M;
            epilogue_columns<BN2>(p, cols, tmem_base + (uint32_t(q * 32) << 16) + uint32_t(half * BN2), acc_empty,
                                  lane, row, row_ok, n0, rc, first, za, run_max, run_neg, st, ready, acc_empty_at);
            acc_ph ^= 1;
        }
        stage_out_drain(st, lane);
        if (p.epi.mode == EPI_SCALE)
            epi_fold_range(p.epi, run_max, run_neg);
    }
    umma::tc_fence_before();
    if constexpr (PAIR) {
        umma::cluster_sync_all();  // the other CTA's MMAs write this CTA's tensor memory too
        if (warp == 1)
            umma::tmem_dealloc_pair(tmem_base, 512);
    } else {
        __syncthreads();
        if (warp == 1)
            umma::tmem_dealloc(tmem_base, 512);
    }
}

// sum_k a[m][k] per row, needed only when the weight's zero point is not 0:
// exits at once otherwise (the zero point is read on the device, never on the host).
__global__ void __launch_bounds__(256)
mmi_rowsum_kernel(const uint8_t *__restrict__ a, int64_t M, int K, int a_signed, const void *b_zp,
                  int b_signed, int32_t *__restrict__ rowsum)
{
    OVK_PDL_LAUNCH_DEPENDENTS();
    OVK_PDL_WAIT();
    if (load_zp(b_zp, b_signed) == 0)
        return;
    const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= M)
        return;
    const uint32_t *aw = reinterpret_cast<const uint32_t *>(a + row * K);  // K % 16 == 0, base 16-byte aligned
    int32_t s = 0;
    for (int w = lane; w < K / 4; w += 32) {
        const uint32_t x = aw[w];
        s = a_signed ? __dp4a(int(x), int(0x01010101), s) : int32_t(__dp4a(x, 0x01010101u, uint32_t(s)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        rowsum[row] = s;
}

// The output of one weight as a [M][N] tensor of 32-bit elements for the bulk stores of the epilogue.
bool out_map(CUtensorMap *map, void *out, int64_t m, int64_t n, bool f32)
{
    return ovk_make_tmap_2d(map, out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_INT32, uint64_t(n),
                            uint64_t(m), uint64_t(n) * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
}

template <int BN>
int32_t launch(ovk_ctx *ctx, const CUtensorMap &tmA, const ovk_mmi_weight *const *ws, int count, TcParams p)
{
    TmGroup tmBs = {}, tmYs = {};
    // 32-bit results (int32, or f32 after scale and bias) of rows that take 16-byte accesses leave by bulk stores
    p.tma_out = p.vec_ok && p.epi.mode != EPI_REQUANT;
    for (int j = 0; j < count && p.tma_out; j++)
        if (!out_map(&tmYs.m[j], p.members ? p.mem[j].out : p.out, p.M, ws[j]->n, p.epi.mode == EPI_SCALE))
            p.tma_out = 0;
    int64_t col_tiles = 0;
    for (int j = 0; j < count; j++) {
        if (!ovk_make_tmap_2d(&tmBs.m[j], ws[j]->bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(ws[j]->k_pad),
                              uint64_t(ws[j]->n_pad), uint64_t(ws[j]->k_pad), BK, BN, CU_TENSOR_MAP_SWIZZLE_128B))
            return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger: cuTensorMapEncodeTiled failed for the packed weight");
        col_tiles += ceil_div64(ws[j]->n, BN);
        if (p.members)
            p.mem[j].tile_end = int(col_tiles);
    }
    OVK_CUDA(ctx, cudaFuncSetAttribute(mmi_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(smem_for<BN>())));
    const int64_t tiles = col_tiles * ceil_div64(p.M, BM);
    const unsigned grid = unsigned(std::min<int64_t>(tiles, ctx->sm_count));
    OVK_CUDA(ctx, ovk_launch_pdl(mmi_tc_kernel<BN>, dim3(grid), dim3(THREADS), smem_for<BN>(), ctx->stream, tmA, tmBs, tmYs, p));
    OVK_LAUNCHED(ctx, BN == 256 ? "mmi_tc_128x256" : (BN == 128 ? "mmi_tc_128x128" : "mmi_tc_128x64"));
    return OVK_OK;
}

// Largest tile that still gives every SM a CTA; the smallest one otherwise
// (the reference picks 64x64 blocks under 64 workgroups, shaders/matmul_integer.rs:467-487).
int32_t launch_by_fill(ovk_ctx *ctx, const CUtensorMap &tmA, const ovk_mmi_weight *const *ws, int count, const TcParams &p)
{
    const int64_t mt = ceil_div64(p.M, BM);
    auto col_tiles = [&](int bn) {
        int64_t t = 0;
        for (int j = 0; j < count; j++)
            t += ceil_div64(ws[j]->n, bn);
        return t;
    };
    int64_t narrowest = ws[0]->n;
    for (int j = 1; j < count; j++)
        narrowest = std::min(narrowest, ws[j]->n);
    if (narrowest >= 256 && mt * col_tiles(256) >= ctx->sm_count)
        return launch<256>(ctx, tmA, ws, count, p);
    if (narrowest >= 128 && mt * col_tiles(128) >= ctx->sm_count)
        return launch<128>(ctx, tmA, ws, count, p);
    return launch<64>(ctx, tmA, ws, count, p);
}

// 256 x 256 tiles: chosen for long K (the epilogue is not overlapped) and enough tiles to keep the
// SMs in whole waves.
#ifndef OVK_MMI_PAIRS
#define OVK_MMI_PAIRS 1
#endif
// How many pairs of CTAs of the pair kernel the GPU runs at once (0: clusters unavailable).
int pair_capacity(ovk_ctx *ctx)
{
    if (ctx->mmi_pairs >= 0)
        return ctx->mmi_pairs;
    ctx->mmi_pairs = 0;
    if (cudaFuncSetAttribute(mmi_tc256_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM2)) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(ctx->sm_count & ~1));
    cfg.blockDim = dim3(THREADS2);
    cfg.dynamicSmemBytes = SMEM2;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, mmi_tc256_kernel<true>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    ctx->mmi_pairs = clusters;
    return clusters;
}

int32_t launch256(ovk_ctx *ctx, const void *a, const ovk_mmi_weight *w, TcParams p)
{
    CUtensorMap tmY = {};
    p.tma_out = p.vec_ok && p.epi.mode != EPI_REQUANT && out_map(&tmY, p.out, p.M, w->n, p.epi.mode == EPI_SCALE);
    const int pairs = OVK_MMI_PAIRS ? pair_capacity(ctx) : 0;
    const bool pair = pairs > 0 && p.M > BM2;  // at least two row blocks to share a B tile
    CUtensorMap tmA, tmB;
    if (!ovk_make_tmap_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->k), uint64_t(p.M), uint64_t(w->k), BK2,
                          BM2, CU_TENSOR_MAP_SWIZZLE_64B) ||
        !ovk_make_tmap_2d(&tmB, w->bt, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->k_pad), uint64_t(w->n_pad),
                          uint64_t(w->k_pad), BK2, pair ? BN2 / 2 : BN2, CU_TENSOR_MAP_SWIZZLE_64B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger: cuTensorMapEncodeTiled failed (256 x 256 tiles)");
    if (pair) {
        const int64_t tiles = ceil_div64(p.N, BN2) * ceil_div64(p.M, 2 * BM2);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2u * unsigned(std::min<int64_t>(tiles, pairs)));
        cfg.blockDim = dim3(THREADS2);
        cfg.dynamicSmemBytes = SMEM2;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        OVK_CUDA(ctx, cudaLaunchKernelEx(&cfg, mmi_tc256_kernel<true>, tmA, tmB, tmY, p));
        OVK_LAUNCHED(ctx, "mmi_tc_pair_512x256");
        return OVK_OK;
    }
    OVK_CUDA(ctx, cudaFuncSetAttribute(mmi_tc256_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM2)));
    const int64_t tiles = ceil_div64(p.N, BN2) * ceil_div64(p.M, BM2);
    const unsigned grid = unsigned(std::min<int64_t>(tiles, ctx->sm_count));
    OVK_CUDA(ctx, ovk_launch_pdl(mmi_tc256_kernel<false>, dim3(grid), dim3(THREADS2), SMEM2, ctx->stream, tmA, tmB, tmY, p));
    OVK_LAUNCHED(ctx, "mmi_tc_256x256");
    return OVK_OK;
}

bool wants256(const ovk_ctx *ctx, const ovk_mmi_weight *w, int64_t m)
{
    if (SMEM2 > ctx->smem_optin || m >= (int64_t(1) << 31) - BM2)
        return false;
    if (w->k < 2048 || w->n < 256 || m < 256)
        return false;
    const int64_t tiles = ceil_div64(w->n, BN2) * ceil_div64(m, BM2);
    // at least three waves, or an almost full last wave
    const int64_t waves = ceil_div64(tiles, ctx->sm_count);
    return tiles >= 3 * int64_t(ctx->sm_count) || (tiles >= ctx->sm_count && tiles * 10 >= waves * ctx->sm_count * 9);
}

}  // namespace

bool ovk_mmi_wants_large_tiles(const ovk_ctx *ctx, const ovk_mmi_weight *w, int64_t m) { return wants256(ctx, w, m); }

int32_t ovk_mmi_tc_launch_with_row_sums(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed, int64_t m,
                                        const void *a_zp, const void *b_zp, const EpiParams &epi, void *out,
                                        const int32_t *row_sums);

// The tensor-core tiles need whole 16-byte rows of A for TMA and enough work
// to fill a tile; everything else stays on the small-shape kernel
// (the split the reference makes with coop_applies, shaders/matmul_integer.rs:501-512).
bool ovk_mmi_tc_applies(const ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int64_t m)
{
    (void)ctx;
    // (a few rows over a large weight - an int8 decode step - stream the weight through the tensor-core kernel
    // too: the one-output-per-thread kernel reads it at a fortieth of the memory bandwidth)
    const bool rows_ok = m >= 16 || (m >= 1 && w->k * w->n >= (int64_t(1) << 20));
    return rows_ok && w->n >= 16 && w->k >= 32 && (w->k % 16) == 0 && aligned_to(a, 16) &&
           m < (int64_t(1) << 31) - BM && ceil_div64(m, BM) * ceil_div64(w->n, 64) < (int64_t(1) << 31);
}

int32_t ovk_mmi_tc_launch(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed, int64_t m,
                          const void *a_zp, const void *b_zp, const EpiParams &epi, void *out)
{
    return ovk_mmi_tc_launch_with_row_sums(ctx, w, a, a_signed, m, a_zp, b_zp, epi, out, nullptr);
}

// `row_sums`: sum over k of a[m][k] for every row, when the caller already has them (A is a constant of the
// graph); null: they are computed here when the weight's zero point may be non-zero.
int32_t ovk_mmi_tc_launch_with_row_sums(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a, int32_t a_signed, int64_t m,
                                        const void *a_zp, const void *b_zp, const EpiParams &epi, void *out,
                                        const int32_t *row_sums)
{
    TcParams p = {};
    p.M = m;
    p.N = int(w->n);
    p.K = int(w->k);
    p.num_kb = int(ceil_div64(w->k, BK));
    p.colsum = w->colsum;
    p.a_zp = a_zp;
    p.b_zp = b_zp;
    p.a_signed = a_signed ? 1 : 0;
    p.b_signed = w->b_signed;
    p.epi = epi;
    p.out = out;
    p.vec_ok = (w->n % 4) == 0 && aligned_to(out, epi.mode == EPI_REQUANT ? 4 : 16);
    p.status = ctx->dev_status;
    if (b_zp && row_sums) {
        p.rowsum = row_sums;
    } else if (b_zp) {
        void *ws = nullptr;
        int32_t rc = ovk_scratch(ctx, size_t(m) * sizeof(int32_t), &ws);
        if (rc != OVK_OK)
            return rc;
        p.rowsum = static_cast<int32_t *>(ws);
        OVK_CUDA(ctx, ovk_launch_pdl(mmi_rowsum_kernel, dim3(unsigned(ceil_div64(m * 32, 256))), dim3(256), 0, ctx->stream,
                                     static_cast<const uint8_t *>(a), m, p.K, p.a_signed, b_zp, p.b_signed,
                                     static_cast<int32_t *>(ws)));
        OVK_LAUNCHED(ctx, "mmi_rowsum");
    }
    if (wants256(ctx, w, m))
        return launch256(ctx, a, w, p);
    CUtensorMap tmA;
    if (!ovk_make_tmap_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->k), uint64_t(m), uint64_t(w->k), BK,
                          BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger: cuTensorMapEncodeTiled failed for A");
    return launch_by_fill(ctx, tmA, &w, 1, p);
}

// Up to four weights over the same A in one launch.  The caller has checked that every member takes
// the tensor-core kernel and shares K and the signedness of B; epis[j] / outs[j] are member j's.
int32_t ovk_mmi_tc_launch_group(ovk_ctx *ctx, int count, const ovk_mmi_weight *const *ws, const void *a, int32_t a_signed,
                                int64_t m, const void *a_zp, const void *b_zp, const EpiParams *epis, void *const *outs)
{
    TcParams p = {};
    p.M = m;
    p.N = int(ws[0]->n);
    p.K = int(ws[0]->k);
    p.num_kb = int(ceil_div64(ws[0]->k, BK));
    p.a_zp = a_zp;
    p.b_zp = b_zp;
    p.a_signed = a_signed ? 1 : 0;
    p.b_signed = ws[0]->b_signed;
    p.epi = epis[0];
    p.status = ctx->dev_status;
    p.members = count;
    p.vec_ok = 1;
    for (int j = 0; j < count; j++) {
        p.mem[j].colsum = ws[j]->colsum;
        p.mem[j].scale = epis[j].scale;
        p.mem[j].product = epis[j].product;
        p.mem[j].fbias = epis[j].fbias;
        p.mem[j].out = outs[j];
        p.mem[j].N = int(ws[j]->n);
        p.vec_ok = p.vec_ok && (ws[j]->n % 4) == 0 && aligned_to(outs[j], 16);
    }
    if (b_zp) {
        void *ws_rows = nullptr;
        int32_t rc = ovk_scratch(ctx, size_t(m) * sizeof(int32_t), &ws_rows);
        if (rc != OVK_OK)
            return rc;
        p.rowsum = static_cast<int32_t *>(ws_rows);
        OVK_CUDA(ctx, ovk_launch_pdl(mmi_rowsum_kernel, dim3(unsigned(ceil_div64(m * 32, 256))), dim3(256), 0, ctx->stream,
                                     static_cast<const uint8_t *>(a), m, p.K, p.a_signed, b_zp, p.b_signed,
                                     static_cast<int32_t *>(ws_rows)));
        OVK_LAUNCHED(ctx, "mmi_rowsum");
    }
    CUtensorMap tmA;
    if (!ovk_make_tmap_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(ws[0]->k), uint64_t(m), uint64_t(ws[0]->k), BK,
                          BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger: cuTensorMapEncodeTiled failed for A");
    return launch_by_fill(ctx, tmA, ws, count, p);
}

// ---------------------------------------------------------------------------
// MatMulInteger for callers that may not allocate device memory.
//
// Some hosts hand out all device memory themselves (an inference runtime whose
// plugin must take every byte from the runtime's own arena, an embedded
// serving loop with a fixed memory plan) or cannot afford the device-wide
// synchronisation an allocation may imply in the middle of a latency-critical
// request.  For them the one piece of scratch this operator needs - the row
// sums of A that enter the zero-point correction when the weight's zero point
// is not 0 - lives in a fixed array inside the library image instead of the
// context's grow-on-demand workspace.  Every GPU that loads the library holds
// these 256 KB until the process exits.
constexpr int64_t OVK_STATIC_ROWS = 65536;  // most rows of A one call may bring
static __device__ __align__(256) int32_t g_static_rowsum[OVK_STATIC_ROWS];

namespace {
constexpr int OVK_MAX_DEVICES = 64;
int32_t *g_static_rowsum_addr[OVK_MAX_DEVICES] = {};  // device address of the array, per device
}  // namespace

extern "C" int32_t ovk_matmul_integer_static_scratch(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a,
                                                     int32_t a_signed, int64_t m, const void *a_zp,
                                                     const void *b_zp, int32_t *out)
{
    if (!ctx || !w)
        return ovk_fail(ctx, OVK_INVALID_ARGUMENT, "MatMulInteger (static scratch): null argument");
    OVK_REQUIRE(ctx, m >= 0, "MatMulInteger (static scratch): %lld rows of A", (long long)m);
    OVK_REQUIRE(ctx, m <= OVK_STATIC_ROWS,
                "MatMulInteger (static scratch): %lld rows of A exceed the fixed scratch of %lld rows; "
                "split the call or use ovk_matmul_integer",
                (long long)m, (long long)OVK_STATIC_ROWS);
    if (m == 0 || w->n == 0)
        return OVK_OK;
    OVK_REQUIRE(ctx, a && out, "MatMulInteger (static scratch): A or the output is null");
    OVK_REFUSE(ctx, w->k > 33025, "MatMulInteger (static scratch): K=%lld could overflow the int32 accumulator",
               (long long)w->k);
    OVK_REQUIRE(ctx, ctx->device >= 0 && ctx->device < OVK_MAX_DEVICES, "MatMulInteger (static scratch): device %d",
                ctx->device);
    OVK_CUDA(ctx, cudaSetDevice(ctx->device));
    if (!ovk_mmi_tc_applies(ctx, w, a, m))
        return ovk_matmul_integer(ctx, w, a, a_signed, m, a_zp, b_zp, out);  // one output per thread: no scratch at all
    // Set-up, once per device, with that device current: in host code the
    // array's name is only a stand-in, the kernels need its device address.
    if (!g_static_rowsum_addr[ctx->device]) {
        void *addr = nullptr;
        OVK_CUDA(ctx, cudaGetSymbolAddress(&addr, g_static_rowsum));
        g_static_rowsum_addr[ctx->device] = static_cast<int32_t *>(addr);
    }
    int32_t *rowsum = g_static_rowsum_addr[ctx->device];
    TcParams p = {};
    p.M = m;
    p.N = int(w->n);
    p.K = int(w->k);
    p.num_kb = int(ceil_div64(w->k, BK));
    p.colsum = w->colsum;
    p.a_zp = a_zp;
    p.b_zp = b_zp;
    p.a_signed = a_signed ? 1 : 0;
    p.b_signed = w->b_signed;
    p.epi = EpiParams{};
    p.epi.mode = EPI_RAW;
    p.out = out;
    p.vec_ok = (w->n % 4) == 0 && aligned_to(out, 16);
    p.status = ctx->dev_status;
    if (b_zp) {
        // rows [0, m) are rewritten whenever the zero point is not 0, and read only then:
        // nothing left over from an earlier call is ever used, so nothing needs clearing
        p.rowsum = rowsum;
        OVK_CUDA(ctx, ovk_launch_pdl(mmi_rowsum_kernel, dim3(unsigned(ceil_div64(m * 32, 256))), dim3(256), 0, ctx->stream,
                                     static_cast<const uint8_t *>(a), m, p.K, p.a_signed, b_zp, p.b_signed, rowsum));
        OVK_LAUNCHED(ctx, "mmi_rowsum");
    }
    CUtensorMap tmA;
    if (!ovk_make_tmap_2d(&tmA, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, uint64_t(w->k), uint64_t(m), uint64_t(w->k), BK,
                          BM, CU_TENSOR_MAP_SWIZZLE_128B))
        return ovk_fail(ctx, OVK_BACKEND, "MatMulInteger (static scratch): cuTensorMapEncodeTiled failed for A");
    return launch_by_fill(ctx, tmA, &w, 1, p);
}
