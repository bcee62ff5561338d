// MatMulNBits decode (M <= 8): the HBM-bound matrix-vector product.
//
// Successor of the reference's wide-column decode kernel
// (crates/onnx-vulkan-core/src/shaders/matmul_nbits.rs:458-516: whole blocks
// read as 128-bit vectors, four accumulators, scale applied once per block).
// The arithmetic per block is the same - an exact sum of (nibble - zero point)
// * a over the block, then ONE multiply by the block's scale accumulated in
// f32 - but the machinery is built for a 6.5 TB/s memory system:
//
//  * ovk_nbits_prepack re-tiles the weight once (the role packed_b plays for
//    MatMulInteger, src/interp.rs:2712): tiles of P 16-column panels x KC
//    quantization blocks, each tile ONE contiguous, 16-byte aligned range that
//    holds its nibbles, scales and zero points, the nibbles already in the
//    order the math unit wants them.  Bytes per weight are unchanged (4 bits
//    + scale + 4-bit zero point).
//  * a persistent CTA per SM streams its tiles with cp.async.bulk into a
//    4-stage shared-memory ring (a producer warp, mbarrier completion), so
//    ~170 KB per SM are in flight without spending registers on it;
//  * sixteen consumer warps unpack with ONE logic op per pair of nibbles (a
//    nibble sitting in the mantissa of an fp16 number whose exponent bits are
//    OR-ed in IS the number bias + n; the prepack rotates every word by two
//    bits so that one rotation per word serves all eight nibbles) and feed
//    mma.sync.m16n8k16: 16 weight columns x 16 k x up to 8 activation rows per
//    instruction, products exact, f32 accumulation; the biases and the zero
//    point leave through one more MMA per block (see do_block).  A block's
//    partial sum is then scaled and added in f32 on the CUDA cores, as the
//    reference does.
//  * f32 activations are split into an fp16 high and low part (two of the
//    eight batch columns), after an exact power-of-two row normalisation, so
//    the result keeps ~22 bits of the activation.
// Without tensor cores the unpack + convert + FMA chain costs ~3 issue slots
// per nibble and caps the kernel well below the memory roofline.
#include "ovk_internal.h"
#include "umma.cuh"

namespace {

constexpr int CONSUMER_WARPS = 16;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int MAX_STAGES = 4;  // ring depth is chosen per launch: as many tiles as fit beside the activations
constexpr int SLICES = 8;      // bulk copies per tile
constexpr uint32_t STAGE_MAX = 70 * 1024;
constexpr size_t ACT_MAX = 64 * 1024;
constexpr long long WAIT_CYCLES = 2000000000ll;

struct DecParams {
    const uint8_t *packed;
    const void *a;
    void *y;
    int M, K, N;
    int P, KC, GB, NKC, ntiles;
    uint32_t s_off, z_off, tile_bytes;
    int g_pad;  // k32 groups covered by the tiles (>= ceil(K/32))
    int rows;   // batch columns in use: M, or 2M for split f32 activations
    int vec_a;  // rows of A start on 16-byte boundaries: groups are read as 128-bit vectors
    int stages; // depth of the weight ring, 2..MAX_STAGES
    // a group of weights that share the activations and the tile shape (q|k|v, gate|up): `ntiles` counts
    // the tiles of all of them, member j owns the tiles below tile_end[j]; member 0 is packed / y / N above
    int members;
    const uint8_t *packed_g[3];
    void *y_g[3];
    int n_g[3];
    int tile_end[4];
    int *status;
};

// Bounded wait; while the phase is incomplete the hardware parks the thread
// (up to a microsecond per attempt) instead of letting it spin in the issue slots.
__device__ __forceinline__ bool wait_bounded(uint64_t *bar, uint32_t parity)
{
    if (umma::mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    for (;;) {
        if (umma::mbar_try_wait_hint(bar, parity, 1000u))
            return true;
        if (clock64() - t0 > WAIT_CYCLES)
            return false;
    }
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi)
{
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}


__device__ __forceinline__ uint2 lds64(uint32_t addr)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// d = A x B (C = 0) for the 16 x 8 (k = 8) shape: two A registers, one B register
__device__ __forceinline__ void mma1688_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "f"(0.0f));
}

// (a & b) | c with all three operands in registers: one LOP3 (two immediates would need two)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct UnpackConsts {
    // held in registers (an immediate pair would cost a second logic op each):
    //   even k: nibble at bits 2-5,  0x003C003C / 0x5C005C00 -> 256 + n
    //   odd k:  nibble at bits 6-9,  0x03C003C0 / 0x4C004C00 ->  16 + n
    //   zero point: bits 4-7,        0x00F000F0 / 0x54005400 ->  64 + z
    uint32_t mask_e, magic_e, mask_o, magic_o, mask_z, magic_z;
};

// One quantization block of one 16-column panel.
//
// A nibble n that sits inside the mantissa field of an fp16 number whose
// exponent bits say "2^e" IS the number 2^e + n when it starts at mantissa bit
// 10 - e: nothing has to be subtracted or converted to unpack it.  The prepack
// stores every 32-bit word of eight nibbles rotated left by two bits, which puts
// nibbles 0 and 4 at bits 2-5 of the two halves (256 + n) and nibbles 1 and 5
// at bits 6-9 (16 + n); ONE rotation by eight bits brings nibbles 2, 6 and 3, 7
// to the same places.  So a word costs one shift and four logic ops.
//
// The block's sum
//     sum_k a_k (n_k - z) = sum_odd a_k (16 + n_k) + sum_even a_k (256 + n_k)
//                           - (64 + z) S + 64 (0.75 S_odd - 3 S_even),   S = S_odd + S_even
// (S_* = sums of the block's activations over odd / even k) is formed entirely
// on the tensor cores: 2*GB MMAs over the nibbles plus ONE k = 8 MMA whose weight
// operand is half2(64 + z, 64) (again just bits) and whose activation operand
// is half2(-S, 0.75 S_odd - 3 S_even), each split into three fp16 parts so that
// it is exact to ~2^-33.  All products are exact and the f32 accumulator only
// ever holds values of about a thousand, so the result differs from the exact
// sum by a few 1e-6 relative.  Then the block's scale, in f32.
template <bool SCALE_F32, int GB, bool ONE>
__device__ __forceinline__ void do_block(float (&acc)[4], const UnpackConsts &uc, uint32_t wa, uint32_t sa,
                                         uint32_t za, uint32_t aa, uint32_t ca)
{
    float s_lo, s_hi;  // scales of columns g and g+8
    if constexpr (SCALE_F32) {
        const uint2 sv = lds64(sa);
        s_lo = __uint_as_float(sv.x);
        s_hi = __uint_as_float(sv.y);
    } else {
        uint32_t sv = lds32(sa);
        const __half2 h = *reinterpret_cast<__half2 *>(&sv);
        s_lo = __low2float(h);
        s_hi = __high2float(h);
    }
    const uint32_t zb = lds8(za);    // z(col g) | z(col g+8) << 4
    const uint32_t corr = lds32(ca);  // half2(-S part_t, (0.75 S_odd - 3 S_even) part_t)
    float d[4];
    mma1688_zero(d, and_or(zb << 4, uc.mask_z, uc.magic_z), and_or(zb, uc.mask_z, uc.magic_z), corr);
#pragma unroll
    for (int gi = 0; gi < GB; gi++) {
        const uint2 wv = lds64(wa + gi * 256);
        const uint4 av = lds128(aa + gi * 64);
        const uint32_t xr = __funnelshift_r(wv.x, wv.x, 8), yr = __funnelshift_r(wv.y, wv.y, 8);
        mma16816(d, and_or(wv.x, uc.mask_e, uc.magic_e), and_or(wv.y, uc.mask_e, uc.magic_e),
                 and_or(wv.x, uc.mask_o, uc.magic_o), and_or(wv.y, uc.mask_o, uc.magic_o), av.x, av.y);
        mma16816(d, and_or(xr, uc.mask_e, uc.magic_e), and_or(yr, uc.mask_e, uc.magic_e),
                 and_or(xr, uc.mask_o, uc.magic_o), and_or(yr, uc.mask_o, uc.magic_o), av.z, av.w);
    }
    acc[0] = fmaf(d[0], s_lo, acc[0]);
    acc[2] = fmaf(d[2], s_hi, acc[2]);
    if constexpr (!ONE) {  // batch columns 1, 3, 5, 7 exist only with more than one row
        acc[1] = fmaf(d[1], s_lo, acc[1]);
        acc[3] = fmaf(d[3], s_hi, acc[3]);
    }
}

// The three fp16 parts of x, to ~2^-33 relative.
__device__ __forceinline__ void split3(double x, __half (&h)[3])
{
    h[0] = __double2half(x);
    const double r1 = x - double(__half2float(h[0]));
    h[1] = __double2half(r1);
    h[2] = __double2half(r1 - double(__half2float(h[1])));
}

// Exact sums of a group's staged (fp16) activations over even and odd k,
// in two chains each; fp16 terms span fewer than 53 bits, so doubles are exact.
struct GroupSums {
    double e0 = 0.0, e1 = 0.0, o0 = 0.0, o1 = 0.0;
};

// Stages eight consecutive k (already rounded to fp16, held as float) as the
// 16-byte unit the fragments read: half2 pairs (0,4) (1,5) (2,6) (3,7).
__device__ __forceinline__ void stage_unit(uint4 *dst, const float (&w)[8], GroupSums &s)
{
    *dst = make_uint4(pack_h2(w[0], w[4]), pack_h2(w[1], w[5]), pack_h2(w[2], w[6]), pack_h2(w[3], w[7]));
    s.e0 += double(w[0]) + double(w[4]);
    s.o0 += double(w[1]) + double(w[5]);
    s.e1 += double(w[2]) + double(w[6]);
    s.o1 += double(w[3]) + double(w[7]);
}

// Sums of a block = of GBT adjacent groups, held by GBT adjacent lanes; the
// first lane of the block writes the correction entry (four words, one per t).
template <int GBT>
__device__ __forceinline__ void finish_block(uint32_t *corr_entry, double s_even, double s_odd, int lane, bool valid)
{
#pragma unroll
    for (int o = 1; o < GBT; o <<= 1) {
        s_even += __shfl_xor_sync(0xffffffffu, s_even, o);
        s_odd += __shfl_xor_sync(0xffffffffu, s_odd, o);
    }
    if (valid && (lane & (GBT - 1)) == 0) {
        __half a[3], b[3];
        split3(-(s_even + s_odd), a);
        split3(0.75 * s_odd - 3.0 * s_even, b);
        uint4 e;
        e.x = uint32_t(__half_as_ushort(a[0])) | uint32_t(__half_as_ushort(b[0])) << 16;
        e.y = uint32_t(__half_as_ushort(a[1])) | uint32_t(__half_as_ushort(b[1])) << 16;
        e.z = uint32_t(__half_as_ushort(a[2])) | uint32_t(__half_as_ushort(b[2])) << 16;
        e.w = 0u;
        *reinterpret_cast<uint4 *>(corr_entry) = e;
    }
}

// Which member of the group owns tile u, and which of its tiles that is.
struct TileOf {
    const uint8_t *packed;
    void *y;
    int n, u;
};
__device__ __forceinline__ TileOf tile_of(const DecParams &p, int u)
{
    TileOf t{p.packed, p.y, p.N, u};
    if (p.members > 1 && u >= p.tile_end[0]) {
        int j = 1;
        while (j + 1 < p.members && u >= p.tile_end[j])
            j++;
        t.packed = p.packed_g[j - 1];
        t.y = p.y_g[j - 1];
        t.n = p.n_g[j - 1];
        t.u = u - p.tile_end[j - 1];
    }
    return t;
}

template <bool SCALE_F32, bool A_F32, bool Y_F32, int GBT, int UNROLL, bool ONE>
__global__ void __launch_bounds__(THREADS, 1) nbits_decode_kernel(DecParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *stage_base = smem;
    uint4 *acts = reinterpret_cast<uint4 *>(smem + size_t(p.stages) * p.tile_bytes);
    // per (batch column, block): half2(-part_t, 0) for t = 0..3, the three fp16 parts of the block's activation sum
    uint32_t *corr = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(acts) + size_t(p.rows) * p.g_pad * 64);
    float4 *red = reinterpret_cast<float4 *>(corr + size_t(p.rows) * (p.g_pad / GBT) * 4);
    float *row_pow2 = reinterpret_cast<float *>(red + CONSUMER_WARPS * 32);
    uint64_t *full = reinterpret_cast<uint64_t *>(row_pow2 + 8);
    uint64_t *empty = full + MAX_STAGES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            umma::mbar_init(&full[s], 1);
            umma::mbar_init(&empty[s], CONSUMER_WARPS);
        }
        umma::fence_barrier_init();
    }

    // barriers visible to everyone, then the producer starts streaming weights at once:
    // the first tiles are in flight while the consumer warps stage the activations
    __syncthreads();
    // Programmatic dependent launch: the next kernel of the stream may start its own
    // prologue and weight streaming now (weights are constants); like this one, it
    // touches activations and outputs only after griddepcontrol.wait, i.e. after
    // every earlier kernel has completed and flushed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------------------------ producer
        // the tile is fetched as SLICES bulk copies issued by as many lanes, all
        // completing on the stage's barrier: more requests in flight per SM
        const uint32_t slice = ((p.tile_bytes / SLICES) + 15u) & ~15u;
        const uint32_t my_off = min(uint32_t(lane) * slice, p.tile_bytes);
        const uint32_t my_len = lane < SLICES ? min(slice, p.tile_bytes - my_off) : 0u;
        int s = 0;
        uint32_t ph = 0;
        bool alive = true;
        for (int ug = blockIdx.x; ug < p.ntiles && alive; ug += gridDim.x) {
            const TileOf tl = tile_of(p, ug);
            const int u = tl.u;
            for (int kc = 0; kc < p.NKC; kc++) {
                bool ok = true;
                if (lane == 0) {
                    ok = wait_bounded(&empty[s], ph ^ 1);
                    if (ok)
                        umma::mbar_expect_tx(&full[s], p.tile_bytes);
                    else
                        atomicExch(p.status, OVK_DEV_TIMEOUT_SLOT);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    alive = false;
                    break;
                }
                if (my_len)
                    umma::bulk_load_1d(stage_base + size_t(s) * p.tile_bytes + my_off,
                                       tl.packed + (size_t(u) * p.NKC + kc) * p.tile_bytes + my_off, my_len, &full[s]);
                if (++s == p.stages) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        return;
    }

    // ---- everything a consumer needs that does not depend on the activations is computed here, while
    // the kernel that produces them may still be running
    const int g = lane >> 2, t = lane & 3;
    // P is a power of two up to the warp count: shifts and masks, no divisions
    const int p_shift = 31 - __clz(p.P);
    const int wp = CONSUMER_WARPS >> p_shift;  // warps sharing one panel
    const int wp_shift = 31 - __clz(wp);
    const int panel = warp & (p.P - 1);
    // each warp owns a contiguous run of the chunk's blocks
    const int per_warp = (p.KC + wp - 1) >> wp_shift;
    const int b_first = min((warp >> p_shift) * per_warp, p.KC);
    const int my_blocks = min(per_warp, p.KC - b_first);
    const int act_row = min(g, p.rows - 1);
    // 32-bit shared-window addresses; every load below is an explicit ld.shared
    const uint32_t stage0 = umma::smem_u32(stage_base);
    const uint32_t act0 = umma::smem_u32(acts) + uint32_t((act_row * p.g_pad) * 4 + t) * 16u;
    constexpr uint32_t SCALE_PAIR = SCALE_F32 ? 8u : 4u;
    constexpr uint32_t W_STEP = GBT * 256u, S_STEP = 8u * SCALE_PAIR, Z_STEP = 8u, A_STEP = GBT * 64u;
    const uint32_t w_rel = uint32_t((panel * p.KC + b_first) * GBT * 32 + lane) * 8u;
    const uint32_t s_rel = p.s_off + uint32_t((panel * p.KC + b_first) * 8 + g) * SCALE_PAIR;
    const uint32_t z_rel = p.z_off + uint32_t((panel * p.KC + b_first) * 8 + g);
    UnpackConsts uc;
    // opaque to the optimiser, so the constants stay in registers
    asm volatile("mov.u32 %0, 0x003C003C;\n\tmov.u32 %1, 0x5C005C00;\n\tmov.u32 %2, 0x03C003C0;\n\t"
                 "mov.u32 %3, 0x4C004C00;\n\tmov.u32 %4, 0x00F000F0;\n\tmov.u32 %5, 0x54005400;"
                 : "=r"(uc.mask_e), "=r"(uc.magic_e), "=r"(uc.mask_o), "=r"(uc.magic_o), "=r"(uc.mask_z),
                   "=r"(uc.magic_z));
    const uint32_t corr0 = umma::smem_u32(corr) + uint32_t((act_row * (p.g_pad / GBT)) * 4 + t) * 4u;
    constexpr uint32_t C_STEP = 16u;
    constexpr int BIG = GBT == 1 ? 9 : (GBT == 2 ? 4 : 2);
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the producers of A have finished
    // ---- activations -> shared memory in the order the fragments are read, one
    // thread per 32-wide k group (unit t of a group: k = 32*group + 8*t + {0,4,1,5,2,6,3,7}),
    // together with the correction entries of do_block: the GBT lanes that hold a
    // block's groups are adjacent, so its sums need at most three shuffle steps
    const int nblk = p.g_pad / GBT;
    const int total_groups = p.M * p.g_pad;
    if constexpr (A_F32) {
        const float *a = static_cast<const float *>(p.a);
        __shared__ float warp_max[CONSUMER_WARPS];
        for (int m = 0; m < p.M; m++) {
            float mx = 0.0f;
            for (int k = threadIdx.x; k < p.K; k += CONSUMER_WARPS * 32)
                mx = fmaxf(mx, fabsf(a[int64_t(m) * p.K + k]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            if (lane == 0)
                warp_max[warp] = mx;
            asm volatile("bar.sync 2, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            if (threadIdx.x == 0) {
                for (int w = 1; w < CONSUMER_WARPS; w++)
                    mx = fmaxf(mx, warp_max[w]);
                int e = 0;
                if (mx > 0.0f && mx < 3.0e38f)
                    frexpf(mx, &e);
                e = max(-100, min(100, e));
                row_pow2[m] = ldexpf(1.0f, e);
            }
            asm volatile("bar.sync 2, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
        }
        for (int base = warp * 32; base < total_groups; base += CONSUMER_WARPS * 32) {
            const int idx = base + lane;
            const bool valid = idx < total_groups;
            const int m = (valid && p.M > 1) ? idx / p.g_pad : 0;
            const int grp = valid ? idx - m * p.g_pad : 0;
            GroupSums sh, sl;
            if (valid) {
                const float inv = 1.0f / row_pow2[m];  // exact power of two
                const float *src = a + int64_t(m) * p.K + grp * 32;
                const bool whole = p.vec_a && grp * 32 + 32 <= p.K;
                float raw[32];  // fetched before anything is stored (see the fp16 path)
                if (whole) {
#pragma unroll
                    for (int t = 0; t < 8; t++) {
                        const float4 f = __ldcg(reinterpret_cast<const float4 *>(src) + t);
                        raw[4 * t] = f.x, raw[4 * t + 1] = f.y, raw[4 * t + 2] = f.z, raw[4 * t + 3] = f.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        raw[i] = grp * 32 + i < p.K ? src[i] : 0.0f;
                }
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    float hi[8], lo[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float x = raw[8 * t + i] * inv;
                        hi[i] = __half2float(__float2half_rn(x));
                        lo[i] = __half2float(__float2half_rn(x - hi[i]));
                    }
                    stage_unit(&acts[(size_t(2 * m) * p.g_pad + grp) * 4 + t], hi, sh);
                    stage_unit(&acts[(size_t(2 * m + 1) * p.g_pad + grp) * 4 + t], lo, sl);
                }
            }
            const int blk = grp / GBT;
            finish_block<GBT>(corr + (size_t(2 * m) * nblk + blk) * 4, sh.e0 + sh.e1, sh.o0 + sh.o1, lane, valid);
            finish_block<GBT>(corr + (size_t(2 * m + 1) * nblk + blk) * 4, sl.e0 + sl.e1, sl.o0 + sl.o1, lane, valid);
        }
    } else {
        const __half *a = static_cast<const __half *>(p.a);
        for (int base = warp * 32; base < total_groups; base += CONSUMER_WARPS * 32) {
            const int idx = base + lane;
            const bool valid = idx < total_groups;
            const int m = (valid && p.M > 1) ? idx / p.g_pad : 0;
            const int grp = valid ? idx - m * p.g_pad : 0;
            GroupSums sg;
            if (valid) {
                const __half *src = a + int64_t(m) * p.K + grp * 32;
                const bool whole = p.vec_a && grp * 32 + 32 <= p.K;
                // all four loads are issued before anything is stored: stores to shared memory in
                // between would serialise them into four round trips to the L2
                uint4 q[4];
                if (whole) {
#pragma unroll
                    for (int t = 0; t < 4; t++)
                        q[t] = __ldcg(reinterpret_cast<const uint4 *>(src) + t);
                } else {
#pragma unroll
                    for (int t = 0; t < 4; t++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int k = grp * 32 + t * 8 + 2 * i;
                            const uint32_t lo = k < p.K ? uint32_t(__half_as_ushort(src[t * 8 + 2 * i])) : 0u;
                            const uint32_t hi = k + 1 < p.K ? uint32_t(__half_as_ushort(src[t * 8 + 2 * i + 1])) : 0u;
                            w[i] = lo | (hi << 16);
                        }
                        q[t] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
#pragma unroll
                for (int t = 0; t < 4; t++) {
                    float v[8];
                    const uint32_t qw[4] = {q[t].x, q[t].y, q[t].z, q[t].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&qw[i]));
                        v[2 * i] = f.x;
                        v[2 * i + 1] = f.y;
                    }
                    stage_unit(&acts[(size_t(m) * p.g_pad + grp) * 4 + t], v, sg);
                }
            }
            finish_block<GBT>(corr + (size_t(m) * nblk + grp / GBT) * 4, sg.e0 + sg.e1, sg.o0 + sg.o1, lane, valid);
        }
    }
    asm volatile("bar.sync 2, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");

    // ---------------------------------------------------------------- consumers
    bool dead = false;
    int s = 0;
    uint32_t ph = 0;
    for (int ug = blockIdx.x; ug < p.ntiles; ug += gridDim.x) {
        const TileOf tl = tile_of(p, ug);
        const int u = tl.u;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int kc = 0; kc < p.NKC; kc++) {
            if (!dead && !wait_bounded(&full[s], ph)) {
                dead = true;
                if (lane == 0)
                    atomicExch(p.status, OVK_DEV_TIMEOUT_TMA);
            }
            if (!dead) {
                const uint32_t tile = stage0 + uint32_t(s) * p.tile_bytes;
                uint32_t wa = tile + w_rel, sa = tile + s_rel, za = tile + z_rel;
                uint32_t aa = act0 + uint32_t((kc * p.KC + b_first) * GBT) * 64u;
                uint32_t ca = corr0 + uint32_t(kc * p.KC + b_first) * 16u;
                int left = my_blocks;
                // runs of BIG, then UNROLL, then single blocks: the offsets of a
                // run are immediates of the loads, only the bases are bumped
#define OVK_RUN(COUNT)                                                                                      \
    for (; left >= (COUNT); left -= (COUNT)) {                                                              \
        _Pragma("unroll") for (int j = 0; j < (COUNT); j++)                                                 \
            do_block<SCALE_F32, GBT, ONE>(acc, uc, wa + j * W_STEP, sa + j * S_STEP, za + j * Z_STEP,            \
                                     aa + j * A_STEP, ca + j * C_STEP);                                     \
        wa += (COUNT) * W_STEP;                                                                             \
        sa += (COUNT) * S_STEP;                                                                             \
        za += (COUNT) * Z_STEP;                                                                             \
        aa += (COUNT) * A_STEP;                                                                             \
        ca += (COUNT) * C_STEP;                                                                             \
    }
                OVK_RUN(BIG)
                OVK_RUN(UNROLL)
                OVK_RUN(1)
#undef OVK_RUN
                __syncwarp();
                if (lane == 0)
                    umma::mbar_arrive(&empty[s]);
            }
            if (++s == p.stages) {
                s = 0;
                ph ^= 1;
            }
        }
        // ---- combine the warps that shared a panel (none when a warp owns a
        // whole panel: then nothing is exchanged and no barrier is taken), then store
        float4 v = make_float4(acc[0], acc[1], acc[2], acc[3]);
        if (wp > 1) {
            red[warp * 32 + lane] = v;
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
            if (warp < p.P) {
                for (int j = 1; j < wp; j++) {
                    const float4 o = red[(warp + j * p.P) * 32 + lane];
                    v.x += o.x;
                    v.y += o.y;
                    v.z += o.z;
                    v.w += o.w;
                }
            }
        }
        if (warp < p.P && !dead) {
            const int col_lo = (u * p.P + warp) * 16 + g, col_hi = col_lo + 8;
            if constexpr (A_F32) {
                // batch columns 2t (high part) and 2t+1 (low part) belong to row t
                if (t < p.M) {
                    const float sc = row_pow2[t];
                    const float y_lo = (v.x + v.y) * sc, y_hi = (v.z + v.w) * sc;
                    if (col_lo < tl.n) {
                        if constexpr (Y_F32) static_cast<float *>(tl.y)[int64_t(t) * tl.n + col_lo] = y_lo;
                        else static_cast<__half *>(tl.y)[int64_t(t) * tl.n + col_lo] = __float2half_rn(y_lo);
                    }
                    if (col_hi < tl.n) {
                        if constexpr (Y_F32) static_cast<float *>(tl.y)[int64_t(t) * tl.n + col_hi] = y_hi;
                        else static_cast<__half *>(tl.y)[int64_t(t) * tl.n + col_hi] = __float2half_rn(y_hi);
                    }
                }
            } else {
                const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int m = 2 * t + (i & 1);
                    const int col = (i < 2) ? col_lo : col_hi;
                    if (m < p.M && col < tl.n) {
                        if constexpr (Y_F32) static_cast<float *>(tl.y)[int64_t(m) * tl.n + col] = vals[i];
                        else static_cast<__half *>(tl.y)[int64_t(m) * tl.n + col] = __float2half_rn(vals[i]);
                    }
                }
            }
        }
        if (wp > 1)
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
    }
}

// ------------------------------------------------------------------- prepack
// One thread per 8-byte weight element, per scale pair, per zero-point byte.
template <bool SCALE_F32>
__global__ void __launch_bounds__(256)
nbits_decode_pack_kernel(const uint32_t *__restrict__ src_w, const void *__restrict__ src_s,
                         const uint8_t *__restrict__ src_z, uint8_t *__restrict__ dst, int N, int n_blocks,
                         int P, int KC, int GB, int NKC, int ntiles, uint32_t s_off, uint32_t z_off,
                         uint32_t tile_bytes)
{
    const int64_t per_tile_w = int64_t(P) * KC * GB * 32;  // 8-byte elements
    const int64_t per_tile_s = int64_t(P) * KC * 8;        // scale pairs
    const int64_t per_tile = per_tile_w + 2 * per_tile_s;  // + zero-point bytes (one per pair)
    const int64_t total = per_tile * ntiles * NKC;
    const int words_per_row = n_blocks * GB * 4;
    const int zp_row = (n_blocks + 1) / 2;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int64_t tile_id = i / per_tile;
        int64_t r = i % per_tile;
        const int nt = int(tile_id / NKC), kc = int(tile_id % NKC);
        uint8_t *tile = dst + size_t(tile_id) * tile_bytes;
        if (r < per_tile_w) {
            const int lane = int(r & 31);
            int64_t q = r >> 5;
            const int gi = int(q % GB);
            q /= GB;
            const int b = int(q % KC), pnl = int(q / KC);
            const int g = lane >> 2, t = lane & 3;
            const int blk = kc * KC + b;
            const int col_lo = (nt * P + pnl) * 16 + g, col_hi = col_lo + 8;
            const int word = (blk * GB + gi) * 4 + t;
            uint2 v = make_uint2(0u, 0u);
            if (blk < n_blocks) {
                if (col_lo < N) v.x = src_w[int64_t(col_lo) * words_per_row + word];
                if (col_hi < N) v.y = src_w[int64_t(col_hi) * words_per_row + word];
                // nibble j of a word moves from bits 4j.. to bits 4j+2.. (mod 32), see do_block
                v.x = __funnelshift_l(v.x, v.x, 2);
                v.y = __funnelshift_l(v.y, v.y, 2);
            }
            reinterpret_cast<uint2 *>(tile)[r] = v;
        } else {
            r -= per_tile_w;
            const bool is_zp = r >= per_tile_s;
            if (is_zp)
                r -= per_tile_s;
            const int g = int(r & 7);
            const int64_t pb = r >> 3;
            const int b = int(pb % KC), pnl = int(pb / KC);
            const int blk = kc * KC + b;
            const int col_lo = (nt * P + pnl) * 16 + g, col_hi = col_lo + 8;
            const bool lo_ok = blk < n_blocks && col_lo < N, hi_ok = blk < n_blocks && col_hi < N;
            if (is_zp) {
                uint32_t zl = 0, zh = 0;
                if (lo_ok) zl = src_z ? (src_z[int64_t(col_lo) * zp_row + blk / 2] >> (4 * (blk & 1))) & 15u : 8u;
                if (hi_ok) zh = src_z ? (src_z[int64_t(col_hi) * zp_row + blk / 2] >> (4 * (blk & 1))) & 15u : 8u;
                tile[z_off + r] = uint8_t(zl | (zh << 4));
            } else if constexpr (SCALE_F32) {
                const float *sp = static_cast<const float *>(src_s);
                reinterpret_cast<float2 *>(tile + s_off)[r] =
                    make_float2(lo_ok ? sp[int64_t(col_lo) * n_blocks + blk] : 0.0f,
                                hi_ok ? sp[int64_t(col_hi) * n_blocks + blk] : 0.0f);
            } else {
                const __half *sp = static_cast<const __half *>(src_s);
                const __half zero = __float2half(0.0f);
                reinterpret_cast<__half2 *>(tile + s_off)[r] =
                    __halves2half2(lo_ok ? sp[int64_t(col_lo) * n_blocks + blk] : zero,
                                   hi_ok ? sp[int64_t(col_hi) * n_blocks + blk] : zero);
            }
        }
    }
}

size_t decode_smem(const ovk_nbits_weight *w, int rows, int stages)
{
    const size_t g_pad = size_t(w->dec_nkc) * w->dec_kc * w->dec_gb;
    return size_t(stages) * w->dec_tile_bytes + size_t(rows) * g_pad * 64 + size_t(rows) * (g_pad / w->dec_gb) * 16 +
           CONSUMER_WARPS * 32 * 16 + 32 + 64 + 128;
}

template <bool SF, bool AF, bool YF, int GB, int UN, bool ONE>
int32_t launch_decode_one(ovk_ctx *ctx, const DecParams &p, size_t smem)
{
    OVK_CUDA(ctx, cudaFuncSetAttribute(nbits_decode_kernel<SF, AF, YF, GB, UN, ONE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    const unsigned grid = unsigned(std::min<int>(p.ntiles, ctx->sm_count));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OVK_CUDA(ctx, cudaLaunchKernelEx(&cfg, nbits_decode_kernel<SF, AF, YF, GB, UN, ONE>, p));
    OVK_LAUNCHED(ctx, "nbits_decode_mma");
    return OVK_OK;
}

template <bool SF, bool AF, bool YF, int GB, int UN>
int32_t launch_decode_gb(ovk_ctx *ctx, const DecParams &p, size_t smem)
{
    if constexpr (!AF) {
        if (p.rows == 1)  // one fp16 row: the odd batch columns are never stored
            return launch_decode_one<SF, AF, YF, GB, UN, true>(ctx, p, smem);
    }
    return launch_decode_one<SF, AF, YF, GB, UN, false>(ctx, p, smem);
}

template <bool SF, bool AF, bool YF>
int32_t launch_decode(ovk_ctx *ctx, const DecParams &p, size_t smem)
{
    switch (p.GB) {
    case 1: return launch_decode_gb<SF, AF, YF, 1, 3>(ctx, p, smem);
    case 2: return launch_decode_gb<SF, AF, YF, 2, 2>(ctx, p, smem);
    case 4: return launch_decode_gb<SF, AF, YF, 4, 1>(ctx, p, smem);
    case 8: return launch_decode_gb<SF, AF, YF, 8, 1>(ctx, p, smem);
    default: return ovk_fail(ctx, OVK_UNSUPPORTED, "MatMulNBits decode: block size %d has no tuned kernel", p.GB * 32);
    }
}

}  // namespace

// Builds the decode copy for block sizes 32, 64, 128 and 256 (a 32-wide k group
// must not straddle two blocks).  Other block sizes keep only the operator layout.
int32_t ovk_nbits_decode_prepack(ovk_ctx *ctx, ovk_nbits_weight *w)
{
    const int64_t bs = w->block_size;
    if ((bs != 32 && bs != 64 && bs != 128 && bs != 256) || !aligned_to(w->b, 4))
        return OVK_OK;
    const int sz = w->scales_dtype == OVK_FLOAT ? 4 : 2;
    if (!aligned_to(w->scales, sz))
        return OVK_OK;
    const int gb = int(w->block_size / 32);
    const int64_t nb = w->n_blocks;
    const uint32_t pb_bytes = uint32_t(gb) * 256u + 16u * sz + 8u;  // one panel x one block
    const int64_t np = ceil_div64(w->n, 16);
    // Tile shape: P panels (a power of two up to the warp count; 16 / P warps share
    // a panel and split its blocks) x KC blocks, K cut into NKC chunks that fit a
    // stage.  Chosen for the shortest critical path, counted in blocks the
    // busiest warp of the busiest CTA works through: per chunk its share of the
    // blocks plus ~0.4 for the hand-over, per tile ~2 for the exchange between
    // warps that share a panel (~0.5 for the store alone when a warp keeps its
    // columns for the whole of K).  A CTA with a single tile gets chunks of at
    // most 32 KB so that arrival and arithmetic overlap.  A larger P is given up
    // only for a gain of more than a tenth: its copies are larger.
    if (pb_bytes > STAGE_MAX)
        return OVK_OK;
    int P = 0, KC = 0, NKC = 0;
    double best = 0.0;
    for (int cand = CONSUMER_WARPS; cand >= 1; cand /= 2) {
        const uint32_t chunk_block = uint32_t(cand) * pb_bytes;  // bytes of one block across the tile's panels
        if (chunk_block > STAGE_MAX)
            continue;
        const int wp = CONSUMER_WARPS / cand;
        const int64_t waves = ceil_div64(ceil_div64(np, cand), ctx->sm_count);
        int64_t kc_cap = STAGE_MAX / chunk_block;
        if (waves == 1)
            kc_cap = std::max<int64_t>(1, std::min<int64_t>(kc_cap, 32768 / chunk_block));
        const int nkc_min = int(ceil_div64(nb, kc_cap));
        int nkc_best = nkc_min;
        double chunk_cost = 0.0;
        for (int nkc = nkc_min; nkc <= nkc_min + 7 && nkc <= nb; nkc++) {
            const int64_t kc = ceil_div64(nb, nkc);
            const double c = double(nkc) * (double(ceil_div64(kc, wp)) + 0.4);
            if (nkc == nkc_min || c < chunk_cost) {
                chunk_cost = c;
                nkc_best = nkc;
            }
        }
        const double cost = double(waves) * (chunk_cost + (wp > 1 ? 2.0 : 0.5));
        if (P == 0 || cost < 0.9 * best) {
            best = cost;
            P = cand;
            NKC = nkc_best;
            KC = int(ceil_div64(nb, nkc_best));
        }
    }
    if (P == 0)
        return OVK_OK;
    const int ntiles = int(ceil_div64(np, P));
    const uint32_t s_off = uint32_t(P) * KC * gb * 256u;
    const uint32_t z_off = s_off + uint32_t(P) * KC * 16u * sz;
    const uint32_t tile_bytes = (z_off + uint32_t(P) * KC * 8u + 127u) & ~127u;
    const size_t bytes = size_t(ntiles) * NKC * tile_bytes;
    void *dst = nullptr;
    OVK_CUDA(ctx, cudaMalloc(&dst, bytes));
    // padding bytes at the end of a tile are never read, but keep the copy deterministic
    OVK_CUDA(ctx, cudaMemsetAsync(dst, 0, bytes, ctx->stream));
    const int64_t total = (int64_t(P) * KC * gb * 32 + 2 * int64_t(P) * KC * 8) * ntiles * NKC;
    const unsigned blocks = unsigned(std::min<int64_t>(ceil_div64(total, 256), int64_t(ctx->sm_count) * 16));
    if (sz == 4)
        nbits_decode_pack_kernel<true><<<blocks, 256, 0, ctx->stream>>>(
            reinterpret_cast<const uint32_t *>(w->b), w->scales, w->zp, static_cast<uint8_t *>(dst), int(w->n),
            int(nb), P, KC, gb, NKC, ntiles, s_off, z_off, tile_bytes);
    else
        nbits_decode_pack_kernel<false><<<blocks, 256, 0, ctx->stream>>>(
            reinterpret_cast<const uint32_t *>(w->b), w->scales, w->zp, static_cast<uint8_t *>(dst), int(w->n),
            int(nb), P, KC, gb, NKC, ntiles, s_off, z_off, tile_bytes);
    ctx->last_kernel = "nbits_decode_pack";
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        cudaFree(dst);
        return ovk_fail(ctx, OVK_BACKEND, "nbits_decode_pack: %s", cudaGetErrorString(e));
    }
    w->decode = dst;
    w->decode_bytes = bytes;
    w->dec_p = P;
    w->dec_kc = KC;
    w->dec_gb = gb;
    w->dec_nkc = NKC;
    w->dec_ntiles = ntiles;
    w->dec_s_off = s_off;
    w->dec_z_off = z_off;
    w->dec_tile_bytes = tile_bytes;
    return OVK_OK;
}

// How one call is cut into launches: batch columns per launch (at most 8; an
// f32 row takes two) and the depth of the weight ring.  Every launch streams
// the whole weight, so all rows in one launch comes first, then a deeper ring.
struct DecodePlan {
    int rows = 0;  // rows of A per launch, 0 = does not fit
    int stages = 0;
};
static DecodePlan decode_plan(const ovk_ctx *ctx, const ovk_nbits_weight *w, int32_t a_dtype, int64_t m)
{
    const int per_row = a_dtype == OVK_FLOAT ? 2 : 1;
    const size_t g_pad = size_t(w->dec_nkc) * w->dec_kc * w->dec_gb;
    const size_t per_col = g_pad * 64 + (g_pad / w->dec_gb) * 16;
    const int want = int(std::min<int64_t>(std::max<int64_t>(m, 1), 8 / per_row));
    const int work = w->dec_nkc * int((w->dec_ntiles + ctx->sm_count - 1) / ctx->sm_count);  // tiles of the busiest CTA
    DecodePlan best;
    for (int stages = std::min(MAX_STAGES, std::max(2, work)); stages >= 2; stages--) {
        const size_t fixed = decode_smem(w, 0, stages);
        if (fixed >= ctx->smem_optin)
            continue;
        const size_t cols = std::min<size_t>(8, std::min(ACT_MAX, ctx->smem_optin - fixed) / per_col);
        const int rows = std::min(want, int(cols) / per_row);
        if (rows > best.rows) {
            best.rows = rows;
            best.stages = stages;
        }
        if (rows == want)
            break;
    }
    if (best.rows == 0 && decode_smem(w, per_row, 1) <= ctx->smem_optin) {
        best.rows = 1;  // a single stage still beats the general kernel
        best.stages = 1;
    }
    return best;
}

// Up to 8 fp16 rows (4 f32 rows) per launch; more rows than that belong to
// the prefill kernel.
bool ovk_nbits_decode_applies(const ovk_ctx *ctx, const ovk_nbits_weight *w, int64_t m, int32_t a_dtype,
                              int32_t y_dtype)
{
    (void)y_dtype;
    return w->decode && m <= 8 && decode_plan(ctx, w, a_dtype, m).rows >= 1;
}

// Weights that can share one launch: same K, block size, scale type and tile shape (then the staged
// activations, the ring slots and every offset inside a tile are the same for all of them).
bool ovk_nbits_decode_group_compatible(const ovk_nbits_weight *a, const ovk_nbits_weight *b)
{
    return a->decode && b->decode && a->k == b->k && a->block_size == b->block_size && a->scales_dtype == b->scales_dtype &&
           a->dec_p == b->dec_p && a->dec_kc == b->dec_kc && a->dec_gb == b->dec_gb && a->dec_nkc == b->dec_nkc &&
           a->dec_s_off == b->dec_s_off && a->dec_z_off == b->dec_z_off && a->dec_tile_bytes == b->dec_tile_bytes;
}

int32_t ovk_nbits_decode_group(ovk_ctx *ctx, int count, const ovk_nbits_weight *const *ws, const void *a, int32_t a_dtype,
                               int64_t m, void *const *ys, int32_t y_dtype)
{
    const ovk_nbits_weight *w = ws[0];
    void *y = ys[0];
    OVK_REQUIRE(ctx, count >= 1 && count <= 4, "MatMulNBits: a group of %d weights", count);
    const bool af = a_dtype == OVK_FLOAT, yf = y_dtype == OVK_FLOAT, sf = w->scales_dtype == OVK_FLOAT;
    for (int j = 0; j < count; j++)
        OVK_REQUIRE(ctx, aligned_to(a, af ? 4 : 2) && aligned_to(ys[j], yf ? 4 : 2), "MatMulNBits: A or Y is misaligned");
    const size_t g_pad = size_t(w->dec_nkc) * w->dec_kc * w->dec_gb;
    const int per_row = af ? 2 : 1;
    const DecodePlan plan = decode_plan(ctx, w, a_dtype, m);
    OVK_REQUIRE(ctx, plan.rows >= 1, "MatMulNBits decode: the tile does not fit in shared memory");
    const int rows_max = plan.rows;  // rows of A per launch
    const size_t a_row = size_t(w->k) * (af ? 4 : 2), y_row = size_t(w->n) * (yf ? 4 : 2);
    for (int64_t m0 = 0; m0 < m; m0 += rows_max) {
        DecParams p = {};
        p.packed = static_cast<const uint8_t *>(w->decode);
        p.a = static_cast<const uint8_t *>(a) + size_t(m0) * a_row;
        p.y = static_cast<uint8_t *>(y) + size_t(m0) * y_row;
        p.M = int(std::min<int64_t>(rows_max, m - m0));
        p.K = int(w->k);
        p.N = int(w->n);
        p.P = w->dec_p;
        p.KC = w->dec_kc;
        p.GB = w->dec_gb;
        p.NKC = w->dec_nkc;
        p.ntiles = w->dec_ntiles;
        p.members = count;
        p.tile_end[0] = w->dec_ntiles;
        for (int j = 1; j < count; j++) {
            p.packed_g[j - 1] = static_cast<const uint8_t *>(ws[j]->decode);
            p.y_g[j - 1] = static_cast<uint8_t *>(ys[j]) + size_t(m0) * size_t(ws[j]->n) * (yf ? 4 : 2);
            p.n_g[j - 1] = int(ws[j]->n);
            p.tile_end[j] = p.tile_end[j - 1] + ws[j]->dec_ntiles;
            p.ntiles = p.tile_end[j];
        }
        p.s_off = w->dec_s_off;
        p.z_off = w->dec_z_off;
        p.tile_bytes = w->dec_tile_bytes;
        p.g_pad = int(g_pad);
        p.rows = p.M * per_row;
        p.vec_a = aligned_to(p.a, 16) && (a_row % 16 == 0);
        p.status = ctx->dev_status;
        p.stages = plan.stages;
        const size_t smem = decode_smem(w, p.rows, plan.stages);
        OVK_REQUIRE(ctx, smem <= ctx->smem_optin, "MatMulNBits decode: %zu bytes of shared memory needed", smem);
        int32_t rc;
#define GO(SF, AF, YF) rc = launch_decode<SF, AF, YF>(ctx, p, smem)
        if (sf && af && yf) GO(true, true, true);
        else if (sf && af && !yf) GO(true, true, false);
        else if (sf && !af && yf) GO(true, false, true);
        else if (sf && !af && !yf) GO(true, false, false);
        else if (!sf && af && yf) GO(false, true, true);
        else if (!sf && af && !yf) GO(false, true, false);
        else if (!sf && !af && yf) GO(false, false, true);
        else GO(false, false, false);
#undef GO
        if (rc != OVK_OK)
            return rc;
    }
    return OVK_OK;
}

int32_t ovk_nbits_decode(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a, int32_t a_dtype, int64_t m,
                         void *y, int32_t y_dtype)
{
    return ovk_nbits_decode_group(ctx, 1, &w, a, a_dtype, m, &y, y_dtype);
}
