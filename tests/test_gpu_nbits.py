"""MatMulNBits parity through the C ABI against the CPU oracle (B200 only)."""
import numpy as np
import pytest
import torch

import cases
import oracle as orc
import ovk_b200
from gpu_util import assert_close, ctx, dev, host

pytestmark = pytest.mark.gpu

# the prefill kernel with per-block scaling: CTAs take whole tiles, or runs of quantization blocks that may share a tile
PER_BLOCK = ("nbits_gemm_tc", "nbits_gemm_tc_shared_k", "nbits_gemm_tc_pair", "nbits_gemm_tc_pair_shared_k")


def run_gpu(a, nib, zp, scale, k, n, bs, out_dtype=None, flags=0):
    b = dev(orc.pack_nibbles(nib, bs))
    s = dev(scale.reshape(-1))
    z = None if zp is None else dev(orc.pack_zero_points(zp))
    w = ctx().nbits_prepack(b, s, z, n, k, bs, flags=flags)
    y = ctx().matmul_nbits(w, dev(a), out_dtype=out_dtype)
    return host(y), ctx().last_kernel


@pytest.mark.parametrize("m,k,n,bs", cases.NBITS_REFERENCE_CASES)
def test_reference_cases(m, k, n, bs):
    """crates/onnx-vulkan-core/tests/matmul_nbits.rs:167-252, same tolerance (:159-164)."""
    a, nib, zp, scale = cases.nbits_reference_case(m, k, n, bs)
    got, _ = run_gpu(a, nib, zp, scale, k, n, bs)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert got.shape == (m, n)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))


@pytest.mark.parametrize("m,k,n,bs", cases.NBITS_REFERENCE_CASES)
def test_reference_cases_general_kernel(m, k, n, bs):
    """The same cases forced onto the general kernel (operator layout only)."""
    import ovk_b200
    a, nib, zp, scale = cases.nbits_reference_case(m, k, n, bs)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs, flags=ovk_b200.NBITS_NO_DECODE_COPY)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))
    if m == 1:
        assert kern == "nbits_rows"


def test_config1_single_op_fp32_no_zero_point():
    """M=1 K=N=2048 bs=32 f32, zero points absent (implicit 8); atol=rtol=1e-4."""
    a, nib, _, scale = cases.nbits_synthetic(1, 1, 2048, 2048, 32, real=np.float32,
                                             scale_lo=0.005, scale_hi=0.02, with_zp=False)
    got, _ = run_gpu(a, nib, None, scale, 2048, 2048, 32)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, None, 2048, 2048, 32)
    assert_close(got, want, 1e-4, 1e-4, "config 1")


GEMMA = [(1152, 1024), (1152, 256), (1024, 1152), (1152, 6912), (6912, 1152)]


@pytest.mark.parametrize("k,n", GEMMA)
@pytest.mark.parametrize("m", [1, 3, 8])
def test_gemma_projections_decode_fp16(k, n, m):
    """Gemma3-1B-shaped projections, fp16 in/out, atol=rtol=1e-3."""
    a, nib, zp, scale = cases.nbits_synthetic(2, m, k, n, 32)
    got, _ = run_gpu(a, nib, zp, scale, k, n, 32)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), k, n, 32)
    assert_close(got, want, 1e-3, 1e-3, f"gemma {k}->{n} M={m}")


def test_gemma_lm_head_decode_full_size():
    """K=1152 N=262144 (151 MB of weights), M=1, every output checked."""
    k, n = 1152, 262144
    a, nib, zp, scale = cases.nbits_synthetic(2, 1, k, n, 32)
    got, _ = run_gpu(a, nib, zp, scale, k, n, 32)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), k, n, 32)
    assert_close(got, want, 1e-3, 1e-3, "gemma lm_head")


@pytest.mark.parametrize("bs", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("real", [np.float32, np.float16])
def test_block_sizes_and_ragged_k(bs, real):
    """K not a multiple of the block or of 32, N not a multiple of any tile."""
    m, k, n = 2, 3 * bs + 40, 77
    a, nib, zp, scale = cases.nbits_synthetic(7, m, k, n, bs, real=real)
    got, _ = run_gpu(a, nib, zp, scale, k, n, bs)
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    tol = 1e-3 if real == np.float16 else 1e-4
    assert_close(got, want, tol, tol, f"bs={bs}")


def test_linearity_in_the_activations_full_size():
    """y(a1 + a2) == y(a1) + y(a2) within float error: a size-independent check
    on the Qwen-sized decode shape K=3584 N=18944 bs=128."""
    k, n, bs = 3584, 18944, 128
    a, nib, zp, scale = cases.nbits_synthetic(5, 2, k, n, bs, real=np.float32, scale_lo=0.001, scale_hi=0.01)
    b = dev(orc.pack_nibbles(nib, bs)); s = dev(scale.reshape(-1)); z = dev(orc.pack_zero_points(zp))
    w = ctx().nbits_prepack(b, s, z, n, k, bs)
    y1 = host(ctx().matmul_nbits(w, dev(a[0:1])))
    y2 = host(ctx().matmul_nbits(w, dev(a[1:2])))
    y12 = host(ctx().matmul_nbits(w, dev(a[0:1] + a[1:2])))
    assert_close(y12, y1 + y2, 2e-4, 2e-4, "linearity")
    cols = np.arange(0, n, 37)
    want = orc.matmul_nbits(a[0:1], orc.pack_nibbles(nib[cols], bs), scale[cols],
                            orc.pack_zero_points(zp[cols]), k, cols.size, bs)
    assert_close(y1[:, cols], want, 1e-4, 1e-4, "sampled columns")


def test_refusals_match_the_reference_predicate():
    """interp.rs:452-464: bits 4 only, block_size a multiple of 8."""
    import ovk_b200
    b = torch.zeros(64, dtype=torch.uint8, device="cuda")
    s = torch.ones(4, dtype=torch.float32, device="cuda")
    for kwargs in ({"bits": 8}, {"block_size": 12}):
        args = dict(n=4, k=32, block_size=32, bits=4)
        args.update(kwargs)
        with pytest.raises(ovk_b200.OvkError) as e:
            ctx().nbits_prepack(b, s, None, args["n"], args["k"], args["block_size"], bits=args["bits"])
        assert e.value.status == ovk_b200.UNSUPPORTED
    w = ctx().nbits_prepack(b, s, None, 4, 32, 32)
    with pytest.raises(ovk_b200.OvkError):
        ctx().matmul_nbits(w, torch.zeros(1, 31, device="cuda"))


# ------------------------------------------------------------------ prefill

@pytest.mark.parametrize("k,n,bs", [(1152, 1024, 32), (1152, 256, 32), (1024, 1152, 32), (1152, 6912, 32),
                                    (6912, 1152, 32), (512, 384, 64), (3584, 512, 128), (1024, 200, 256)])
@pytest.mark.parametrize("m", [9, 130, 512])
def test_prefill_against_the_oracle(k, n, bs, m):
    """M > 8 takes the tensor-core dequant-GEMM; fp16, atol=rtol=1e-3.  The
    Gemma3-shaped projections at M=512 are config 2's prefill case."""
    a, nib, zp, scale = cases.nbits_synthetic(2, m, k, n, bs)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    # blocks of 32 and 64 with fp16 scales: the scale goes into the weight as two exact fp16 terms;
    # larger blocks: integer weights, each block's partial sum scaled in f32
    assert kern == "nbits_gemm_tc_split" if bs <= 64 else kern in PER_BLOCK
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert_close(got, want, 1e-3, 1e-3, f"prefill {k}->{n} bs={bs} M={m}")


@pytest.mark.parametrize("n", [1793, 1921, 2049, 2368, 4000])
@pytest.mark.parametrize("m,bs", [(200, 128), (97, 64), (130, 256)])
def test_prefill_on_pairs_of_ctas_with_a_ragged_last_tile(n, m, bs):
    """Pairs of CTAs compute tiles of 256 weight columns (tcgen05.mma.cta_group::2); widths whose last tile leaves
    the second CTA of the pair one column (1921 = 15 x 128 + 1), nothing at all (1793, 2049), half a tile (2368) or
    a ragged piece (4000), with token counts whose halves are ragged too.  Blocks of 64 take f32 scales here, which
    keep them on the per-block kernel.  Every output against the CPU port."""
    k = 512
    a, nib, zp, scale = cases.nbits_synthetic(11, m, k, n, bs)
    if bs == 64:
        scale = scale.astype(np.float32)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    assert kern in PER_BLOCK
    import torch
    if torch.cuda.get_device_capability(0)[0] >= 9:
        assert "pair" in kern, kern
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert_close(got, want, 1e-3, 1e-3, f"pair prefill N={n} M={m} bs={bs}")


def test_prefill_repeats_bit_for_bit():
    """The same product a hundred times: barriers that cross a pair of CTAs, K ranges shared between CTAs and the
    fixed order of their partial sums leave no room for a result that depends on timing."""
    import torch
    for m, k, n, bs in ((700, 1024, 2368, 128), (333, 2048, 4000, 256)):
        a, nib, zp, scale = cases.nbits_synthetic(13, m, k, n, bs)
        w = ctx().nbits_prepack(dev(orc.pack_nibbles(nib, bs)), dev(scale.reshape(-1)), dev(orc.pack_zero_points(zp)), n, k, bs)
        x = dev(a)
        first = ctx().matmul_nbits(w, x).clone()
        assert ctx().last_kernel in PER_BLOCK
        for _ in range(100):
            assert torch.equal(ctx().matmul_nbits(w, x), first)
        ctx().flush()


@pytest.mark.parametrize("m,bs", [(90, 128), (150, 128), (190, 128), (200, 128), (385, 128), (200, 256)])
def test_prefill_every_token_tile_width(m, bs):
    """The per-block kernel picks 96, 128, 160 or 192 tokens per tile (with 4, 3,
    2 and 2 accumulators in flight) from the token count and the number of
    weight tiles; with 150 weight tiles on 148 SMs these token counts reach each
    width, every one with a ragged last tile.  Sampled columns against the oracle."""
    k, n = 512, 150 * 128
    a, nib, zp, scale = cases.nbits_synthetic(5, m, k, n, bs)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    assert kern in PER_BLOCK
    cols = np.r_[0:130, 9000:9130, n - 130:n]  # the first, a middle and the last weight tiles
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib[cols], bs), scale[cols], orc.pack_zero_points(zp[cols]), k,
                            cols.size, bs)
    assert_close(got[:, cols], want, 1e-3, 1e-3, f"prefill M={m} bs={bs}, sampled columns")
    # every output was written: the rows of one ragged token tile, all columns, against a float64 product
    rows = np.r_[0:3, m - 3:m]
    ref = cases.nbits_expected_f64(a[rows].astype(np.float32), nib, zp, scale.astype(np.float32), bs)
    assert_close(got[rows], ref, 2e-3, 2e-3, "prefill, whole rows")


def test_prefill_f32_output_and_missing_zero_points():
    a, nib, _, scale = cases.nbits_synthetic(6, 77, 640, 300, 32, with_zp=False)
    got, kern = run_gpu(a, nib, None, scale, 640, 300, 32, out_dtype=torch.float32)
    assert kern == "nbits_gemm_tc_split" and got.dtype == np.float32
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, None, 640, 300, 32, out_dtype=np.float32)
    assert_close(got, want, 1e-4, 1e-4, "prefill f32 out")


@pytest.mark.parametrize("m,k,n,bs", [(40, 256, 200, 32), (70, 192, 300, 64), (300, 1088, 260, 64)])
def test_prefill_small_blocks_with_f32_scales_keep_the_per_block_kernel(m, k, n, bs):
    """An f32 scale is not one fp16 number: the scale stays outside the MMA.
    Blocks of 32 are two per 64-k slab (one issuing warp), blocks of 64 one per
    slab (two issuing warps on alternate slabs, here with an odd slab count)."""
    a, nib, zp, scale = cases.nbits_synthetic(6, m, k, n, bs)
    scale32 = (scale.astype(np.float32) * np.float32(1.0001)).astype(np.float32)
    got, kern = run_gpu(a, nib, zp, scale32, k, n, bs)
    assert kern in PER_BLOCK
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale32, orc.pack_zero_points(zp), k, n, bs)
    assert_close(got, want, 1e-3, 1e-3, "prefill, f32 scales")


@pytest.mark.parametrize("m,k,n,bs", [(77, 1096, 300, 128), (200, 520, 140, 256)])
def test_prefill_per_block_kernel_f32_output_and_ragged_k(m, k, n, bs):
    """K that ends inside a quantization block, f32 output (atol = rtol = 1e-4)."""
    a, nib, zp, scale = cases.nbits_synthetic(6, m, k, n, bs)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs, out_dtype=torch.float32)
    assert kern in PER_BLOCK and got.dtype == np.float32
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs,
                            out_dtype=np.float32)
    assert_close(got, want, 1e-4, 1e-4, "prefill f32 out, ragged K")


@pytest.mark.parametrize("k,n,bs,f32_scales", [(1152, 1024, 32, False), (512, 384, 64, True), (3584, 512, 128, False),
                                               (1024, 200, 256, True), (2048, 2048, 32, True)])
@pytest.mark.parametrize("m", [9, 130, 512])
def test_prefill_with_f32_activations_takes_the_tensor_core_kernels(k, n, bs, f32_scales, m):
    """The reference computes in f32 and its models feed f32 activations: at M > 8 every row is split into two
    fp16 rows (hi + lo after a power-of-two normalisation, ~22 bits, as the decode kernel does), the prefill kernel
    runs over twice the rows, and a last pass adds the pairs.  Against the CPU port at the f32 tolerance, with rows
    of very different magnitudes, a row of zeros, and both output types."""
    a, nib, zp, scale = cases.nbits_synthetic(17, m, k, n, bs, real=np.float32)
    a = a.astype(np.float32)
    a[1] *= np.float32(3.0e4)
    a[2] *= np.float32(2.0e-6)
    a[3] = 0.0
    scale = scale.astype(np.float32 if f32_scales else np.float16)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    assert kern == "nbits_join_rows", kern
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, bs), scale, orc.pack_zero_points(zp), k, n, bs)
    assert got.dtype == np.float32
    # the reference's tolerance, 1e-4 * max(|want|, 1) for rows of N(0,1) activations
    # (tests/matmul_nbits.rs:159-164), with the 1 scaled to the row: its root mean square output
    rms = np.maximum(np.sqrt((want.astype(np.float64) ** 2).mean(axis=1, keepdims=True)), 1e-30)
    assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), rms)), (np.abs(got - want) / rms).max()
    got16, _ = run_gpu(a[4:], nib, zp, scale, k, n, bs, out_dtype=torch.float16)
    assert got16.dtype == np.float16
    assert_close(got16, want[4:], 2e-3, 2e-3, "f32 activations, fp16 output")


def test_prefill_ragged_k_and_f32_activations_fall_back_to_the_general_kernel():
    a, nib, zp, scale = cases.nbits_synthetic(6, 20, 100, 48, 32, real=np.float32)
    got, kern = run_gpu(a, nib, zp, scale, 100, 48, 32)
    assert kern == "nbits_rows"
    want = orc.matmul_nbits(a, orc.pack_nibbles(nib, 32), scale, orc.pack_zero_points(zp), 100, 48, 32)
    assert_close(got, want, 1e-4, 1e-4, "general kernel, M=20")


def test_qwen_prefill_full_size_sampled():
    """Config 5's gate/up shape at M=4096: K=3584 N=18944 bs=128, fp16; the
    oracle checks 48 token rows x 296 weight columns spread over every tile."""
    m, k, n, bs = 4096, 3584, 18944, 128
    a, nib, zp, scale = cases.nbits_synthetic(5, m, k, n, bs, scale_lo=0.001, scale_hi=0.01)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    assert kern in PER_BLOCK
    rows = np.arange(5, m, 86)
    cols = np.arange(3, n, 64)
    want = orc.matmul_nbits(a[rows], orc.pack_nibbles(nib[cols], bs), scale[cols],
                            orc.pack_zero_points(zp[cols]), k, cols.size, bs)
    assert_close(got[np.ix_(rows, cols)], want, 1e-3, 1e-3, "qwen gate/up prefill")
    assert np.isfinite(got.astype(np.float32)).all()


def _sampled(a, nib, zp, scale, k, bs, rows, cols):
    return orc.matmul_nbits(a[rows], orc.pack_nibbles(nib[cols], bs), scale[cols], orc.pack_zero_points(zp[cols]), k,
                            cols.size, bs)


def test_qwen_down_projection_full_size_sampled():
    """Config 5's down projection at M=4096: K=18944 N=3584 bs=128 - the longest K of
    the configurations, 148 quantization blocks summed per output, where error
    accumulated over K is largest.  48 token rows x 299 weight columns spread over
    every tile, atol = rtol = 1e-3 (fp16 out)."""
    m, k, n, bs = 4096, 18944, 3584, 128
    a, nib, zp, scale = cases.nbits_synthetic(5, m, k, n, bs, scale_lo=0.001, scale_hi=0.01)
    got, kern = run_gpu(a, nib, zp, scale, k, n, bs)
    assert kern in PER_BLOCK
    rows, cols = np.arange(5, m, 86), np.arange(3, n, 12)
    assert_close(got[np.ix_(rows, cols)], _sampled(a, nib, zp, scale, k, bs, rows, cols), 1e-3, 1e-3, "qwen down prefill")
    assert np.isfinite(got.astype(np.float32)).all()


def test_qwen_lm_head_full_size_sampled():
    """Config 5's lm_head at M=4096: K=3584 N=152064 bs=128 (a 1.25 GB fp16 output);
    48 token rows x 298 weight columns spread over the 1188 weight tiles."""
    m, k, n, bs = 4096, 3584, 152064, 128
    a, nib, zp, scale = cases.nbits_synthetic(5, m, k, n, bs, scale_lo=0.001, scale_hi=0.01)
    b = dev(orc.pack_nibbles(nib, bs)); s = dev(scale.reshape(-1)); z = dev(orc.pack_zero_points(zp))
    w = ctx().nbits_prepack(b, s, z, n, k, bs)
    y = ctx().matmul_nbits(w, dev(a))
    assert ctx().last_kernel in PER_BLOCK
    rows, cols = np.arange(5, m, 86), np.arange(3, n, 511)
    ctx().flush()
    got = y[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    assert_close(got, _sampled(a, nib, zp, scale, k, bs, rows, cols), 1e-3, 1e-3, "qwen lm_head prefill")
    assert bool(torch.isfinite(y).all())


def test_gemma_lm_head_prefill_full_size_sampled():
    """Config 2's lm_head at M=512: K=1152 N=262144 bs=32 with fp16 scales, the shape
    the two-term-scale kernel is benchmarked on; 32 token rows x 512 weight columns
    spread over the 2048 weight tiles, and every output finite."""
    m, k, n, bs = 512, 1152, 262144, 32
    a, nib, zp, scale = cases.nbits_synthetic(2, m, k, n, bs)
    b = dev(orc.pack_nibbles(nib, bs)); s = dev(scale.reshape(-1)); z = dev(orc.pack_zero_points(zp))
    w = ctx().nbits_prepack(b, s, z, n, k, bs)
    y = ctx().matmul_nbits(w, dev(a))
    assert ctx().last_kernel == "nbits_gemm_tc_split"
    rows, cols = np.arange(3, m, 16), np.arange(5, n, 512)
    ctx().flush()
    got = y[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    assert_close(got, _sampled(a, nib, zp, scale, k, bs, rows, cols), 1e-3, 1e-3, "gemma lm_head prefill")
    assert bool(torch.isfinite(y).all())


@pytest.mark.parametrize("shapes,m", [(((1152, 1024), (1152, 256), (1152, 256)), 1), (((1152, 6912), (1152, 6912)), 1),
                                      (((1152, 1024), (1152, 256), (1152, 256)), 3),
                                      (((256, 96), (128, 96)), 1), (((640, 300), (640, 80)), 20)])
def test_group_of_weights_over_the_same_activations(shapes, m):
    """q|k|v and gate|up in one launch: every member's result is that of its own call (bit for bit when
    the group runs as one launch, which a decode kernel name after the call shows)."""
    k0 = shapes[0][0]
    ws, packed = [], []
    a = None
    for j, (k, n) in enumerate(shapes):
        aj, nib, zp, scale = cases.nbits_synthetic(30 + j, m, k, n, 32)
        a = aj if a is None else a
        packed.append((nib, zp, scale, k, n))
        ws.append(ctx().nbits_prepack(dev(orc.pack_nibbles(nib, 32)), dev(scale.reshape(-1)),
                                      dev(orc.pack_zero_points(zp)), n, k, 32))
    same_k = all(k == k0 for k, _ in shapes)
    if not same_k:
        with pytest.raises(ovk_b200.OvkError):
            ctx().matmul_nbits_group(ws, dev(a))
        return
    before = ctx().launches
    outs = ctx().matmul_nbits_group(ws, dev(a))
    launched = ctx().launches - before
    if m <= 8:
        assert launched == 1 and ctx().last_kernel == "nbits_decode_mma"
    else:
        assert launched >= len(ws)  # one prefill launch per member (plus the lazy prefill copies)
    for w, y in zip(ws, outs):
        alone = ctx().matmul_nbits(w, dev(a))
        assert np.array_equal(host(y).view(np.uint16), host(alone).view(np.uint16))
