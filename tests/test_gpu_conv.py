"""GPU parity of the tcgen05 conv against the CPU oracle, through the C ABI.  Tolerance: conv outputs within 1e-3 relative L2 of
the oracle's fp32 accumulation of the same dequantised operands (the summation order is the only freedom); with exact operands
(every product and partial sum representable) the fp32 outputs must be bit-identical."""
import numpy as np
import pytest

import gpu_util as G
import orc
import synth
from test_oracle import exact_operands

pytestmark = pytest.mark.gpu
TOL = 1e-3


oracle_conv = orc.conv_case
run_pm32 = G.run_pm32


CASES = [
    # kind, N, Ci, Co, D, H, W
    ("conv3", 1, 32, 32, 4, 16, 8),        # one tile per plane
    ("conv3", 1, 32, 32, 3, 19, 11),       # ragged: H, W not multiples of the tile
    ("conv3", 2, 64, 96, 2, 20, 9),        # two input blocks, N tile 96, batch 2
    ("conv3", 1, 96, 320, 2, 8, 8),        # three column tiles (128, 128, 64), H smaller than the tile
    ("conv3", 1, 1, 32, 5, 16, 16),        # the one-channel stem (31 zero channels)
    ("conv3", 1, 40, 33, 2, 7, 5),         # channel counts that are not multiples of 32
    ("conv1", 1, 32, 7, 3, 17, 9),         # the head
    ("conv1", 1, 320, 40, 2, 16, 8),       # ten K blocks: three stages, the last partial
    ("down2", 1, 32, 64, 4, 32, 16),       # K = 8 blocks through the space-to-depth copy
    ("down2", 1, 64, 128, 2, 6, 10),
    ("tconv2", 1, 64, 32, 2, 9, 5),        # N = 8 x 32 columns, scattered
    ("tconv2", 1, 320, 256, 1, 4, 4),
    ("conv3", 2, 256, 128, 3, 16, 16),     # a deep level: few tiles, eight input blocks split over the blocks of a tile
    ("conv3", 1, 320, 320, 2, 8, 8),       # the bottleneck: ten input blocks, three column tiles
    ("down2", 1, 256, 320, 4, 8, 8),       # K = 64 blocks in 16 stages, split
]
S2_CASES = [
    # N, Ci, Co, D, H, W of the input grid
    (1, 32, 32, 8, 32, 16),                # even grid, one input block
    (2, 64, 96, 5, 19, 11),                # odd grid (the last output voxel sees one input voxel and padding), two blocks, batch 2
    (1, 40, 33, 4, 6, 10),                 # channel counts that are not multiples of 32
    (1, 128, 256, 4, 16, 16),              # 108 K items, two column tiles, K split
]


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("kind,N,Ci,Co,D,H,W", CASES)
def test_conv_parity(dev, kind, N, Ci, Co, D, H, W, bits):
    taps = {"conv3": 27, "conv1": 1, "down2": 8, "tconv2": 8}[kind]
    x = synth.rng(11).standard_normal(N * Ci * D * H * W).astype(np.float32)
    w = synth.kaiming(12, Co, Ci, taps, transposed=(kind == "tconv2"))
    b = synth.bias(13, Co, 0.1)
    mx, want = oracle_conv(kind, x, w, b, N, Ci, D, H, W, Co, bits)
    got = run_pm32(kind, mx, w, b, N, Ci, D, H, W, Co, bits)
    assert np.isfinite(got).all()
    e = orc.rel_l2(got, want)
    assert e < TOL, "relative L2 %.3g" % e


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Ci,Co,D,H,W", S2_CASES + [(2, 96, 32, 4, 8, 16)])      # three input blocks: with MX-fp4 the second K item of a tap is half padding, also at the last sample's end
def test_conv3_stride2_parity(dev, N, Ci, Co, D, H, W, bits):
    x = synth.rng(41).standard_normal(N * Ci * D * H * W).astype(np.float32)
    w, b = synth.kaiming(42, Co, Ci, 27), synth.bias(43, Co, 0.1)
    mx, want = oracle_conv("conv3s2", x, w, b, N, Ci, D, H, W, Co, bits)
    got = run_pm32("conv3s2", mx, w, b, N, Ci, D, H, W, Co, bits)
    assert got.size == want.size and np.isfinite(got).all()
    e = orc.rel_l2(got, want)
    assert e < TOL, "relative L2 %.3g" % e
    assert np.array_equal(got, run_pm32("conv3s2", mx, w, b, N, Ci, D, H, W, Co, bits, split=False))    # reference-layout input


@pytest.mark.parametrize("Ci,Co,ybf", [(32, 32, 3), (64, 40, 4), (96, 64, 3), (8, 16, 4), (16, 32, 3)])
def test_lp_conv_fwd_s2_mxfp4_input(dev, Ci, Co, ybf):
    """lp_conv_fwd_s2_f8 on an MX-fp4 tensor computes in MX-fp4 and says so (returns 3: src/lp_s2.cu:652-716), also for inputs and outputs of
    16 channels or fewer, which are stored in rows of 8 / 16 (src/lp_common.cuh:132); exact operands, so the MX output is the oracle's bytes."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    D, H, W = 6, 10, 16
    S, So = D * H * W, (D // 2) * (H // 2) * (W // 2)
    x = exact_operands(61, (Ci, D, H, W), 0).reshape(-1)
    w = exact_operands(62, (Co, Ci, 27), 1)
    b = (synth.rng(63).integers(-8, 8, Co) * 0.5).astype(np.float32)
    mx = orc.pm_to_mx(x, 0, 1, Ci, S, 4)                       # the storage rule's row width: 8, 16 or 32 channels
    mx32 = orc.pm_to_mx(x, 0, 1, Ci, S, 4, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(mx32, 4, 1, Ci, S), 1, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 4), b, Co, 3, 2, 1)
    ob = 8 if ybf == 3 else 4
    want = orc.pm_to_mx(orc.blocked_to_pm(acc, 1, Co, So), 0, 1, Co, So, ob)       # rows of the storage rule's width, from the accumulators
    L = ufsm_b200.lib()
    xd, wd, bd = DevBuf(data=mx), DevBuf(data=w), DevBuf(data=b)
    yd = DevBuf(want.size).fill(0xEE)
    rc = L.lp_conv_fwd_s2_f8(xd.ptr, 4, Shape5(1, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, ybf, Shape5(1, Co, D // 2, H // 2, W // 2), Gnp())
    ufsm_b200.check()
    assert rc == 3
    assert np.array_equal(yd.download(), want)


def test_conv3_stride2_exact_operands_and_lp_entry(dev):
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    Ci, Co, D, H, W = 64, 40, 6, 18, 9
    x = exact_operands(51, (Ci, D, H, W), 0).reshape(-1)
    w = exact_operands(52, (Co, Ci, 27), 1)
    b = (synth.rng(53).integers(-8, 8, Co) * 0.5).astype(np.float32)
    mx, want = oracle_conv("conv3s2", x, w, b, 1, Ci, D, H, W, Co, 8)
    got = run_pm32("conv3s2", mx, w, b, 1, Ci, D, H, W, Co, 8)
    assert np.array_equal(got, want), "%d of %d differ" % (np.count_nonzero(got != want), want.size)
    # the reference's entry point: fp16 plane-major in and out
    L = ufsm_b200.lib()
    Do, Ho, Wo = (D + 1) // 2, (H + 1) // 2, (W + 1) // 2
    x16 = x.astype(np.float16)
    xd, wd, bd = DevBuf(data=x16), DevBuf(data=w), DevBuf(data=b)
    yd = DevBuf(Co * Do * Ho * Wo * 2).fill(0xEE)
    rc = L.lp_conv_fwd_s2_f8(xd.ptr, 2, Shape5(1, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, Shape5(1, Co, Do, Ho, Wo), Gnp())
    ufsm_b200.check()
    assert rc == 0
    mx16 = orc.pm_to_mx(x16, 2, 1, Ci, D * H * W, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(mx16, 8, 1, Ci, D * H * W), 1, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 8), b, Co, 3, 2, 1)
    want16 = orc.blocked_to_pm(orc.round_h16(acc), 1, Co, Do * Ho * Wo)
    assert np.array_equal(yd.download(np.float16).astype(np.float32), want16)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("kind,Ci,Co,D,H,W", [("conv3", 64, 40, 4, 18, 9), ("conv1", 96, 32, 2, 16, 8), ("down2", 32, 32, 4, 8, 16), ("tconv2", 64, 64, 2, 5, 8)])
def test_conv_exact_operands_bit_identical(dev, kind, Ci, Co, D, H, W, bits):
    taps = {"conv3": 27, "conv1": 1, "down2": 8, "tconv2": 8}[kind]
    x = exact_operands(21, (Ci, D, H, W), 0).reshape(-1)
    w = exact_operands(22, (Ci, Co, taps), 0) if kind == "tconv2" else exact_operands(22, (Co, Ci, taps), 1)
    b = (synth.rng(23).integers(-8, 8, Co) * 0.5).astype(np.float32)
    mx, want = oracle_conv(kind, x, w, b, 1, Ci, D, H, W, Co, bits)
    got = run_pm32(kind, mx, w, b, 1, Ci, D, H, W, Co, bits)
    assert np.array_equal(got, want), "%d of %d differ" % (np.count_nonzero(got != want), want.size)


def test_k_split_is_batch_invariant(dev):
    # the deep-level convs split K over several blocks per tile; the split is chosen per sample, so a sample's bytes do not depend on the batch
    Ci, Co, D, H, W = 256, 256, 4, 16, 16
    S = D * H * W
    x = synth.rng(31).standard_normal(Ci * S).astype(np.float32)
    w, b = synth.kaiming(32, Co, Ci, 27), synth.bias(33, Co, 0.1)
    mx1 = orc.pm_to_mx(x, 0, 1, Ci, S, 8, 32)
    mx2 = orc.pm_to_mx(np.concatenate([x, x]), 0, 2, Ci, S, 8, 32)
    one = run_pm32("conv3", mx1, w, b, 1, Ci, D, H, W, Co, 8)
    two = run_pm32("conv3", mx2, w, b, 2, Ci, D, H, W, Co, 8).reshape(2, -1)
    assert np.array_equal(two[0], one.reshape(-1)) and np.array_equal(two[1], one.reshape(-1))
    assert np.array_equal(one, run_pm32("conv3", mx1, w, b, 1, Ci, D, H, W, Co, 8))


def test_reference_layout_input_and_output(dev):
    # MX-fp8 tensors in the reference's own row layout (what lp_conv_fwd_f8 receives): same results as the split layout
    N, Ci, Co, D, H, W = 1, 64, 64, 3, 19, 11
    S = D * H * W
    x = synth.rng(15).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(16, Co, Ci, 27), synth.bias(17, Co, 0.1)
    mx, want = oracle_conv("conv3", x, w, b, N, Ci, D, H, W, Co, 8)
    got = run_pm32("conv3", mx, w, b, N, Ci, D, H, W, Co, 8, split=False)
    assert np.array_equal(got, run_pm32("conv3", mx, w, b, N, Ci, D, H, W, Co, 8, split=True)) and orc.rel_l2(got, want) < TOL
    c = G.Conv("conv3", w, b, Co, Ci, 8)
    a = c.fwd(mx, N, D, H, W, G.OUT_MXRAW, 8, split=False)[0]
    assert np.array_equal(a, c.fwd(mx, N, D, H, W, G.OUT_MXRAW, 8, split=True)[0])
    c.free()


@pytest.mark.parametrize("bits", [8, 4])
def test_weight_quantisation_is_the_oracles(dev, bits):
    # one-hot activations read the prepared weights back: x = e_ci at one voxel makes y[co] at that voxel = dequantised w[co][ci][centre]
    Ci, Co, D, H, W = 64, 64, 1, 16, 8
    w = synth.kaiming(31, Co, Ci, 27)
    wdq = orc.prep_w(w, Co, Ci, 27, bits).reshape(27, 64, 64)
    x = np.zeros((Ci, D * H * W), np.float32)
    for ci in range(Ci):
        x[ci, ci] = 1.0                                    # voxel ci carries channel ci alone
    mx = orc.pm_to_mx(x, 0, 1, Ci, D * H * W, bits, 32)
    got = run_pm32("conv3", mx, w, None, 1, Ci, D, H, W, Co, bits).reshape(Co, D * H * W)
    want = wdq[13].T                                       # [co][ci], centre tap
    # voxels 0..63 sit at (y, x) = (v // 8, v % 8); neighbours contribute other taps, so compare only through a second run with the centre tap alone
    w_c = np.zeros_like(w); w_c[:, :, 13] = w[:, :, 13]
    got_c = run_pm32("conv3", mx, w_c, None, 1, Ci, D, H, W, Co, bits).reshape(Co, D * H * W)
    assert np.array_equal(got_c[:, :Ci], want)
    assert np.isfinite(got).all()


@pytest.mark.parametrize("bits", [8, 4])
def test_output_modes(dev, bits):
    N, Ci, Co, D, H, W = 1, 32, 64, 2, 16, 8
    S = D * H * W
    x = synth.rng(41).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(42, Co, Ci, 27), synth.bias(43, Co, 0.1)
    mx, _ = oracle_conv("conv3", x, w, b, N, Ci, D, H, W, Co, bits)
    c = G.Conv("conv3", w, b, Co, Ci, bits)
    acc = c.fwd(mx, N, D, H, W, G.OUT_PM32)[0].view(np.float32)                     # the device's own accumulators
    acc_b = orc.pm_to_blocked(acc, N, Co, S)
    # every other epilogue is a deterministic function of those accumulators: bit-exact against the oracle's arithmetic on them
    h16 = c.fwd(mx, N, D, H, W, G.OUT_PM16)[0].view(np.float16)
    assert np.array_equal(h16, acc.astype(np.float16))
    h16b = c.fwd(mx, N, D, H, W, G.OUT_H16B)[0].view(np.float16)
    assert np.array_equal(h16b, acc_b.astype(np.float16))
    for ob in (8, 4):
        raw = c.fwd(mx, N, D, H, W, G.OUT_MXRAW, ob)[0]
        assert np.array_equal(raw, orc.blocked_to_mx(acc_b, ob, N, Co, S))
        rnd = c.fwd(mx, N, D, H, W, G.OUT_MX, ob)[0]
        assert np.array_equal(rnd, orc.blocked_to_mx(orc.round_h16(acc_b), ob, N, Co, S))
    # into the second half of a wider tensor (the decoder's concat): only blocks [2, 4) of 4 are written
    wide = c.fwd(mx, N, D, H, W, G.OUT_MX, 8, nb_dst=4, b0=2)[0]
    one = orc.blocked_to_mx(orc.round_h16(acc_b), 8, N, Co, S)
    assert np.array_equal(wide[2 * S * 32:4 * S * 32], one[:2 * S * 32]) and np.array_equal(wide[4 * S * 32 + 2 * S:], one[2 * S * 32:])
    assert np.all(wide[:2 * S * 32] == 0xEE) and np.all(wide[4 * S * 32:4 * S * 32 + 2 * S] == 0xEE)
    c.free()


def test_instance_norm_sums_and_apply(dev):
    N, Ci, Co, D, H, W = 2, 32, 96, 3, 19, 11
    S = D * H * W
    x = synth.rng(51).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(52, Co, Ci, 27), synth.bias(53, Co, 0.1)
    mx, _ = oracle_conv("conv3", x, w, b, N, Ci, D, H, W, Co, 8)
    c = G.Conv("conv3", w, b, Co, Ci, 8)
    raw, part = c.fwd(mx, N, D, H, W, G.OUT_H16B, want_part=True)
    y = raw.view(np.float16).astype(np.float32)                    # blocked fp16 the device stored
    coef, _ = G.in_coef(part, N, Co, D, H, W)
    want_coef = orc.in_coef(orc.in_sums(y, N, Co, S), N, Co, S)   # statistics of the stored values, fp64
    assert np.array_equal(coef, want_coef), "max diff %g" % np.abs(coef - want_coef).max()
    for _ in range(2):      # the one-launch form (the ticket counters reset themselves: twice in a row)
        assert np.array_equal(G.in_stats_coef(raw.view(np.float16), N, Co, D, H, W), want_coef)
    for bits in (8, 4):
        q, s2d, h = G.in_apply(y, coef, N, Co, D, H, W, 2, bits, want_h=True)
        a = orc.in_apply(y, coef, N, Co, S, 2)
        assert np.array_equal(h.astype(np.float32), a)
        assert np.array_equal(q, orc.blocked_to_mx(a, bits, N, Co, S))
    c.free()


@pytest.mark.parametrize("N,Ci,Co,D,H,W", [(2, 32, 32, 5, 20, 16), (1, 64, 64, 4, 16, 32), (2, 32, 96, 3, 9, 16), (1, 128, 64, 3, 16, 16), (2, 64, 64, 6, 16, 16), (2, 32, 96, 3, 19, 11)])
def test_conv_with_fused_norm(dev, N, Ci, Co, D, H, W):
    """umx_conv_fwd_norm: the stored tensor is the conv's; the coefficients are those of the oracle's fp64 statistics of it bit for bit,
    by the separate pass (default) and with the sums taken in the z-marching kernel's epilogue (UMX_STATS_EPILOGUE: fp64 sums of the
    stored fp16 values, exact, so no order can change them; the last shape takes the general kernel, which has no such epilogue: the
    pass again).  They do not depend on the batch."""
    S = D * H * W
    x = synth.rng(71).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(72, Co, Ci, 27), synth.bias(73, Co, 0.1)
    mx, _ = oracle_conv("conv3", x, w, b, N, Ci, D, H, W, Co, 8)
    c = G.Conv("conv3", w, b, Co, Ci, 8)
    raw, _ = c.fwd(mx, N, D, H, W, G.OUT_H16B)
    yf = raw.view(np.float16).astype(np.float32)
    exact = orc.in_coef(orc.in_sums(yf, N, Co, S), N, Co, S)
    y, coef = c.fwd_norm(mx, N, D, H, W)
    assert np.array_equal(y.view(np.uint16), raw.view(np.uint16)) and np.array_equal(coef, exact)
    for _ in range(2):          # twice: the ticket counters reset themselves
        y, coef = c.fwd_norm(mx, N, D, H, W, epilogue_stats=True)
        assert np.array_equal(y.view(np.uint16), raw.view(np.uint16))
        assert np.array_equal(coef, exact), "max diff %g" % np.abs(coef - exact).max()
    if N == 2:                  # a sample's coefficients do not depend on the batch it is in
        for n in range(2):
            one = orc.pm_to_mx(x[n * Ci * S:(n + 1) * Ci * S], 0, 1, Ci, S, 8, 32)
            _, coef1 = c.fwd_norm(one, 1, D, H, W, epilogue_stats=True)
            assert np.array_equal(coef1, coef[n * 2 * Co:(n + 1) * 2 * Co]), n
    c.free()


def test_apply_space_to_depth_and_concat(dev):
    N, Cn, D, H, W = 1, 64, 4, 6, 8
    S = D * H * W
    y = orc.round_h16(orc.pm_to_blocked(synth.rng(61).standard_normal(N * Cn * S).astype(np.float32) * 2, N, Cn, S))
    coef = np.stack([synth.rng(62).uniform(0.5, 2, N * Cn), synth.rng(63).standard_normal(N * Cn)], -1).astype(np.float32).ravel()
    a = orc.in_apply(y, coef, N, Cn, S, 2)
    q, s2d, _ = G.in_apply(y, coef, N, Cn, D, H, W, 2, 8, nb_dst=4, b0=2, want_s2d=True)
    one = orc.blocked_to_mx(a, 8, N, Cn, S)
    assert np.array_equal(q[2 * S * 32:4 * S * 32], one[:2 * S * 32]) and np.array_equal(q[4 * S * 32 + 2 * S:], one[2 * S * 32:])
    assert np.array_equal(s2d, orc.blocked_to_mx(orc.s2d_blocked(a, N, Cn, D, H, W), 8, N, 8 * Cn, S // 8))


def test_apply_scale_ranges(dev):
    """The apply's requantiser across block scales: rows whose scale 2^-e is a normal fp16 take the packed-half path, very small and
    very large rows (and inf / NaN rows) the fp32 path; all must match the oracle bit for bit."""
    N, Cn, D, H, W = 1, 64, 2, 8, 16
    S = D * H * W
    r = synth.rng(91)
    mag = 2.0 ** r.integers(-24, 16, (N, 2, S, 1)).astype(np.float64)               # per (block, voxel) magnitude from 2^-24 to 2^15
    y = (r.standard_normal((N, 2, S, 32)) * mag).astype(np.float16)
    y[0, 0, 5, 3] = np.float16(np.inf); y[0, 1, 7, 9] = np.float16(np.nan); y[0, 0, 9, :] = 0; y[0, 1, 11, 2] = np.float16(65504)
    y = y.astype(np.float32).ravel()
    coef = np.tile(np.array([1, 0], np.float32), N * Cn)                             # identity map: fmaf(x, 1, 0) == x
    a = orc.in_apply(y, coef, N, Cn, S, 0)
    for bits in (8, 4):
        q, _, h = G.in_apply(y, coef, N, Cn, D, H, W, 0, bits, want_h=True)
        assert np.array_equal(h.astype(np.float32), a, equal_nan=True)
        assert np.array_equal(q, orc.blocked_to_mx(a, bits, N, Cn, S))


def test_config2_mxfp4_down_up_pair(dev):
    """The benchmark's configuration 2 at full size: 1 x 64 x 96^3 fp16 N(0,1); a 2^3 stride-2 conv 64 -> 128 (to 48^3), then a 2^3 stride-2
    transposed conv 128 -> 64 (back to 96^3) on the fp16 result; E2M1 operands with an E8M0 scale per 32 channels, fp32 accumulate.  Each
    layer against the oracle on identical MX operands."""
    N, Ci, Cm, D = 1, 64, 128, 96
    S, Sc = D ** 3, (D // 2) ** 3
    x = synth.rng(201).standard_normal(N * Ci * S).astype(np.float16).astype(np.float32)
    w1, b1 = synth.kaiming(202, Cm, Ci, 8), synth.bias(203, Cm, 0.01)
    mxs, want1 = oracle_conv("down2", x, w1, b1, N, Ci, D, D, D, Cm, 4)
    got1 = run_pm32("down2", mxs, w1, b1, N, Ci, D, D, D, Cm, 4)
    e1 = orc.rel_l2(got1, want1)
    y = got1.astype(np.float16).astype(np.float32)                  # the fp16 output of the first layer feeds the second
    w2, b2 = synth.kaiming(204, Ci, Cm, 8, transposed=True), synth.bias(205, Ci, 0.01)
    mx2, want2 = oracle_conv("tconv2", y, w2, b2, N, Cm, D // 2, D // 2, D // 2, Ci, 4)
    got2 = run_pm32("tconv2", mx2, w2, b2, N, Cm, D // 2, D // 2, D // 2, Ci, 4)
    e2 = orc.rel_l2(got2, want2)
    print("configuration 2: down rel-L2 %.3g, up rel-L2 %.3g" % (e1, e2))
    assert got1.size == N * Cm * Sc and got2.size == N * Ci * S
    assert e1 < TOL and e2 < TOL


def test_lp_conv_fwd_f8_config1(dev):
    """The benchmark's configuration 1 through the reference's entry point: 1 x 32 x 64^3 fp16 N(0,1), 32 -> 32, MX-fp8, fp16 output."""
    import ctypes as C
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    N, Cn, D = 1, 32, 64
    S = D ** 3
    x16 = synth.act_h16(1, N * Cn * S)
    w = synth.kaiming(2, Cn, Cn, 27).astype(np.float16).astype(np.float32)
    b = synth.bias(3, Cn).astype(np.float16).astype(np.float32)
    xd, wd, bd = DevBuf(data=x16), DevBuf(data=w), DevBuf(data=b)
    yd = DevBuf(N * Cn * S * 2).fill(0xEE)
    L = ufsm_b200.lib()
    rc = L.lp_conv_fwd_f8(xd.ptr, 2, Shape5(N, Cn, D, D, D), wd.ptr, bd.ptr, Cn, yd.ptr, 2, Gnp(), None, 0, Split())
    ufsm_b200.check()
    assert rc == 0
    got = yd.download(np.float16).astype(np.float32)
    mx = orc.pm_to_mx(x16, 2, N, Cn, S, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(mx, 8, N, Cn, S), N, Cn, D, D, D, orc.prep_w(w, Cn, Cn, 27, 8), b, Cn, 3, 1, 1)
    want = orc.blocked_to_pm(orc.round_h16(acc), N, Cn, S)
    e = orc.rel_l2(got, want)
    assert e < TOL, "relative L2 %.3g" % e
    # MX in, MX out (the form the mainloop is fed in a network): codes and scales of the device's own accumulators are covered by
    # test_output_modes; here the reference's dtype codes 3 -> 3 must run and agree with the fp16 path's values to fp8 precision
    xm = DevBuf(data=mx)
    ym = DevBuf(L.lp_mx8_bytes(N, Cn, S)).fill(0xEE)
    sp = Split(); sp.wkey = 7
    for _ in range(2):     # the second call takes the memoised weights
        L.lp_conv_fwd_f8(xm.ptr, 3, Shape5(N, Cn, D, D, D), wd.ptr, bd.ptr, Cn, ym.ptr, 3, Gnp(), None, 0, sp)
    ufsm_b200.check()
    dq = orc.mx_to_pm(ym.download(), 8, N, Cn, S)
    assert orc.rel_l2(dq, want) < 0.04
    L.lp_wmemo_clear()


def test_lp_conv_fwd_f4_entry(dev):
    """lp_conv_fwd_f4 (src/nn_lp.h:54, src/lp_f4fwd.cu:30-51): E2M1 operands.  fp16 plane-major in and out on configuration 1's tensor
    (1 x 32 x 64^3) and on a 64 -> 64 layer; MX-fp4 in and out with the prepared weights memoised under split_t.wkey."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    for N, Ci, Co, D in ((1, 32, 32, 64), (2, 64, 64, 24)):
        S = D ** 3
        x16 = synth.act_h16(401, N * Ci * S)
        w = synth.kaiming(402, Co, Ci, 27)
        b = synth.bias(403, Co)
        xd, wd, bd = DevBuf(data=x16), DevBuf(data=w), DevBuf(data=b)
        yd = DevBuf(N * Co * S * 2).fill(0xEE)
        rc = L.lp_conv_fwd_f4(xd.ptr, 2, Shape5(N, Ci, D, D, D), wd.ptr, bd.ptr, Co, yd.ptr, 2, Gnp(), None, 0, Split())
        ufsm_b200.check()
        assert rc == 0
        got = yd.download(np.float16).astype(np.float32)
        mx = orc.pm_to_mx(x16, 2, N, Ci, S, 4, 32)
        acc = orc.conv_blocked(orc.mx_to_blocked(mx, 4, N, Ci, S), N, Ci, D, D, D, orc.prep_w(w, Co, Ci, 27, 4), b, Co, 3, 1, 1)
        want = orc.blocked_to_pm(orc.round_h16(acc), N, Co, S)
        e = orc.rel_l2(got, want)
        assert e < TOL, "relative L2 %.3g" % e
        # MX-fp4 in, MX-fp4 out, memoised weights: the output rows are the requantised accumulators (src/lp_common.cuh:1465-1536); against
        # the oracle's rows of its own accumulators all but the rows where the summation order moved a value across a rounding boundary
        xm = DevBuf(data=mx)
        ym = DevBuf(L.lp_mx4_bytes(N, Co, S)).fill(0xEE)
        sp = Split(); sp.wkey = 11 + Ci
        outs = []
        for _ in range(2):     # the second call takes the memoised weights
            assert L.lp_conv_fwd_f4(xm.ptr, 4, Shape5(N, Ci, D, D, D), wd.ptr, bd.ptr, Co, ym.ptr, 4, Gnp(), None, 0, sp) == 0
            ufsm_b200.check()
            outs.append(ym.download())
        assert np.array_equal(outs[0], outs[1])
        want_mx = orc.blocked_to_mx(acc, 4, N, Co, S)
        frac = np.mean(outs[0] != want_mx)
        dq = orc.mx_to_pm(outs[0], 4, N, Co, S)
        print("lp_conv_fwd_f4 %d -> %d on %d^3: fp16 out rel-L2 %.3g; MX-fp4 out: %.2e of the bytes differ from the oracle's rows" % (Ci, Co, D, e, frac))
        assert frac < 1e-4 and orc.rel_l2(dq, orc.mx_to_pm(want_mx, 4, N, Co, S)) < 5e-3
    L.lp_wmemo_clear()


def _gn_silu_oracle(dq, N, Cn, S, Gn, gamma, beta, mean, rstd, form):
    """form 0 = ((x - mean) rstd) gamma + beta (src/lp_mx_gn.cu:17), form 1 = fma(x, a, b) with a = rstd gamma, b = fma(-mean, a, beta)
    (src/lp_common.cuh:244-261, 474-476); then v / (1 + exp(-v)): the oracle's orc_gn_silu"""
    return orc.gn_silu(dq, N, Cn, S, Gn, gamma, beta, mean, rstd, form)


def _gn_params(seed, N, Cn, Gn):
    g = synth.rng(seed)
    return ((1 + 0.2 * g.standard_normal(Cn)).astype(np.float32), (0.1 * g.standard_normal(Cn)).astype(np.float32),
            (0.3 * g.standard_normal(N * Gn)).astype(np.float32), (0.5 + g.random(N * Gn)).astype(np.float32))


@pytest.mark.parametrize("shape", [(2, 64, 8, 3, 10, 12), (1, 40, 5, 5, 21, 23), (2, 16, 4, 3, 10, 12), (1, 8, 2, 2, 9, 7)])      # the second: several runs of voxels, a ragged channel block; the last two: rows of 16 / 8 channels
@pytest.mark.parametrize("xdt,ybits", [(3, 8), (4, 4), (3, 4), (2, 8), (0, 4)])
def test_gn_silu_apply_mx(dev, xdt, ybits, shape):
    """Tolerance: a transcendental (expf) sits between the operands and the requantiser, so codes may differ from the CPU evaluation where a
    value lands on a rounding boundary: at most 2e-4 of the code bytes, and 1e-3 relative L2 on the decoded tensor."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5
    L = ufsm_b200.lib()
    N, Cn, Gn, D, H, W = shape
    S = D * H * W
    x = (synth.rng(71).standard_normal(N * Cn * S) * 2).astype(np.float32)
    gamma, beta, mean, rstd = _gn_params(72, N, Cn, Gn)
    if xdt >= 3:
        src = orc.pm_to_mx(x, 0, N, Cn, S, 8 if xdt == 3 else 4)           # rows of the storage rule's width (8, 16 or 32 channels)
        dq = orc.mx_to_pm(src, 8 if xdt == 3 else 4, N, Cn, S)
    elif xdt == 2:
        src = x.astype(np.float16); dq = src.astype(np.float32)
    else:
        src = x; dq = x
    want_f = _gn_silu_oracle(dq, N, Cn, S, Gn, gamma, beta, mean, rstd, 0)
    want = orc.pm_to_mx(want_f, 0, N, Cn, S, ybits)
    xd, yd = DevBuf(data=src), DevBuf(want.size).fill(0xEE)
    bufs = [DevBuf(data=a) for a in (gamma, beta, mean, rstd)]
    L.lp_gn_silu_apply_mx(xd.ptr, xdt, Shape5(N, Cn, D, H, W), Gn, bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, yd.ptr, 3 if ybits == 8 else 4)
    ufsm_b200.check()
    got = yd.download()
    assert got.size == want.size
    assert np.count_nonzero(got != want) <= 2e-4 * want.size, "%d of %d bytes differ" % (np.count_nonzero(got != want), want.size)
    assert orc.rel_l2(orc.mx_to_pm(got, ybits, N, Cn, S), orc.mx_to_pm(want, ybits, N, Cn, S)) < TOL


@pytest.mark.parametrize("Ci,Gn", [(64, 8), (16, 2), (8, 1)])         # 16 and 8 channels: the MX input in rows of 16 / 8
@pytest.mark.parametrize("s2", [False, True])
def test_conv_entry_with_gn_silu_input_transform(dev, s2, Ci, Gn):
    """lp_conv_fwd_f8 / lp_conv_fwd_s2_f8 with gnp_t.G != 0: silu(fma(x, a, b)) quantised to MX-fp8, then the conv; fp16 plane-major out."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Co, D, H, W = 1, 32, 4, 16, 16
    S = D * H * W
    x = (synth.rng(81).standard_normal(N * Ci * S) * 2).astype(np.float32)
    w, b = synth.kaiming(82, Co, Ci, 27), synth.bias(83, Co, 0.1)
    gamma, beta, mean, rstd = _gn_params(84, N, Ci, Gn)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, 8)                       # rows of the storage rule's width
    act = _gn_silu_oracle(orc.mx_to_pm(mx, 8, N, Ci, S), N, Ci, S, Gn, gamma, beta, mean, rstd, 1)
    amx = orc.pm_to_mx(act, 0, N, Ci, S, 8, 32)
    st = 2 if s2 else 1
    Do, Ho, Wo = (D + st - 1) // st, (H + st - 1) // st, (W + st - 1) // st
    acc = orc.conv_blocked(orc.mx_to_blocked(amx, 8, N, Ci, S), N, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 8), b, Co, 3, st, 1)
    want = orc.blocked_to_pm(orc.round_h16(acc), N, Co, Do * Ho * Wo)
    xd, wd, bd = DevBuf(data=mx), DevBuf(data=w), DevBuf(data=b)
    bufs = [DevBuf(data=a) for a in (gamma, beta, mean, rstd)]
    gp = Gnp(); gp.gamma, gp.beta, gp.mean, gp.rstd, gp.G = bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, Gn
    yd = DevBuf(N * Co * Do * Ho * Wo * 2).fill(0xEE)
    if s2:
        rc = L.lp_conv_fwd_s2_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, Shape5(N, Co, Do, Ho, Wo), gp)
    else:
        rc = L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, gp, None, 0, Split())
    ufsm_b200.check()
    assert rc == 0
    e = orc.rel_l2(yd.download(np.float16).astype(np.float32), want)
    assert e < TOL, "relative L2 %.3g" % e


@pytest.mark.parametrize("xbf", [3, 2])
def test_conv_entry_with_slab_local_groupnorm(dev, xbf):
    """gnp_t.ns != 0 (src/nn_lp.h:15-18, src/lp_slab.cuh:7-12): mean and rstd per (sample, z slab), plane z in slab (z + zo) / zs clamped to
    [0, ns).  The expected tensor applies the oracle's transform slab by slab."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Ci, Co, Gn, D, H, W = 2, 64, 32, 8, 7, 8, 16
    ns, zs, zo = 3, 3, 1                          # planes 0-1, 2-4, 5-6
    S, hw = D * H * W, H * W
    x = (synth.rng(91).standard_normal(N * Ci * S) * 2).astype(np.float32)
    w, b = synth.kaiming(92, Co, Ci, 27), synth.bias(93, Co, 0.1)
    gamma, beta, mean, rstd = _gn_params(94, N * ns, Ci, Gn)
    if xbf == 3:
        src = orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
        dq = orc.mx_to_pm(src, 8, N, Ci, S, 32)
    else:
        src = x.astype(np.float16)
        dq = src.astype(np.float32)
    dq = dq.reshape(N, Ci, D, hw)
    act = np.zeros_like(dq)
    for sl in range(ns):
        zz = [z for z in range(D) if min(max((z + zo) // zs, 0), ns - 1) == sl]
        sub = np.ascontiguousarray(dq[:, :, zz[0]:zz[-1] + 1]).reshape(-1)
        m, r = mean.reshape(N, ns, Gn)[:, sl].reshape(-1), rstd.reshape(N, ns, Gn)[:, sl].reshape(-1)
        act[:, :, zz[0]:zz[-1] + 1] = _gn_silu_oracle(sub, N, Ci, len(zz) * hw, Gn, gamma, beta, np.ascontiguousarray(m), np.ascontiguousarray(r), 1).reshape(N, Ci, len(zz), hw)
    amx = orc.pm_to_mx(act.reshape(-1), 0, N, Ci, S, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(amx, 8, N, Ci, S), N, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 8), b, Co, 3, 1, 1)
    want = orc.blocked_to_pm(orc.round_h16(acc), N, Co, S)
    xd, wd, bd = DevBuf(data=src), DevBuf(data=w), DevBuf(data=b)
    bufs = [DevBuf(data=a) for a in (gamma, beta, mean, rstd)]
    gp = Gnp(); gp.gamma, gp.beta, gp.mean, gp.rstd, gp.G = bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, Gn
    gp.ns, gp.zs, gp.zo, gp.zhw = ns, zs, zo, hw
    yd = DevBuf(N * Co * S * 2).fill(0xEE)
    assert L.lp_conv_fwd_f8(xd.ptr, xbf, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, gp, None, 0, Split()) == 0
    ufsm_b200.check()
    e = orc.rel_l2(yd.download(np.float16).astype(np.float32), want)
    assert e < TOL, "relative L2 %.3g" % e


@pytest.mark.parametrize("bits,Ci,Co,N,D,H,W", [(8, 32, 7, 2, 4, 16, 16), (4, 64, 3, 1, 3, 8, 16), (8, 32, 40, 1, 2, 8, 16), (8, 32, 7, 1, 3, 5, 7)])
def test_probability_bytes_from_the_head(dev, bits, Ci, Co, N, D, H, W):
    """UMX_OUT_PROB8: the 1^3 conv writes round(254 sigmoid(fp16 logit)) itself; the bytes must be those of umx_h16_to_prob_u8 on the conv's
    fp16 plane-major output (the head's shape takes them in its epilogue from a table of all fp16 values, other shapes through that pass)."""
    import ufsm_b200
    from ufsm_b200 import DevBuf
    S = D * H * W
    x = (synth.rng(101).standard_normal(N * Ci * S) * 2).astype(np.float32)
    w = (synth.rng(102).standard_normal((Co, Ci, 1)) * 3 / np.sqrt(Ci)).astype(np.float32)
    b = synth.bias(103, Co, 0.5)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, bits, 32)
    c = G.Conv("conv1", w, b, Co, Ci, bits)
    lg, _ = c.fwd(mx, N, D, H, W, G.OUT_PM16)
    pb, _ = c.fwd(mx, N, D, H, W, G.OUT_PROB8)
    c.free()
    L = ufsm_b200.lib()
    ld, od = DevBuf(data=lg), DevBuf(lg.size // 2).fill(0xEE)
    L.umx_h16_to_prob_u8(ld.ptr, lg.size // 2, od.ptr)
    ufsm_b200.check()
    assert np.array_equal(pb, od.download())
    p = 1.0 / (1.0 + np.exp(-lg.view(np.float16).astype(np.float64)))
    assert np.abs(pb.astype(np.float64) - 254.0 * p).max() <= 0.5 + 1e-3
