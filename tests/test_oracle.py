"""The CPU oracle against the reference's golden definitions: its own conversions compiled from src/mx_sw.cuh (when built), the
committed vectors generated from that build, the host formulas of the reference's tests (tests/test_mx4.c:36-54,
tests/test_mx4_wide.c:123-148) restated in numpy, and the exact-operand conv construction of tests/test_mx4_wide.c:1-30."""
import ctypes as C
import os

import numpy as np
import pytest

import orc
import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mx_golden.npz")
G8 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)


def test_golden_vectors():
    g = np.load(GOLD)
    x = g["x_bits"].view(np.float32)
    assert np.array_equal(orc.enc(x, 8), g["e4m3"])
    assert np.array_equal(orc.enc(x, 4), g["e2m1"])
    o = orc.o()
    d8 = np.array([o.orc_dec_e4m3(b) for b in range(256)], np.float32).view(np.uint32)
    d4 = np.array([o.orc_dec_e2m1(b) for b in range(16)], np.float32).view(np.uint32)
    nan8 = np.isnan(g["dec_e4m3_bits"].view(np.float32))
    assert np.array_equal(d8[~nan8], g["dec_e4m3_bits"][~nan8]) and np.all(np.isnan(d8.view(np.float32)[nan8]))
    assert np.array_equal(d4, g["dec_e2m1_bits"])


def test_encoders_against_reference_build():
    r = orc.ref()
    if r is None:
        pytest.skip("oracle/_ref not built (reference tree absent); the golden vectors cover this")
    o = orc.o()
    bad = C.c_uint32(0)
    # every 251st fp32 bit pattern (17.1 M inputs) and the whole neighbourhood of the e4m3 saturation and subnormal thresholds
    for fmt, fn in ((8, o.orc_enc_e4m3), (4, o.orc_enc_e2m1)):
        f = C.cast(fn, C.c_void_p)
        assert r.ref_sweep_diff(fmt, f, 0, 251, (1 << 32) // 251, C.byref(bad)) == 0, hex(bad.value)
        for lo in (0x43d00000, 0x3c000000, 0x39800000, 0x40900000, 0x3e700000, 0x7f700000, 0xc3d00000):
            assert r.ref_sweep_diff(fmt, f, lo, 1, 1 << 21, C.byref(bad)) == 0, hex(bad.value)


@pytest.mark.skipif(not os.environ.get("UFSM_FULL_SWEEP"), reason="all 2^32 inputs: set UFSM_FULL_SWEEP=1 (about 20 s)")
def test_encoders_all_inputs():
    r = orc.ref()
    if r is None:
        pytest.skip("oracle/_ref not built")
    o = orc.o()
    for fmt, fn in ((8, o.orc_enc_e4m3), (4, o.orc_enc_e2m1)):
        assert r.ref_sweep_diff(fmt, C.cast(fn, C.c_void_p), 0, 1, 1 << 32, None) == 0


def test_mx_exp_known_answers():
    e = orc.o().orc_mx_exp
    q8, q4 = np.float32(1.0) / np.float32(448.0), np.float32(1.0) / np.float32(6.0)
    assert e(448.0, q8) == 0 and e(449.0, q8) == 1 and e(224.0, q8) == -1 and e(224.5, q8) == 0
    assert e(6.0, q4) == 0 and e(3.0, q4) == -1 and e(6.5, q4) == 1 and e(12.0, q4) == 1
    assert e(0.0, q8) == -126 and e(1e-45, q4) == -126 and e(3e38, q8) == 120
    assert e(np.inf, q8) == 128 and e(np.nan, q4) == 128 and e(3.4e38, np.float32(4.0)) == 128


def _host_mx_exp(am, inv):
    """tests/test_mx4_wide.c:123-128 in numpy (vectorised)."""
    p = (am.astype(np.float32) * np.float32(inv)).astype(np.float32)
    u = p.view(np.uint32)
    e = ((u >> 23) & 255).astype(np.int64) - 127 + ((u & 0x7fffff) != 0)
    return np.clip(e, -126, 126)


def _host_e2m1(a):
    """tests/test_mx4.c:38-45: nearest grid point, ties to the even code, a >= 0."""
    a = np.minimum(a, 6.0)
    i = np.clip(np.searchsorted(G8, a, side="right") - 1, 0, 6)
    lo, hi = G8[i], G8[i + 1]
    d, u = a - lo, hi - a
    up = (u < d) | ((u == d) & (i % 2 == 1))
    return np.where(a >= 6.0, 6.0, np.where(up, hi, lo)).astype(np.float32)


@pytest.mark.parametrize("scale", [1.0, 4.0, 1e-3, 300.0])
def test_quantiser_against_host_formula_fp4(scale):
    # the decoded values of the oracle's MX-fp4 quantiser == the host quantiser of the reference's tests on the same data
    N, Cn, S = 2, 32, 512
    x = (synth.rng(7).standard_normal(N * Cn * S) * scale).astype(np.float32)
    mx = orc.pm_to_mx(x, 0, N, Cn, S, 4)
    got = orc.mx_to_pm(mx, 4, N, Cn, S).reshape(N, Cn, S)
    xr = x.reshape(N, Cn, S)
    am = np.abs(xr).max(axis=1)
    e = _host_mx_exp(am, np.float32(1.0) / np.float32(6.0))
    m = np.ldexp(np.float32(1.0), -e).astype(np.float32)[:, None, :]
    want = np.copysign(_host_e2m1(np.abs(xr) * m) / m, xr)
    assert np.array_equal(got, want.astype(np.float32))


def test_storage_layout_and_sizes():
    # sizes and the 8 / 16 / 32 block widths of src/lp_common.cuh:132-134, nibble order, scale plane after the data
    assert orc.mx_bytes(8, 1, 32, 64 ** 3) == 64 ** 3 * 33 and orc.mx_bytes(4, 1, 64, 96 ** 3) == 2 * 96 ** 3 * 17
    assert orc.mx_bytes(8, 2, 4, 10) == 2 * 10 * 9 and orc.mx_bytes(4, 1, 16, 10) == 10 * 9 and orc.mx_bytes(8, 1, 40, 10) == 2 * 10 * 33
    N, Cn, S = 1, 40, 6
    x = np.zeros((N, Cn, S), np.float32)
    x[0, 1, 2] = 6.0      # block 0, voxel 2, channel 1 -> high nibble of byte 0 of that row
    x[0, 33, 5] = -3.0    # block 1, voxel 5, channel 1
    mx = orc.pm_to_mx(x, 0, N, Cn, S, 4)
    rows = mx[:2 * S * 16].reshape(2, S, 16)
    sc = mx[2 * S * 16:].reshape(2, S)
    assert rows[0, 2, 0] == 0x70 and sc[0, 2] == 127 and rows[1, 5, 0] == 0xf0 and sc[1, 5] == 126   # -3 at scale 2^-1 is the code of -6
    assert sc[0, 0] == 1          # an all-zero block: exponent -126
    assert np.count_nonzero(rows) == 2


def test_nan_inf_policy():
    # a NaN or inf anywhere in a block: scale byte 0xFF, the block decodes non-finite (tests/test_mx4.c:139-168)
    for bits in (8, 4):
        for bad in (np.nan, np.inf, -np.inf):
            x = (0.5 * (np.arange(32 * 4) % 7)).astype(np.float32).reshape(1, 32, 4)
            x[0, 5, 0] = bad
            mx = orc.pm_to_mx(x, 0, 1, 32, 4, bits)
            rb = 32 * bits // 8
            assert mx[4 * rb] == 0xff and np.all(mx[4 * rb + 1:] != 0xff)
            d = orc.mx_to_pm(mx, bits, 1, 32, 4).reshape(32, 4)
            assert not np.isfinite(d[:, 0]).any() and np.isfinite(d[:, 1:]).all()


def _np_conv(x, w, b, k, stride, pad):
    """Direct conv in float64: x [Ci][D][H][W], w [Co][Ci][k^3] -> [Co][Do][Ho][Wo]."""
    Ci, D, H, W = x.shape
    Co = w.shape[0]
    xp = np.pad(x.astype(np.float64), ((0, 0), (pad, pad), (pad, pad), (pad, pad)))
    Do, Ho, Wo = (D + 2 * pad - k) // stride + 1, (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    y = np.zeros((Co, Do, Ho, Wo))
    wr = w.astype(np.float64).reshape(Co, Ci, k, k, k)
    for kz in range(k):
        for ky in range(k):
            for kx in range(k):
                sl = xp[:, kz:kz + stride * Do:stride, ky:ky + stride * Ho:stride, kx:kx + stride * Wo:stride]
                y += np.einsum("oc,cdhw->odhw", wr[:, :, kz, ky, kx], sl)
    return y + (b.astype(np.float64)[:, None, None, None] if b is not None else 0)


def exact_operands(seed, shape, block_axis):
    """Values on the e2m1 grid with a +-6 in every 32-block along block_axis: every MX scale is 1, codes are lossless."""
    g = synth.rng(seed)
    v = (G8[g.integers(0, 8, shape)] * np.where(g.integers(0, 2, shape) > 0, 1, -1)).astype(np.float32)
    v = np.moveaxis(v, block_axis, -1)
    n = v.shape[-1]
    for b0 in range(0, n, 32):
        v[..., b0 + g.integers(0, min(32, n - b0))] = 6.0
    return np.ascontiguousarray(np.moveaxis(v, -1, block_axis))


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("k,stride,pad", [(3, 1, 1), (1, 1, 0), (2, 2, 0)])
def test_conv_exact_operands(bits, k, stride, pad):
    # exact-operand construction: all products and sums exact, so the fp32-accumulating oracle equals the float64 conv bit for bit
    Ci, Co, D, H, W = 64, 40, 4, 6, 8
    x = exact_operands(1, (Ci, D, H, W), 0)
    w = exact_operands(2, (Co, Ci, k ** 3), 1)
    b = (synth.rng(3).integers(-8, 8, Co) * 0.5).astype(np.float32)
    S = D * H * W
    mx = orc.pm_to_mx(x.reshape(1, Ci, S), 0, 1, Ci, S, bits, 32)
    assert np.all(mx[-orc.nb32(Ci) * S:] == (127 if bits == 4 else 121))   # amax 6: scale 1 (fp4) or 2^-6 (fp8), codes lossless either way
    xb = orc.mx_to_blocked(mx, bits, 1, Ci, S)
    wdq = orc.prep_w(w, Co, Ci, k ** 3, bits)
    y = orc.conv_blocked(xb, 1, Ci, D, H, W, wdq, b, Co, k, stride, pad)
    want = _np_conv(x, w, b, k, stride, pad)
    got = orc.blocked_to_pm(y, 1, Co, want[0].size).reshape(want.shape)
    assert np.array_equal(got.astype(np.float64), want)


def test_tconv_exact_operands():
    Ci, Co, D, H, W = 64, 32, 3, 4, 5
    x = exact_operands(4, (Ci, D, H, W), 0)
    w = exact_operands(5, (Ci, Co, 8), 0)          # PyTorch ConvTranspose3d order [ci][co][8]; blocks run along ci
    b = (synth.rng(6).integers(-8, 8, Co) * 0.5).astype(np.float32)
    S = D * H * W
    xb = orc.pm_to_blocked(x.reshape(1, Ci, S), 1, Ci, S)
    wdq = orc.prep_w(w, Co, Ci, 8, 8, layout=1)
    y = orc.blocked_to_pm(orc.tconv_blocked(xb, 1, Ci, D, H, W, wdq, b, Co), 1, Co, 8 * S).reshape(Co, 2 * D, 2 * H, 2 * W)
    want = np.zeros((Co, 2 * D, 2 * H, 2 * W))
    for a in range(2):
        for bb in range(2):
            for e in range(2):
                want[:, a::2, bb::2, e::2] = np.einsum("co,cdhw->odhw", w[:, :, (a * 2 + bb) * 2 + e].astype(np.float64), x.astype(np.float64))
    want += b[:, None, None, None]
    assert np.array_equal(y.astype(np.float64), want)


def test_space_to_depth_is_the_stride2_conv():
    # a 2^3 stride-2 conv == a 1^3 conv over the space-to-depth copy with K blocks ordered (tap, block)
    Ci, Co, D = 64, 32, 4
    x = synth.rng(8).standard_normal((Ci, D, D, D)).astype(np.float32)
    w = synth.kaiming(9, Co, Ci, 8)
    S = D ** 3
    xb = orc.fake_quant_blocked(orc.pm_to_blocked(x.reshape(1, Ci, S), 1, Ci, S), 8)
    y2 = orc.conv_blocked(xb, 1, Ci, D, D, D, orc.prep_w(w, Co, Ci, 8, 8), None, Co, 2, 2, 0)
    xs = orc.s2d_blocked(xb, 1, Ci, D, D, D)
    w1 = np.ascontiguousarray(w.transpose(0, 2, 1).reshape(Co, 8 * Ci))      # [co][tap * Ci + ci]
    y1 = orc.conv_blocked(xs, 1, 8 * Ci, D // 2, D // 2, D // 2, orc.prep_w(w1, Co, 8 * Ci, 1, 8), None, Co, 1, 1, 0)
    assert orc.rel_l2(y1, y2) < 1e-6


def test_instance_norm_apply():
    N, Cn, S = 2, 40, 300
    y = orc.round_h16(orc.pm_to_blocked(synth.rng(10).standard_normal(N * Cn * S).astype(np.float32) * 3 + 1, N, Cn, S))
    sums = orc.in_sums(y, N, Cn, S)
    ypm = orc.blocked_to_pm(y, N, Cn, S).reshape(N, Cn, S).astype(np.float64)
    assert np.allclose(sums.reshape(N, Cn, 2)[..., 0], ypm.sum(-1), rtol=1e-12) and np.allclose(sums.reshape(N, Cn, 2)[..., 1], (ypm ** 2).sum(-1), rtol=1e-12)
    coef = orc.in_coef(sums, N, Cn, S)
    out = orc.blocked_to_pm(orc.in_apply(y, coef, N, Cn, S, 2), N, Cn, S).reshape(N, Cn, S)
    m, v = ypm.mean(-1, keepdims=True), ypm.var(-1, keepdims=True)
    ref = (ypm - m) / np.sqrt(v + 1e-5)
    ref = np.where(ref < 0, 0.01 * ref, ref)
    assert np.abs(out - ref).max() < 4e-3          # fp16 rounding of the result
    assert np.array_equal(out, out.astype(np.float16).astype(np.float32))


def test_unet_small_runs():
    cfg = orc.unet_cfg(16, [32, 64])
    w = synth.unet_weights(1, [32, 64])
    assert w.size == orc.unet_nweights(cfg)
    x = (synth.ct_u8(2, 16 ** 3).astype(np.float32) / np.float32(255)).astype(np.float16)
    y = orc.unet_forward(cfg, w, x, 1)
    assert np.isfinite(y).all() and y.std() > 0
    assert np.array_equal(y, orc.unet_forward(cfg, w, x, 1))


def test_elementwise_operator_restatements():
    """orc_up2, orc_conv1, orc_gn_silu against independent float64 evaluations"""
    r = np.random.default_rng(5)
    N, Cn, D, H, W = 2, 3, 3, 4, 5
    S = D * H * W
    x = r.standard_normal(N * Cn * S).astype(np.float32)
    # trilinear 2x, align_corners false with clamped edges: the separable float64 form
    def lin(a, axis):
        n = a.shape[axis]
        o = np.arange(2 * n)
        near, far = o >> 1, np.clip((o >> 1) + np.where(o & 1, 1, -1), 0, n - 1)
        return 0.75 * np.take(a, near, axis) + 0.25 * np.take(a, far, axis)
    want = lin(lin(lin(x.reshape(N, Cn, D, H, W).astype(np.float64), 2), 3), 4)
    got = orc.up2(x, N, Cn, D, H, W).reshape(want.shape)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    assert np.array_equal(orc.up2(np.full(N * Cn * S, 1.5, np.float32), N, Cn, D, H, W), np.full(8 * N * Cn * S, 1.5, np.float32))   # weights sum to one exactly
    w, b = r.standard_normal((4, Cn)).astype(np.float32), r.standard_normal(4).astype(np.float32)
    c1 = orc.conv1(x, w, b, N, Cn, 4, S).reshape(N, 4, S)
    assert np.allclose(c1, np.einsum("oc,ncs->nos", w.astype(np.float64), x.reshape(N, Cn, S).astype(np.float64)) + b[None, :, None], rtol=1e-5, atol=1e-5)
    Gn = 3
    gamma, beta = (1 + 0.2 * r.standard_normal(Cn)).astype(np.float32), (0.1 * r.standard_normal(Cn)).astype(np.float32)
    mean, rstd = (0.3 * r.standard_normal(N * Gn)).astype(np.float32), (0.5 + r.random(N * Gn)).astype(np.float32)
    u = ((x.reshape(N, Cn, S).astype(np.float64) - mean.reshape(N, Gn, 1)) * rstd.reshape(N, Gn, 1)) * gamma[None, :, None] + beta[None, :, None]
    silu = u / (1 + np.exp(-u))
    for form in (0, 1):
        assert np.allclose(orc.gn_silu(x, N, Cn, S, Gn, gamma, beta, mean, rstd, form).reshape(N, Cn, S), silu, rtol=2e-6, atol=2e-6)
    # a channel segment of a larger tensor takes the larger tensor's groups and parameters
    whole = orc.gn_silu(x, N, Cn, S, Gn, gamma, beta, mean, rstd, 1).reshape(N, Cn, S)
    seg = orc.gn_silu(np.ascontiguousarray(x.reshape(N, Cn, S)[:, 1:]), N, Cn - 1, S, Gn, gamma, beta, mean, rstd, 1, 1, Cn).reshape(N, Cn - 1, S)
    assert np.array_equal(seg, whole[:, 1:])


def test_one_channel_fp8_row_is_rounding_to_four_bits():
    """An MX-fp8 row with one real channel (the network's input) holds its value rounded to nearest-even at four significant bits: the
    block scale puts |x| 2^-e into (224, 448], where E4M3 neither saturates nor is subnormal.  Checked for every finite fp16 value; the
    tap-packed first conv quantises its fp16 input by this rule."""
    h = np.arange(65536, dtype=np.uint16).view(np.float16)
    x = h[np.isfinite(h)].astype(np.float32)
    mx = orc.pm_to_mx(x, 0, 1, 1, x.size, 8, 32)
    want = orc.mx_to_blocked(mx, 8, 1, 1, x.size).reshape(-1, 32)[:, 0]
    u = x.view(np.uint32).astype(np.uint64)
    got = ((u + 0x7FFFF + ((u >> 20) & 1)) & 0xFFF00000).astype(np.uint32).view(np.float32)
    assert np.array_equal(got, want) and np.array_equal(np.signbit(got), np.signbit(want))


def test_predict_back_end_restatement():
    """prob255 / pred_place / ctmask (the predict back end, src/nn_elem.cu:1096-1178): known answers and the box arithmetic"""
    assert list(orc.prob255([0.0, 40.0, -40.0, -200.0, np.log(3.0)])) == [128, 255, 0, 0, 191]      # 127.5 + 0.5; 255; 0; exp overflow; 191.25 + 0.5
    W, halo, shard = 8, 2, 10
    lg = np.zeros(W ** 3, np.float32)
    mat = np.ones(W ** 3, bool)
    mat[(3 * W + 3) * W + 3] = False
    out = orc.pred_place(lg, mat, W, W, halo, halo, -3, 0, 5, 10, 10, 9, shard, np.full(shard ** 3, 7, np.uint8)).reshape(shard, shard, shard)
    want = np.full((shard, shard, shard), 7, np.uint8)
    want[0:3, 2:6, 7:9] = 128                   # z: window planes 3..5 (0..2 lie below the shard), y: 2..5, x: 2..3 (the extent ends at 9)
    want[0, 3, 8] = 0                           # the voxel that is not material
    assert np.array_equal(out, want)
    ct = np.arange(70, dtype=np.uint8)
    bits = orc.ctmask(ct, 33)
    assert bits.size == 3 and bits[0] == 0 and bits[1] == 0xFFFFFFFE and bits[2] == 0x3F


def test_feather_restatement_partition_of_unity():
    """the seam feather's weights (src/predict.c:282-296): with every neighbour present the weights of a lower-shell voxel sum to 1, so windows
    that all predict the same byte blend to that byte; with none present the window's own bytes come back"""
    S, B, osh = 6, 3, 6
    E = S + B
    e = np.full(E ** 3, 77, np.uint8)
    sizes = {d: (B * E * E if d & 4 else S * B * E if d & 2 else S * S * B) for d in range(1, 8)}
    nb = [None] + [np.full(sizes[d], 77, np.uint8) for d in range(1, 8)]
    out = orc.feather_blend(e, nb, S, B, (0, 0, 0), (S, S, S), osh, np.zeros(osh ** 3, np.uint8))
    assert (out == 77).all()
    u = orc.feather_u(B)
    assert np.allclose(u[0] + u[1], 1, atol=1e-7) and u[0][0] < u[0][-1]
    r = synth.rng(5).integers(0, 256, E ** 3, dtype=np.uint8)
    out = orc.feather_blend(r, [None] * 8, S, B, (0, 0, 0), (S, S, S), osh, np.zeros(osh ** 3, np.uint8))
    assert np.array_equal(out.reshape(osh, osh, osh), r.reshape(E, E, E)[:S, :S, :S])
