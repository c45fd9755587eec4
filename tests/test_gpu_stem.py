"""GPU parity of the tap-packed one-channel 3^3 conv (the network's first layer reading the fp16 patch itself, UMX_X_H16) against the CPU
oracle's MX conv of the quantised input and against the library's own quantise-then-conv path.  The operands are the same MX-fp8
values in both paths and every product is exact, so the only freedom is the order of the fp32 additions: outputs within 1e-3
relative L2 of the oracle (the tolerance of all conv outputs), and the stored fp16 values of the two GPU paths at most one fp16 step
apart (or 2e-6 where the sum cancels).  Shapes the kernel does not take (W not a multiple of 8, MX-fp4, another output mode) must give exactly what quantise-then-
conv gives, since they run it."""
import numpy as np
import pytest

import gpu_util as G
import orc
import synth
from ufsm_b200 import npapi

pytestmark = pytest.mark.gpu
TOL = 1e-3

CASES = [
    # N, Co, D, H, W, input
    (1, 32, 5, 16, 16, "normal"),          # two tiles a plane
    (2, 32, 4, 20, 24, "normal"),          # H not a multiple of the tile, batch 2
    (1, 20, 3, 7, 8, "normal"),            # fewer than 32 outputs, H smaller than the tile
    (1, 32, 1, 16, 8, "u8"),               # one plane
    (1, 32, 64, 64, 64, "u8"),             # blocks walk several runs of planes and cross from one tile to the next
]


def make_x(kind, n):
    r = synth.rng(71)
    if kind == "u8":
        return (r.integers(0, 256, n).astype(np.float32) / 255.0).astype(np.float16)
    x = r.standard_normal(n).astype(np.float32)
    x[::97] = 0.0
    x[5::113] *= 1e-4           # small values: the one-channel rows get their own scale, far from their neighbours'
    return x.astype(np.float16)


def h16b_pm(raw, N, Co, S):
    return orc.blocked_to_pm(raw.view(np.float16).astype(np.float32), N, Co, S)


@pytest.mark.parametrize("N,Co,D,H,W,kind", CASES)
def test_stem_parity(dev, N, Co, D, H, W, kind):
    S = D * H * W
    x16 = make_x(kind, N * S)
    w, b = synth.kaiming(72, Co, 1, 27), synth.bias(73, Co, 0.1)
    mx, want = orc.conv_case("conv3", x16.astype(np.float32), w, b, N, 1, D, H, W, Co, 8)
    c = npapi.Conv("conv3", w, b, Co, 1, 8)
    raw, _, k = c.fwd_h16(x16, N, D, H, W)
    assert k == 3, "the tap-packed kernel did not run"
    got = h16b_pm(raw, N, Co, S)
    assert np.isfinite(got).all()
    e = orc.rel_l2(got, want.astype(np.float16).astype(np.float32))
    assert e < TOL, "relative L2 %.3g" % e
    # the library's other path on the same operands: the quantiser's MX tensor through the MX conv
    raw2, _ = c.fwd(mx, N, D, H, W, npapi.OUT_H16B)
    a, r = raw.view(np.float16), raw2.view(np.float16)
    assert a.size == r.size
    ai, ri = a.view(np.int16).astype(np.int32), r.view(np.int16).astype(np.int32)
    near = (np.abs(ai - ri) <= 1) | (np.abs(a.astype(np.float32) - r.astype(np.float32)) <= 2e-6)     # one fp16 step, or fp32 rounding of a cancelling sum
    assert near.all()
    assert (ai != ri).mean() < 0.02
    # and the coefficients of the InstanceNorm that follows are those of the stored tensor
    raw3, coef, k3 = c.fwd_h16(x16, N, D, H, W, norm=True)
    assert k3 == 3 and np.array_equal(raw3, raw)
    assert np.array_equal(coef, npapi.in_stats_coef(raw.view(np.float16), N, Co, D, H, W))
    if kind == "u8":
        # CT bytes as the input (UMX_X_U8): the bytes of the fp16 input byte / 255, in the kernel and in the quantise-first path (W = 12)
        ct = (x16.astype(np.float32) * 255).round().astype(np.uint8)
        assert np.array_equal((ct.astype(np.float32) / np.float32(255)).astype(np.float16), x16)
        raw8, _, k8 = c.fwd_h16(ct, N, D, H, W, u8=True)
        assert k8 == 3 and np.array_equal(raw8, raw)
    c.free()


@pytest.mark.parametrize("Ci,Co,D,H,W,bits,mode", [
    (1, 32, 3, 16, 12, 8, "h16b"),         # W not a multiple of 8
    (1, 32, 3, 16, 16, 4, "h16b"),         # MX-fp4
    (1, 32, 3, 16, 16, 8, "pm32"),         # another output mode
    (1, 48, 2, 16, 16, 8, "h16b"),         # more than 32 outputs
    (5, 32, 2, 16, 16, 8, "h16b"),         # more than one input channel
])
def test_fp16_input_other_shapes(dev, Ci, Co, D, H, W, bits, mode):
    S = D * H * W
    x16 = make_x("normal", Ci * S)
    w, b = synth.kaiming(74, Co, Ci, 27), synth.bias(75, Co, 0.1)
    mx = orc.pm_to_mx(x16.astype(np.float32), 0, 1, Ci, S, bits, 32)
    c = npapi.Conv("conv3", w, b, Co, Ci, bits)
    om = npapi.OUT_H16B if mode == "h16b" else npapi.OUT_PM32
    raw, _, k = c.fwd_h16(x16, 1, D, H, W, out_mode=om)
    assert k != 3
    raw2, _ = c.fwd(mx, 1, D, H, W, om)
    assert np.array_equal(raw, raw2)
    if Ci == 1 and bits == 8 and mode == "h16b":
        ct = synth.ct_u8(76, S)
        r8, _, k8 = c.fwd_h16(ct, 1, D, H, W, out_mode=om, u8=True)
        r16, _, _ = c.fwd_h16((ct.astype(np.float32) / np.float32(255)).astype(np.float16), 1, D, H, W, out_mode=om)
        assert (k8 == 3) == (W % 8 == 0 and Co <= 32) and np.array_equal(r8, r16)
    c.free()
