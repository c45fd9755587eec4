"""GPU quantiser against the CPU oracle: codes and scale bytes bit-exact, through the reference-named entry points."""
import numpy as np
import pytest

import gpu_util as G
import orc
import synth

pytestmark = pytest.mark.gpu


def edge_values(n):
    g = synth.rng(5)
    v = g.standard_normal(n).astype(np.float32)
    sp = np.array([0.0, -0.0, 448.0, -448.0, 464.0, 465.0, 6.0, 5.0, 7.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -126, 2.0 ** -140, 1e-30, 3e38, 0.25, 0.75,
                   1.25, 1.75, 2.5, 3.5, 224.0, 224.5, 3.0, 12.0, 65504.0], np.float32)
    idx = g.integers(0, n, 4 * sp.size)
    v[idx] = np.tile(np.concatenate([sp, -sp]), 2)[: idx.size]
    v[g.integers(0, n, n // 50)] *= np.float32(1e-4)      # blocks with tiny amax
    v[g.integers(0, n, n // 50)] *= np.float32(1e3)
    return v


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Cn,S", [(1, 32, 4096), (2, 64, 1000), (1, 40, 777), (1, 4, 513), (3, 16, 300), (1, 1, 4096), (1, 320, 64)])
def test_f32_to_mx(dev, bits, N, Cn, S):
    x = edge_values(N * Cn * S)
    got = G.quantise_pm(x, 0, N, Cn, S, bits)
    want = orc.pm_to_mx(x, 0, N, Cn, S, bits)
    assert got.size == want.size and np.array_equal(got, want), "%d bytes differ" % np.count_nonzero(got != want)


@pytest.mark.parametrize("bits", [8, 4])
def test_bf16_source(dev, bits):
    """lp_h16_to_mx8 / 4 with dt 1 (bf16 plane-major, src/nn_lp.h:113-116): a bf16 value is the fp32 value with the same upper 16 bits"""
    N, Cn, S = 2, 40, 1500
    x = edge_values(N * Cn * S)
    hi = (x.view(np.uint32) >> 16).astype(np.uint16)                  # truncation is as good as any rounding for making test inputs
    xf = (hi.astype(np.uint32) << 16).view(np.float32)
    got = G.quantise_pm(hi, 1, N, Cn, S, bits)
    assert np.array_equal(got, orc.pm_to_mx(xf, 0, N, Cn, S, bits))


@pytest.mark.parametrize("bits", [8, 4])
def test_h16_to_mx_and_back(dev, bits):
    N, Cn, S = 1, 32, 32 ** 3
    x = synth.act_h16(1, N * Cn * S)
    got = G.quantise_pm(x, 2, N, Cn, S, bits)
    assert np.array_equal(got, orc.pm_to_mx(x, 2, N, Cn, S, bits))
    assert np.array_equal(G.dequantise(got, bits, N, Cn, S), orc.mx_to_pm(got, bits, N, Cn, S))
    # the all-zero tensor: codes 0, scale byte 1 (exponent -126)
    z = G.quantise_pm(np.zeros(N * Cn * 64, np.float16), 2, N, Cn, 64, bits)
    assert np.all(z[: 64 * 32 * bits // 8] == 0) and np.all(z[64 * 32 * bits // 8:] == 1)


@pytest.mark.parametrize("bits", [8, 4])
def test_nan_inf_blocks(dev, bits):
    x = (0.5 * (np.arange(32 * 8) % 7)).astype(np.float32).reshape(32, 8)
    x[5, 0], x[6, 1], x[7, 2] = np.nan, np.inf, -np.inf
    got = G.quantise_pm(x, 0, 1, 32, 8, bits)
    want = orc.pm_to_mx(x, 0, 1, 32, 8, bits)
    assert np.array_equal(got, want)
    d = G.dequantise(got, bits, 1, 32, 8).reshape(32, 8)
    assert not np.isfinite(d[:, :3]).any() and np.isfinite(d[:, 3:]).all()


@pytest.mark.parametrize("bits", [8, 4])
def test_wide32_one_channel(dev, bits):
    # the network input: one channel kept in a 32-wide block
    S = 4096
    x = (synth.ct_u8(9, S).astype(np.float32) / np.float32(255)).astype(np.float16)
    want = orc.pm_to_mx(x, 2, 1, 1, S, bits, 32)
    assert np.array_equal(G.quantise_pm(x, 2, 1, 1, S, bits, wide32=True), want)
    assert np.array_equal(G.from_split(G.quantise_pm(x, 2, 1, 1, S, bits, wide32=True, layout=1), 1, 32, S, bits), want)   # the split layout holds the same bytes
    # special values in a one-channel block (its own code path): zeros, subnormals, the largest fp16, inf and NaN
    x2 = x.copy()
    x2[:8] = np.array([0.0, -0.0, 6e-8, -6.1e-5, 65504.0, np.inf, -np.inf, np.nan], np.float16)
    want2 = orc.pm_to_mx(x2, 2, 1, 1, S, bits, 32)
    assert np.array_equal(G.quantise_pm(x2, 2, 1, 1, S, bits, wide32=True), want2)
    # narrow rows (the reference's 8-wide block for C <= 8) with one channel
    assert np.array_equal(G.quantise_pm(x2, 2, 1, 1, S, bits), orc.pm_to_mx(x2, 2, 1, 1, S, bits))


def _slots(raw):
    """decode the three-word fixed-point slots: fraction in 2^-64, signed integer part, count of non-finite terms"""
    w = raw.view(np.uint64).reshape(-1, 3)
    v = w[:, 1].astype(np.int64).astype(np.float64) + w[:, 0].astype(np.float64) * 2.0 ** -64
    v[w[:, 2] != 0] = np.nan
    return v


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("N,Cn,Gn,S", [(1, 32, 8, 5000), (2, 64, 8, 4097), (1, 40, 5, 777), (2, 96, 32, 1300), (1, 64, 64, 2000), (2, 16, 4, 3000), (1, 8, 1, 1025)])      # the last two: rows of 16 / 8 channels
def test_gn_sums_mx(dev, bits, N, Cn, Gn, S):
    import ufsm_b200
    from ufsm_b200 import DevBuf
    L = ufsm_b200.lib()
    x = (synth.rng(61).standard_normal(N * Cn * S) * 3 + 1.5).astype(np.float32)
    mx = orc.pm_to_mx(x, 0, N, Cn, S, bits)
    dq = orc.mx_to_pm(mx, bits, N, Cn, S).astype(np.float64).reshape(N, Gn, -1)
    want = np.stack([dq.sum(2), (dq * dq).sum(2)], 2).reshape(-1)
    xd, sd = DevBuf(data=mx), DevBuf(N * Gn * 2 * 24).fill(0)
    dt = 3 if bits == 8 else 4
    cut = S // 3
    assert L.lp_gn_sums_mx(xd.ptr, dt, N, Cn, Gn, S, sd.ptr, 0, cut) == 0          # two spatial parts accumulate into the same slots
    assert L.lp_gn_sums_mx(xd.ptr, dt, N, Cn, Gn, S, sd.ptr, cut, S) == 0
    ufsm_b200.check()
    got = _slots(sd.download())
    assert np.allclose(got, want, rtol=1e-13, atol=1e-9), np.abs(got - want).max()
    # a second run gives the same words (integer adds: no dependence on the order of the blocks)
    s2 = DevBuf(N * Gn * 2 * 24).fill(0)
    L.lp_gn_sums_mx(xd.ptr, dt, N, Cn, Gn, S, s2.ptr, 0, cut); L.lp_gn_sums_mx(xd.ptr, dt, N, Cn, Gn, S, s2.ptr, cut, S)
    assert np.array_equal(sd.download(), s2.download())
    # finalise
    md, rd = DevBuf(N * Gn * 4), DevBuf(N * Gn * 4)
    ln = (Cn // Gn) * S
    L.umx_gn_finalize(sd.ptr, N * Gn, ln, np.float32(1e-5), md.ptr, rd.ptr)
    ufsm_b200.check()
    m = want[0::2] / ln
    v = np.maximum(want[1::2] / ln - m * m, 0)
    assert np.allclose(md.download(np.float32), m.astype(np.float32), rtol=1e-6, atol=1e-7)
    assert np.allclose(rd.download(np.float32), (1 / np.sqrt(v + 1e-5)).astype(np.float32), rtol=1e-6)
    # unsupported combinations answer -1 as the reference does
    assert L.lp_gn_sums_mx(xd.ptr, dt, N, Cn, 7 if Cn % 7 else 9, S, sd.ptr, 0, S) == -1


def test_gn_sums_mx_non_finite(dev):
    import ufsm_b200
    from ufsm_b200 import DevBuf
    L = ufsm_b200.lib()
    N, Cn, Gn, S = 1, 64, 2, 1024
    x = synth.rng(62).standard_normal(N * Cn * S).astype(np.float32)
    x[5 * S + 17] = np.inf                    # channel 5 (group 0): its block's scale byte becomes 0xFF
    mx = orc.pm_to_mx(x, 0, N, Cn, S, 8, 32)
    xd, sd = DevBuf(data=mx), DevBuf(N * Gn * 2 * 24).fill(0)
    assert L.lp_gn_sums_mx(xd.ptr, 3, N, Cn, Gn, S, sd.ptr, 0, S) == 0
    ufsm_b200.check()
    got = _slots(sd.download())
    assert np.isnan(got[0]) and np.isnan(got[1]) and np.isfinite(got[2]) and np.isfinite(got[3])
