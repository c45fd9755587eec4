"""GPU parity of the reference interface's elementwise MX operators (trilinear 2x upsample, 1^3 conv with fp32 weights) against the
oracle's restatements of the reference's arithmetic order (orc_up2, orc_conv1, orc_gn_silu; src/lp_mx_gn.cu:32-72, src/lp_mx_conv1.cu:4-22)."""
import numpy as np
import pytest

import orc
import synth

pytestmark = pytest.mark.gpu
f32, f64 = np.float32, np.float64


def gn_params(seed, N, Cn, Gn):
    g = synth.rng(seed)
    return ((1 + 0.2 * g.standard_normal(Cn)).astype(f32), (0.1 * g.standard_normal(Cn)).astype(f32),
            (0.3 * g.standard_normal(N * Gn)).astype(f32), (0.5 + g.random(N * Gn)).astype(f32))


def make_gp(Gn, arrays):
    from ufsm_b200 import DevBuf, Gnp
    bufs = [DevBuf(data=a) for a in arrays]
    gp = Gnp()
    gp.gamma, gp.beta, gp.mean, gp.rstd, gp.G = bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, Gn
    return gp, bufs


def slab_gn_silu(dq, N, Cn, D, hw, Gn, pr, ns, zs, zo):
    """silu(gn(x)) with statistics per (sample, z slab): plane z in slab (z + zo) // zs clamped to [0, ns) (src/lp_slab.cuh:7-12), slab by slab"""
    gamma, beta, mean, rstd = pr
    x = dq.reshape(N, Cn, D, hw)
    out = np.zeros_like(x)
    for sl in range(ns):
        zz = [z for z in range(D) if min(max((z + zo) // zs, 0), ns - 1) == sl]
        if not zz:
            continue
        sub = np.ascontiguousarray(x[:, :, zz[0]:zz[-1] + 1]).reshape(-1)
        m = np.ascontiguousarray(mean.reshape(N, ns, Gn)[:, sl]).reshape(-1)
        r = np.ascontiguousarray(rstd.reshape(N, ns, Gn)[:, sl]).reshape(-1)
        out[:, :, zz[0]:zz[-1] + 1] = orc.gn_silu(sub, N, Cn, len(zz) * hw, Gn, gamma, beta, m, r, 1).reshape(N, Cn, len(zz), hw)
    return out.reshape(-1)


@pytest.mark.parametrize("bits", [8, 4])
def test_slab_local_groupnorm_in_up2_and_conv1(dev, bits):
    """gnp_t.ns != 0 in lp_up2_fwd_mx and lp_conv1_fwd_mx: the statistics of the slab a (coarse) plane lies in"""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5
    L = ufsm_b200.lib()
    dt = 3 if bits == 8 else 4
    # upsample: six coarse planes in three slabs (0 | 1 2 | 3 4 5)
    N, Cn, Gn, D, H, W, ns, zs, zo = 2, 40, 5, 6, 9, 11, 3, 2, 1
    S, hw = D * H * W, H * W
    x = (synth.rng(401).standard_normal(N * Cn * S) * 2).astype(f32)
    mx = orc.pm_to_mx(x, 0, N, Cn, S, bits, 32)
    pr = gn_params(402, N * ns, Cn, Gn)
    gp, keep = make_gp(Gn, pr)
    gp.ns, gp.zs, gp.zo, gp.zhw = ns, zs, zo, hw
    act = slab_gn_silu(orc.mx_to_pm(mx, bits, N, Cn, S, 32), N, Cn, D, hw, Gn, pr, ns, zs, zo)
    want = orc.pm_to_mx(orc.up2(act, N, Cn, D, H, W), 0, N, Cn, 8 * S, bits, 32)
    xd, yd = DevBuf(data=mx), DevBuf(want.size).fill(0xEE)
    L.lp_up2_fwd_mx(xd.ptr, dt, Shape5(N, Cn, D, H, W), yd.ptr, dt, gp)
    ufsm_b200.check()
    bad = np.count_nonzero(yd.download() != want)
    assert bad <= 2e-4 * want.size, "%d of %d bytes differ" % (bad, want.size)
    # 1^3 conv: planes of 117 voxels, so a block of 512 voxels touches up to three slabs (0 1 | 2 3 | 4)
    N, Ci, Co, D, H, W, ns, zs, zo = 2, 64, 7, 5, 9, 13, 3, 2, 0
    S, hw = D * H * W, H * W
    x = (synth.rng(403).standard_normal(N * Ci * S) * 2).astype(f32)
    w = (synth.rng(404).standard_normal((Co, Ci)) / np.sqrt(Ci)).astype(f32)
    b = (0.1 * synth.rng(405).standard_normal(Co)).astype(f32)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, bits, 32)
    pr = gn_params(406, N * ns, Ci, 8)
    gp, keep2 = make_gp(8, pr)
    gp.ns, gp.zs, gp.zo, gp.zhw = ns, zs, zo, hw
    act = slab_gn_silu(orc.mx_to_pm(mx, bits, N, Ci, S, 32), N, Ci, D, hw, 8, pr, ns, zs, zo)
    want = orc.conv1(act, w, b, N, Ci, Co, S).reshape(N, Co, S)
    xd, wd, bd, yd = DevBuf(data=mx), DevBuf(data=w), DevBuf(data=b), DevBuf(N * Co * S * 4).fill(0xEE)
    L.lp_conv1_fwd_mx(xd.ptr, dt, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, gp)
    ufsm_b200.check()
    assert orc.rel_l2(yd.download(f32).reshape(N, Co, S), want) < 1e-5


# the second shape spans several tiles of the kernel on every axis (4 x 4 x 16 cells of the dual grid), with ragged last tiles
@pytest.mark.parametrize("shape", [(2, 40, 5, 3, 5, 7), (1, 64, 8, 6, 9, 35), (2, 16, 2, 3, 5, 7), (1, 8, 1, 2, 6, 5)])      # the last two: rows of 16 / 8 channels
@pytest.mark.parametrize("xbits,ybits,gn", [(8, 8, False), (4, 4, False), (8, 4, False), (4, 8, False), (8, 8, True), (4, 4, True)])
def test_up2_fwd_mx(dev, xbits, ybits, gn, shape):
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    L = ufsm_b200.lib()
    N, Cn, Gn, D, H, W = shape
    S = D * H * W
    x = (synth.rng(91).standard_normal(N * Cn * S) * 2).astype(f32)
    mx = orc.pm_to_mx(x, 0, N, Cn, S, xbits)                 # rows of the storage rule's width
    dq = orc.mx_to_pm(mx, xbits, N, Cn, S)
    gp, keep = Gnp(), None
    if gn:
        pr = gn_params(92, N, Cn, Gn)
        gp, keep = make_gp(Gn, pr)
        dq = orc.gn_silu(dq, N, Cn, S, Gn, *pr, 1)
    want = orc.pm_to_mx(orc.up2(dq, N, Cn, D, H, W), 0, N, Cn, 8 * S, ybits)
    xd, yd = DevBuf(data=mx), DevBuf(want.size).fill(0xEE)
    L.lp_up2_fwd_mx(xd.ptr, 3 if xbits == 8 else 4, Shape5(N, Cn, D, H, W), yd.ptr, 3 if ybits == 8 else 4, gp)
    ufsm_b200.check()
    got = yd.download()
    bad = np.count_nonzero(got != want)
    if gn:      # a transcendental ahead of the requantiser: codes on a rounding boundary may differ (tolerance as for lp_gn_silu_apply_mx)
        assert bad <= 2e-4 * want.size, "%d of %d bytes differ" % (bad, want.size)
    else:
        assert bad == 0, "%d of %d bytes differ" % (bad, want.size)


@pytest.mark.parametrize("bits,Ci,Co,N,h16,gn", [(8, 32, 7, 1, False, False), (4, 64, 16, 2, False, False), (8, 40, 3, 1, True, False), (8, 64, 32, 2, False, False), (8, 64, 7, 2, False, True), (4, 96, 10, 1, False, True),
                                                   (8, 16, 7, 2, False, False), (4, 8, 3, 1, True, True)])          # rows of 16 / 8 channels
def test_conv1_fwd_mx(dev, bits, Ci, Co, N, h16, gn):
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    L = ufsm_b200.lib()
    D, H, W = 5, 9, 13                # 585 voxels: a full trip of 512 a block and a ragged one
    S = D * H * W
    x = (synth.rng(95).standard_normal(N * Ci * S) * 2).astype(f32)
    w = (synth.rng(96).standard_normal((Co, Ci)) / np.sqrt(Ci)).astype(f32)
    b = (0.1 * synth.rng(97).standard_normal(Co)).astype(f32)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, bits)
    dq = orc.mx_to_pm(mx, bits, N, Ci, S)
    gp, keep = Gnp(), None
    if gn:
        pr = gn_params(98, N, Ci, 8)
        gp, keep = make_gp(8, pr)
        dq = orc.gn_silu(dq, N, Ci, S, 8, *pr, 1)
    acc = orc.conv1(dq, w, b, N, Ci, Co, S).reshape(N, Co, S)
    xd, wd, bd = DevBuf(data=mx), DevBuf(data=w), DevBuf(data=b)
    yd = DevBuf(N * Co * S * (2 if h16 else 4)).fill(0xEE)
    fn = L.lp_conv1_fwd_mx_h16 if h16 else L.lp_conv1_fwd_mx
    fn(xd.ptr, 3 if bits == 8 else 4, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, gp)
    ufsm_b200.check()
    got = yd.download(np.float16 if h16 else f32).astype(f32).reshape(N, Co, S)
    want = acc.astype(np.float16).astype(f32) if h16 else acc
    if gn:
        assert orc.rel_l2(got, want) < 1e-5
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("bits", [8, 4])
def test_up2_blocks_conv1_ranges_and_add(dev, bits):
    """lp_up2_fwd_mx_blocks (the upsample of a range of 32-channel blocks), lp_conv1_fwd_mx_r / _h16_r (a range of voxels: the bits of the
    whole-tensor call), lp_add_mx (y += x, rows re-encoded)."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    L = ufsm_b200.lib()
    dt = 3 if bits == 8 else 4
    N, Cn, D, H, W = 2, 96, 3, 5, 9
    S = D * H * W
    x = (synth.rng(301).standard_normal(N * Cn * S) * 2).astype(f32)
    mx = orc.pm_to_mx(x, 0, N, Cn, S, bits, 32)
    dq = orc.mx_to_pm(mx, bits, N, Cn, S, 32).reshape(N, Cn, S)
    xd = DevBuf(data=mx)
    # blocks 1 and 2 (channels 32 .. 95) upsampled alone
    part = np.ascontiguousarray(dq[:, 32:96]).reshape(-1)
    want = orc.pm_to_mx(orc.up2(part, N, 64, D, H, W), 0, N, 64, 8 * S, bits, 32)
    yd = DevBuf(want.size).fill(0xEE)
    L.lp_up2_fwd_mx_blocks(xd.ptr, dt, Shape5(N, Cn, D, H, W), 1, 2, yd.ptr, dt)
    ufsm_b200.check()
    assert np.array_equal(yd.download(), want)
    # a range of voxels of the 1^3 conv: one sample (the fp32 form takes no batch), planes of their own length or inside a wider buffer
    Co = 7
    w = (synth.rng(302).standard_normal((Co, Cn)) / np.sqrt(Cn)).astype(f32)
    b = (0.1 * synth.rng(303).standard_normal(Co)).astype(f32)
    mx1 = orc.pm_to_mx(x[:Cn * S], 0, 1, Cn, S, bits, 32)
    x1, wd, bd = DevBuf(data=mx1), DevBuf(data=w), DevBuf(data=b)
    whole = orc.conv1(orc.mx_to_pm(mx1, bits, 1, Cn, S, 32), w, b, 1, Cn, Co, S).reshape(Co, S)
    vb, nv, ly = 17, 77, 100
    y32 = DevBuf(Co * ly * 4).fill(0xEE)
    assert L.lp_conv1_fwd_mx_r(x1.ptr, dt, Shape5(1, Cn, D, H, W), wd.ptr, bd.ptr, Co, y32.ptr, Gnp(), vb, nv, ly) == 0
    y16 = DevBuf(Co * nv * 2).fill(0xEE)
    L.lp_conv1_fwd_mx_h16_r(x1.ptr, dt, Shape5(1, Cn, D, H, W), wd.ptr, bd.ptr, Co, y16.ptr, Gnp(), vb, nv)
    ufsm_b200.check()
    g32 = y32.download(f32).reshape(Co, ly)
    assert np.array_equal(g32[:, :nv], whole[:, vb:vb + nv]) and (y32.download().reshape(Co, ly * 4)[:, nv * 4:] == 0xEE).all()
    assert np.array_equal(y16.download(np.float16).reshape(Co, nv), whole[:, vb:vb + nv].astype(np.float16))
    assert L.lp_conv1_fwd_mx_r(xd.ptr, dt, Shape5(N, Cn, D, H, W), wd.ptr, bd.ptr, Co, y32.ptr, Gnp(), vb, nv, ly) == -1       # a batch: refused as in the reference
    # y += x
    x2 = (synth.rng(304).standard_normal(N * Cn * S) * 3).astype(f32)
    mx2 = orc.pm_to_mx(x2, 0, N, Cn, S, bits, 32)
    want = orc.pm_to_mx((dq.reshape(-1) + orc.mx_to_pm(mx2, bits, N, Cn, S, 32)).astype(f32), 0, N, Cn, S, bits, 32)
    yd, x2d = DevBuf(data=mx), DevBuf(data=mx2)
    L.lp_add_mx(yd.ptr, x2d.ptr, Shape5(N, Cn, D, H, W), bits, 0)
    ufsm_b200.check()
    assert np.array_equal(yd.download(), want)
    # the same on a tensor of 16 channels: rows of 16 (src/lp_common.cuh:132)
    Cs = 16
    a16 = (synth.rng(305).standard_normal(N * Cs * S) * 3).astype(f32)
    b16 = (synth.rng(306).standard_normal(N * Cs * S) * 3).astype(f32)
    ma, mb = orc.pm_to_mx(a16, 0, N, Cs, S, bits), orc.pm_to_mx(b16, 0, N, Cs, S, bits)
    want = orc.pm_to_mx((orc.mx_to_pm(ma, bits, N, Cs, S) + orc.mx_to_pm(mb, bits, N, Cs, S)).astype(f32), 0, N, Cs, S, bits)
    yd, x2d = DevBuf(data=ma), DevBuf(data=mb)
    L.lp_add_mx(yd.ptr, x2d.ptr, Shape5(N, Cs, D, H, W), bits, 0)
    ufsm_b200.check()
    assert np.array_equal(yd.download(), want)
