"""GPU parity of the conv entry points' split_t fields (src/nn_lp.h:20-37 of the reference): concat input (x2 / c_split / gp2), the x
part stored at half resolution (up), split output (y2 / o_split), GroupNorm sums of the stored output (osum / Go / stored_stats /
zlo / zhi).  The expected values are built from the oracle's pieces in the order the reference's kernels apply them while staging:
transform, blend, quantise rows of 32 channels to the conv's format, per-tensor 32-channel segments (src/lp_f8fwd.cuh:617-623), conv."""
import numpy as np
import pytest

import orc
import synth

pytestmark = pytest.mark.gpu
f32 = np.float32
TOL = 1e-3


def up32(c):
    return (c + 31) // 32 * 32


def gn_params(seed, N, Cn, Gn):
    g = synth.rng(seed)
    return ((1 + 0.2 * g.standard_normal(Cn)).astype(f32), (0.1 * g.standard_normal(Cn)).astype(f32),
            (0.3 * g.standard_normal(N * Gn)).astype(f32), (0.5 + g.random(N * Gn)).astype(f32))


def make_gp(Gn, arrays, keep):
    from ufsm_b200 import DevBuf, Gnp
    bufs = [DevBuf(data=a) for a in arrays]
    keep.extend(bufs)
    gp = Gnp()
    gp.gamma, gp.beta, gp.mean, gp.rstd, gp.G = bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, Gn
    return gp


def expand_w(w, b, Co, Ci, Cx, cin, Ox, cout_c):
    """weights of the conv on padded segments: input channel ci at ci (ci < Cx) or up32(Cx) + ci - Cx, output channel likewise"""
    wp = np.zeros((cout_c, cin, 27), f32)
    bp = np.zeros(cout_c, f32)
    pi = np.array([c if c < Cx else up32(Cx) + c - Cx for c in range(Ci)])
    po = np.array([c if c < Ox else up32(Ox) + c - Ox for c in range(Co)])
    wp[np.ix_(po, pi)] = w.reshape(Co, Ci, 27)
    bp[po] = b
    return wp, bp


def padded_segments(a, b, N, Ca, Cb, S):
    """two plane-major tensors as one with each part padded to whole 32-channel blocks"""
    out = np.zeros((N, up32(Ca) + up32(Cb), S), f32)
    out[:, :Ca] = a.reshape(N, Ca, S)
    out[:, up32(Ca):up32(Ca) + Cb] = b.reshape(N, Cb, S)
    return out.reshape(-1)


CASES = [
    # storage, bits, Cx, C2, up, gn ("", "seg" = one GroupNorm per part, "all" = one over both parts)
    (2, 8, 40, 24, False, ""),          # plane-major parts, split inside a block
    (3, 8, 40, 32, False, ""),          # MX parts, the x part padded to two blocks
    (4, 4, 32, 64, False, ""),
    (3, 8, 64, 32, True, ""),           # decoder form: [upsampled coarse | skip]
    (4, 4, 32, 32, True, "seg"),
    (3, 8, 40, 40, False, "seg"),
    (3, 8, 32, 32, False, "all"),
    (2, 8, 32, 48, False, "seg"),
    (4, 8, 32, 32, True, "seg"),        # MX-fp4 storage into an MX-fp8 conv: the transform requantises
    (3, 8, 16, 32, False, ""),          # an MX part of 16 channels: rows of 16 (src/lp_common.cuh:132)
    (4, 4, 8, 8, False, ""),            # two parts in rows of 8
]


@pytest.mark.parametrize("xbf,bits,Cx,C2,up,gn", CASES)
def test_concat_input(dev, xbf, bits, Cx, C2, up, gn):
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Co, D, H, W = 2, 32, 4, 8, 16
    Ci, S = Cx + C2, D * H * W
    Dc, Hc, Wc = (D // 2, H // 2, W // 2) if up else (D, H, W)
    Sc = Dc * Hc * Wc
    sb = 8 if xbf == 3 else 4
    xa = (synth.rng(201).standard_normal(N * Cx * Sc) * 2).astype(f32)
    xb = (synth.rng(202).standard_normal(N * C2 * S) * 2).astype(f32)
    w, b = synth.kaiming(203, Co, Ci, 27), synth.bias(204, Co, 0.1)
    keep = []
    if xbf == 2:
        sa, sb_ = xa.astype(np.float16), xb.astype(np.float16)
        da, db = sa.astype(f32), sb_.astype(f32)
    else:
        sa, sb_ = orc.pm_to_mx(xa, 0, N, Cx, Sc, sb), orc.pm_to_mx(xb, 0, N, C2, S, sb)           # rows of the storage rule's width
        da, db = orc.mx_to_pm(sa, sb, N, Cx, Sc), orc.mx_to_pm(sb_, sb, N, C2, S)
    gp, sp = Gnp(), Split()
    if gn == "seg":
        pa, pb = gn_params(205, N, Cx, 8), gn_params(206, N, C2, 4)
        gp = make_gp(8, pa, keep)
        sp.gp2 = make_gp(4, pb, keep)
        da, db = orc.gn_silu(da, N, Cx, Sc, 8, *pa, 1), orc.gn_silu(db, N, C2, S, 4, *pb, 1)
    elif gn == "all":
        pa = gn_params(207, N, Ci, 8)
        gp = make_gp(8, pa, keep)
        da, db = orc.gn_silu(da, N, Cx, S, 8, *pa, 1, 0, Ci), orc.gn_silu(db, N, C2, S, 8, *pa, 1, Cx, Ci)
    if up:
        da = orc.up2(da, N, Cx, Dc, Hc, Wc)
    if xbf == 2 and not gn:                  # plane-major parts: blocks over the concatenated index
        cin = Ci
        cat = np.concatenate([da.reshape(N, Cx, S), db.reshape(N, C2, S)], 1).reshape(-1)
        wp, bp = w.reshape(Co, Ci, 27), b
    else:
        cin = up32(Cx) + up32(C2)
        cat = padded_segments(da, db, N, Cx, C2, S)
        wp, bp = expand_w(w, b, Co, Ci, Cx, cin, Co, Co)
    amx = orc.pm_to_mx(cat, 0, N, cin, S, bits, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(amx, bits, N, cin, S), N, cin, D, H, W, orc.prep_w(wp, Co, cin, 27, bits), bp, Co, 3, 1, 1)
    want = orc.blocked_to_pm(orc.round_h16(acc), N, Co, S)
    xd, x2d, wd, bd = DevBuf(data=sa), DevBuf(data=sb_), DevBuf(data=w), DevBuf(data=b)
    sp.x2, sp.c_split, sp.up = x2d.ptr, Cx, 1 if up else 0
    yd = DevBuf(N * Co * S * 2).fill(0xEE)
    fn = L.lp_conv_fwd_f8 if bits == 8 else L.lp_conv_fwd_f4
    assert fn(xd.ptr, xbf, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, gp, None, 0, sp) == 0
    ufsm_b200.check()
    got = yd.download(np.float16).astype(f32)
    e = orc.rel_l2(got, want)
    print("concat input storage %d -> MX-fp%d conv, %d + %d channels%s%s: rel-L2 %.3g" % (xbf, bits, Cx, C2, ", up" if up else "", ", gn " + gn if gn else "", e))
    # a transcendental ahead of the requantiser flips a code now and then (a 6 % step of that element in fp8, 25 % in fp4)
    assert e < TOL


def test_concat_up_with_slab_local_groupnorm(dev):
    """the decoder form [upsample(silu(gn(coarse))) | silu(gn(skip))] with the coarse part's statistics per z slab of the coarse tensor
    (gnp_t.ns / zs / zo / zhw count its planes) and the skip part's per sample"""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    from test_gpu_mxops import slab_gn_silu
    L = ufsm_b200.lib()
    N, Cx, C2, Co, D, H, W = 2, 32, 32, 32, 4, 8, 16
    Dc, Hc, Wc = D // 2, H // 2, W // 2
    Ci, S, Sc, hwc = Cx + C2, D * H * W, Dc * Hc * Wc, Hc * Wc
    ns, zs, zo = 2, 1, 0                                     # one coarse plane a slab
    xa = (synth.rng(261).standard_normal(N * Cx * Sc) * 2).astype(f32)
    xb = (synth.rng(262).standard_normal(N * C2 * S) * 2).astype(f32)
    w, b = synth.kaiming(263, Co, Ci, 27), synth.bias(264, Co, 0.1)
    sa, sb_ = orc.pm_to_mx(xa, 0, N, Cx, Sc, 8, 32), orc.pm_to_mx(xb, 0, N, C2, S, 8, 32)
    pa, pb = gn_params(265, N * ns, Cx, 8), gn_params(266, N, C2, 4)
    keep = []
    gp = make_gp(8, pa, keep)
    gp.ns, gp.zs, gp.zo, gp.zhw = ns, zs, zo, hwc
    sp = Split()
    sp.gp2 = make_gp(4, pb, keep)
    da = slab_gn_silu(orc.mx_to_pm(sa, 8, N, Cx, Sc, 32), N, Cx, Dc, hwc, 8, pa, ns, zs, zo)
    db = orc.gn_silu(orc.mx_to_pm(sb_, 8, N, C2, S, 32), N, C2, S, 4, *pb, 1)
    cat = padded_segments(orc.up2(da, N, Cx, Dc, Hc, Wc), db, N, Cx, C2, S)
    amx = orc.pm_to_mx(cat, 0, N, Ci, S, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(amx, 8, N, Ci, S), N, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 8), b, Co, 3, 1, 1)
    want = orc.blocked_to_pm(orc.round_h16(acc), N, Co, S)
    xd, x2d, wd, bd = DevBuf(data=sa), DevBuf(data=sb_), DevBuf(data=w), DevBuf(data=b)
    sp.x2, sp.c_split, sp.up = x2d.ptr, Cx, 1
    yd = DevBuf(N * Co * S * 2).fill(0xEE)
    assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, gp, None, 0, sp) == 0
    ufsm_b200.check()
    assert orc.rel_l2(yd.download(np.float16).astype(f32), want) < TOL


@pytest.mark.parametrize("ybf,Ox,O2", [(2, 40, 24), (3, 32, 32), (3, 40, 56), (4, 64, 32), (3, 16, 16), (4, 8, 40), (3, 40, 8)])
def test_split_output_and_stored_stats(dev, ybf, Ox, O2):
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Ci, D, H, W = 2, 32, 4, 8, 16
    Co, S = Ox + O2, D * H * W
    x = (synth.rng(211).standard_normal(N * Ci * S) * 2).astype(f32)
    w, b = synth.kaiming(212, Co, Ci, 27), synth.bias(213, Co, 0.1)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(mx, 8, N, Ci, S), N, Ci, D, H, W, orc.prep_w(w, Co, Ci, 27, 8), b, Co, 3, 1, 1)
    want = orc.blocked_to_pm(acc, N, Co, S).reshape(N, Co, S)
    xd, wd, bd = DevBuf(data=mx), DevBuf(data=w), DevBuf(data=b)
    sp = Split()
    ob = 8 if ybf == 3 else 4
    nbytes = (lambda c: N * c * S * 2) if ybf == 2 else (lambda c: orc.mx_bytes(ob, N, c, S))      # parts of 16 channels or fewer in rows of 8 / 16
    yd, y2d = DevBuf(nbytes(Ox)).fill(0xEE), DevBuf(nbytes(O2)).fill(0xEE)
    sp.y2, sp.o_split = y2d.ptr, Ox
    if Ox <= 16 and O2 <= 16:
        sp.o_pad = 16                                        # what the reference's caller passes for two such tensors (src/nn_lp.h:32)
    assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, ybf, Gnp(), None, 0, sp) == 0
    ufsm_b200.check()
    for buf, c0, c in ((yd, 0, Ox), (y2d, Ox, O2)):
        part = np.ascontiguousarray(want[:, c0:c0 + c]).reshape(-1)
        if ybf == 2:
            got = buf.download(np.float16).astype(f32)
            assert orc.rel_l2(got, part.astype(np.float16).astype(f32)) < TOL
        else:
            got = buf.download()
            wmx = orc.pm_to_mx(part, 0, N, c, S, ob)              # each part an MX tensor of its own blocks
            assert got.size == wmx.size
            frac = np.count_nonzero(got != wmx) / got.size
            assert frac < (2e-3 if ob == 8 else 1e-3), frac           # accumulation order flips a code now and then
            assert orc.rel_l2(orc.mx_to_pm(got, ob, N, c, S), orc.mx_to_pm(wmx, ob, N, c, S)) < (5e-3 if ob == 8 else 2e-2)
    if ybf == 2:
        return
    # the same conv, one MX output, with the GroupNorm sums of the stored values over the planes [zlo, D - zhi)
    Go, zlo, zhi = 8, 1, 1
    yall, sums = DevBuf(orc.mx_bytes(ob, N, Co, S, 32)).fill(0xEE), DevBuf(N * Go * 2 * 24).fill(0)
    sp = Split()
    sp.stored_stats, sp.zlo, sp.zhi = 1, zlo, zhi
    assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yall.ptr, ybf, Gnp(), sums.ptr, Go, sp) == 0
    ufsm_b200.check()
    stored = orc.mx_to_pm(yall.download(), ob, N, Co, S, 32).astype(np.float64).reshape(N, Go, Co // Go, D, H * W)[:, :, :, zlo:D - zhi]
    ws = sums.download().view(np.uint64).reshape(-1, 3)
    got = ws[:, 1].astype(np.int64).astype(np.float64) + ws[:, 0].astype(np.float64) * 2.0 ** -64
    exp = np.stack([stored.sum((2, 3, 4)), (stored * stored).sum((2, 3, 4))], 2).reshape(-1)
    assert (ws[:, 2] == 0).all() and np.allclose(got, exp, rtol=1e-13, atol=1e-9)
    # stored_stats 0: the sums of acc + bias before the rounding to MX; the output tensor is the same
    yraw, sraw = DevBuf(orc.mx_bytes(ob, N, Co, S, 32)).fill(0xEE), DevBuf(N * Go * 2 * 24).fill(0)
    sp0 = Split()
    sp0.zlo, sp0.zhi = zlo, zhi
    assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yraw.ptr, ybf, Gnp(), sraw.ptr, Go, sp0) == 0
    ufsm_b200.check()
    assert np.array_equal(yraw.download(), yall.download())
    unr = want.astype(np.float64).reshape(N, Go, Co // Go, D, H * W)[:, :, :, zlo:D - zhi]
    wr = sraw.download().view(np.uint64).reshape(-1, 3)
    gotr = wr[:, 1].astype(np.int64).astype(np.float64) + wr[:, 0].astype(np.float64) * 2.0 ** -64
    expr = np.stack([unr.sum((2, 3, 4)), (unr * unr).sum((2, 3, 4))], 2).reshape(-1)
    assert (wr[:, 2] == 0).all() and np.allclose(gotr, expr, rtol=2e-5, atol=1e-3)          # the oracle's accumulators, another summation order
    if Ox % 32 or O2 <= 16:
        return
    # and of a split output whose first part ends on a block: the same sums, the same bytes in the two tensors
    sums2 = DevBuf(N * Go * 2 * 24).fill(0)
    sp.y2, sp.o_split = y2d.fill(0xEE).ptr, Ox
    assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.fill(0xEE).ptr, ybf, Gnp(), sums2.ptr, Go, sp) == 0
    ufsm_b200.check()
    assert np.array_equal(sums2.download(), sums.download())
    whole = orc.mx_to_pm(yall.download(), ob, N, Co, S, 32).reshape(N, Co, S)
    assert np.array_equal(orc.mx_to_pm(yd.download(), ob, N, Ox, S, 32).reshape(N, Ox, S), whole[:, :Ox])
    assert np.array_equal(orc.mx_to_pm(y2d.download(), ob, N, O2, S, 32).reshape(N, O2, S), whole[:, Ox:])


def test_unbuilt_fields_stop(dev):
    """what is not built says so (checked here through the checks that run ahead of any launch: a child process, since the entry aborts)"""
    import subprocess
    import sys
    code = ("import ufsm_b200, ctypes as C\nfrom ufsm_b200 import Shape5, Gnp, Split\nL = ufsm_b200.lib()\nassert L.nn_init(0) == 0\n"
            "sp = Split(); sp.sr = 7\nL.lp_conv_fwd_f8(None, 3, Shape5(1, 32, 4, 8, 16), None, None, 32, None, 3, Gnp(), None, 0, sp)\n")
    r = subprocess.run([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=orc.ROOT)
    assert r.returncode != 0 and "not built" in r.stderr


@pytest.mark.parametrize("bits,hd,axis", [(8, 2, 1), (4, 2, -1), (8, 1, 1), (8, 0, 0)])
def test_pred_input_mx_and_narrow_rows(dev, bits, hd, axis):
    """lp_pred_input_mx: bytes equal to the oracle's values quantised to rows of 8 channels; then those rows (4 channels, 8 wide) as the
    input of a stem conv through lp_conv_fwd_f8 / _f4, and a conv with an MX output of 16 channels (16-wide rows)."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    W, depth, z0, nz = 16, 7, 2, 4
    S = nz * W * W
    ct = synth.ct_u8(221, depth * W * W)
    g = synth.rng(222)
    dyo, dxo = (g.standard_normal(depth) * 3 - 8).astype(f32), (g.standard_normal(depth) * 3 - 7).astype(f32)
    mean, isd = f32(110.0), f32(1 / 40.0)
    vals = orc.pred_input(ct, W, mean, isd, dyo, dxo, axis, z0, nz, hd)
    want = orc.pm_to_mx(vals, 0, 1, 4, S, bits)                       # 4 channels: one block of 8 a voxel
    ctd, dyd, dxd = DevBuf(data=ct), DevBuf(data=dyo), DevBuf(data=dxo)
    yd = DevBuf(want.size).fill(0xEE)
    L.lp_pred_input_mx(ctd.ptr, W, mean, isd, dyd.ptr, dxd.ptr, axis, z0, nz, yd.ptr, hd, bits)
    ufsm_b200.check()
    got = yd.download()
    assert np.array_equal(got, want), "%d of %d bytes differ" % (np.count_nonzero(got != want), want.size)
    # stem conv 4 -> 32 on the narrow rows, fp16 out; then 32 -> 16 with an MX output of 16-wide rows
    Co = 32
    w, b = synth.kaiming(223, Co, 4, 27), synth.bias(224, Co, 0.1)
    dq = orc.mx_to_pm(want, bits, 1, 4, S)
    wide = orc.pm_to_mx(dq, 0, 1, 4, S, bits, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(wide, bits, 1, 4, S), 1, 4, nz, W, W, orc.prep_w(w, Co, 4, 27, bits), b, Co, 3, 1, 1)
    wh = orc.blocked_to_pm(orc.round_h16(acc), 1, Co, S)
    wd, bd, od = DevBuf(data=w), DevBuf(data=b), DevBuf(Co * S * 2).fill(0xEE)
    fn = L.lp_conv_fwd_f8 if bits == 8 else L.lp_conv_fwd_f4
    assert fn(yd.ptr, 3 if bits == 8 else 4, Shape5(1, 4, nz, W, W), wd.ptr, bd.ptr, Co, od.ptr, 2, Gnp(), None, 0, Split()) == 0
    ufsm_b200.check()
    assert orc.rel_l2(od.download(np.float16).astype(f32), wh) < TOL
    w2, b2 = synth.kaiming(225, 16, Co, 27), synth.bias(226, 16, 0.1)
    xin = orc.pm_to_mx(wh, 0, 1, Co, S, bits, 32)
    acc2 = orc.conv_blocked(orc.mx_to_blocked(xin, bits, 1, Co, S), 1, Co, nz, W, W, orc.prep_w(w2, 16, Co, 27, bits), b2, 16, 3, 1, 1)
    want2 = orc.pm_to_mx(orc.blocked_to_pm(acc2, 1, 16, S), 0, 1, 16, S, bits)       # rows of 16 channels
    xd2, wd2, bd2, od2 = DevBuf(data=xin), DevBuf(data=w2), DevBuf(data=b2), DevBuf(want2.size).fill(0xEE)
    assert fn(xd2.ptr, 3 if bits == 8 else 4, Shape5(1, Co, nz, W, W), wd2.ptr, bd2.ptr, 16, od2.ptr, 3 if bits == 8 else 4, Gnp(), None, 0, Split()) == 0
    ufsm_b200.check()
    got2 = od2.download()
    assert got2.size == want2.size and np.count_nonzero(got2 != want2) < 2e-3 * got2.size
    assert orc.rel_l2(orc.mx_to_pm(got2, bits, 1, 16, S), orc.mx_to_pm(want2, bits, 1, 16, S)) < (5e-3 if bits == 8 else 2e-2)


def _full_conv(L, xbf, x_store, N, Ci, D, H, W, w, b, Co, ybf, gp=None):
    """the whole-tensor conv through the same entry (itself checked against the oracle elsewhere in this suite): what a slab run must reproduce"""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    S = D * H * W
    nby = N * Co * S * 2 if ybf == 2 else orc.mx_bytes(8 if ybf == 3 else 4, N, Co, S, 32)
    xd, wd, bd, yd = DevBuf(data=x_store), DevBuf(data=w), DevBuf(data=b), DevBuf(nby).fill(0xEE)
    assert L.lp_conv_fwd_f8(xd.ptr, xbf, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, ybf, gp if gp is not None else Gnp(), None, 0, Split()) == 0
    ufsm_b200.check()
    return yd.download()


@pytest.mark.parametrize("xbf,ybf,gn", [(3, 2, False), (2, 2, False), (3, 3, False), (3, 2, True), (3, 2, "slabs")])
def test_z_range_window_and_slab_output(dev, xbf, ybf, gn):
    """split_t.zi0 / Di (a conv over planes of a deeper input), zw0 / zw1 (a window of output planes), yD / yzo (the output placed in a deeper
    tensor): each run must give the planes of the whole-tensor conv, with zero padding only at the tensor's own ends."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Ci, Co, D, H, W = 2, 32, 32, 12, 8, 16
    S, hw = D * H * W, H * W
    x = (synth.rng(231).standard_normal(N * Ci * S) * 2).astype(f32)
    w, b = synth.kaiming(232, Co, Ci, 27), synth.bias(233, Co, 0.1)
    xs = x.astype(np.float16) if xbf == 2 else orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
    keep = []
    gp = Gnp()
    if gn == "slabs":                        # statistics per (sample, z slab): planes 0-2, 3-7, 8-11 (gnp_t.ns / zs / zo / zhw, src/nn_lp.h:15-18)
        gp = make_gp(8, gn_params(234, N * 3, Ci, 8), keep)
        gp.ns, gp.zs, gp.zo, gp.zhw = 3, 5, 2, hw
    elif gn:
        gp = make_gp(8, gn_params(234, N, Ci, 8), keep)
    full = _full_conv(L, xbf, xs, N, Ci, D, H, W, w, b, Co, ybf, gp)
    xd, wd, bd = DevBuf(data=xs), DevBuf(data=w), DevBuf(data=b)

    def planes(buf, z0, z1):                 # planes [z0, z1) of a stored output tensor as a flat array (codes and scale rows for MX)
        if ybf == 2:
            return buf.view(np.float16).reshape(N * Co, D, hw)[:, z0:z1].copy()
        rows = N * (Co // 32)
        return np.concatenate([buf[:rows * S * 32].reshape(rows, D, hw * 32)[:, z0:z1].ravel(), buf[rows * S * 32:].reshape(rows, D, hw)[:, z0:z1].ravel()])

    def same(a, c):
        if ybf == 2:
            return orc.rel_l2(a.astype(f32), c.astype(f32)) < 1e-5
        return np.count_nonzero(a != c) < 1e-3 * a.size
    # a window of output planes: the rest of y stays as it was
    for z0, z1 in ((0, 4), (4, 8), (8, 12)):
        yd = DevBuf(full.size).fill(0xEE)
        sp = Split(); sp.zw0, sp.zw1 = z0, z1
        assert L.lp_conv_fwd_f8(xd.ptr, xbf, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, ybf, gp, None, 0, sp) == 0
        ufsm_b200.check()
        got = yd.download()
        assert same(planes(got, z0, z1), planes(full, z0, z1)), (z0, z1)
        rest = np.ones(D, bool); rest[z0:z1] = False
        other = got.view(np.float16).reshape(N * Co, D, hw)[:, rest].view(np.uint8) if ybf == 2 else got[:N * (Co // 32) * S * 32].reshape(-1, D, hw * 32)[:, rest]
        assert (other == 0xEE).all()
    # a z range of a deeper input, written as a tensor of its own depth, and (MX or fp16 alike) straight into the deep output tensor
    for zi0, nz in ((0, 4), (4, 4), (8, 4), (2, 7)):
        sp = Split(); sp.zi0, sp.Di = zi0, D
        nby = N * Co * nz * hw * 2 if ybf == 2 else orc.mx_bytes(8, N, Co, nz * hw, 32)
        yd = DevBuf(nby).fill(0xEE)
        assert L.lp_conv_fwd_f8(xd.ptr, xbf, Shape5(N, Ci, nz, H, W), wd.ptr, bd.ptr, Co, yd.ptr, ybf, gp, None, 0, sp) == 0
        sp.yD, sp.yzo = D, zi0
        yd2 = DevBuf(full.size).fill(0xEE)
        assert L.lp_conv_fwd_f8(xd.ptr, xbf, Shape5(N, Ci, nz, H, W), wd.ptr, bd.ptr, Co, yd2.ptr, ybf, gp, None, 0, sp) == 0
        ufsm_b200.check()
        want = planes(full, zi0, zi0 + nz)
        got = yd.download()
        got = got.view(np.float16).reshape(N * Co, nz, hw) if ybf == 2 else got
        assert same(got.ravel() if ybf == 2 else got, want.ravel() if ybf == 2 else want), (zi0, nz)
        assert same(planes(yd2.download(), zi0, zi0 + nz), want), (zi0, nz)


def test_z_window_with_split_output_and_statistics(dev):
    """A z window and a z range together with a split MX output and the GroupNorm sums of the stored output: the two output tensors hold the
    window's planes of the whole-tensor conv's, and the sums are those of exactly these planes (less zlo / zhi of them)."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Ci, Ox, O2, D, H, W, Go = 2, 32, 32, 32, 10, 8, 16, 8
    Co, S, hw = Ox + O2, D * H * W, H * W
    x = (synth.rng(251).standard_normal(N * Ci * S) * 2).astype(f32)
    w, b = synth.kaiming(252, Co, Ci, 27), synth.bias(253, Co, 0.1)
    xs = orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
    full = _full_conv(L, 3, xs, N, Ci, D, H, W, w, b, Co, 3)
    stored = orc.mx_to_pm(full, 8, N, Co, S, 32).reshape(N, Co, D, hw)
    xd, wd, bd = DevBuf(data=xs), DevBuf(data=w), DevBuf(data=b)

    def check(sp, shape_d, z0, z1, zlo, zhi, deep):
        nz = z1 - z0
        Dy = D if deep else nz
        yd, y2d = DevBuf(orc.mx_bytes(8, N, Ox, Dy * hw, 32)).fill(0xEE), DevBuf(orc.mx_bytes(8, N, O2, Dy * hw, 32)).fill(0xEE)
        sums = DevBuf(N * Go * 2 * 24).fill(0)
        sp.y2, sp.o_split, sp.stored_stats, sp.zlo, sp.zhi = y2d.ptr, Ox, 1, zlo, zhi
        assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, shape_d, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 3, Gnp(), sums.ptr, Go, sp) == 0
        ufsm_b200.check()
        for buf, c0, c in ((yd, 0, Ox), (y2d, Ox, O2)):
            got = orc.mx_to_pm(buf.download(), 8, N, c, Dy * hw, 32).reshape(N, c, Dy, hw)
            got = got[:, :, z0:z1] if deep else got
            assert np.array_equal(got, stored[:, c0:c0 + c, z0:z1]), (z0, z1, c0)
        ws = sums.download().view(np.uint64).reshape(-1, 3)
        got = ws[:, 1].astype(np.int64).astype(np.float64) + ws[:, 0].astype(np.float64) * 2.0 ** -64
        part = stored[:, :, z0 + zlo:z1 - zhi].astype(np.float64).reshape(N, Go, Co // Go, -1)
        exp = np.stack([part.sum((2, 3)), (part * part).sum((2, 3))], 2).reshape(-1)
        assert (ws[:, 2] == 0).all() and np.allclose(got, exp, rtol=1e-13, atol=1e-9)

    sp = Split(); sp.zw0, sp.zw1 = 3, 8                     # a window of the output planes, written into the whole-depth tensors
    check(sp, D, 3, 8, 1, 0, True)
    sp = Split(); sp.zi0, sp.Di = 4, D                      # a z range of the deeper input, outputs of the range's own depth
    check(sp, 5, 4, 9, 0, 2, False)


def test_accumulate(dev):
    """split_t.accum: y += conv (fp16 plane-major), also on a window of planes"""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    L = ufsm_b200.lib()
    N, Ci, Co, D, H, W = 1, 32, 32, 8, 8, 16
    S = D * H * W
    x = (synth.rng(241).standard_normal(N * Ci * S) * 2).astype(f32)
    w, b = synth.kaiming(242, Co, Ci, 27), synth.bias(243, Co, 0.1)
    xs = orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
    full = _full_conv(L, 3, xs, N, Ci, D, H, W, w, b, Co, 2).view(np.float16).astype(f32)
    y0 = synth.rng(244).standard_normal(N * Co * S).astype(np.float16)
    xd, wd, bd = DevBuf(data=xs), DevBuf(data=w), DevBuf(data=b)
    for zw in (None, (2, 6)):
        yd = DevBuf(data=y0)
        sp = Split(); sp.accum = 1
        add = full.reshape(N * Co, D, -1).copy()
        if zw:
            sp.zw0, sp.zw1 = zw
            add[:, :zw[0]] = 0; add[:, zw[1]:] = 0
        assert L.lp_conv_fwd_f8(xd.ptr, 3, Shape5(N, Ci, D, H, W), wd.ptr, bd.ptr, Co, yd.ptr, 2, Gnp(), None, 0, sp) == 0
        ufsm_b200.check()
        want = (y0.astype(f32) + add.ravel()).astype(np.float16)
        assert np.array_equal(yd.download(np.float16), want)
