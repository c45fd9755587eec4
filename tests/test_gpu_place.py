"""GPU parity of the predict back end (nn_pred_place and its variants, src/nn.h:871-885 of the reference) against the oracle's
restatement: halo crop, clipping to the shard, the material test (CT threshold or mask bits), fp32 and fp16 logits, and the byte
trunc(255 sigmoid + 0.5).  Voxels outside the placed box must stay untouched, the placed box and the zeros of non-material voxels
exact; the byte itself may differ by one where 255 sigmoid + 0.5 lands within rounding of an integer (the GPU's exp and division are
the hardware approximations, as in the reference's kernel): at most one voxel in a thousand."""
import numpy as np
import pytest

import orc
import synth

pytestmark = pytest.mark.gpu


def close_bytes(got, want):
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    if not d.size:
        return
    assert d.max() <= 1, d.max()
    assert (d != 0).mean() < 1e-3, (d != 0).mean()


def make(seed, D, W, h16):
    g = synth.rng(seed)
    lg = (g.standard_normal(D * W * W) * 3).astype(np.float32)
    lg[::53] = 40.0
    lg[7::61] = -40.0
    lg[11::97] = -120.0                     # exp overflows: probability 0
    if h16:
        lg = lg.astype(np.float16)
    ct = synth.ct_u8(seed + 1, D * W * W)
    ct[::5] = 0
    return lg, ct


CASES = [
    # D, W, hz, halo, (oz, oy, ox), (ez, ey, ex), shard, iso, h16
    (32, 32, 4, 4, (0, 0, 0), (40, 40, 40), 40, 1, False),          # the whole interior
    (32, 32, 4, 4, (-6, 20, -9), (40, 30, 40), 40, 1, False),       # clipped at the low end in z and x, at the extent in y
    (20, 32, 2, 6, (15, 3, 11), (30, 40, 37), 48, 90, True),        # D != W, own z halo, a CT threshold, fp16 logits, odd row starts
    (16, 24, 4, 4, (40, 0, 0), (32, 32, 32), 48, 1, False),         # entirely outside: nothing written
]


@pytest.mark.parametrize("D,W,hz,halo,o,e,shard,iso,h16", CASES)
def test_pred_place(dev, D, W, hz, halo, o, e, shard, iso, h16):
    import ufsm_b200
    from ufsm_b200 import DevBuf
    L = ufsm_b200.lib()
    lg, ct = make(301, D, W, h16)
    lgd, ctd = DevBuf(data=lg), DevBuf(data=ct)
    L.nn_set_logits_h16(1 if h16 else 0)
    L.nn_set_pred_iso(iso)
    assert L.nn_get_pred_iso() == iso
    try:
        dsh = DevBuf(shard ** 3).fill(0xEE)
        L.nn_pred_place_d(lgd.ptr, ctd.ptr, D, W, hz, halo, *o, *e, shard, dsh.ptr)
        ufsm_b200.check()
        want = orc.pred_place(lg.astype(np.float32), ct >= iso, D, W, hz, halo, *o, *e, shard, np.full(shard ** 3, 0xEE, np.uint8))
        got = dsh.download()
        box = want == orc.pred_place(lg.astype(np.float32), ct >= iso, D, W, hz, halo, *o, *e, shard, np.full(shard ** 3, 0x11, np.uint8))     # where nothing is placed the prefill shows
        assert np.array_equal(got[~box], want[~box])
        close_bytes(got[box], want[box])
        # the same through the mask bits
        bits = DevBuf(((D * W * W + 31) // 32) * 4).fill(0)
        L.nn_pred_ctmask_t(ctd.ptr, D * W * W, bits.ptr, iso)
        ufsm_b200.check()
        assert np.array_equal(bits.download(np.uint32), orc.ctmask(ct, iso))
        dsh2 = DevBuf(shard ** 3).fill(0xEE)
        L.nn_pred_place_m_d(lgd.ptr, bits.ptr, D, W, hz, halo, *o, *e, shard, dsh2.ptr)
        ufsm_b200.check()
        assert np.array_equal(dsh2.download(), got)
        if D == W and hz == halo:
            dsh3 = DevBuf(shard ** 3).fill(0xEE)
            if iso == 1:
                L.nn_pred_place(lgd.ptr, ctd.ptr, W, halo, *o, *e, shard, dsh3.ptr)
            else:
                L.nn_pred_place_m(lgd.ptr, bits.ptr, W, halo, *o, *e, shard, dsh3.ptr)
            ufsm_b200.check()
            assert np.array_equal(dsh3.download(), got)
    finally:
        L.nn_set_logits_h16(0)
        L.nn_set_pred_iso(1)


def test_pred_place_split_window_and_output(dev):
    """nn_pred_place_mz: the two halves of a window split in z (each held from its own first plane, with the bits of its own planes) place
    what the whole window places; nn_pred_output: every voxel, material where CT != 0; nn_pred_ctmask on a length that is not a
    multiple of 32 and on an unaligned pointer."""
    import ufsm_b200
    from ufsm_b200 import DevBuf
    L = ufsm_b200.lib()
    W, halo, shard = 32, 4, 40
    o, e = (3, -2, 5), (40, 40, 33)
    lg, ct = make(311, W, W, False)
    lgd, ctd = DevBuf(data=lg), DevBuf(data=ct)
    whole = DevBuf(shard ** 3).fill(0xEE)
    L.nn_pred_place(lgd.ptr, ctd.ptr, W, halo, *o, *e, shard, whole.ptr)
    halves = DevBuf(shard ** 3).fill(0xEE)
    zc = 18
    for zoff, zlo, zhi in ((0, 0, zc), (zc - 2, zc, W)):            # the upper half is held from plane zc - 2 on
        part_lg, part_ct = lg[zoff * W * W:], ct[zoff * W * W:]
        pl, pb = DevBuf(data=part_lg), DevBuf(((part_ct.size + 31) // 32) * 4).fill(0)
        pc = DevBuf(data=part_ct)
        L.nn_pred_ctmask(pc.ptr, part_ct.size, pb.ptr)
        L.nn_pred_place_mz(pl.ptr, pb.ptr, W, halo, zlo, zhi, zoff, *o, *e, shard, halves.ptr)
    ufsm_b200.check()
    assert np.array_equal(halves.download(), whole.download())
    want = orc.pred_place(lg, ct >= 1, W, W, halo, halo, *o, *e, shard, np.full(shard ** 3, 0xEE, np.uint8))
    box = want == orc.pred_place(lg, ct >= 1, W, W, halo, halo, *o, *e, shard, np.full(shard ** 3, 0x11, np.uint8))
    assert np.array_equal(whole.download()[~box], want[~box])
    close_bytes(whole.download()[box], want[box])
    # nn_pred_output
    n = 5003
    out = DevBuf(n).fill(0xEE)
    L.nn_pred_output(lgd.ptr, ctd.ptr, n, out.ptr)
    ufsm_b200.check()
    close_bytes(out.download(), np.where(ct[:n] != 0, orc.prob255(lg[:n]), 0).astype(np.uint8))
    # mask of an odd length from an odd address
    big = DevBuf(data=np.concatenate([np.zeros(3, np.uint8), ct[:n]]))
    mb = DevBuf(((n + 31) // 32) * 4).fill(0xEE)
    L.nn_pred_ctmask_t(big.ptr + 3, n, mb.ptr, 100)
    ufsm_b200.check()
    assert np.array_equal(mb.download(np.uint32), orc.ctmask(ct[:n], 100))


@pytest.mark.parametrize("present,oo,on", [((1, 2, 3, 4, 5, 6, 7), (0, 0, 0), (12, 12, 12)), ((4, 1), (0, 3, 0), (7, 9, 12)), ((), (5, 0, 2), (6, 12, 10)), ((2, 6, 7), (0, 0, 0), (4, 12, 5))])
def test_feather_blend_and_keep(dev, present, oo, on):
    """The seam feather on the device (src/predict.c:282-376): the blended interior bytes equal the restatement's (fp32 in the same order: exact),
    for every subset of neighbours tried and for partial output boxes; the kept slabs are the window's upper slabs."""
    import ctypes as C
    import ufsm_b200
    from ufsm_b200 import DevBuf, Feather
    L = ufsm_b200.lib()
    S, B, osh = 12, 4, 13
    E = S + B
    g = synth.rng(321)
    e = g.integers(0, 256, E ** 3, dtype=np.uint8)
    sizes = {d: (B * E * E if d & 4 else S * B * E if d & 2 else S * S * B) for d in range(1, 8)}
    nb = [None] * 8
    for d in present:
        nb[d] = g.integers(0, 256, sizes[d], dtype=np.uint8)
    want = orc.feather_blend(e, nb, S, B, oo, on, osh, np.full(osh ** 3, 0xEE, np.uint8))
    ed, od = DevBuf(data=e), DevBuf(osh ** 3).fill(0xEE)
    bufs = {d: DevBuf(data=nb[d]) for d in present}
    f = Feather()
    f.S, f.B, f.e, f.osh, f.out = S, B, ed.ptr, osh, od.ptr
    for d in range(8):
        f.nb[d] = bufs[d].ptr if d in bufs else None
    for k in range(3):
        f.oo[k], f.on[k] = oo[k], on[k]
    assert L.umx_feather_blend(C.byref(f)) == 0
    ufsm_b200.check()
    assert np.array_equal(od.download(), want)
    # what is kept of a window for those after it
    zs, ys, xs = DevBuf(B * E * E).fill(0), DevBuf(S * B * E).fill(0), DevBuf(S * S * B).fill(0)
    L.umx_feather_keep(ed.ptr, S, B, zs.ptr, ys.ptr, xs.ptr)
    ufsm_b200.check()
    e3 = e.reshape(E, E, E)
    assert np.array_equal(zs.download(), e3[S:].ravel())
    assert np.array_equal(ys.download(), e3[:S, S:, :].ravel())
    assert np.array_equal(xs.download(), e3[:S, :S, S:].ravel())
