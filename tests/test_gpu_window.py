"""Sliding-window scheduler on the GPU: umx_window_run's blended planes against a numpy blend of the library's own per-patch logits
(the arithmetic of k_i3_blend, src/nn_ink3dext.cu:58-73: acc += w * logit with the separable Gaussian window, in patch order), and the
shards of two ranks against the single-rank run (src/predict.c:2696-2717: contiguous z-slabs of patch rows, the host adds the planes two
ranks share)."""
import ctypes as C

import numpy as np
import pytest

import gpu_util as G
import synth
import ufsm_b200

pytestmark = pytest.mark.gpu

V, P, OV, CW, NH = 72, 32, 8, [32, 64], 7


def run_share(L, u, w, vol, first, count, batch=2):
    lo, hi = C.c_int(), C.c_int()
    L.umx_window_extent(C.byref(w), first, count, C.byref(lo), C.byref(hi))
    zext = hi.value - lo.value
    acc = np.full(NH * zext * V * V, np.nan, np.float32)
    ws = np.full(zext * V * V, np.nan, np.float32)
    rc = L.umx_window_run(u.h, C.byref(w), vol.ctypes.data, first, count, batch, acc.ctypes.data, ws.ctypes.data)
    assert rc == 0, (L.lp_check() or b"").decode()
    return lo.value, hi.value, acc.reshape(NH, zext, V, V), ws.reshape(zext, V, V)


def test_window_blend_and_two_rank_shards(dev):
    L = G.L()
    cfg = G.make_cfg(P, CW, NH, (8, 8, 8))
    u = G.Unet(cfg, synth.unet_weights(7, CW, NH), 2)
    vol = synth.ct_u8(71, V ** 3).reshape(V, V, V)
    w = L.umx_window_make(V, P, OV)
    assert w.nper == 3 and w.npatch == 27                   # origins 0, 24, 40 (the last patch pulled back to the edge)
    lo, hi, acc, ws = run_share(L, u, w, vol, 0, w.npatch)
    assert (lo, hi) == (0, V) and np.isfinite(acc).all() and (ws > 0).all()
    # numpy restatement of the blend from the library's per-patch logits (host entry, fp16 -> the device path's fp32 logits differ by the
    # fp16 rounding only, so compare through the fp32 device entry)
    sg, c = P / 8.0, float(P // 2)
    w1 = np.exp(-0.5 * ((np.arange(P) - c) / sg) ** 2).astype(np.float32)
    w3 = ((w1[:, None, None] * w1[None, :, None]).astype(np.float32) * w1[None, None, :]).astype(np.float32)
    want = np.zeros((NH, V, V, V), np.float32)
    wsum = np.zeros((V, V, V), np.float32)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    for i in range(w.npatch):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        z0, y0, x0 = z.value, y.value, x.value
        patch = vol[z0:z0 + P, y0:y0 + P, x0:x0 + P]
        x16 = (patch.astype(np.float32) / np.float32(255)).astype(np.float16)
        lg = u.forward(x16.ravel(), 1).reshape(NH, P, P, P)
        # one fused multiply-add per voxel and channel, as the kernel does: float64 product + sum rounded once to fp32
        sl = (slice(None), slice(z0, z0 + P), slice(y0, y0 + P), slice(x0, x0 + P))
        want[sl] = (w3.astype(np.float64)[None] * lg.astype(np.float64) + want[sl].astype(np.float64)).astype(np.float32)
        wsum[sl[1:]] += w3
    assert np.array_equal(ws, wsum)
    assert np.array_equal(acc, want), "max diff %g" % np.abs(acc - want).max()
    # two ranks: each runs its contiguous share; the planes both touch are added on the host
    tot = np.zeros_like(acc)
    tws = np.zeros_like(ws)
    seen = 0
    for r in range(2):
        f, cnt = C.c_int(), C.c_int()
        L.umx_window_share(C.byref(w), r, 2, C.byref(f), C.byref(cnt))
        assert f.value == seen
        seen += cnt.value
        lo_r, hi_r, a_r, w_r = run_share(L, u, w, vol, f.value, cnt.value, batch=1)
        tot[:, lo_r:hi_r] += a_r
        tws[lo_r:hi_r] += w_r
    assert seen == w.npatch
    assert np.allclose(tws, ws, rtol=1e-6, atol=0) and np.allclose(tot, acc, rtol=1e-5, atol=1e-6)
    out1, out2 = acc / ws[None], tot / tws[None]
    assert np.abs(out1 - out2).max() <= 1e-5 * max(1.0, np.abs(out1).max())
    u.free()
