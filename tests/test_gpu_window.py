"""Sliding-window scheduler on the GPU.  One rank: umx_window_run_fx's finished volume against the oracle's exact blend of the library's own
per-patch logits (orc.blend_add_fx / orc.emit_fx: the weight arithmetic of k_i3_blend and the emit of k_i3_emit, src/nn_ink3dext.cu:48-100,
with the sums taken as 64-bit integers) bit for bit.  Several ranks (each rank's share run in turn on the one device, the rows they
share handed over with umx_wplan_pack / umx_wplan_add): the assembled volume is the single-rank volume byte for byte, whatever the number of
ranks and the batch size (the reference's multi-GPU contract, tests/test_predict_gpus2.sh)."""
import ctypes as C

import numpy as np
import pytest

import gpu_util as G
import orc
import synth
import ufsm_b200
from ufsm_b200 import DevBuf

pytestmark = pytest.mark.gpu

V, P, OV, CW, NH = 72, 32, 8, [32, 64], 7
F16, U8 = 2, 100


def run_ranks(L, u, vol, world, batch, fmt):
    """every rank's share in turn, then the hand-over of shared rows, then the assembly of the rows each rank owns"""
    w = L.umx_window_make(V, P, OV)
    el = 2 if fmt == F16 else 1
    plans, outs, exts = [], [], []
    for r in range(world):
        p = L.umx_wplan_create(C.byref(w), r, world, NH)
        f, c, lo, hi = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        L.umx_wplan_info(p, C.byref(f), C.byref(c), C.byref(lo), C.byref(hi))
        n = NH * (hi.value - lo.value) * V * V * el
        host = L.nn_malloc_host(n)
        C.memset(host, 0xEE, n)
        assert L.umx_window_run_fx(u.h, p, vol.ctypes.data, batch, fmt, host) == 0, (L.lp_check() or b"").decode()
        plans.append(p); outs.append(host); exts.append((lo.value, hi.value))
    for a in range(world):
        for b in range(a):
            n = L.umx_wplan_rows(plans[a], b, 0, None)
            assert n == L.umx_wplan_rows(plans[b], a, 1, None)
            if n:
                buf = DevBuf(n * L.umx_wplan_row_bytes(plans[a]))
                assert L.umx_wplan_pack(plans[a], b, buf.ptr) == 0 and L.umx_wplan_add(plans[b], a, buf.ptr) == 0
    full = np.zeros((NH, V, V, V), np.uint16 if fmt == F16 else np.uint8)
    cover = np.zeros((V, V), np.int32)
    for r in range(world):
        assert L.umx_wplan_finish(plans[r], outs[r]) == 0, (L.lp_check() or b"").decode()
        lo, hi = exts[r]
        out = np.ctypeslib.as_array((C.c_uint8 * (NH * (hi - lo) * V * V * el)).from_address(outs[r])).view(full.dtype).reshape(NH, hi - lo, V, V)
        mode = np.zeros((hi - lo, V), np.uint8)
        L.umx_wplan_mode(plans[r], mode.ctypes.data)
        mine = (mode == 1) | (mode == 2)
        full[:, lo:hi][:, mine, :] = out[:, mine, :]
        cover[lo:hi][mine] += 1
        L.umx_wplan_free(plans[r])
        L.nn_free_host(outs[r])
    ufsm_b200.check()
    assert np.all(cover == 1)
    return full


def test_window_single_rank_against_the_oracle_and_rank_invariance(dev):
    L = G.L()
    u = G.Unet(G.make_cfg(P, CW, NH, (8, 8, 8)), synth.unet_weights(7, CW, NH), 2)
    vol = synth.ct_u8(71, V ** 3).reshape(V, V, V)
    w = L.umx_window_make(V, P, OV)
    assert w.nper == 3 and w.npatch == 27                   # origins 0, 24, 40 (the last patch pulled back to the edge)
    one = run_ranks(L, u, vol, 1, 2, F16)
    # the oracle's blend of the library's per-patch logits
    acc, ws = np.zeros((NH, V ** 3), np.int64), np.zeros(V ** 3, np.int64)
    w1 = orc.gauss_window(P)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    for i in range(w.npatch):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        z0, y0, x0 = z.value, y.value, x.value
        x16 = (vol[z0:z0 + P, y0:y0 + P, x0:x0 + P].astype(np.float32) / np.float32(255)).astype(np.float16)
        orc.blend_add_fx(u.forward(x16.ravel(), 1), NH, P, V, z0, y0, x0, w1, acc, ws)
    assert (ws > 0).all()
    want = orc.emit_fx(acc, ws, NH, F16).view(np.uint16).reshape(NH, V, V, V)
    assert np.array_equal(one, want), "%d of %d differ" % (np.count_nonzero(one != want), want.size)
    # the ideal blend in float64 is within fp16 rounding of it
    ideal = (acc.astype(np.float64) / ws.astype(np.float64)[None]).reshape(NH, V, V, V)
    got = one.view(np.float16).astype(np.float64)
    assert np.abs(got - ideal).max() <= 6e-4 * max(1.0, np.abs(ideal).max())
    # any number of ranks, any batch: the same bytes
    for world, batch in ((2, 1), (3, 2), (5, 2)):
        assert np.array_equal(run_ranks(L, u, vol, world, batch, F16), one), (world, batch)
    # uint8 output (round(254 sigmoid)): the device's expf against the host's may move a value on a rounding boundary by one
    u8 = run_ranks(L, u, vol, 2, 2, U8)
    want8 = orc.emit_fx(acc, ws, NH, U8).reshape(NH, V, V, V)
    d = np.abs(u8.astype(np.int32) - want8.astype(np.int32))
    assert d.max() <= 1 and np.mean(d != 0) < 1e-3
    assert np.array_equal(run_ranks(L, u, vol, 1, 1, U8), u8)
    u.free()


def test_reference_blend_operator(dev):
    """umx_blend_add, the reference's own arithmetic (fp32 fma per patch in call order, k_i3_blend): two overlapping patches against numpy"""
    L = G.L()
    Vb, Pb, nh = 24, 16, 2
    g = synth.rng(5)
    lg = [g.standard_normal((nh, Pb, Pb, Pb)).astype(np.float32) for _ in range(2)]
    org = [(0, 0, 0), (8, 4, 8)]
    w1 = orc.gauss_window(Pb)
    w3 = ((w1[:, None, None] * w1[None, :, None]).astype(np.float32) * w1[None, None, :]).astype(np.float32)
    acc, ws = DevBuf(nh * Vb ** 3 * 4).zero(), DevBuf(Vb ** 3 * 4).zero()
    w1d = DevBuf(data=w1)
    want, wsum = np.zeros((nh, Vb, Vb, Vb), np.float32), np.zeros((Vb, Vb, Vb), np.float32)
    for l, (z0, y0, x0) in zip(lg, org):
        ld = DevBuf(data=l)
        L.umx_blend_add(ld.ptr, 0, nh, Pb, Vb, 0, Vb, z0, y0, x0, w1d.ptr, acc.ptr, ws.ptr)
        sl = (slice(None), slice(z0, z0 + Pb), slice(y0, y0 + Pb), slice(x0, x0 + Pb))
        want[sl] = (w3.astype(np.float64)[None] * l.astype(np.float64) + want[sl].astype(np.float64)).astype(np.float32)      # one fused multiply-add
        wsum[sl[1:]] += w3
    ufsm_b200.check()
    assert np.array_equal(acc.download(np.float32).reshape(want.shape), want) and np.array_equal(ws.download(np.float32).reshape(wsum.shape), wsum)
