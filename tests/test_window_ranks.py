"""The multi-rank path of the window scheduler on CPU.  The library's plan (umx_wplan_*: host-only code) deals the (z, y) patch rows to
ranks in contiguous z-slab-first shares (src/predict.c:2696-2717), decides which rank owns each row (z, y) of the volume and lists
the rows whose partial sums go from one rank to another.  Here gloo ranks follow their plans with the oracle's exact (64-bit
fixed-point) blend of synthetic per-patch logits, exchange exactly the listed rows, and assemble the volume; it must be the single-rank
volume byte for byte (the reference's multi-GPU contract, tests/test_predict_gpus2.sh).  No GPU, no compute entry of the library."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
V, P, OV, NH = 40, 16, 4, 2


def _fake_logits(i):
    r = np.random.default_rng(1000 + i)
    return (r.standard_normal((NH, P, P, P)) * 3).astype(np.float32)


def _plan(L, rank, world):
    w = L.umx_window_make(V, P, OV)
    p = L.umx_wplan_create(C.byref(w), rank, world, NH)
    f, c, lo, hi = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    L.umx_wplan_info(p, C.byref(f), C.byref(c), C.byref(lo), C.byref(hi))
    return w, p, f.value, c.value, lo.value, hi.value


def _rows(L, p, peer, d):
    n = L.umx_wplan_rows(p, peer, d, None)
    zy = np.zeros((max(n, 1), 2), np.int32)
    L.umx_wplan_rows(p, peer, d, zy.ctypes.data)
    return zy[:n]


def _blend_share(L, orc, w, first, count):
    """this rank's patches into full-volume integer accumulators (only the rows the plan names are ever read)"""
    acc, ws = np.zeros((NH, V, V, V), np.int64), np.zeros((V, V, V), np.int64)
    w1 = orc.gauss_window(P)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    for i in range(first, first + count):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        orc.blend_add_fx(_fake_logits(i), NH, P, V, z.value, y.value, x.value, w1, acc, ws)
    return acc, ws


def _rank(rank, world, port, q):
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))
    import torch
    import torch.distributed as dist
    import orc
    import ufsm_b200
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = ufsm_b200.lib()
    w, p, first, count, lo, hi = _plan(L, rank, world)
    acc, ws = _blend_share(L, orc, w, first, count)
    # hand the rows that lower ranks own to them, receive those of higher ranks (exactly the plan's lists, in their order)
    reqs, sendbufs = [], []
    for peer in range(world):
        zy = _rows(L, p, peer, 0)
        if len(zy):
            buf = np.concatenate([acc[:, zy[:, 0], zy[:, 1], :].transpose(1, 0, 2), ws[zy[:, 0], zy[:, 1], :][:, None, :]], 1)       # [row][nh + 1][V]
            t = torch.from_numpy(np.ascontiguousarray(buf))
            sendbufs.append(t)
            reqs.append(dist.isend(t, peer))
    for peer in range(world):
        zy = _rows(L, p, peer, 1)
        if len(zy):
            t = torch.zeros(len(zy), NH + 1, V, dtype=torch.int64)
            dist.recv(t, peer)
            b = t.numpy()
            for r, (zz, yy) in enumerate(zy):
                acc[:, zz, yy, :] += b[r, :NH]
                ws[zz, yy, :] += b[r, NH]
    for r in reqs:
        r.wait()
    # this rank's rows of the finished volume: the ones it owns (its plan's modes are not exposed: owned = touched and not sent away)
    out = orc.emit_fx(acc.reshape(NH, -1), ws.ravel(), NH, 2).reshape(NH, V, V, V)
    mine = np.zeros((V, V), bool)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    for i in range(first, first + count, w.nper):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        mine[z.value:z.value + P, y.value:y.value + P] = True
    for peer in range(world):
        zy = _rows(L, p, peer, 0)
        mine[zy[:, 0], zy[:, 1]] = False
    full = torch.zeros(NH, V, V, V, dtype=torch.int32)
    cover = torch.zeros(V, V, dtype=torch.int32)
    full.numpy()[:, mine, :] = out.view(np.uint16)[:, mine, :]
    cover.numpy()[mine] = 1
    dist.reduce(full, 0)
    dist.reduce(cover, 0)
    if rank == 0:
        q.put((full.numpy().astype(np.uint16), cover.numpy()))
    dist.barrier()
    L.umx_wplan_free(p)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ranks_assemble_the_single_rank_volume(world):
    sys.path.insert(0, os.path.dirname(HERE))
    import orc
    import ufsm_b200
    L = ufsm_b200.lib()
    w, p, first, count, lo, hi = _plan(L, 0, 1)
    assert (first, count, lo, hi) == (0, w.npatch, 0, V) and all(L.umx_wplan_rows(p, r, d, None) == 0 for r in range(4) for d in (0, 1))
    L.umx_wplan_free(p)
    acc, ws = _blend_share(L, orc, w, 0, w.npatch)
    want = orc.emit_fx(acc.reshape(NH, -1), ws.ravel(), NH, 2).view(np.uint16).reshape(NH, V, V, V)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    got, cover = q.get(timeout=180)
    for pr in procs:
        pr.join(60)
        assert pr.exitcode == 0
    assert np.all(cover == 1), "every row of the volume has exactly one owner"
    assert np.array_equal(got, want)


def test_plan_lists_are_consistent():
    """what rank a hands to rank b is what b expects from a, row for row; only higher ranks hand over to lower ones"""
    sys.path.insert(0, os.path.dirname(HERE))
    import ufsm_b200
    L = ufsm_b200.lib()
    for world in (2, 3, 5, 8):
        plans = [_plan(L, r, world) for r in range(world)]
        total = 0
        for a in range(world):
            for b in range(world):
                s, r = _rows(L, plans[a][1], b, 0), _rows(L, plans[b][1], a, 1)
                assert np.array_equal(s, r), (world, a, b)
                assert len(s) == 0 or b < a
                total += len(s)
        assert total > 0
        first = 0
        for r in range(world):
            assert plans[r][2] == first
            first += plans[r][3]
        assert first == plans[0][0].npatch
        for pl in plans:
            L.umx_wplan_free(pl[1])
