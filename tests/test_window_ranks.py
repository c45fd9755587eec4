"""The multi-rank path of the window scheduler on CPU: two gloo ranks take their shares from umx_window_share (host-only code of the
library; the reference deals contiguous z-slabs of patch rows, src/predict.c:2696-2717), blend synthetic per-patch logits with the
oracle-side numpy blend, and rank 0 gathers the slabs and adds the planes both touch; the result must equal the single-process blend.
No GPU and no compute entry of the library is used."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
V, P, OV, NH = 40, 16, 4, 2


def _fake_logits(i):
    r = np.random.default_rng(1000 + i)
    return r.standard_normal((NH, P, P, P)).astype(np.float32)


def _blend(L, w, first, count):
    lo, hi = C.c_int(), C.c_int()
    L.umx_window_extent(C.byref(w), first, count, C.byref(lo), C.byref(hi))
    zext = hi.value - lo.value
    acc, ws = np.zeros((NH, zext, V, V), np.float32), np.zeros((zext, V, V), np.float32)
    sg, c = P / 8.0, float(P // 2)
    w1 = np.exp(-0.5 * ((np.arange(P) - c) / sg) ** 2).astype(np.float32)
    w3 = ((w1[:, None, None] * w1[None, :, None]).astype(np.float32) * w1[None, None, :]).astype(np.float32)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    for i in range(first, first + count):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        z0, y0, x0 = z.value - lo.value, y.value, x.value
        acc[:, z0:z0 + P, y0:y0 + P, x0:x0 + P] += w3[None] * _fake_logits(i)
        ws[z0:z0 + P, y0:y0 + P, x0:x0 + P] += w3
    return lo.value, hi.value, acc, ws


def _rank(rank, world, port, q):
    sys.path.insert(0, os.path.dirname(HERE))
    import torch
    import torch.distributed as dist
    import ufsm_b200
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = ufsm_b200.lib()
    w = L.umx_window_make(V, P, OV)
    f, cnt = C.c_int(), C.c_int()
    L.umx_window_share(C.byref(w), rank, world, C.byref(f), C.byref(cnt))
    lo, hi, acc, ws = _blend(L, w, f.value, cnt.value)
    # every rank sends (lo, hi) and its slabs padded to the full volume; rank 0 adds them: no data-path collective is needed for the
    # forwards themselves, only this gather of results
    full_a, full_w = torch.zeros(NH, V, V, V), torch.zeros(V, V, V)
    full_a[:, lo:hi] = torch.from_numpy(acc)
    full_w[lo:hi] = torch.from_numpy(ws)
    dist.reduce(full_a, 0)
    dist.reduce(full_w, 0)
    meta = torch.tensor([f.value, cnt.value], dtype=torch.int64)
    metas = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(metas, meta)
    if rank == 0:
        q.put((full_a.numpy(), full_w.numpy(), [m.tolist() for m in metas]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_window_shards_equal_single_process():
    sys.path.insert(0, os.path.dirname(HERE))
    import ufsm_b200
    L = ufsm_b200.lib()
    w = L.umx_window_make(V, P, OV)
    lo, hi, acc, ws = _blend(L, w, 0, w.npatch)
    assert (lo, hi) == (0, V)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    a2, w2, metas = q.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert metas[0][0] == 0 and metas[1][0] == metas[0][1] and metas[0][1] + metas[1][1] == w.npatch     # contiguous, complete shares
    assert np.allclose(w2, ws, rtol=1e-6) and np.allclose(a2, acc, rtol=1e-5, atol=1e-6)
    assert np.allclose(a2 / w2[None], acc / ws[None], rtol=1e-4, atol=1e-5)
