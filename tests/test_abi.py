"""CPU checks of the boundary: the library loads, exports every function include/ufsm_mx.h declares, the structs have the
reference's sizes, the host-only scheduler logic is right, and compute entries fail loudly without a B200."""
import ctypes as C
import os
import re

import numpy as np

import ufsm_b200
from ufsm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    src = open(os.path.join(ROOT, "include", "ufsm_mx.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b((?:lp|nn|umx)_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound():
    L = ufsm_b200.lib()
    names = header_functions()
    assert len(names) > 40
    for n in names:
        assert hasattr(L, n), "not exported: " + n
        assert n in _lib.SYMBOLS, "no ctypes signature: " + n
    for n in _lib.SYMBOLS:
        assert n in names, "bound but not declared in the header: " + n


def test_struct_sizes_match_the_reference():
    assert C.sizeof(ufsm_b200.Shape5) == 20
    assert C.sizeof(ufsm_b200.Split) <= 128 and C.sizeof(ufsm_b200.Split) == 128   # static_assert of src/nn_lp.h:38-41
    assert C.sizeof(ufsm_b200.Gnp) == 56
    assert C.sizeof(ufsm_b200.Feather) == 120        # umx_feather_t: 2 ints, 9 pointers, 7 ints, padding, 1 pointer


def test_storage_sizes():
    L = ufsm_b200.lib()
    assert L.lp_mx8_bytes(1, 32, 64 ** 3) == 64 ** 3 * 33 and L.lp_mx4_bytes(1, 64, 96 ** 3) == 2 * 96 ** 3 * 17
    assert L.lp_mx8_bytes(2, 4, 10) == 2 * 10 * 9 and L.lp_mx4_bytes(1, 16, 10) == 10 * 9
    assert L.umx_mx_bytes32(8, 1, 1, 100) == 3300 and L.umx_mx_bytes32(4, 2, 40, 10) == 2 * 2 * 10 * 17


def test_window_plan():
    L = ufsm_b200.lib()
    w = L.umx_window_make(1024, 128, 16)
    assert (w.nper, w.npatch) == (9, 729)
    z, y, x = C.c_int(), C.c_int(), C.c_int()
    L.umx_window_origin(C.byref(w), 728, C.byref(z), C.byref(y), C.byref(x))
    assert (z.value, y.value, x.value) == (896, 896, 896)
    covered = np.zeros(1024, bool)
    for i in range(9):
        L.umx_window_origin(C.byref(w), i, C.byref(z), C.byref(y), C.byref(x))
        covered[x.value:x.value + 128] = True
    assert covered.all()
    for world in (1, 2, 3, 4, 8):
        f, c = C.c_int(), C.c_int()
        seen = []
        for r in range(world):
            L.umx_window_share(C.byref(w), r, world, C.byref(f), C.byref(c))
            assert c.value % 9 == 0                       # whole (z, y) rows
            seen += list(range(f.value, f.value + c.value))
        assert seen == list(range(729))                   # every patch once, contiguous z-slab order
    w2 = L.umx_window_make(300, 128, 16)                  # the last patch is pulled back to the edge
    L.umx_window_origin(C.byref(w2), w2.npatch - 1, C.byref(z), C.byref(y), C.byref(x))
    assert w2.nper == 3 and x.value == 300 - 128
    lo, hi = C.c_int(), C.c_int()
    L.umx_window_share(C.byref(w), 1, 8, C.byref(f), C.byref(c))
    L.umx_window_extent(C.byref(w), f.value, c.value, C.byref(lo), C.byref(hi))
    assert 0 <= lo.value < hi.value <= 1024 and (hi.value - lo.value) % 16 == 0


def test_network_sizes():
    L = ufsm_b200.lib()
    cfg = ufsm_b200.UnetCfg()
    cfg.L = 5
    for i, v in enumerate([32, 64, 128, 256, 320]):
        cfg.cw[i] = v
    cfg.nh, cfg.P, cfg.bits_first, cfg.bits_mid, cfg.bits_last = 7, 128, 8, 8, 8
    import orc
    assert L.umx_unet_nweights(C.byref(cfg)) == orc.unet_nweights(orc.unet_cfg(128, [32, 64, 128, 256, 320]))
    assert abs(L.umx_unet_flops(C.byref(cfg)) / 1e9 - 1012.8) < 0.5     # the benchmark's figure for one 128^3 patch


def test_no_cpu_fallback():
    """Without a B200 a compute entry must latch an error, not compute something."""
    import torch
    if torch.cuda.is_available():
        return
    L = ufsm_b200.lib()
    L.lp_check()
    buf = np.zeros(64, np.float32)
    out = np.zeros(128, np.uint8)
    L.lp_f32_to_mx8(buf.ctypes.data, 1, 32, 2, out.ctypes.data)
    e = L.lp_check()
    assert e and b"no CPU path" in e or b"no other path" in e
    assert not out.any()
