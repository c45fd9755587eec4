"""umx_in_coef_static: the entry point for callers that cannot allocate (their own pool owns the device memory, or allocation is
forbidden once the pipeline runs).  It must give the coefficients of the existing path (conv epilogue partial sums in a caller buffer
+ umx_in_coef) from the stored tensor alone, on two calls in a row that share the library's built-in scratch array, and must refuse
sizes the array cannot hold.  This file is collected last so a failure here cannot hide another test's."""
import ctypes as C

import numpy as np
import pytest

import gpu_util as G
import orc
import synth
import ufsm_b200
from ufsm_b200 import DevBuf

pytestmark = pytest.mark.gpu


def coefs_both_ways(L, seed, N, Ci, Co, D, H, W):
    S = D * H * W
    x = synth.rng(seed).standard_normal(N * Ci * S).astype(np.float32)
    w, b = synth.kaiming(seed + 1, Co, Ci, 27), synth.bias(seed + 2, Co, 0.1)
    mx = orc.pm_to_mx(x, 0, N, Ci, S, 8, 32)
    conv = G.Conv("conv3", w, b, Co, Ci, 8)
    yd = DevBuf(N * orc.nb32(Co) * S * 64).fill(0xEE)
    _, part = conv.fwd(mx, N, D, H, W, G.OUT_H16B, want_part=True, dst=yd)       # existing path: caller-allocated partial sums
    ref, _ = G.in_coef(part, N, Co, D, H, W)
    out = DevBuf(N * Co * 8).fill(0xEE)
    rc = L.umx_in_coef_static(yd.ptr, N, Co, D, H, W, None, None, C.c_float(1e-5), out.ptr)   # new path: no allocation inside
    ufsm_b200.check()
    assert rc == 0
    conv.free()
    want = orc.in_coef(orc.in_sums(yd.download(np.float16).astype(np.float32), N, Co, S), N, Co, S)   # the oracle's fp64 statistics of the stored tensor
    return out.download(np.float32), ref, want


def test_two_calls_in_a_row_match_the_existing_entry(dev):
    # the second call is smaller than the first: it must not see what the first left in the shared array
    for seed, shape in ((70, (2, 32, 96, 3, 19, 11)), (80, (1, 32, 40, 2, 7, 5))):
        got, ref, want = coefs_both_ways(dev, seed, *shape)
        assert np.isfinite(got).all()
        assert np.array_equal(got, want), "max diff to the oracle %g" % np.abs(got - want).max()
        # the two paths add the same fp64 terms in different groupings: equal to a float32 rounding
        assert np.allclose(got, ref, rtol=3e-7, atol=3e-7 * np.abs(ref).max()), "max diff %g" % np.abs(got - ref).max()


def test_sizes_beyond_the_array_are_refused(dev):
    out = DevBuf(64).fill(0xEE)
    rc = dev.umx_in_coef_static(out.ptr, 16, 512, 2, 2, 2, None, None, C.c_float(1e-5), out.ptr)   # 16 x 64 x 512 x 2 doubles > 524288
    e = dev.lp_check()
    assert rc == -1 and e and b"built-in array" in e
    assert np.all(out.download() == 0xEE)                                                          # nothing ran
    rc = dev.umx_in_coef_static(out.ptr, 1, 32, 0, 2, 2, None, None, C.c_float(1e-5), out.ptr)     # an empty grid
    e = dev.lp_check()
    assert rc == -1 and e and b"at least 1" in e
