"""Generates tests/golden/mx_golden.npz from the reference's own conversions (oracle/_ref/libmxsw_ref.so, built from the reference's
src/mx_sw.cuh by oracle/Makefile).  Needs the reference tree at build time only; the fixture it writes is committed.

    python tests/golden/make_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import orc  # noqa: E402


def main():
    r = orc.ref()
    assert r is not None, "build oracle/_ref first (make -C oracle)"
    g = np.random.Generator(np.random.PCG64(20261125))
    parts = [g.standard_normal(4096).astype(np.float32) * s for s in (1.0, 6.0, 100.0, 448.0, 1e-3)]
    # every e4m3 / e2m1 value, the midpoints between neighbours, and one ulp either side of each midpoint
    e4 = np.array([r.ref_dec_e4m3(b) for b in range(0x7f)], np.float32)
    e2 = np.array([r.ref_dec_e2m1(b) for b in range(8)], np.float32)
    for grid in (e4, e2):
        mid = ((grid[:-1].astype(np.float64) + grid[1:].astype(np.float64)) / 2).astype(np.float32)
        for v in (grid, mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf))):
            parts += [v, -v]
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 448.0, 464.0, 465.0, 480.0, 1e38, 6.0, 5.0, 5.0000005, 7.0, 2.0 ** -9, 2.0 ** -10, 2.0 ** -11, 1.5 * 2.0 ** -10,
                        2.0 ** -126, 2.0 ** -140, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5], np.float32)
    parts += [special, -special]
    bits = g.integers(0, 2 ** 32, 8192, dtype=np.uint64).astype(np.uint32).view(np.float32)   # random bit patterns
    x = np.concatenate(parts + [bits]).astype(np.float32)
    c8, c4 = np.empty(x.size, np.uint8), np.empty(x.size, np.uint8)
    r.ref_enc_e4m3_n(x.ctypes.data_as(C.c_void_p), C.c_size_t(x.size), c8.ctypes.data_as(C.c_void_p))
    r.ref_enc_e2m1_n(x.ctypes.data_as(C.c_void_p), C.c_size_t(x.size), c4.ctypes.data_as(C.c_void_p))
    d8 = np.array([r.ref_dec_e4m3(b) for b in range(256)], np.float32)
    d4 = np.array([r.ref_dec_e2m1(b) for b in range(16)], np.float32)
    np.savez_compressed(os.path.join(HERE, "mx_golden.npz"), x_bits=x.view(np.uint32), e4m3=c8, e2m1=c4, dec_e4m3_bits=d8.view(np.uint32), dec_e2m1_bits=d4.view(np.uint32))
    print("wrote", x.size, "vectors")


if __name__ == "__main__":
    main()
