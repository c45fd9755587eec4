"""Time one conv layer of the MX U-Net path on the current GPU.

    python -m ufsm_b200.layer_bench --kind conv3 --ci 32 --co 32 --size 128 [--bits 8] [--reps 5] [--out h16b|mx|pm32]

The input is an MX tensor of arbitrary finite codes (split layout for fp8), the weights are Kaiming-normal.  Prints the best of
`reps` device times (events around the launch) and the algorithmic TFLOP/s.  Also the command used for the profiler captures
summarised under profiles/."""
import argparse
import ctypes as C

import numpy as np

import ufsm_b200
from ufsm_b200 import DevBuf

KIND = {"conv3": 0, "conv1": 1, "down2": 2, "tconv2": 3, "conv3s2": 4}
OUT = {"h16b": 0, "mx": 1, "pm32": 2}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="conv3", choices=list(KIND))
    ap.add_argument("--ci", type=int, default=32)
    ap.add_argument("--co", type=int, default=32)
    ap.add_argument("--size", type=int, default=128, help="edge of the cubic grid of GEMM rows (the conv's input grid; for down2 the output grid; for conv3s2 the input grid, output = half)")
    ap.add_argument("--bits", type=int, default=8)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--out", default="h16b", choices=list(OUT))
    a = ap.parse_args()
    L = ufsm_b200.lib()
    assert L.nn_init(0) == 0, (L.lp_check() or b"").decode()
    D = a.size
    S = D ** 3
    nbi = (a.ci + 31) // 32 * (8 if a.kind == "down2" else 1)
    rb = 32 * a.bits // 8
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.integers(0, 120, nbi * S * rb, dtype=np.uint8), rng.integers(100, 130, nbi * S, dtype=np.uint8)])
    taps = {"conv3": 27, "conv1": 1, "down2": 8, "tconv2": 8, "conv3s2": 27}[a.kind]
    w = (rng.standard_normal((a.co, a.ci, taps)) * np.sqrt(2.0 / (a.ci * taps))).astype(np.float32)
    if a.kind == "tconv2":
        w = np.ascontiguousarray(w.transpose(1, 0, 2))
    h = L.umx_conv_create(KIND[a.kind], w.ctypes.data, None, a.co, a.ci, a.bits)
    ufsm_b200.check()
    f = 8 if a.kind == "tconv2" else 1
    nbo = (a.co + 31) // 32
    mode = OUT[a.out]
    So = ((D + 1) // 2) ** 3 if a.kind == "conv3s2" else S * f
    nbytes = {0: nbo * So * 64, 1: nbo * So * (rb + 1), 2: a.co * So * 4}[mode]
    xd, yd = DevBuf(data=x), DevBuf(nbytes)
    best, ms, fl = 1e30, C.c_double(), C.c_double()
    for _ in range(a.reps):
        L.umx_prof_begin()
        rc = L.umx_conv_fwd(h, xd.ptr, 1, D, D, D, yd.ptr, mode, a.bits if mode == 1 else 0, 0, 0, None, 3)
        L.umx_prof_end(C.byref(ms), C.byref(fl))
        assert rc == 0
        best = min(best, ms.value)
    ufsm_b200.check()
    print("%s %d->%d on %d^3 MX-fp%d out %s: %.1f us, %.0f TFLOP/s" % (a.kind, a.ci, a.co, D, a.bits, a.out, best * 1e3, fl.value / best / 1e9))
    L.umx_conv_free(h)


if __name__ == "__main__":
    main()
