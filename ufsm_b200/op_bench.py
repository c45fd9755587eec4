"""Time the elementwise MX operators of the reference interface on the current GPU and print their algorithmic GB/s.

    python -m ufsm_b200.op_bench [--c 32] [--size 128] [--bits 8] [--reps 5]

Operators: lp_gn_sums_mx, lp_gn_silu_apply_mx, lp_up2_fwd_mx (from size / 2), lp_conv1_fwd_mx (7 outputs), lp_conv_fwd_s2_f8's
kernel is timed by layer_bench --kind conv3s2.  Inputs are MX tensors of arbitrary finite codes on a size^3 grid (larger than L2 at the
defaults); times are the best of `reps` (events around the call)."""
import argparse
import ctypes as C

import numpy as np

import ufsm_b200
from ufsm_b200 import DevBuf, Shape5, Gnp


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--c", type=int, default=32)
    ap.add_argument("--size", type=int, default=128)
    ap.add_argument("--bits", type=int, default=8)
    ap.add_argument("--reps", type=int, default=5)
    a = ap.parse_args()
    L = ufsm_b200.lib()
    assert L.nn_init(0) == 0, (L.lp_check() or b"").decode()
    D, Cn, G = a.size, a.c, 8
    S, nb, rb, dt = D ** 3, (a.c + 31) // 32, 32 * a.bits // 8, 3 if a.bits == 8 else 4
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.integers(0, 120, nb * S * rb, dtype=np.uint8), rng.integers(120, 130, nb * S, dtype=np.uint8)])
    xd, yd = DevBuf(data=x), DevBuf(nb * S * (rb + 1))
    par = [DevBuf(data=v) for v in (np.ones(Cn, np.float32), np.zeros(Cn, np.float32), np.zeros(G, np.float32), np.ones(G, np.float32))]
    gp = Gnp()
    sums = DevBuf(G * 2 * 24).fill(0)
    w = DevBuf(data=(rng.standard_normal((7, Cn)) / np.sqrt(Cn)).astype(np.float32))
    logits = DevBuf(7 * S * 4)
    Dh = D // 2
    t = L.umx_timer_new()

    def run(name, fn, nbytes):
        best = 1e30
        for _ in range(a.reps):
            L.umx_timer_start(t)
            fn()
            best = min(best, L.umx_timer_stop_ms(t))
        ufsm_b200.check()
        print("%-22s %d ch on %d^3 MX-fp%d: %.1f us, %.0f GB/s (algorithmic %.1f MB)" % (name, Cn, D, a.bits, best * 1e3, nbytes / best / 1e6, nbytes / 1e6))

    mxb = nb * S * (rb + 1)
    run("lp_gn_sums_mx", lambda: L.lp_gn_sums_mx(xd.ptr, dt, 1, Cn, G, S, sums.ptr, 0, S), mxb)
    run("lp_gn_silu_apply_mx", lambda: L.lp_gn_silu_apply_mx(xd.ptr, dt, Shape5(1, Cn, D, D, D), G, par[0].ptr, par[1].ptr, par[2].ptr, par[3].ptr, yd.ptr, dt), 2 * mxb)
    run("lp_up2_fwd_mx", lambda: L.lp_up2_fwd_mx(xd.ptr, dt, Shape5(1, Cn, Dh, Dh, Dh), yd.ptr, dt, gp), mxb + mxb // 8)
    run("lp_conv1_fwd_mx (7)", lambda: L.lp_conv1_fwd_mx(xd.ptr, dt, Shape5(1, Cn, D, D, D), w.ptr, None, 7, logits.ptr, gp), mxb + 7 * S * 4)
    L.umx_timer_free(t)


if __name__ == "__main__":
    main()
