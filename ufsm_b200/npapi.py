"""numpy-facing helpers over the C ABI for the benchmark, the smoke test and the tests: they upload numpy arrays, call the
library's entry points and download the results (device memory through nn_malloc).  Not part of the product interface."""
import ctypes as C

import numpy as np


from ._lib import DevBuf, UnetCfg, check as _check, lib as _libf

KIND = {"conv3": 0, "conv1": 1, "down2": 2, "tconv2": 3, "conv3s2": 4}
OUT_H16B, OUT_MX, OUT_PM32, OUT_PM16, OUT_MXRAW, OUT_PROB8 = 0, 1, 2, 3, 4, 5


def nb32(Cn):
    return (Cn + 31) // 32


def L():
    return _libf()


def to_split(mx, N, Cn, S, bits):
    """MX bytes (32-wide blocks) from the reference layout to the split layout (fp8 only; fp4 rows are 16 bytes already)."""
    if bits != 8:
        return mx
    rows = N * nb32(Cn) * S
    codes = mx[: rows * 32].reshape(N * nb32(Cn), S, 2, 16).transpose(0, 2, 1, 3)
    return np.concatenate([np.ascontiguousarray(codes).ravel(), mx[rows * 32:]])


def from_split(mx, N, Cn, S, bits):
    if bits != 8:
        return mx
    rows = N * nb32(Cn) * S
    codes = mx[: rows * 32].reshape(N * nb32(Cn), 2, S, 16).transpose(0, 2, 1, 3)
    return np.concatenate([np.ascontiguousarray(codes).ravel(), mx[rows * 32:]])


def quantise_pm(x, dt, N, Cn, S, bits, wide32=False, layout=0):
    """plane-major fp32 (dt 0) / fp16 (dt 2) -> MX bytes via the reference-named entry points (or the 32-wide variant)."""
    xd = DevBuf(data=x)
    nbytes = L().umx_mx_bytes32(bits, N, Cn, S) if wide32 else (L().lp_mx8_bytes if bits == 8 else L().lp_mx4_bytes)(N, Cn, S)
    yd = DevBuf(nbytes).fill(0xEE)
    if wide32:
        L().umx_pm_to_mx32(xd.ptr, dt, N, Cn, S, yd.ptr, bits, layout)
    elif dt == 0:
        (L().lp_f32_to_mx8 if bits == 8 else L().lp_f32_to_mx4)(xd.ptr, N, Cn, S, yd.ptr)
    else:
        (L().lp_h16_to_mx8 if bits == 8 else L().lp_h16_to_mx4)(xd.ptr, dt, N, Cn, S, yd.ptr)
    _check()
    return yd.download()


def dequantise(mx, bits, N, Cn, S):
    xd = DevBuf(data=mx)
    yd = DevBuf(N * Cn * S * 4).fill(0xEE)
    (L().lp_mx8_to_f32 if bits == 8 else L().lp_mx4_to_f32)(xd.ptr, N, Cn, S, yd.ptr)
    _check()
    return yd.download(np.float32)


class Conv:
    def __init__(self, kind, w, b, co, ci, bits):
        w = np.ascontiguousarray(w, np.float32)
        bp = np.ascontiguousarray(b, np.float32) if b is not None else None
        self.h = L().umx_conv_create(KIND[kind], w.ctypes.data, bp.ctypes.data if bp is not None else None, co, ci, bits)
        _check()
        assert self.h
        self.kind, self.co, self.ci, self.bits = kind, co, ci, bits

    def fwd(self, x_mx, N, D, H, W, out_mode, out_bits=0, nb_dst=0, b0=0, want_part=False, dst=None, split=True):
        """x_mx: numpy MX bytes (32-wide blocks, reference layout).  split: hand the conv fp8 tensors in the split layout (what the graph
        does) and bring MX outputs back to the reference layout; otherwise the reference layout goes through the C ABI as it is.
        Returns (output bytes as uint8 array, partial sums or None)."""
        cin_t = (8 if self.kind == "down2" else 1) * nb32(self.ci) * 32
        xd = DevBuf(data=to_split(x_mx, N, cin_t, D * H * W, self.bits) if split else x_mx)
        flags = 3 if split else 0
        f = 8 if self.kind == "tconv2" else 1
        So = D * H * W * f
        if self.kind == "conv3s2":      # D, H, W are the input grid
            So = ((D + 1) // 2) * ((H + 1) // 2) * ((W + 1) // 2)
        nbo = nb_dst if nb_dst else nb32(self.co)
        if out_mode == OUT_H16B:
            nbytes = N * nbo * So * 64
        elif out_mode in (OUT_MX, OUT_MXRAW):
            nbytes = N * nbo * So * (32 * out_bits // 8 + 1)
        elif out_mode == OUT_PM32:
            nbytes = N * self.co * So * 4
        elif out_mode == OUT_PROB8:
            nbytes = N * self.co * So
        else:
            nbytes = N * self.co * So * 2
        yd = dst if dst is not None else DevBuf(nbytes).fill(0xEE)
        pd = None
        if want_part:
            pd = DevBuf(L().umx_stats_doubles(N, self.co, D, H, W) * 8).fill(0xEE)
        rc = L().umx_conv_fwd(self.h, xd.ptr, N, D, H, W, yd.ptr, out_mode, out_bits, nb_dst, b0, pd.ptr if pd else None, flags)
        _check()
        assert rc == 0
        out = yd.download()
        if split and out_mode in (OUT_MX, OUT_MXRAW):
            out = from_split(out, N, nbo * 32, So, out_bits)
        return out, (pd if want_part else None)

    def fwd_h16(self, x16, N, D, H, W, out_mode=OUT_H16B, norm=False, eps=1e-5, u8=False):
        """the conv on the planar fp16 tensor itself (UMX_X_H16: quantised on the way in), or (u8) on CT bytes read as byte / 255 (UMX_X_U8).
        Returns (output bytes, coef or None, the kernel that ran: umx_conv_last_kernel)."""
        xd = DevBuf(data=np.ascontiguousarray(x16, np.uint8 if u8 else np.float16))
        xflag = 16 if u8 else 8
        S = D * H * W
        yd = DevBuf(N * nb32(self.co) * S * 64 if out_mode == OUT_H16B else N * self.co * S * 4).fill(0xEE)
        cd = None
        if norm:
            pd = DevBuf(L().umx_stats_doubles(N, self.co, D, H, W) * 8).fill(0xEE)
            cd = DevBuf(N * self.co * 8).fill(0xEE)
            rc = L().umx_conv_fwd_norm(self.h, xd.ptr, N, D, H, W, yd.ptr, pd.ptr, None, None, C.c_float(eps), cd.ptr, xflag)
        else:
            rc = L().umx_conv_fwd(self.h, xd.ptr, N, D, H, W, yd.ptr, out_mode, 0, 0, 0, None, xflag)
        _check()
        assert rc == 0
        return yd.download(), (cd.download(np.float32) if cd else None), L().umx_conv_last_kernel()

    def fwd_norm(self, x_mx, N, D, H, W, eps=1e-5, epilogue_stats=False):
        """conv -> blocked fp16 + InstanceNorm coefficients in one call; returns (fp16 blocked values, coef [N * co * 2])"""
        xd = DevBuf(data=to_split(x_mx, N, nb32(self.ci) * 32, D * H * W, self.bits))
        yd = DevBuf(N * nb32(self.co) * D * H * W * 64).fill(0xEE)
        pd = DevBuf(L().umx_stats_doubles(N, self.co, D, H, W) * 8).fill(0xEE)
        cd = DevBuf(N * self.co * 8).fill(0xEE)
        rc = L().umx_conv_fwd_norm(self.h, xd.ptr, N, D, H, W, yd.ptr, pd.ptr, None, None, C.c_float(eps), cd.ptr, 3 | (4 if epilogue_stats else 0))
        _check()
        assert rc == 0
        return yd.download(np.float16), cd.download(np.float32)

    def free(self):
        if self.h:
            L().umx_conv_free(self.h)
            self.h = None


def run_pm32(kind, mx, w, b, N, Ci, D, H, W, Co, bits, split=True):
    """one conv on MX bytes (reference layout) -> acc + bias as plane-major fp32; D, H, W: the input grid (down2: the fine grid)"""
    c = Conv(kind, w, b, Co, Ci, bits)
    g = (D // 2, H // 2, W // 2) if kind == "down2" else (D, H, W)
    raw, _ = c.fwd(mx, N, *g, OUT_PM32, split=split)
    c.free()
    return raw.view(np.float32)


def h16b_to_blocked_f32(raw, n_elems=None):
    return raw.view(np.float16).astype(np.float32)


def in_coef(part, N, Cn, D, H, W, eps=1e-5):
    cd = DevBuf(N * Cn * 8).fill(0xEE)
    L().umx_in_coef(part.ptr, N, Cn, D, H, W, None, None, C.c_float(eps), cd.ptr)
    _check()
    return cd.download(np.float32), cd


def in_stats_coef(y16_blocked, N, Cn, D, H, W, eps=1e-5):
    """statistics + coefficients of a stored blocked-fp16 tensor in one launch"""
    yd = DevBuf(data=np.ascontiguousarray(y16_blocked, np.float16))
    pd = DevBuf(L().umx_stats_doubles(N, Cn, D, H, W) * 8).fill(0xEE)
    cd = DevBuf(N * Cn * 8).fill(0xEE)
    L().umx_in_stats_coef(yd.ptr, N, Cn, D, H, W, None, None, C.c_float(eps), pd.ptr, cd.ptr)
    _check()
    return cd.download(np.float32)


def in_apply(y16_blocked, coef, N, Cn, D, H, W, act, bits, nb_dst=0, b0=0, want_s2d=False, want_h=False, split=True):
    S = D * H * W
    nb = nb32(Cn)
    xd = DevBuf(data=np.ascontiguousarray(y16_blocked, np.float16))
    cd = DevBuf(data=np.ascontiguousarray(coef, np.float32)) if coef is not None else None
    rb = 32 * bits // 8 + 1
    qd = DevBuf(N * (nb_dst or nb) * S * rb).fill(0xEE)
    sd = DevBuf(N * 8 * nb * (S // 8) * rb).fill(0xEE) if want_s2d else None
    hd = DevBuf(N * nb * S * 64).fill(0xEE) if want_h else None
    L().umx_in_apply(xd.ptr, cd.ptr if cd else None, N, Cn, D, H, W, act, qd.ptr, bits, nb_dst, b0, sd.ptr if sd else None, hd.ptr if hd else None, 1 if split else 0)
    _check()
    q, s2 = qd.download(), (sd.download() if sd else None)
    if split:
        q = from_split(q, N, (nb_dst or nb) * 32, S, bits)
        if s2 is not None:
            s2 = from_split(s2, N, 8 * nb * 32, S // 8, bits)
    return q, s2, (hd.download(np.float16) if hd else None)


def make_cfg(P, cw, nh=7, bits=(8, 8, 8)):
    c = UnetCfg()
    c.L = len(cw)
    for i, v in enumerate(cw):
        c.cw[i] = v
    c.nh, c.P = nh, P
    c.bits_first, c.bits_mid, c.bits_last = bits
    return c


class Unet:
    def __init__(self, cfg, weights, max_batch=1):
        weights = np.ascontiguousarray(weights, np.float32)
        assert weights.size == L().umx_unet_nweights(C.byref(cfg))
        self.cfg = cfg
        self.h = L().umx_unet_create(C.byref(cfg), weights.ctypes.data, max_batch)
        assert self.h, (L().lp_check() or b"").decode()

    def forward(self, x16, N):
        xd = DevBuf(data=np.ascontiguousarray(x16, np.float16))
        yd = DevBuf(N * self.cfg.nh * self.cfg.P ** 3 * 4).fill(0xEE)
        rc = L().umx_unet_forward(self.h, xd.ptr, N, yd.ptr)
        _check()
        assert rc == 0
        return yd.download(np.float32)

    def forward_host(self, ct_u8, N):
        ct_u8 = np.ascontiguousarray(ct_u8, np.uint8)
        out = np.empty(N * self.cfg.nh * self.cfg.P ** 3, np.float16)
        rc = L().umx_unet_forward_host(self.h, ct_u8.ctypes.data, N, out.ctypes.data)
        assert rc == 0, (L().lp_check() or b"").decode()
        return out

    def free(self):
        if self.h:
            L().umx_unet_free(self.h)
            self.h = None
