"""numpy wrappers around the CPU oracle (liboracle.so beside this file).  Test infrastructure only: imported by the tests, the smoke
test and the CPU-baseline legs of the benchmark, never by the library."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))   # the repository root: this file sits in oracle/
ORC_DIR = os.path.join(ROOT, "oracle")
_o = None


class UnetCfg(C.Structure):
    _fields_ = [("L", C.c_int), ("cw", C.c_int * 8), ("nh", C.c_int), ("P", C.c_int), ("bits_first", C.c_int), ("bits_mid", C.c_int), ("bits_last", C.c_int)]


def o():
    global _o
    if _o is None:
        so = os.path.join(ORC_DIR, "liboracle.so")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(os.path.join(ORC_DIR, "mx_oracle.c")):
            subprocess.run(["make", "-C", ORC_DIR], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
        _o = C.CDLL(so)
        _o.orc_mx_exp.restype = C.c_int
        _o.orc_mx_exp.argtypes = [C.c_float, C.c_float]
        for f in ("orc_enc_e4m3", "orc_enc_e2m1"):
            getattr(_o, f).restype = C.c_uint
            getattr(_o, f).argtypes = [C.c_float]
        for f in ("orc_dec_e4m3", "orc_dec_e2m1", "orc_dec_scale"):
            getattr(_o, f).restype = C.c_float
            getattr(_o, f).argtypes = [C.c_uint]
        _o.orc_mx_bytes.restype = C.c_size_t
        _o.orc_mx_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_int]
        _o.orc_unet_nweights.restype = C.c_size_t
        _o.orc_threads.restype = C.c_int
    return _o


def ref():
    """The reference's own conversions (oracle/_ref/libmxsw_ref.so), or None when it was not built."""
    so = os.path.join(ORC_DIR, "_ref", "libmxsw_ref.so")
    if not os.path.exists(so):
        return None
    r = C.CDLL(so)
    r.ref_sweep_diff.restype = C.c_size_t
    r.ref_sweep_diff.argtypes = [C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_size_t, C.POINTER(C.c_uint32)]
    for f in ("ref_dec_e4m3", "ref_dec_e2m1"):
        getattr(r, f).restype = C.c_float
        getattr(r, f).argtypes = [C.c_uint]
    return r


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def enc(x, bits):
    x = f32(x).ravel()
    y = np.empty(x.size, np.uint8)
    (o().orc_enc_e2m1_n if bits == 4 else o().orc_enc_e4m3_n)(_p(x), C.c_size_t(x.size), _p(y))
    return y


def mx_bytes(bits, N, Cn, S, bw_force=0):
    return o().orc_mx_bytes(bits, N, Cn, C.c_size_t(S), bw_force)


def pm_to_mx(x, dt, N, Cn, S, bits, bw_force=0):
    x = np.ascontiguousarray(x)
    y = np.zeros(mx_bytes(bits, N, Cn, S, bw_force), np.uint8)
    o().orc_pm_to_mx(_p(x), dt, N, Cn, C.c_size_t(S), bits, bw_force, _p(y))
    return y


def mx_to_pm(mx, bits, N, Cn, S, bw_force=0):
    y = np.zeros(N * Cn * S, np.float32)
    o().orc_mx_to_pm(_p(mx), bits, N, Cn, C.c_size_t(S), bw_force, _p(y))
    return y


def nb32(Cn):
    return (Cn + 31) // 32


def mx_to_blocked(mx, bits, N, Cn, S):
    y = np.zeros(N * nb32(Cn) * S * 32, np.float32)
    o().orc_mx_to_blocked(_p(mx), bits, N, Cn, C.c_size_t(S), _p(y))
    return y


def blocked_to_mx(x, bits, N, Cn, S):
    x = f32(x)
    y = np.zeros(N * nb32(Cn) * S * (32 * bits // 8 + 1), np.uint8)
    o().orc_blocked_to_mx(_p(x), bits, N, Cn, C.c_size_t(S), _p(y))
    return y


def pm_to_blocked(x, N, Cn, S):
    x = f32(x)
    y = np.zeros(N * nb32(Cn) * S * 32, np.float32)
    o().orc_pm_to_blocked(_p(x), N, Cn, C.c_size_t(S), _p(y))
    return y


def blocked_to_pm(x, N, Cn, S):
    x = f32(x)
    y = np.zeros(N * Cn * S, np.float32)
    o().orc_blocked_to_pm(_p(x), N, Cn, C.c_size_t(S), _p(y))
    return y


def prep_w(w, Co, Ci, taps, bits, layout=0, want_codes=False):
    w = f32(w)
    Cip, Cop = nb32(Ci) * 32, nb32(Co) * 32
    wdq = np.zeros(taps * Cip * Cop, np.float32)
    if want_codes:
        wq = np.zeros(taps * (Cip // 32) * Cop * 32, np.uint8)
        ws = np.zeros(taps * (Cip // 32) * Cop, np.uint8)
        o().orc_prep_w(_p(w), Co, Ci, taps, bits, layout, _p(wdq), _p(wq), _p(ws))
        return wdq, wq, ws
    o().orc_prep_w(_p(w), Co, Ci, taps, bits, layout, _p(wdq), None, None)
    return wdq


def conv_blocked(x, N, Ci, D, H, W, wdq, bias, Co, k, stride, pad):
    x, wdq = f32(x), f32(wdq)
    Do, Ho, Wo = (D + 2 * pad - k) // stride + 1, (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    y = np.zeros(N * nb32(Co) * Do * Ho * Wo * 32, np.float32)
    b = f32(bias) if bias is not None else None
    o().orc_conv_blocked(_p(x), N, Ci, D, H, W, _p(wdq), _p(b) if b is not None else None, Co, k, stride, pad, _p(y))
    return y


def tconv_blocked(x, N, Ci, D, H, W, wdq, bias, Co):
    x, wdq = f32(x), f32(wdq)
    y = np.zeros(N * nb32(Co) * D * H * W * 8 * 32, np.float32)
    b = f32(bias) if bias is not None else None
    o().orc_tconv_blocked(_p(x), N, Ci, D, H, W, _p(wdq), _p(b) if b is not None else None, Co, _p(y))
    return y


def round_h16(v):
    v = f32(v).copy()
    o().orc_round_h16(_p(v), C.c_size_t(v.size))
    return v


def in_sums(y, N, Cn, S):
    y = f32(y)
    s = np.zeros(N * Cn * 2, np.float64)
    o().orc_in_sums(_p(y), N, Cn, C.c_size_t(S), _p(s))
    return s


def in_coef(sums, N, Cn, S, eps=1e-5):
    coef = np.zeros(N * Cn * 2, np.float32)
    o().orc_in_coef(_p(sums), N, Cn, C.c_double(S), None, None, C.c_float(eps), _p(coef))
    return coef


def in_apply(y, coef, N, Cn, S, act=2):
    y, coef = f32(y), f32(coef)
    out = np.zeros_like(y)
    o().orc_in_apply(_p(y), _p(coef), N, Cn, C.c_size_t(S), act, _p(out))
    return out


def s2d_blocked(x, N, Cn, D, H, W):
    x = f32(x)
    y = np.zeros(x.size, np.float32)
    o().orc_s2d_blocked(_p(x), N, Cn, D, H, W, _p(y))
    return y


def fake_quant_blocked(x, bits):
    x = f32(x).copy()
    o().orc_fake_quant_blocked(_p(x), C.c_size_t(x.size // 32), bits)
    return x


def unet_cfg(P, cw, nh=7, bits=(8, 8, 8)):
    c = UnetCfg()
    c.L = len(cw)
    for i, v in enumerate(cw):
        c.cw[i] = v
    c.nh, c.P = nh, P
    c.bits_first, c.bits_mid, c.bits_last = bits
    return c


def unet_nweights(cfg):
    return o().orc_unet_nweights(C.byref(cfg))


def unet_forward(cfg, weights, x16, N, descending=False):
    """descending: add the taps in the opposite order (another valid fp32 summation order of the same operands)."""
    o().orc_set_tap_order(1 if descending else 0)
    try:
        return _unet_forward(cfg, weights, x16, N)
    finally:
        o().orc_set_tap_order(0)


def _unet_forward(cfg, weights, x16, N):
    weights = f32(weights)
    x16 = np.ascontiguousarray(x16, dtype=np.float16)
    logits = np.zeros(N * cfg.nh * cfg.P ** 3, np.float32)
    o().orc_unet_forward(C.byref(cfg), _p(weights), _p(x16), N, _p(logits), None, None)
    return logits


def gauss_window(P):
    w = np.zeros(P, np.float32)
    o().orc_gauss_window(P, _p(w))
    return w


def blend_add_fx(logits, nh, P, V, z0, y0, x0, w1d, acc, wsum):
    """acc [nh][V^3] int64, wsum [V^3] int64, updated in place"""
    o().orc_blend_add_fx(_p(f32(logits)), nh, P, V, z0, y0, x0, _p(w1d), _p(acc), _p(wsum))


def emit_fx(acc, wsum, nh, fmt):
    """fmt 2: fp16 blended logits, else uint8"""
    out = np.zeros(acc.size, np.float16 if fmt == 2 else np.uint8)
    o().orc_emit_fx(_p(acc), _p(wsum), nh, C.c_size_t(wsum.size), fmt, _p(out))
    return out


def gn_silu(x, N, Cn, S, Gn, gamma, beta, mean, rstd, form, c_off=0, C_all=None):
    """silu(groupnorm(x)) of a plane-major fp32 tensor (or of a channel segment of a tensor of C_all channels), flat fp32"""
    x = f32(x)
    y = np.empty(N * Cn * S, np.float32)
    g, b, m, r = f32(gamma), f32(beta), f32(mean), f32(rstd)
    o().orc_gn_silu(_p(x), N, Cn, C.c_size_t(S), Gn, _p(g), _p(b), _p(m), _p(r), form, c_off, Cn if C_all is None else C_all, _p(y))
    return y


def up2(x, N, Cn, D, H, W):
    """exact-2x trilinear upsample in the reference's order of roundings, flat fp32 [N][Cn][2D][2H][2W]"""
    x = f32(x)
    y = np.empty(N * Cn * 8 * D * H * W, np.float32)
    o().orc_up2(_p(x), N, Cn, D, H, W, _p(y))
    return y


def conv1(x, w, b, N, Ci, Co, S):
    """1^3 conv with fp32 weights, bias first then ascending input channel, flat fp32 [N][Co][S]"""
    x, w = f32(x), f32(w)
    y = np.empty(N * Co * S, np.float32)
    bb = f32(b) if b is not None else None
    o().orc_conv1(_p(x), _p(w), _p(bb) if bb is not None else None, N, Ci, Co, C.c_size_t(S), _p(y))
    return y


def pred_input(ct, W, mean, isd, dyo, dxo, axis, z0, nz, hd):
    """the predict network input of planes [z0, z0 + nz): flat fp32 [4][nz W W]"""
    ct = np.ascontiguousarray(ct, dtype=np.uint8)
    dyo, dxo = f32(dyo), f32(dxo)
    out = np.empty(4 * nz * W * W, np.float32)
    o().orc_pred_input(_p(ct), W, C.c_float(mean), C.c_float(isd), _p(dyo), _p(dxo), axis, z0, nz, hd, _p(out))
    return out


def prob255(lg):
    """the probability byte of the reference's predict back end (src/nn_elem.cu:1100, 1123): trunc(255 / (1 + exp(-logit)) + 0.5), fp32"""
    lg = np.asarray(lg, np.float32)
    with np.errstate(over="ignore"):
        e = np.exp(-lg, dtype=np.float32)
    return (np.float32(255) / (np.float32(1) + e) + np.float32(0.5)).astype(np.uint8)


def pred_place(lg, material, D, W, hz, halo, oz, oy, ox, ez, ey, ex, shard, dsh, zoff=0, zlo=None, zhi=None):
    """nn_pred_place_d / _m_d / _mz (src/nn_elem.cu:1107-1178): the interior of a window (held from plane zoff on: lg and material are
    [D - zoff.., W, W] arrays indexed by z - zoff) into the shard buffer dsh [shard]^3 (modified in place) at (oz, oy, ox), clipped to
    [0, ez) x [0, ey) x [0, ex); only planes [zlo, zhi) when given."""
    lg = np.asarray(lg, np.float32).reshape(-1, W, W)
    material = np.asarray(material, bool).reshape(-1, W, W)
    out = dsh.reshape(shard, shard, shard)
    z0, z1 = max(hz, -oz), min(D - hz, ez - oz)
    if zlo is not None:
        z0, z1 = max(z0, zlo), min(z1, zhi)
    y0, y1 = max(halo, -oy), min(W - halo, ey - oy)
    x0, x1 = max(halo, -ox), min(W - halo, ex - ox)
    if z1 <= z0 or y1 <= y0 or x1 <= x0:
        return dsh
    sub = (slice(z0 - zoff, z1 - zoff), slice(y0, y1), slice(x0, x1))
    out[oz + z0:oz + z1, oy + y0:oy + y1, ox + x0:ox + x1] = np.where(material[sub], prob255(lg[sub]), 0).astype(np.uint8)
    return dsh


def ctmask(ct, t=1):
    """nn_pred_ctmask_t (src/nn_elem.cu:1135-1144): bit k & 31 of word k >> 5 = ct[k] >= t"""
    ct = np.asarray(ct, np.uint8).ravel()
    b = np.zeros((ct.size + 31) // 32 * 32, np.uint8)
    b[:ct.size] = ct >= max(t, 1)
    return np.packbits(b.reshape(-1, 32), axis=1, bitorder="little").view(np.uint32).ravel()


def feather_u(B):
    """the seam feather's ramp (feather_init, src/predict.c:334-336): u[0][j] = sin^2(pi / 2 (j + 0.5) / B), u[1][j] = 1 - that, cast to fp32"""
    j = np.arange(B, dtype=np.float64)
    s = np.sin(np.pi / 2 * (j + 0.5) / B)
    return np.stack([(s * s).astype(np.float32), (1 - s * s).astype(np.float32)])


def feather_blend(e, nb, S, B, oo, on, osh, out):
    """fe_val / fe_blend / fe_rows (src/predict.c:296-333): e [E][E][E] (E = S + B), nb[d] the spill slab of the window back by d's bits (bit 0
    x, 1 y, 2 z) or None: z slab [B][E][E] if d & 4, else y slab [S][B][E] if d & 2, else x slab [S][S][B]; the interior box [oo, oo + on) goes to
    out[(lz osh + ly) osh + lx] (modified in place).  fp32 products and sums in the reference's order."""
    E = S + B
    e = np.asarray(e, np.uint8).reshape(E, E, E)
    u = feather_u(B)
    o = out.reshape(osh, osh, osh)
    f32 = np.float32

    def val(d, z, y, x):
        if not d:
            return e[z, y, x]
        p = nb[d]
        uz, uy, ux = z + (S if d & 4 else 0), y + (S if d & 2 else 0), x + (S if d & 1 else 0)
        if uz >= S:
            return p.reshape(B, E, E)[uz - S, uy, ux]
        if uy >= S:
            return p.reshape(S, B, E)[uz, uy - S, ux]
        return p.reshape(S, S, B)[uz, uy, ux - S]

    for lz in range(on[0]):
        for ly in range(on[1]):
            for lx in range(on[2]):
                z, y, x = oo[0] + lz, oo[1] + ly, oo[2] + lx
                if z >= B and y >= B and x >= B:
                    o[lz, ly, lx] = e[z, y, x]
                    continue
                s, w = f32(0), f32(0)
                for d in range(8):
                    if d and nb[d] is None:
                        continue
                    dz, dy, dx = d >> 2 & 1, d >> 1 & 1, d & 1
                    if (dz and z >= B) or (dy and y >= B) or (dx and x >= B):
                        continue
                    wi = f32(f32(u[dz][z] if z < B else f32(1)) * f32(u[dy][y] if y < B else f32(1))) * f32(u[dx][x] if x < B else f32(1))
                    s = f32(s + f32(wi * f32(val(d, z, y, x))))
                    w = f32(w + wi)
                o[lz, ly, lx] = np.uint8(min(f32(255), f32(f32(s / w) + f32(0.5)))) if w > 0 else 0
    return out


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def conv_case(kind, x, w, b, N, Ci, D, H, W, Co, bits):
    """One conv layer on identical operands.  x: plane-major fp32 [N][Ci][S].  Returns (the MX bytes a conv under test reads, in the
    reference layout with 32-wide blocks; the oracle's acc + bias as plane-major fp32 [N][Co][So])."""
    S = D * H * W
    mx = pm_to_mx(x, 0, N, Ci, S, bits, 32)
    xb = mx_to_blocked(mx, bits, N, Ci, S)
    if kind == "conv3":
        acc = conv_blocked(xb, N, Ci, D, H, W, prep_w(w, Co, Ci, 27, bits), b, Co, 3, 1, 1)
        return mx, blocked_to_pm(acc, N, Co, S)
    if kind == "conv1":
        acc = conv_blocked(xb, N, Ci, D, H, W, prep_w(w, Co, Ci, 1, bits), b, Co, 1, 1, 0)
        return mx, blocked_to_pm(acc, N, Co, S)
    if kind == "down2":
        acc = conv_blocked(xb, N, Ci, D, H, W, prep_w(w, Co, Ci, 8, bits), b, Co, 2, 2, 0)
        mxs = blocked_to_mx(s2d_blocked(xb, N, Ci, D, H, W), bits, N, 8 * nb32(Ci) * 32, S // 8)
        return mxs, blocked_to_pm(acc, N, Co, S // 8)
    if kind == "conv3s2":
        acc = conv_blocked(xb, N, Ci, D, H, W, prep_w(w, Co, Ci, 27, bits), b, Co, 3, 2, 1)
        return mx, blocked_to_pm(acc, N, Co, ((D + 1) // 2) * ((H + 1) // 2) * ((W + 1) // 2))
    acc = tconv_blocked(xb, N, Ci, D, H, W, prep_w(w, Co, Ci, 8, bits, layout=1), b, Co)
    return mx, blocked_to_pm(acc, N, Co, 8 * S)
