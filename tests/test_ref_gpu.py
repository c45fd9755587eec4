"""The oracle and the library against the reference's own code for this path, built for sm_100a from the reference tree where it lies
(oracle/_ref/libref_gpu.so, recipe in oracle/Makefile; oracle/ref_gpu.cu describes what is built):

  * the host weight rounding of the emulated-MX path, fq_host (src/nn_xnet.cu:168-173), which takes its block exponent from
    frexpf(am / q) with a true division, against the oracle's weight quantiser, which follows mx_exp (a multiply by 1 / q): the
    disagreements are counted, on random blocks and on blocks whose amax sits on and beside q 2^k (CPU test);
  * on a B200: the quantiser entry points lp_f32_to_mx8/4 and lp_h16_to_mx8/4 (src/lp_mx_cvt.cu:59-79) byte for byte against the
    library and the oracle; the emulated-MX convs (UFSM_XNET_FQ, src/nn_xnet.cu:128-232, 1467-1476) on the benchmark's
    configurations 1 and 2 against the oracle and the library within 1e-3 relative L2; the InstanceNorm coefficient and apply kernels
    k_in_coef / k_inq (src/nn_xnet.cu:1565-1620) bit for bit against the oracle's orc_in_coef / orc_in_apply."""
import ctypes as C
import os

import numpy as np
import pytest

import orc
import synth

SO = os.path.join(orc.ORC_DIR, "_ref", "libref_gpu.so")
TOL = 1e-3
_r = None


def ref():
    global _r
    if _r is None:
        if not os.path.exists(SO):
            pytest.skip("oracle/_ref/libref_gpu.so not built (reference tree absent when the oracle was made)")
        r = C.CDLL(SO)
        r.refgpu_fq_host.argtypes = [C.c_void_p, C.c_int, C.c_int]
        r.refgpu_mx_bytes.restype = C.c_size_t
        r.refgpu_mx_bytes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t]
        r.refgpu_to_mx.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p]
        r.refgpu_mx_to_f32.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]
        r.refgpu_conv.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [C.c_void_p] + [C.c_int] * 4 + [C.c_void_p, C.c_void_p]
        r.refgpu_tconv3.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p] + [C.c_int] * 4 + [C.c_void_p]
        r.refgpu_in.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p, C.c_int]
        _r = r
    return _r


def test_host_weight_rounding_frexp_against_mx_exp():
    r = ref()
    g = synth.rng(5)
    for bits, q in ((8, 448.0), (4, 6.0)):
        blocks = []
        for t in range(4000):
            blocks.append((g.standard_normal(32) * 2.0 ** g.integers(-24, 12)).astype(np.float32))
        # amax on q 2^k and one float to either side: where a true division and a multiply by the rounded reciprocal could part
        for k in range(-30, 30):
            for step in (-1, 0, 1):
                am = np.float32(q * 2.0 ** k)
                if step:
                    am = np.nextafter(am, np.float32(np.inf if step > 0 else 0), dtype=np.float32)
                v = (g.uniform(-1, 1, 32) * am).astype(np.float32)
                v[int(g.integers(32))] = am if g.integers(2) else -am
                blocks.append(v)
        differ = 0
        for v in blocks:
            a = v.copy()
            r.refgpu_fq_host(a.ctypes.data, 32, bits)
            differ += not np.array_equal(a, orc.fake_quant_blocked(v, bits))
        print("MX-fp%d: %d of %d blocks differ between frexpf(am / q) and mx_exp(am, 1 / q)" % (bits, differ, len(blocks)))
        assert differ == 0


def ndhwc(blocked, N, Cn, S):
    """blocked [n][blk][voxel][32] -> [n][voxel][Cn]"""
    nb = orc.nb32(Cn)
    return np.ascontiguousarray(blocked.reshape(N, nb, S, 32).transpose(0, 2, 1, 3).reshape(N, S, nb * 32)[:, :, :Cn])


def to_blocked(x_ndhwc, N, Cn, S):
    nb = orc.nb32(Cn)
    t = np.zeros((N, S, nb * 32), x_ndhwc.dtype)
    t[:, :, :Cn] = x_ndhwc.reshape(N, S, Cn)
    return np.ascontiguousarray(t.reshape(N, S, nb, 32).transpose(0, 2, 1, 3)).ravel()


@pytest.mark.gpu
@pytest.mark.parametrize("N,Cn,S,dt", [(1, 32, 64 ** 3, 2), (2, 40, 1000, 0), (1, 8, 999, 2), (1, 16, 501, 0), (3, 5, 77, 2)])
def test_reference_quantiser_bytes(dev, N, Cn, S, dt):
    """lp_h16_to_mx8/4 and lp_f32_to_mx8/4 of the reference build == the library == the oracle (configuration 1's input first;
    then ragged channel counts and the 8- and 16-wide rows of C <= 8 / <= 16)."""
    import gpu_util as G
    r = ref()
    x = synth.rng(1).standard_normal(N * Cn * S).astype(np.float16 if dt == 2 else np.float32)
    if dt == 0:
        x[::97] *= np.float32(1e-30)
        x[5] = np.inf
        x[11] = np.nan
    for bits in (8, 4):
        y = np.zeros(r.refgpu_mx_bytes(bits, N, Cn, S), np.uint8)
        assert r.refgpu_to_mx(bits, x.ctypes.data, dt, N, Cn, S, y.ctypes.data) == 0
        assert np.array_equal(y, orc.pm_to_mx(x, dt, N, Cn, S, bits)), "reference != oracle (MX-fp%d)" % bits
        assert np.array_equal(y, G.quantise_pm(x, dt, N, Cn, S, bits)), "reference != library (MX-fp%d)" % bits
        back = np.zeros(N * Cn * S, np.float32)
        assert r.refgpu_mx_to_f32(bits, y.ctypes.data, N, Cn, S, back.ctypes.data) == 0
        assert np.array_equal(back, orc.mx_to_pm(y, bits, N, Cn, S), equal_nan=True)
        assert np.array_equal(back, G.dequantise(y, bits, N, Cn, S), equal_nan=True)


def run_ref_conv(r, bits, k, s, p, w, b, Co, Ci, x16, N, D, H, W, want_st=False):
    Do, Ho, Wo = (D + 2 * p - k) // s + 1, (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
    y = np.zeros(N * Do * Ho * Wo * Co, np.float16)
    st = np.zeros(N * Co * 2, np.float64) if want_st else None
    r.refgpu_set_fq(bits, bits)
    assert r.refgpu_init(0) == 0
    w = np.ascontiguousarray(w, np.float32)
    rc = r.refgpu_conv(w.ctypes.data, b.ctypes.data if b is not None else None, Co, Ci, k, s, p, x16.ctypes.data, N, D, H, W, y.ctypes.data, st.ctypes.data if want_st else None)
    assert rc == 0
    return y, st


@pytest.mark.gpu
def test_reference_emulated_mx_conv_config1(dev):
    """Configuration 1 (1 x 32 x 64^3 fp16 N(0,1), 3^3 conv 32 -> 32, MX-fp8, fp16 bias and output) on the reference's emulated-MX conv,
    the oracle and the library's lp_conv_fwd_f8."""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp, Split
    r = ref()
    N, Cn, D = 1, 32, 64
    S = D ** 3
    x_pm = synth.act_h16(1, N * Cn * S)                                          # plane-major [n][c][voxel]
    w = synth.kaiming(2, Cn, Cn, 27).astype(np.float16).astype(np.float32)
    b = synth.bias(3, Cn).astype(np.float16).astype(np.float32)
    x_cl = np.ascontiguousarray(x_pm.reshape(N, Cn, S).transpose(0, 2, 1))       # channels last
    got_ref, st = run_ref_conv(r, 8, 3, 1, 1, w, b, Cn, Cn, x_cl, N, D, D, D, want_st=True)
    mx = orc.pm_to_mx(x_pm, 2, N, Cn, S, 8, 32)
    acc = orc.conv_blocked(orc.mx_to_blocked(mx, 8, N, Cn, S), N, Cn, D, D, D, orc.prep_w(w, Cn, Cn, 27, 8), b, Cn, 3, 1, 1)
    want = ndhwc(orc.round_h16(acc), N, Cn, S).ravel()
    e = orc.rel_l2(got_ref.astype(np.float32), want)
    same = np.mean(got_ref.astype(np.float32) == want)
    print("configuration 1, reference emulated MX-fp8 vs oracle: rel-L2 %.3g, %.4f of the fp16 outputs identical" % (e, same))
    assert e < TOL
    # the reference's own InstanceNorm sums (fp32 per thread, fp64 atomics) against the oracle's fp64 sums of the reference's stored values
    sums = orc.in_sums(to_blocked(got_ref.astype(np.float32), N, Cn, S), N, Cn, S)
    assert np.allclose(st, sums, rtol=1e-5, atol=1e-3)
    # the library through the reference's entry point, against the reference's output
    L = ufsm_b200.lib()
    xd, wd, bd = DevBuf(data=x_pm), DevBuf(data=w), DevBuf(data=b)
    yd = DevBuf(N * Cn * S * 2).fill(0xEE)
    assert L.lp_conv_fwd_f8(xd.ptr, 2, Shape5(N, Cn, D, D, D), wd.ptr, bd.ptr, Cn, yd.ptr, 2, Gnp(), None, 0, Split()) == 0
    ufsm_b200.check()
    got_lib = yd.download(np.float16).reshape(N, Cn, S).transpose(0, 2, 1).astype(np.float32).ravel()
    e2 = orc.rel_l2(got_lib, got_ref.astype(np.float32))
    print("configuration 1, library vs reference emulated MX-fp8: rel-L2 %.3g" % e2)
    assert e2 < TOL


@pytest.mark.gpu
def test_reference_emulated_mx_conv_config2(dev):
    """Configuration 2's layer pair in MX-fp4 on a 1 x 64 x 48^3 input (an eighth of the benchmark's volume: the reference's fp16 conv
    is slow): the 2^3 stride-2 conv 64 -> 128 and the transposed conv 128 -> 64, reference against oracle and library."""
    import gpu_util as G
    r = ref()
    N, Ci, Cm, D = 1, 64, 128, 48
    S, Sc = D ** 3, (D // 2) ** 3
    x_pm = synth.rng(201).standard_normal(N * Ci * S).astype(np.float16)
    w1, b1 = synth.kaiming(202, Cm, Ci, 8), synth.bias(203, Cm, 0.01)
    x_cl = np.ascontiguousarray(x_pm.reshape(N, Ci, S).transpose(0, 2, 1))
    got1, _ = run_ref_conv(r, 4, 2, 2, 0, w1, b1, Cm, Ci, x_cl, N, D, D, D)
    mxs, want1_pm = orc.conv_case("down2", x_pm.astype(np.float32), w1, b1, N, Ci, D, D, D, Cm, 4)
    want1 = orc.round_h16(want1_pm).reshape(N, Cm, Sc).transpose(0, 2, 1).ravel()
    e1 = orc.rel_l2(got1.astype(np.float32), want1)
    lib1 = G.run_pm32("down2", mxs, w1, b1, N, Ci, D, D, D, Cm, 4).astype(np.float16).astype(np.float32).reshape(N, Cm, Sc).transpose(0, 2, 1).ravel()
    e1l = orc.rel_l2(lib1, got1.astype(np.float32))
    # the transposed conv on the reference's fp16 result, without a bias (the reference's unfused path rounds before it adds the bias)
    w2 = synth.kaiming(204, Ci, Cm, 8, transposed=True)
    y16 = got1                                                                   # [n][voxel][Cm] fp16
    r.refgpu_set_fq(4, 4)
    got2 = np.zeros(N * S * Ci, np.float16)
    assert r.refgpu_tconv3(np.ascontiguousarray(w2).ctypes.data, None, Cm, Ci, y16.ctypes.data, N, D // 2, D // 2, D // 2, got2.ctypes.data) == 0
    y_pm = np.ascontiguousarray(y16.reshape(N, Sc, Cm).transpose(0, 2, 1)).astype(np.float32).ravel()
    mx2, want2_pm = orc.conv_case("tconv2", y_pm, w2, None, N, Cm, D // 2, D // 2, D // 2, Ci, 4)
    want2 = orc.round_h16(want2_pm).reshape(N, Ci, S).transpose(0, 2, 1).ravel()
    e2 = orc.rel_l2(got2.astype(np.float32), want2)
    lib2 = G.run_pm32("tconv2", mx2, w2, None, N, Cm, D // 2, D // 2, D // 2, Ci, 4).astype(np.float16).astype(np.float32).reshape(N, Ci, S).transpose(0, 2, 1).ravel()
    e2l = orc.rel_l2(lib2, got2.astype(np.float32))
    print("configuration 2 (48^3), reference emulated MX-fp4: down vs oracle %.3g, vs library %.3g; up vs oracle %.3g, vs library %.3g" % (e1, e1l, e2, e2l))
    assert max(e1, e1l, e2, e2l) < TOL


@pytest.mark.gpu
def test_reference_instance_norm_kernels_bit_for_bit(dev):
    """k_in_coef and k_inq of the reference (from the oracle's fp64 sums of a stored fp16 tensor) against orc_in_coef / orc_in_apply: the
    coefficients' float bits and the fp16 outputs must be identical (this settles how the reference's a * x + b and beta - mean * a
    are contracted by its compiler)."""
    r = ref()
    N, Cn, S = 2, 64, 5000
    g = synth.rng(77)
    y = (g.standard_normal((N, S, Cn)) * g.uniform(0.2, 3.0, Cn) + g.uniform(-1, 1, Cn)).astype(np.float16)
    gamma = (1 + 0.3 * g.standard_normal(Cn)).astype(np.float32)
    beta = (0.2 * g.standard_normal(Cn)).astype(np.float32)
    yb = to_blocked(y.astype(np.float32), N, Cn, S)
    sums = orc.in_sums(yb, N, Cn, S)
    coef_o = np.zeros(N * Cn * 2, np.float32)
    orc.o().orc_in_coef(sums.ctypes.data_as(C.c_void_p), N, Cn, C.c_double(S), gamma.ctypes.data_as(C.c_void_p), beta.ctypes.data_as(C.c_void_p), C.c_float(1e-5), coef_o.ctypes.data_as(C.c_void_p))
    want = ndhwc(orc.in_apply(yb, coef_o, N, Cn, S, 2), N, Cn, S)
    assert r.refgpu_init(0) == 0
    coef_r = np.zeros(N * Cn * 2, np.float32)
    out = y.copy()
    assert r.refgpu_in(sums.ctypes.data, N, Cn, S, gamma.ctypes.data, beta.ctypes.data, C.c_float(1e-5), coef_r.ctypes.data, out.ctypes.data, 2) == 0
    assert np.array_equal(coef_r.view(np.uint32), coef_o.view(np.uint32)), "%d coefficients differ" % np.count_nonzero(coef_r != coef_o)
    assert np.array_equal(out.astype(np.float32), want), "%d outputs differ" % np.count_nonzero(out.astype(np.float32) != want)
