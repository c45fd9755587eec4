"""ctypes declarations for every entry point of include/ufsm_mx.h."""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("UFSM_MX_LIB") or os.path.join(HERE, "libufsm_mx.so")     # UFSM_MX_LIB: another build of the library (e.g. one with the kernels' cycle counters)


class Shape5(C.Structure):
    _fields_ = [("n", C.c_int), ("c", C.c_int), ("d", C.c_int), ("h", C.c_int), ("w", C.c_int)]


class Gnp(C.Structure):
    _fields_ = [("gamma", C.c_void_p), ("beta", C.c_void_p), ("mean", C.c_void_p), ("rstd", C.c_void_p), ("G", C.c_int),
                ("zs", C.c_int), ("zo", C.c_int), ("ns", C.c_int), ("zhw", C.c_int)]


class Split(C.Structure):
    _fields_ = [("x2", C.c_void_p), ("c_split", C.c_int), ("y2", C.c_void_p), ("o_split", C.c_int), ("accum", C.c_int), ("gp2", Gnp),
                ("up", C.c_int16), ("yD", C.c_int16), ("sr", C.c_uint), ("wkey", C.c_uint), ("zlo", C.c_int), ("zhi", C.c_int),
                ("stored_stats", C.c_int), ("osr", C.c_uint), ("zi0", C.c_int16), ("Di", C.c_int16), ("o_pad", C.c_int16),
                ("zw0", C.c_int16), ("zw1", C.c_int16), ("yzo", C.c_int16)]


class Feather(C.Structure):
    _fields_ = [("S", C.c_int), ("B", C.c_int), ("e", C.c_void_p), ("nb", C.c_void_p * 8), ("oo", C.c_int * 3), ("on", C.c_int * 3), ("osh", C.c_int), ("out", C.c_void_p)]


class UnetCfg(C.Structure):
    _fields_ = [("L", C.c_int), ("cw", C.c_int * 8), ("nh", C.c_int), ("P", C.c_int), ("bits_first", C.c_int), ("bits_mid", C.c_int), ("bits_last", C.c_int)]


class Window(C.Structure):
    _fields_ = [("V", C.c_int), ("P", C.c_int), ("overlap", C.c_int), ("nper", C.c_int), ("npatch", C.c_int)]


_SIG = {
    "nn_init": (C.c_int, [C.c_int]),
    "nn_malloc": (C.c_void_p, [C.c_size_t]),
    "nn_free": (None, [C.c_void_p]),
    "nn_zero": (None, [C.c_void_p, C.c_size_t]),
    "nn_h2d": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "nn_d2h": (None, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "nn_sync": (None, []),
    "nn_check": (C.c_char_p, []),
    "lp_check": (C.c_char_p, []),
    "nn_malloc_host": (C.c_void_p, [C.c_size_t]),
    "nn_free_host": (None, [C.c_void_p]),
    "umx_timer_new": (C.c_void_p, []),
    "umx_timer_start": (None, [C.c_void_p]),
    "umx_timer_stop_ms": (C.c_float, [C.c_void_p]),
    "umx_timer_mark": (None, [C.c_void_p]),
    "umx_timer_read_ms": (C.c_float, [C.c_void_p]),
    "umx_timer_free": (None, [C.c_void_p]),
    "umx_prof_begin": (None, []),
    "umx_prof_end": (C.c_int, [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "umx_prof_get": (C.c_int, [C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "lp_mx8_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_size_t]),
    "lp_gn_silu_apply_mx": (None, [C.c_void_p, C.c_int, Shape5, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "lp_up2_fwd_mx": (None, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_int, Gnp]),
    "lp_conv1_fwd_mx": (None, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, Gnp]),
    "lp_conv1_fwd_mx_h16": (None, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, Gnp]),
    "lp_conv1_fwd_mx_h16_r": (None, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, Gnp, C.c_size_t, C.c_size_t]),
    "lp_conv1_fwd_mx_r": (C.c_int, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, Gnp, C.c_size_t, C.c_size_t, C.c_size_t]),
    "lp_up2_fwd_mx_blocks": (None, [C.c_void_p, C.c_int, Shape5, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "lp_add_mx": (None, [C.c_void_p, C.c_void_p, Shape5, C.c_int, C.c_uint]),
    "lp_gn_sums_mx": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t]),
    "lp_gn_sums_mx_n": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_int]),
    "umx_gn_finalize": (None, [C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_void_p, C.c_void_p]),
    "lp_mx4_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_size_t]),
    "lp_f32_to_mx8": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_f32_to_mx4": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_h16_to_mx8": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_h16_to_mx4": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_mx8_to_f32": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_mx4_to_f32": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "umx_mx_bytes32": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_size_t]),
    "umx_pm_to_mx32": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int, C.c_int]),
    "umx_mx_rewidth": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int]),
    "lp_pred_input_mx": (None, [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int]),
    "lp_pred_input_mx8": (None, [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "umx_pm_to_mx32_cat": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int, C.c_int]),
    "umx_mx_relayout": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int]),
    "umx_mx32_to_f32": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int]),
    "umx_h16b_to_f32": (None, [C.c_void_p, C.c_int, C.c_int, C.c_size_t, C.c_void_p]),
    "lp_conv_fwd_f8": (C.c_int, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, Gnp, C.c_void_p, C.c_int, Split]),
    "lp_conv_fwd_s2_f8": (C.c_int, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, Shape5, Gnp]),
    "lp_conv_fwd_f4": (C.c_int, [C.c_void_p, C.c_int, Shape5, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, Gnp, C.c_void_p, C.c_int, Split]),
    "lp_wmemo_clear": (None, []),
    "umx_conv_create": (C.c_void_p, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "umx_conv_create_dev": (C.c_void_p, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "umx_conv_free": (None, [C.c_void_p]),
    "umx_conv_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "umx_conv_fwd_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_int]),
    "umx_conv_r_block_cap": (None, [C.c_int]),
    "umx_conv_last_kernel": (C.c_int, []),
    "umx_stats_doubles": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "umx_in_coef": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]),
    "umx_in_stats_coef": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]),
    "umx_in_coef_static": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]),
    "umx_in_apply": (None, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "umx_unet_nweights": (C.c_size_t, [C.POINTER(UnetCfg)]),
    "umx_unet_create": (C.c_void_p, [C.POINTER(UnetCfg), C.c_void_p, C.c_int]),
    "umx_unet_free": (None, [C.c_void_p]),
    "umx_unet_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umx_unet_forward_h16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umx_unet_forward_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umx_unet_submit_host_u8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umx_h16_to_prob_u8": (None, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "umx_feather_blend": (C.c_int, [C.POINTER(Feather)]),
    "umx_feather_keep": (None, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "nn_set_logits_h16": (None, [C.c_int]),
    "nn_set_pred_iso": (None, [C.c_int]),
    "nn_get_pred_iso": (C.c_int, []),
    "nn_pred_output": (None, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "nn_pred_place": (None, [C.c_void_p, C.c_void_p] + [C.c_int] * 9 + [C.c_void_p]),
    "nn_pred_place_d": (None, [C.c_void_p, C.c_void_p] + [C.c_int] * 11 + [C.c_void_p]),
    "nn_pred_ctmask": (None, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "nn_pred_ctmask_t": (None, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]),
    "nn_pred_place_m": (None, [C.c_void_p, C.c_void_p] + [C.c_int] * 9 + [C.c_void_p]),
    "nn_pred_place_m_d": (None, [C.c_void_p, C.c_void_p] + [C.c_int] * 11 + [C.c_void_p]),
    "nn_pred_place_mz": (None, [C.c_void_p, C.c_void_p] + [C.c_int] * 12 + [C.c_void_p]),
    "umx_unet_submit_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "umx_unet_wait": (C.c_int, [C.c_void_p]),
    "umx_wait_selftest": (C.c_int, [C.c_longlong]),
    "umx_stream_new": (C.c_void_p, []),
    "umx_stream_free": (None, [C.c_void_p]),
    "umx_event_new": (C.c_void_p, []),
    "umx_event_free": (None, [C.c_void_p]),
    "umx_event_record": (None, [C.c_void_p, C.c_void_p]),
    "umx_stream_wait": (None, [C.c_void_p, C.c_void_p]),
    "umx_stream_sync": (None, [C.c_void_p]),
    "umx_event_sync": (None, [C.c_void_p]),
    "umx_copy2d_async": (None, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p]),
    "umx_copy_async": (None, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "umx_unet_flops": (C.c_double, [C.POINTER(UnetCfg)]),
    "umx_unet_launches": (C.c_long, [C.c_void_p]),
    "umx_launch_count": (C.c_long, []),
    "umx_u8_to_h16": (None, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "umx_blend_add": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umx_window_make": (Window, [C.c_int, C.c_int, C.c_int]),
    "umx_window_share": (None, [C.POINTER(Window), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "umx_window_origin": (None, [C.POINTER(Window), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "umx_window_extent": (None, [C.POINTER(Window), C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "umx_wplan_create": (C.c_void_p, [C.POINTER(Window), C.c_int, C.c_int, C.c_int]),
    "umx_wplan_free": (None, [C.c_void_p]),
    "umx_wplan_info": (None, [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "umx_wplan_rows": (C.c_long, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "umx_wplan_mode": (None, [C.c_void_p, C.c_void_p]),
    "umx_wplan_row_bytes": (C.c_size_t, [C.c_void_p]),
    "umx_wplan_prepare": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "umx_window_run_fx": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "umx_wplan_pack": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "umx_wplan_add": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "umx_wplan_finish": (C.c_int, [C.c_void_p, C.c_void_p]),
    "umx_blend_add_fx": (None, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "umx_emit_fx": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "umx_emit_rows_fx": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "umx_rows_fx": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
}
SYMBOLS = tuple(_SIG)
_lib = None


def lib():
    """The loaded library with argument types set; raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("libufsm_mx.so is missing: run `python -c 'import __graft_entry__ as g; g.build()'` (there is no fallback path)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIG.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check():
    """Synchronise, then raise when the library latched an error."""
    L = lib()
    L.nn_sync()
    e = L.lp_check()
    if e:
        raise RuntimeError(e.decode())


class DevBuf:
    """Device memory owned through nn_malloc / nn_free, with numpy upload / download."""

    def __init__(self, nbytes=None, data=None):
        L = lib()
        if data is not None:
            data = np.ascontiguousarray(data)
            nbytes = data.nbytes
        self.nbytes = int(nbytes)
        self.ptr = L.nn_malloc(self.nbytes)
        if not self.ptr:
            raise RuntimeError("nn_malloc(%d) failed: %s" % (self.nbytes, (L.lp_check() or b"").decode()))
        if data is not None:
            L.nn_h2d(self.ptr, data.ctypes.data, self.nbytes)

    def zero(self):
        lib().nn_zero(self.ptr, self.nbytes)
        return self

    def fill(self, byte):
        self.upload(np.full(self.nbytes, byte, np.uint8))
        return self

    def upload(self, data):
        data = np.ascontiguousarray(data)
        assert data.nbytes <= self.nbytes
        lib().nn_h2d(self.ptr, data.ctypes.data, data.nbytes)

    def download(self, dtype=np.uint8, count=None):
        dtype = np.dtype(dtype)
        n = self.nbytes // dtype.itemsize if count is None else count
        out = np.empty(n, dtype)
        lib().nn_d2h(out.ctypes.data, self.ptr, n * dtype.itemsize)
        return out

    def free(self):
        if self.ptr:
            lib().nn_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
