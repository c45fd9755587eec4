"""ufsm_b200: ctypes access to libufsm_mx.so, the B200 (sm_100a) implementation of ufsm's MX block-scaled 3-D conv forward path.

The product is the C-ABI shared library (include/ufsm_mx.h); this package only loads it for the tests, the smoke test and the
benchmark.  There is no fallback: a missing library raises."""
from ._lib import lib, LIB_PATH, Shape5, Gnp, Split, Feather, UnetCfg, Window, DevBuf, check  # noqa: F401
