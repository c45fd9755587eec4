"""The numpy-facing wrappers of the package under the name the tests use."""
from ufsm_b200.npapi import *  # noqa: F401,F403
from ufsm_b200.npapi import L, Conv, Unet, make_cfg  # noqa: F401
