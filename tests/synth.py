"""The seeded synthetic inputs of the package under the name the tests use."""
from ufsm_b200.synth import *  # noqa: F401,F403
