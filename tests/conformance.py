"""The checks live in the package (``python -m pytorches_b200.conformance``); tests import them from here."""

from pytorches_b200.conformance import *  # noqa: F401,F403
from pytorches_b200.conformance import ALL_CHECKS, edge_values, f32_bits  # noqa: F401
