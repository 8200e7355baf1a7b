"""The helpers live in the package (the conformance tool uses them too); tests import them from here."""

from pytorches_b200.harness import *  # noqa: F401,F403
from pytorches_b200.harness import Buf, assert_bit_equal, bits, close, exec_op, lcg_data, strided_view_numpy, ulp_distance  # noqa: F401
