"""Default hyper-parameters, with the reference's values (quashkv/constants.py:15-26)."""

import math

SUPPORTED_BITS = {1, 2, 3, 4}
DEFAULT_TOTAL_BITS = 3          # keys: 2-bit codes + 1 sign bit; values: 3-bit codes
DEFAULT_SEED = 42
QJL_COEFF = math.sqrt(math.pi / 2)
LLOYD_MAX_ITER = 300
LLOYD_MAX_TOL = 1e-12
LLOYD_MAX_RANGE_SIGMAS = 4.0
