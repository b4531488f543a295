"""deepstrix_b200 -- B200 (sm_100a) routed-MoE path for deepstrix.

The package is a thin Python mirror of the C ABI in ``include/dsx_moe.h``
(``libdsx_moe.so``, built in-tree by ``deepstrix_b200._build``).  There is no
fallback: importing :mod:`deepstrix_b200.moe` raises if the library is missing.
"""
from .config import MoeConfig, RouterConfig, CONFIGS, FMT_MXFP4, FMT_Q8_0, SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS  # noqa: F401

__all__ = ["MoeConfig", "RouterConfig", "CONFIGS", "FMT_MXFP4", "FMT_Q8_0", "SCORE_SIGMOID", "SCORE_SQRT_SOFTPLUS"]
