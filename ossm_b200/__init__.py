"""ossm_b200 -- B200-native (sm_100a) recurrent scans behind ossm's op signatures."""
from . import kernels  # noqa: F401

__all__ = ["kernels"]
