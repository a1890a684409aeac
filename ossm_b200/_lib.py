"""ctypes binding of ``libossm_b200.so`` (the C ABI declared in ``include/ossm_b200.h``).

There is no fallback: if the shared library is missing the import of any op
raises, so a GPU run can never silently take another path.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("OSSM_B200_LIB") or os.path.join(_PKG, "libossm_b200.so")

_lib = None

# name -> (restype, argtypes); kept in one table so a test can check that every
# symbol of the header is exported and bound.
SIGNATURES = {
    "ossm_b200_version": (c_int, []),
    "ossm_b200_last_error": (c_char_p, []),
    "ossm_b200_device_status": (c_int, [POINTER(c_int), c_int]),
    "ossm_b200_selftest_wait_timeout": (c_int, [ctypes.c_uint64, c_void_p, c_void_p]),
    "ossm_b200_lti_chunk": (c_int, []),
    "ossm_b200_lti_carry_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "ossm_b200_lti_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "ossm_b200_lti_forward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "ossm_b200_lti_scan_forward_ws": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_scan_forward": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_scan_backward": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                            c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_scan_forward_slice": (c_int, [c_int] + [c_void_p] * 8 + [c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_scan_backward_slice": (c_int, [c_int] + [c_void_p] * 14 + [c_size_t, c_int64, c_int64, c_int64,
                                                                             c_void_p]),
    "ossm_b200_lti_scan_backward_states": (c_int, [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_size_t, c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_scan_backward_static_max_series": (c_size_t, []),
    "ossm_b200_lti_scan_backward_static": (c_int, [c_int] + [c_void_p] * 10 + [c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_lti_set_tuning": (c_int, [c_char_p, c_int]),
    "ossm_b200_selective_scan_chunk": (c_int, [c_int64]),
    "ossm_b200_selective_scan_state_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "ossm_b200_selective_scan_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int64]),
    "ossm_b200_selective_scan_forward": (c_int, [c_void_p] * 8 + [c_int] + [c_void_p] * 2 + [c_int64] * 4
                                         + [c_int, c_void_p]),
    "ossm_b200_selective_scan_backward": (c_int, [c_void_p] * 8 + [c_int] + [c_void_p] * 11 + [c_size_t]
                                          + [c_int64] * 4 + [c_int, c_void_p]),
    "ossm_b200_selective_scan_step_major_bc": (c_int, [c_int64]),
    "ossm_b200_selective_scan_forward_step_major_bc": (c_int, [c_void_p] * 8 + [c_int] + [c_void_p] * 2 + [c_int64] * 5
                                                       + [c_int, c_void_p]),
    "ossm_b200_selective_scan_backward_step_major_bc": (c_int, [c_void_p] * 8 + [c_int] + [c_void_p] * 11 + [c_size_t]
                                                        + [c_int64] * 5 + [c_int, c_void_p]),
    "ossm_b200_split_tf32": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "ossm_b200_gemm_tf32x3": (c_int, [c_void_p] * 6 + [c_int64] * 6 + [c_int, c_int64, c_int64, c_void_p]),
    "ossm_b200_wgrad_tf32x3_workspace_bytes": (c_size_t, [c_int64] * 4),
    "ossm_b200_wgrad_tf32x3": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_size_t, POINTER(c_int)]
                               + [c_int64] * 4 + [c_void_p]),
    "ossm_b200_layer_set_tuning": (c_int, [c_char_p, c_int]),
    "ossm_b200_colwise_dot_partials": (c_int, [c_int64]),
    "ossm_b200_colwise_dot": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "ossm_b200_conv1d_silu_forward": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                              c_int64, c_int, c_void_p]),
    "ossm_b200_conv1d_silu_backward": (c_int, [c_void_p, c_int64] + [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_int,
                                                                                     c_void_p]),
    "ossm_b200_linoss_scan_forward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_linoss_scan_backward_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "ossm_b200_linoss_scan_backward": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_size_t, c_int64, c_int64, c_int64,
                                               c_void_p]),
    "ossm_b200_sdlinoss_forward": (c_int, [c_int, c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p,
                                           POINTER(c_int64), c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                           c_int64, c_int64, c_void_p]),
    "ossm_b200_sdlinoss_backward": (c_int, [c_int, c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p,
                                            POINTER(c_int64), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "ossm_b200_sdlinoss_set_tuning": (c_int, [c_char_p, c_int]),
    "ossm_b200_selective_scan_set_tuning": (c_int, [c_char_p, c_int]),
    "ossm_b200_sdlinoss_carry_interval": (c_int, []),
    "ossm_b200_sdlinoss_carry_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
}


def load():
    """Returns the loaded library, loading it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        # a source checkout without the built library: compile it once (needs nvcc); anything
        # else is an error -- there is no CPU or PyTorch fallback to take instead
        try:
            from . import build as _build

            _build.build()
        except Exception as exc:
            raise RuntimeError(
                f"ossm_b200: {LIB_PATH} is missing and could not be built ({exc}); build it with "
                "`python -m ossm_b200.build` (there is no CPU or PyTorch fallback)") from exc
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    """Raises ``RuntimeError`` (what the reference's TORCH_CHECK surfaces as) on a non-zero return code."""
    if rc != 0:
        msg = load().ossm_b200_last_error()
        raise RuntimeError(f"ossm_b200 {what} failed ({rc}): {msg.decode() if msg else 'unknown error'}")


def device_status(clear: bool = True) -> int:
    out = c_int(0)
    check(load().ossm_b200_device_status(ctypes.byref(out), 1 if clear else 0), "device_status")
    return out.value
