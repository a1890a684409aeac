"""Optional record of the errors the parity tests measure.

With ``OSSM_B200_PARITY_REPORT=<file>`` every call of :func:`record` appends one JSON line
(case, tensor, measured max-norm relative error, asserted bound) to that file; without it
nothing is written.  The table of measured errors in the design notes is made from such a file.
"""
import json
import os


def record(case: str, tensor: str, err: float, bound: float) -> float:
    path = os.environ.get("OSSM_B200_PARITY_REPORT")
    if path:
        with open(path, "a") as fh:
            fh.write(json.dumps({"case": case, "tensor": tensor, "err": float(err), "bound": float(bound)}) + "\n")
    return err
