"""Loader for the committed golden fixtures (produced by make_golden.py from the reference's CPU code)."""
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def load(name: str = "reference_cpu.npz") -> dict:
    """Return {case: {field: ndarray}}; ``:bf16`` fields are widened back to float32."""
    raw = np.load(os.path.join(_HERE, name))
    cases: dict = {}
    for key in raw.files:
        case, field = key.split(".", 1)
        val = raw[key]
        if field.endswith(":bf16"):
            field = field[: -len(":bf16")]
            val = (val.astype(np.uint32) << 16).view(np.float32)
        cases.setdefault(case, {})[field] = val
    return cases
