"""Loader for tests/golden/*.npz (see tests/golden/make_golden.py for the format)."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name: str) -> dict:
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if k.endswith("__bf16"):
            out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.bfloat16)
        elif k.endswith("__e4m3"):
            out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)
        elif a.ndim == 0:
            out[k] = a.item()
        else:
            out[k] = torch.from_numpy(a.copy())
    return out
