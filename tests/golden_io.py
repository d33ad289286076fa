"""Loader for the fixtures under tests/golden/ (written by tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    """Returns {key: torch tensor or python int}; bf16 / e4m3 payloads get their dtype back."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for key in z.files:
        a = z[key]
        if key.endswith("::bf16"):
            out[key[:-6]] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        elif key.endswith("::e4m3"):
            out[key[:-6]] = torch.from_numpy(a.copy())          # raw bytes (uint8)
        elif a.ndim == 0:
            out[key] = a.item()
        else:
            out[key] = torch.from_numpy(a.copy())
    return out


def names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))
