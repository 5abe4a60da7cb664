"""Loader for the fixtures under tests/golden (written by tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class Golden:
    def __init__(self, name):
        self._z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))

    def keys(self):
        return [k[:-6] if k.endswith("__bf16") else k for k in self._z.files]

    def __contains__(self, k):
        return k in self._z.files or (k + "__bf16") in self._z.files

    def __getitem__(self, k) -> torch.Tensor:
        if (k + "__bf16") in self._z.files:
            bits = self._z[k + "__bf16"]
            return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)
        a = self._z[k]
        if a.dtype.kind in "US":
            return a
        return torch.from_numpy(np.array(a))

    def scalar(self, k):
        return self._z[k].item()


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / max(|b|, tiny) over the tensor (the parity metric used for float outputs)."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    den = max(float(b.abs().max()), 1e-30)
    return float((a - b).abs().max()) / den
