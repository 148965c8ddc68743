"""Shared helpers for the test-suite: golden-fixture loading and the parity metrics."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def load_golden(name):
    """Load a fixture written by tests/golden/make_golden.py. 16-bit float tensors were stored as
    raw int16 bit patterns; ``dtype_of`` maps array name -> torch dtype for those."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: z[k] for k in z.files}


def unpack(arr, dtype):
    t = torch.from_numpy(np.ascontiguousarray(arr))
    if t.dtype == torch.int16:
        return t.view(dtype)
    return t


def cos_sim(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-300))


def rel_l1(a, b):
    """sum|a-b| / sum|b| (b is the reference)."""
    a, b = a.double(), b.double()
    return float((a - b).abs().sum() / (b.abs().sum() + 1e-300))


def assert_close_parity(got, ref, cos_min=0.999, l1_max=1e-2, what=""):
    if float(ref.double().abs().max()) == 0.0:      # an all-zero reference: cosine is undefined, the result must be zero too
        assert float(got.double().abs().max()) <= 1e-30, f"{what}: reference is zero, result is not"
        return 1.0, 0.0
    c, l = cos_sim(got, ref), rel_l1(got, ref)
    assert c >= cos_min and l <= l1_max, f"{what}: cos={c:.6f} (>= {cos_min}), relL1={l:.3e} (<= {l1_max})"
    return c, l
