"""Loader for the golden fixtures written by tests/golden/make_golden.py."""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.dirname(HERE))

from make_golden import CASES, build_case  # noqa: E402  (the generator's own case table)

ALL_CASES = list(CASES)
F32_CASES = [n for n in ALL_CASES if CASES[n][3] == "float32"]
BF16_CASES = [n for n in ALL_CASES if CASES[n][3] == "bfloat16"]


def _sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def load_case(name):
    """Returns (shape, x, factors, dtype, golden) with inputs verified against the stored hashes."""
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    shape, x, f, dtype, _ = build_case(name)
    assert _sha(x) == str(z["sha_x"]), f"{name}: regenerated x differs from the fixture's input"
    for k, v in f.items():
        assert _sha(v) == str(z["sha_" + k]), f"{name}: regenerated factor {k} differs from the fixture's"
    if "x" in z.files:
        assert torch.equal(x.float(), torch.from_numpy(z["x"]).reshape(x.shape))
    golden = {
        "y": torch.from_numpy(z["y"]), "scores": torch.from_numpy(z["scores"]),
        "idx": torch.from_numpy(z["idx"]), "gates": torch.from_numpy(z["gates"]),
    }
    return shape, x, f, dtype, golden
