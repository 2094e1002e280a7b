"""Shared helpers for the test-suite: golden-fixture loading and tolerances."""
from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = ["normal_s256_d64", "normal_s200_d128", "clustered_s512_d128", "clustered_s389_d64"]

# Output tolerance for bf16 inputs with fp32 accumulation (max-abs, mean-abs).
OUT_MAX_ABS = 2e-2
OUT_MEAN_ABS = 2e-3
# Mask entries whose score lies within this relative distance of tau may differ.
TAU_REL = 1e-3


def load_golden(name):
    z = np.load(GOLDEN / f"{name}.npz")
    d = {k: z[k] for k in z.files}
    for t in ("q", "k", "v"):
        bits = torch.from_numpy(d.pop(f"{t}_bf16").copy())
        d[t] = bits.view(torch.bfloat16)
    d["tau"] = float(d["tau"])
    return d


def unpack_bitmask(packed, n):
    return torch.from_numpy(np.unpackbits(packed, axis=-1)[..., :n].astype(bool))
