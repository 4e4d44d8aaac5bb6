"""Shared helpers for the tests: golden fixtures, model construction, parity metric."""
import json
import os

import numpy as np

from lumi_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ["tiny_mamba", "tiny_hybrid", "tiny_hybrid_ext", "tiny_bytelevel"]


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = synth.tiny_config(**json.loads(str(z["cfg"])))
    tens = list(synth.iter_tensors(cfg, seed=int(z["seed"]), perturb_ones=float(z["perturb"])))
    return z, cfg, tens


def rel_err(got, ref):
    """The parity metric: max_i |g_i - r_i| / max_i |r_i|."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def top2_margin(logits):
    s = np.sort(np.asarray(logits, dtype=np.float64))
    return float(s[-1] - s[-2])
