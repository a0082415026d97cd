"""Loader for the golden vectors produced by tests/golden/make_moe_block_golden.py from the
reference's f64 NumPy implementation of one qwen3moe block."""
import glob
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# The reference's own comparator limits (tools/compare_block.py:14-18): expert selections
# exact, routing weights max-abs 1e-6, hidden state rel-L2 1e-6.
ROUTING_MAX_ABS = 1e-6
HIDDEN_REL_L2 = 1e-6


def names():
    return sorted(os.path.splitext(os.path.basename(p))[0] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    return {k: z[k] for k in z.files}


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.sqrt(((got - want) ** 2).sum()) / np.sqrt((want ** 2).sum()))
