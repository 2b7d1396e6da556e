"""Access to the committed golden vectors (tests/golden/*.npz)."""
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN_DIR, f"ops_{name}.npz"))
