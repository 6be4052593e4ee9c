"""Loads the golden model case (tests/golden/case_fcc32_L2_C32.npz)."""
import os

import numpy as np
import torch

from tace_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_case(name="case_fcc32_L2_C32.npz"):
    blob = dict(np.load(os.path.join(GOLDEN, name)))
    sd = {k[3:]: torch.from_numpy(v.astype(np.float64) if v.dtype == np.float32 else v)
          for k, v in blob.items() if k.startswith("sd:")}
    cfg = synth.model_config(2, 32, float(blob["cutoff"]), [29], float(blob["avg_num_neighbors"]))
    structure = synth.Structure(positions=blob["positions"], atomic_numbers=blob["atomic_numbers"], cell=blob["cell"],
                                pbc=(True, True, True))
    return blob, sd, cfg, structure
