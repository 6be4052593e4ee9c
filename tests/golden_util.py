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
    if "cfg_json" in blob:  # newer cases carry their model configuration
        import json
        cfg = json.loads(str(blob["cfg_json"]))
        for st in cfg["statistics"]:  # JSON turned the integer keys of the per-element tables into strings
            for key in ("atomic_energy", "rms_forces"):
                st[key] = {int(k): v for k, v in st[key].items()}
    else:
        cfg = synth.model_config(2, 32, float(blob["cutoff"]), [29], float(blob["avg_num_neighbors"]))
    structure = synth.Structure(positions=blob["positions"], atomic_numbers=blob["atomic_numbers"], cell=blob["cell"],
                                pbc=(True, True, True))
    return blob, sd, cfg, structure
