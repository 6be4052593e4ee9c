"""Batch construction: structures -> the ``data`` dictionary ``TensorModel.forward`` consumes
(the role of ``from_atoms`` + PyG collation in the reference, ``tace/dataset/graph.py:36-161``,
``tace/interface/ase/calculator.py:132-152``), with the neighbour list built on the device."""

from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch

from .neighbour_list import complete_cell, neighbor_list_batch


def z_to_index(atomic_numbers: Sequence[int], model_numbers: Sequence[int]) -> np.ndarray:
    """tace/dataset/element.py:41-61 (TorchElement.z2idx): position of each Z in the sorted element list."""
    table = np.full(max(max(model_numbers), int(np.max(atomic_numbers))) + 1, -1, dtype=np.int64)
    for i, z in enumerate(sorted(model_numbers)):
        table[z] = i
    idx = table[np.asarray(atomic_numbers, dtype=np.int64)]
    if (idx < 0).any():
        raise ValueError("structure contains an element the model was not built for")
    return idx


def build_batch(batch: Dict[str, np.ndarray], model_numbers: Sequence[int], cutoff: float, dtype: torch.dtype,
                device: torch.device) -> Dict[str, torch.Tensor]:
    """``batch`` as returned by ``tace_b200.synth.collate`` (host arrays).  Uploads the structure,
    builds the neighbour list on ``device`` and returns the model input dictionary."""
    n_el = len(model_numbers)
    pos64 = torch.as_tensor(batch["positions"], dtype=torch.float64).to(device)
    cells = np.stack([complete_cell(c, batch["positions"][a:b], p, cutoff)
                      for c, p, a, b in zip(batch["lattice"], batch["pbc"], batch["ptr"][:-1], batch["ptr"][1:])])
    lat64 = torch.as_tensor(cells, dtype=torch.float64).to(device)
    ptr = torch.as_tensor(batch["ptr"], dtype=torch.int64).to(device)
    pbc = torch.as_tensor(np.asarray(batch["pbc"], dtype=np.uint8)).to(device)
    edge_index, shifts = neighbor_list_batch(pos64, lat64, pbc, ptr.to(torch.int32), cutoff)
    species = torch.as_tensor(z_to_index(batch["atomic_numbers"], model_numbers)).to(device)
    return {
        "positions": pos64.to(dtype),
        "lattice": torch.as_tensor(batch["lattice"], dtype=torch.float64).to(device).to(dtype),
        "node_attrs": torch.nn.functional.one_hot(species, n_el).to(dtype),
        "species": species.to(torch.int32),
        "edge_index": edge_index,
        "edge_shifts": shifts.to(dtype),
        "batch": torch.as_tensor(batch["batch"], dtype=torch.int64).to(device),
        "ptr": ptr,
    }
