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
    """``batch`` as returned by ``tace_b200.synth.collate``: host numpy arrays or (pinned) CPU
    tensors; an optional ``species`` entry (index into the model's element list) replaces the
    lookup from ``atomic_numbers``.  Uploads the structure, builds the neighbour list on ``device``
    and returns the model input dictionary."""
    n_el = len(model_numbers)
    pbc_host = np.asarray(batch["pbc"], dtype=np.uint8)
    lattice_host = batch["lattice"]
    if pbc_host.all():
        cells = lattice_host  # fully periodic: the cell is used as given
    else:
        pos_np, lat_np, ptr_np = (np.asarray(batch[k]) for k in ("positions", "lattice", "ptr"))
        cells = np.stack([complete_cell(c, pos_np[a:b], p, cutoff)
                          for c, p, a, b in zip(lat_np, pbc_host, ptr_np[:-1], ptr_np[1:])])
    up = lambda x, dt: torch.as_tensor(x, dtype=dt).to(device, non_blocking=True)
    pos64 = up(batch["positions"], torch.float64)
    lat64 = up(cells, torch.float64)
    ptr = up(batch["ptr"], torch.int64)
    pbc = up(pbc_host, torch.uint8)
    edge_index, shifts = neighbor_list_batch(pos64, lat64, pbc, ptr.to(torch.int32), cutoff)
    if "species" in batch:
        species = up(batch["species"], torch.int64)
    else:
        species = up(z_to_index(np.asarray(batch["atomic_numbers"]), model_numbers), torch.int64)
    return {
        "positions": pos64.to(dtype),
        "lattice": up(lattice_host, torch.float64).to(dtype),
        "node_attrs": torch.nn.functional.one_hot(species, n_el).to(dtype),
        "species": species.to(torch.int32),
        "edge_index": edge_index,
        "edge_shifts": shifts.to(dtype),
        "batch": up(batch["batch"], torch.int64),
        "ptr": ptr,
    }
