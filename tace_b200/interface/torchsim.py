"""TorchSim entry point with the reference's ``TACETorchSimCalc`` contract
(``tace/interface/torchsim/torchsim.py:28-305``): ``forward(state)`` takes an object with
``positions [n,3]``, ``row_vector_cell [n_systems,3,3]``, ``pbc``, ``atomic_numbers [n]`` and
``system_idx [n]`` and returns ``energy [n_systems]``, ``forces [n,3]``, ``stress [n_systems,3,3]``.

The default ``neighbor_list_fn`` is this package's GPU cell list behind TorchSim's neighbour-list
signature ``(positions, cell, pbc, cutoff, system_idx) -> (edge_index, mapping_system, unit_shifts)``
(``torchsim.py:250-256``), so a batched-MD driver never leaves the device.  ``torch_sim`` itself is
optional: when it is installed the class derives from its ``ModelInterface``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Dict, List, Optional, Union

import torch

from ..graph import z_to_index  # noqa: F401  (re-exported for drivers that prepare species themselves)
from ..models import TensorModel
from ..neighbour_list import neighbor_list_batch
from .ase_calculator import load_tace

try:  # pragma: no cover - torch_sim is not part of the test environment
    from torch_sim.models.interface import ModelInterface as _Base
except ImportError:
    _Base = torch.nn.Module


def tace_b200_nl(positions: torch.Tensor, cell: torch.Tensor, pbc, cutoff: float, system_idx: torch.Tensor):
    """Neighbour list of a batch of systems on the GPU.  ``cell``: row vectors ``[n_systems,3,3]``; ``pbc``: one
    triple for all systems or ``[n_systems,3]``.  Atoms must be grouped by system (ascending ``system_idx``)."""
    n_systems = int(cell.reshape(-1, 3, 3).shape[0])
    counts = torch.bincount(system_idx, minlength=n_systems)
    ptr = torch.cat([counts.new_zeros(1), counts.cumsum(0)]).to(torch.int32)
    pbc_t = torch.as_tensor(pbc, device=positions.device).to(torch.uint8).reshape(-1, 3)
    if pbc_t.shape[0] == 1 and n_systems > 1:
        pbc_t = pbc_t.expand(n_systems, 3)
    edge_index, shifts = neighbor_list_batch(positions.to(torch.float64), cell.to(torch.float64), pbc_t.contiguous(), ptr, float(cutoff))
    mapping_system = system_idx[edge_index[0]]
    return edge_index, mapping_system, shifts


class TACETorchSimCalc(_Base):
    def __init__(self, model: Union[str, Path, TensorModel, None] = None, *, device: Optional[torch.device] = None,
                 dtype: torch.dtype = torch.float32, neighbor_list_fn: Optional[Callable] = None, compute_forces: bool = True,
                 compute_stress: bool = True, atomic_numbers: Optional[torch.Tensor] = None,
                 system_idx: Optional[torch.Tensor] = None, fidelity_idx: Optional[int] = None,
                 target_property: Optional[List[str]] = None, **unsupported) -> None:
        super().__init__()
        for key, value in unsupported.items():  # enable_oeq / enable_cue / enable_eqt / enable_compile / enable_eqx
            if value:
                raise NotImplementedError(f"{key}: tace_b200 has one execution path (its own sm_100a kernels)")
        self._device = torch.device(device if device is not None else "cuda")
        self._compute_forces, self._compute_stress = bool(compute_forces), bool(compute_stress)
        self.neighbor_list_fn = tace_b200_nl if neighbor_list_fn is None else neighbor_list_fn
        self._memory_scales_with = "n_atoms_x_density"
        model = load_tace(model, self._device, dtype=dtype, target_property=target_property).to(self._device)
        self._dtype = model.get_model_dtype()
        model.flags.compute_forces = self._compute_forces
        model.flags.compute_stress = self._compute_stress
        model.reset_fidelity_idx(fidelity_idx)
        model.eval()
        for p in model.parameters():
            p.requires_grad = False
        self.model = model
        self.r_max = float(model.get_cutoff())
        self._z_list = [int(z) for z in model.get_atomic_numbers()]
        table = torch.full((max(self._z_list) + 1,), -1, dtype=torch.int64)
        table[torch.tensor(self._z_list)] = torch.arange(len(self._z_list))
        self._z_table = table.to(self._device)
        self.atomic_numbers_in_init = atomic_numbers is not None
        self.system_idx_in_init = system_idx is not None
        if atomic_numbers is not None:
            self.atomic_numbers = atomic_numbers.to(device=self._device, dtype=torch.int64)
            self._setup_node_attrs(self.atomic_numbers)
        if system_idx is not None:
            self.system_idx = system_idx.to(device=self._device, dtype=torch.int64)
            self._setup_ptr(self.system_idx)
        if atomic_numbers is not None and system_idx is not None and system_idx.shape[0] != atomic_numbers.shape[0]:
            raise ValueError(f"system_idx length {system_idx.shape[0]} must match atomic_numbers length {atomic_numbers.shape[0]}.")

    # ModelInterface properties when torch_sim is absent
    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def compute_forces(self) -> bool:
        return self._compute_forces

    @property
    def compute_stress(self) -> bool:
        return self._compute_stress

    def _setup_ptr(self, system_idx: torch.Tensor) -> None:
        counts = torch.bincount(system_idx)
        self.n_systems = len(counts)
        self.n_atoms_per_system = counts.tolist()
        self.ptr = torch.cat([counts.new_zeros(1), counts.cumsum(0)])

    def _setup_node_attrs(self, atomic_numbers: torch.Tensor) -> None:
        if int(atomic_numbers.max()) >= self._z_table.numel():
            raise ValueError("structure contains an element the model was not built for")
        species = self._z_table[atomic_numbers]
        if bool((species < 0).any()):
            raise ValueError("structure contains an element the model was not built for")
        self.species = species.to(torch.int32)
        self.node_attrs = torch.nn.functional.one_hot(species, len(self._z_list)).to(self._dtype)

    def forward(self, state, **_kwargs) -> Dict[str, torch.Tensor]:
        if self.atomic_numbers_in_init:
            if state.positions.shape[0] != self.atomic_numbers.shape[0]:
                raise ValueError(f"Expected {self.atomic_numbers.shape[0]} atoms, got {state.positions.shape[0]}.")
        else:
            z = state.atomic_numbers.to(device=self._device, dtype=torch.int64)
            if not hasattr(self, "atomic_numbers") or not torch.equal(z, self.atomic_numbers):
                self._setup_node_attrs(z)
                self.atomic_numbers = z
        if self.system_idx_in_init:
            if state.system_idx.shape[0] != self.system_idx.shape[0]:
                raise ValueError(f"Expected system_idx of length {self.system_idx.shape[0]}, got {state.system_idx.shape[0]}.")
        else:
            sidx = state.system_idx.to(device=self._device, dtype=torch.int64)
            if not hasattr(self, "system_idx") or not torch.equal(sidx, self.system_idx):
                self._setup_ptr(sidx)
                self.system_idx = sidx
        edge_index, _mapping, unit_shifts = self.neighbor_list_fn(state.positions, state.row_vector_cell, state.pbc, self.r_max,
                                                                  self.system_idx)
        out = self.model({
            "ptr": self.ptr, "node_attrs": self.node_attrs, "species": self.species, "batch": self.system_idx, "pbc": state.pbc,
            "lattice": state.row_vector_cell, "positions": state.positions, "edge_index": edge_index, "edge_shifts": unit_shifts,
        })
        results: Dict[str, torch.Tensor] = {}
        results["energy"] = out["energy"].detach() if out["energy"] is not None else torch.zeros(self.n_systems, device=self._device)
        if self._compute_forces and out.get("forces") is not None:
            results["forces"] = out["forces"].detach()
        if self._compute_stress and out.get("stress") is not None:
            results["stress"] = out["stress"].detach()
        for key, val in out.items():
            if key not in ("energy", "forces", "stress") and isinstance(val, torch.Tensor):
                results[key] = val.detach()
        return results
