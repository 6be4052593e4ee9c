"""ASE calculator with the reference's constructor and result contract
(``tace/interface/ase/calculator.py:26-178``): ``calculate(atoms)`` fills
``results["energy", "free_energy", "forces", "stress"]`` (stress as a 3x3 array, as the
reference returns it).  Unlike the reference, which rebuilds the neighbour list on the CPU and
re-uploads a collated graph on every call, the structure is uploaded once per call and the
neighbour list is built on the GPU.
"""

from __future__ import annotations

from typing import List, Optional, Union

import numpy as np
import torch

from ..graph import build_batch
from ..models import TensorModel, create_model

try:  # ASE is optional: without it the class still works with any object exposing the four getters below
    from ase.calculators.calculator import Calculator, all_changes
except ImportError:  # pragma: no cover - exercised where ase is absent
    all_changes = ["positions", "numbers", "cell", "pbc"]

    class Calculator:  # minimal stand-in for ase.calculators.calculator.Calculator
        implemented_properties: List[str] = []

        def __init__(self, **kwargs):
            self.results = {}
            self.atoms = None

        def calculate(self, atoms=None, properties=None, system_changes=all_changes):
            if atoms is not None:
                self.atoms = atoms

        def get_potential_energy(self, atoms=None):
            self.calculate(atoms)
            return self.results["energy"]

        def get_forces(self, atoms=None):
            self.calculate(atoms)
            return self.results["forces"]

        def get_stress(self, atoms=None):
            self.calculate(atoms)
            return self.results["stress"]


def load_tace(path_or_model, device, dtype=None, target_property=None) -> TensorModel:
    """The ``.pt`` contract of the reference (tace/lightning/lit_model.py:587-609,664-677): a dict with
    ``state_dict``, ``cfg`` (model section), ``statistics``, ``target_property``."""
    if isinstance(path_or_model, TensorModel):
        model = path_or_model
    else:
        blob = torch.load(path_or_model, map_location="cpu", weights_only=False)
        prev = torch.get_default_dtype()
        want = {"float32": torch.float32, "float64": torch.float64, None: None}.get(dtype, dtype)
        first = next(v for v in blob["state_dict"].values() if v.is_floating_point())
        torch.set_default_dtype(want or first.dtype)
        try:
            model = create_model(blob["cfg"], blob.get("statistics"), target_property or blob.get("target_property"))
        finally:
            torch.set_default_dtype(prev)
        own = model.state_dict()
        model.load_state_dict({k: v.to(own[k].dtype) for k, v in blob["state_dict"].items() if k in own}, strict=True)
    if target_property is not None:
        model.reset_target_property(list(target_property))
    return model


def export_tace(model: TensorModel, path: str) -> None:
    """Writes the reference's portable ``.pt`` dictionary (tace/lightning/lit_model.py:664-677)."""
    rf = model.readout_fn
    torch.save({"state_dict": model.state_dict(), "cfg": rf.model_config, "target_property": rf.target_property,
                "embedding_property": [], "statistics": rf.statistics}, path)


class TACEAseCalc(Calculator):
    def __init__(self, model: Union[str, TensorModel], *, dtype: Optional[str] = None, device: Optional[str] = None,
                 fidelity_idx: Optional[int] = None, target_property: Optional[List[str]] = None,
                 neighborlist_backend: str = "tace_b200", **kwargs):
        for flag in ("enable_oeq", "enable_cue", "enable_eqt", "enable_compile", "enable_eqx"):
            if kwargs.pop(flag, False):
                raise NotImplementedError(f"{flag}: third-party acceleration back ends are not part of tace_b200")
        super().__init__(**kwargs)
        self.device = torch.device(device or "cuda")
        if self.device.type != "cuda":
            raise RuntimeError("tace_b200 runs on CUDA devices only")
        self.model = load_tace(model, self.device, dtype=dtype, target_property=target_property)
        self.dtype = self.model.get_model_dtype()
        self.target_property = self.model.get_target_property()
        self.cutoff = self.model.get_cutoff()
        self.atomic_numbers = self.model.get_atomic_numbers()
        self.neighborlist_backend = neighborlist_backend
        self.fidelity_idx = 0 if fidelity_idx is None else fidelity_idx
        self.model.reset_fidelity_idx(self.fidelity_idx)
        self.implemented_properties = []
        for p in self.target_property:
            self.implemented_properties.extend(["energy", "free_energy"] if p == "energy" else [p])

    def calculate(self, atoms=None, properties=None, system_changes=all_changes):
        Calculator.calculate(self, atoms)
        positions = np.asarray(atoms.get_positions(), dtype=np.float64)
        n = len(positions)
        host = {
            "positions": positions,
            "atomic_numbers": np.asarray(atoms.get_atomic_numbers(), dtype=np.int64),
            "lattice": np.asarray(atoms.get_cell(), dtype=np.float64).reshape(1, 3, 3),
            "pbc": np.asarray(atoms.get_pbc(), dtype=np.uint8).reshape(1, 3),
            "batch": np.zeros(n, dtype=np.int64),
            "ptr": np.array([0, n], dtype=np.int64),
        }
        data = build_batch(host, self.atomic_numbers, self.cutoff, self.dtype, self.device)
        outs = self.model(data)
        self.results = {}
        for p in self.target_property:
            if outs.get(p) is None:
                continue
            if p == "energy":
                self.results["energy"] = float(outs[p].cpu().item())
                self.results["free_energy"] = self.results["energy"]
            elif p in ("stress", "virials"):
                self.results[p] = outs[p].cpu().numpy().squeeze(0)
            else:
                self.results[p] = outs[p].cpu().numpy()
