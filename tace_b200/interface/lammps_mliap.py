"""LAMMPS ML-IAP (unified, Kokkos CUDA) entry point with the reference's contract
(``tace/interface/lammps/mliap.py:25-151``): ``compute_forces(data)`` reads
``data.{nlocal, ntotal, npairs, elems, rij, pair_i, pair_j, eatoms}``, writes ``data.eatoms`` and
``data.energy`` and calls ``data.update_pair_forces`` with fp64 pair forces.  Ghost-atom features
are refreshed between interaction layers through ``data.forward_exchange`` and their gradients are
returned through ``data.reverse_exchange`` (``tace/models/lammps.py:82-129``).
"""

from __future__ import annotations

import logging
from typing import Dict, Tuple

import torch

from ..models import TensorModel

try:
    from lammps.mliap.mliap_unified_abc import MLIAPUnified

    LAMMPS_ML_IAP_AVAILABLE = True
except ImportError:  # the class stays importable (and testable with a stand-in `data`) without LAMMPS
    LAMMPS_ML_IAP_AVAILABLE = False

    class MLIAPUnified:  # minimal stand-in for lammps.mliap.mliap_unified_abc.MLIAPUnified
        def __init__(self, interface=None, element_types=None, ndescriptors=None, nparams=None, rcutfac=None):
            self.interface, self.element_types = interface, element_types
            self.ndescriptors, self.nparams, self.rcutfac = ndescriptors, nparams, rcutfac


_SYMBOLS = ("X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr "
            "Nb Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt "
            "Au Hg Tl Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr").split()


class EdgeForcesWrapper(torch.nn.Module):
    """tace/interface/lammps/mliap.py:25-52: switches the model to edge-vector input and pair-force output."""

    def __init__(self, model: TensorModel, **kwargs):
        super().__init__()
        model._set_lammps_mliap(True)
        model.flags.compute_forces = False
        model.flags.compute_stress = False
        model.flags.compute_virials = False
        model.flags.compute_edge_forces = True
        self.model = model
        self.register_buffer("cutoff", model.readout_fn.cutoff)
        self.register_buffer("atomic_numbers", model.readout_fn.atomic_numbers)

    def forward(self, data: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        outs = self.model(data)
        pair_forces = outs["edge_forces"]
        if pair_forces is None:
            pair_forces = torch.zeros_like(data["edge_vector"])
        return outs["energy"][0], outs["node_energy"], pair_forces


class TACELammpsCalc(MLIAPUnified):
    def __init__(self, model: TensorModel, **kwargs):
        super().__init__()
        self.model = EdgeForcesWrapper(model, **kwargs)
        self.element_types = [_SYMBOLS[int(z)] for z in model.readout_fn.atomic_numbers]
        self.num_species = len(self.element_types)
        self.rcutfac = 0.5 * float(model.readout_fn.cutoff)
        self.nparams = 1
        self.ndescriptors = 1
        self.dtype = model.readout_fn.cutoff.dtype
        self.device = torch.device("cpu")
        self.initialized = False

    def _initialize_device(self, data):
        device = torch.as_tensor(data.elems).device
        self._validate_lammps_data(data, device)
        self.device = device
        self.model = self.model.to(device)
        logging.info(f"TACE model initialized on device: {device}")
        self.initialized = True

    @staticmethod
    def _validate_lammps_data(data, device):
        if not all(hasattr(data, m) for m in ("forward_exchange", "reverse_exchange")):
            raise RuntimeError("TACE requires the KOKKOS ML-IAP interface for ghost exchange. "
                               "Run LAMMPS with '-k on g <Ng> -sf kk'.")
        if device.type != "cuda":
            raise RuntimeError("TACE LAMMPS ML-IAP currently requires a CUDA KOKKOS backend. "
                               "LAMMPS host-side ML-IAP ghost exchange is not supported.")

    def compute_forces(self, data):
        nlocal, ntotal, npairs = data.nlocal, data.ntotal, data.npairs
        nghosts = ntotal - nlocal
        species = torch.as_tensor(data.elems, dtype=torch.int64)
        if not self.initialized:
            self._initialize_device(data)
        if nlocal == 0 or npairs <= 1:
            return
        batch = self._prepare_batch(data, nlocal, nghosts, species)
        _, node_energy, pair_forces = self.model(batch)
        torch.cuda.synchronize(self.device)
        self._update_lammps_data(data, node_energy, pair_forces, nlocal)

    def _prepare_batch(self, data, nlocal, nghosts, species):
        species = species.to(self.device)
        return {
            "edge_vector": torch.as_tensor(data.rij).to(self.dtype).to(self.device),
            "node_attrs": torch.nn.functional.one_hot(species, num_classes=self.num_species).to(self.dtype),
            "species": species.to(torch.int32),
            "edge_index": torch.stack([torch.as_tensor(data.pair_j, dtype=torch.int64).to(self.device),
                                       torch.as_tensor(data.pair_i, dtype=torch.int64).to(self.device)], dim=0),
            "batch": torch.zeros(nlocal, dtype=torch.int64, device=self.device),
            "ptr": torch.tensor([0, nlocal], dtype=torch.int64, device=self.device),
            "lmp_data": data,
            "natoms": (nlocal, nghosts),
        }

    @staticmethod
    def _update_lammps_data(data, node_energy, pair_forces, nlocal):
        pair_forces = pair_forces.to(dtype=torch.float64).contiguous()
        node_energy = node_energy.to(dtype=torch.float64).contiguous()
        eatoms = torch.as_tensor(data.eatoms)
        eatoms.copy_(node_energy[:nlocal])
        data.energy = node_energy[:nlocal].sum().item()
        data.update_pair_forces(pair_forces)

    def compute_descriptors(self, data):
        pass

    def compute_gradients(self, data):
        pass
