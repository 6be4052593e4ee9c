"""LAMMPS ML-IAP "unified" plug-in backed by the CUDA evaluation path.

Same contract as the reference's plug-in (``tace/interface/lammps/mliap.py:55-151``), so ``pair_style mliap unified``
can load an object of this class in its place:

* attributes LAMMPS reads: ``element_types`` (chemical symbols in the model's element order), ``rcutfac`` (half the
  cutoff), ``nparams`` = ``ndescriptors`` = 1;
* ``compute_forces(data)`` takes the pair list of one rank (``data.rij`` = neighbour minus centre, ``data.pair_i`` the
  centre, ``data.pair_j`` the neighbour, owned atoms first, then ghosts), writes per-atom energies into
  ``data.eatoms``, their sum into ``data.energy`` and hands fp64 dE/d(rij) to ``data.update_pair_forces``;
* between interaction layers the features of ghost atoms come from their owners through ``data.forward_exchange``
  and the gradients go back through ``data.reverse_exchange`` (``tace/models/lammps.py:82-142``): that is wired
  inside ``TensorModel.forward`` (``tace_set_exchange``), this file only passes ``data`` along;
* the object is pickled on the host and binds to the device of ``data.elems`` at its first call.

The evaluation is one ``tace_forward`` call in edge-vector mode; nothing here touches autograd.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from ..models import TensorModel

try:
    from lammps.mliap.mliap_unified_abc import MLIAPUnified

    LAMMPS_ML_IAP_AVAILABLE = True
except ImportError:  # without LAMMPS the class can still be built, pickled and driven by a stand-in `data` object
    LAMMPS_ML_IAP_AVAILABLE = False

    class MLIAPUnified:  # the constructor signature of lammps.mliap.mliap_unified_abc.MLIAPUnified
        def __init__(self, interface=None, element_types=None, ndescriptors=None, nparams=None, rcutfac=None):
            self.interface, self.element_types = interface, element_types
            self.ndescriptors, self.nparams, self.rcutfac = ndescriptors, nparams, rcutfac


_SYMBOLS = ("X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr "
            "Nb Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt "
            "Au Hg Tl Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr").split()


def _pair_force_mode(model: TensorModel) -> TensorModel:
    """Edge vectors in, dE/d(edge vector) out; no per-atom forces, no strain derivative."""
    model._set_lammps_mliap(True)
    flags = model.flags
    flags.compute_forces = flags.compute_stress = flags.compute_virials = False
    flags.compute_edge_forces = True
    return model


class TACELammpsCalc(MLIAPUnified):
    def __init__(self, model: TensorModel, **kwargs):
        super().__init__()
        head = model.readout_fn
        self.model = _pair_force_mode(model)
        self.element_types: List[str] = [_SYMBOLS[int(z)] for z in head.atomic_numbers]
        self.num_species = len(self.element_types)
        self.rcutfac = float(head.cutoff) / 2.0
        self.nparams = self.ndescriptors = 1
        self.dtype = head.cutoff.dtype
        self.device: Optional[torch.device] = None  # bound at the first compute_forces call

    # -- device binding ----------------------------------------------------------------------------------------------
    def _bind(self, data) -> torch.device:
        """The rank's GPU is the one LAMMPS put ``data.elems`` on.  Ghost features travel through LAMMPS' own
        device-side exchange, which only the KOKKOS build of ML-IAP offers."""
        missing = [name for name in ("forward_exchange", "reverse_exchange") if not callable(getattr(data, name, None))]
        if missing:
            raise RuntimeError(f"the ML-IAP data object has no {' / '.join(missing)}: this model needs the KOKKOS ML-IAP "
                               "interface (start LAMMPS with '-k on g <gpus per node> -sf kk')")
        device = torch.as_tensor(data.elems).device
        if device.type != "cuda":
            raise RuntimeError(f"ML-IAP data lives on '{device}': tace_b200 evaluates on CUDA devices only, run the KOKKOS "
                               "CUDA back end")
        self.model = self.model.to(device)
        self.device = device
        return device

    # -- one evaluation ----------------------------------------------------------------------------------------------
    def compute_forces(self, data):
        device = self.device if self.device is not None else self._bind(data)
        n_owned, n_pairs = int(data.nlocal), int(data.npairs)
        if n_owned == 0 or n_pairs <= 1:  # nothing to evaluate on this rank (the reference returns here as well)
            return
        n_ghost = int(data.ntotal) - n_owned
        species = torch.as_tensor(data.elems).to(device=device, dtype=torch.int32)
        centre = torch.as_tensor(data.pair_i).to(device=device, dtype=torch.int64)
        neighbour = torch.as_tensor(data.pair_j).to(device=device, dtype=torch.int64)
        result = self.model({
            "species": species,
            "edge_index": torch.stack((neighbour, centre)),  # messages flow neighbour -> centre
            "edge_vector": torch.as_tensor(data.rij).to(device=device, dtype=self.dtype),
            "natoms": (n_owned, n_ghost),
            "lmp_data": data,
        })
        torch.cuda.synchronize(device)  # LAMMPS reads the results on its own stream
        per_atom = result["node_energy"][:n_owned].to(torch.float64)
        torch.as_tensor(data.eatoms).copy_(per_atom)
        data.energy = float(per_atom.sum())
        data.update_pair_forces(result["edge_forces"].to(torch.float64).contiguous())

    # descriptors and their gradients are not a separate stage of this model
    def compute_descriptors(self, data):
        return None

    def compute_gradients(self, data):
        return None
