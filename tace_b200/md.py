"""Velocity-Verlet molecular dynamics (NVE, or NVT with a Langevin thermostat) of one periodic system on one or
several GPUs.

Every rank owns the atoms of one block of the cell (``tace_b200.domain``), keeps positions and
velocities in fp64 on its GPU and, per step: half kick + drift, ghost positions from the owning
ranks, a fresh neighbour list over owned targets, one model evaluation in edge-vector mode (the
LAMMPS contract of the reference: ghost feature rows refreshed between interaction layers, ghost
gradients returned to their owners, ``tace/models/lammps.py:82-142``), forces that landed on ghost
rows returned to their owners, second half kick.  Ownership and ghost lists are rebuilt when an atom
has moved more than half the skin.  With ``friction`` set, every step ends with the exact Ornstein-Uhlenbeck
velocity update ``v <- c1 v + sqrt((1 - c1^2) kT / m) xi``, ``c1 = exp(-friction dt)``, whose random numbers depend
only on (seed, step, atom id), so the trajectory is the same for any number of ranks.  ``thermo()`` returns the usual
thermodynamic output line.

Units: eV, Angstrom, atomic mass units, femtoseconds.
"""

from __future__ import annotations

import ctypes
import time
from typing import Dict, Optional, Sequence, Tuple

import numpy as np
import torch

from . import lib as _lib
from .domain import Domain
from .graph import z_to_index
from .neighbour_list import neighbor_list_batch

# 1 eV / amu in Angstrom^2 / fs^2, and Boltzmann's constant in eV / K
ACCEL = 9.64853321233e-3
KB = 8.617333262e-5

# standard atomic weights of the elements the synthetic workloads use (amu)
_MASSES = {1: 1.008, 6: 12.011, 7: 14.007, 8: 15.999, 13: 26.9815385, 14: 28.085, 22: 47.867, 23: 50.9415, 24: 51.9961,
           26: 55.845, 27: 58.933194, 28: 58.6934, 29: 63.546}


def masses_for(atomic_numbers: Sequence[int]) -> np.ndarray:
    try:
        return np.array([_MASSES[int(z)] for z in atomic_numbers], dtype=np.float64)
    except KeyError as exc:  # pragma: no cover - message only
        raise ValueError(f"no tabulated mass for Z={exc.args[0]}; pass `masses` explicitly") from None


def maxwell_boltzmann(masses: np.ndarray, temperature: float, seed: int) -> np.ndarray:
    """Velocities (Angstrom / fs) at ``temperature`` with zero total momentum, rescaled to the exact
    kinetic temperature."""
    rng = np.random.default_rng(seed)
    sigma = np.sqrt(KB * temperature * ACCEL / masses)[:, None]
    v = rng.normal(size=(len(masses), 3)) * sigma
    v -= (masses[:, None] * v).sum(0) / masses.sum()
    ke = 0.5 * (masses[:, None] * v * v).sum() / ACCEL
    t_now = 2.0 * ke / (3.0 * len(masses) * KB)
    return v * np.sqrt(temperature / t_now) if t_now > 0 else v


class DomainMD:
    """``model``: a ``tace_b200.models.TensorModel``.  ``positions`` [N,3], ``atomic_numbers`` [N],
    ``velocities`` [N,3] describe the WHOLE system and must be identical on every rank (each rank keeps
    only its own block).  ``group``: the ``torch.distributed`` process group (``None`` = default group;
    unused when ``world_size == 1``)."""

    def __init__(self, model, cell: np.ndarray, positions: np.ndarray, atomic_numbers: np.ndarray,
                 velocities: Optional[np.ndarray] = None, masses: Optional[np.ndarray] = None, dt: float = 1.0,
                 skin: float = 0.5, rank: int = 0, world_size: int = 1, device: Optional[torch.device] = None,
                 grid: Optional[Tuple[int, int, int]] = None, group=None, temperature: Optional[float] = None,
                 friction: float = 0.0, seed: int = 0):
        """``friction`` (1/fs) > 0 with ``temperature`` (K) switches the Langevin thermostat on."""
        self.model = model
        if friction < 0.0 or (friction > 0.0 and (temperature is None or temperature < 0.0)):
            raise ValueError("the Langevin thermostat needs friction >= 0 and a target temperature >= 0")
        self.friction, self.target_temperature, self.seed = float(friction), temperature, int(seed)
        self.device = torch.device(device if device is not None else "cuda")
        self.rank, self.world_size, self.group = rank, world_size, group
        self.dt = float(dt)
        self.cutoff = float(model.get_cutoff())
        self.dtype = model.get_model_dtype()
        self.lib = _lib.load()
        model._set_lammps_mliap(True)
        model.reset_target_property(["energy", "forces"])
        self.domain = Domain(cell, self.cutoff, skin, rank, world_size, self.device, grid=grid, group=group,
                             high_priority_halo=bool(getattr(model, "_exchange_overlap", False)))

        positions = np.asarray(positions, dtype=np.float64)
        n = positions.shape[0]
        z = np.asarray(atomic_numbers)
        if masses is None:
            masses = masses_for(z)
        if velocities is None:
            velocities = np.zeros((n, 3))
        species = z_to_index(z, model.get_atomic_numbers())
        # every rank starts from the same global arrays and keeps its own block: rank r contributes
        # the r-th slice to the first partition, which then moves every atom to its owner
        lo, hi = (n * rank) // world_size, (n * (rank + 1)) // world_size
        dev = self.device
        state = {
            "positions": torch.as_tensor(positions[lo:hi], dtype=torch.float64, device=dev),
            "velocities": torch.as_tensor(np.asarray(velocities, dtype=np.float64)[lo:hi], device=dev),
            "species": torch.as_tensor(np.asarray(species[lo:hi], dtype=np.int64), device=dev),
            "mass": torch.as_tensor(np.asarray(masses, dtype=np.float64)[lo:hi], device=dev),
            "ids": torch.arange(lo, hi, dtype=torch.int64, device=dev),
        }
        self.n_global = n
        self.step_count = 0
        self.timings: Dict[str, float] = {}
        self.skin = float(skin)
        self._skin_edges: Optional[torch.Tensor] = None  # neighbour list within cutoff + skin, built once per partition
        self.n_list_builds = 0
        self._next_check = 0                              # step at which the displacement is looked at again
        self._repartition(state)
        self.forces = None
        self.potential_energy = None
        self._evaluate()

    # -- state -------------------------------------------------------------------------------------
    def _repartition(self, state: Dict[str, torch.Tensor]) -> None:
        new = self.domain.partition(state)
        self.positions = new["positions"].contiguous()
        self.velocities = new["velocities"].contiguous()
        self.species = new["species"].contiguous()
        self.mass = new["mass"].contiguous()
        self.ids = new["ids"].contiguous()
        self.inv_mass = (1.0 / self.mass).contiguous()
        self.local_species = self.domain.local_rows(self.species).to(torch.int32).contiguous()
        self._ke_scratch = torch.empty(1025, dtype=torch.float64, device=self.device)
        self._skin_edges = None  # ownership and ghosts changed: the list is rebuilt at the next evaluation

    def _state(self) -> Dict[str, torch.Tensor]:
        return {"positions": self.positions, "velocities": self.velocities, "species": self.species, "mass": self.mass,
                "ids": self.ids}

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # -- one force evaluation ------------------------------------------------------------------------
    def _evaluate(self) -> None:
        dom = self.domain
        n, g = dom.n_owned, dom.n_ghost
        t0 = time.perf_counter()
        local_pos = dom.local_positions(self.positions)
        t1 = time.perf_counter()
        # open (non-periodic) neighbour list over owned + ghost atoms, owned targets only
        lattice = torch.eye(3, dtype=torch.float64, device=self.device)[None]
        pbc = torch.zeros(1, 3, dtype=torch.uint8, device=self.device)
        ptr = torch.tensor([0, n + g], dtype=torch.int32, device=self.device)
        if n == 0:  # a block of vacuum: no target atom, no edge (the evaluation still answers its peers' exchanges)
            edge_index = torch.empty(2, 0, dtype=torch.int64, device=self.device)
        else:
            # Verlet list: all pairs within cutoff + skin, built once per partition.  Ownership, ghost lists and this
            # list stay valid until an atom has moved more than half the skin; every step only filters the list down
            # to the pairs that are inside the cutoff now (the same fp64 test a fresh list would apply).
            if self._skin_edges is None:
                t_l = time.perf_counter()
                self._skin_edges, _ = neighbor_list_batch(local_pos, lattice, pbc, ptr, self.cutoff + self.skin, n_targets=n)
                self._skin_edges = self._skin_edges.contiguous()
                self.n_list_builds += 1
                self.timings["list_build"] = self.timings.get("list_build", 0.0) + time.perf_counter() - t_l
            wide = self._skin_edges
            Ew = int(wide.shape[1])
            keep = torch.empty(Ew, dtype=torch.uint8, device=self.device)
            position = torch.empty(Ew, dtype=torch.int32, device=self.device)
            total = torch.empty(1, dtype=torch.int64, device=self.device)
            nbytes = ctypes.c_size_t()
            _lib.check(self.lib.tace_edges_scan_workspace_bytes(Ew, ctypes.byref(nbytes)), "tace_edges_scan_workspace_bytes")
            scratch = torch.empty(int(nbytes.value), dtype=torch.uint8, device=self.device)
            with torch.cuda.device(self.device):
                _lib.check(self.lib.tace_edges_within(local_pos.data_ptr(), wide.data_ptr(), Ew, self.cutoff, keep.data_ptr(),
                                                      self._stream()), "tace_edges_within")
                _lib.check(self.lib.tace_edges_scan(keep.data_ptr(), Ew, position.data_ptr(), total.data_ptr(), scratch.data_ptr(),
                                                    scratch.numel(), self._stream()), "tace_edges_scan")
            E = int(total.item())  # the one host read of the step: sizes of the edge arrays
            edge_index = torch.empty(2, E, dtype=torch.int64, device=self.device)
            vec = torch.empty(E, 3, dtype=self.dtype, device=self.device)
            with torch.cuda.device(self.device):
                _lib.check(self.lib.tace_edges_compact(local_pos.data_ptr(), wide.data_ptr(), Ew, keep.data_ptr(), position.data_ptr(), E,
                                                       edge_index.data_ptr(), vec.data_ptr(), _lib.dtype_code(self.dtype), self._stream()),
                           "tace_edges_compact")
        if n == 0:
            E = 0
            vec = torch.empty(0, 3, dtype=self.dtype, device=self.device)
        t2 = time.perf_counter()
        out = self.model({"species": self.local_species, "edge_index": edge_index, "edge_vector": vec, "natoms": (n, g),
                          "lmp_data": dom.exchange})
        forces = out["forces"]
        if g:
            dom.exchange.reverse_exchange(forces, forces, 3)
        self.forces = forces[:n].contiguous()
        self.node_energy = out["node_energy"]
        self.n_edges = E
        t3 = time.perf_counter()
        for k, v in (("halo_positions", t1 - t0), ("neighbour_list", t2 - t1), ("model", t3 - t2)):
            self.timings[k] = self.timings.get(k, 0.0) + v

    # -- integration ---------------------------------------------------------------------------------
    def step(self, n_steps: int = 1, log_every: int = 0, log=None) -> None:
        """Advance ``n_steps``; every ``log_every`` steps ``log(self.thermo())`` is called (collective)."""
        kick = 0.5 * self.dt * ACCEL
        fcode = _lib.dtype_code(self.dtype)
        for _ in range(n_steps):
            n = self.domain.n_owned
            if n > 0:
                with torch.cuda.device(self.device):
                    _lib.check(self.lib.tace_md_kick_drift(self.positions.data_ptr(), self.velocities.data_ptr(), self.forces.data_ptr(),
                                                           fcode, self.inv_mass.data_ptr(), n, kick, self.dt, self._stream()),
                               "tace_md_kick_drift")
            if self.step_count >= self._next_check:
                moved, fastest = self.domain.displacement(self.positions, self.velocities)
                if moved > 0.5 * self.skin:
                    t_r = time.perf_counter()
                    self._repartition(self._state())
                    self.timings["repartition"] = self.timings.get("repartition", 0.0) + time.perf_counter() - t_r
                    moved = 0.0
                # no atom can cross half the skin before it has travelled the remaining margin: look again after half
                # the steps the fastest atom would need at twice its present speed (at most 16 steps)
                margin = 0.5 * self.skin - moved
                safe = int(margin / max(2.0 * fastest * self.dt, 1e-12) / 2.0)
                self._next_check = self.step_count + max(1, min(16, safe))
            self._evaluate()
            n = self.domain.n_owned
            with torch.cuda.device(self.device):
                if n > 0:
                    _lib.check(self.lib.tace_md_kick_drift(None, self.velocities.data_ptr(), self.forces.data_ptr(), fcode,
                                                           self.inv_mass.data_ptr(), n, kick, 0.0, self._stream()), "tace_md_kick_drift")
                if self.friction > 0.0 and n > 0:
                    _lib.check(self.lib.tace_md_langevin(self.velocities.data_ptr(), self.inv_mass.data_ptr(), self.ids.data_ptr(), n,
                                                         float(np.exp(-self.friction * self.dt)), KB * self.target_temperature * ACCEL,
                                                         self.seed, self.step_count, self._stream()), "tace_md_langevin")
            self.step_count += 1
            if log is not None and log_every > 0 and self.step_count % log_every == 0:
                log(self.thermo())

    # -- observables (collective: every rank must call) ---------------------------------------------
    def _all_sum(self, x: torch.Tensor) -> float:
        if self.world_size > 1:
            import torch.distributed as dist

            x = x.clone()
            dist.all_reduce(x, group=self.group)
        return float(x.item())

    def kinetic_energy(self) -> float:
        out = self._ke_scratch[1024:1025]
        if self.domain.n_owned == 0:
            return self._all_sum(torch.zeros((), dtype=torch.float64, device=self.device)) / ACCEL
        with torch.cuda.device(self.device):
            _lib.check(self.lib.tace_md_kinetic_energy(self.velocities.data_ptr(), self.mass.data_ptr(), self.domain.n_owned,
                                                       self._ke_scratch.data_ptr(), out.data_ptr(), self._stream()),
                       "tace_md_kinetic_energy")
        return self._all_sum(out.clone().reshape(())) / ACCEL

    def potential(self) -> float:
        return self._all_sum(self.node_energy.to(torch.float64).sum())

    def temperature(self) -> float:
        return 2.0 * self.kinetic_energy() / (3.0 * self.n_global * KB)

    def thermo(self) -> Dict[str, float]:
        """Step, time (fs), potential / kinetic / total energy (eV) and temperature (K) of the whole system (collective)."""
        ke, pe = self.kinetic_energy(), self.potential()
        return {"step": self.step_count, "time": self.step_count * self.dt, "potential": pe, "kinetic": ke, "total": pe + ke,
                "temperature": 2.0 * ke / (3.0 * self.n_global * KB)}

    def gather(self) -> Dict[str, np.ndarray]:
        """Whole-system positions, velocities and forces ordered by atom id (collective)."""
        parts = {"ids": self.ids, "positions": self.positions, "velocities": self.velocities,
                 "forces": self.forces.to(torch.float64)}
        full = {k: torch.cat(self.domain._all_gather_rows(v.contiguous())) for k, v in parts.items()}
        order = torch.argsort(full["ids"])
        return {k: v[order].cpu().numpy() for k, v in full.items()}
