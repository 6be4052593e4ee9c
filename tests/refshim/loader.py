"""Imports the reference's ``tace.models`` package from its source tree with stand-ins for the third-party packages
that are absent here.  TEST INFRASTRUCTURE ONLY.

What is real: every file under the reference's ``tace/`` that the energy / force path executes.  What is a stand-in:
``e3nn`` (``mini_e3nn.py``, conventions from ``oracle/o3.py``), ``ase.data`` (tables of the right length; the covalent
radii are supplied by the caller because only ZBL reads them), ``torch_geometric.utils.scatter / segment`` (ten lines
of torch), ``opt_einsum_fx`` (unused: the reference only calls it behind a flag that is off by default,
``tace/models/o2/wigner.py:183``), and empty placeholder modules for packages the model code imports but never calls on
this path (lightning, hydra, matscipy, ...).
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import os
import sys
import types

import numpy as np
import torch

from . import mini_e3nn

# The reference's source tree: TACE_REFERENCE_ROOT, or a directory named "reference" beside this repository.
_REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REFERENCE_ROOT = os.environ.get("TACE_REFERENCE_ROOT", os.path.join(os.path.dirname(_REPO_ROOT), "reference"))
_PLACEHOLDER_ROOTS = ("matscipy", "lightning", "pytorch_lightning", "hydra", "omegaconf", "torch_scatter",
                      "h5py", "lmdb", "vesin", "torch_ema", "torchmetrics", "wandb", "opt_einsum", "cuequivariance",
                      "cuequivariance_torch", "openequivariance", "equitorch", "ase", "torch_geometric", "nvalchemiops",
                      "torch_sim", "lammps")


class _Placeholder(types.ModuleType):
    """A module whose attributes exist (so ``from x import Y`` works) but do nothing."""

    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        if name[0].islower():
            try:
                sub = importlib.import_module(self.__name__ + "." + name)
                setattr(self, name, sub)
                return sub
            except ImportError:
                pass
        cls = type(name, (), {"__init__": lambda self, *a, **k: None})
        setattr(self, name, cls)
        return cls


class _PlaceholderFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path, target=None):
        if fullname.split(".")[0] in _PLACEHOLDER_ROOTS and fullname not in sys.modules:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Placeholder(spec.name)
        m.__path__ = []
        return m

    def exec_module(self, module):
        pass


def _scatter(src, index, dim=0, dim_size=None, reduce="sum"):
    if dim != 0:
        raise NotImplementedError
    n = int(index.max()) + 1 if dim_size is None else dim_size
    idx = index.view((-1,) + (1,) * (src.dim() - 1)).expand_as(src)
    if reduce in ("sum", "add"):
        return torch.zeros((n,) + tuple(src.shape[1:]), dtype=src.dtype).scatter_add_(0, idx, src)
    if reduce == "max":
        out = torch.full((n,) + tuple(src.shape[1:]), -float("inf"), dtype=src.dtype)
        out = out.scatter_reduce(0, idx, src, "amax")
        return torch.where(torch.isinf(out), torch.zeros_like(out), out)  # torch_geometric fills empty rows with 0
    raise NotImplementedError(reduce)


def _segment(src, ptr, reduce="sum"):
    ptr = ptr.reshape(-1)
    return torch.stack([getattr(src[a:b], {"sum": "sum", "max": "amax"}[reduce])(dim=0) for a, b in zip(ptr[:-1], ptr[1:])])


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_ROOT, "tace", "models"))


_state = {}


def load(covalent_radii=None):
    """Returns the reference's ``tace.models`` module (imported once per process)."""
    if "models" in _state:
        return _state["models"]
    if not available():
        raise FileNotFoundError(REFERENCE_ROOT)
    try:
        import e3nn  # noqa: F401  (a real e3nn would make the stand-in unnecessary)
    except ImportError:
        mini_e3nn.install()
    if "ase.data" not in sys.modules:
        ase = types.ModuleType("ase")
        ase.__path__ = []
        data = types.ModuleType("ase.data")
        data.chemical_symbols = ["X"] + [f"El{z}" for z in range(1, 119)]
        data.atomic_numbers = {s: z for z, s in enumerate(data.chemical_symbols)}
        data.atomic_names = [""] * 119
        data.atomic_masses = np.ones(119)
        data.vdw_radii = np.ones(119)
        data.ground_state_magnetic_moments = np.zeros(119)
        data.covalent_radii = np.full(119, 0.2) if covalent_radii is None else np.asarray(covalent_radii, dtype=float)
        ase.data = data
        sys.modules["ase"], sys.modules["ase.data"] = ase, data
    if "torch_geometric" not in sys.modules:
        tg = types.ModuleType("torch_geometric")
        tg.__path__ = []
        utils = types.ModuleType("torch_geometric.utils")
        utils.__path__ = []
        utils.scatter, utils.segment = _scatter, _segment
        nn_mod = types.ModuleType("torch_geometric.utils.num_nodes")
        nn_mod.maybe_num_nodes = lambda index, num_nodes=None: int(index.max()) + 1 if num_nodes is None else num_nodes
        utils.num_nodes = nn_mod
        tg.utils = utils
        sys.modules.update({"torch_geometric": tg, "torch_geometric.utils": utils, "torch_geometric.utils.num_nodes": nn_mod})
    if "opt_einsum_fx" not in sys.modules:  # only reorders einsum contractions; the traced module is returned as it is
        oe = types.ModuleType("opt_einsum_fx")
        oe.optimize_einsums_full = lambda model, example_inputs=None, **kw: model
        sys.modules["opt_einsum_fx"] = oe
    sys.meta_path.append(_PlaceholderFinder())
    if REFERENCE_ROOT not in sys.path:
        sys.path.append(REFERENCE_ROOT)
    _state["models"] = importlib.import_module("tace.models")
    return _state["models"]
