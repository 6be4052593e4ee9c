"""Drop-in mirror of ``tace.models`` for the energy / force / stress path.

``e3nnTACE`` (alias ``cartTACE``) keeps the reference constructor signature
(``tace/models/_e3nn/tace.py:29-62``) and parameter names, so a reference ``.pt`` checkpoint's
``state_dict`` loads unchanged; ``TensorModel`` keeps the reference wrapper contract
(``tace/models/adapter.py:23-41``): ``forward(data) -> dict`` with ``energy``, ``node_energy``,
``forces``, ``virials``, ``stress``, ``edge_forces``.  All arithmetic happens in
``libtace_b200.so`` (hand-written CUDA, forward and backward); PyTorch only owns the device
buffers and the stream.  There is no autograd and no CPU fallback, and ``forward`` never
mutates ``data``.
"""

from __future__ import annotations

import copy
import ctypes
import os
import math
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch

from . import lib as _lib
from .pack import RADIAL_TABLE_INTERVALS, ModelPlan, pack_weights

# Options of the reference constructor that this path implements; anything else raises.
_DEFAULTS: Dict[str, Any] = {
    "mmax": 2, "Lmax": 2, "lmax": 3, "mag_Lmax": 1, "parity": False, "num_channel": 64, "num_layers": 2,
    "target_property": ["energy", "forces"], "embedding_property": [],
    "fidelity": {"name": "PBE", "atomic_energy": None},
    "node_embedding": {"type": "linear"}, "edge_embedding": {"type": "identity"}, "edge_update": {"type": "identity"},
    "radial_basis": {"bias": False, "r_min": 0.0, "radial_basis": "j0", "num_radial_basis": 8, "distance_transform": None,
                     "cutoff_fn": "c2poly", "polynomial_cutoff": 5, "trainable": False, "apply_cutoff": True,
                     "hidden": [64, 64, 64], "use_dydynamic_cutoff": False},
    "atomic_basis": {"type": "cgtp", "l1l2": None, "scatter_norm": "avg_num_neighbors", "nonlinear": "sigmoid_gate",
                     "edge_nonlinear": "so2_sigmoid_gate", "gate_m0": True, "scalar_act": None, "tensor_act": None,
                     "node_wise_hidden": None, "edge_wise_hidden": None, "edge_ace_hidden": None, "num_head": None},
    "resnet": {"type": "BB", "linear_type": "aware", "use_first_resnet": False},
    "layer_norm": {"pre_norm_type": None, "final_norm_type": None, "use_first_pre_norm": False},
    "product_basis": {"type": "cgtp", "l1l2": None, "correlation": 2, "return_components": None, "num_expert": None,
                      "num_channel_per_expert": None, "use_shared_expert": False, "nonlinear": None, "agnostic": False},
    "readout_emlp": {"bias": False, "hidden": [16], "use_alllayer": False, "use_uie": False},
    "scale_shift": {"enable": True, "scale_type": "rms_forces", "shift_type": None, "scale_trainable": False,
                    "shift_trainable": False, "all_atoms": False, "scale_zbl": True},
    "short_range": {"zbl": {"enable": False, "trainable": False}},
    "long_range": {"les": {"enable": False}},
    "dropout": {"use_first_dropout": False, "stochastic_depth": 0.0},
}

_SUPPORTED_TARGETS = {"energy", "forces", "stress", "virials", "edge_forces"}


def _merge(default: Dict, user: Dict) -> Dict:
    """tace/models/_e3nn/default.py:180-212 (recursive_update)."""
    out = {}
    for k, dv in default.items():
        if k not in user:
            out[k] = copy.deepcopy(dv)
        elif isinstance(dv, dict) and isinstance(user[k], dict):
            out[k] = _merge(dv, user[k])
        else:
            out[k] = copy.deepcopy(user[k])
    for k, v in user.items():
        if k not in out:
            out[k] = copy.deepcopy(v)
    return out


def _require(cond: bool, what: str) -> None:
    if not cond:
        raise NotImplementedError(f"tace_b200 implements the cgtp energy/force path only: {what}")


def check_model_config(cfg: Dict) -> Dict:
    """The part of tace/models/_e3nn/default.py:231-316 this path needs, plus refusal of
    every option that is not implemented (never silently ignored)."""
    cfg = _merge(_DEFAULTS, {k: v for k, v in cfg.items() if v is not None or k == "max_neighbors"})
    if cfg.get("max_neighbors") is not None:
        raise ValueError("TACE does not truncate neighbor lists. Set `max_neighbors: null` in the model configuration.")
    stats = cfg.get("statistics")
    if not isinstance(stats, (list, tuple)) or not stats:
        raise ValueError("statistics must be a non-empty list of dicts")
    _require(1 <= len(stats) <= 8, "one to eight fidelities (entries of statistics)")
    cfg["atomic_numbers"] = sorted({int(z) for s in stats for z in s["atomic_numbers"]})
    cfg["avg_num_neighbors"] = sum(float(s["avg_num_neighbors"]) for s in stats) / len(stats)
    cfg["atomic_energies"] = [s["atomic_energy"] for s in stats]
    _require(1 <= cfg["Lmax"] <= cfg["lmax"] <= 3, "1 <= Lmax <= lmax <= 3")
    _require(not cfg["parity"], "parity=False")
    _require(1 <= cfg["num_channel"] <= 256, "1 <= num_channel <= 256 (counts that are not multiples of 32 run zero-padded)")
    _require(1 <= cfg["num_layers"] <= 4, "1..4 layers")
    _require(set(cfg["target_property"]) <= _SUPPORTED_TARGETS and "energy" in cfg["target_property"],
             f"target_property within {sorted(_SUPPORTED_TARGETS)} including energy")
    _require(not cfg["embedding_property"], "no universal embeddings")
    for section, key, allowed in [
        ("node_embedding", "type", {"linear"}), ("edge_embedding", "type", {"identity"}), ("edge_update", "type", {"identity", "element2"}),
        ("radial_basis", "radial_basis", {"j0", "bessel"}), ("radial_basis", "cutoff_fn", {"c2poly", "polynomial"}),
        ("radial_basis", "distance_transform", {None}), ("radial_basis", "apply_cutoff", {True, False}),
        ("radial_basis", "bias", {False, True}), ("radial_basis", "use_dydynamic_cutoff", {False}),
        ("radial_basis", "num_radial_basis", {8}),
        ("atomic_basis", "scatter_norm", {"avg_num_neighbors", "density", "no_cutoff_density"}), ("atomic_basis", "gate_m0", {True, False}),
        ("atomic_basis", "l1l2", {None}), ("atomic_basis", "scalar_act", {None, "sigmoid"}),
        ("atomic_basis", "tensor_act", {None, "sigmoid"}), ("atomic_basis", "node_wise_hidden", {None}),
        ("resnet", "type", {"BB"}), ("resnet", "linear_type", {"aware", "agnostic", "identity"}), ("resnet", "use_first_resnet", {False}),
        ("layer_norm", "pre_norm_type", {None}), ("layer_norm", "final_norm_type", {None}),
        ("product_basis", "l1l2", {None}), ("product_basis", "return_components", {None}),
        ("product_basis", "num_expert", {None, 1}), ("product_basis", "nonlinear", {None, "silu_bilineargate"}),
        ("product_basis", "agnostic", {False, True}), ("product_basis", "use_shared_expert", {False}),
        ("readout_emlp", "bias", {False}), ("readout_emlp", "use_alllayer", {False, True}), ("readout_emlp", "use_uie", {False}),
        ("scale_shift", "enable", {True}), ("scale_shift", "all_atoms", {False}), ("scale_shift", "shift_type", {None}),
    ]:
        _require(cfg[section][key] in allowed, f"{section}.{key} in {allowed}, got {cfg[section][key]!r}")
    hidden = list(cfg["radial_basis"]["hidden"])
    _require(1 <= len(hidden) <= 3 and all(h == 64 for h in hidden), "radial_basis.hidden: one to three layers of width 64")
    _require(len(cfg["readout_emlp"]["hidden"]) == 1 and cfg["readout_emlp"]["hidden"][0] <= 64, "one read-out hidden layer <= 64")
    _require(cfg["atomic_basis"]["scatter_norm"] == "avg_num_neighbors" or cfg["edge_update"]["type"] == "identity",
             "a learned edge density (atomic_basis.scatter_norm) only with edge_update.type = identity")
    if cfg["short_range"]["zbl"]["enable"]:
        cfg["short_range"]["zbl"]["covalent_radii"] = _covalent_radii(cfg)
    _require(not cfg["long_range"]["les"]["enable"], "no LES")
    _require(cfg["dropout"]["stochastic_depth"] == 0.0, "no stochastic depth")

    def to_list(x):
        return [x] * cfg["num_layers"] if not isinstance(x, list) else x

    for section, key in [("atomic_basis", "type"), ("product_basis", "type"), ("atomic_basis", "nonlinear"),
                         ("product_basis", "correlation")]:
        cfg[section][key] = to_list(cfg[section][key])
    _require(all(t in ("cgtp", "uv_so2") for t in cfg["atomic_basis"]["type"]), "atomic_basis.type in {cgtp, uv_so2}")
    if "uv_so2" in cfg["atomic_basis"]["type"]:  # the TECE edge block (tace/models/_e3nn/inter.py:440-519)
        ab = cfg["atomic_basis"]
        _require(cfg["atomic_basis"]["type"][0] == "cgtp", "atomic_basis.type: uv_so2 needs input ranks above 0, so not on the first layer")
        _require(cfg["Lmax"] == cfg["lmax"], "Lmax == lmax with uv_so2 interactions")
        _require(0 <= cfg["mmax"] <= min(2, cfg["lmax"]), "mmax <= 2 with uv_so2 interactions")
        _require(ab["edge_wise_hidden"] in (None, cfg["num_channel"]), "atomic_basis.edge_wise_hidden == num_channel")
        _require(ab["edge_nonlinear"] in ("so2_sigmoid_gate", "so2_silu_gate"), "atomic_basis.edge_nonlinear in {so2_sigmoid_gate, so2_silu_gate}")
        _require(cfg["num_channel"] % (ab["num_head"] or 1) == 0, "num_head divides num_channel")
        _require(ab["scatter_norm"] == "avg_num_neighbors", "scatter_norm = avg_num_neighbors next to uv_so2 interactions")
    _require(all(t in ("cgtp", "spatial", "coupled") for t in cfg["product_basis"]["type"]), "product_basis.type == cgtp")
    _require(all(n == "sigmoid_gate" for n in cfg["atomic_basis"]["nonlinear"]), "atomic_basis.nonlinear == sigmoid_gate")
    corr = cfg["product_basis"]["correlation"]
    _require(len(set(corr)) == 1 and corr[0] in (1, 2, 3), "product_basis.correlation in {1, 2, 3}, equal on all layers")
    _require(corr[0] >= 2 or cfg["Lmax"] == cfg["lmax"], "Lmax == lmax when product_basis.correlation == 1")
    return cfg


def _covalent_radii(cfg: Dict) -> Dict[int, float]:
    """Covalent radius per element for the ZBL envelope.  The reference reads ``ase.data.covalent_radii``
    (tace/models/radial.py:809-815); this does the same when ase is installed, and otherwise needs the radii of the
    model's elements in ``short_range.zbl.covalent_radii`` (a {Z: radius in Angstrom} dictionary)."""
    given = {int(k): float(v) for k, v in (cfg["short_range"]["zbl"].get("covalent_radii") or {}).items()}
    missing = [z for z in cfg["atomic_numbers"] if z not in given]
    if missing:
        try:
            from ase.data import covalent_radii as table
        except ImportError:
            _require(False, f"ZBL needs short_range.zbl.covalent_radii for elements {missing} when ase is not installed")
        for z in missing:
            given[z] = float(table[z])
    return given


def _set_nested(root: torch.nn.Module, dotted: str, tensor: torch.Tensor, buffer: bool) -> None:
    parts = dotted.split(".")
    mod = root
    for p in parts[:-1]:
        if p not in mod._modules:
            mod.add_module(p, torch.nn.Module())
        mod = mod._modules[p]
    if buffer:
        mod.register_buffer(parts[-1], tensor)
    else:
        mod.register_parameter(parts[-1], torch.nn.Parameter(tensor, requires_grad=False))


class e3nnTACE(torch.nn.Module):
    """Parameter container with the reference constructor and state_dict layout.

    Weights are drawn like the reference's initialisers (unit normal for the equivariant
    linears, U(-sqrt3, sqrt3) for the radial MLP, zero biases; ``tace/models/linear.py:260-261,
    331-337, 428-431``) from the global torch generator."""

    def __init__(self, Lmax: int = None, lmax: int = None, num_layers: int = None, num_channel: int = None,
                 cutoff: float = None, statistics: List[Dict] = None, target_property: List[str] = None,
                 max_neighbors: Union[int, None] = None, fidelity: Dict = None, node_embedding: Dict = None,
                 edge_embedding: Dict = None, edge_update: Dict = None, radial_basis: Dict = None, atomic_basis: Dict = None,
                 product_basis: Dict = None, readout_emlp: Dict = None, scale_shift: Dict = None, short_range: Dict = None,
                 long_range: Dict = None, universal_embedding: Dict = None, special: Dict = {}, resnet: Dict = {},
                 layer_norm: Dict = {}, normalizer: Dict = {}, parity: bool = False, mmax: int = 2, mag_Lmax: int = 1,
                 dropout: Dict = {}, embedding_property=[], atomic_numbers=None, **kwargs):
        cfg = {k: v for k, v in locals().items() if k not in ("self", "kwargs", "__class__") and not k.startswith("_")}
        cfg.update(kwargs)
        self.model_config = copy.deepcopy(cfg)
        if universal_embedding:
            _require(not any(v.get("enable") for v in universal_embedding.values()), "no universal embeddings")
        cfg.pop("universal_embedding", None)
        for k in ("special", "resnet", "layer_norm", "normalizer", "dropout"):
            if not cfg.get(k):
                cfg.pop(k, None)
        if cutoff is None:
            raise ValueError("cutoff is required")
        cfg = check_model_config(cfg)
        super().__init__()
        self.cfg = cfg
        self.fidelity = [cfg["fidelity"]] if isinstance(cfg["fidelity"], dict) else cfg["fidelity"]
        self.num_fidelities = len(cfg["statistics"])
        self.max_neighbors = None
        self.target_property = list(cfg["target_property"])
        self.num_layers = cfg["num_layers"]
        self.statistics = cfg["statistics"]
        self.embedding_property = []
        self.num_elements = len(cfg["atomic_numbers"])
        self.num_channel = cfg["num_channel"]
        dt = torch.get_default_dtype()
        rc = float(cfg["cutoff"])
        nb = cfg["radial_basis"]["num_radial_basis"]
        self.plan = ModelPlan(cfg["lmax"], cfg["num_layers"], cfg["num_channel"], self.num_elements,
                              cfg["product_basis"]["correlation"][0], cfg["readout_emlp"]["hidden"][0], nb, 64,
                              Lnode=cfg["Lmax"], use_alllayer=cfg["readout_emlp"]["use_alllayer"], gate_m0=cfg["atomic_basis"]["gate_m0"],
                              mlp_layers=len(cfg["radial_basis"]["hidden"]), mlp_bias=cfg["radial_basis"]["bias"],
                              apply_cutoff=cfg["radial_basis"]["apply_cutoff"],
                              element2=cfg["edge_update"]["type"] == "element2", num_fidelities=self.num_fidelities,
                              product_bilinear=cfg["product_basis"]["nonlinear"] == "silu_bilineargate",
                              tece_layers=[t for t, k in enumerate(cfg["atomic_basis"]["type"]) if k == "uv_so2"], mmax=cfg["mmax"],
                              num_head=cfg["atomic_basis"]["num_head"], edge_ace_hidden=cfg["atomic_basis"]["edge_ace_hidden"],
                              edge_act=cfg["atomic_basis"]["edge_nonlinear"].split("_")[1],
                              resnet_type=cfg["resnet"]["linear_type"], product_agnostic=cfg["product_basis"]["agnostic"],
                              density={"avg_num_neighbors": 0, "density": 1, "no_cutoff_density": 2}[cfg["atomic_basis"]["scatter_norm"]],
                              zbl=0 if not cfg["short_range"]["zbl"]["enable"] else (1 if cfg["scale_shift"]["scale_zbl"] else 2))
        self.register_buffer("cutoff", torch.tensor(rc, dtype=dt))
        self.register_buffer("atomic_numbers", torch.tensor(cfg["atomic_numbers"], dtype=torch.int64))
        for name, shape in self.plan.parameter_shapes().items():
            if name.endswith(".bias"):
                value = torch.zeros(shape, dtype=dt)
            elif ".edge_updates." in name:  # tace/models/_e3nn/edge.py:216-221
                value = torch.empty(shape, dtype=dt).uniform_(-0.001, 0.001)
            elif name.endswith("rejector.temperature_logit"):  # oam_2026_07_05.py:687-697: temperature 1
                value = torch.full(shape, math.log((1.0 - 0.25) / (4.0 - 1.0)), dtype=dt)
            elif "rejector.radial_proj" in name:  # zero-initialised (oam_2026_07_05.py:681-682)
                value = torch.zeros(shape, dtype=dt)
            elif name.endswith(".alpha"):  # tace/models/_e3nn/inter.py:109-110
                value = torch.tensor(float(cfg["avg_num_neighbors"]), dtype=dt)
            elif name.endswith(".beta"):
                value = torch.zeros((), dtype=dt)
            elif ".edge_density.mlp." in name:
                value = torch.empty(shape, dtype=dt).uniform_(-math.sqrt(3.0), math.sqrt(3.0))
            elif ".edge_info.mlp." in name and len(shape) == 1:  # LayerNorm scale (torch.nn.LayerNorm default)
                value = torch.ones(shape, dtype=dt)
            elif ".edge_info.mlp." in name:
                value = torch.empty(shape, dtype=dt).uniform_(-math.sqrt(3.0), math.sqrt(3.0))
            else:
                value = torch.randn(shape, dtype=dt)
            _set_nested(self, name, value, buffer=False)
        rb = "representation.radial_basis."
        _set_nested(self, "representation.atomic_numbers", torch.tensor(cfg["atomic_numbers"], dtype=torch.int64), True)
        _set_nested(self, rb + "radial_fn.bessel_weights", math.pi / rc * torch.linspace(1.0, nb, nb, dtype=dt), True)
        _set_nested(self, rb + "radial_fn.cutoff", torch.tensor(rc, dtype=dt), True)
        _set_nested(self, rb + "radial_fn.prefactor", torch.tensor(math.sqrt(2.0 / rc), dtype=dt), True)
        _set_nested(self, rb + "cutoff_fn.p", torch.tensor(cfg["radial_basis"]["polynomial_cutoff"], dtype=torch.int), True)
        _set_nested(self, rb + "cutoff_fn.cutoff", torch.tensor(rc, dtype=dt), True)
        zs = cfg["atomic_numbers"]
        ae = [{int(k): float(v) for k, v in d.items()} for d in cfg["atomic_energies"]]
        _set_nested(self, "atomic_energy_layer.atomic_energy",
                    torch.tensor([[d.get(int(z), 0.0) for z in zs] for d in ae], dtype=dt), True)
        sk = cfg["scale_shift"]["scale_type"]
        scale = [[float({int(k): float(v) for k, v in (s[sk] if sk else {}).items()}.get(int(z), 1.0)) for z in zs]
                 for s in cfg["statistics"]]
        _set_nested(self, "scale_shift.scale", torch.tensor(scale, dtype=dt), True)
        _set_nested(self, "scale_shift.shift", torch.zeros(len(scale), len(zs), dtype=dt), True)
        _set_nested(self, "scale_shift.atomic_numbers", torch.tensor(zs, dtype=torch.int64), True)
        if cfg["short_range"]["zbl"]["enable"]:  # buffers of the reference's ZBLBasis (tace/models/radial.py:797-819)
            _require(not cfg["short_range"]["zbl"].get("trainable", False), "short_range.zbl.trainable = False")
            radii = torch.zeros(max(119, max(zs) + 1), dtype=dt)
            for z, r in cfg["short_range"]["zbl"]["covalent_radii"].items():
                radii[int(z)] = float(r)
            _set_nested(self, "zbl.c", torch.tensor([0.1818, 0.5099, 0.2802, 0.02817], dtype=dt), True)
            _set_nested(self, "zbl.p", torch.tensor(cfg["radial_basis"]["polynomial_cutoff"], dtype=torch.int), True)
            _set_nested(self, "zbl.covalent_radii", radii, True)
            _set_nested(self, "zbl.a_exp", torch.tensor(0.300), True)
            _set_nested(self, "zbl.a_prefactor", torch.tensor(0.4543), True)

    def forward(self, data, graph=None):
        raise RuntimeError("call the TensorModel wrapper; the model body runs inside libtace_b200.so")


cartTACE = e3nnTACE  # the reference exports the same architecture under both names (tace/models/__init__.py:4-7)


class _Flags:
    pass


class TensorModel(torch.nn.Module):
    """``TensorModel(readout_fn)`` with the reference's ``forward(data)`` contract."""

    def __init__(self, readout_fn: e3nnTACE):
        super().__init__()
        self.readout_fn = readout_fn
        self.num_fidelities = readout_fn.num_fidelities
        self.lmp = False
        self.fidelity_idx = 0
        self._handle = None
        self._handle_key = None
        self._workspace = None
        self._graph_mode = os.environ.get("TACE_B200_GRAPHS", "1") != "0"
        self._sized_for, self._sized_bytes = None, 0  # batch shape the workspace size was last computed for
        self._radial_table = True   # see set_radial_table
        self._exchange_overlap = os.environ.get("TACE_B200_EXCHANGE_OVERLAP", "0") == "1"  # see set_exchange_overlap
        self._exchange_stream = None
        self.uses_radial_table = False
        # TACE_B200_CHUNK_EDGES=<n>: fixed edge-chunk size for every model instead of the automatic choice
        self._chunk_edges = int(os.environ["TACE_B200_CHUNK_EDGES"]) if os.environ.get("TACE_B200_CHUNK_EDGES") else None
        self._auto_chunk = None
        self._set_target_property()

    # ---- reference getters (tace/models/adapter.py:386-452) ----------------------------------
    def get_fidelity_idx(self) -> int:
        return int(self.fidelity_idx)

    def reset_fidelity_idx(self, fidelity_idx: Union[int, None] = 0) -> None:
        """tace/models/adapter.py:389-391: the head used when ``data`` carries no ``fidelity_idx``."""
        if fidelity_idx is not None:
            if not 0 <= int(fidelity_idx) < self.num_fidelities:
                raise ValueError(f"fidelity_idx {fidelity_idx} outside 0..{self.num_fidelities - 1}")
            self.fidelity_idx = int(fidelity_idx)

    def get_embedding_property(self) -> List[str]:
        return []

    def get_target_property(self) -> List[str]:
        return list(set(self.readout_fn.target_property))

    def reset_target_property(self, target_property: List[str]) -> None:
        assert isinstance(target_property, list)
        _require(set(target_property) <= _SUPPORTED_TARGETS, f"targets within {sorted(_SUPPORTED_TARGETS)}")
        self.readout_fn.target_property = target_property
        self._set_target_property()

    def _set_target_property(self) -> None:
        self.flags = _Flags()
        for k in _SUPPORTED_TARGETS:
            setattr(self.flags, f"compute_{k}", k in self.get_target_property())

    def _set_lammps_mliap(self, enable: bool = False) -> None:
        self.lmp = enable

    def get_model_dtype(self) -> torch.dtype:
        return self.readout_fn.cutoff.dtype

    def get_max_neighbors(self):
        return None

    def get_cutoff(self) -> float:
        return float(self.readout_fn.cutoff.item())

    def get_atomic_numbers(self) -> List[int]:
        return [int(z) for z in self.readout_fn.atomic_numbers.cpu().tolist()]

    # ---- native model handle ----------------------------------------------------------------------
    def _native(self, device: torch.device):
        rf = self.readout_fn
        dtype = self.get_model_dtype()
        key = (device.index, dtype, sum(int(p._version) for p in rf.state_dict().values()))
        if self._handle is not None and key == self._handle_key:
            return self._handle
        self.release()
        self._auto_chunk = None
        self._sized_for = None
        lib = _lib.load()
        plan = rf.plan
        cfg = _lib.TaceConfig(
            dtype=_lib.TACE_F64 if dtype == torch.float64 else _lib.TACE_F32, L=plan.L, num_layers=plan.num_layers,
            num_channel=plan.Cp, num_elements=plan.n_el, correlation=plan.correlation, num_bessel=plan.num_bessel,
            mlp_hidden=plan.mlp_hidden, envelope_p=int(rf.cfg["radial_basis"]["polynomial_cutoff"]), readout_hidden=plan.H,
            cutoff=self.get_cutoff(), avg_num_neighbors=float(rf.cfg["avg_num_neighbors"]), Lnode=plan.Lnode,
            use_alllayer=int(plan.use_alllayer), gate_m0_off=int(not plan.gate_m0), mlp_layers=plan.mlp_layers,
            mlp_bias=int(plan.mlp_bias), env_after_mlp=int(not plan.apply_cutoff), edge_update_element2=int(plan.element2),
            num_fidelities=plan.n_fid, zbl=plan.zbl, scatter_norm_density=plan.density,
            resnet_identity=int(plan.resnet_type == "identity"), product_bilinear=int(plan.bilinear),
            tece_layers=sum(1 << t for t in plan.tece_layers), mmax=plan.mmax, num_head=plan.num_head,
            edge_ace_hidden=plan.edge_ace_hidden, edge_act=0 if plan.edge_act == "sigmoid" else 1)
        # With the identity edge update the radial MLP's output depends on the edge length only: fp32 models read it
        # from a table (TaceConfig.radial_table) instead of evaluating the MLP per edge.  TACE_B200_RADIAL_TABLE=0
        # keeps the per-edge MLP.
        table = (dtype == torch.float32 and not plan.element2 and not plan.tece_layers
                 and os.environ.get("TACE_B200_RADIAL_TABLE", "1") != "0" and self._radial_table)
        env_p = int(rf.cfg["radial_basis"]["polynomial_cutoff"])
        cfg.radial_table = RADIAL_TABLE_INTERVALS if table else 0
        self.uses_radial_table = bool(table)
        handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(lib.tace_create(ctypes.byref(cfg), ctypes.byref(handle)), "tace_create")
            packed = pack_weights(plan, rf.state_dict(), float(rf.cfg["avg_num_neighbors"]),
                                  radial_table_spec=(self.get_cutoff(), env_p, RADIAL_TABLE_INTERVALS) if table else None)
            npdt = np.float64 if dtype == torch.float64 else np.float32
            name, numel = ctypes.c_char_p(), ctypes.c_int64()
            for i in range(lib.tace_weight_count(handle)):
                _lib.check(lib.tace_weight_info(handle, i, ctypes.byref(name), ctypes.byref(numel)), "tace_weight_info")
                arr = np.ascontiguousarray(packed[name.value.decode()], dtype=npdt).reshape(-1)
                if arr.size != numel.value:
                    raise _lib.TaceError(f"weight {name.value.decode()}: packed {arr.size} elements, library expects {numel.value}")
                _lib.check(lib.tace_set_weight(handle, name.value, arr.ctypes.data_as(ctypes.c_void_p), arr.size), "tace_set_weight")
            _lib.check(lib.tace_set_graph_mode(handle, int(self._graph_mode)), "tace_set_graph_mode")
            if self._chunk_edges is not None:
                _lib.check(lib.tace_set_chunk_edges(handle, int(self._chunk_edges)), "tace_set_chunk_edges")
        self._handle, self._handle_key = handle, key
        return handle

    def set_graph_mode(self, enable: bool = True) -> None:
        """Replay repeated evaluations of one batch shape as a CUDA graph (default on; the environment
        variable TACE_B200_GRAPHS=0 turns it off for every model)."""
        self._graph_mode = bool(enable)
        if self._handle is not None:
            _lib.check(_lib.load().tace_set_graph_mode(self._handle, int(self._graph_mode)), "tace_set_graph_mode")

    def set_radial_table(self, enable: bool = True) -> None:
        """fp32 models with the identity edge update read the radial path weights from a per-(path, channel) table of
        the edge length (cubic Hermite, 512 intervals) instead of evaluating the radial MLP for every edge; ``False``
        goes back to the per-edge MLP.  Takes effect when the native model is (re)built."""
        if bool(enable) != self._radial_table:
            self._radial_table = bool(enable)
            self.release()

    def set_exchange_overlap(self, enable: bool = True) -> None:
        """Run stream-ordered ghost exchanges (``tace_b200.domain.HaloExchange``) on a stream of their own while the layer
        works on the atoms without ghost neighbours (``tace_set_exchange_stream``).  Off by default (the environment
        variable TACE_B200_EXCHANGE_OVERLAP=1 turns it on for every model): over NVLink the exchange inside an evaluation
        is about 1 % of a step of the 1 M-atom benchmark, less than what splitting the tensor-product passes costs; it
        is meant for interconnects where the exchange is slow."""
        self._exchange_overlap = bool(enable)

    def set_chunk_edges(self, max_edges: Optional[int]) -> None:
        """Batches with more edges than this are evaluated chunk by chunk of target atoms with the per-edge tensors
        recomputed in the backward pass (library default 2**21 edges)."""
        self._chunk_edges = None if max_edges is None else int(max_edges)
        self._sized_for = None
        if self._handle is not None and max_edges is not None:
            _lib.check(_lib.load().tace_set_chunk_edges(self._handle, int(max_edges)), "tace_set_chunk_edges")

    def graph_replays(self) -> int:
        return int(_lib.load().tace_graph_replays(self._handle)) if self._handle is not None else 0

    def release(self) -> None:
        if self._handle is not None:
            _lib.load().tace_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    def __getstate__(self):
        state = self.__dict__.copy()
        state["_handle"], state["_handle_key"], state["_workspace"] = None, None, None
        state["_exchange_stream"] = None
        return state

    def _get_workspace(self, nbytes: int, device: torch.device) -> torch.Tensor:
        ws = self._workspace
        if ws is None or ws.numel() < nbytes or ws.device != device:
            self._workspace = None
            # head room for batches that grow a little (an MD run re-partitions every few dozen steps and its edge count
            # drifts by a per cent or so): growing means a second allocation of the full size beside the cached old one
            # and tens of milliseconds in the allocator
            ws = torch.empty(int(nbytes + min(0.1 * nbytes, 4 << 30)) + 4096, dtype=torch.uint8, device=device)
            self._workspace = ws
        return ws

    # ---- forward -------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, data: Dict[str, torch.Tensor]) -> Dict[str, Optional[torch.Tensor]]:
        lib = _lib.load()
        dtype = self.get_model_dtype()
        node_attrs = data.get("node_attrs")
        device = (node_attrs if node_attrs is not None else data["species"]).device
        if device.type != "cuda":
            raise _lib.TaceError("tace_b200 runs on CUDA devices only (no CPU path)")
        handle = self._native(device)
        flags = self.flags
        species = data["species"] if "species" in data else node_attrs.argmax(dim=-1)
        species = species.to(torch.int32).contiguous()
        edge_index = data["edge_index"].to(torch.int64).contiguous()
        E = int(edge_index.shape[1])
        keep = [species, edge_index]

        def real(x):
            x = x.detach().to(dtype).contiguous()
            keep.append(x)
            return x

        batch = _lib.TaceBatch()
        if self.lmp:
            nlocal, nghost = int(data["natoms"][0]), int(data["natoms"][1])
            n_atoms, n_local, n_graphs = nlocal + nghost, nlocal, 1
            graph_ptr = torch.tensor([0, nlocal], dtype=torch.int32, device=device)
            if n_atoms == 0:  # a rank of a domain decomposition that neither owns nor sees any atom
                zeros = lambda *shape: torch.zeros(*shape, dtype=dtype, device=device)
                return {"energy": zeros(1), "node_energy": zeros(0), "forces": zeros(0, 3) if flags.compute_forces else None,
                        "virials": None, "stress": None, "edge_forces": zeros(0, 3)}
            # an empty edge list (a rank that owns no atom) still has to say "edge-vector mode": never a NULL pointer
            vec = data["edge_vector"] if E > 0 else torch.zeros(1, 3, dtype=dtype, device=device)
            batch.edge_vector = real(vec).data_ptr()
        else:
            n_atoms = n_local = int(species.shape[0])
            graph_ptr = data["ptr"].to(torch.int32).contiguous()
            n_graphs = int(graph_ptr.numel() - 1)
            batch.positions = real(data["positions"]).data_ptr()
            batch.lattice = real(data["lattice"]).reshape(-1, 3, 3).data_ptr()
            batch.edge_shifts = real(data["edge_shifts"]).data_ptr()
        keep.append(graph_ptr)
        batch.n_atoms, batch.n_local, batch.n_edges, batch.n_graphs = n_atoms, n_local, E, n_graphs
        batch.species, batch.graph_ptr, batch.edge_index = species.data_ptr(), graph_ptr.data_ptr(), edge_index.data_ptr()
        if self.num_fidelities > 1:  # tace/models/adapter.py:280-284
            if "fidelity_idx" in data:
                fid = data["fidelity_idx"].to(device=device, dtype=torch.int32).contiguous()
                if fid.numel() != n_graphs or int(fid.min()) < 0 or int(fid.max()) >= self.num_fidelities:
                    raise ValueError("fidelity_idx must hold one head index in 0..num_fidelities-1 per graph")
            else:
                fid = torch.full((n_graphs,), int(self.fidelity_idx), dtype=torch.int32, device=device)
            keep.append(fid)
            batch.fidelity = fid.data_ptr()

        out = _lib.TaceOutputs()
        res: Dict[str, Optional[torch.Tensor]] = {k: None for k in
                                                   ("energy", "node_energy", "forces", "virials", "stress", "edge_forces")}
        res["energy"] = torch.empty(n_graphs, dtype=dtype, device=device)
        res["node_energy"] = torch.empty(n_local, dtype=dtype, device=device)
        out.energy, out.node_energy = res["energy"].data_ptr(), res["node_energy"].data_ptr()
        if flags.compute_forces:  # edge-vector mode: rows of ghost atoms hold the force parts that belong to their owners
            res["forces"] = torch.empty(n_atoms, 3, dtype=dtype, device=device)
            out.forces = res["forces"].data_ptr()
        if (flags.compute_stress or flags.compute_virials) and not self.lmp:
            res["virials"] = torch.empty(n_graphs, 3, 3, dtype=dtype, device=device)
            res["stress"] = torch.empty(n_graphs, 3, 3, dtype=dtype, device=device)
            out.virials, out.stress = res["virials"].data_ptr(), res["stress"].data_ptr()
        if flags.compute_edge_forces or self.lmp:
            res["edge_forces"] = torch.empty(E, 3, dtype=dtype, device=device)
            out.edge_forces = res["edge_forces"].data_ptr()

        exchange_cb = None
        if self.lmp and n_atoms != n_local and self.readout_fn.num_layers > 1:
            # an exchange object that enqueues everything on the current stream (tace_b200.domain.HaloExchange) says so
            # with `stream_ordered`; LAMMPS' own exchange does not, and gets a synchronised stream on both sides
            ordered = bool(getattr(data["lmp_data"], "stream_ordered", False))
            # such an exchange can also run on a stream of its own while the layer works on the edges between owned atoms
            side = None
            if ordered and self._exchange_overlap:
                if self._exchange_stream is None or self._exchange_stream.device != device:
                    self._exchange_stream = torch.cuda.Stream(device, priority=-1)
                side = self._exchange_stream
            exchange_cb = self._make_exchange(data["lmp_data"], dtype, device, sync=not ordered, stream=side)
            _lib.check(lib.tace_set_exchange(handle, exchange_cb, None), "tace_set_exchange")
            _lib.check(lib.tace_set_exchange_sync(handle, 0 if ordered else 1), "tace_set_exchange_sync")
            _lib.check(lib.tace_set_exchange_stream(handle, side.cuda_stream if side is not None else None), "tace_set_exchange_stream")
        with torch.cuda.device(device):
            nbytes = ctypes.c_size_t()

            def needed() -> int:
                _lib.check(lib.tace_workspace_bytes(handle, n_atoms, n_local, E, n_graphs, ctypes.byref(nbytes)), "tace_workspace_bytes")
                return int(nbytes.value)

            shape_key = (n_atoms, n_local, E, n_graphs, device.index)

            def set_limit(limit: int) -> None:
                if limit != self._auto_chunk:
                    _lib.check(lib.tace_set_chunk_edges(handle, int(limit)), "tace_set_chunk_edges")
                    self._auto_chunk = limit

            if self._chunk_edges is None and shape_key != self._sized_for:
                # automatic edge chunking: keep every per-edge tensor resident when the workspace fits in
                # 80 % of the memory this model may use, otherwise halve the chunk size until it does.  Decided once
                # per batch shape, and without asking the driver when the whole batch fits into the workspace this
                # model already holds: the memory query can take longer than the evaluation itself (up to ~20 ms seen).
                whole = max(E, 1 << 21)
                held = self._workspace.numel() - 512 if self._workspace is not None and self._workspace.device == device else -1
                fits = False
                for limit in (whole, self._auto_chunk):  # the whole batch, else the chunk size chosen last time
                    if limit is not None and limit <= whole and not fits:
                        set_limit(limit)
                        fits = needed() <= held
                if not fits:
                    free, _total = torch.cuda.mem_get_info(device)
                    budget = 0.8 * (free + (self._workspace.numel() if self._workspace is not None else 0))
                    whole_only = bool(self.readout_fn.plan.tece_layers)  # the TECE edge block is evaluated on the whole batch only
                    for limit in ((whole,) if whole_only else (whole, 1 << 22, 1 << 21, 1 << 20, 1 << 19, 1 << 18)):
                        set_limit(limit)
                        if needed() <= budget or limit == 1 << 18:
                            break
                        if whole_only:
                            raise _lib.TaceError(f"tace_b200: this batch needs {needed() / 2**30:.1f} GiB of workspace with the TECE edge block "
                                                 f"(all per-edge tensors resident), {budget / 2**30:.1f} GiB are available; use smaller batches")
            if shape_key != self._sized_for or self._workspace is None:
                needed()
                self._sized_bytes = int(nbytes.value)
                self._sized_for = shape_key
            ws = self._get_workspace(self._sized_bytes, device)
            ws_ptr = (ws.data_ptr() + 255) & ~255
            stream = torch.cuda.current_stream(device).cuda_stream
            self._exchange_error = None
            try:
                _lib.check(lib.tace_forward(handle, ctypes.byref(batch), ctypes.byref(out), ws_ptr,
                                            ws.numel() - (ws_ptr - ws.data_ptr()), stream), "tace_forward")
            except _lib.TaceError as exc:
                if self._exchange_error is not None:  # the callback failed: show its exception, not the bare status
                    raise self._exchange_error from exc
                raise
            finally:
                # the handle must never keep a pointer to a callback object that dies with this frame
                if exchange_cb is not None:
                    lib.tace_set_exchange(handle, _lib.EXCHANGE_FN(0), None)
        return res

    def _make_exchange(self, lmp_data, dtype: torch.dtype, device: torch.device, sync: bool = True, stream=None):
        """ctypes callback handing the workspace rows to ``lmp_data.forward_exchange`` /
        ``reverse_exchange`` as torch views (tace/models/lammps.py:82-102).  With ``stream`` the exchange's own work is
        enqueued on that stream (the library orders it against the evaluation, tace_set_exchange_stream)."""
        import contextlib
        itemsize = torch.empty((), dtype=dtype).element_size()

        def view(ptr: int, rows: int, cols: int) -> torch.Tensor:
            ws = self._workspace
            off = ptr - ws.data_ptr()
            return ws[off:off + rows * cols * itemsize].view(dtype).view(rows, cols)

        def callback(_user, reverse, in_ptr, out_ptr, n_rows, vec_len):
            try:
                src, dst = view(in_ptr, n_rows, vec_len), view(out_ptr, n_rows, vec_len)
                with (torch.cuda.stream(stream) if stream is not None else contextlib.nullcontext()):
                    if reverse:
                        lmp_data.reverse_exchange(src, dst, vec_len)
                    else:
                        lmp_data.forward_exchange(src, dst, vec_len)
                if sync:
                    torch.cuda.synchronize(device)
                return 0
            except Exception as exc:  # an exception must not cross the C boundary
                self._exchange_error = exc
                return 1

        return _lib.EXCHANGE_FN(callback)

    def device_error(self) -> int:
        """Non-zero if a bounded wait inside a kernel expired since the last check (synchronises)."""
        if self._handle is None:
            return 0
        code = ctypes.c_int32()
        _lib.check(_lib.load().tace_device_error(self._handle, ctypes.byref(code)), "tace_device_error")
        return int(code.value)

    def launch_count(self) -> int:
        """Kernels of libtace_b200.so enqueued by this model's forward calls so far."""
        return int(_lib.load().tace_launch_count(self._handle)) if self._handle is not None else 0

    def enable_profile(self, enable: bool = True) -> None:
        """Record a CUDA event at every phase boundary of forward (see ``read_profile``)."""
        if self._handle is None:
            raise _lib.TaceError("run one forward call before enabling the profile")
        _lib.check(_lib.load().tace_profile_enable(self._handle, int(enable)), "tace_profile_enable")

    def read_profile(self) -> Dict[str, float]:
        """Phase name -> device milliseconds of the last forward call (synchronises)."""
        lib = _lib.load()
        out: Dict[str, float] = {}
        name, ms = ctypes.c_char_p(), ctypes.c_float()
        for i in range(lib.tace_profile_count(self._handle)):
            _lib.check(lib.tace_profile_read(self._handle, i, ctypes.byref(name), ctypes.byref(ms)), "tace_profile_read")
            out[name.value.decode()] = out.get(name.value.decode(), 0.0) + float(ms.value)
        return out

    def debug_read(self, name: str, numel: int) -> torch.Tensor:
        """Copy a named intermediate of the last forward call (parity tests)."""
        lib = _lib.load()
        device = self._workspace.device
        buf = torch.empty(numel, dtype=self.get_model_dtype(), device=device)
        n = lib.tace_debug_read(self._handle, name.encode(), buf.data_ptr(), numel, torch.cuda.current_stream(device).cuda_stream)
        if n < 0:
            raise _lib.TaceError(f"tace_debug_read({name}): status {n}")
        return buf[:n]


def create_model(model_config: Dict, statistics=None, target_property=None, **_) -> TensorModel:
    """``TensorModel(e3nnTACE(**model_config))`` as tace/lightning/torch_model.py:54-114 builds it."""
    cfg = dict(model_config)
    cfg.pop("_target_", None)
    if statistics is not None:
        cfg["statistics"] = statistics
    if target_property is not None:
        cfg["target_property"] = target_property
    return TensorModel(e3nnTACE(**cfg))
