"""Model plan (path bookkeeping) and repacking of reference-named parameters into the
arrays ``libtace_b200.so`` consumes.

Parameter names, flat-weight order and normalisation constants follow the reference
(paths relative to its project root):

* flat linear weights = concatenation, in (input block, output block) order, of
  ``[mul_in, mul_out]`` matrices, each used with the factor 1/sqrt(fan_in)
  (``tace/models/linear.py:282-374`` over e3nn ``o3.Linear``);
* tensor-product paths are enumerated output-rank major, then first input, then second
  (``tace/models/_e3nn/paths.py:30-71``); the radial MLP emits one weight per (path, channel),
  path major (``tace/models/_e3nn/inter.py:92-99,180``);
* radial MLP layers carry 1/sqrt(fan_in) and, after the first, a sqrt(2) gain
  (``tace/models/mlp.py:155-170``);
* messages are divided by ``avg_num_neighbors`` after ``linear_down``
  (``tace/models/_e3nn/base.py:240-249``), folded into that layer's weights here.
"""

from __future__ import annotations

import math
from typing import Dict, List

import numpy as np


def tp_paths(in1_ls, in2_ls, out_ls):
    return [(l1, l2, l3) for l3 in out_ls for l1 in in1_ls for l2 in in2_ls
            if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0]


class LayerPlan:
    """``L``: rank of the angular features and of the atomic basis A (the reference's ``lmax``); ``Lnode``: rank of
    the node features between layers (``Lmax``), tace/models/_e3nn/base.py:113-360."""

    def __init__(self, t: int, num_layers: int, L: int, Lnode: int = None, correlation: int = 2, bilinear: bool = False,
                 tece: bool = False, mmax: int = 2):
        Lnode = L if Lnode is None else Lnode
        self.tece = bool(tece)  # the interaction is the TECE edge block (atomic_basis.type = uv_so2)
        self.t = t
        self.scalar_src = t == 0 or Lnode == 0
        self.last = t == num_layers - 1
        self.has_res = t > 0
        all_ls = list(range(L + 1))
        node_ls = list(range(Lnode + 1))
        self.in_ls = [0] if t == 0 else node_ls
        self.out_ls = [0] if self.last else node_ls
        self.tp_paths = tp_paths(self.in_ls, all_ls, all_ls)
        self.k = [sum(1 for p in self.tp_paths if p[2] == l) for l in all_ls]
        self.radial_out = len(self.tp_paths)  # radial-MLP outputs per channel
        if self.tece:
            # messages arrive as one block of channels per rank; the radial MLP weights every (order, rank >= order) row of the
            # source | target features (tace/models/_e3nn/archive/oam_2026_07_05.py:586-588)
            self.k = [1] * (L + 1)
            self.radial_out = 2 * sum(L + 1 - m for m in range(mmax + 1))
        # second-order product basis: with a third order behind it every rank <= L keeps its paths (each path is a
        # slot of the next product), otherwise only the output ranks (tace/models/_e3nn/prod.py:216-266)
        self.pb_paths = tp_paths(all_ls, all_ls, all_ls if correlation >= 3 else self.out_ls)
        if bilinear:
            # gated bilinear product (tace/models/_e3nn/prod.py:87-111): the second factor carries an extra block of ones
            # (l2 = -1 here), which adds the path l1 = l3; no symmetry between the factors
            self.pb_paths = [q for l3 in self.out_ls for l1 in all_ls
                             for q in ([(l1, l2, l3) for l2 in all_ls if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0]
                                       + ([(l1, -1, l3)] if l1 == l3 else []))]
        self.kp = [sum(1 for p in self.pb_paths if p[2] == l) for l in self.out_ls]
        self.pb3_paths = []
        if correlation >= 3:
            self.pb3_paths = [(s, lb, l3) for l3 in self.out_ls for s, (_, _, ls_) in enumerate(self.pb_paths) for lb in all_ls
                              if abs(ls_ - lb) <= l3 <= ls_ + lb and (ls_ + lb + l3) % 2 == 0]
        self.kp3 = [sum(1 for p in self.pb3_paths if p[2] == l) for l in self.out_ls]


class ModelPlan:
    def __init__(self, L: int, num_layers: int, num_channel: int, num_elements: int, correlation: int,
                 readout_hidden: int = 16, num_bessel: int = 8, mlp_hidden: int = 64, Lnode: int = None,
                 use_alllayer: bool = False, gate_m0: bool = True, mlp_layers: int = 3, mlp_bias: bool = False,
                 apply_cutoff: bool = True, element2: bool = False, num_fidelities: int = 1, zbl: int = 0,
                 density: int = 0, resnet_type: str = "aware", product_agnostic: bool = False, product_bilinear: bool = False,
                 tece_layers=(), mmax: int = 2, num_head: int = 1, edge_ace_hidden: int = None, edge_act: str = "sigmoid"):
        self.L, self.num_layers, self.C, self.n_el = L, num_layers, num_channel, num_elements
        self.Cp = 32 * ((num_channel + 31) // 32)  # channel count the kernels run with (zero-padded, see pad_channels)
        self.Lnode = L if Lnode is None else Lnode
        self.use_alllayer = bool(use_alllayer)
        # read-out heads (one per `statistics` entry); ZBL repulsion: 0 off, 1 inside the species scale, 2 outside
        self.n_fid, self.zbl = int(num_fidelities), int(zbl)
        # atomic_basis.scatter_norm: 0 avg_num_neighbors, 1 density, 2 no_cutoff_density (learned edge density)
        self.density = int(density)
        # resnet.linear_type: aware (per-species linear), agnostic (one linear), identity (copy); product_basis.agnostic:
        # one coefficient matrix for all species instead of one per species
        self.resnet_type, self.product_agnostic = resnet_type, bool(product_agnostic)
        self.bilinear = bool(product_bilinear)  # product_basis.nonlinear = silu_bilineargate
        if self.bilinear and (correlation != 2 or self.Cp != self.C):
            raise NotImplementedError("tace_b200: silu_bilineargate needs correlation 2 and a channel count that is a multiple of 32")
        self.gate_m0 = bool(gate_m0)  # False: scalars are not gated, so linear_down emits one scalar block less
        # radial MLP: hidden layers (all mlp_hidden wide), biases, envelope before (True) or after the MLP; edge update
        self.mlp_layers, self.mlp_bias, self.apply_cutoff, self.element2 = int(mlp_layers), bool(mlp_bias), bool(apply_cutoff), bool(element2)
        self.correlation, self.H, self.num_bessel, self.mlp_hidden = correlation, readout_hidden, num_bessel, mlp_hidden
        # TECE edge block: which interactions use it, orders kept, heads, width of the edge cluster expansion, activation
        self.tece_layers, self.mmax, self.num_head = tuple(sorted(tece_layers)), int(mmax), int(num_head or 1)
        self.edge_ace_hidden, self.edge_act = int(edge_ace_hidden or num_channel), edge_act
        if self.tece_layers and (self.Cp != self.C or self.Lnode != L or 0 in self.tece_layers or not 0 <= self.mmax <= min(2, L)
                                 or self.C % self.num_head or self.edge_ace_hidden % 4):
            raise NotImplementedError("tace_b200: uv_so2 interactions need Lmax == lmax, mmax <= 2, a channel count that is a multiple "
                                      "of 32 and of num_head, and cannot be the first layer")
        self.layers = [LayerPlan(t, num_layers, L, self.Lnode, correlation, self.bilinear, t in self.tece_layers, self.mmax)
                       for t in range(num_layers)]

    @property
    def mlp_layer_norm(self) -> bool:
        """Edge features wider than the radial basis (the element-dependent edge update) put a LayerNorm between every
        hidden linear of the radial MLP and its activation (tace/models/_e3nn/base.py:183-185, tace/models/mlp.py:172-176)."""
        return self.element2

    def mlp_index(self, i: int) -> int:
        """Position of the i-th linear inside the radial MLP's ``Sequential`` (linear, [LayerNorm], SiLU, ...)."""
        return (3 if self.mlp_layer_norm else 2) * i

    def so2_linears(self):
        """The six SO(2) linears of the edge block (oam_2026_07_05.py:612-676): reference name, packed name, channels in / out,
        rows per order in / out."""
        n, mm, C, Ca = self.L + 1, self.mmax, self.C, self.edge_ace_hidden
        red, full = [n - m for m in range(mm + 1)], [n] * (mm + 1)
        gates = n * (mm + 1 - (0 if self.gate_m0 else 1))
        n_paths = sum(1 for m3 in range(mm + 1) for m1 in range(mm + 1) for m2 in range(m1 + 1) if m1 + m2 == m3 or m1 - m2 == m3)
        return [("key_proj", "key", C, C, red, red), ("query_proj", "query", C, C, red, red),
                ("linear_up", "up", 2 * C, Ca, red, [gates + n] + full[1:]), ("linear_glu", "glu", 2 * C, Ca, red, full),
                ("linear_coefs", "coefs", 2 * C, 1, red[:1], [n_paths * n * Ca]), ("linear_down", "down", Ca, C, full, red)]

    def tece_shapes(self) -> Dict[str, tuple]:
        out = {}
        for ref, _, ci, co, n_in, n_out in self.so2_linears():
            out[f"rejector.{ref}.m0_rlinear.weight"] = (n_out[0] * co, n_in[0] * ci)
            out[f"rejector.{ref}.m0_rlinear.bias"] = (n_out[0] * co,)
            for m in range(1, len(n_in)):
                out[f"rejector.{ref}.ms_clinear.{m - 1}.fc.weight"] = (n_out[m] * co, n_in[m] * ci)
        out["rejector.radial_proj.weight"] = (2 * self.num_head, self.num_bessel)
        out["rejector.radial_proj.bias"] = (2 * self.num_head,)
        out["rejector.temperature_logit"] = (self.num_head,)
        return out

    def parameter_shapes(self) -> Dict[str, tuple]:
        """Reference parameter names (without the ``readout_fn.`` prefix) and shapes."""
        C, n_el, L = self.C, self.n_el, self.L
        out = {"representation.node_embedding.elem_emb1.weight": (n_el * C,)}
        for lp in self.layers:
            pre = f"representation.interactions.{lp.t}."
            out[pre + "linear_up.weight"] = (len(lp.in_ls) * C * C,)
            out[pre + "linear_up.bias"] = (C,)
            edge_dim = self.num_bessel + (2 * C if self.element2 else 0)
            dims = [edge_dim] + [self.mlp_hidden] * self.mlp_layers + [lp.radial_out * C]
            for i, (a, b) in enumerate(zip(dims, dims[1:])):
                out[pre + f"edge_info.mlp.{self.mlp_index(i)}.weight"] = (a, b)
                if self.mlp_bias:
                    out[pre + f"edge_info.mlp.{self.mlp_index(i)}.bias"] = (b,)
                if self.mlp_layer_norm and i < self.mlp_layers:
                    out[pre + f"edge_info.mlp.{self.mlp_index(i) + 1}.weight"] = (b,)
                    out[pre + f"edge_info.mlp.{self.mlp_index(i) + 1}.bias"] = (b,)
            if lp.tece:
                out.update({pre + k: v for k, v in self.tece_shapes().items()})
            if self.density:  # tace/models/_e3nn/inter.py:102-110
                out[pre + "edge_density.mlp.0.weight"] = (self.num_bessel, self.mlp_hidden)
                out[pre + "edge_density.mlp.2.weight"] = (self.mlp_hidden, 1)
                if self.mlp_bias:
                    out[pre + "edge_density.mlp.0.bias"] = (self.mlp_hidden,)
                    out[pre + "edge_density.mlp.2.bias"] = (1,)
                out[pre + "alpha"] = ()
                out[pre + "beta"] = ()
            if self.element2:  # tace/models/_e3nn/edge.py:190-257
                out[f"representation.edge_updates.{lp.t}.source_embedding.weight"] = (n_el * C,)
                out[f"representation.edge_updates.{lp.t}.target_embedding.weight"] = (n_el * C,)
            n0 = (L + 2) * C if self.gate_m0 else (L + 1) * C
            out[pre + "linear_down.weight"] = (sum(lp.k[l] * C * (n0 if l == 0 else C) for l in range(L + 1)),)
            out[pre + "linear_down.bias"] = (n0,)
            out[pre + "linear_nonlinearity.weight"] = ((L + 1) * C * C,)
            out[pre + "linear_nonlinearity.bias"] = (C,)
            res_lead = (n_el,) if self.resnet_type == "aware" else ()
            if lp.has_res and self.resnet_type != "identity":
                out[pre + "resnetBB.weight"] = res_lead + (len(lp.out_ls) * C * C,)
                out[pre + "resnetBB.bias"] = res_lead + (C,)
            pp = f"representation.products.{lp.t}."
            co_lead = () if self.product_agnostic else (n_el,)
            if self.bilinear:  # prod.py:128-141: gates for every product path, then both factors per rank
                out[pp + "linear_up.weight"] = (C * len(lp.pb_paths) * C + (L + 1) * C * 2 * C,)
                out[pp + "linear_up.bias"] = (len(lp.pb_paths) * C + 2 * C,)
            out[pp + "coefs.0.weight"] = co_lead + (len(lp.out_ls) * C * C,)
            out[pp + "coefs.0.bias"] = co_lead + (C,)
            if self.correlation >= 2:
                out[pp + "coefs.1.weight"] = co_lead + (sum(kp * C * C for kp in lp.kp),)
                out[pp + "coefs.1.bias"] = co_lead + (C,)
            if self.correlation >= 3:
                out[pp + "coefs.2.weight"] = co_lead + (sum(kp * C * C for kp in lp.kp3),)
                out[pp + "coefs.2.bias"] = co_lead + (C,)
            out[pp + "linear.weight"] = (len(lp.out_ls) * C * C,)
            out[pp + "linear.bias"] = (C,)
        # tace/models/_e3nn/readout.py:192-221: with use_alllayer every layer has a read-out (a single linear on
        # the scalar block below the last layer), otherwise the list holds only the last layer's MLP
        ro = self.num_layers - 1 if self.use_alllayer else 0
        if self.use_alllayer:
            for t in range(self.num_layers - 1):
                out[f"energy_readouts.{t}.linear1.0.weight"] = (C * self.n_fid,)
        # hidden width and output count are multiplied by the number of heads (tace/models/_e3nn/base.py:386-396)
        out[f"energy_readouts.{ro}.linear2.0.weight"] = (C * self.H * self.n_fid,)
        out[f"energy_readouts.{ro}.linear2.1.weight"] = (self.H * self.n_fid * self.n_fid,)
        return out


def split_tf32(w: np.ndarray):
    """fp32 value = hi + lo with hi exactly representable in TF32 (low 13 mantissa bits zero)."""
    w32 = np.ascontiguousarray(w, dtype=np.float32)
    hi = (w32.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    return hi, w32 - hi


def tile_k_major(w: np.ndarray, tile: int = 32) -> np.ndarray:
    """[..., N, K] -> [..., K/tile, N, tile] (same number of elements)."""
    n, k = w.shape[-2], w.shape[-1]
    if k % tile:
        raise ValueError("contraction length must be a multiple of the K tile")
    lead = w.shape[:-2]
    return np.ascontiguousarray(np.swapaxes(w.reshape(lead + (n, k // tile, tile)), -3, -2))


def _pad_axis(arr: np.ndarray, axis: int, C: int, Cp: int) -> np.ndarray:
    """An axis made of blocks of C channels -> the same blocks of Cp channels, zero-filled."""
    axis = axis % arr.ndim
    n = arr.shape[axis]
    assert n % C == 0, (arr.shape, axis, C)
    shp = arr.shape[:axis] + (n // C, C) + arr.shape[axis + 1:]
    a = arr.reshape(shp)
    width = [(0, 0)] * a.ndim
    width[axis + 1] = (0, Cp - C)
    a = np.pad(a, width)
    return a.reshape(arr.shape[:axis] + ((n // C) * Cp,) + arr.shape[axis + 1:])


def pad_channels(out: Dict[str, np.ndarray], C: int, Cp: int) -> None:
    """The kernels work on channel counts that are multiples of 32.  Other counts (the reference's example uses 48)
    run with the channel dimension zero-padded: padded channels stay exactly zero through every layer (zero weights
    and biases in, zero out; SiLU, gates and products of zeros are zero) and the fan-in factors were taken from the
    true channel count before this step."""
    if Cp == C:
        return
    both = {"up", "upT", "nl", "nlT", "lin", "linT", "c0", "c0T", "c1", "c1T", "c2", "c2T", "res", "resT", "down", "downT"}
    last_only = {"W3", "b", "b3"}
    for name in list(out):
        parts = name.split(".")
        arr = out[name]
        if name == "emb":
            out[name] = _pad_axis(arr, -1, C, Cp)
        elif name == "ro.W1":
            out[name] = _pad_axis(arr, -2, C, Cp)
        elif name.startswith("ro.lin"):
            out[name] = _pad_axis(arr, -1, C, Cp)
        elif len(parts) >= 2 and parts[0].startswith("t") and parts[0][1:].isdigit():
            stem = parts[1]
            if stem in both and len(parts) == 3 and parts[2].startswith("l"):
                out[name] = _pad_axis(_pad_axis(arr, -2, C, Cp), -1, C, Cp)
            elif stem == "W3t":
                out[name] = _pad_axis(arr, -2, C, Cp)
            elif stem == "W3" or stem == "b3" or (len(parts) == 3 and parts[2] == "b" and stem in ("up", "nl", "lin", "down", "c", "res")):
                out[name] = _pad_axis(arr, -1, C, Cp)


def _silu(z):
    return z / (1.0 + np.exp(-z))


def _silu_grad(z):
    sg = 1.0 / (1.0 + np.exp(-z))
    return sg * (1.0 + z * (1.0 - sg))


def radial_table(out: Dict[str, np.ndarray], layer: int, plan: "ModelPlan", cutoff: float, envelope_p: int, intervals: int) -> np.ndarray:
    """Path weights of interaction ``layer`` as a function of the edge length, tabulated for cubic Hermite interpolation.

    With the identity edge update the radial MLP sees nothing but the radial basis of the edge length
    (tace/models/_e3nn/edge.py:15-35,169-189, inter.py:166-183), so its output W(d) [paths * channels] is a smooth
    function of one variable.  Returns [intervals + 1][paths * channels][2] (fp64): W at the knots d_k = k * cutoff /
    intervals and h * dW/dd there (h = knot spacing), both from an fp64 forward-mode pass through the packed layers of
    ``out`` (normalisation factors already folded in).  With ``apply_cutoff`` the envelope is part of the features;
    otherwise the table holds the bare MLP output and the kernels multiply by the envelope as before."""
    tp = f"t{layer}."
    K = int(intervals)
    h = cutoff / K
    d = np.arange(K + 1, dtype=np.float64) * h
    d[0] = 1e-3 * h  # sin(w d) / d and its derivative are finite at 0; evaluate just beside it
    w = out["bessel"].reshape(1, -1)
    pref = float(out["bessel_pref"].reshape(-1)[0])
    s, c = np.sin(w * d[:, None]), np.cos(w * d[:, None])
    f = pref * s / d[:, None]
    df = pref * (w * c * d[:, None] - s) / d[:, None] ** 2
    if plan.apply_cutoff:
        x = d / cutoff
        pp = float(envelope_p)
        u = 1.0 - (pp + 1) * (pp + 2) / 2 * x**pp + pp * (pp + 2) * x ** (pp + 1) - pp * (pp + 1) / 2 * x ** (pp + 2)
        du = -(pp * (pp + 1) * (pp + 2) / 2) * x ** (pp - 1) * (1 - x) ** 2 / cutoff
        inside = d < cutoff
        u, du = np.where(inside, u, 0.0), np.where(inside, du, 0.0)
        f, df = f * u[:, None], df * u[:, None] + f * du[:, None]
    nh = plan.mlp_layers
    z = f @ out[tp + "A0"] + (out[tp + "b0"] if plan.mlp_bias else 0.0)
    dz = df @ out[tp + "A0"]
    a, da = _silu(z), _silu_grad(z) * dz
    for j, name in ((1, "A1"), (2, "A2")):
        if nh > j:
            z = a @ out[tp + name] + (out[tp + f"b{j}"] if plan.mlp_bias else 0.0)
            dz = da @ out[tp + name]
            a, da = _silu(z), _silu_grad(z) * dz
    val = a @ out[tp + "W3"] + (out[tp + "b3"] if plan.mlp_bias else 0.0)
    slope = da @ out[tp + "W3"]
    knots = np.stack([val, slope * h], axis=-1)  # [K + 1][paths * channels][2]
    return knots


def radial_table_intervals(knots: np.ndarray) -> np.ndarray:
    """The device layout of ``radial_table``'s result: [K][paths * channels][4] = the (value, h * slope) pairs of both
    ends of interval k, so that one 16-byte load feeds the interpolation of one (path, channel) weight."""
    return np.ascontiguousarray(np.concatenate([knots[:-1], knots[1:]], axis=-1))


def hermite_weights(table: np.ndarray, d: np.ndarray, cutoff: float):
    """Host restatement of the kernels' interpolation: (W(d), dW/dd) from a table of ``radial_table``."""
    K = table.shape[0] - 1
    h = cutoff / K
    u = np.asarray(d, dtype=np.float64) / h
    k = np.clip(np.floor(u).astype(np.int64), 0, K - 1)
    t = (u - k)[:, None]
    v0, m0, v1, m1 = table[k, :, 0], table[k, :, 1], table[k + 1, :, 0], table[k + 1, :, 1]
    t2, t3 = t * t, t * t * t
    val = (2 * t3 - 3 * t2 + 1) * v0 + (t3 - 2 * t2 + t) * m0 + (-2 * t3 + 3 * t2) * v1 + (t3 - t2) * m1
    der = ((6 * t2 - 6 * t) * v0 + (3 * t2 - 4 * t + 1) * m0 + (-6 * t2 + 6 * t) * v1 + (3 * t2 - 2 * t) * m1) / h
    return val, der


def _np(t) -> np.ndarray:
    return t.detach().cpu().double().numpy() if hasattr(t, "detach") else np.asarray(t, dtype=np.float64)


RADIAL_TABLE_INTERVALS = 512  # knot spacing cutoff / 512: interpolation error below fp32 round-off of the table itself


def pack_weights(plan: ModelPlan, sd: Dict[str, "object"], avg_num_neighbors: float, prefix: str = "", radial_table_spec=None
                 ) -> Dict[str, np.ndarray]:
    """fp64 arrays keyed by the names ``tace_weight_info`` reports.  ``radial_table_spec`` = (cutoff, envelope power,
    intervals) adds the tabulated radial weights "t<i>.rtab" of every interaction (``radial_table``)."""
    C, n_el, L = plan.C, plan.n_el, plan.L
    g = lambda k: _np(sd[prefix + k])
    out: Dict[str, np.ndarray] = {}
    out["emb"] = g("representation.node_embedding.elem_emb1.weight").reshape(n_el, C) / math.sqrt(n_el)
    out["bessel"] = g("representation.radial_basis.radial_fn.bessel_weights").reshape(-1)
    out["bessel_pref"] = g("representation.radial_basis.radial_fn.prefactor").reshape(1)

    def split(flat: np.ndarray, shapes: List[tuple]) -> List[np.ndarray]:
        res, off = [], 0
        for shp in shapes:
            n = int(np.prod(shp))
            res.append(flat[..., off:off + n].reshape(flat.shape[:-1] + shp))
            off += n
        assert off == flat.shape[-1], (off, flat.shape)
        return res

    def put(name: str, mat: np.ndarray, transposed_name: str = None):
        out[name] = np.ascontiguousarray(mat)
        if transposed_name:
            out[transposed_name] = np.ascontiguousarray(np.swapaxes(mat, -1, -2))

    def per_species(key: str, shared: bool) -> np.ndarray:
        """A per-species parameter; one shared (species-agnostic) array is repeated for every species."""
        arr = g(key)
        return np.broadcast_to(arr[None], (n_el,) + arr.shape).copy() if shared else arr

    for lp in plan.layers:
        t = lp.t
        pre = f"representation.interactions.{t}."
        pp = f"representation.products.{t}."
        tp = f"t{t}."
        for l, m in zip(lp.in_ls, split(g(pre + "linear_up.weight"), [(C, C)] * len(lp.in_ls))):
            put(tp + f"up.l{l}", m / math.sqrt(C), tp + f"upT.l{l}")
        out[tp + "up.b"] = g(pre + "linear_up.bias")
        nb, hd, nh = plan.num_bessel, plan.mlp_hidden, plan.mlp_layers
        # first layer: fan-in = radial features (+ both species embeddings with the element-dependent edge update, whose
        # rows become per-species tables added to the first pre-activation: tace/models/_e3nn/edge.py:190-257)
        w0 = g(pre + "edge_info.mlp.0.weight")
        out[tp + "A0"] = w0[:nb] / math.sqrt(w0.shape[0])
        if plan.element2:
            eu = f"representation.edge_updates.{t}."
            temb = g(eu + "target_embedding.weight").reshape(n_el, C) / math.sqrt(n_el)
            semb = g(eu + "source_embedding.weight").reshape(n_el, C) / math.sqrt(n_el)
            out[tp + "tdst"] = temb @ w0[nb:nb + C] / math.sqrt(w0.shape[0])
            out[tp + "tsrc"] = semb @ w0[nb + C:nb + 2 * C] / math.sqrt(w0.shape[0])
        mi = plan.mlp_index
        if nh >= 2:
            put(tp + "A1", g(pre + f"edge_info.mlp.{mi(1)}.weight") * math.sqrt(2.0 / hd), tp + "A1t")
        if nh >= 3:
            put(tp + "A2", g(pre + f"edge_info.mlp.{mi(2)}.weight") * math.sqrt(2.0 / hd), tp + "A2t")
        put(tp + "W3", g(pre + f"edge_info.mlp.{mi(nh)}.weight") * math.sqrt(2.0 / hd), tp + "W3t")
        if plan.mlp_bias:
            for j in range(nh):
                out[tp + f"b{j}"] = g(pre + f"edge_info.mlp.{mi(j)}.bias")
            out[tp + "b3"] = g(pre + f"edge_info.mlp.{mi(nh)}.bias")
        if plan.mlp_layer_norm:
            for j in range(nh):
                out[tp + f"ln{j}g"] = g(pre + f"edge_info.mlp.{mi(j) + 1}.weight")
                out[tp + f"ln{j}b"] = g(pre + f"edge_info.mlp.{mi(j) + 1}.bias")
        down_shapes = [(lp.k[l] * C, ((L + 2) * C if plan.gate_m0 else (L + 1) * C) if l == 0 else C) for l in range(L + 1)]
        # the constant message normalisation is folded into linear_down; a learned density divides at run time instead
        norm = 1.0 if (plan.density or lp.tece) else avg_num_neighbors  # the edge block is not normalised (inter.py:466)
        if lp.tece:  # torch-style linears [out, in] with 1 / sqrt(fan_in) (tace/models/linear.py:210-244) -> [K][N]
            for ref, name, ci, co, n_in, n_out in plan.so2_linears():
                w0 = g(pre + f"rejector.{ref}.m0_rlinear.weight")
                put(tp + f"so2.{name}.m0", w0.T / math.sqrt(w0.shape[1]), tp + f"so2.{name}T.m0")
                out[tp + f"so2.{name}.b"] = g(pre + f"rejector.{ref}.m0_rlinear.bias")
                for m in range(1, len(n_in)):
                    wm = g(pre + f"rejector.{ref}.ms_clinear.{m - 1}.fc.weight")
                    put(tp + f"so2.{name}.m{m}", wm.T / math.sqrt(wm.shape[1]), tp + f"so2.{name}T.m{m}")
            n, H = plan.L + 1, plan.num_head
            rows = n + 2 * n * plan.mmax  # oam_2026_07_05.py:597-600,683-685
            scale = 1.0 / math.sqrt((plan.C // H) * rows)
            logit = g(pre + "rejector.temperature_logit").reshape(H)
            out[tp + "att.temp"] = scale * (0.25 + (4.0 - 0.25) / (1.0 + np.exp(-logit)))
            rw = g(pre + "rejector.radial_proj.weight")
            out[tp + "att.rw"] = rw.T / math.sqrt(rw.shape[1])
            out[tp + "att.rb"] = g(pre + "rejector.radial_proj.bias")
        for l, m in enumerate(split(g(pre + "linear_down.weight"), down_shapes)):
            put(tp + f"down.l{l}", m / math.sqrt(lp.k[l] * C) / norm, tp + f"downT.l{l}")
        out[tp + "down.b"] = g(pre + "linear_down.bias") / norm
        if plan.density:  # MLP 8 -> 64 -> 1 with the MLP gains (1 / sqrt(fan_in), sqrt(2) after the first layer)
            out[tp + "dA0"] = g(pre + "edge_density.mlp.0.weight") / math.sqrt(nb)
            out[tp + "dw1"] = g(pre + "edge_density.mlp.2.weight").reshape(hd) * math.sqrt(2.0 / hd)
            out[tp + "dab"] = np.array([float(g(pre + "alpha")), float(g(pre + "beta"))])
            if plan.mlp_bias:
                out[tp + "db0"] = g(pre + "edge_density.mlp.0.bias")
                out[tp + "db1"] = g(pre + "edge_density.mlp.2.bias")
        for l, m in enumerate(split(g(pre + "linear_nonlinearity.weight"), [(C, C)] * (L + 1))):
            put(tp + f"nl.l{l}", m / math.sqrt(C), tp + f"nlT.l{l}")
        out[tp + "nl.b"] = g(pre + "linear_nonlinearity.bias")
        if plan.bilinear:
            # e3nn Linear order: input block major; the scalars feed the gates and the rank-0 factors, rank l its factors
            npth = len(lp.pb_paths)
            mats = split(g(pp + "linear_up.weight"), [(C, npth * C)] + [(C, 2 * C)] * (L + 1))
            put(tp + "pg", mats[0] / math.sqrt(C), tp + "pgT")
            for l in range(L + 1):
                put(tp + f"pu.l{l}", mats[1 + l] / math.sqrt(C), tp + f"puT.l{l}")
            bias = g(pp + "linear_up.bias")
            out[tp + "pg.b"], out[tp + "pu.b"] = bias[:npth * C], bias[npth * C:]
        for l, m in zip(lp.out_ls, split(per_species(pp + "coefs.0.weight", plan.product_agnostic), [(C, C)] * len(lp.out_ls))):
            put(tp + f"c0.l{l}", m / math.sqrt(C), tp + f"c0T.l{l}")
        bias = per_species(pp + "coefs.0.bias", plan.product_agnostic).copy()
        if plan.correlation >= 2:
            for l, kp, m in zip(lp.out_ls, lp.kp, split(per_species(pp + "coefs.1.weight", plan.product_agnostic), [(kp * C, C) for kp in lp.kp])):
                put(tp + f"c1.l{l}", m / math.sqrt(kp * C), tp + f"c1T.l{l}")
            bias = bias + per_species(pp + "coefs.1.bias", plan.product_agnostic)
        if plan.correlation >= 3:
            for l, kp, m in zip(lp.out_ls, lp.kp3, split(per_species(pp + "coefs.2.weight", plan.product_agnostic), [(kp * C, C) for kp in lp.kp3])):
                put(tp + f"c2.l{l}", m / math.sqrt(kp * C), tp + f"c2T.l{l}")
            bias = bias + per_species(pp + "coefs.2.bias", plan.product_agnostic)
        out[tp + "c.b"] = bias
        for l, m in zip(lp.out_ls, split(g(pp + "linear.weight"), [(C, C)] * len(lp.out_ls))):
            put(tp + f"lin.l{l}", m / math.sqrt(C), tp + f"linT.l{l}")
        out[tp + "lin.b"] = g(pp + "linear.bias")
        if lp.has_res and plan.resnet_type != "identity":
            shared = plan.resnet_type == "agnostic"
            for l, m in zip(lp.out_ls, split(per_species(pre + "resnetBB.weight", shared), [(C, C)] * len(lp.out_ls))):
                put(tp + f"res.l{l}", m / math.sqrt(C), tp + f"resT.l{l}")
            out[tp + "res.b"] = per_species(pre + "resnetBB.bias", shared)
    ro = plan.num_layers - 1 if plan.use_alllayer else 0
    # multi-head read-out (tace/models/_e3nn/readout.py:18-33,72-84): the hidden layer is [head][H] wide, the mask keeps
    # the block of the atom's head and the head's output column is taken, so head f only ever uses W1[:, f, :] and
    # W2[f, :, f]; the second linear's fan-in is the full hidden width
    nf, H = plan.n_fid, plan.H
    w1 = g(f"energy_readouts.{ro}.linear2.0.weight").reshape(C, nf, H) / math.sqrt(C)
    w2 = g(f"energy_readouts.{ro}.linear2.1.weight").reshape(nf, H, nf) / math.sqrt(H * nf)
    out["ro.W1"] = np.ascontiguousarray(np.transpose(w1, (1, 0, 2)))
    out["ro.W2"] = np.stack([w2[f, :, f] for f in range(nf)])
    if plan.use_alllayer:
        for t in range(plan.num_layers - 1):
            out[f"ro.lin{t}"] = np.ascontiguousarray(g(f"energy_readouts.{t}.linear1.0.weight").reshape(C, nf).T) / math.sqrt(C)
    pad_channels(out, C, plan.Cp)
    # TF32 high part / residual of every plain channel-mixing matrix (tensor-core path of fp32 models)
    for name in list(out):
        stem = name.split(".")[1] if name.startswith("t") and "." in name else ""
        if (stem in ("up", "upT", "down", "downT", "nl", "nlT", "lin", "linT", "c0", "c0T", "c1", "c1T", "c2", "c2T", "res", "resT", "pu", "puT")
                and name.split(".")[-1].startswith("l")) \
                or stem in ("A1", "A1t", "A2", "A2t", "W3", "W3t") or name.split(".")[-1] in ("pg", "pgT") \
                or (stem == "so2" and name.split(".")[-1].startswith("m")):
            hi, lo = split_tf32(out[name])
            if stem in ("c0", "c0T", "c1", "c1T", "c2", "c2T", "res", "resT"):
                # per-species matrices [species][N][K] are read once per pass: store them K-tile-major,
                # [species][K/32][N][32], so every operand block of the tensor-core GEMM is contiguous
                hi, lo = tile_k_major(hi), tile_k_major(lo)
            out[name + "_hi"], out[name + "_lo"] = hi, lo
    out["scale"] = g("scale_shift.scale").reshape(nf, n_el)
    out["e0"] = g("atomic_energy_layer.atomic_energy").reshape(nf, n_el)
    if plan.zbl:  # tace/models/radial.py:788-874
        zs = g("atomic_numbers").reshape(-1).astype(np.int64)
        out["zbl.z"] = zs.astype(np.float64)
        out["zbl.rcov"] = g("zbl.covalent_radii").reshape(-1)[zs]
        out["zbl.par"] = np.array([0.529 * float(g("zbl.a_prefactor")), float(g("zbl.a_exp"))])
    if radial_table_spec is not None:
        rc, env_p, intervals = radial_table_spec
        for lp in plan.layers:
            out[f"t{lp.t}.rtab"] = radial_table_intervals(radial_table(out, lp.t, plan, float(rc), int(env_p), int(intervals)))
    shift = g("scale_shift.shift")
    if np.any(shift != 0.0):
        raise NotImplementedError("a non-zero energy shift (scale_shift.shift_type) is not supported")
    return out
