"""CPU restatement of the reference energy / force / virial path.  TEST INFRASTRUCTURE ONLY.

Plain PyTorch (fp64 or fp32), forces by reverse-mode autograd exactly as the
reference does.  Module and parameter names mirror the reference so that one
``state_dict`` drives both this oracle and the CUDA implementation.  Each
class cites the reference file:line it follows (paths relative to the
reference project root).  PARITY UNPINNED at the e3nn boundary, see
``oracle/__init__.py``.
"""

from __future__ import annotations

import copy
import math
from typing import Dict, List, Optional, Tuple

import torch

from . import o3
from .o3 import Irreps

SILU_CST = 1.6791767923989418  # tace/models/mlp.py:34
SIGMOID_CST = 1.8467055342154763  # tace/models/mlp.py:43


def scatter_sum(src: torch.Tensor, index: torch.Tensor, dim_size: int) -> torch.Tensor:
    """tace/utils/torch_scatter.py:43-62 (zeros().scatter_add_())."""
    out = torch.zeros((dim_size,) + tuple(src.shape[1:]), dtype=src.dtype)
    idx = index.view((-1,) + (1,) * (src.dim() - 1)).expand_as(src)
    return out.scatter_add_(0, idx, src)


# ----------------------------------------------------------------------------
# irreps rules
# ----------------------------------------------------------------------------
def possible_tp_irreps(in1: Irreps, in2: Irreps, lmax: int) -> Irreps:
    """tace/models/_e3nn/base.py:16-30 with parity=False (natural parity only)."""
    ls = set()
    for _, l1 in in1:
        for _, l2 in in2:
            for l3 in range(abs(l1 - l2), l1 + l2 + 1):
                if l3 <= lmax and (l1 + l2 + l3) % 2 == 0:
                    ls.add(l3)
    return Irreps([(1, l) for l in ls]).regroup()


def generate_paths(irreps_out: Irreps, in1: Irreps, in2: Irreps, mode: str, identical_inputs: bool = False):
    """tace/models/_e3nn/paths.py:30-71: out-irrep major, then in1, then in2."""
    paths, out = [], []
    for _, l3 in irreps_out:
        for i, (mul, l1) in enumerate(in1):
            for j, (_, l2) in enumerate(in2):
                if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0:
                    if identical_inputs and i == j and (l1 + l2 - l3) % 2 == 1:
                        continue
                    paths.append((i, j, len(out), mode))
                    out.append((mul, l3))
    return paths, Irreps(out)


# ----------------------------------------------------------------------------
# e3nn-style modules
# ----------------------------------------------------------------------------
class Linear(torch.nn.Module):
    """tace/models/linear.py:282-374 over e3nn ``o3.Linear``: one ``[mul_in, mul_out]``
    block per (i_in, i_out) pair of equal l, i_in-major, flat weights, each path scaled by
    1/sqrt(sum of mul_in feeding that output); bias on 0e outputs only."""

    def __init__(self, irreps_in: Irreps, irreps_out: Irreps, bias: bool = True, num_elements: Optional[int] = None):
        super().__init__()
        self.irreps_in, self.irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        self.num_elements = num_elements
        self.instr = [
            (i, o)
            for i, (_, li) in enumerate(self.irreps_in)
            for o, (_, lo) in enumerate(self.irreps_out)
            if li == lo
        ]
        fan = {o: 0 for _, o in self.instr}
        for i, o in self.instr:
            fan[o] += self.irreps_in[i][0]
        self.path_weight = [fan[o] ** -0.5 for _, o in self.instr]
        self.weight_numel = sum(self.irreps_in[i][0] * self.irreps_out[o][0] for i, o in self.instr)
        nbias = sum(m for m, l in self.irreps_out if l == 0)
        lead = () if num_elements is None else (num_elements,)
        self.weight = torch.nn.Parameter(torch.randn(lead + (self.weight_numel,)))
        if bias and nbias > 0:
            self.bias = torch.nn.Parameter(torch.zeros(lead + (nbias,)))
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, attrs: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0]
        if self.num_elements is None:
            w = self.weight.unsqueeze(0).expand(n, -1)
            b = None if self.bias is None else self.bias.unsqueeze(0).expand(n, -1)
        else:  # tace/models/linear.py:442-478
            node_type = attrs.argmax(dim=-1)
            w = self.weight[node_type]
            b = None if self.bias is None else torch.einsum("bz,zi->bi", attrs, self.bias)
        in_sl, out_sl = self.irreps_in.slices(), self.irreps_out.slices()
        outs = [x.new_zeros(n, m, 2 * l + 1) for m, l in self.irreps_out]
        off = 0
        for (i, o), pw in zip(self.instr, self.path_weight):
            mi, l = self.irreps_in[i]
            mo = self.irreps_out[o][0]
            wi = w[:, off : off + mi * mo].reshape(n, mi, mo)
            off += mi * mo
            xi = x[:, in_sl[i]].reshape(n, mi, 2 * l + 1)
            outs[o] = outs[o] + pw * torch.einsum("zuw,zui->zwi", wi, xi)
        if b is not None:
            boff = 0
            for o, (m, l) in enumerate(self.irreps_out):
                if l == 0:
                    outs[o] = outs[o] + b[:, boff : boff + m].unsqueeze(-1)
                    boff += m
        return torch.cat([t.reshape(n, -1) for t in outs], dim=-1)


class TensorProduct(torch.nn.Module):
    """e3nn ``o3.TensorProduct`` as used in tace/models/_e3nn/fused.py:44-51,203-210:
    'component' irrep normalisation, 'element' path normalisation, one instruction per
    output slot, so every path carries the factor sqrt(2 l3 + 1)."""

    def __init__(self, in1: Irreps, in2: Irreps, out: Irreps, paths):
        super().__init__()
        self.in1, self.in2, self.out, self.paths = Irreps(in1), Irreps(in2), Irreps(out), paths
        # "uvu": one weight per (u, v); "uuuw": the channel-wise product with one weight per channel (trainable = True in
        # tace/models/_e3nn/paths.py:66-69)
        self.weight_numel = sum(self.in1[i][0] * (self.in2[j][0] if mode == "uvu" else 1) for i, j, _, mode in paths
                                if mode in ("uvu", "uuuw"))

    def forward(self, x1: torch.Tensor, x2: torch.Tensor, w: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x1.shape[0]
        s1, s2 = self.in1.slices(), self.in2.slices()
        outs, woff = [], 0
        for i, j, k, mode in self.paths:
            (m1, l1), (m2, l2), (_, l3) = self.in1[i], self.in2[j], self.out[k]
            c = o3.wigner_3j(l1, l2, l3, dtype=x1.dtype) * math.sqrt(2 * l3 + 1)
            a = x1[:, s1[i]].reshape(n, m1, 2 * l1 + 1)
            b = x2[:, s2[j]].reshape(n, m2, 2 * l2 + 1)
            if mode == "uvu":
                wk = w[:, woff : woff + m1 * m2].reshape(n, m1, m2)
                woff += m1 * m2
                o = torch.einsum("zuv,ijk,zui,zvj->zuk", wk, c, a, b)
            elif mode == "uuuw":
                wk = w[:, woff : woff + m1]
                woff += m1
                o = torch.einsum("zu,ijk,zui,zuj->zuk", wk, c, a, b)
            else:  # uuu, no weights
                o = torch.einsum("ijk,zui,zuj->zuk", c, a, b)
            outs.append(o.reshape(n, m1 * (2 * l3 + 1)))  # explicit width: n may be 0 (a batch without edges)
        return torch.cat(outs, dim=-1)


class MlpLinear(torch.nn.Module):
    """tace/models/linear.py:247-279."""

    def __init__(self, in_dim: int, out_dim: int, alpha: float, bias: bool = False):
        super().__init__()
        self.alpha = alpha
        self.weight = torch.nn.Parameter(torch.empty(in_dim, out_dim).uniform_(-math.sqrt(3), math.sqrt(3)))
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_dim))
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        y = torch.mm(x, self.weight * self.alpha)
        return y if self.bias is None else y + self.bias


class MLP(torch.nn.Module):
    """tace/models/mlp.py:136-191 (plain SiLU, gain sqrt(2) after layer 0, optional bias on every layer, optional
    LayerNorm between every hidden linear and its activation)."""

    def __init__(self, dims: List[int], bias: bool = False, layer_norm: bool = False):
        super().__init__()
        mods = []
        for layer, (a, b) in enumerate(zip(dims, dims[1:])):
            gain = 1.0 if layer == 0 else math.sqrt(2.0)
            mods.append(MlpLinear(a, b, gain / math.sqrt(a), bias=bias))
            if layer != len(dims) - 2:
                if layer_norm:
                    mods.append(torch.nn.LayerNorm(b))
                mods.append(torch.nn.SiLU())
        self.mlp = torch.nn.Sequential(*mods)

    def forward(self, x):
        return self.mlp(x)


class Gate(torch.nn.Module):
    """tace/models/_e3nn/nonlinear.py:27-42,93-143 with gate_m0=True: input =
    [(L+1)*C gate scalars | gated blocks]; every block, l = 0 included, is scaled channel-wise by
    1.8467*sigmoid(gate)."""

    def __init__(self, irreps_gated: Irreps):
        super().__init__()
        self.irreps_gated = Irreps(irreps_gated)
        self.irreps_gates = Irreps([(m, 0) for m, _ in self.irreps_gated])
        self.irreps_in = (self.irreps_gates.simplify() + self.irreps_gated).sort().simplify()
        self.irreps_out = self.irreps_gated
        self.m0 = True

    def forward(self, x):
        n = x.shape[0]
        if not self.m0:
            return self._forward_scalars_ungated(x)
        ng = self.irreps_gates.dim
        gates = SIGMOID_CST * torch.sigmoid(x[:, :ng])
        gated = x[:, ng:]
        outs, goff = [], 0
        for (m, l), sl in zip(self.irreps_gated, self.irreps_gated.slices()):
            g = gates[:, goff : goff + m]
            goff += m
            outs.append((gated[:, sl].reshape(n, m, 2 * l + 1) * g.unsqueeze(-1)).reshape(n, -1))
        return torch.cat(outs, dim=-1)


class ScalarActGate(Gate):
    """tace/models/_e3nn/nonlinear.py:43-70 (gate_m0=False) over e3nn ``Gate``: input = [scalars | one gate scalar
    block per rank >= 1 | blocks of rank >= 1]; scalars go through 1.6792*silu, rank l >= 1 is scaled channel-wise
    by 1.8467*sigmoid(gate l); output = [activated scalars | gated blocks]."""

    def __init__(self, irreps: Irreps):
        super().__init__(irreps)
        irreps = Irreps(irreps)
        self.m0 = False
        self.n_scalar = sum(m for m, l in irreps if l == 0)
        self.irreps_gated = Irreps([(m, l) for m, l in irreps if l > 0])
        self.irreps_gates = Irreps([(m, 0) for m, _ in self.irreps_gated])
        scalars = Irreps([(self.n_scalar, 0)])
        self.irreps_in = (scalars + self.irreps_gates.simplify() + self.irreps_gated).sort().simplify()
        self.irreps_out = (scalars + self.irreps_gated).simplify()

    def _forward_scalars_ungated(self, x):
        n, ns, ng = x.shape[0], self.n_scalar, self.irreps_gates.dim
        outs = [SILU_CST * torch.nn.functional.silu(x[:, :ns])]
        gates = SIGMOID_CST * torch.sigmoid(x[:, ns:ns + ng])
        gated = x[:, ns + ng:]
        goff = 0
        for (m, l), sl in zip(self.irreps_gated, self.irreps_gated.slices()):
            g = gates[:, goff:goff + m]
            goff += m
            outs.append((gated[:, sl].reshape(n, m, 2 * l + 1) * g.unsqueeze(-1)).reshape(n, -1))
        return torch.cat(outs, dim=-1)


# ----------------------------------------------------------------------------
# model blocks
# ----------------------------------------------------------------------------
class J0Bessel(torch.nn.Module):
    """tace/models/radial.py:43-84."""

    def __init__(self, cutoff: float, num_basis: int):
        super().__init__()
        self.register_buffer("bessel_weights", math.pi / cutoff * torch.linspace(1.0, num_basis, num_basis))
        self.register_buffer("cutoff", torch.tensor(cutoff))
        self.register_buffer("prefactor", torch.tensor(math.sqrt(2.0 / cutoff)))

    def forward(self, r):
        return self.prefactor * (torch.sin(self.bessel_weights * r) / r)


class C2Poly(torch.nn.Module):
    """tace/models/radial.py:437-472."""

    def __init__(self, cutoff: float, p: int):
        super().__init__()
        self.register_buffer("p", torch.tensor(p, dtype=torch.int))
        self.register_buffer("cutoff", torch.tensor(cutoff))

    def forward(self, r):
        p = self.p.to(torch.int)
        x = r / self.cutoff
        env = (
            1.0
            - ((p + 1.0) * (p + 2.0) / 2.0) * torch.pow(x, p)
            + p * (p + 2.0) * torch.pow(x, p + 1)
            - (p * (p + 1.0) / 2) * torch.pow(x, p + 2)
        )
        return env * (r < self.cutoff)


class RadialBasis(torch.nn.Module):
    """tace/models/radial.py:877-993: returns (radial features, envelope or None); with apply_cutoff the envelope is
    already in the features, otherwise the caller multiplies the radial MLP's output by it (:987-993)."""

    def __init__(self, cutoff, num_basis, p, apply_cutoff=True):
        super().__init__()
        self.cutoff_fn = C2Poly(cutoff, p)
        self.radial_fn = J0Bessel(cutoff, num_basis)
        self.num_basis = num_basis
        self.apply_cutoff = apply_cutoff

    def forward(self, edge_length):
        env = self.cutoff_fn(edge_length)
        radial = self.radial_fn(edge_length)
        return (radial * env, None) if self.apply_cutoff else (radial, env)


class ZBLBasis(torch.nn.Module):
    """tace/models/radial.py:788-874: screened nuclear repulsion (ZBL universal screening function) per pair, cut by the
    polynomial envelope at the sum of the two covalent radii; half of every directed edge's energy goes to its target.
    ``covalent_radii`` is a table indexed by atomic number (the reference reads ``ase.data.covalent_radii``)."""

    def __init__(self, covalent_radii, p: int = 5):
        super().__init__()
        self.register_buffer("c", torch.tensor([0.1818, 0.5099, 0.2802, 0.02817]))
        self.register_buffer("p", torch.tensor(p, dtype=torch.int))
        self.register_buffer("covalent_radii", torch.as_tensor(covalent_radii, dtype=torch.get_default_dtype()))
        self.register_buffer("a_exp", torch.tensor(0.300))
        self.register_buffer("a_prefactor", torch.tensor(0.4543))

    def forward(self, x, node_attrs, edge_index, atomic_numbers):
        source, target = edge_index[0], edge_index[1]
        z = atomic_numbers[torch.argmax(node_attrs, dim=1)].unsqueeze(-1)
        zu, zv = z[source], z[target]
        a = self.a_prefactor * 0.529 / (torch.pow(zu, self.a_exp) + torch.pow(zv, self.a_exp))
        ra = x / a
        phi = (self.c[0] * torch.exp(-3.2 * ra) + self.c[1] * torch.exp(-0.9423 * ra)
               + self.c[2] * torch.exp(-0.4028 * ra) + self.c[3] * torch.exp(-0.2016 * ra))
        v = (14.3996 * zu * zv) / x * phi
        r_max = self.covalent_radii[zu] + self.covalent_radii[zv]
        p = self.p.to(torch.int)
        xr = x / r_max  # tace/models/radial.py:458-469 with a per-edge cutoff
        env = (1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * torch.pow(xr, p) + p * (p + 2.0) * torch.pow(xr, p + 1)
               - (p * (p + 1.0) / 2) * torch.pow(xr, p + 2)) * (x < r_max)
        v = 0.5 * v * env
        return scatter_sum(v, target, node_attrs.size(0)).squeeze(-1)


class Element2EdgeUpdate(torch.nn.Module):
    """tace/models/_e3nn/edge.py:190-257: radial features followed by the species embeddings of the target and
    of the source (in that order; ``ElementEdgeUpdate`` has them the other way round)."""

    def __init__(self, num_elements, num_channel):
        super().__init__()
        irr_in, irr_out = Irreps([(num_elements, 0)]), Irreps([(num_channel, 0)])
        self.source_embedding = Linear(irr_in, irr_out, bias=False)
        self.target_embedding = Linear(irr_in, irr_out, bias=False)

    def forward(self, node_attrs, edge_feats, edge_index):
        return torch.cat([edge_feats, self.target_embedding(node_attrs[edge_index[1]]),
                          self.source_embedding(node_attrs[edge_index[0]])], dim=-1)


class NodeEmbedding(torch.nn.Module):
    """tace/models/_e3nn/node.py:22-52."""

    def __init__(self, num_elements, num_channel):
        super().__init__()
        self.irreps_out = Irreps([(num_channel, 0)])
        self.elem_emb1 = Linear(Irreps([(num_elements, 0)]), self.irreps_out, bias=False)

    def forward(self, node_attrs):
        return self.elem_emb1(node_attrs)


class SkipIdentity(torch.nn.Module):
    """tace/models/_e3nn/residual.py:170-250: the skip connection without weights.  Equal irreps pass through; a smaller
    output keeps the first input block of every irrep it has (ProjectDown); a larger one is zero-filled (ProjectUp)."""

    def __init__(self, irreps_in: Irreps, irreps_out: Irreps):
        super().__init__()
        self.irreps_in, self.irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        small, big = (self.irreps_out, self.irreps_in) if self.irreps_out.dim <= self.irreps_in.dim else (self.irreps_in, self.irreps_out)
        big_slices, used, idx = big.slices(), set(), []
        for mul_ir in small:
            for k, (target, sl) in enumerate(zip(big, big_slices)):
                if k not in used and tuple(mul_ir) == tuple(target):
                    idx.append(torch.arange(sl.start, sl.stop))
                    used.add(k)
                    break
            else:
                raise ValueError(f"{small} is not a sub-representation of {big}")
        self.register_buffer("idx", torch.cat(idx), persistent=False)

    def forward(self, x, attrs=None):
        if self.irreps_in.dim >= self.irreps_out.dim:
            return x[:, self.idx]
        out = x.new_zeros(x.shape[0], self.irreps_out.dim)
        out[:, self.idx] = x
        return out


class Interaction(torch.nn.Module):
    """tace/models/_e3nn/inter.py:28-285 (O3CgtpInteraction), irreps from
    tace/models/_e3nn/base.py:113-249."""

    def __init__(self, layer, num_layers, num_elements, avg_num_neighbors, Lmax, lmax, correlation,
                 num_channel, num_radial_basis, radial_mlp, irreps_in, target_irreps, gate_m0=True, mlp_bias=False, mlp_layer_norm=False,
                 scatter_norm="avg_num_neighbors", resnet_linear_type="aware", radial_dim=8):
        super().__init__()
        self.layer, self.avg_num_neighbors = layer, avg_num_neighbors
        self.scatter_norm = scatter_norm
        C = num_channel
        self.num_channel, self.gate_m0, self.num_radial_basis = C, gate_m0, radial_dim
        self.mlp_bias, self.mlp_layer_norm = mlp_bias, mlp_layer_norm
        self.irreps_in = Irreps(irreps_in)
        self.irreps_sh = Irreps.spherical_harmonics(lmax)
        tp_out = possible_tp_irreps(self.irreps_in, self.irreps_sh, Lmax if correlation == 1 else lmax)
        self.irreps_out = (tp_out * C).regroup()
        if layer == num_layers - 1:
            self.irreps_sc = (Irreps(target_irreps) * C).regroup()
        else:
            self.irreps_sc = (possible_tp_irreps(self.irreps_in, self.irreps_sh, Lmax) * C).regroup()

        self.linear_up = Linear(self.irreps_in, self.irreps_in, bias=True)
        paths, tp_irreps_out = generate_paths(self.irreps_out, self.irreps_in, self.irreps_sh, "uvu")
        self.rejector = TensorProduct(self.irreps_in, self.irreps_sh, tp_irreps_out, paths)
        gate_cls = Gate if gate_m0 else ScalarActGate
        self.nonlinearity = gate_cls(Irreps([(C, l) for _, l in self.irreps_out]))
        self.linear_nonlinearity = Linear(self.nonlinearity.irreps_out, self.irreps_out, bias=True)
        self.linear_down = Linear(tp_irreps_out.simplify(), self.nonlinearity.irreps_in, bias=True)
        # tace/models/_e3nn/base.py:183-185: edge features wider than the radial basis (an element-dependent edge
        # update) switch LayerNorm on inside the radial MLP
        self.edge_info_dims = [num_radial_basis] + list(radial_mlp) + [self.rejector.weight_numel]
        self.edge_info = MLP(self.edge_info_dims, bias=mlp_bias, layer_norm=mlp_layer_norm)
        if scatter_norm in ("density", "no_cutoff_density"):  # inter.py:102-110 (the edge density of MACE)
            self.edge_density = MLP([num_radial_basis, 64, 1], bias=mlp_bias, layer_norm=mlp_layer_norm)
            self.alpha = torch.nn.Parameter(torch.tensor(float(avg_num_neighbors)))
            self.beta = torch.nn.Parameter(torch.tensor(0.0))
        if layer > 0:  # resnet type "BB", use_first_resnet False; tace/models/_e3nn/residual.py:145-168
            if resnet_linear_type == "identity":
                self.resnetBB = SkipIdentity(self.irreps_in, self.irreps_sc)
            else:
                self.resnetBB = Linear(self.irreps_in, self.irreps_sc, bias=True,
                                       num_elements=num_elements if resnet_linear_type == "aware" else None)

    def messages(self, x, edge_feats, edge_attrs, edge_index, edge_cutoff, edge_vector, radial_basis):
        """inter.py:166-183: per-edge weights from the radial MLP, weighted tensor product with the angular basis, sum
        over the edges into every atom."""
        w = self.edge_info(edge_feats)
        if edge_cutoff is not None:  # inter.py:174-183
            w = w * edge_cutoff
        msg = self.rejector(x[edge_index[0]], edge_attrs, w)  # tace/models/_e3nn/fused.py:269-271
        return scatter_sum(msg, edge_index[1], x.shape[0])

    def forward(self, node_feats, node_attrs, edge_feats, edge_attrs, edge_index, edge_cutoff=None, edge_vector=None,
                radial_basis=None):
        sc = self.resnetBB(node_feats, node_attrs) if hasattr(self, "resnetBB") else None
        x = self.linear_up(node_feats)
        m = self.messages(x, edge_feats, edge_attrs, edge_index, edge_cutoff, edge_vector, radial_basis)
        m = self.linear_down(m)
        m = self.normalise(m, edge_feats, edge_index, edge_cutoff)
        m = self.linear_nonlinearity(self.nonlinearity(m))
        return m, sc

    def normalise(self, m, edge_feats, edge_index, edge_cutoff):
        if hasattr(self, "edge_density"):  # inter.py:249-260, base.py:240-249
            density = torch.tanh(self.edge_density(edge_feats) ** 2)
            if edge_cutoff is not None and self.scatter_norm == "density":
                density = density * edge_cutoff
            density = scatter_sum(density, edge_index[1], m.shape[0])
            density = density * self.beta + self.alpha
            density = density.masked_fill(density == 0, 1e-9)
            return m / density
        return m / self.avg_num_neighbors  # base.py:240-249


class Product(torch.nn.Module):
    """tace/models/_e3nn/prod.py:20-266 (CgtpACE, one expert, per-species coefficients),
    irreps from tace/models/_e3nn/base.py:252-360."""

    def __init__(self, layer, num_layers, num_elements, Lmax, lmax, num_channel, correlation, irreps_in,
                 target_irreps, agnostic=False, bilinear=False):
        super().__init__()
        C = num_channel
        self.correlation = correlation
        self.bilinear = bilinear
        if agnostic:  # prod.py:49-50: one coefficient linear for every species
            num_elements = None
        last = layer == num_layers - 1
        self.irreps_in = Irreps(irreps_in)
        hidden = Irreps([(C, l) for _, l in self.irreps_in])
        tp_out_list = []
        for nu in range(2, correlation + 1):
            if nu == correlation:
                if last:
                    tp_out_list.append((Irreps(target_irreps) * C).regroup())
                else:
                    tp_out_list.append((possible_tp_irreps(hidden, hidden, Lmax) * C).regroup())
            else:
                tp_out_list.append(possible_tp_irreps(hidden, hidden, lmax))
        if correlation == 1:
            coefs_out = Irreps([(C, l) for _, l in self.irreps_in if l <= Lmax])
        else:
            coefs_out = (possible_tp_irreps(self.irreps_in, self.irreps_in, Lmax) * C).regroup()
        if last:
            coefs_out = (Irreps(target_irreps) * C).regroup()
        self.irreps_out = Irreps([(C, l) for _, l in coefs_out])

        self.coefs = torch.nn.ModuleList([Linear(hidden.simplify(), coefs_out, bias=True, num_elements=num_elements)])
        self.aces = torch.nn.ModuleList()
        in1 = hidden
        base = hidden
        if bilinear:  # prod.py:87-92: the second factor gets a block of ones, so the product also carries the factor itself
            assert correlation == 2
            base = Irreps(list(hidden) + [(C, 0)])
        for nu in range(2, correlation + 1):
            if bilinear:
                paths, out = generate_paths(tp_out_list[nu - 2], in1, base, "uuuw")
            else:
                paths, out = generate_paths(tp_out_list[nu - 2], in1, hidden, "uuu", identical_inputs=(nu == 2))
            self.aces.append(TensorProduct(in1, base, out, paths))
            self.coefs.append(
                Linear(Irreps([(C, l) for _, l in out]).simplify(), coefs_out, bias=True, num_elements=num_elements)
            )
            in1 = out
        self.linear = Linear(Irreps([(C, l) for _, l in coefs_out]), self.irreps_out, bias=True)
        if bilinear:  # prod.py:128-155: gate scalars for every product path and both factors from one linear
            self.num_gates = self.aces[0].weight_numel
            self.hidden = hidden
            self.linear_up = Linear(self.irreps_in, Irreps([(self.num_gates, 0)] + [(2 * C, l) for _, l in hidden]), bias=True)

    def forward(self, node_feats, node_attrs, sc):
        base_feats, gates = node_feats, None
        if self.bilinear:  # prod.py:183-221
            x = self.linear_up(node_feats)
            gates = torch.nn.functional.silu(x[:, :self.num_gates])
            n, off, first, second = x.shape[0], self.num_gates, [], []
            for mul, l in self.hidden:
                field = x[:, off:off + 2 * mul * (2 * l + 1)].reshape(n, 2 * mul, 2 * l + 1)
                off += 2 * mul * (2 * l + 1)
                first.append(field[:, :mul].reshape(n, -1))
                second.append(field[:, mul:].reshape(n, -1))
            node_feats = torch.cat(first, dim=-1)
            base_feats = torch.cat(second + [x.new_ones(n, self.hidden[0][0])], dim=-1)
        corr = {1: node_feats}
        outs = self.coefs[0](corr[1], node_attrs)
        for nu in range(2, self.correlation + 1):
            if self.bilinear:
                corr[nu] = self.aces[nu - 2](corr[nu - 1], base_feats, gates)
                outs = outs + self.coefs[nu - 1](corr[nu], node_attrs)
                continue
            corr[nu] = self.aces[nu - 2](corr[nu - 1], node_feats)
            outs = outs + self.coefs[nu - 1](corr[nu], node_attrs)
        outs = self.linear(outs)
        if sc is not None:
            outs = outs + sc
        return outs


class Representation(torch.nn.Module):
    """tace/models/_e3nn/representation.py:28-300,302-429 (default options)."""

    def __init__(self, cfg):
        super().__init__()
        n_el = len(cfg["atomic_numbers"])
        C, L, l = cfg["num_channel"], cfg["Lmax"], cfg["lmax"]
        rb = cfg["radial_basis"]
        self.lmax = l
        self.register_buffer("atomic_numbers", torch.tensor(cfg["atomic_numbers"], dtype=torch.int64))
        self.radial_basis = RadialBasis(cfg["cutoff"], rb["num_radial_basis"], rb["polynomial_cutoff"],
                                        apply_cutoff=rb.get("apply_cutoff", True))
        self.element2 = cfg.get("edge_update", {}).get("type", "identity") == "element2"
        if self.element2:
            self.edge_updates = torch.nn.ModuleList([Element2EdgeUpdate(n_el, C) for _ in range(cfg["num_layers"])])
        edge_dim = rb["num_radial_basis"] + (2 * C if self.element2 else 0)
        self.node_embedding = NodeEmbedding(n_el, C)
        self.interactions = torch.nn.ModuleList()
        self.products = torch.nn.ModuleList()
        for layer in range(cfg["num_layers"]):
            irreps_in = self.node_embedding.irreps_out if layer == 0 else self.products[layer - 1].irreps_out
            ab = cfg.get("atomic_basis", {})
            kinds = ab.get("type", "cgtp")
            kind = kinds[layer] if isinstance(kinds, (list, tuple)) else kinds
            cls, extra = Interaction, {}
            if kind == "uv_so2":  # the TECE edge block (tace/models/_e3nn/inter.py:440-519,779)
                from .tece import build_tece_interaction

                cls = build_tece_interaction(Interaction)
                edge_nl = ab.get("edge_nonlinear", "so2_sigmoid_gate")
                edge_nl = edge_nl[layer] if isinstance(edge_nl, (list, tuple)) else edge_nl
                extra = dict(mmax=cfg.get("mmax", 2), num_head=ab.get("num_head") or 1, edge_ace_hidden=ab.get("edge_ace_hidden"),
                             edge_wise_hidden=ab.get("edge_wise_hidden"), edge_act=edge_nl.split("_")[1])
            self.interactions.append(
                cls(layer, cfg["num_layers"], n_el, cfg["avg_num_neighbors"], L, l,
                    cfg["product_basis"]["correlation"][layer], C, edge_dim, rb["hidden"],
                    irreps_in, [(1, 0)], gate_m0=ab.get("gate_m0", True),
                    mlp_bias=rb.get("bias", False), mlp_layer_norm=self.element2,
                    scatter_norm=ab.get("scatter_norm", "avg_num_neighbors"),
                    resnet_linear_type=cfg.get("resnet", {}).get("linear_type", "aware"),
                    radial_dim=rb["num_radial_basis"], **extra)
            )
            self.products.append(
                Product(layer, cfg["num_layers"], n_el, L, l, C, cfg["product_basis"]["correlation"][layer],
                        self.interactions[layer].irreps_out, [(1, 0)],
                        agnostic=cfg["product_basis"].get("agnostic", False),
                        bilinear=cfg["product_basis"].get("nonlinear") == "silu_bilineargate")
            )

    def forward(self, node_attrs, edge_index, edge_vector, edge_length):
        edge_feats, edge_cutoff = self.radial_basis(edge_length)  # identity edge embedding
        edge_attrs = o3.spherical_harmonics(self.lmax, edge_vector / edge_length, "component")
        h = self.node_embedding(node_attrs)
        descriptors = []
        for inter, prod in zip(self.interactions, self.products):
            ef = self.edge_updates[len(descriptors)](node_attrs, edge_feats, edge_index) if self.element2 else edge_feats
            h, sc = inter(h, node_attrs, ef, edge_attrs, edge_index, edge_cutoff, edge_vector, edge_feats)
            h = prod(h, node_attrs, sc)
            descriptors.append(h)
        return descriptors


class ScalarReadOut(torch.nn.Module):
    """tace/models/_e3nn/readout.py:36-84.  Last layer: C -> 16 -> 1 with normalised SiLU, no bias
    (``linear2``); earlier layers (only built with ``use_alllayer``): one linear from the scalar block of
    the layer's features to the energy (``linear1``)."""

    def __init__(self, num_channel, hidden, irreps_in=None, last=True, num_fidelities=1):
        super().__init__()
        self.last = last
        self.num_fidelities = nf = num_fidelities
        if last:  # hidden widths and the output are multiplied by the number of fidelities (base.py:386-396)
            dims = [num_channel] + [h * nf for h in hidden] + [nf]
            self.linear2 = torch.nn.ModuleList(
                [Linear(Irreps([(a, 0)]), Irreps([(b, 0)]), bias=False) for a, b in zip(dims, dims[1:])]
            )
        else:
            self.linear1 = torch.nn.ModuleList([Linear(Irreps(irreps_in), Irreps([(nf, 0)]), bias=False)])

    def forward(self, x, node_fidelity=None):
        if not self.last:
            return self.linear1[0](x)
        for lin in self.linear2[:-1]:
            x = SILU_CST * torch.nn.functional.silu(lin(x))
            if self.num_fidelities > 1:  # readout.py:18-33 (mh_mask): only the hidden block of the atom's fidelity survives
                mask = torch.zeros(x.shape[0], self.num_fidelities, x.shape[1] // self.num_fidelities, dtype=x.dtype)
                mask[torch.arange(x.shape[0]), node_fidelity, :] = 1
                x = x * mask.reshape(x.shape[0], -1)
        return self.linear2[-1](x)


class AtomicEnergy(torch.nn.Module):
    """tace/models/blocks.py:250-273."""

    def __init__(self, atomic_energies, atomic_numbers):
        super().__init__()
        rows = [[float({int(k): float(v) for k, v in ae.items()}.get(int(z), 0.0)) for z in atomic_numbers]
                for ae in atomic_energies]
        self.register_buffer("atomic_energy", torch.tensor(rows))

    def forward(self, x):
        return torch.matmul(x, self.atomic_energy.T)


class ScaleShift(torch.nn.Module):
    """tace/models/blocks.py:289-379 (all_atoms=False, fixed scale, zero shift)."""

    def __init__(self, atomic_numbers, scale_dicts, shift_dicts):
        super().__init__()
        self.register_buffer("atomic_numbers", torch.tensor([int(z) for z in atomic_numbers], dtype=torch.int64))
        self.register_buffer("scale", torch.tensor([[d.get(int(z), 1.0) for z in atomic_numbers] for d in scale_dicts]))
        self.register_buffer("shift", torch.tensor([[d.get(int(z), 0.0) for z in atomic_numbers] for d in shift_dicts]))

    def forward(self, node_energy, node_attrs, ptr, edge_index, batch, node_fidelity):
        num_graphs = ptr.numel() - 1
        num_nodes = ptr[1:] - ptr[:-1]
        if edge_index.numel() == 0:
            num_edges = torch.zeros(num_graphs, dtype=torch.int64)
        else:
            eb = batch[edge_index[1]]
            num_edges = scatter_sum(torch.ones_like(eb), eb, num_graphs)
        isolated = ((num_nodes == 1) & (num_edges == 0))[batch]
        scale = (node_attrs * self.scale[node_fidelity]).sum(-1)
        node_energy = node_energy * torch.where(isolated, torch.zeros_like(scale), scale)
        shift = (node_attrs * self.shift[node_fidelity]).sum(-1)
        return node_energy + torch.where(isolated, torch.zeros_like(shift), shift)


def resolve_config(user_cfg: Dict) -> Dict:
    """The subset of tace/models/_e3nn/default.py:10-177,231-316 this path uses."""
    cfg = {
        "Lmax": 2, "lmax": 3, "num_channel": 64, "num_layers": 2,
        "radial_basis": {"num_radial_basis": 8, "polynomial_cutoff": 5, "hidden": [64, 64, 64], "bias": False,
                         "apply_cutoff": True},
        "edge_update": {"type": "identity"},
        "product_basis": {"correlation": 2},
        "readout_emlp": {"hidden": [16], "use_alllayer": False},
        "scale_shift": {"scale_type": "rms_forces", "shift_type": None, "scale_zbl": True},
        "short_range": {"zbl": {"enable": False}},
    }
    for k, v in copy.deepcopy(user_cfg).items():
        if isinstance(v, dict) and isinstance(cfg.get(k), dict):
            cfg[k].update(v)
        else:
            cfg[k] = v
    stats = cfg["statistics"]
    cfg["atomic_numbers"] = sorted({int(z) for s in stats for z in s["atomic_numbers"]})
    cfg["avg_num_neighbors"] = sum(s["avg_num_neighbors"] for s in stats) / len(stats)
    cfg["atomic_energies"] = [s["atomic_energy"] for s in stats]
    corr = cfg["product_basis"]["correlation"]
    if isinstance(corr, int):
        cfg["product_basis"]["correlation"] = [corr] * cfg["num_layers"]
    return cfg


class OracleTACE(torch.nn.Module):
    """tace/models/_e3nn/tace.py:29-337 (constructor), :356-417 (energy readout), :788-790."""

    def __init__(self, **user_cfg):
        super().__init__()
        cfg = resolve_config(user_cfg)
        self.cfg = cfg
        self.register_buffer("cutoff", torch.tensor(float(cfg["cutoff"])))
        self.register_buffer("atomic_numbers", torch.tensor(cfg["atomic_numbers"], dtype=torch.int64))
        self.representation = Representation(cfg)
        # tace/models/_e3nn/readout.py:192-221: one read-out per layer with use_alllayer, else only the last
        C, hid = cfg["num_channel"], cfg["readout_emlp"]["hidden"]
        self.use_alllayer = bool(cfg["readout_emlp"].get("use_alllayer", False))
        nf = len(cfg["statistics"])  # one statistics entry per fidelity (tace/models/_e3nn/tace.py:75-76)
        if self.use_alllayer:
            prods = self.representation.products
            self.energy_readouts = torch.nn.ModuleList(
                [ScalarReadOut(C, hid, irreps_in=prods[t].irreps_out, last=(t == len(prods) - 1), num_fidelities=nf)
                 for t in range(len(prods))])
        else:
            self.energy_readouts = torch.nn.ModuleList([ScalarReadOut(C, hid, num_fidelities=nf)])
        zbl = cfg["short_range"]["zbl"]
        if zbl.get("enable"):  # tace/models/_e3nn/tace.py:222-228
            radii = torch.zeros(max(119, max(cfg["atomic_numbers"]) + 1))  # ase.data.covalent_radii has 119 entries
            for z, r in zbl["covalent_radii"].items():
                radii[int(z)] = float(r)
            self.zbl = ZBLBasis(radii, cfg["radial_basis"]["polynomial_cutoff"])
        self.scale_zbl = bool(cfg["scale_shift"].get("scale_zbl", True))
        self.atomic_energy_layer = AtomicEnergy(cfg["atomic_energies"], cfg["atomic_numbers"])
        sk, hk = cfg["scale_shift"]["scale_type"], cfg["scale_shift"]["shift_type"]
        scale_d, shift_d = [], []
        for s in cfg["statistics"]:
            scale_d.append({int(k): float(v) for k, v in (s[sk] if sk else {}).items()})
            shift_d.append({int(k): float(v) for k, v in (s[hk] if hk else {}).items()})
        self.scale_shift = ScaleShift(cfg["atomic_numbers"], scale_d, shift_d)


class OracleTensorModel(torch.nn.Module):
    """tace/models/adapter.py:23-41 (forward), :278-384 (prepare_graph), :59-174
    (first_derivative_fn); strain from tace/models/utils.py:50-79."""

    def __init__(self, readout_fn: OracleTACE):
        super().__init__()
        self.readout_fn = readout_fn

    def forward(self, data: Dict[str, torch.Tensor], compute_stress: bool = True,
                compute_edge_forces: bool = False) -> Dict[str, torch.Tensor]:
        m = self.readout_fn
        node_attrs = data["node_attrs"]
        batch, ptr, edge_index = data["batch"], data["ptr"], data["edge_index"]
        num_graphs = ptr.numel() - 1
        n = node_attrs.shape[0]
        # tace/models/adapter.py:280-284: the graph's fidelity for each of its atoms
        node_fidelity = data["fidelity_idx"][batch] if "fidelity_idx" in data else torch.zeros_like(batch)
        arange = torch.arange(n)
        lmp = "edge_vector" in data and "positions" not in data
        inputs = []
        if lmp:
            edge_vector = data["edge_vector"].detach().clone().requires_grad_(True)
            lattice = None
        else:
            positions = data["positions"].detach().clone().requires_grad_(True)
            lattice = data["lattice"].detach().clone()
            pos_in = positions
            inputs.append(positions)
            if compute_stress:
                displacement = torch.zeros(num_graphs, 3, 3, dtype=positions.dtype, requires_grad=True)
                sym = 0.5 * (displacement + displacement.transpose(-1, -2))
                pos_in = positions + torch.einsum("be,bec->bc", positions, sym[batch])
                lattice = lattice + torch.matmul(lattice, sym)
                inputs.append(displacement)
            src, dst = edge_index[0], edge_index[1]
            edge_vector = pos_in[dst] - pos_in[src] + torch.einsum(
                "ni,nij->nj", data["edge_shifts"], lattice[batch[src]])
            if compute_edge_forces:
                edge_vector.retain_grad()
        edge_length = (edge_vector**2).sum(dim=1, keepdim=True).sqrt() + 1e-9

        desc = m.representation(node_attrs, edge_index, edge_vector, edge_length)
        e_base_node = m.atomic_energy_layer(node_attrs)[arange, node_fidelity]
        e_base_graph = scatter_sum(e_base_node, batch, num_graphs)
        if m.use_alllayer:  # tace/models/_e3nn/tace.py:367-386: every layer's read-out, summed before scale / shift
            e_node = sum(ro(d, node_fidelity)[arange, node_fidelity] for ro, d in zip(m.energy_readouts, desc))
        else:
            e_node = m.energy_readouts[0](desc[-1], node_fidelity)[arange, node_fidelity]
        if hasattr(m, "zbl"):  # tace/models/_e3nn/tace.py:387-408: before the scale when scale_zbl, after it otherwise
            e_zbl = m.zbl(edge_length, node_attrs, edge_index, m.atomic_numbers)
            if m.scale_zbl:
                e_node = e_node + e_zbl
        e_node = m.scale_shift(e_node, node_attrs, ptr, edge_index, batch, node_fidelity)
        if hasattr(m, "zbl") and not m.scale_zbl:
            e_node = e_node + e_zbl
        e_graph = scatter_sum(e_node, batch, num_graphs)
        energy = e_base_graph + e_graph
        out = {"energy": energy.detach(), "node_energy": (e_base_node + e_node).detach(),
               "forces": None, "virials": None, "stress": None, "edge_forces": None}
        if lmp:
            (g,) = torch.autograd.grad(energy, [edge_vector], torch.ones_like(energy), allow_unused=True)
            out["edge_forces"] = torch.zeros_like(edge_vector) if g is None else g
            return out
        if compute_edge_forces:
            inputs.append(edge_vector)
        grads = torch.autograd.grad(energy, inputs, torch.ones_like(energy), allow_unused=True)
        out["forces"] = torch.zeros_like(positions) if grads[0] is None else -grads[0]
        idx = 1
        if compute_stress:
            v = torch.zeros_like(data["lattice"]) if grads[idx] is None else -grads[idx]
            vol = torch.linalg.det(data["lattice"]).abs().view(-1, 1, 1)
            s = -v / vol
            out["virials"] = v
            out["stress"] = torch.where(torch.abs(s) < 1e10, s, torch.zeros_like(s))
            idx += 1
        if compute_edge_forces:
            out["edge_forces"] = torch.zeros_like(edge_vector) if grads[idx] is None else grads[idx]
        return out


def build_oracle(cfg: Dict, state_dict: Optional[Dict[str, torch.Tensor]] = None,
                 dtype: torch.dtype = torch.float64) -> OracleTensorModel:
    """Construct the oracle under ``dtype`` and load a reference-named state_dict
    (keys prefixed ``readout_fn.``, tace/lightning/lit_model.py:664-677)."""
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        model = OracleTensorModel(OracleTACE(**cfg))
    finally:
        torch.set_default_dtype(prev)
    if state_dict is not None:
        own = model.state_dict()
        missing = [k for k in own if k not in state_dict]
        if missing:
            raise KeyError(f"state_dict lacks {missing[:5]} ...")
        model.load_state_dict({k: state_dict[k].to(own[k].dtype) for k in own}, strict=True)
    return model.to(dtype)
