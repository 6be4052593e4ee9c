"""A small stand-in for the third-party package ``e3nn``.  TEST INFRASTRUCTURE ONLY.

The reference (xvzemin/tace) delegates irreps bookkeeping, Wigner-3j symbols, spherical harmonics, the
weighted tensor product, the irreps-aware linear layer and the gate building blocks to ``e3nn``, which
is absent from the reference tree and cannot be installed offline.  To run the reference's OWN source
files here (``tests/refshim/loader.py``) this module offers the part of the ``e3nn`` interface those
files touch, written from e3nn's documented behaviour.  All arithmetic conventions (real 3j symbols,
harmonics with y as polar axis, "component" / "element" normalisation, 1/sqrt(fan-in) linears, second
moment constants) come from ``oracle/o3.py``; so a comparison "reference files + this stand-in" against
the oracle pins everything the reference itself implements, and leaves exactly these conventions
unpinned.
"""

from __future__ import annotations

import collections
import math
import re
import sys
import types
from typing import List, Optional

import torch

from oracle import o3 as _o3


# ---------------------------------------------------------------------------------------------------
# Irrep / Irreps
# ---------------------------------------------------------------------------------------------------
class Irrep(tuple):
    """(l, p) with p = +1 ("e") or -1 ("o")."""

    def __new__(cls, l, p=None):
        if p is None:
            if isinstance(l, Irrep):
                return l
            if isinstance(l, str):
                m = re.fullmatch(r"\s*(\d+)([eoy])\s*", l)
                if m is None:
                    raise ValueError(f"cannot read irrep {l!r}")
                ll = int(m.group(1))
                p = {"e": 1, "o": -1, "y": (-1) ** ll}[m.group(2)]
                l = ll
            elif isinstance(l, (tuple, list)):
                l, p = l
            else:
                raise ValueError(f"cannot read irrep {l!r}")
        return super().__new__(cls, (int(l), int(p)))

    @property
    def l(self) -> int:
        return self[0]

    @property
    def p(self) -> int:
        return self[1]

    @property
    def dim(self) -> int:
        return 2 * self[0] + 1

    def _key(self):
        return (self.l, -self.p * (-1) ** self.l)

    def __lt__(self, other):
        return self._key() < Irrep(other)._key()

    def __le__(self, other):
        return self._key() <= Irrep(other)._key()

    def __gt__(self, other):
        return self._key() > Irrep(other)._key()

    def __ge__(self, other):
        return self._key() >= Irrep(other)._key()

    def __eq__(self, other):
        try:
            other = Irrep(other)
        except (ValueError, TypeError):
            return False
        return tuple(self) == tuple(other)

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(tuple(self))

    def __mul__(self, other):
        other = Irrep(other)
        return [Irrep(l, self.p * other.p) for l in range(abs(self.l - other.l), self.l + other.l + 1)]

    def __rmul__(self, mul):
        return Irreps([(int(mul), self)])

    def __repr__(self):
        return f"{self.l}{'e' if self.p == 1 else 'o'}"

    def is_scalar(self):
        return self.l == 0 and self.p == 1


class _MulIr(tuple):
    def __new__(cls, mul, ir):
        return super().__new__(cls, (int(mul), Irrep(ir)))

    @property
    def mul(self) -> int:
        return self[0]

    @property
    def ir(self) -> Irrep:
        return self[1]

    @property
    def dim(self) -> int:
        return self.mul * self.ir.dim

    def __repr__(self):
        return f"{self.mul}x{self.ir}"


_SortResult = collections.namedtuple("sort", ["irreps", "p", "inv"])


class Irreps(tuple):
    def __new__(cls, irreps=None):
        if isinstance(irreps, Irreps):
            return super().__new__(cls, tuple(irreps))
        out = []
        if irreps is None:
            pass
        elif isinstance(irreps, Irrep):
            out.append(_MulIr(1, irreps))
        elif isinstance(irreps, str):
            text = irreps.strip()
            if text:
                for part in text.split("+"):
                    part = part.strip()
                    if "x" in part:
                        mul, ir = part.split("x")
                        out.append(_MulIr(int(mul), Irrep(ir)))
                    else:
                        out.append(_MulIr(1, Irrep(part)))
        else:
            for item in irreps:
                if isinstance(item, _MulIr):
                    out.append(item)
                elif isinstance(item, Irrep):
                    out.append(_MulIr(1, item))
                elif isinstance(item, str):
                    out.extend(Irreps(item))
                else:
                    mul, ir = item
                    out.append(_MulIr(mul, Irrep(ir)))
        return super().__new__(cls, tuple(out))

    @staticmethod
    def spherical_harmonics(lmax: int, p: int = -1) -> "Irreps":
        return Irreps([(1, (l, p ** l)) for l in range(lmax + 1)])

    @property
    def dim(self) -> int:
        return sum(mi.dim for mi in self)

    @property
    def num_irreps(self) -> int:
        return sum(mi.mul for mi in self)

    @property
    def ls(self) -> List[int]:
        return [mi.ir.l for mi in self for _ in range(mi.mul)]

    @property
    def lmax(self) -> int:
        if len(self) == 0:
            raise ValueError("empty irreps have no lmax")
        return max(mi.ir.l for mi in self)

    def slices(self):
        out, acc = [], 0
        for mi in self:
            out.append(slice(acc, acc + mi.dim))
            acc += mi.dim
        return out

    def simplify(self) -> "Irreps":
        out = []
        for mi in self:
            if mi.mul == 0:
                continue
            if out and out[-1][1] == mi.ir:
                out[-1] = (out[-1][0] + mi.mul, mi.ir)
            else:
                out.append((mi.mul, mi.ir))
        return Irreps(out)

    def remove_zero_multiplicities(self) -> "Irreps":
        return Irreps([(mi.mul, mi.ir) for mi in self if mi.mul > 0])

    def sort(self):
        order = sorted(range(len(self)), key=lambda i: (self[i].ir._key(), i))  # stable in the original position
        inv = tuple(order)
        p = [0] * len(self)
        for new, old in enumerate(order):
            p[old] = new
        return _SortResult(Irreps([self[i] for i in order]), tuple(p), inv)

    def regroup(self) -> "Irreps":
        return self.sort().irreps.simplify()

    def count(self, ir) -> int:
        ir = Irrep(ir)
        return sum(mi.mul for mi in self if mi.ir == ir)

    def __contains__(self, ir) -> bool:
        try:
            ir = Irrep(ir)
        except (ValueError, TypeError):
            return False
        return any(mi.ir == ir for mi in self)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return Irreps(tuple.__getitem__(self, i))
        return tuple.__getitem__(self, i)

    def __add__(self, other) -> "Irreps":
        return Irreps(tuple(self) + tuple(Irreps(other)))

    def __radd__(self, other) -> "Irreps":
        return Irreps(other) + self

    def __mul__(self, n) -> "Irreps":
        if isinstance(n, Irreps):
            raise NotImplementedError
        return Irreps(tuple(self) * int(n))

    __rmul__ = __mul__

    def __eq__(self, other):
        try:
            other = Irreps(other)
        except (ValueError, TypeError):
            return False
        return tuple(self) == tuple(other)

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash(tuple(self))

    def __repr__(self):
        return "+".join(repr(mi) for mi in self)

    def randn(self, *size, **kw):
        size = [self.dim if s == -1 else s for s in size]
        return torch.randn(*size, **kw)


# ---------------------------------------------------------------------------------------------------
# arithmetic conventions (from the oracle)
# ---------------------------------------------------------------------------------------------------
def wigner_3j(l1, l2, l3, dtype=None, device=None):
    return _o3.wigner_3j(int(l1), int(l2), int(l3), dtype=dtype or torch.get_default_dtype())


def _spherical_harmonics(lmax: int, x: torch.Tensor, y: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """The raw polynomial table: component normalisation, blocks l = 0..lmax."""
    return _o3.spherical_harmonics(int(lmax), torch.stack([x, y, z], dim=-1), "component")


def spherical_harmonics(l, x, normalize, normalization="integral"):
    if isinstance(l, int):
        ls = [l]
    elif isinstance(l, (list, tuple)) and all(isinstance(k, int) for k in l):
        ls = list(l)
    else:
        ls = [mi.ir.l for mi in Irreps(l) for _ in range(mi.mul)]
    if normalize:
        x = torch.nn.functional.normalize(x, dim=-1)
    sh = _spherical_harmonics(max(ls), x[..., 0], x[..., 1], x[..., 2])
    sh = torch.cat([sh[..., k * k:(k + 1) ** 2] for k in ls], dim=-1)
    if normalization == "integral":
        sh = sh / math.sqrt(4 * math.pi)
    elif normalization == "norm":
        sh = sh / torch.cat([math.sqrt(2 * k + 1) * torch.ones(2 * k + 1, dtype=sh.dtype) for k in ls])
    return sh


def _second_moment_constant(act) -> float:
    gen = torch.Generator(device="cpu").manual_seed(0)
    z = torch.randn(1_000_000, generator=gen, dtype=torch.float64, device="cpu")
    with torch.no_grad():
        c = act(z).pow(2).mean().pow(-0.5).item()
    return 1.0 if abs(c - 1.0) < 1e-4 else c


class _Normalised(torch.nn.Module):
    def __init__(self, act):
        super().__init__()
        self.act = act
        self.cst = _second_moment_constant(act)

    def forward(self, x):
        return self.act(x) * self.cst


# ---------------------------------------------------------------------------------------------------
# o3.Linear
# ---------------------------------------------------------------------------------------------------
_LinIns = collections.namedtuple("Instruction", ["i_in", "i_out", "path_shape", "path_weight"])


class Linear(torch.nn.Module):
    """One [mul_in, mul_out] block for every pair (input block, output block) of equal irrep, input-major; every
    block scaled by 1 / sqrt(total multiplicity feeding that output block) ("element" path normalisation)."""

    def __init__(self, irreps_in, irreps_out, internal_weights=None, shared_weights=None, biases=False, **_):
        super().__init__()
        self.irreps_in, self.irreps_out = Irreps(irreps_in), Irreps(irreps_out)
        pairs = [(i, o) for i, mi in enumerate(self.irreps_in) for o, mo in enumerate(self.irreps_out) if mi.ir == mo.ir]
        fan = collections.Counter()
        for i, o in pairs:
            fan[o] += self.irreps_in[i].mul
        self.instructions = [
            _LinIns(i, o, (self.irreps_in[i].mul, self.irreps_out[o].mul), fan[o] ** -0.5) for i, o in pairs]
        self.weight_numel = sum(a * b for _, _, (a, b), _ in self.instructions)
        if shared_weights is None:
            shared_weights = True if internal_weights is None else bool(internal_weights)
        if internal_weights is None:
            internal_weights = shared_weights
        self.shared_weights, self.internal_weights = shared_weights, internal_weights
        if internal_weights:
            self.weight = torch.nn.Parameter(torch.randn(self.weight_numel))
        if biases:
            raise NotImplementedError("the reference adds its own biases")

    def forward(self, x, weight=None):
        if weight is None:
            weight = self.weight
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        n = x2.shape[0]
        w = weight.reshape(-1, self.weight_numel) if weight.dim() > 1 else weight.unsqueeze(0)
        outs = [x2.new_zeros(n, mo.mul, mo.ir.dim) for mo in self.irreps_out]
        sl, off = self.irreps_in.slices(), 0
        for ins in self.instructions:
            a, b = ins.path_shape
            wi = w[:, off:off + a * b].reshape(-1, a, b)
            off += a * b
            xi = x2[:, sl[ins.i_in]].reshape(n, a, self.irreps_in[ins.i_in].ir.dim)
            if wi.shape[0] == 1:
                term = torch.einsum("uw,zui->zwi", wi[0], xi)
            else:
                term = torch.einsum("zuw,zui->zwi", wi, xi)
            outs[ins.i_out] = outs[ins.i_out] + ins.path_weight * term
        out = torch.cat([t.reshape(n, -1) for t in outs], dim=-1) if outs else x2.new_zeros(n, 0)
        return out.reshape(*lead, self.irreps_out.dim)

    def __repr__(self):
        return f"Linear({self.irreps_in} -> {self.irreps_out} | {self.weight_numel} weights)"


# ---------------------------------------------------------------------------------------------------
# o3.TensorProduct
# ---------------------------------------------------------------------------------------------------
_TpIns = collections.namedtuple("Instruction", ["i_in1", "i_in2", "i_out", "connection_mode", "has_weight", "path_weight", "path_shape"])


class TensorProduct(torch.nn.Module):
    """Weighted tensor product with explicit instructions; "component" irrep normalisation (factor 2 l_out + 1 under
    the root) and "element" path normalisation (divide by the number of summed products feeding the output block)."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, instructions, in1_var=None, in2_var=None, out_var=None,
                 irrep_normalization="component", path_normalization="element", internal_weights=None,
                 shared_weights=None, **_):
        super().__init__()
        self.irreps_in1, self.irreps_in2, self.irreps_out = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        if irrep_normalization != "component" or path_normalization != "element":
            raise NotImplementedError
        raw = []
        for ins in instructions:
            ins = tuple(ins)
            if len(ins) == 5:
                ins = ins + (1.0,)
            i1, i2, io, mode, has_w, pw = ins
            m1, m2, mo = self.irreps_in1[i1].mul, self.irreps_in2[i2].mul, self.irreps_out[io].mul
            shape = {"uvw": (m1, m2, mo), "uvu": (m1, m2), "uvv": (m1, m2), "uuw": (m1, mo), "uuu": (m1,), "uvuv": (m1, m2)}[mode]
            raw.append((i1, i2, io, mode, bool(has_w), float(pw), shape))

        def n_sum(i1, i2, mode):
            m1, m2 = self.irreps_in1[i1].mul, self.irreps_in2[i2].mul
            return {"uvw": m1 * m2, "uvu": m2, "uvv": m1, "uuw": m1, "uuu": 1, "uvuv": 1}[mode]

        total = collections.Counter()
        for i1, i2, io, mode, _, _, _ in raw:
            total[io] += n_sum(i1, i2, mode)
        self.instructions = []
        for i1, i2, io, mode, has_w, pw, shape in raw:
            alpha = self.irreps_out[io].ir.dim * pw / total[io]
            self.instructions.append(_TpIns(i1, i2, io, mode, has_w, math.sqrt(alpha), shape))
        self.weight_numel = sum(math.prod(i.path_shape) for i in self.instructions if i.has_weight)
        if shared_weights is None:
            shared_weights = True if internal_weights is None else bool(internal_weights)
        if internal_weights is None:
            internal_weights = shared_weights and self.weight_numel > 0
        self.shared_weights, self.internal_weights = shared_weights, internal_weights
        if internal_weights and self.weight_numel > 0:
            self.weight = torch.nn.Parameter(torch.randn(self.weight_numel))

    def forward(self, x1, x2, weight=None):
        if weight is None and self.weight_numel > 0:
            weight = self.weight
        n = x1.shape[0]
        s1, s2 = self.irreps_in1.slices(), self.irreps_in2.slices()
        outs = [None] * len(self.irreps_out)
        off = 0
        for ins in self.instructions:
            mi1, mi2, mo = self.irreps_in1[ins.i_in1], self.irreps_in2[ins.i_in2], self.irreps_out[ins.i_out]
            c = wigner_3j(mi1.ir.l, mi2.ir.l, mo.ir.l, dtype=x1.dtype) * ins.path_weight
            a = x1[:, s1[ins.i_in1]].reshape(n, mi1.mul, mi1.ir.dim)
            b = x2[:, s2[ins.i_in2]].reshape(n, mi2.mul, mi2.ir.dim)
            w = None
            if ins.has_weight:
                k = math.prod(ins.path_shape)
                w = weight[..., off:off + k]
                w = w.reshape((-1,) + tuple(ins.path_shape))
                if w.shape[0] == 1 and n != 1:
                    w = w.expand((n,) + tuple(ins.path_shape))
                off += k
            mode = ins.connection_mode
            if mode == "uvu":
                o = torch.einsum("zuv,ijk,zui,zvj->zuk", w, c, a, b) if w is not None else torch.einsum("ijk,zui,zvj->zuk", c, a, b)
            elif mode == "uuu":
                o = torch.einsum("zu,ijk,zui,zuj->zuk", w, c, a, b) if w is not None else torch.einsum("ijk,zui,zuj->zuk", c, a, b)
            elif mode == "uvw":
                o = torch.einsum("zuvw,ijk,zui,zvj->zwk", w, c, a, b)
            else:
                raise NotImplementedError(mode)
            o = o.reshape(n, mo.mul * mo.ir.dim)
            outs[ins.i_out] = o if outs[ins.i_out] is None else outs[ins.i_out] + o
        outs = [x1.new_zeros(n, mo.dim) if o is None else o for o, mo in zip(outs, self.irreps_out)]
        return torch.cat(outs, dim=-1) if outs else x1.new_zeros(n, 0)


class ElementwiseTensorProduct(TensorProduct):
    """Channel-wise product of two inputs with the same total multiplicity, no weights."""

    def __init__(self, irreps_in1, irreps_in2, filter_ir_out=None, irrep_normalization=None, **kw):
        a, b = list(Irreps(irreps_in1).simplify()), list(Irreps(irreps_in2).simplify())
        a = [(mi.mul, mi.ir) for mi in a]
        b = [(mi.mul, mi.ir) for mi in b]
        if sum(m for m, _ in a) != sum(m for m, _ in b):
            raise ValueError("both inputs need the same number of irreps")
        i = 0
        while i < len(a):  # cut both lists into pieces of equal multiplicity
            m1, ir1 = a[i]
            m2, ir2 = b[i]
            if m1 < m2:
                b[i] = (m1, ir2)
                b.insert(i + 1, (m2 - m1, ir2))
            elif m2 < m1:
                a[i] = (m2, ir1)
                a.insert(i + 1, (m1 - m2, ir1))
            i += 1
        out, instr = [], []
        for i, ((mul, ir1), (_, ir2)) in enumerate(zip(a, b)):
            for ir in ir1 * ir2:
                if filter_ir_out is not None and ir not in [Irrep(f) for f in filter_ir_out]:
                    continue
                instr.append((i, i, len(out), "uuu", False))
                out.append((mul, ir))
        super().__init__(a, b, out, instr, **kw)


# ---------------------------------------------------------------------------------------------------
# e3nn.nn
# ---------------------------------------------------------------------------------------------------
class Activation(torch.nn.Module):
    """One scalar function (or None) per block of scalar irreps, each rescaled to unit second moment."""

    def __init__(self, irreps_in, acts):
        super().__init__()
        self.irreps_in = Irreps(irreps_in)
        if len(self.irreps_in) != len(acts):
            raise ValueError("one activation per irreps block")
        self.acts = torch.nn.ModuleList([None if a is None else _Normalised(a) for a in acts])
        for mi, a in zip(self.irreps_in, acts):
            if a is not None and mi.ir.l != 0:
                raise ValueError("activations act on scalars only")
        self.irreps_out = self.irreps_in

    def forward(self, x):
        out = []
        for sl, a in zip(self.irreps_in.slices(), self.acts):
            out.append(x[..., sl] if a is None else a(x[..., sl]))
        return torch.cat(out, dim=-1) if out else x


class _Sortcut(torch.nn.Module):
    """Splits one input, laid out as the sorted concatenation of several irreps lists, back into those lists."""

    def __init__(self, *irreps_outs):
        super().__init__()
        outs = [Irreps(i) for i in irreps_outs]
        blocks = [(k, j, mi) for k, irr in enumerate(outs) for j, mi in enumerate(irr)]
        order = sorted(range(len(blocks)), key=lambda i: (blocks[i][2].ir._key(), i))
        self.irreps_in = Irreps([blocks[i][2] for i in order]).simplify()
        start, where = 0, {}
        for i in order:
            k, j, mi = blocks[i]
            where[(k, j)] = (start, start + mi.dim)
            start += mi.dim
        self._pieces = [[where[(k, j)] for j in range(len(irr))] for k, irr in enumerate(outs)]
        self.irreps_outs = tuple(irr.simplify() for irr in outs)

    def forward(self, x):
        res = []
        for pieces in self._pieces:
            res.append(torch.cat([x[..., a:b] for a, b in pieces], dim=-1) if pieces else x[..., :0])
        return tuple(res)


class Gate(torch.nn.Module):
    """[scalars | gate scalars | gated] -> [act(scalars) | gated * act(gates)]."""

    def __init__(self, irreps_scalars, act_scalars, irreps_gates, act_gates, irreps_gated):
        super().__init__()
        irreps_scalars, irreps_gates, irreps_gated = Irreps(irreps_scalars), Irreps(irreps_gates), Irreps(irreps_gated)
        if irreps_gates.num_irreps != irreps_gated.num_irreps:
            raise ValueError("one gate scalar per gated irrep")
        self.sc = _Sortcut(irreps_scalars, irreps_gates, irreps_gated)
        self.irreps_scalars, self.irreps_gates, self.irreps_gated = self.sc.irreps_outs
        self._irreps_in = self.sc.irreps_in
        self.act_scalars = Activation(irreps_scalars, act_scalars)
        self.act_gates = Activation(irreps_gates, act_gates)
        self.mul = ElementwiseTensorProduct(irreps_gated, irreps_gates)
        self._irreps_out = Irreps(irreps_scalars) + self.mul.irreps_out

    @property
    def irreps_in(self):
        return self._irreps_in

    @property
    def irreps_out(self):
        return self._irreps_out

    def forward(self, x):
        scalars, gates, gated = self.sc(x)
        scalars = self.act_scalars(scalars)
        if gates.shape[-1]:
            gated = self.mul(gated.reshape(-1, gated.shape[-1]), self.act_gates(gates).reshape(-1, gates.shape[-1]))
            gated = gated.reshape(*x.shape[:-1], gated.shape[-1])
            return torch.cat([scalars, gated], dim=-1)
        return scalars


# ---------------------------------------------------------------------------------------------------
# module objects
# ---------------------------------------------------------------------------------------------------
def _compile_mode(_mode):
    def deco(cls):
        return cls
    return deco


def _unavailable(name):
    def fail(*a, **k):
        raise NotImplementedError(f"e3nn.{name} is not part of the stand-in")
    return fail


def install() -> None:
    """Register the stand-in as ``e3nn`` in ``sys.modules`` (no-op when a real e3nn is importable)."""
    if "e3nn" in sys.modules and not getattr(sys.modules["e3nn"], "_tace_b200_stand_in", False):
        return

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    opt = {"jit_mode": "eager", "specialized_code": True, "optimize_einsums": False, "jit_script_fx": False}
    e3nn = mod("e3nn", _tace_b200_stand_in=True, get_optimization_defaults=lambda: dict(opt),
               set_optimization_defaults=lambda **k: opt.update(k), __version__="0.0-stand-in")
    irreps_mod = mod("e3nn.o3._irreps", Irrep=Irrep, Irreps=Irreps, _MulIr=_MulIr)
    sh_mod = mod("e3nn.o3._spherical_harmonics", _spherical_harmonics=_spherical_harmonics, spherical_harmonics=spherical_harmonics)
    sub_mod = mod("e3nn.o3._tensor_product._sub", ElementwiseTensorProduct=ElementwiseTensorProduct)
    tp_mod = mod("e3nn.o3._tensor_product", TensorProduct=TensorProduct, _sub=sub_mod)
    red_mod = mod("e3nn.o3._reduce", ReducedTensorProducts=_unavailable("o3.ReducedTensorProducts"))
    o3 = mod("e3nn.o3", Irrep=Irrep, Irreps=Irreps, wigner_3j=wigner_3j, Linear=Linear, TensorProduct=TensorProduct,
             ElementwiseTensorProduct=ElementwiseTensorProduct, spherical_harmonics=spherical_harmonics,
             Norm=_unavailable("o3.Norm"), FullyConnectedTensorProduct=_unavailable("o3.FullyConnectedTensorProduct"),
             _irreps=irreps_mod, _spherical_harmonics=sh_mod, _tensor_product=tp_mod, _reduce=red_mod)
    gate_mod = mod("e3nn.nn._gate", _Sortcut=_Sortcut, Gate=Gate)
    nn = mod("e3nn.nn", Activation=Activation, Gate=Gate, _gate=gate_mod,
             BatchNorm=_unavailable("nn.BatchNorm"), FullyConnectedNet=_unavailable("nn.FullyConnectedNet"))
    jit = mod("e3nn.util.jit", compile_mode=_compile_mode, script=lambda m: m, compile=lambda m: m)
    util = mod("e3nn.util", jit=jit)
    math_mod = mod("e3nn.math", normalize2mom=_Normalised)
    io_mod = mod("e3nn.io", CartesianTensor=_unavailable("io.CartesianTensor"))
    e3nn.o3, e3nn.nn, e3nn.util, e3nn.math, e3nn.io = o3, nn, util, math_mod, io_mod
