"""CPU restatement of the reference's TECE edge block.  TEST INFRASTRUCTURE ONLY.

The block (``atomic_basis.type = uv_so2``) rotates the features of both ends of an edge into a frame whose polar axis
is the edge, mixes them there with SO(2)-equivariant linears, a gate and a second / third order "edge cluster
expansion", weights every message with a per-head attention coefficient normalised over the incoming edges of the
target atom, rotates back and sums per target.  Every class cites the reference file:line it follows (paths relative to
the reference repository).

PARITY UNPINNED: the reference cannot be imported here (e3nn is absent) and none of its tests pins values of this
block; what the CPU tests pin instead is internal consistency: the Wigner matrices built here rotate this package's
spherical harmonics (``D(R) Y(v) = Y(R v)``), compose like a representation, the edge frame puts the edge on the polar
axis, and the whole block is equivariant under global rotations.
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from . import o3
from .model import SILU_CST, scatter_sum

SIGMOID_CST = 1.8467055342154763  # tace/models/mlp.py:40-46


# ---- edge frame ------------------------------------------------------------------------------------
def _norm(x: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    return torch.sqrt(torch.sum(x * x, dim=-1, keepdim=True) + eps * eps)


def _smooth_step(x: torch.Tensor) -> torch.Tensor:
    """tace/models/o2/rotation_matrix.py:25-36: C-infinity step from 0 (x <= 0) to 1 (x >= 1)."""
    x = x.clamp(0.0, 1.0)
    eps = torch.finfo(x.dtype).eps
    left = torch.exp(-1.0 / torch.clamp(x, min=eps))
    right = torch.exp(-1.0 / torch.clamp(1.0 - x, min=eps))
    interior = left / (left + right)
    return torch.where(x <= 0.0, torch.zeros_like(x), torch.where(x >= 1.0, torch.ones_like(x), interior))


def edge_rotation(edge_vector: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """tace/models/o2/rotation_matrix.py:74-88: the rotation that puts the edge on the y axis.  Two quaternions (one
    regular away from -y, one away from +y) are blended with a smooth step in the y component and renormalised."""
    unit = edge_vector / _norm(edge_vector, eps)
    x, y, z = unit.unbind(dim=-1)
    zero = torch.zeros_like(x)
    q_pos = torch.stack([1.0 + y, -z, zero, x], dim=-1)
    q_pos = q_pos / _norm(q_pos, eps)
    q_neg = torch.stack([-z, 1.0 - y, x, zero], dim=-1)
    q_neg = q_neg / _norm(q_neg, eps)
    blend = _smooth_step(0.5 * (y + 1.0))
    dot = torch.sum(q_neg * q_pos, dim=-1, keepdim=True)
    q1 = torch.where(dot < 0.0, -q_pos, q_pos)  # rotation_matrix.py:39-49 (nlerp from q_neg to q_pos)
    q = (1.0 - blend.unsqueeze(-1)) * q_neg + blend.unsqueeze(-1) * q1
    q = q / _norm(q, eps)
    w, qx, qy, qz = q.unbind(dim=-1)
    x2, y2, z2 = qx * qx, qy * qy, qz * qz
    xy, xz, yz = qx * qy, qx * qz, qy * qz
    wx, wy, wz = w * qx, w * qy, w * qz
    return torch.stack([
        torch.stack([1.0 - 2.0 * (y2 + z2), 2.0 * (xy - wz), 2.0 * (xz + wy)], dim=-1),
        torch.stack([2.0 * (xy + wz), 1.0 - 2.0 * (x2 + z2), 2.0 * (yz - wx)], dim=-1),
        torch.stack([2.0 * (xz - wy), 2.0 * (yz + wx), 1.0 - 2.0 * (x2 + y2)], dim=-1),
    ], dim=-2)


def wigner_blocks(rotation: torch.Tensor, lmax: int) -> List[torch.Tensor]:
    """tace/models/o2/wigner.py:316-357: D^0 = 1, D^1 = R (e3nn's l = 1 basis is (x, y, z) itself), and
    D^l = (2l+1) * C^T (D^1 (x) D^(l-1)) C with C = wigner_3j(1, l-1, l)."""
    blocks = [rotation.new_ones(rotation.shape[0], 1, 1)]
    if lmax >= 1:
        blocks.append(rotation)
    for l in range(2, lmax + 1):
        cg = o3.wigner_3j(1, l - 1, l, dtype=rotation.dtype)
        left = torch.einsum("abm,eac->ebmc", cg, blocks[1])
        left = torch.einsum("ebmc,ebd->emcd", left, blocks[l - 1])
        blocks.append(torch.einsum("emcd,cdn->emn", left, cg) * (2 * l + 1))
    return blocks


def m_layout(lmax: int, mmax: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """tace/models/o2/wigner.py:22-167 (CoefficientMappingModule): for every row of the order-major layout
    [m = 0: l = 0..lmax | m = 1: l = 1..lmax, then the same for -1 | m = 2 ...] its index in the (l, m) layout of the
    full (lmax+1)^2 vector, and its rank l."""
    rows, ranks = [], []
    for m in range(mmax + 1):
        for sign in ((1,) if m == 0 else (1, -1)):
            for l in range(m, lmax + 1):
                rows.append(l * l + l + sign * m)
                ranks.append(l)
    return torch.tensor(rows, dtype=torch.int64), torch.tensor(ranks, dtype=torch.int64)


class WignerD(torch.nn.Module):
    """tace/models/o2/wigner.py:178-239: per edge, the rows of blockdiag(D^0..D^lmax) of the edge frame that belong to
    orders |m| <= mmax, in order-major layout ([n_m, (lmax+1)^2]), and the inverse map ([(lmax+1)^2, n_m]) = its
    transpose, where ranks l > mmax are rescaled by sqrt((2l+1) / (2 mmax+1)) to make up for the dropped orders."""

    def __init__(self, mmax: int, lmax: int):
        super().__init__()
        self.mmax, self.lmax = mmax, lmax
        rows, ranks = m_layout(lmax, mmax)
        self.register_buffer("rows", rows, persistent=False)
        scale = torch.tensor([math.sqrt((2 * int(l) + 1) / (2 * mmax + 1)) if int(l) > mmax else 1.0 for l in ranks])
        self.register_buffer("inv_rescale", scale, persistent=False)

    def get_wigner(self, edge_vector: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        blocks = wigner_blocks(edge_rotation(edge_vector), self.lmax)
        full = edge_vector.new_zeros(edge_vector.shape[0], (self.lmax + 1) ** 2, (self.lmax + 1) ** 2)
        for l, blk in enumerate(blocks):
            full[:, l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = blk
        wigner = full[:, self.rows, :]
        wigner_inv = wigner.transpose(1, 2) * self.inv_rescale.to(wigner.dtype)
        return wigner, wigner_inv.contiguous()


# ---- SO(2) building blocks ---------------------------------------------------------------------------
class TorchLinear(torch.nn.Module):
    """tace/models/linear.py:210-244: y = x W^T / sqrt(fan_in) + b, unit-normal weights [out, in]."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.randn(out_features, in_features))
        self.bias = torch.nn.Parameter(torch.zeros(out_features)) if bias else None
        self.alpha = 1.0 / math.sqrt(in_features)

    def forward(self, x):
        y = torch.matmul(x, self.weight.t()) * self.alpha
        return y if self.bias is None else y + self.bias


class SO2MLinear(torch.nn.Module):
    """tace/models/_e3nn/archive/oam_2026_07_05.py:46-135, weight type "w1" (the one the block uses): one real matrix
    applied to the +m and to the -m components alike."""

    def __init__(self, c_in: int, c_out: int, n_in: int, n_out: int):
        super().__init__()
        self.fc = TorchLinear(n_in * c_in, n_out * c_out, bias=False)

    def forward(self, x):  # [E, 2, n_in * c_in]
        return self.fc(x)


class SO2Linear(torch.nn.Module):
    """oam_2026_07_05.py:138-229: features [E, components, C] in order-major layout; the m = 0 block goes through one
    real linear with bias, every m > 0 block through its own SO2MLinear."""

    def __init__(self, mmax: int, lmax: int, c_in: int, c_out: int, n_in: Optional[List[int]] = None,
                 n_out: Optional[List[int]] = None):
        super().__init__()
        self.mmax, self.lmax, self.c_in, self.c_out = mmax, lmax, c_in, c_out
        self.n_in = n_in if n_in is not None else [lmax + 1 - m for m in range(mmax + 1)]
        self.n_out = n_out if n_out is not None else [lmax + 1 - m for m in range(mmax + 1)]
        self.m0_rlinear = TorchLinear(c_in * self.n_in[0], c_out * self.n_out[0], bias=True)
        self.ms_clinear = torch.nn.ModuleList(
            [SO2MLinear(c_in, c_out, self.n_in[m], self.n_out[m]) for m in range(1, mmax + 1)])

    def forward(self, x):
        E = x.shape[0]
        outs = [self.m0_rlinear(x[:, :self.n_in[0]].reshape(E, -1)).view(E, self.n_out[0], self.c_out)]
        offset = self.lmax + 1  # oam_2026_07_05.py:211 (the m = 0 block always spans lmax + 1 rows of the input)
        for m in range(1, self.mmax + 1):
            xm = x[:, offset:offset + 2 * self.n_in[m]].reshape(E, 2, self.n_in[m] * self.c_in)
            offset += 2 * self.n_in[m]
            ym = self.ms_clinear[m - 1](xm)
            outs.append(ym[:, 0].reshape(E, self.n_out[m], self.c_out))
            outs.append(ym[:, 1].reshape(E, self.n_out[m], self.c_out))
        return torch.cat(outs, dim=1)


def so2_expand_index(mmax: int, lmax: int, start: int = 0) -> Tuple[int, torch.Tensor]:
    """oam_2026_07_05.py:18-31: one index per (m, l >= m) pair, repeated for +m and -m."""
    idx, offset = [], 0
    for m in range(start, mmax + 1):
        block = torch.arange(lmax + 1 - m) + offset
        idx.append(block)
        if m > 0:
            idx.append(block)
        offset += lmax + 1 - m
    return offset, torch.cat(idx).long()


class SO2Gate(torch.nn.Module):
    """oam_2026_07_05.py:250-309."""

    def __init__(self, mmax, lmax, num_channel, scalar_act, tensor_act, channel_wise=False, gate_m0=True):
        super().__init__()
        self.num_channel, self.gate_m0, self.n_m0 = num_channel, gate_m0, lmax + 1
        start = 0 if gate_m0 else 1
        if not channel_wise:
            self.num_components, idx = so2_expand_index(mmax, lmax, start) if start <= mmax else (0, torch.empty(0, dtype=torch.long))
        else:  # every order carries lmax + 1 rows (the layout of the edge cluster expansion)
            parts, offset = [], 0
            for m in range(start, mmax + 1):
                block = torch.arange(lmax + 1) + offset
                parts.append(block)
                if m > 0:
                    parts.append(block)
                offset += lmax + 1
            idx = torch.cat(parts).long() if parts else torch.empty(0, dtype=torch.long)
            self.num_components = offset
        self.register_buffer("expand_index", idx, persistent=False)
        self.scalar_act, self.tensor_act = scalar_act, tensor_act

    def forward(self, x, g):
        E = x.shape[0]
        g = self.tensor_act(g).view(E, self.num_components, self.num_channel)[:, self.expand_index]
        if self.gate_m0:
            return g * x
        return torch.cat((self.scalar_act(x[:, :self.n_m0]), g * x[:, self.n_m0:]), dim=1)


class SO2Product(torch.nn.Module):
    """oam_2026_07_05.py:312-488 with ``m1m2 = ">="`` and external weights (ComplexProductBasis :519-544): channel-wise
    products of the complex order-m components of x and y, every order carrying lmax + 1 rows; path (m1, m2) feeds
    m3 = m1 + m2 ("sum", x y) or |m1 - m2| ("diff", x conj(y)); per path one weight per (row, channel); every output
    order is divided by sqrt(number of paths into it)."""

    def __init__(self, mmax: int, lmax: int, num_channel: int):
        super().__init__()
        self.mmax, self.lmax, self.C = mmax, lmax, num_channel
        self.paths = []
        for m3 in range(mmax + 1):
            ps = []
            for m1 in range(mmax + 1):
                for m2 in range(mmax + 1):
                    if m1 >= m2:
                        if m1 + m2 == m3:
                            ps.append((m1, m2, "sum"))
                        elif abs(m1 - m2) == m3:
                            ps.append((m1, m2, "diff"))
            self.paths.append(ps)
        n = lmax + 1
        self.weight_numel = num_channel * n * sum(len(p) for p in self.paths)
        scales = [torch.full((n,), 1.0 / math.sqrt(len(self.paths[0])))]
        for m3 in range(1, mmax + 1):
            scales.append(torch.full((2 * n,), 1.0 / math.sqrt(len(self.paths[m3]))))
        self.register_buffer("output_scales", torch.cat(scales), persistent=False)

    def _split(self, x):
        E, n = x.shape[0], self.lmax + 1
        out, off = [x[:, :n]], n
        for _ in range(1, self.mmax + 1):
            out.append(x[:, off:off + 2 * n].view(E, 2, n, self.C))
            off += 2 * n
        return out

    @staticmethod
    def _cmul(x, y, mode):
        a, b, c, d = x[:, 0], x[:, 1], y[:, 0], y[:, 1]
        if mode == "sum":
            return torch.stack([a * c - b * d, a * d + b * c], dim=1)
        return torch.stack([a * c + b * d, b * c - a * d], dim=1)

    def forward(self, x, y, ws):
        xs, ys = self._split(x), self._split(y)
        n, C = self.lmax + 1, self.C
        w_off, wn = 0, C * n
        outs = []
        m0 = 0.0
        for m1, m2, _mode in self.paths[0]:
            w = ws[:, w_off:w_off + wn].view(-1, n, C)
            w_off += wn
            if m1 == 0 and m2 == 0:
                m0 = m0 + xs[0] * ys[0] * w
            elif m1 > 0 and m2 > 0:  # real part of x conj(y)
                m0 = m0 + self._cmul(xs[m1], ys[m2], "diff")[:, 0] * w
        outs.append(m0)
        for m3 in range(1, self.mmax + 1):
            real, imag = 0.0, 0.0
            for m1, m2, mode in self.paths[m3]:
                w = ws[:, w_off:w_off + wn].view(-1, 1, n, C)
                w_off += wn
                if m1 == 0:
                    z = xs[m1].unsqueeze(1) * ys[m2]
                elif m2 == 0:
                    z = xs[m1] * ys[m2].unsqueeze(1)
                elif m1 < m2 and mode == "diff":
                    z = self._cmul(ys[m2], xs[m1], mode)
                else:
                    z = self._cmul(xs[m1], ys[m2], mode)
                z = z * w
                real, imag = real + z[:, 0], imag + z[:, 1]
            outs += [real, imag]
        return torch.cat(outs, dim=1) * self.output_scales.view(1, -1, 1)


def graph_softmax(src, index, num_nodes, exp_rescale=None, eps=1e-16):
    """tace/models/softmax.py:80-114 (index form): softmax over the edges that share a target, every exponential
    multiplied by ``exp_rescale`` (the cutoff envelope) before the normalisation."""
    src_max = torch.full((num_nodes,) + src.shape[1:], -float("inf"), dtype=src.dtype)
    src_max = src_max.scatter_reduce(0, index.view(-1, *([1] * (src.dim() - 1))).expand_as(src), src.detach(), "amax")
    out = (src - src_max[index]).exp()
    if exp_rescale is not None:
        out = out * exp_rescale
    out_sum = scatter_sum(out, index, num_nodes) + eps
    return out / out_sum[index]


class EdgeConvolution(torch.nn.Module):
    """oam_2026_07_05.py:547-823 (OAM20260705Convolution) with the switches the interaction sets
    (tace/models/_e3nn/inter.py:451-455,468-492): SO(2) linears of type "w1", temperature, edge cluster expansion, graph
    softmax and radial phase all on.  Node features are [N, (lmax+1)^2, C] here (the reference's LayoutTransform gives
    the same view of its e3nn-layout rows, tace/models/layout.py:48-86)."""

    def __init__(self, mmax, lmax, num_channel, num_head, edge_ace_hidden, edge_wise_hidden, num_radial_basis, gate_m0,
                 scalar_act, tensor_act):
        super().__init__()
        self.mmax, self.lmax, self.C, self.H = mmax, lmax, num_channel, num_head
        self.ace_hidden = edge_ace_hidden
        self.hidden = edge_wise_hidden or num_channel
        assert self.hidden % num_head == 0
        self.c_head = self.hidden // num_head
        self.num_components, idx = so2_expand_index(mmax, lmax)
        self.weight_numel = self.num_components * num_channel * 2
        self.register_buffer("expand_index", idx, persistent=False)
        n = lmax + 1
        start_m = 0 if gate_m0 else 1
        self.num_gates = sum(n for _ in range(start_m, mmax + 1))
        full = [n for _ in range(mmax + 1)]
        self.split = [self.num_gates, n + sum(2 * n for _ in range(1, mmax + 1))]
        self.linear_up = SO2Linear(mmax, lmax, 2 * num_channel, edge_ace_hidden, n_out=[self.num_gates + n] + full[1:])
        self.nonlinearity = SO2Gate(mmax, lmax, edge_ace_hidden, scalar_act, tensor_act, channel_wise=True, gate_m0=gate_m0)
        self.linear_glu = SO2Linear(mmax, lmax, 2 * num_channel, edge_ace_hidden, n_out=list(full))
        self.ece = SO2Product(mmax, lmax, edge_ace_hidden)
        self.linear_coefs = SO2Linear(0, lmax, 2 * num_channel, 1, n_out=[self.ece.weight_numel])
        self.linear_down = SO2Linear(mmax, lmax, edge_ace_hidden, self.hidden, n_in=list(full))
        self.query_proj = SO2Linear(mmax, lmax, num_channel, self.hidden)
        self.key_proj = SO2Linear(mmax, lmax, num_channel, self.hidden)
        self.radial_proj = TorchLinear(num_radial_basis, 2 * num_head)
        torch.nn.init.zeros_(self.radial_proj.weight)
        self.attention_scale = 1.0 / math.sqrt(self.c_head * self.split[1])
        self.t_min, self.t_max = 0.25, 4.0
        self.temperature_logit = torch.nn.Parameter(torch.full((num_head,), math.log((1.0 - self.t_min) / (self.t_max - 1.0))))

    def _attention(self, query, key, radial_basis):
        """oam_2026_07_05.py:699-754: per head, <q, k> over rows and channels with the order-m part of the key turned by
        m * pi * tanh(radial projection), scaled by the temperature, plus a radial bias."""
        E, H, Ch = query.shape[0], self.H, self.c_head
        proj = self.radial_proj(radial_basis)
        bias, phase = proj[:, :H], math.pi * torch.tanh(proj[:, H:])
        n = self.lmax + 1
        score = (query[:, :n].view(E, n, H, Ch) * key[:, :n].view(E, n, H, Ch)).sum(dim=(1, 3))
        off = n
        for m in range(1, self.mmax + 1):
            n = self.lmax + 1 - m
            q = query[:, off:off + 2 * n].view(E, 2, n, H, Ch)
            k = key[:, off:off + 2 * n].view(E, 2, n, H, Ch)
            off += 2 * n
            ph = (m * phase).view(E, 1, H, 1)
            k_re = torch.cos(ph) * k[:, 0] - torch.sin(ph) * k[:, 1]
            k_im = torch.sin(ph) * k[:, 0] + torch.cos(ph) * k[:, 1]
            score = score + (q[:, 0] * k_re + q[:, 1] * k_im).sum(dim=(1, 3))
        temperature = self.t_min + (self.t_max - self.t_min) * torch.sigmoid(self.temperature_logit)
        return score * self.attention_scale * temperature + bias

    def forward(self, x, w, edge_index, cutoff, wigner, wigner_inv, radial_basis):
        N, E = x.shape[0], w.shape[0]
        if E == 0:  # no edge, no message (the sums below are empty)
            return x.new_zeros(N, x.shape[1], self.hidden)
        m_ij = torch.cat((x[edge_index[0]], x[edge_index[1]]), dim=-1)  # source | target channels
        m_ij = torch.bmm(wigner, m_ij)
        key = self.key_proj(m_ij[:, :, :self.C])
        query = self.query_proj(m_ij[:, :, self.C:])
        alpha = self._attention(query, key, radial_basis)
        w = w.view(E, self.num_components, 2 * self.C)[:, self.expand_index]
        m_ij = w * m_ij
        coefs = self.nonlinearity.scalar_act(self.linear_coefs(m_ij).squeeze(-1))
        glu = self.linear_glu(m_ij)
        up = self.linear_up(m_ij)
        gate, m_ij = up[:, :self.split[0]], up[:, self.split[0]:self.split[0] + self.split[1]]
        m_ij = m_ij + self.nonlinearity(m_ij, gate) + self.ece(m_ij, glu, coefs)
        m_ij = self.linear_down(m_ij)
        alpha = graph_softmax(alpha, edge_index[1], N, exp_rescale=cutoff)
        if cutoff is not None:
            alpha = alpha * cutoff
        m_ij = (alpha.view(E, 1, self.H, 1) * m_ij.view(E, m_ij.shape[1], self.H, self.c_head)).reshape(E, -1, self.hidden)
        m_ij = torch.bmm(wigner_inv, m_ij)
        return scatter_sum(m_ij, edge_index[1], N)


class ScaledSigmoid(torch.nn.Module):
    def forward(self, x):
        return torch.sigmoid(x) * SIGMOID_CST


class ScaledSiLU(torch.nn.Module):
    def forward(self, x):
        return torch.nn.functional.silu(x) * SILU_CST


def to_rows(x: torch.Tensor, irreps) -> torch.Tensor:
    """tace/models/layout.py:48-86 (LayoutTransform.forward): e3nn rows (per rank a [mul, 2l+1] block) -> [N, (L+1)^2, mul]."""
    n, start, out = x.shape[0], 0, []
    for mul, l in irreps:
        d = 2 * l + 1
        out.append(x[:, start:start + mul * d].reshape(n, mul, d))
        start += mul * d
    return torch.cat(out, dim=-1).transpose(-1, -2).contiguous()


def from_rows(x: torch.Tensor, irreps) -> torch.Tensor:
    """LayoutTransform.inverse."""
    x = x.transpose(-1, -2)
    n, start, out = x.shape[0], 0, []
    for _, l in irreps:
        d = 2 * l + 1
        out.append(x[:, :, start:start + d].reshape(n, -1))
        start += d
    return torch.cat(out, dim=-1)


def build_tece_interaction(base_cls):
    """The interaction of ``atomic_basis.type = uv_so2`` (tace/models/_e3nn/inter.py:440-519): the cgtp interaction with
    its scattered tensor product replaced by the edge convolution above, no message normalisation, the radial MLP
    emitting one weight per (order-reduced row, channel of source | target), and the cutoff handled inside the block."""
    from .model import MLP, Linear
    from .o3 import Irreps

    class TeceInteraction(base_cls):
        def __init__(self, *args, mmax=2, num_head=1, edge_ace_hidden=None, edge_wise_hidden=None, edge_act="sigmoid", **kw):
            super().__init__(*args, **kw)
            C = self.num_channel
            lmax = max(l for _, l in self.irreps_out)
            assert max(l for _, l in self.irreps_in) > 0, "the block needs input ranks above 0 (inter.py:458-461)"
            act = ScaledSigmoid() if edge_act == "sigmoid" else ScaledSiLU()
            hidden = edge_wise_hidden or C
            self.rejector = EdgeConvolution(mmax, lmax, C, num_head, edge_ace_hidden or C, hidden, self.num_radial_basis,
                                            self.gate_m0, act, act)
            self.conv_irreps = Irreps([(hidden, l) for _, l in self.irreps_out])
            self.linear_down = Linear(self.conv_irreps, self.nonlinearity.irreps_in, bias=True)
            dims = list(self.edge_info_dims)
            dims[-1] = self.rejector.weight_numel
            self.edge_info = MLP(dims, bias=self.mlp_bias, layer_norm=self.mlp_layer_norm)
            self.wigner = WignerD(mmax, lmax)

        def messages(self, x, edge_feats, edge_attrs, edge_index, edge_cutoff, edge_vector, radial_basis):
            wig, wig_inv = self.wigner.get_wigner(edge_vector)
            rows = to_rows(x, self.irreps_in)
            out = self.rejector(rows, self.edge_info(edge_feats), edge_index, edge_cutoff, wig, wig_inv, radial_basis)
            return from_rows(out, self.conv_irreps)

        def normalise(self, m, edge_feats, edge_index, edge_cutoff):
            return m  # scatter_norm = None (inter.py:466)

    return TeceInteraction
