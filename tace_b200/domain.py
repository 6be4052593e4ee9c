"""Spatial domain decomposition of ONE large periodic system over several GPUs.

The reference runs multi-GPU molecular dynamics through LAMMPS: every MPI rank owns the atoms of one
block of the box, carries copies ("ghosts") of the atoms within the cutoff of its block, and the model
asks LAMMPS to refresh ghost feature rows between interaction layers and to return gradients that
landed on ghost rows to their owners (``tace/models/lammps.py:82-142``; ``forward_exchange`` /
``reverse_exchange``).  This module provides the same contract without LAMMPS:

* ``choose_grid`` / ``DomainGrid`` - 3-D block decomposition of the (possibly triclinic) cell in
  fractional coordinates;
* ``build_halo_plan`` - who owns what, which periodic images every rank needs as ghosts, and the
  matching send lists, computed identically on every rank from the all-gathered fractional
  coordinates (no negotiation);
* ``HaloExchange`` - ``forward_exchange(src, dst, vec_len)`` and ``reverse_exchange(src, dst, vec_len)``
  with the LAMMPS semantics, over ``torch.distributed`` point-to-point messages (NCCL on GPUs, gloo on
  CPU for tests).  Data received from a peer lands in this rank's own memory before any kernel reads it.

Ghost order on every rank: by owning rank, then by periodic shift (fixed order), then by the owner's
local index.  A rank may be its own peer (fewer than three blocks along an axis): those ghosts are
local copies.
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

SHIFTS: Tuple[Tuple[int, int, int], ...] = tuple(itertools.product((-1, 0, 1), repeat=3))


def cell_heights(cell: np.ndarray) -> np.ndarray:
    """Perpendicular height of the cell along each lattice direction."""
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    inv = np.linalg.inv(cell)  # frac = pos @ inv
    return 1.0 / np.linalg.norm(inv, axis=0)


def choose_grid(world_size: int, heights: Sequence[float]) -> Tuple[int, int, int]:
    """Block counts (px, py, pz) with px*py*pz = world_size that minimise the surface of one block;
    ties go to the lexicographically smallest triple so every rank picks the same grid."""
    best, best_area = None, None
    h = [float(x) for x in heights]
    for px in range(1, world_size + 1):
        if world_size % px:
            continue
        for py in range(1, world_size // px + 1):
            if (world_size // px) % py:
                continue
            pz = world_size // (px * py)
            a, b, c = h[0] / px, h[1] / py, h[2] / pz
            area = a * b + b * c + a * c
            if best is None or area < best_area - 1e-12:
                best, best_area = (px, py, pz), area
    return best


@dataclass
class DomainGrid:
    """Blocks of the unit cube of fractional coordinates; rank = (ix * py + iy) * pz + iz."""

    grid: Tuple[int, int, int]

    @property
    def world_size(self) -> int:
        return self.grid[0] * self.grid[1] * self.grid[2]

    def coords(self, rank: int) -> Tuple[int, int, int]:
        px, py, pz = self.grid
        return rank // (py * pz), (rank // pz) % py, rank % pz

    def bounds(self, rank: int) -> Tuple[np.ndarray, np.ndarray]:
        c = np.array(self.coords(rank), dtype=np.float64)
        p = np.array(self.grid, dtype=np.float64)
        return c / p, (c + 1.0) / p

    def owner_of(self, frac: torch.Tensor) -> torch.Tensor:
        """Owning rank of wrapped fractional coordinates ``[n, 3]`` (values in [0, 1))."""
        p = torch.tensor(self.grid, dtype=frac.dtype, device=frac.device)
        idx = torch.floor(frac * p).to(torch.int64)
        for k in range(3):
            idx[:, k].clamp_(0, self.grid[k] - 1)
        return (idx[:, 0] * self.grid[1] + idx[:, 1]) * self.grid[2] + idx[:, 2]


@dataclass
class HaloPlan:
    rank: int
    world_size: int
    n_owned: int
    n_ghost: int
    # peers in ascending rank order (this rank included when it holds images of its own atoms)
    peers: List[int] = field(default_factory=list)
    send_index: Dict[int, torch.Tensor] = field(default_factory=dict)   # owned-local rows sent to each peer
    send_parts: Dict[int, List[Tuple[int, int]]] = field(default_factory=dict)  # (start, count) per periodic shift
    recv_slice: Dict[int, Tuple[int, int]] = field(default_factory=dict)  # (offset, count) in the ghost block
    ghost_shift: Optional[torch.Tensor] = None   # int64 [n_ghost, 3] periodic image of each ghost
    ghost_owner: Optional[torch.Tensor] = None   # int64 [n_ghost] owning rank
    ghost_owner_index: Optional[torch.Tensor] = None  # int64 [n_ghost] row on the owning rank


def _in_box(frac: torch.Tensor, lo: np.ndarray, hi: np.ndarray) -> torch.Tensor:
    lo_t = torch.tensor(lo, dtype=frac.dtype, device=frac.device)
    hi_t = torch.tensor(hi, dtype=frac.dtype, device=frac.device)
    return ((frac >= lo_t) & (frac < hi_t)).all(dim=1)


def _overlaps(lo_a, hi_a, lo_b, hi_b) -> bool:
    return bool(np.all(lo_a < hi_b) and np.all(lo_b < hi_a))


def build_halo_plan(grid: DomainGrid, rank: int, frac_by_rank: Sequence[torch.Tensor], ghost_width: Sequence[float]) -> HaloPlan:
    """``frac_by_rank[r]`` = wrapped fractional coordinates of the atoms rank ``r`` owns, in ``r``'s
    local order (identical tensors on every rank, e.g. from an all-gather).  ``ghost_width`` = halo
    thickness per axis in fractional units ((cutoff + skin) / cell height); it must be below 1 so that
    the 27 nearest periodic images suffice."""
    gw = np.asarray(ghost_width, dtype=np.float64)
    if np.any(gw >= 1.0):
        raise ValueError("halo wider than the periodic cell: use a larger cell or a smaller cutoff + skin")
    W = grid.world_size
    dev = frac_by_rank[rank].device
    plan = HaloPlan(rank=rank, world_size=W, n_owned=int(frac_by_rank[rank].shape[0]), n_ghost=0)
    my_lo, my_hi = grid.bounds(rank)
    ext_lo, ext_hi = my_lo - gw, my_hi + gw

    # receive side: images of rank r's atoms inside my extended block
    g_shift, g_owner, g_index = [], [], []
    offset = 0
    for r in range(W):
        r_lo, r_hi = grid.bounds(r)
        count = 0
        for s in SHIFTS:
            if r == rank and s == (0, 0, 0):
                continue
            sv = np.array(s, dtype=np.float64)
            if not _overlaps(r_lo + sv, r_hi + sv, ext_lo, ext_hi):
                continue
            fr = frac_by_rank[r]
            idx = torch.nonzero(_in_box(fr + torch.tensor(sv, dtype=fr.dtype, device=fr.device), ext_lo, ext_hi)).flatten()
            if idx.numel() == 0:
                continue
            g_index.append(idx)
            g_owner.append(torch.full_like(idx, r))
            g_shift.append(torch.tensor(s, dtype=torch.int64, device=dev).expand(idx.numel(), 3))
            count += int(idx.numel())
        if count:
            plan.peers.append(r)
            plan.recv_slice[r] = (offset, count)
            offset += count
    plan.n_ghost = offset
    if offset:
        plan.ghost_shift = torch.cat(g_shift).contiguous()
        plan.ghost_owner = torch.cat(g_owner)
        plan.ghost_owner_index = torch.cat(g_index)
    else:
        plan.ghost_shift = torch.zeros(0, 3, dtype=torch.int64, device=dev)
        plan.ghost_owner = torch.zeros(0, dtype=torch.int64, device=dev)
        plan.ghost_owner_index = torch.zeros(0, dtype=torch.int64, device=dev)

    # send side: my atoms whose image lies inside peer q's extended block (same rule, same order)
    mine = frac_by_rank[rank]
    for q in range(W):
        q_lo, q_hi = grid.bounds(q)
        q_ext_lo, q_ext_hi = q_lo - gw, q_hi + gw
        parts = []
        for s in SHIFTS:
            if q == rank and s == (0, 0, 0):
                continue
            sv = np.array(s, dtype=np.float64)
            if not _overlaps(my_lo + sv, my_hi + sv, q_ext_lo, q_ext_hi):
                continue
            idx = torch.nonzero(_in_box(mine + torch.tensor(sv, dtype=mine.dtype, device=dev), q_ext_lo, q_ext_hi)).flatten()
            if idx.numel():
                parts.append(idx)
        if parts:
            plan.send_index[q] = torch.cat(parts).contiguous()
            starts = np.cumsum([0] + [int(x.numel()) for x in parts])
            plan.send_parts[q] = [(int(starts[i]), int(parts[i].numel())) for i in range(len(parts))]
            if q not in plan.peers:  # a peer that only receives from this rank
                plan.peers.append(q)
                plan.recv_slice.setdefault(q, (plan.n_ghost, 0))
    plan.peers.sort()
    for q in plan.peers:
        plan.send_index.setdefault(q, torch.zeros(0, dtype=torch.int64, device=dev))
        plan.send_parts.setdefault(q, [])
        plan.recv_slice.setdefault(q, (plan.n_ghost, 0))
    return plan


class HaloExchange:
    """Ghost-row exchange with the semantics the reference expects from ``lmp_data``
    (tace/models/lammps.py:82-102):

    * ``forward_exchange(src, dst, vec_len)``: ``dst`` = ``src`` with every ghost row replaced by its
      owner's row;
    * ``reverse_exchange(src, dst, vec_len)``: ``dst`` = ``src`` with every ghost row's value added to
      its owner's row (ghost rows of ``dst`` are copied unchanged).

    Rows are ``[n_owned + n_ghost, vec_len]``.  Remote rows travel as point-to-point messages of the
    process group; sums into owner rows are applied peer by peer in ascending rank order.
    """

    # every operation below is enqueued on the current CUDA stream (NCCL send / receive are ordered against it by
    # torch.distributed), so a caller on that stream needs no host synchronisation around an exchange
    stream_ordered = True

    def __init__(self, plan: HaloPlan, group=None):
        self.plan = plan
        self.group = group
        self.calls = 0
        self.bytes_sent = 0
        self.timed = False      # record a CUDA event pair around every exchange (read with exchange_ms)
        self._events = []

    def _mark(self, tensor: torch.Tensor):
        if not (self.timed and tensor.is_cuda):
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(tensor.device))
        return ev

    def exchange_ms(self, reset: bool = True) -> float:
        """Device time spent between the start and the end of every exchange since the last reset (synchronises)."""
        total = 0.0
        for a, b in self._events:
            b.synchronize()
            total += a.elapsed_time(b)
        if reset:
            self._events = []
        return total

    # -- helpers -----------------------------------------------------------------------------------
    @staticmethod
    def _gather_rows(src2: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Packed copy of rows ``idx``: the library's gather kernel on the GPU, torch on the CPU (tests)."""
        if not src2.is_cuda or src2.element_size() not in (4, 8) or not src2.is_contiguous():
            return src2.index_select(0, idx).contiguous()
        from . import lib as _lib

        out = torch.empty(idx.numel(), src2.shape[1], dtype=src2.dtype, device=src2.device)
        with torch.cuda.device(src2.device):
            _lib.check(_lib.load().tace_rows_gather(src2.data_ptr(), idx.data_ptr(), idx.numel(), src2.shape[1], src2.element_size(),
                                                    out.data_ptr(), torch.cuda.current_stream(src2.device).cuda_stream),
                       "tace_rows_gather")
        return out

    def _add_rows(self, dst2: torch.Tensor, q: int, rows: torch.Tensor) -> None:
        """dst2[send_index[q]] += rows, one launch per periodic shift (indices are distinct within a shift)."""
        idx = self.plan.send_index[q]
        if not dst2.is_cuda or dst2.dtype not in (torch.float32, torch.float64) or not dst2.is_contiguous():
            dst2[: self.plan.n_owned].index_add_(0, idx, rows)
            return
        from . import lib as _lib

        lib = _lib.load()
        rows = rows.contiguous()
        width = dst2.shape[1]
        with torch.cuda.device(dst2.device):
            stream = torch.cuda.current_stream(dst2.device).cuda_stream
            for start, count in self.plan.send_parts[q]:
                _lib.check(lib.tace_rows_scatter_add(rows.data_ptr() + start * width * rows.element_size(),
                                                     idx.data_ptr() + start * 8, count, width, rows.element_size(),
                                                     dst2.data_ptr(), stream), "tace_rows_scatter_add")

    def _p2p(self, sends: List[Tuple[torch.Tensor, int]], recvs: List[Tuple[torch.Tensor, int]]) -> None:
        import torch.distributed as dist

        ops = []
        for t, q in sends:
            ops.append(dist.P2POp(dist.isend, t, q, group=self.group))
            self.bytes_sent += t.numel() * t.element_size()
        for t, q in recvs:
            ops.append(dist.P2POp(dist.irecv, t, q, group=self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def forward_exchange(self, src: torch.Tensor, dst: torch.Tensor, vec_len: int = 0) -> None:
        p = self.plan
        n = p.n_owned
        t_start = self._mark(src)
        src2, dst2 = src.reshape(src.shape[0], -1), dst.reshape(dst.shape[0], -1)
        if dst2.data_ptr() != src2.data_ptr():
            dst2[:n].copy_(src2[:n])
        sends, recvs = [], []
        for q in p.peers:
            off, cnt = p.recv_slice[q]
            sidx = p.send_index[q]
            if q == p.rank:
                if cnt:
                    dst2[n + off:n + off + cnt].copy_(self._gather_rows(src2, sidx))
                continue
            if sidx.numel():
                sends.append((self._gather_rows(src2, sidx), q))
            if cnt:
                recvs.append((dst2[n + off:n + off + cnt], q))
        self._p2p(sends, recvs)
        self.calls += 1
        if t_start is not None:
            self._events.append((t_start, self._mark(src)))

    def reverse_exchange(self, src: torch.Tensor, dst: torch.Tensor, vec_len: int = 0) -> None:
        p = self.plan
        n = p.n_owned
        t_start = self._mark(src)
        src2, dst2 = src.reshape(src.shape[0], -1), dst.reshape(dst.shape[0], -1)
        if dst2.data_ptr() != src2.data_ptr():
            dst2.copy_(src2)
        sends, recvs, landed = [], [], {}
        for q in p.peers:
            off, cnt = p.recv_slice[q]
            sidx = p.send_index[q]
            if q == p.rank:
                if cnt:
                    landed[q] = src2[n + off:n + off + cnt].clone()
                continue
            if cnt:
                sends.append((src2[n + off:n + off + cnt].contiguous(), q))
            if sidx.numel():
                buf = torch.empty(sidx.numel(), src2.shape[1], dtype=src2.dtype, device=src2.device)
                landed[q] = buf
                recvs.append((buf, q))
        self._p2p(sends, recvs)
        for q in p.peers:
            if q in landed:
                self._add_rows(dst2, q, landed[q])
        self.calls += 1
        if t_start is not None:
            self._events.append((t_start, self._mark(src)))


class Domain:
    """Owned + ghost atoms of one rank, rebuilt from the global state whenever atoms may have moved
    more than half the skin.

    ``partition`` takes every rank's owned atoms (positions, velocities, species, persistent ids),
    all-gathers them, wraps positions into the cell, reassigns owners by block and builds the halo
    plan.  Between two calls the ownership and the ghost lists stay fixed and positions are not
    wrapped; ``refresh_ghost_positions`` sends current owner positions to the ghost copies and adds
    the image translation.
    """

    def __init__(self, cell: np.ndarray, cutoff: float, skin: float, rank: int, world_size: int, device: torch.device,
                 grid: Optional[Tuple[int, int, int]] = None, group=None, high_priority_halo: bool = False):
        self.cell_np = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.heights = cell_heights(self.cell_np)
        self.cutoff, self.skin = float(cutoff), float(skin)
        self.rank, self.world_size, self.device, self.group = rank, world_size, torch.device(device), group
        # high_priority_halo: halo messages travel on a group of their own whose NCCL streams have high priority, so that an
        # exchange that runs beside the evaluation (TensorModel.set_exchange_overlap) does not queue behind the
        # evaluation's thread blocks.
        self.halo_group = group
        if high_priority_halo and world_size > 1 and self.device.type == "cuda":
            import torch.distributed as dist

            if dist.get_backend(group) == "nccl":
                ranks = None if group is None else dist.get_process_group_ranks(group)
                options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
                self.halo_group = dist.new_group(ranks=ranks, backend="nccl", pg_options=options)  # collective: every rank builds its Domain
        self.grid = DomainGrid(tuple(grid) if grid is not None else choose_grid(world_size, self.heights))
        if self.grid.world_size != world_size:
            raise ValueError(f"grid {self.grid.grid} does not match world size {world_size}")
        self.cell = torch.tensor(self.cell_np, dtype=torch.float64, device=self.device)
        self.inv_cell = torch.linalg.inv(self.cell)
        self.ghost_width = (self.cutoff + self.skin) / self.heights
        self.plan: Optional[HaloPlan] = None
        self.exchange: Optional[HaloExchange] = None
        self.reference_positions: Optional[torch.Tensor] = None
        self.n_partitions = 0
        self.time_exchanges = False  # CUDA-event timing of every exchange (halo_stats)
        self._halo_ms, self._halo_bytes = 0.0, 0

    def _all_gather_rows(self, x: torch.Tensor) -> List[torch.Tensor]:
        """Every rank's rows of ``x`` ([n_r, ...], n_r differs per rank)."""
        if self.world_size == 1:
            return [x]
        import torch.distributed as dist

        n = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
        counts = [torch.zeros_like(n) for _ in range(self.world_size)]
        dist.all_gather(counts, n, group=self.group)
        counts = [int(c.item()) for c in counts]
        m = max(counts) if counts else 0
        pad = torch.zeros((m,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        pad[: x.shape[0]] = x
        out = [torch.empty_like(pad) for _ in range(self.world_size)]
        dist.all_gather(out, pad, group=self.group)
        return [o[:c] for o, c in zip(out, counts)]

    def partition(self, state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """``state``: this rank's per-atom tensors, at least ``positions`` fp64 [n,3]; every other entry
        ([n] or [n,k]) moves with its atom.  Returns the new owned state (positions wrapped)."""
        gathered = {k: torch.cat(self._all_gather_rows(v.contiguous())) for k, v in state.items()}
        pos = gathered["positions"].to(torch.float64)
        frac = pos @ self.inv_cell
        frac = frac - torch.floor(frac)
        frac = torch.where(frac >= 1.0, torch.zeros_like(frac), frac)  # -1e-17 wraps to exactly 1.0
        owner = self.grid.owner_of(frac)
        # stable order by persistent id when present, so the local order does not depend on history
        order_key = gathered["ids"] if "ids" in gathered else torch.arange(pos.shape[0], device=pos.device)
        frac_by_rank, rows_by_rank = [], []
        for r in range(self.world_size):
            rows = torch.nonzero(owner == r).flatten()
            rows = rows[torch.argsort(order_key[rows], stable=True)]
            rows_by_rank.append(rows)
            frac_by_rank.append(frac[rows])
        mine = rows_by_rank[self.rank]
        new_state = {k: v[mine].clone() for k, v in gathered.items()}
        new_state["positions"] = (frac[mine] @ self.cell).contiguous()
        self.plan = build_halo_plan(self.grid, self.rank, frac_by_rank, self.ghost_width)
        if self.exchange is not None:  # keep the totals of the exchange object this partition retires
            self._halo_ms += self.exchange.exchange_ms()
            self._halo_bytes += self.exchange.bytes_sent
        self.exchange = HaloExchange(self.plan, self.halo_group)
        self.exchange.timed = self.time_exchanges
        self.ghost_offset = (self.plan.ghost_shift.to(torch.float64) @ self.cell).contiguous()
        self.reference_positions = new_state["positions"].clone()
        self.n_partitions += 1
        return new_state

    def halo_stats(self, reset: bool = False):
        """(device milliseconds inside exchanges, bytes sent) since construction or the last reset; the time is only
        collected while ``time_exchanges`` is set."""
        ms = self._halo_ms + (self.exchange.exchange_ms(reset=reset) if self.exchange is not None else 0.0)
        nbytes = self._halo_bytes + (self.exchange.bytes_sent if self.exchange is not None else 0)
        if reset:
            self._halo_ms, self._halo_bytes = 0.0, 0
            if self.exchange is not None:
                self.exchange.bytes_sent = 0
        return ms, nbytes

    def set_time_exchanges(self, enable: bool) -> None:
        self.time_exchanges = bool(enable)
        if self.exchange is not None:
            self.exchange.timed = self.time_exchanges

    @property
    def n_owned(self) -> int:
        return self.plan.n_owned

    @property
    def n_ghost(self) -> int:
        return self.plan.n_ghost

    def local_positions(self, owned_positions: torch.Tensor) -> torch.Tensor:
        """[n_owned + n_ghost, 3] fp64: owned rows followed by the translated ghost copies."""
        n, g = self.plan.n_owned, self.plan.n_ghost
        full = torch.empty(n + g, 3, dtype=torch.float64, device=owned_positions.device)
        full[:n] = owned_positions
        self.exchange.forward_exchange(full, full, 3)
        full[n:] += self.ghost_offset
        return full

    def local_rows(self, owned: torch.Tensor) -> torch.Tensor:
        """Any per-atom tensor extended with its ghost copies (species, masses, ...)."""
        n, g = self.plan.n_owned, self.plan.n_ghost
        full = torch.empty((n + g,) + tuple(owned.shape[1:]), dtype=owned.dtype, device=owned.device)
        full[:n] = owned
        self.exchange.forward_exchange(full, full, 0)
        return full

    def displacement(self, owned_positions: torch.Tensor, velocities: torch.Tensor):
        """(largest distance any atom of any rank has moved since the last partition, largest speed of any atom), read
        back with one collective and one host synchronisation."""
        d2 = ((owned_positions - self.reference_positions) ** 2).sum(dim=1)
        v2 = (velocities ** 2).sum(dim=1)
        zero = torch.zeros((), dtype=torch.float64, device=owned_positions.device)
        both = torch.stack([d2.max() if d2.numel() else zero, v2.max() if v2.numel() else zero])
        if self.world_size > 1:
            import torch.distributed as dist

            dist.all_reduce(both, op=dist.ReduceOp.MAX, group=self.group)
        moved2, fastest2 = both.tolist()
        return moved2 ** 0.5, fastest2 ** 0.5

    def needs_partition(self, owned_positions: torch.Tensor) -> bool:
        """True on every rank as soon as an atom of any rank moved more than half the skin since the
        last partition."""
        d2 = ((owned_positions - self.reference_positions) ** 2).sum(dim=1)
        worst = d2.max() if d2.numel() else torch.zeros((), dtype=torch.float64, device=owned_positions.device)
        if self.world_size > 1:
            import torch.distributed as dist

            worst = worst.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX, group=self.group)
        return bool(worst.item() > (0.5 * self.skin) ** 2)
