"""Data-parallel evaluation of a batch of independent structures on several GPUs.

Graphs of one batch are disjoint components (``batch`` / ``ptr`` in the reference's input
dictionary, ``tace/models/adapter.py:326-340``), so the batch shards across ranks with no
model-level communication: every rank evaluates its own sub-batch with replicated weights and
only the small per-structure results are gathered.  Structures are assigned with the
longest-processing-time heuristic on their estimated edge counts, the same balancing rule the
reference uses for its training sampler (``tace/dataset/sampler.py:17-145``).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Sequence

import numpy as np


def estimate_edges(structure, cutoff: float) -> float:
    """Atoms x mean neighbour count at the structure's number density."""
    n = len(structure["positions"])
    vol = abs(float(np.linalg.det(np.asarray(structure["cell"], dtype=np.float64))))
    if vol <= 0.0:
        return float(n * n)
    return n * (4.0 / 3.0) * np.pi * cutoff**3 * n / vol


def partition_lpt(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Indices per rank: heaviest first, each to the currently lightest rank; ties by rank id so
    every rank computes the identical assignment without communication."""
    order = sorted(range(len(costs)), key=lambda i: (-float(costs[i]), i))
    load = [0.0] * world_size
    parts: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        parts[r].append(i)
        load[r] += float(costs[i])
    return [sorted(p) for p in parts]


def evaluate_sharded(structures: Sequence, cutoff: float, evaluate: Callable[[List], Dict[str, np.ndarray]],
                     rank: int, world_size: int, gather: Callable[[object], List[object]]) -> Dict[str, List[np.ndarray]]:
    """Evaluate ``structures`` across ``world_size`` ranks.

    ``evaluate(list_of_structures)`` returns per-structure arrays: ``energy [n]``, ``stress [n,3,3]``
    and ``forces`` as a list of ``[atoms_i, 3]`` arrays (one per structure).  ``gather(obj)``
    returns the list of every rank's ``obj`` (``torch.distributed.all_gather_object`` in
    production).  Every rank returns the results in the original structure order.
    """
    parts = partition_lpt([estimate_edges(s, cutoff) for s in structures], world_size)
    mine = parts[rank]
    local = evaluate([structures[i] for i in mine]) if mine else {"energy": np.zeros(0), "stress": np.zeros((0, 3, 3)), "forces": []}
    gathered = gather({"index": mine, "result": local})
    n = len(structures)
    out = {"energy": [None] * n, "stress": [None] * n, "forces": [None] * n}
    for item in gathered:
        for j, i in enumerate(item["index"]):
            out["energy"][i] = item["result"]["energy"][j]
            out["stress"][i] = item["result"]["stress"][j]
            out["forces"][i] = item["result"]["forces"][j]
    if any(v is None for v in out["energy"]):
        raise RuntimeError("a rank did not report its share of the batch")
    return out
