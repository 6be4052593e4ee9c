"""On-disk formats next to the hot path: extended-XYZ structures in and results out (the format of the
reference's example data, ``example/data/*.xyz``, which the reference reads through ase), and a flat binary
weight file for hosts that drive the C ABI without Python.

Weight file layout (little endian): ``b"TACEW001"``, int32 dtype code (0 = fp32, 1 = fp64), int32 count, then per
array: int32 name length, name bytes, int64 element count, the elements.  Names and element counts are the ones
``tace_weight_info`` reports, so a host loops over the file and calls ``tace_set_weight`` for every record.
"""

from __future__ import annotations

import re
import struct
from typing import Dict, Iterable, List, Optional, Sequence

import numpy as np

_SYMBOLS = ("X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr Nb Mo "
            "Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt Au Hg Tl "
            "Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr").split()
_Z = {s: z for z, s in enumerate(_SYMBOLS)}
_KV = re.compile(r'(\w+)=("([^"]*)"|(\S+))')


def _parse_properties(spec: str):
    fields = spec.split(":")
    return [(fields[i], fields[i + 1], int(fields[i + 2])) for i in range(0, len(fields), 3)]


def read_extxyz(path: str) -> List[Dict[str, np.ndarray]]:
    """Frames as dictionaries with ``positions [n,3]``, ``atomic_numbers [n]``, ``cell [3,3]`` (row vectors; zeros
    when absent), ``pbc [3]``, plus ``energy`` / ``forces`` / ``stress`` when the file carries them."""
    frames = []
    with open(path) as fh:
        lines = fh.read().splitlines()
    i = 0
    while i < len(lines):
        if not lines[i].strip():
            i += 1
            continue
        n = int(lines[i].split()[0])
        info = {m.group(1): (m.group(3) if m.group(3) is not None else m.group(4)) for m in _KV.finditer(lines[i + 1])}
        props = _parse_properties(info.get("Properties", "species:S:1:pos:R:3"))
        rows = [ln.split() for ln in lines[i + 2:i + 2 + n]]
        frame: Dict[str, np.ndarray] = {}
        col = 0
        for name, kind, width in props:
            block = [r[col:col + width] for r in rows]
            col += width
            if name == "species":
                frame["atomic_numbers"] = np.array([_Z[b[0]] if not b[0].isdigit() else int(b[0]) for b in block], dtype=np.int64)
            elif name == "Z":
                frame["atomic_numbers"] = np.array([int(b[0]) for b in block], dtype=np.int64)
            elif name == "pos":
                frame["positions"] = np.array(block, dtype=np.float64)
            elif kind == "R":
                frame[name] = np.array(block, dtype=np.float64)
        frame["cell"] = (np.array(info["Lattice"].split(), dtype=np.float64).reshape(3, 3) if "Lattice" in info
                         else np.zeros((3, 3)))
        pbc = info.get("pbc")
        frame["pbc"] = (np.array([t.upper().startswith("T") for t in pbc.split()]) if pbc
                        else np.array(["Lattice" in info] * 3))
        for key in ("energy", "free_energy"):
            if key in info:
                frame[key] = np.float64(info[key])
        for key in ("stress", "virial"):
            if key in info:
                frame[key] = np.array(info[key].split(), dtype=np.float64).reshape(3, 3)
        frames.append(frame)
        i += 2 + n
    return frames


def write_extxyz(path: str, frames: Iterable[Dict[str, np.ndarray]]) -> None:
    """Inverse of ``read_extxyz``; ``energy``, ``forces`` and ``stress`` entries are written when present."""
    with open(path, "w") as fh:
        for f in frames:
            n = len(f["positions"])
            props = "species:S:1:pos:R:3" + (":forces:R:3" if "forces" in f else "")
            head = [f'Lattice="{" ".join(repr(float(x)) for x in np.asarray(f["cell"]).reshape(-1))}"', f"Properties={props}"]
            if "energy" in f:
                head.append(f"energy={float(f['energy'])!r}")
            if "stress" in f:
                head.append(f'stress="{" ".join(repr(float(x)) for x in np.asarray(f["stress"]).reshape(-1))}"')
            head.append('pbc="' + " ".join("T" if b else "F" for b in np.asarray(f.get("pbc", [True] * 3))) + '"')
            fh.write(f"{n}\n{' '.join(head)}\n")
            for k in range(n):
                row = [_SYMBOLS[int(f["atomic_numbers"][k])]] + [repr(float(x)) for x in f["positions"][k]]
                if "forces" in f:
                    row += [repr(float(x)) for x in f["forces"][k]]
                fh.write(" ".join(row) + "\n")


_MAGIC = b"TACEW001"


def write_weight_file(path: str, packed: Dict[str, np.ndarray], names: Sequence[str], dtype=np.float32) -> None:
    """``packed``: the dictionary of ``tace_b200.pack.pack_weights``; ``names``: the arrays the library asks for
    (``tace_weight_info`` order)."""
    code = {np.dtype(np.float32): 0, np.dtype(np.float64): 1}[np.dtype(dtype)]
    with open(path, "wb") as fh:
        fh.write(_MAGIC + struct.pack("<ii", code, len(names)))
        for name in names:
            arr = np.ascontiguousarray(packed[name], dtype=dtype).reshape(-1)
            raw = name.encode()
            fh.write(struct.pack("<i", len(raw)) + raw + struct.pack("<q", arr.size) + arr.tobytes())


def read_weight_file(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as fh:
        blob = fh.read()
    if blob[:8] != _MAGIC:
        raise ValueError("not a tace_b200 weight file")
    code, count = struct.unpack_from("<ii", blob, 8)
    dtype = np.float32 if code == 0 else np.float64
    off, out = 16, {}
    for _ in range(count):
        (ln,) = struct.unpack_from("<i", blob, off); off += 4
        name = blob[off:off + ln].decode(); off += ln
        (numel,) = struct.unpack_from("<q", blob, off); off += 8
        nbytes = numel * np.dtype(dtype).itemsize
        out[name] = np.frombuffer(blob, dtype=dtype, count=numel, offset=off).copy(); off += nbytes
    return out
