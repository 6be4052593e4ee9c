"""Extended-XYZ and weight-file round trips (host code only)."""
import numpy as np
import torch

from tace_b200 import synth
from tace_b200.io import read_extxyz, read_weight_file, write_extxyz, write_weight_file
from tace_b200.models import create_model
from tace_b200.pack import pack_weights


def test_extxyz_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    frames = []
    for s in synth.random_crystals(3, seed=4, nmin=3, nmax=7, zmax=30):
        n = len(s["positions"])
        frames.append({"positions": s["positions"], "atomic_numbers": s["atomic_numbers"], "cell": s["cell"], "pbc": s["pbc"],
                       "energy": rng.normal(), "forces": rng.normal(size=(n, 3)), "stress": rng.normal(size=(3, 3))})
    path = tmp_path / "frames.xyz"
    write_extxyz(str(path), frames)
    back = read_extxyz(str(path))
    assert len(back) == 3
    for a, b in zip(frames, back):
        for key in ("positions", "cell", "forces", "stress"):
            assert np.array_equal(np.asarray(a[key], dtype=np.float64), b[key]), key
        assert np.array_equal(a["atomic_numbers"], b["atomic_numbers"])
        assert float(a["energy"]) == float(b["energy"])
        assert list(b["pbc"]) == [True, True, True]


def test_extxyz_reads_a_minimal_frame(tmp_path):
    path = tmp_path / "min.xyz"
    path.write_text('2\nLattice="4.0 0 0 0 4.0 0 0 0 4.0" Properties=species:S:1:pos:R:3 pbc="T T F"\nCu 0 0 0\nAl 1.5 1.5 1.5\n')
    (f,) = read_extxyz(str(path))
    assert list(f["atomic_numbers"]) == [29, 13] and list(f["pbc"]) == [True, True, False]
    assert np.allclose(f["cell"], 4.0 * np.eye(3)) and f["positions"].shape == (2, 3)


def test_weight_file_round_trip(tmp_path):
    torch.manual_seed(0)
    cfg = synth.model_config(2, 32, 4.0, [13, 29], 20.0)
    model = create_model(cfg)
    rf = model.readout_fn
    packed = pack_weights(rf.plan, rf.state_dict(), 20.0)
    names = sorted(packed)
    path = tmp_path / "weights.bin"
    write_weight_file(str(path), packed, names, dtype=np.float32)
    back = read_weight_file(str(path))
    assert list(back) == names
    for k in names:
        assert np.array_equal(back[k], np.asarray(packed[k], dtype=np.float32).reshape(-1)), k
