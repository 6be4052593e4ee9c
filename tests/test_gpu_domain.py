"""Domain-decomposed evaluation and MD on the GPU.

One rank (the block is the whole cell, ghosts are periodic images of the rank's own atoms) must give the
oracle's energy and forces; two ranks on two GPUs (skipped on a single-GPU machine) must give the same
forces as one; the MD support kernels are checked against torch; NVE dynamics must conserve energy and
momentum."""
import os
import socket

import numpy as np
import pytest
import torch

from helpers import make_models, oracle_batch
from tace_b200 import lib as _lib
from tace_b200 import synth
from tace_b200.md import ACCEL, DomainMD, masses_for, maxwell_boltzmann

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _system(seed=7):
    return synth.fcc_supercell(3, 3.61, 0.05, seed=seed, species=(13, 29), fractions=(0.3, 0.7))


@pytest.mark.parametrize("num_layers", [1, 2])
def test_single_rank_domain_matches_oracle(num_layers):
    s = _system()
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, num_layers=num_layers, targets=("energy", "forces"))
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64))
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], skin=0.4, device=DEV)
    assert md.domain.n_ghost > 0
    got = md.gather()
    assert abs(md.potential() - float(ref["energy"][0])) / len(s["positions"]) < 1e-8
    assert np.abs(got["forces"] - ref["forces"].detach().numpy()).max() < 1e-7
    assert model.device_error() == 0


@pytest.mark.parametrize("dtype,num_layers", [(torch.float64, 2), (torch.float64, 3), (torch.float32, 2)])
def test_exchange_on_its_own_stream_gives_the_serial_result(dtype, num_layers):
    """The ghost exchange may run on a second stream while the layer works on the atoms without ghost neighbours
    (tace_set_exchange_stream).  Every atom's message sum keeps its order, so both schedules must give the same energy
    bit for bit; the gradient rows of an atom with several ghost copies add the arrivals before the rank's own sum
    instead of after it, so forces agree to rounding.  Both must give the oracle's numbers."""
    s = synth.fcc_supercell(4, 3.61, 0.05, seed=21, species=(13, 29), fractions=(0.4, 0.6))
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, dtype, num_layers=num_layers, targets=("energy", "forces"))
    ref = oracle(oracle_batch([s], [13, 29], 4.0, dtype))
    model = model.to(DEV)
    got, launches = {}, {}
    for overlap in (False, True):
        model.set_exchange_overlap(overlap)
        before = model.launch_count()
        md = DomainMD(model, s["cell"], s["positions"], s["atomic_numbers"], skin=0.4, device=DEV)
        assert md.domain.n_ghost > 0
        got[overlap] = (md.potential(), md.gather()["forces"])
        launches[overlap] = model.launch_count() - before
        assert model.device_error() == 0
    # the split passes are extra launches: a schedule that silently fell back to the serial exchange would not add any
    assert launches[True] > launches[False]
    tol_e, tol_f = (1e-8, 1e-7) if dtype == torch.float64 else (1e-5, 1e-4)
    n = len(s["positions"])
    for overlap in (False, True):
        assert abs(got[overlap][0] - float(ref["energy"][0])) / n < tol_e
        assert np.abs(got[overlap][1] - ref["forces"].detach().double().numpy()).max() < tol_f
    assert got[True][0] == got[False][0]
    assert np.abs(got[True][1] - got[False][1]).max() < (1e-12 if dtype == torch.float64 else 1e-5)


def test_single_rank_domain_with_the_tece_edge_block():
    """The same check for a model whose second interaction is the TECE edge block: ghost features through the exchange,
    gradients of ghost sources back through it, the edge-frame gradient inside the forces."""
    s = _system(seed=8)
    model, oracle, cfg = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"),
                                     radial={"apply_cutoff": False}, tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64))
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], skin=0.4, device=DEV)
    assert md.domain.n_ghost > 0
    got = md.gather()
    assert abs(md.potential() - float(ref["energy"][0])) / len(s["positions"]) < 1e-8
    assert np.abs(got["forces"] - ref["forces"].detach().numpy()).max() < 1e-7
    assert model.device_error() == 0
    # with an exchange stream the edge block still waits for its ghost rows before it starts: same numbers
    model.set_exchange_overlap(True)
    md2 = DomainMD(model, s["cell"], s["positions"], s["atomic_numbers"], skin=0.4, device=DEV)
    assert md2.potential() == md.potential()
    assert np.abs(md2.gather()["forces"] - got["forces"]).max() < 1e-12
    assert model.device_error() == 0


def test_md_support_kernels_match_torch():
    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(0)
    n = 1000
    pos = torch.randn(n, 3, generator=g, dtype=torch.float64).to(DEV)
    vel = torch.randn(n, 3, generator=g, dtype=torch.float64).to(DEV)
    mass = (torch.rand(n, generator=g, dtype=torch.float64) + 0.5).to(DEV)
    inv_mass = 1.0 / mass
    stream = torch.cuda.current_stream(DEV).cuda_stream
    for dtype in (torch.float32, torch.float64):
        f = torch.randn(n, 3, generator=g, dtype=torch.float64).to(DEV).to(dtype)
        p2, v2 = pos.clone(), vel.clone()
        _lib.check(lib.tace_md_kick_drift(p2.data_ptr(), v2.data_ptr(), f.data_ptr(), _lib.dtype_code(dtype), inv_mass.data_ptr(), n,
                                          0.25, 2.0, stream), "kick_drift")
        v_ref = vel + 0.25 * f.to(torch.float64) * inv_mass[:, None]
        assert torch.allclose(v2, v_ref, rtol=0, atol=1e-14)
        assert torch.allclose(p2, pos + 2.0 * v_ref, rtol=0, atol=1e-13)
        v3 = vel.clone()
        _lib.check(lib.tace_md_kick_drift(None, v3.data_ptr(), f.data_ptr(), _lib.dtype_code(dtype), inv_mass.data_ptr(), n, 0.25, 0.0,
                                          stream), "kick")
        assert torch.equal(v3, v2)
    scratch = torch.empty(1024, dtype=torch.float64, device=DEV)
    out = torch.empty(1, dtype=torch.float64, device=DEV)
    _lib.check(lib.tace_md_kinetic_energy(vel.data_ptr(), mass.data_ptr(), n, scratch.data_ptr(), out.data_ptr(), stream), "ke")
    assert abs(out.item() - float((0.5 * mass[:, None] * vel * vel).sum())) < 1e-9
    # edge vectors
    E = 5000
    ei = torch.randint(0, n, (2, E), generator=g).to(DEV)
    for dtype in (torch.float32, torch.float64):
        vec = torch.empty(E, 3, dtype=dtype, device=DEV)
        _lib.check(lib.tace_edge_vectors(pos.data_ptr(), ei.data_ptr(), E, vec.data_ptr(), _lib.dtype_code(dtype), stream), "vec")
        assert torch.equal(vec, (pos[ei[1]] - pos[ei[0]]).to(dtype))
    # row gather / scatter-add (distinct indices)
    for dtype in (torch.float32, torch.float64, torch.int64, torch.int32):
        src = (torch.randn(n, 7, generator=g, dtype=torch.float64) * 100).to(DEV).to(dtype).contiguous()
        idx = torch.randperm(n, generator=g)[:300].to(DEV)
        dst = torch.empty(300, 7, dtype=dtype, device=DEV)
        _lib.check(lib.tace_rows_gather(src.data_ptr(), idx.data_ptr(), 300, 7, src.element_size(), dst.data_ptr(), stream), "gather")
        assert torch.equal(dst, src[idx])
        if dtype.is_floating_point:
            acc = src.clone()
            _lib.check(lib.tace_rows_scatter_add(dst.data_ptr(), idx.data_ptr(), 300, 7, src.element_size(), acc.data_ptr(), stream),
                       "scatter_add")
            ref = src.clone()
            ref[idx] += dst
            assert torch.equal(acc, ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_filtered_edge_list_matches_a_boolean_mask(dtype):
    """tace_edges_within + tace_edges_scan + tace_edges_compact against torch: the kept edges in list order and their
    vectors (the fp64 difference rounded once), bit for bit."""
    import ctypes

    lib = _lib.load()
    g = torch.Generator(device="cpu").manual_seed(5)
    n, E = 500, 20000
    pos = (torch.rand(n, 3, generator=g, dtype=torch.float64) * 12.0).to(DEV)
    ei = torch.randint(0, n, (2, E), generator=g, dtype=torch.int64).to(DEV)
    cutoff = 5.0
    stream = torch.cuda.current_stream(DEV).cuda_stream
    keep = torch.empty(E, dtype=torch.uint8, device=DEV)
    position = torch.empty(E, dtype=torch.int32, device=DEV)
    total = torch.empty(1, dtype=torch.int64, device=DEV)
    nbytes = ctypes.c_size_t()
    _lib.check(lib.tace_edges_scan_workspace_bytes(E, ctypes.byref(nbytes)), "ws")
    scratch = torch.empty(int(nbytes.value), dtype=torch.uint8, device=DEV)
    _lib.check(lib.tace_edges_within(pos.data_ptr(), ei.data_ptr(), E, cutoff, keep.data_ptr(), stream), "within")
    _lib.check(lib.tace_edges_scan(keep.data_ptr(), E, position.data_ptr(), total.data_ptr(), scratch.data_ptr(), scratch.numel(), stream),
               "scan")
    n_kept = int(total.item())
    mask = keep.view(torch.bool)
    assert 0 < n_kept < E and n_kept == int(mask.sum())
    out_index = torch.empty(2, n_kept, dtype=torch.int64, device=DEV)
    out_vec = torch.empty(n_kept, 3, dtype=dtype, device=DEV)
    _lib.check(lib.tace_edges_compact(pos.data_ptr(), ei.data_ptr(), E, keep.data_ptr(), position.data_ptr(), n_kept,
                                      out_index.data_ptr(), out_vec.data_ptr(), _lib.dtype_code(dtype), stream), "compact")
    ref_index = ei[:, mask]
    assert torch.equal(out_index, ref_index)
    assert torch.equal(out_vec, (pos[ref_index[1]] - pos[ref_index[0]]).to(dtype))
    # an empty list is legal
    _lib.check(lib.tace_edges_scan(None, 0, None, total.data_ptr(), None, 0, stream), "scan of nothing")
    assert int(total.item()) == 0


def test_nve_conserves_energy_and_momentum():
    s = _system(seed=9)
    model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"))
    masses = masses_for(s["atomic_numbers"])
    vel = maxwell_boltzmann(masses, 300.0, seed=1)
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], velocities=vel, dt=1.0, skin=0.3, device=DEV)
    assert abs(md.temperature() - 300.0) < 1e-6
    e0 = md.potential() + md.kinetic_energy()
    scale = abs(md.kinetic_energy())
    md.step(25)
    e1 = md.potential() + md.kinetic_energy()
    # random weights give a rough energy surface; velocity Verlet with dt = 1 fs still keeps the total
    # energy to a small fraction of the kinetic energy
    assert abs(e1 - e0) < 2e-3 * scale, (e0, e1, scale)
    out = md.gather()
    p = (masses[:, None] * out["velocities"]).sum(0)
    assert np.abs(p).max() < 1e-9 * np.abs(masses[:, None] * out["velocities"]).sum()
    assert model.device_error() == 0


def test_repartition_keeps_the_trajectory():
    """Same dynamics with a tiny skin (re-partition nearly every step) and a large one."""
    s = _system(seed=11)
    masses = masses_for(s["atomic_numbers"])
    vel = maxwell_boltzmann(masses, 600.0, seed=2)
    outs = []
    for skin in (0.02, 1.0):
        model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"))
        md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], velocities=vel, dt=1.0, skin=skin, device=DEV)
        md.step(10)
        outs.append((md.gather(), md.domain.n_partitions))
    assert outs[0][1] > outs[1][1] >= 1
    a, b = outs[0][0], outs[1][0]
    cell = s["cell"]
    d = a["positions"] - b["positions"]
    d -= np.round(d @ np.linalg.inv(cell)) @ cell  # positions are wrapped at every partition
    assert np.abs(d).max() < 1e-9
    assert np.abs(a["forces"] - b["forces"]).max() < 1e-8


def _two_rank_worker(rank, world, port, ret, overlap=False):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        s = _system(seed=13)
        model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"))
        model.set_exchange_overlap(overlap)  # exchange on its own stream, NCCL messages on a high-priority group
        masses = masses_for(s["atomic_numbers"])
        vel = maxwell_boltzmann(masses, 300.0, seed=3)
        md = DomainMD(model.to(dev), s["cell"], s["positions"], s["atomic_numbers"], velocities=vel, skin=0.4, rank=rank,
                      world_size=world, device=dev)
        e = md.potential()
        md.step(3)
        out = md.gather()
        ret[rank] = {"energy": e, "forces": out["forces"], "positions": out["positions"], "owned": md.domain.n_owned,
                     "err": model.device_error()}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_two_ranks_match_one(overlap):
    import torch.multiprocessing as mp

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, port, ret, overlap)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    s = _system(seed=13)
    model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"))
    masses = masses_for(s["atomic_numbers"])
    vel = maxwell_boltzmann(masses, 300.0, seed=3)
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], velocities=vel, skin=0.4, device=DEV)
    e = md.potential()
    md.step(3)
    one = md.gather()
    for r in range(2):
        assert ret[r]["err"] == 0 and 0 < ret[r]["owned"] < len(s["positions"])
        assert abs(ret[r]["energy"] - e) < 1e-8 * len(s["positions"])
        assert np.abs(ret[r]["forces"] - one["forces"]).max() < 1e-8
        assert np.abs(ret[r]["positions"] - one["positions"]).max() < 1e-10


def test_langevin_kernel_statistics_and_determinism():
    lib = _lib.load()
    n = 200000
    g = torch.Generator().manual_seed(0)
    mass = (torch.rand(n, generator=g, dtype=torch.float64) * 50 + 1).to(DEV)
    inv_mass = 1.0 / mass
    ids = torch.randperm(n, generator=g).to(DEV)
    kt = 0.7
    stream = torch.cuda.current_stream(DEV).cuda_stream
    v = torch.ones(n, 3, dtype=torch.float64, device=DEV)
    # c1 = 0: the old velocities are forgotten, every component is N(0, kT / m)
    _lib.check(lib.tace_md_langevin(v.data_ptr(), inv_mass.data_ptr(), ids.data_ptr(), n, 0.0, kt, 7, 3, stream), "langevin")
    z = v * torch.sqrt(mass / kt)[:, None]
    assert abs(z.mean().item()) < 0.01 and abs(z.var().item() - 1.0) < 0.01
    assert abs((z ** 4).mean().item() - 3.0) < 0.1  # Gaussian fourth moment
    assert abs((z[:, 0] * z[:, 1]).mean().item()) < 0.01 and abs((z[:, 1] * z[:, 2]).mean().item()) < 0.01
    # the noise of an atom depends on its id, not on its row: a permuted call gives the permuted result
    perm = torch.randperm(n, generator=g).to(DEV)
    v2 = torch.ones(n, 3, dtype=torch.float64, device=DEV)
    inv_mass_p, ids_p = inv_mass[perm].contiguous(), ids[perm].contiguous()
    _lib.check(lib.tace_md_langevin(v2.data_ptr(), inv_mass_p.data_ptr(), ids_p.data_ptr(), n, 0.0, kt, 7, 3, stream), "langevin")
    assert torch.equal(v2, v[perm])
    v3 = torch.ones(n, 3, dtype=torch.float64, device=DEV)
    _lib.check(lib.tace_md_langevin(v3.data_ptr(), inv_mass.data_ptr(), ids.data_ptr(), n, 0.0, kt, 7, 4, stream), "langevin")
    assert not torch.equal(v3, v)  # another step, other numbers
    # c1 = 1: no friction, nothing changes
    v4 = v.clone()
    _lib.check(lib.tace_md_langevin(v4.data_ptr(), inv_mass.data_ptr(), ids.data_ptr(), n, 1.0, kt, 7, 5, stream), "langevin")
    assert torch.equal(v4, v)


def test_langevin_dynamics_reaches_the_target_temperature():
    s = synth.fcc_supercell(4, 3.61, 0.02, seed=15, species=(13, 29), fractions=(0.3, 0.7))
    model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, targets=("energy", "forces"))
    md = DomainMD(model.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], dt=1.0, skin=0.3, device=DEV,
                  temperature=300.0, friction=0.05, seed=5)
    lines = []
    md.step(150, log_every=10, log=lines.append)
    assert len(lines) == 15 and lines[-1]["step"] == 150 and abs(lines[-1]["total"] - lines[-1]["potential"] - lines[-1]["kinetic"]) < 1e-9
    temps = [ln["temperature"] for ln in lines[-8:]]
    # 256 atoms: the instantaneous temperature fluctuates by about 5 %; the mean of the last samples is near the target
    assert 240.0 < sum(temps) / len(temps) < 360.0, temps
    assert model.device_error() == 0


def test_rank_without_owned_atoms_answers_its_exchanges():
    """A block of vacuum in a decomposition (a slab in a long box): the rank owns nothing but holds ghost rows.  Its
    evaluation must return zeros and still call the exchange once per exchanged layer and direction - its neighbours'
    point-to-point messages have to meet a partner."""
    model, _, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, num_layers=3, targets=("energy", "forces"))
    model = model.to(DEV)
    model._set_lammps_mliap(True)
    calls = []

    class Exchange:
        def forward_exchange(self, src, dst, vec_len):
            calls.append(("forward", tuple(src.shape)))
            dst.copy_(src)

        def reverse_exchange(self, src, dst, vec_len):
            calls.append(("reverse", tuple(src.shape)))
            dst.copy_(src)

    g = 7
    out = model({"species": torch.zeros(g, dtype=torch.int32, device=DEV), "edge_index": torch.empty(2, 0, dtype=torch.int64, device=DEV),
                 "edge_vector": torch.empty(0, 3, dtype=torch.float64, device=DEV), "natoms": (0, g), "lmp_data": Exchange()})
    torch.cuda.synchronize()
    assert [c[0] for c in calls] == ["forward", "forward", "reverse", "reverse"]  # layers 1 and 2 read exchanged features
    assert all(c[1][0] == g for c in calls)
    assert out["forces"].shape == (g, 3) and float(out["forces"].abs().max()) == 0.0
    assert out["node_energy"].numel() == 0 and float(out["energy"].abs().max()) == 0.0
    assert model.device_error() == 0
    # the next ordinary evaluation on the same handle is unaffected
    s = _system()
    model2, oracle, _ = make_models(2, 32, [13, 29], 4.0, 20.0, torch.float64, num_layers=3, targets=("energy", "forces"))
    md = DomainMD(model2.to(DEV), s["cell"], s["positions"], s["atomic_numbers"], skin=0.4, device=DEV)
    ref = oracle(oracle_batch([s], [13, 29], 4.0, torch.float64))
    assert abs(md.potential() - float(ref["energy"][0])) / len(s["positions"]) < 1e-8


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_one_process_two_devices(dtype):
    """Models on cuda:0 and then cuda:1 in one process: kernel attributes (opt-in shared memory) are set per device."""
    from helpers import check_parity, to_device

    s = synth.fcc_supercell(2, 3.61, 0.05, seed=0)
    for dev in (torch.device("cuda:0"), torch.device("cuda:1")):
        model, oracle, _ = make_models(3, 128, [29], 4.0, 20.0, dtype)
        data = oracle_batch([s], [29], 4.0, dtype)
        out = model(to_device(data, dev))
        check_parity(out, oracle(data), data["ptr"], dtype, f"L3 C128 on {dev}")
        assert model.device_error() == 0
