"""Constructor / configuration checks that need no GPU: which reference options are accepted, which are refused."""
import pytest
import torch

from tace_b200 import synth
from tace_b200.models import check_model_config, create_model

# the `model.config` section of the reference's example training file (example/train/tace.yaml), values only
EXAMPLE_MODEL_SECTION = {
    "cutoff": 6.0, "max_neighbors": None, "target_property": ["energy", "forces", "stress"], "embedding_property": [],
    "node_embedding": {"type": "linear"}, "edge_embedding": {"type": "identity"}, "edge_update": {"type": "element2"},
    "mmax": 3, "Lmax": 2, "lmax": 3, "mag_Lmax": 1, "num_layers": 3, "num_channel": 48, "parity": False,
    "radial_basis": {"radial_basis": "j0", "num_radial_basis": 8, "distance_transform": None, "cutoff_fn": "c2poly",
                     "polynomial_cutoff": 5, "order": 0, "trainable": False, "apply_cutoff": False, "hidden": [64, 64],
                     "bias": True, "use_dydynamic_cutoff": False},
    "resnet": {"type": "BB", "linear_type": "aware", "use_first_resnet": False},
    "layer_norm": {"pre_norm_type": None, "final_norm_type": None, "use_first_pre_norm": False},
    "atomic_basis": {"type": "cgtp", "l1l2": None, "scatter_norm": "avg_num_neighbors", "nonlinear": "sigmoid_gate",
                     "gate_m0": False, "scalar_act": None, "tensor_act": None},
    "product_basis": {"type": "cgtp", "l1l2": None, "correlation": 2, "return_components": None, "num_expert": None,
                      "nonlinear": None, "use_shared_expert": False, "agnostic": False},
    "readout_emlp": {"bias": False, "hidden": [16], "use_alllayer": False, "use_uie": False},
    "scale_shift": {"enable": True, "scale_type": "rms_forces", "shift_type": None, "all_atoms": False},
}


def test_example_training_configuration_is_accepted_and_builds():
    cfg = dict(EXAMPLE_MODEL_SECTION, statistics=synth.statistics([1, 6, 8], 30.0))
    torch.manual_seed(0)
    model = create_model(cfg)
    rf = model.readout_fn
    assert rf.plan.C == 48 and rf.plan.Cp == 64 and rf.plan.L == 3 and rf.plan.Lnode == 2
    assert rf.plan.mlp_layers == 2 and rf.plan.mlp_bias and not rf.plan.apply_cutoff and rf.plan.element2 and not rf.plan.gate_m0
    sd = model.state_dict()
    assert sd["readout_fn.representation.interactions.0.edge_info.mlp.0.weight"].shape == (8 + 2 * 48, 64)
    assert sd["readout_fn.representation.edge_updates.2.target_embedding.weight"].shape == (3 * 48,)
    # edge features wider than the radial basis: linear, LayerNorm, SiLU, linear, LayerNorm, SiLU, linear
    assert sd["readout_fn.representation.interactions.0.edge_info.mlp.1.weight"].shape == (64,)
    assert sd["readout_fn.representation.interactions.0.edge_info.mlp.3.weight"].shape == (64, 64)
    assert sd["readout_fn.representation.interactions.0.edge_info.mlp.4.bias"].shape == (64,)
    assert "readout_fn.representation.interactions.0.edge_info.mlp.6.bias" in sd
    assert "readout_fn.representation.interactions.0.edge_info.mlp.2.weight" not in sd
    assert "readout_fn.representation.interactions.0.edge_info.mlp.9.weight" not in sd


@pytest.mark.parametrize("override,needle", [
    ({"Lmax": 3, "lmax": 2}, "Lmax"),
    ({"parity": True}, "parity"),
    ({"product_basis": {"correlation": 4}}, "correlation"),
    ({"radial_basis": {"hidden": [32, 32]}}, "hidden"),
    ({"radial_basis": {"cutoff_fn": "cosine"}}, "cutoff_fn"),
    ({"atomic_basis": {"type": "uv_so2"}}, "atomic_basis.type"),
    ({"short_range": {"zbl": {"enable": True}}}, "ZBL"),
    ({"num_channel": 300}, "num_channel"),
])
def test_unsupported_options_are_refused_loudly(override, needle):
    cfg = synth.model_config(2, 32, 4.0, [29], 20.0)
    for k, v in override.items():
        if isinstance(v, dict) and isinstance(cfg.get(k), dict):
            cfg[k] = {**cfg[k], **v}
        else:
            cfg[k] = v
    with pytest.raises(NotImplementedError) as err:
        check_model_config({k: v for k, v in cfg.items()})
    assert needle in str(err.value)


def test_tece_configuration_builds_with_reference_parameter_names():
    """atomic_basis.type = [cgtp, uv_so2]: accepted, parameters of the edge block named and shaped like the reference's
    (tace/models/_e3nn/archive/oam_2026_07_05.py:612-697), and the matching oracle loads the same state_dict."""
    from oracle.model import build_oracle

    cfg = synth.model_config(3, 32, 5.0, [1, 8], 20.0, gate_m0=False, radial={"apply_cutoff": False},
                             tece={"num_head": 4, "edge_ace_hidden": 8, "mmax": 2})
    torch.manual_seed(0)
    model = create_model(cfg)
    sd = model.state_dict()
    pre = "readout_fn.representation.interactions.1."
    n, C, Ca = 4, 32, 8
    assert sd[pre + "rejector.linear_up.m0_rlinear.weight"].shape == ((2 * n + n) * Ca, n * 2 * C)  # gates for m = 1, 2 + features
    assert sd[pre + "rejector.linear_up.ms_clinear.1.fc.weight"].shape == (n * Ca, (n - 2) * 2 * C)
    assert sd[pre + "rejector.linear_coefs.m0_rlinear.weight"].shape == (7 * n * Ca, n * 2 * C)       # 7 cluster paths for mmax = 2
    assert sd[pre + "rejector.linear_down.ms_clinear.0.fc.weight"].shape == ((n - 1) * C, n * Ca)
    assert sd[pre + "rejector.key_proj.m0_rlinear.bias"].shape == (n * C,)
    assert sd[pre + "rejector.radial_proj.weight"].shape == (8, 8) and sd[pre + "rejector.temperature_logit"].shape == (4,)
    assert sd[pre + "edge_info.mlp.6.weight"].shape == (64, (4 + 3 + 2) * 2 * C)                      # one weight per (row, source | target channel)
    assert sd[pre + "linear_down.weight"].numel() == (3 + 1) * C * C + 3 * C * C                      # one C-block per rank in
    build_oracle(cfg, sd, torch.float64)  # raises on any missing or mis-shaped name
    for bad in ({"Lmax": 2}, {"mmax": 3}):
        with pytest.raises(NotImplementedError):
            check_model_config({**cfg, **bad})


def test_checkpoint_written_from_the_reference_models_own_state_dict_loads(tmp_path):
    """A ``.pt`` dictionary in the reference's export format (tace/lightning/lit_model.py:664-677) whose state_dict is the
    reference model's own (``tests/golden/ref_model_tece_L2_C32.npz`` was written by running the reference's source files:
    it carries the reference's parameter names and the persistent Wigner buffers this implementation has no use for)."""
    import json
    import os

    import numpy as np

    from tace_b200.interface.ase_calculator import load_tace

    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_model_tece_L2_C32.npz"))
    cfg = json.loads(str(z["cfg_json"]))
    for s in cfg["statistics"]:
        for k, v in list(s.items()):
            if isinstance(v, dict):
                s[k] = {int(a): b for a, b in v.items()}
    sd = {k[3:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("sd:")}
    extra = [k for k in sd if "so2_angular_basis" in k]
    assert extra, "the reference's state_dict holds persistent Wigner buffers"
    statistics = cfg.pop("statistics")
    target = cfg.pop("target_property")
    path = str(tmp_path / "reference_export.pt")
    torch.save({"state_dict": sd, "cfg": cfg, "target_property": target, "embedding_property": [], "statistics": statistics}, path)
    model = load_tace(path, "cpu", dtype="float64")
    own = model.state_dict()
    assert set(own) == set(sd) - set(extra)
    for k, v in own.items():
        assert torch.equal(v, sd[k].to(v.dtype)), k
