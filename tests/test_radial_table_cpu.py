"""The tabulated radial weights (tace_b200.pack.radial_table) against the radial MLP they replace.

For models with the identity edge update the fp32 kernels read the path weights W(d) from a per-(path, channel) table
with cubic Hermite interpolation instead of running the radial MLP per edge.  Here the host restatement of that
interpolation is compared with the oracle's MLP (fp64) at random edge lengths: values and d/dd."""
import numpy as np
import pytest
import torch

from helpers import make_models
from tace_b200.pack import hermite_weights, pack_weights, radial_table


@pytest.mark.parametrize("radial", [{}, {"apply_cutoff": False, "bias": True, "hidden": [64, 64]}, {"hidden": [64]}])
def test_table_reproduces_the_radial_mlp(radial):
    cutoff = 5.0
    model, oracle, cfg = make_models(2, 32, [13, 29], cutoff, 20.0, torch.float64, radial=radial)
    rf = model.readout_fn
    packed = pack_weights(rf.plan, rf.state_dict(), 20.0)
    rep = oracle.readout_fn.representation
    rng = np.random.default_rng(0)
    d = np.concatenate([rng.uniform(0.6, cutoff, 400), [cutoff - 1e-9, cutoff * (1 - 1e-7), 0.75, 4.999]])
    dt = torch.tensor(d, dtype=torch.float64).unsqueeze(-1).requires_grad_(True)
    feats, env = rep.radial_basis(dt)
    for layer, inter in enumerate(rep.interactions):
        w = inter.edge_info(feats)  # the envelope (when applied after the MLP) stays outside the table
        table = radial_table(packed, layer, rf.plan, cutoff, 5, 1024)
        assert table.shape == (1025, w.shape[1], 2)
        val, der = hermite_weights(table, d, cutoff)
        ref_val = w.detach().numpy()
        cols = rng.choice(w.shape[1], 12, replace=False)
        ref_der = np.stack([torch.autograd.grad(w[:, c].sum(), dt, retain_graph=True)[0].reshape(-1).numpy() for c in cols], axis=1)
        scale = max(1.0, np.abs(ref_val).max())
        assert np.abs(val - ref_val).max() <= 2e-7 * scale, np.abs(val - ref_val).max()
        assert np.abs(der[:, cols] - ref_der).max() <= 2e-5 * max(1.0, np.abs(ref_der).max()), np.abs(der[:, cols] - ref_der).max()
