"""Host-side parts of the Togalorn design that need no GPU: the configuration reader (looped layer ranges become
layer runs that share weights), the registry, synthetic weights under the checkpoint's names, and properties of the
float64 oracle itself (causality, the state-space recurrence cut into parts, the experts' limits)."""
import pytest
import torch

from oracle import togalorn_ref as R
from test_togalorn_engine_gpu import cfg_a, cfg_b, cfg_c, prompt


def test_loop_becomes_layer_runs_that_share_weights():
    from dli_b200 import models, togalorn

    cfg = cfg_a()
    assert models.family(cfg) == "togalorn" and models.supports_float32(cfg)
    spec = models.spec_from_config(cfg)
    assert [L.ckpt for L in spec.layers] == [0, 1, 2, 1, 2, 3] == [i for i, _ in R.layer_runs(cfg)]
    assert [L.weights_of for L in spec.layers] == [None, None, None, 1, 2, None]
    assert [L.reenter for L in spec.layers] == [None, 0, None, 1, None, None]
    assert all(L.parallel for L in spec.layers) and spec.layers[5].moe is None and spec.layers[0].moe.total_ff == 4 * 24 + 16
    assert spec.loop_passes == 2 and spec.norm_groups == 4
    nl = togalorn.spec_from_config(cfg_b())
    assert nl.loop_passes == 0 and all(L.reenter is None and L.weights_of is None for L in nl.layers)
    whole = togalorn.spec_from_config(cfg_c())
    assert [L.reenter for L in whole.layers] == [0, None, 1, None, 2, None]
    with pytest.raises(ValueError):
        togalorn.spec_from_config(dict(cfg, loop={"start": 2, "stop": 9, "times": 2}))
    with pytest.raises(ValueError):
        bad = cfg_b()
        bad["layers"][0]["type"] = "convolution"
        togalorn.spec_from_config(bad)


def test_synthetic_weights_have_the_checkpoint_names_and_shapes():
    from dli_b200 import togalorn

    cfg = cfg_a()
    spec = togalorn.spec_from_config(cfg)
    sd = togalorn.random_state_dict(spec, seed=3)
    assert sd["loop.in"].shape == (48, 96) and sd["loop.step"].shape == (2, 48)
    assert sd["l0.mix.in"].shape == (2 * 24 + 2 * 20 + 4, 48) and sd["l0.mix.conv"].shape == (24 + 40, 3)
    assert sd["l1.mix.dkv"].shape == (20 + 4, 48) and sd["l1.mix.uq"].shape == (3 * 12, 14)
    assert sd["l1.mlp.router"].shape == (6, 48) and "l1.mlp.e3.down" in sd and "l3.mlp.router" not in sd
    t = togalorn.model_tensors(spec, sd)
    assert sorted(t["layers"]) == [0, 1, 2, 5] and t["layers"][5]["o"] is sd["l3.mix.o"]
    R.forward(cfg, sd, prompt(5, cfg["vocab"], 0))   # the oracle finds every tensor it needs


def test_oracle_is_causal_and_its_recurrence_can_be_cut():
    from dli_b200 import togalorn

    cfg = cfg_a()
    sd = togalorn.random_state_dict(togalorn.spec_from_config(cfg), seed=1, std=0.15)
    toks = prompt(14, cfg["vocab"], 7)
    full, trace = R.forward(cfg, sd, toks)
    part, _ = R.forward(cfg, sd, toks[:9])
    assert torch.allclose(full[:9], part, atol=1e-10)
    assert trace.shape == (6, 14, 48)
    # experts: the gate is cut from above only, the up projection on both sides
    h = torch.tensor([[10.0, -10.0]], dtype=torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    y = R.expert(h, eye, eye, eye, 1.5)
    g0 = 1.5 * torch.sigmoid(torch.tensor(1.702 * 1.5, dtype=torch.float64)) * 2.5
    g1 = -10.0 * torch.sigmoid(torch.tensor(-17.02, dtype=torch.float64)) * (-0.5)
    assert torch.allclose(y, torch.stack((g0, g1))[None], atol=1e-12)
