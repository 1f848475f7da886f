"""Host-side parts of the Fubepel design that need no GPU: the configuration reader (which layer owns a cache and
which reads another's), the registry, synthetic weights under the checkpoint's names, and properties of the float64
oracle itself (causality, the window with kept first positions, the sink, the rotation's pairing)."""
import math

import pytest
import torch

from oracle import fubepel_ref as R
from test_fubepel_engine_gpu import cfg_a, cfg_b, cfg_d, prompt


def test_configuration_reader_and_registry():
    from dli_b200 import fubepel, models

    cfg = cfg_a()
    assert models.family(cfg) == "fubepel" and models.supports_float32(cfg)
    spec = models.spec_from_config(cfg)
    assert [L.mixer.kind for L in spec.layers] == ["latent_attention", "delta", "attention", "latent_attention", "delta",
                                                   "latent_attention"]
    assert [L.mixer.kv_from for L in spec.layers] == [None, None, None, 0, None, None]
    assert all(L.post_only and not L.parallel for L in spec.layers) and spec.taps == 1 and spec.norm_groups == 1
    assert [L.side_off for L in spec.layers] == [0, 6, 12, 18, 24, 30] and spec.side_width == 36
    a = spec.layers[2].mixer
    assert (a.window, a.keep_first, a.qk_norm, a.rot_dims, a.sink) == (9, 3, True, 0, False)
    l0 = spec.layers[0].mixer
    assert l0.rot_halves and l0.sink and l0.q_rank == 0 and not l0.out_gate
    assert spec.layers[1].mixer.scale == 8 ** -0.5 and spec.layers[4].ff == 0 and spec.layers[2].ff_limit == 0.7
    assert fubepel.spec_from_config(cfg_b()).side_width == 0
    assert fubepel.config_from_spec(spec)["layers"][3]["mixer"]["kv_from"] == 0
    assert fubepel.spec_from_config(fubepel.config_from_spec(spec)) == spec
    for bad_src in (3, 1, 7):     # itself, a layer of another kind, a layer that does not exist
        bad = cfg_a()
        bad["layers"][3]["mixer"]["kv_from"] = bad_src
        with pytest.raises(ValueError):
            fubepel.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][3]["mixer"]["kv_rank"] = 24   # another latent size than the cache it reads
    with pytest.raises(ValueError):
        fubepel.spec_from_config(bad)
    bad = cfg_b()
    bad["layers"][5]["mixer"]["kv_from"] = 3    # a layer that itself reads another layer's cache
    with pytest.raises(ValueError):
        fubepel.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][1]["type"] = "convolution"
    with pytest.raises(ValueError):
        fubepel.spec_from_config(bad)


def test_synthetic_weights_have_the_checkpoint_names_and_shapes():
    from dli_b200 import fubepel

    cfg = cfg_a()
    spec = fubepel.spec_from_config(cfg)
    sd = fubepel.random_state_dict(spec, seed=3)
    assert sd["side.embed"].shape == (97, 36) and sd["final.norm"].shape == (48,)
    assert sd["l0.mix.q"].shape == (3 * 12, 48) and sd["l0.mix.dkv"].shape == (24, 48) and sd["l0.mix.sink"].shape == (3,)
    assert "l3.mix.dkv" not in sd and "l3.mix.dkv.norm" not in sd and sd["l3.mix.uk"].shape == (12, 20)
    assert sd["l1.mix.q"].shape == (16, 48) and sd["l1.mix.v.conv"].shape == (24, 3) and sd["l1.mix.norm"].shape == (6,)
    assert sd["l2.mix.k"].shape == (16, 48) and sd["l2.mix.v"].shape == (20, 48) and "l2.mix.sink" not in sd
    assert "l4.mlp.gate" not in sd and sd["l4.side.proj"].shape == (48, 6)
    t = fubepel.model_tensors(spec, sd)
    assert sorted(t["layers"]) == list(range(6)) and t["layers"][1]["conv"].shape == (16 + 16 + 24, 3)
    assert "dkv" not in t["layers"][3] and t["side_embed"] is sd["side.embed"]
    R.forward(cfg, sd, prompt(5, cfg["vocab"], 0))   # the oracle finds every tensor it needs


def test_oracle_masks_sink_and_rotation():
    vis = R.visible(12, 4, 2)
    assert vis[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9] and vis[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert R.visible(5).tolist() == torch.ones(5, 5).tril().bool().tolist()
    # the sink takes weight but adds nothing
    s = torch.zeros(1, 1, dtype=torch.float64)
    v = torch.ones(1, 3, dtype=torch.float64)
    out = R.softmax_attend(s, v, torch.ones(1, 1, dtype=torch.bool), sink=math.log(3.0))
    assert torch.allclose(out, torch.full((1, 3), 0.25, dtype=torch.float64))
    # entry i turns with entry i + dims/2; what lies beyond `dims` passes; scores depend on the distance only
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]], dtype=torch.float64)
    y = R.rotate_half_pairs(x, torch.tensor([1]), 100.0, 4)
    a0, a1 = 1.0, 100.0 ** -0.5
    assert torch.allclose(y[0], torch.tensor([math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                              3 * math.cos(a0) + math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0],
                                             dtype=torch.float64))
    q, k = torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64)
    d1 = R.rotate_half_pairs(q, torch.tensor([7]), 50.0, 8) @ R.rotate_half_pairs(k, torch.tensor([4]), 50.0, 8).T
    d2 = R.rotate_half_pairs(q, torch.tensor([103]), 50.0, 8) @ R.rotate_half_pairs(k, torch.tensor([100]), 50.0, 8).T
    assert torch.allclose(d1, d2, atol=1e-9)


def test_oracle_is_causal():
    from dli_b200 import fubepel

    for make in (cfg_a, cfg_d):
        cfg = make()
        sd = fubepel.random_state_dict(fubepel.spec_from_config(cfg), seed=1, std=0.15)
        toks = prompt(21, cfg["vocab"], 7)
        layers = []
        full = R.forward(cfg, sd, toks, layers)
        assert torch.allclose(full[:13], R.forward(cfg, sd, toks[:13]), atol=1e-10)
        assert len(layers) == len(cfg["layers"]) and layers[0].shape == (21, cfg["width"])
