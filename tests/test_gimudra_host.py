"""Host-side parts of the Gimudra design that need no GPU: the configuration reader (which layer owns a cache and which
reads another's, router groups), the registry, synthetic weights under the checkpoint's names, and properties of the
float64 oracle itself (causality, blocks, the distance penalty, the token shift, the router's groups)."""
import math

import pytest
import torch

from oracle import gimudra_ref as R
from test_gimudra_engine_gpu import cfg_a, cfg_b, cfg_c, prompt


def test_configuration_reader_and_registry():
    from dli_b200 import gimudra, models

    cfg = cfg_a()
    assert models.family(cfg) == "gimudra" and models.supports_float32(cfg)
    spec = models.spec_from_config(cfg)
    assert [L.mixer.kind for L in spec.layers] == ["attention"] * 6
    assert [L.mixer.kv_from for L in spec.layers] == [None, None, 1, 0, None, 4]
    assert all(L.pre_norm and L.token_shift and L.layer_scale and L.depth_avg and not L.post_only and not L.parallel
               for L in spec.layers)
    assert spec.taps == 1 and spec.norm_groups == 1 and spec.pos_sinusoid and spec.pos_base == 10000.0 and spec.embed_scale == 3.0
    a = spec.layers[1].mixer
    assert (a.chunk, a.window, a.bias, a.dist_penalty, a.qk_norm, a.rot_dims, a.sink) == (7, 0, True, True, False, 0, False)
    assert [L.ff for L in spec.layers] == [40, 0, 0, 0, 0, 24] and [L.ff_bias for L in spec.layers] == [True] + [False] * 4 + [True]
    e = spec.layers[1].moe
    assert (e.experts, e.identity, e.top, e.ff, e.groups, e.keep, e.route_scale, e.renorm, e.gated, e.shared_ff) == \
           (6, 2, 2, 12, 4, 2, 1.5, False, False, 0)
    assert spec.layers[3].moe is None and spec.layers[4].moe.groups == 1
    assert gimudra.config_from_spec(spec)["layers"][2]["mixer"]["kv_from"] == 1
    assert gimudra.spec_from_config(gimudra.config_from_spec(spec)) == spec
    for bad_src in (2, 3, 9):                 # a layer that itself reads another's cache, itself, a layer that does not exist
        bad = cfg_a()
        bad["layers"][3]["mixer"]["kv_from"] = bad_src
        with pytest.raises(ValueError):
            gimudra.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][3]["mixer"]["vdim"] = 12     # another value size than the cache it reads
    with pytest.raises(ValueError):
        gimudra.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][1]["mlp"]["router"]["groups"] = {"count": 3, "keep": 1}   # 8 outputs do not form 3 equal groups
    with pytest.raises(ValueError):
        gimudra.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][1]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}   # 2 candidates for the 2 chosen: fine
    gimudra.spec_from_config(bad)
    bad["layers"][1]["mlp"]["router"]["top"] = 3                            # 2 candidates for 3
    with pytest.raises(ValueError):
        gimudra.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][1]["type"] = "convolution"
    with pytest.raises(ValueError):
        gimudra.spec_from_config(bad)
    bad = cfg_a()
    bad["layers"][0]["mlp"]["kind"] = "maxout"
    with pytest.raises(ValueError):
        gimudra.spec_from_config(bad)


def test_synthetic_weights_have_the_checkpoint_names_and_shapes():
    from dli_b200 import gimudra

    cfg = cfg_a()
    spec = gimudra.spec_from_config(cfg)
    sd = gimudra.random_state_dict(spec, seed=3)
    assert sd["embed"].shape == (97, 48) and sd["final.norm"].shape == (48,)
    assert sd["l0.mix.q"].shape == (32, 48) and sd["l0.mix.k.b"].shape == (16,) and sd["l0.mix.v"].shape == (20, 48)
    assert sd["l0.mix.r1"].shape == (4,) and sd["l0.mlp.gate.b"].shape == (40,) and sd["l0.mlp.down.b"].shape == (48,)
    assert "l2.mix.k" not in sd and "l2.mix.v.b" not in sd and sd["l2.mix.q.b"].shape == (36,)
    assert sd["l1.mlp.router"].shape == (8, 48) and sd["l1.mlp.correction"].shape == (8,) and sd["l1.mlp.e5.up"].shape == (12, 48)
    assert "l1.mlp.e6.up" not in sd and "l3.norm2" not in sd and "l3.ls2" not in sd and sd["l3.ls1"].shape == (48,)
    assert [sd[f"l{i}.dwa"].shape[0] for i in range(6)] == [2, 3, 4, 5, 6, 7] and sd["l4.shift"].shape == (48,)
    t = gimudra.model_tensors(spec, sd)
    assert sorted(t["layers"]) == list(range(6)) and "k" not in t["layers"][5] and len(t["layers"][1]["experts"]) == 6
    R.forward(cfg, sd, prompt(5, cfg["vocab"], 0))   # the oracle finds every tensor it needs


def test_oracle_blocks_penalty_shift_and_positions():
    vis = R.block_visible(12, 5)
    assert vis[9].nonzero().flatten().tolist() == [5, 6, 7, 8, 9] and vis[10].nonzero().flatten().tolist() == [10]
    assert vis[4].nonzero().flatten().tolist() == [0, 1, 2, 3, 4]
    assert R.block_visible(5, 0).tolist() == torch.ones(5, 5).tril().bool().tolist()
    pen = R.distance_penalty(6, torch.tensor([2.0, 0.0]), torch.tensor([0.5, 3.0]))
    assert abs(float(pen[0, 5, 1]) - 2.0 * math.log(1 + 0.5 * 4)) < 1e-12 and float(pen[0, 3, 3]) == 0.0
    assert float(pen[1].abs().max()) == 0.0
    h = torch.arange(12, dtype=torch.float64).reshape(4, 3)
    s = torch.tensor([0.0, 1.0, 0.5], dtype=torch.float64)
    out = R.token_shift(h, s)
    assert out[0].tolist() == [0.0, 0.0, 1.0] and out[2].tolist() == [6.0, 4.0, 6.5]
    assert R.token_shift(h[2:], s, before=h[1]).tolist() == out[2:].tolist()
    p = R.sinusoid(torch.tensor([0, 3]), 6)
    assert p[0].tolist() == [0.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    f1 = 10000.0 ** (-2.0 / 6)
    assert torch.allclose(p[1], torch.tensor([math.sin(3), math.cos(3), math.sin(3 * f1), math.cos(3 * f1), math.sin(3 * f1 * f1),
                                              math.cos(3 * f1 * f1)], dtype=torch.float64))


def test_oracle_router_groups():
    """Two groups of three, one kept: the kept group is the one that holds the single best choice score, and the choice
    stays inside it although the other group's members all beat its second best."""
    w = torch.eye(6, dtype=torch.float64)
    h = torch.tensor([[2.0, -5.0, -5.0, 1.5, 1.4, 1.3]], dtype=torch.float64)
    c = torch.full((6,), -3.0, dtype=torch.float64)
    r = {"experts": 5, "identity": 1, "top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}}
    idx, wt = R.route(h, w, c, r)
    assert idx[0].tolist() == [0, 1]
    s = torch.softmax(h, dim=-1)
    assert torch.allclose(wt[0], 2.0 * s[0, [0, 1]])
    idx2, _ = R.route(h, w, c, dict(r, groups={"count": 2, "keep": 2}))
    assert idx2[0].tolist() == [0, 3]
    c2 = c.clone()
    c2[0] = -9.0                               # the correction moves the choice, not the weights
    idx3, wt3 = R.route(h, w, c2, r)
    assert idx3[0].tolist() == [3, 4] and torch.allclose(wt3[0], 2.0 * s[0, [3, 4]])


def test_oracle_is_causal():
    from dli_b200 import gimudra

    for make in (cfg_a, cfg_b, cfg_c):
        cfg = make()
        sd = gimudra.random_state_dict(gimudra.spec_from_config(cfg), seed=1, std=0.15)
        toks = prompt(21, cfg["vocab"], 7)
        layers = []
        full = R.forward(cfg, sd, toks, layers)
        assert torch.allclose(full[:13], R.forward(cfg, sd, toks[:13]), atol=1e-10)
        assert len(layers) == len(cfg["layers"]) and layers[0].shape == (21, cfg["width"])
