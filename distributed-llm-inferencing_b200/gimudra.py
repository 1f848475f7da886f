"""The Gimudra design: a pre-norm decoder whose layers are listed in config.json.  Every layer has softmax attention
inside blocks of positions (no rotation: a sinusoidal vector is added to the embedding, and a logarithmic distance
penalty r1 ln(1 + r2 (i - j)) is taken off the scores), with biased q / k / v projections, grouped key/value heads and
optionally ANOTHER layer's cached keys and values; then a feed-forward: gated SiLU with biases, or a mixture of
squared-ReLU experts without gates whose router chooses inside the best groups of experts and has outputs that pass
the input through.  Around them: RMS norms with a weight vector before each sublayer, a layer scale vector on each
sublayer's result, a token shift (the mixer's normed input is blended with the previous position's), and after every
layer a weighted average over the embedding output and all layers' results so far.  This module is the model
definition only — the configuration reader, the checkpoint's tensor names and synthetic weights; the step function,
caches and kernels are ragged_engine.RaggedEngine's.

config.json keys read here: architecture, vocab, width, embedding.scale, norm.eps, layers[] with type (attention),
mixer {heads, kv_heads, dim, vdim, scale, mask {size}, kv_from} and mlp: null, {kind: dense, ff} or {kind: moe,
expert {ff}, router {experts, identity, top, scale, groups {count, keep}}}.
Tensor names: embed, head, final.norm [width]; l<i>.norm1 / norm2 / ls1 / ls2 / shift [width], l<i>.dwa [i + 2];
l<i>.mix.{q, k, v} with biases <name>.b (no k / v in a layer that reads another layer's cache), l<i>.mix.{r1, r2} [heads],
l<i>.mix.o; dense l<i>.mlp.{gate, up, down} with biases; experts l<i>.mlp.e<k>.{up, down}, l<i>.mlp.router
[experts + identity, width], l<i>.mlp.correction.  A layer without shift, ls1 / ls2 or dwa tensors runs without that step.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .ragged_engine import HybridSpec, LayerSpec, MixerSpec, MoESpec

ARCHITECTURE = "Gimudra"
POS_BASE = 10000.0     # the sinusoidal position vector's frequencies are POS_BASE^(-2i/width)


def _mixer(i: int, L: dict, layers: list) -> MixerSpec:
    if L.get("type") != "attention":
        raise ValueError(f"layer {i}: unknown mixer type {L.get('type')!r}")
    m = L["mixer"]
    H, G = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
    if H % G:
        raise ValueError(f"layer {i}: {H} query heads over {G} key/value heads")
    src = m.get("kv_from")
    if src is not None:
        src = int(src)
        o = layers[src]["mixer"] if 0 <= src < i and layers[src].get("type") == "attention" else None
        if o is None or o.get("kv_from") is not None or int(o.get("kv_heads", o["heads"])) != G or \
                int(o["dim"]) != int(m["dim"]) or int(o["vdim"]) != int(m["vdim"]):
            raise ValueError(f"layer {i}: kv_from {src} is not an earlier attention layer with a cache of its own and the "
                             f"same key/value heads and sizes")
    return MixerSpec(kind="attention", heads=H, kv_heads=G, dim=int(m["dim"]), vdim=int(m["vdim"]), scale=float(m["scale"]),
                     chunk=int((m.get("mask") or {}).get("size", 0)), bias=True, dist_penalty=True, kv_from=src)


def _moe(i: int, mlp: dict) -> MoESpec:
    r = mlp["router"]
    n_out = int(r["experts"]) + int(r.get("identity", 0))
    g = r.get("groups") or {}
    count = int(g.get("count", 1))
    keep = int(g.get("keep", count))
    if count < 1 or n_out % count or not 1 <= keep <= count or keep * (n_out // count) < int(r["top"]):
        raise ValueError(f"layer {i}: {n_out} router outputs in {count} groups, {keep} kept, top {r['top']}")
    return MoESpec(experts=int(r["experts"]), identity=int(r.get("identity", 0)), top=int(r["top"]), ff=int(mlp["expert"]["ff"]),
                   limit=0.0, gated=False, groups=count, keep=keep, route_scale=float(r.get("scale", 1.0)), renorm=False)


def spec_from_config(cfg: dict) -> HybridSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    layers: List[LayerSpec] = []
    for i, L in enumerate(cfg["layers"]):
        mlp = L.get("mlp")
        kind = None if mlp is None else mlp.get("kind", "dense")
        if kind not in (None, "dense", "moe"):
            raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
        layers.append(LayerSpec(mixer=_mixer(i, L, cfg["layers"]), ff=int(mlp["ff"]) if kind == "dense" else 0,
                                moe=_moe(i, mlp) if kind == "moe" else None, pre_norm=True, token_shift=True, layer_scale=True,
                                depth_avg=True, ff_bias=kind == "dense"))
    return HybridSpec(arch="gimudra", vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                      taps=1, layers=layers, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), norm_groups=1,
                      pos_sinusoid=True, pos_base=POS_BASE)


def layer_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor], i: int) -> dict:
    """The checkpoint's tensors of layer i under the names the engine uses."""
    L, m = spec.layers[i], spec.layers[i].mixer
    p = f"l{i}."
    out = {"norm1": sd[p + "norm1"], "q": sd[p + "mix.q"], "q_b": sd[p + "mix.q.b"], "o": sd[p + "mix.o"],
           "r1": sd[p + "mix.r1"], "r2": sd[p + "mix.r2"]}
    if m.kv_from is None:
        out.update(k=sd[p + "mix.k"], k_b=sd[p + "mix.k.b"], v=sd[p + "mix.v"], v_b=sd[p + "mix.v.b"])
    for k in ("shift", "ls1", "ls2", "dwa"):
        if p + k in sd:
            out[k] = sd[p + k]
    if L.ff:
        out.update(norm2=sd[p + "norm2"], gate=sd[p + "mlp.gate"], up=sd[p + "mlp.up"], down=sd[p + "mlp.down"],
                   gate_b=sd[p + "mlp.gate.b"], up_b=sd[p + "mlp.up.b"], down_b=sd[p + "mlp.down.b"])
    if L.moe is not None:
        out.update(norm2=sd[p + "norm2"], router=sd[p + "mlp.router"], correction=sd[p + "mlp.correction"],
                   experts=[(None, sd[p + f"mlp.e{k}.up"], sd[p + f"mlp.e{k}.down"]) for k in range(L.moe.experts)])
    return out


def model_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor]) -> dict:
    return {"embed": sd["embed"], "head": sd["head"], "final_norm": sd["final.norm"],
            "layers": {i: layer_tensors(spec, sd, i) for i in range(spec.n_layers)}}


def random_state_dict(spec: HybridSpec, seed: int = 0, std: float = 0.05, device="cpu") -> Dict[str, torch.Tensor]:
    """Synthetic weights under the checkpoint's names (benchmarks and tests; there are no checkpoints offline)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = spec.width

    def n(*shape, s=std, mean=0.0):
        return (mean + s * torch.randn(tuple(shape), generator=g)).to(torch.bfloat16).to(device)

    def u(*shape, lo=0.0, hi=1.0):
        return (lo + (hi - lo) * torch.rand(tuple(shape), generator=g)).to(torch.bfloat16).to(device)

    sd = {"embed": n(spec.vocab, W, s=1.0 / max(spec.embed_scale, 1e-6)), "head": n(spec.vocab, W),
          "final.norm": n(W, mean=1.0, s=0.1)}
    for i, L in enumerate(spec.layers):
        m, p = L.mixer, f"l{i}."
        H, G, D, V = m.heads, m.kv_heads, m.dim, m.vdim
        sd[p + "norm1"] = n(W, mean=1.0, s=0.1)
        sd[p + "mix.q"], sd[p + "mix.q.b"] = n(H * D, W), n(H * D, s=0.3)
        if m.kv_from is None:
            sd[p + "mix.k"], sd[p + "mix.k.b"] = n(G * D, W), n(G * D, s=0.3)
            sd[p + "mix.v"], sd[p + "mix.v.b"] = n(G * V, W), n(G * V, s=0.3)
        sd[p + "mix.r1"], sd[p + "mix.r2"] = u(H, lo=0.0, hi=2.0), u(H, lo=0.05, hi=0.5)
        sd[p + "mix.o"] = n(W, H * V)
        if L.token_shift:
            sd[p + "shift"] = u(W, lo=0.0, hi=0.8)
        if L.layer_scale:
            sd[p + "ls1"] = u(W, lo=0.2, hi=1.4)
        if L.depth_avg:
            a = 0.3 * torch.randn(i + 2, generator=g)
            a[-1] += 1.0
            sd[p + "dwa"] = a.to(torch.bfloat16).to(device)
        if L.ff or L.moe is not None:
            sd[p + "norm2"] = n(W, mean=1.0, s=0.1)
            if L.layer_scale:
                sd[p + "ls2"] = u(W, lo=0.2, hi=1.4)
        if L.ff:
            sd[p + "mlp.gate"], sd[p + "mlp.up"], sd[p + "mlp.down"] = n(L.ff, W), n(L.ff, W), n(W, L.ff)
            sd[p + "mlp.gate.b"], sd[p + "mlp.up.b"], sd[p + "mlp.down.b"] = n(L.ff, s=0.2), n(L.ff, s=0.2), n(W, s=0.2)
        if L.moe is not None:
            e = L.moe
            for k in range(e.experts):
                sd[p + f"mlp.e{k}.up"], sd[p + f"mlp.e{k}.down"] = n(e.ff, W, s=2 * std), n(W, e.ff, s=2 * std)
            sd[p + "mlp.router"] = n(e.experts + e.identity, W, s=0.5)
            sd[p + "mlp.correction"] = n(e.experts + e.identity, mean=-1.0, s=0.5)
    return sd


def config_from_spec(spec: HybridSpec) -> dict:
    """The config.json of a spec (tests and benchmarks write model directories with it)."""
    layers = []
    for L in spec.layers:
        m = L.mixer
        mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
              "mask": {"size": m.chunk}}
        if m.kv_from is not None:
            mx["kv_from"] = m.kv_from
        if L.moe is not None:
            e = L.moe
            mlp = {"kind": "moe", "expert": {"ff": e.ff},
                   "router": {"experts": e.experts, "identity": e.identity, "top": e.top, "scale": e.route_scale,
                              "groups": {"count": e.groups, "keep": e.keep}}}
        else:
            mlp = {"kind": "dense", "ff": L.ff} if L.ff else None
        layers.append({"type": "attention", "mixer": mx, "mlp": mlp})
    return {"architecture": ARCHITECTURE, "vocab": spec.vocab, "width": spec.width, "embedding": {"scale": spec.embed_scale},
            "norm": {"eps": spec.eps}, "layers": layers}
