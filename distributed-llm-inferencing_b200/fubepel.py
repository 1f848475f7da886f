"""The Fubepel design: a decoder whose layers are listed in config.json, each with one of three token mixers — a
gated delta-rule recurrence, softmax attention without positions under a sliding window that keeps the first tokens,
or latent attention with a rotated shared key part and a softmax sink (optionally reading ANOTHER layer's cache) —
then a clamped gated feed-forward and a per-layer token input.  Sublayers read the residual stream itself and are
RMS-normed on their output only: x += norm(sublayer(x)).  This module is the model definition only — the
configuration reader, the checkpoint's tensor names and synthetic weights; the step function, caches and kernels are
ragged_engine.RaggedEngine's.

config.json keys read here: architecture, vocab, width, embedding.scale, norm.eps, token_side.dim, layers[] with type,
mlp (null or {kind: dense, ff, limit}) and mixer: delta {heads, kv_heads, dim, vdim, conv}, attention {heads,
kv_heads, dim, vdim, scale, mask {size, keep_first}}, latent_attention {heads, dim, rot_dim, vdim, kv_rank, scale,
rot {base, dims}, kv_from}.
Tensor names: embed, head, final.norm [width], side.embed [vocab, layers * token_side.dim], l<i>.norm1 / norm2 [width],
l<i>.side.{gate, proj, norm}, l<i>.mlp.{gate, up, down}; delta l<i>.mix.{q, q.conv, k, k.conv, v, v.conv, b, a, A_log,
dt_bias, norm, g, o}; attention l<i>.mix.{q, k, v, o}; latent attention l<i>.mix.{q, dkv, dkv.norm, uk, uv, sink, o}
(no dkv / dkv.norm in a layer that reads another layer's cache).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .ragged_engine import HybridSpec, LayerSpec, MixerSpec

ARCHITECTURE = "Fubepel"
FF_ALPHA = 1.702       # g * sigmoid(alpha * g) in the feed-forward
UNIT_EPS = 1e-6        # under the root when the delta rule's queries and keys are made unit vectors


def _mixer(i: int, L: dict, layers: list) -> MixerSpec:
    m = L["mixer"]
    kind = L["type"]
    if kind == "delta":
        return MixerSpec(kind="delta", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                         vdim=int(m["vdim"]), conv_taps=int(m.get("conv", 1)), scale=float(m["dim"]) ** -0.5,
                         unit_eps=UNIT_EPS)
    if kind == "attention":
        mask = m.get("mask") or {}
        return MixerSpec(kind="attention", heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])),
                         dim=int(m["dim"]), vdim=int(m["vdim"]), scale=float(m["scale"]), window=int(mask.get("size", 0)),
                         keep_first=int(mask.get("keep_first", 0)), qk_norm=True)
    if kind == "latent_attention":
        rot = m.get("rot") or {}
        rd = int(m.get("rot_dim", 0))
        if rd and int(rot.get("dims", rd)) != rd:
            raise ValueError(f"layer {i}: rot.dims {rot.get('dims')} differs from rot_dim {rd}")
        src = m.get("kv_from")
        if src is not None:
            src = int(src)
            o = layers[src]["mixer"] if 0 <= src < i and layers[src]["type"] == "latent_attention" else None
            if o is None or o.get("kv_from") is not None or int(o["kv_rank"]) != int(m["kv_rank"]) or int(o.get("rot_dim", 0)) != rd:
                raise ValueError(f"layer {i}: kv_from {src} is not an earlier latent-attention layer with a cache of its own "
                                 f"and the same kv_rank / rot_dim")
        return MixerSpec(kind="latent_attention", heads=int(m["heads"]), kv_heads=1, dim=int(m["dim"]), vdim=int(m["vdim"]),
                         scale=float(m["scale"]), rot_dims=rd, rot_base=float(rot.get("base", 10000.0)), rot_halves=True,
                         kv_rank=int(m["kv_rank"]), q_rank=0, sink=True, kv_from=src)
    raise ValueError(f"layer {i}: unknown mixer type {kind!r}")


def spec_from_config(cfg: dict) -> HybridSpec:
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    side = cfg.get("token_side") or {}
    sdim = int(side.get("dim", 0))
    layers: List[LayerSpec] = []
    for i, L in enumerate(cfg["layers"]):
        mlp = L.get("mlp")
        if mlp is not None and mlp.get("kind", "dense") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(LayerSpec(mixer=_mixer(i, L, cfg["layers"]), ff=int(mlp["ff"]) if mlp else 0, post_only=True,
                                ff_limit=float(mlp["limit"]) if mlp else 0.0, ff_alpha=FF_ALPHA, side_dim=sdim,
                                side_off=i * sdim))
    return HybridSpec(arch="fubepel", vocab=int(cfg["vocab"]), width=int(cfg["width"]), eps=float(cfg["norm"]["eps"]),
                      taps=1, layers=layers, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), norm_groups=1,
                      side_width=sdim * len(layers))


def layer_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor], i: int) -> dict:
    """The checkpoint's tensors of layer i under the names the engine uses."""
    L, m = spec.layers[i], spec.layers[i].mixer
    p = f"l{i}."
    out = {"norm1": sd[p + "norm1"], "q": sd[p + "mix.q"], "o": sd[p + "mix.o"]}
    if m.kind == "delta":
        for k in ("k", "v", "g", "b", "a", "A_log", "dt_bias"):
            out[k] = sd[p + "mix." + k]
        out["conv"] = torch.cat([sd[p + f"mix.{k}.conv"] for k in "qkv"], dim=0)
        out["out_norm"] = sd[p + "mix.norm"]
    elif m.kind == "attention":
        out.update(k=sd[p + "mix.k"], v=sd[p + "mix.v"])
    else:
        out.update(uk=sd[p + "mix.uk"], uv=sd[p + "mix.uv"], sink=sd[p + "mix.sink"])
        if m.kv_from is None:
            out.update(dkv=sd[p + "mix.dkv"], dkv_norm=sd[p + "mix.dkv.norm"])
    if L.ff:
        out.update(norm2=sd[p + "norm2"], gate=sd[p + "mlp.gate"], up=sd[p + "mlp.up"], down=sd[p + "mlp.down"])
    if L.side_dim:
        out.update(side_gate=sd[p + "side.gate"], side_proj=sd[p + "side.proj"], side_norm=sd[p + "side.norm"])
    return out


def model_tensors(spec: HybridSpec, sd: Dict[str, torch.Tensor]) -> dict:
    out = {"embed": sd["embed"], "head": sd["head"], "final_norm": sd["final.norm"],
           "layers": {i: layer_tensors(spec, sd, i) for i in range(spec.n_layers)}}
    if spec.side_width:
        out["side_embed"] = sd["side.embed"]
    return out


def random_state_dict(spec: HybridSpec, seed: int = 0, std: float = 0.05, device="cpu") -> Dict[str, torch.Tensor]:
    """Synthetic weights under the checkpoint's names (benchmarks and tests; there are no checkpoints offline)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = spec.width

    def n(*shape, s=std, mean=0.0):
        return (mean + s * torch.randn(tuple(shape), generator=g)).to(torch.bfloat16).to(device)

    sd = {"embed": n(spec.vocab, W, s=1.0 / max(spec.embed_scale, 1e-6)), "head": n(spec.vocab, W),
          "final.norm": n(W, mean=1.0, s=0.1)}
    if spec.side_width:
        sd["side.embed"] = n(spec.vocab, spec.side_width, s=1.0)
    for i, L in enumerate(spec.layers):
        m, p = L.mixer, f"l{i}."
        sd[p + "norm1"] = n(W, mean=1.0, s=0.1)
        H, G, D, V = m.heads, m.kv_heads, m.dim, m.vdim
        if m.kind == "delta":
            sd[p + "mix.q"], sd[p + "mix.k"], sd[p + "mix.v"] = n(G * D, W), n(G * D, W), n(H * V, W)
            for k, c in (("q", G * D), ("k", G * D), ("v", H * V)):
                sd[p + f"mix.{k}.conv"] = n(c, m.conv_taps, s=0.5)
            sd[p + "mix.b"], sd[p + "mix.a"] = n(H, W), n(H, W)
            sd[p + "mix.A_log"], sd[p + "mix.dt_bias"] = n(H, mean=-1.0, s=0.7), n(H, mean=-1.0, s=1.0)
            sd[p + "mix.norm"], sd[p + "mix.g"] = n(V, mean=1.0, s=0.1), n(H * V, W)
        elif m.kind == "attention":
            sd[p + "mix.q"], sd[p + "mix.k"], sd[p + "mix.v"] = n(H * D, W), n(G * D, W), n(G * V, W)
        else:
            K, R = m.kv_rank, m.rot_dims
            sd[p + "mix.q"] = n(H * (D + R), W)
            if m.kv_from is None:
                sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = n(K + R, W), n(K, mean=1.0, s=0.1)
            sd[p + "mix.uk"], sd[p + "mix.uv"] = n(H * D, K, s=1.0 / K ** 0.5), n(H * V, K, s=1.0 / K ** 0.5)
            sd[p + "mix.sink"] = n(H, s=1.0)
        sd[p + "mix.o"] = n(W, H * V)
        if L.ff:
            sd[p + "norm2"] = n(W, mean=1.0, s=0.1)
            sd[p + "mlp.gate"], sd[p + "mlp.up"], sd[p + "mlp.down"] = n(L.ff, W), n(L.ff, W), n(W, L.ff)
        if L.side_dim:
            sd[p + "side.gate"], sd[p + "side.proj"] = n(L.side_dim, W), n(W, L.side_dim, s=0.2)
            sd[p + "side.norm"] = n(W, mean=1.0, s=0.1)
    return sd


def config_from_spec(spec: HybridSpec) -> dict:
    """The config.json of a spec (tests and benchmarks write model directories with it)."""
    layers = []
    for L in spec.layers:
        m = L.mixer
        if m.kind == "delta":
            mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv_taps}
        elif m.kind == "attention":
            mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                  "mask": {"size": m.window, "keep_first": m.keep_first}}
        else:
            mx = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dims, "vdim": m.vdim, "kv_rank": m.kv_rank,
                  "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dims}}
            if m.kv_from is not None:
                mx["kv_from"] = m.kv_from
        layers.append({"type": m.kind, "mixer": mx,
                       "mlp": {"kind": "dense", "ff": L.ff, "limit": L.ff_limit} if L.ff else None})
    sdim = spec.layers[0].side_dim if spec.layers else 0
    cfg = {"architecture": ARCHITECTURE, "vocab": spec.vocab, "width": spec.width, "embedding": {"scale": spec.embed_scale},
           "norm": {"eps": spec.eps}, "layers": layers}
    if sdim:
        cfg["token_side"] = {"dim": sdim}
    return cfg
