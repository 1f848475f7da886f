"""Plain restatement of the Fubepel design in float64: whole sequences, one function per mechanism.

It is the oracle of the tests and imports nothing of the product.  A model is (cfg, sd): the dictionary of
config.json and the tensors under the checkpoint's names.  Notation: T tokens, W width, positions are 0-based per
sequence.  Every function takes and returns float64 tensors.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w when there is one."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def short_conv(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, C], w [C, taps]: out_t = sum_j w[:, j] h_(t - taps + 1 + j); nothing before the start."""
    T, taps = h.shape[0], w.shape[1]
    out = torch.zeros_like(h)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[:T - back]
    return out


def rotate_half_pairs(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [T, ..., n], pos [T]: entry i of the first `dims` is paired with entry i + dims/2 and the pair is turned by
    pos * base^(-2i/dims); the rest passes."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = pos.to(F64)[:, None] * f[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = a.cos().reshape(shape), a.sin().reshape(shape)
    u, w = v[..., :half], v[..., half:dims]
    return torch.cat((u * c - w * s, w * c + u * s, v[..., dims:]), dim=-1)


def visible(T: int, window: int = 0, keep_first: int = 0) -> torch.Tensor:
    """bool [T, T]: query i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window > 0:
        ok &= (i - j < window) | (j < keep_first)
    return ok


def softmax_attend(scores: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, sink: Optional[float] = None) -> torch.Tensor:
    """scores [T, T], v [T, V]: softmax over the visible keys; a sink adds exp(sink) to the denominator only."""
    s = scores.masked_fill(~mask, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.clamp(m, min=float(sink))
    p = torch.exp(s - m)
    den = p.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(torch.tensor(float(sink), dtype=F64) - m)
    return (p / den) @ v


def window_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Softmax attention without positions: q and k divided by their root mean square per head (no weight), grouped
    key/value heads, a sliding window that also keeps the first tokens.  P: q, k, v, o."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    vis = visible(T, int(mask.get("size", 0)), int(mask.get("keep_first", 0)))
    q = rms_norm((h @ P["q"].T).reshape(T, H, D), None, eps)
    k = rms_norm((h @ P["k"].T).reshape(T, G, D), None, eps)
    v = (h @ P["v"].T).reshape(T, G, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        out[:, hh] = softmax_attend((q[:, hh] @ k[:, g].T) * m["scale"], v[:, g], vis)
    return out.reshape(T, H * V) @ P["o"].T


def latent_kv(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float):
    """What a latent-attention layer caches per position: the normed latent c [T, K] and the rotated shared key part
    [T, R]."""
    T, K, R = h.shape[0], m["kv_rank"], m["rot_dim"]
    kv = h @ P["dkv"].T
    c = rms_norm(kv[:, :K], P["dkv.norm"], eps)
    kr = rotate_half_pairs(kv[:, K:], torch.arange(T), float(m["rot"]["base"]), int(m["rot"]["dims"]))
    return c, kr


def latent_attention(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float, cached=None) -> torch.Tensor:
    """Causal attention whose keys and values are up-projections of a cached latent, plus one rotated key part shared
    by the heads; the softmax has a per-head sink.  `cached`: (c, kr) of the layer whose cache this layer reads
    (None: its own).  P: q, [dkv, dkv.norm], uk, uv, sink, o."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = latent_kv(h, P, m, eps) if cached is None else cached
    q = (h @ P["q"].T).reshape(T, H, D + R)
    qr = rotate_half_pairs(q[..., D:], torch.arange(T), float(m["rot"]["base"]), int(m["rot"]["dims"]))
    kn = (c @ P["uk"].T).reshape(T, H, D)
    v = (c @ P["uv"].T).reshape(T, H, V)
    vis = visible(T)
    out = torch.zeros(T, H, V, dtype=F64)
    for hh in range(H):
        s = (q[:, hh, :D] @ kn[:, hh].T + qr[:, hh] @ kr.T) * m["scale"]
        out[:, hh] = softmax_attend(s, v[:, hh], vis, sink=float(P["sink"][hh]))
    return out.reshape(T, H * V) @ P["o"].T


def delta_rule(q, k, v, beta, g):
    """One head.  q, k [T, D], v [T, V], beta, g [T].  S starts at zero; per token S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q (the read-out sees the token's own write)."""
    T, D = q.shape
    S = torch.zeros(D, v.shape[1], dtype=F64)
    o = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o


def gated_delta(h: torch.Tensor, P: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Gated delta-rule mixer.  P: q, q.conv, k, k.conv, v, v.conv, b, a, A_log, dt_bias, norm, g, o."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ P["q"].T, P["q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ P["k"].T, P["k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ P["v"].T, P["v.conv"])).reshape(T, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P["b"].T)
    decay = torch.exp(-torch.exp(P["A_log"]) * softplus(h @ P["a"].T + P["dt_bias"]))
    o = torch.zeros(T, H, V, dtype=F64)
    for hh in range(H):
        gq = hh // (H // G)
        o[:, hh] = delta_rule(q[:, gq], k[:, gq], v[:, hh], beta[:, hh], decay[:, hh])
    o = rms_norm(o, P["norm"], eps) * silu(h @ P["g"].T).reshape(T, H, V)
    return o.reshape(T, H * V) @ P["o"].T


def clamped_ff(h: torch.Tensor, P: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    """down(g sigmoid(1.702 g) (u + 1)) with g = min(gate h, limit) and u = clamp(up h, -limit, limit)."""
    g = torch.clamp(h @ P["gate"].T, max=limit)
    u = torch.clamp(h @ P["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P["down"].T


def token_side(x: torch.Tensor, e: torch.Tensor, P: Dict[str, torch.Tensor], eps: float) -> torch.Tensor:
    """The per-layer token input: x + rms_norm(proj(gelu(gate x) * e)) * norm, e [T, dim] the layer's part of the
    tokens' side embedding."""
    y = (gelu_tanh(x @ P["gate"].T) * e) @ P["proj"].T
    return x + rms_norm(y, P["norm"], eps)


def _sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(F64) for k, v in sd.items() if k.startswith(prefix)}


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; layers_out collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x = sd["embed"].to(F64)[tok] * float(cfg["embedding"]["scale"])
    side = cfg.get("token_side")
    sdim = int(side["dim"]) if side else 0
    cache = {}
    for i, L in enumerate(cfg["layers"]):
        m, P = L["mixer"], _sub(sd, f"l{i}.mix.")
        if L["type"] == "delta":
            y = gated_delta(x, P, m, eps)
        elif L["type"] == "attention":
            y = window_attention(x, P, m, eps)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                cache[i] = latent_kv(x, P, m, eps)
            y = latent_attention(x, P, m, eps, cached=cache[i if src is None else int(src)])
        else:
            raise ValueError(L["type"])
        x = x + rms_norm(y, sd[f"l{i}.norm1"].to(F64), eps)
        if L.get("mlp") is not None:
            y = clamped_ff(x, _sub(sd, f"l{i}.mlp."), float(L["mlp"]["limit"]))
            x = x + rms_norm(y, sd[f"l{i}.norm2"].to(F64), eps)
        if sdim:
            e = sd["side.embed"].to(F64)[tok][:, i * sdim:(i + 1) * sdim]
            x = token_side(x, e, _sub(sd, f"l{i}.side."), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, sd["final.norm"].to(F64), eps) @ sd["head"].to(F64).T


def greedy(cfg: dict, sd: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[-1].argmax()))
    return toks
