"""Plain restatement of the Gimudra design in float64: whole sequences, one function per mechanism.

It is the oracle of the tests and imports nothing of the product.  A model is (cfg, sd): the dictionary of
config.json and the tensors under the checkpoint's names.  Notation: T tokens, W width, positions are 0-based per
sequence.  Every function takes and returns float64 tensors.

The design: x_0 = embed[token] * scale + sinusoid(position).  Layer i reads u_i = sum_(j <= i) a_(i-1)[j] X_j (u_0 = X_0 = x_0),
computes X_(i+1) = r + ls2 * ff(norm2(r)) with r = u_i + ls1 * mixer(shift(norm1(u_i))), and hands on
u_(i+1) = sum_(j <= i+1) a_i[j] X_j.  shift(h)_t = h_t + (h_(t-1) - h_t) * s.  The mixer is softmax attention inside
blocks of positions with a logarithmic distance penalty; the feed-forward is gated (SiLU) with biases, or a mixture of
squared-ReLU experts routed in groups, some of whose router outputs pass the input through.
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


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def sinusoid(pos: torch.Tensor, width: int) -> torch.Tensor:
    """[T, width]: entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos of the same angle."""
    out = torch.zeros(pos.shape[0], width, dtype=F64)
    for c in range(width):
        i = c // 2
        ang = pos.to(F64) * (10000.0 ** (-2.0 * i / width))
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def embed(tokens: List[int], table: torch.Tensor, scale: float, first_pos: int = 0) -> torch.Tensor:
    T = len(tokens)
    x = table.to(F64)[torch.tensor(tokens, dtype=torch.long)] * scale
    return x + sinusoid(torch.arange(first_pos, first_pos + T), table.shape[1])


def token_shift(h: torch.Tensor, s: torch.Tensor, before: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, W]: row t becomes h_t + (h_(t-1) - h_t) * s, with h_(-1) = `before` (zeros at the start of a sequence)."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * s


def block_visible(T: int, size: int) -> torch.Tensor:
    """bool [T, T]: query i sees key j when j <= i and both lie in the same block of `size` positions (size 0: causal)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if size > 0:
        ok = ok & ((i // size) == (j // size))
    return ok


def distance_penalty(T: int, r1: torch.Tensor, r2: torch.Tensor) -> torch.Tensor:
    """[H, T, T]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (0 elsewhere)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).clamp(min=0).to(F64)
    return r1.to(F64)[:, None, None] * torch.log1p(r2.to(F64)[:, None, None] * dist[None])


def attention_scores_softmax(q, k, v, scale, size, r1, r2):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]; head h reads key/value head h // (H / G)."""
    T, H, D = q.shape
    G = k.shape[1]
    vis = block_visible(T, size)
    pen = distance_penalty(T, r1, r2)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale - pen[h]
        s = s.masked_fill(~vis, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention(h: torch.Tensor, sd: Dict[str, torch.Tensor], p: str, m: dict, kv=None):
    """The mixer on its (shifted) input h [T, W].  kv: another layer's (k, v) to read instead of projecting.  Returns
    (output [T, W], (k, v))."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ sd[p + "q"].to(F64).T + sd[p + "q.b"].to(F64)).reshape(T, H, D)
    if kv is None:
        k = (h @ sd[p + "k"].to(F64).T + sd[p + "k.b"].to(F64)).reshape(T, G, D)
        v = (h @ sd[p + "v"].to(F64).T + sd[p + "v.b"].to(F64)).reshape(T, G, V)
    else:
        k, v = kv
    size = int((m.get("mask") or {}).get("size", 0))
    o = attention_scores_softmax(q, k, v, float(m["scale"]), size, sd[p + "r1"], sd[p + "r2"])
    return o.reshape(T, H * V) @ sd[p + "o"].to(F64).T, (k, v)


def dense_ff(h: torch.Tensor, sd: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ sd[p + "gate"].to(F64).T + sd[p + "gate.b"].to(F64)
    u = h @ sd[p + "up"].to(F64).T + sd[p + "up.b"].to(F64)
    return (silu(g) * u) @ sd[p + "down"].to(F64).T + sd[p + "down.b"].to(F64)


def route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict):
    """Per row the chosen router outputs and their weights: (idx [T, top], weight [T, top]).  Scores are the softmax over
    all outputs; the choice is by score + correction among the outputs of the `keep` groups whose best choice score is
    largest; the weight is the score itself times `scale`."""
    n = w_router.shape[0]
    top = int(r["top"])
    groups = r.get("groups") or {}
    count, keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
    s = torch.softmax(h @ w_router.to(F64).T, dim=-1)
    c = s + correction.to(F64)
    T = h.shape[0]
    idx = torch.zeros(T, top, dtype=torch.long)
    wt = torch.zeros(T, top, dtype=F64)
    per = n // count
    for t in range(T):
        best = [max(c[t, g * per:(g + 1) * per].tolist()) for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-best[g], g))[:keep]
        allowed = [o for o in range(n) if o // per in kept]
        order = sorted(allowed, key=lambda o: (-float(c[t, o]), o))[:top]
        for k_, o in enumerate(order):
            idx[t, k_] = o
            wt[t, k_] = s[t, o] * float(r.get("scale", 1.0))
    return idx, wt


def moe_ff(h: torch.Tensor, sd: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    E, I = int(r["experts"]), int(r.get("identity", 0))
    idx, wt = route(h, sd[p + "router"], sd[p + "correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k_ in range(idx.shape[1]):
            e = int(idx[t, k_])
            if e >= E:  # passes its input through
                y = h[t]
            else:
                a = torch.relu(sd[p + f"e{e}.up"].to(F64) @ h[t]) ** 2
                y = sd[p + f"e{e}.down"].to(F64) @ a
            out[t] += wt[t, k_] * y
    assert E + I == sd[p + "router"].shape[0]
    return out


def forward(cfg: dict, sd: Dict[str, torch.Tensor], tokens: List[int], trace: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; trace (a list) collects the stream handed on after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, sd["embed"], float((cfg.get("embedding") or {}).get("scale", 1.0)))
    X = [x]
    kvs = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = rms_norm(x, sd[p + "norm1"].to(F64), eps)
        if p + "shift" in sd:
            h = token_shift(h, sd[p + "shift"].to(F64))
        src = m.get("kv_from")
        y, kvs[i] = attention(h, sd, p + "mix.", m, kv=None if src is None else kvs[int(src)])
        x = x + y * sd[p + "ls1"].to(F64) if p + "ls1" in sd else x + y
        mlp = L.get("mlp")
        if mlp is not None:
            h2 = rms_norm(x, sd[p + "norm2"].to(F64), eps)
            f = dense_ff(h2, sd, p + "mlp.") if mlp.get("kind", "dense") == "dense" else moe_ff(h2, sd, p + "mlp.", mlp)
            x = x + f * sd[p + "ls2"].to(F64) if p + "ls2" in sd else x + f
        X.append(x)
        if p + "dwa" in sd:
            a = sd[p + "dwa"].to(F64)
            x = sum(a[j] * X[j] for j in range(len(X)))
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, sd["final.norm"].to(F64), eps) @ sd["head"].to(F64).T


def greedy(cfg: dict, sd: Dict[str, torch.Tensor], prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[-1].argmax()))
    return toks
