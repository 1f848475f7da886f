"""RaggedEngine — a decoder whose layers are of different kinds, run on RAGGED steps.

ShardEngine (engine.py) serves uniform Llama / GPT-2 stacks on rectangular batches with a bf16 residual stream.
This engine serves stacks described layer by layer (HybridSpec): every layer has a token mixer — softmax attention
with its options, latent attention, or a recurrent cell with a matrix state (mLSTM, state-space, gated delta rule) —
and optionally a feed-forward (dense or a mixture of experts).  Four layer styles: sublayers in sequence, each
wrapped in a pre-norm and a post-norm with one weight and reading its input through a short causal convolution;
mixer and feed-forward side by side on one grouped norm; sublayers that read the residual stream itself and are
normed on their output only, followed by a per-layer token input; pre-normed sublayers with a weight vector per
norm, a layer scale on each result, a token shift in front of the mixer and an average over all layers' results
after the layer.  Layers may share another layer's weights while
keeping a cache / state of their own, or read another layer's cache.  The residual stream, norms, rotation
angles, scores, softmax weights, convolution and recurrent state are fp32; projections run in the element type of the
engine (bf16 on the tcgen05 / GEMV kernels of ops.linear, or float32 on the CUDA-core GEMM).

One call of step() takes the NEXT TOKENS of any number of live sequences — a portion of a prompt of any length
beside single decoded tokens — as one batch: projections and feed-forwards run over all rows at once, attention
reads and extends the paged key/value cache (engine.PagedKVCache), recurrent layers and the input convolutions
read and advance the sequence's state slot (state_cache.StateSlots).  The result at a position does not depend
on how the sequence was cut into steps, on the other rows, or on the pages and slot it got, beyond rounding.
batching.RaggedBatcher schedules requests onto step(); generate() is that scheduler behind ShardEngine's signature.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import ops
from .engine import PagedKVCache
from .state_cache import StateSlots

BF = torch.bfloat16


@dataclass
class MixerSpec:
    kind: str                      # "attention", "mlstm", "latent_attention", "mamba2" or "delta"
    heads: int
    kv_heads: int
    dim: int                       # query / key size per head
    vdim: int                      # value size per head
    # attention
    scale: float = 1.0
    rot_dims: int = 0              # leading dims of q / k that are rotated (interleaved pairs); 0 = none
    rot_base: float = 10000.0
    rot_scaling: Optional[dict] = None   # {factor, low, high, original}: wavelength-dependent frequency scaling
    chunk: int = 0                 # > 0: a position sees only its own block of `chunk` positions
    window: int = 0                # > 0: a position sees the last `window` positions
    keep_first: int = 0            # with a chunk or window: the first `keep_first` positions stay visible
    qk_norm: bool = False          # per-head RMS norm of q and k (weights q_norm / k_norm; without them: plain division)
    rotate_values: bool = False    # values rotated by their position, outputs turned back by theirs
    sink: bool = False             # one extra softmax term per head without key or value
    head_gate: bool = False        # sigmoid gate per head on the output
    # mlstm
    gate_cap: float = 0.0
    # latent attention: queries and keys/values pass through low-rank latents; `dim` is the unrotated and `rot_dims`
    # the rotated query/key size per head; the cache holds kv_rank + rot_dims numbers per position
    kv_rank: int = 0
    q_rank: int = 0                # 0: queries are projected directly, without a latent
    out_gate: bool = False         # sigmoid gate per output channel (head_gate: one per head)
    rot_halves: bool = False       # rotation pairs (i, i + rot_dims/2) instead of interleaved (2i, 2i+1)
    kv_from: Optional[int] = None  # the layer reads that (earlier) layer's cache and writes none of its own
    bias: bool = False             # attention: q / k / v projections have biases
    dist_penalty: bool = False     # attention: r1[h] ln(1 + r2[h] (i - j)) is taken off the scaled scores
    # mamba2: state rows per head, B/C groups, groups of the gated output norm, taps of the x/B/C convolution
    state: int = 0
    groups: int = 1
    norm_groups: int = 1
    conv_taps: int = 0
    # delta (gated delta rule): heads value heads of size vdim, kv_heads query/key heads of size dim, conv_taps of the
    # q / k / v convolution, scale on the unit queries, unit_eps under the root of the unit vectors
    unit_eps: float = 1e-6


@dataclass
class MoESpec:
    """Mixture-of-experts feed-forward: `experts` gated experts of size ff, then `identity` router outputs that pass
    the input through; `top` are used per token; a shared expert (shared_ff > 0) runs for every token."""
    experts: int
    identity: int
    top: int
    ff: int
    limit: float                   # gate is cut at +limit, up at +-limit
    shared_ff: int = 0
    shared_limit: float = 0.0
    alpha: float = 1.702           # g * sigmoid(alpha * g)
    gated: bool = True             # False: experts are down(max(up x, 0)^2), no gate, no clamps
    groups: int = 1                # > 1: router outputs form that many equal groups; only the `keep` best groups' outputs
    keep: int = 1                  # can be chosen
    route_scale: float = 1.0       # factor on the routing weights
    renorm: bool = True            # weights divided by the sum of the chosen scores (False: the scores themselves)

    @property
    def total_ff(self) -> int:
        return self.experts * self.ff + self.shared_ff


@dataclass
class LayerSpec:
    mixer: MixerSpec
    ff: int = 0                    # dense feed-forward size, 0 = none
    weights_of: Optional[int] = None
    moe: Optional[MoESpec] = None  # mixture-of-experts feed-forward
    parallel: bool = False         # True: ONE grouped norm; mixer (through the input convolution) and feed-forward both
                                   # read it and x += mixer + feed-forward.  False: pre-/post-normed sublayers in sequence
    ckpt: Optional[int] = None     # the checkpoint's layer number when it differs from the position in `layers`
    reenter: Optional[int] = None  # t: before this layer x <- W_loop [x | embedding output] + step[t]
    post_only: bool = False        # True: sublayers read x itself and x += rmsnorm(sublayer(x)) * weight vector; no input
                                   # convolution
    ff_limit: float = 0.0          # > 0: the dense feed-forward is min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u) + 1)
    ff_alpha: float = 1.702
    side_dim: int = 0              # > 0: after the feed-forward, the per-layer token input of this size ...
    side_off: int = 0              # ... read at this column of the side embedding table
    pre_norm: bool = False         # True: x += ls1 * mixer(norm1(x)); x += ls2 * ff(norm2(x)) with weight vectors, and:
    token_shift: bool = False      # the mixer reads h_t + (h_(t-1) - h_t) * shift of its normed input (a row per slot)
    layer_scale: bool = False      # vectors ls1 / ls2 on the sublayers' results
    depth_avg: bool = False        # after the layer x <- sum_j dwa[j] X_j over the embedding output and all results so far
    ff_bias: bool = False          # the dense feed-forward's projections have biases


@dataclass
class HybridSpec:
    arch: str
    vocab: int
    width: int
    eps: float
    taps: int                      # taps of the input convolutions (1: the current input only, no state)
    layers: List[LayerSpec] = field(default_factory=list)
    embed_scale: float = 1.0
    norm_groups: int = 0           # > 0: the final norm (and the norm of parallel layers) is grouped with a weight vector
    loop_passes: int = 0           # > 0: the model has the loop re-entry projection and per-pass vectors
    side_width: int = 0            # > 0: columns of the side embedding table [vocab, side_width]
    pos_sinusoid: bool = False     # the embedding output gets sin / cos (position * pos_base^(-2i/width)) added
    pos_base: float = 10000.0

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def source(self, i: int) -> int:
        j = self.layers[i].weights_of
        return i if j is None else j


def rot_frequencies(base: float, dims: int, scaling: Optional[dict]) -> torch.Tensor:
    """float64 [dims/2]: f_i = base^(-2i/dims), then the wavelength-dependent scaling of long-context Llama
    checkpoints: wavelengths below original/high keep f, above original/low use f/factor, between them a linear
    blend in original/wavelength."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if not scaling:
        return f
    fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wl = 2.0 * math.pi / fi
        if wl < orig / hi:
            out.append(fi)
        elif wl > orig / lo:
            out.append(fi / fac)
        else:
            s = (orig / wl - lo) / (hi - lo)
            out.append((1.0 - s) * fi / fac + s * fi)
    return torch.tensor(out, dtype=torch.float64)


def _ceil(a: int, b: int) -> int:
    return (a + b - 1) // b * b


class RaggedEngine:
    def __init__(self, spec: HybridSpec, device: str = "cuda:0", max_batch: int = 4, max_seq_len: int = 2048,
                 page_size: int = 16, kv_pool_tokens: Optional[int] = None, dtype=BF):
        if not torch.cuda.is_available():
            raise RuntimeError("RaggedEngine needs a CUDA device: this package has no CPU path")
        if dtype not in (BF, torch.float32):
            raise ValueError("dtype: torch.bfloat16 or torch.float32")
        self.spec, self.dtype = spec, dtype
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.max_batch, self.max_seq_len = int(max_batch), int(max_seq_len)
        self.is_first = self.is_last = self.has_head = True
        # layers that own a paged cache (a layer with kv_from reads its source's)
        self.attn_layers = [i for i, L in enumerate(spec.layers)
                            if L.mixer.kind in ("attention", "latent_attention") and L.mixer.kv_from is None]
        # latent attention caches ONE row [latent | rotated key part] per position and no values of its own
        shapes = [(1, m.kv_rank + m.rot_dims, 0) if m.kind == "latent_attention" else (m.kv_heads, m.dim, m.vdim)
                  for m in (spec.layers[i].mixer for i in self.attn_layers)]
        self.kv = PagedKVCache(len(shapes), 0, 0, page_size, self.max_batch, self.max_seq_len, self.device,
                               pool_tokens=kv_pool_tokens, layer_shapes=shapes, dtype=dtype)
        self.kv_index = {li: n for n, li in enumerate(self.attn_layers)}
        for i, L in enumerate(spec.layers):
            if L.mixer.kv_from is not None:
                self.kv_index[i] = self.kv_index[L.mixer.kv_from]
        self.slots = StateSlots(self.max_batch, self.device)
        for i, L in enumerate(spec.layers):
            if spec.taps > 1 and not L.post_only and not L.pre_norm:
                self.slots.add(("tail1", i), spec.taps - 1, spec.width)
                if L.ff:
                    self.slots.add(("tail2", i), spec.taps - 1, spec.width)
            if L.pre_norm and L.token_shift:
                self.slots.add(("shift", i), spec.width)  # the previous position's normed mixer input
            if L.mixer.kind == "delta":
                m = L.mixer
                self.slots.add(("S", i), m.heads, m.vdim, m.dim)  # value-major: the transposed state
                if m.conv_taps > 1:
                    self.slots.add(("ctail", i), m.conv_taps - 1, 2 * m.kv_heads * m.dim + m.heads * m.vdim)
            if L.mixer.kind == "mlstm":
                m = L.mixer
                self.slots.add(("S", i), m.heads, m.dim, m.vdim)
                self.slots.add(("n", i), m.heads, m.dim)
                self.slots.add(("m", i), m.heads)
            if L.mixer.kind == "mamba2":
                m = L.mixer
                self.slots.add(("S", i), m.heads, m.state, m.vdim)
                if m.conv_taps > 1:
                    self.slots.add(("ctail", i), m.conv_taps - 1, m.heads * m.vdim + 2 * m.groups * m.state)
        self.lengths: Dict[int, int] = {}          # slot -> tokens the sequence holds
        self.w: Dict[str, object] = {}
        self.layers: Dict[int, dict] = {}
        self._tables: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._ws_rows = 0
        self._meta_cap = 0
        self._graphs: Dict[tuple, object] = {}
        self.use_cuda_graph = os.environ.get("DLI_RAGGED_GRAPH", "1") == "1"
        self.eos_token_ids: tuple = ()
        self.pad_token_id: Optional[int] = None
        self.prefill_chunk: Optional[int] = None   # tokens of a prompt per step (None: the scheduler's default)
        self.tc_min_rows = int(os.environ.get("DLI_RAGGED_TC_MIN_ROWS", "16"))  # portions from this size: tensor-core attention
        self.moe_sel_max_rows = 8                  # up to this many rows a step reads only the chosen experts' weights ...
        self.moe_sel_share = 3.0                   # ... if what the rows choose is at most 1/3 of all expert weights ...
        self.moe_sel_min_bytes = 512 << 20         # ... and a layer's experts are at least this large: the two gathering kernels
                                                   # take ~75 us whatever they read, the stream over all experts runs at 0.6-0.95
                                                   # of the HBM peak (measured: 235 MB of experts, 4 of 14 chosen: 81 against 69 us;
                                                   # 822 MB: 100 against 143 us)
        self.delta_blocked = False                 # portions of prompts through the delta rule 16 rows at a time; off: row by row,
                                                   # which is faster while one sequence's columns leave a warp per scheduler
                                                   # (0.89 against 1.15 ms for 2 048 rows, 8 heads of 128 x 256)
        self.side_fused_max_rows = 16              # up to this many rows the per-layer token input is one kernel ...
        self.side_fused_max_bytes = 64 << 10       # ... if its two matrices are at most this large (else: weight streams)
        self.latent_expand_max_elems = 1 << 31     # scratch bound (4 GiB in bf16) of the per-head expansion of cached latents
        self.mlstm_parallel_max_floats = 1 << 28   # scratch bound (1 GiB) of the block-parallel mLSTM / state-space scan; beyond it: blocks in order
        self.layer_trace: Optional[list] = None    # set to [] to collect the residual stream after every layer
        ops.set_pdl(os.environ.get("DLI_PDL", "1") == "1")
        self._sms = ops.sm_count()

    # ------------------------------------------------------------------ weights
    def _table(self, base: float, dims: int, scaling: Optional[dict]):
        """fp32 cos / sin [max_seq_len, dims/2] of position * frequency, angles taken in float64 on the host."""
        key = (base, dims, tuple(sorted(scaling.items())) if scaling else None)
        if key not in self._tables:
            f = rot_frequencies(base, dims, scaling)
            ang = torch.arange(self.max_seq_len, dtype=torch.float64)[:, None] * f[None, :]
            self._tables[key] = (ang.cos().float().contiguous().to(self.device),
                                 ang.sin().float().contiguous().to(self.device))
        return self._tables[key]

    def load_tensors(self, t: dict) -> None:
        """t: {"embed", "head", "final_norm", "layers": {i: {...}}} (+ "loop_in", "loop_step") with the layer tensors
        named as in sokevik.layer_tensors / togalorn.layer_tensors (any dtype / device); linear weights [out, in]."""
        dev, E = self.device, self.dtype
        s = self.spec

        def mat(*ws, pad_rows=True):
            """Rows of several [out, in] matrices stacked (padded to a multiple of 16 rows with zeros)."""
            w = torch.cat([x.reshape(-1, x.shape[-1]) for x in ws], dim=0).to(E)
            pad = _ceil(w.shape[0], 16) - w.shape[0] if pad_rows else 0
            if pad:
                w = torch.cat((w, torch.zeros(pad, w.shape[1], dtype=E, device=w.device)), dim=0)
            return w.contiguous().to(dev)

        def vec(x):
            return x.to(torch.float32).reshape(-1).contiguous().to(dev)

        def f32(x):
            return x.to(torch.float32).contiguous().to(dev)

        self.w = {"embed": t["embed"].to(E).contiguous().to(dev), "head": mat(t["head"]),
                  "final_norm": vec(t["final_norm"]) if s.norm_groups else float(t["final_norm"])}
        if s.side_width:
            self.w["side_embed"] = t["side_embed"].to(E).contiguous().to(dev)
        if s.loop_passes:
            self.w["loop_in"] = mat(t["loop_in"], pad_rows=False)
            self.w["loop_step"] = f32(t["loop_step"])
        if s.pos_sinusoid:
            # frequencies in float64 on the host, rounded once; the angle position * frequency is formed in fp32
            self.w["pos_freq"] = torch.tensor([s.pos_base ** (-2.0 * i / s.width) for i in range((s.width + 1) // 2)],
                                              dtype=torch.float64).to(torch.float32).to(dev)
        self.layers = {}
        for i, src in t["layers"].items():
            L, m = s.layers[i], s.layers[i].mixer
            d = {} if (L.post_only or L.pre_norm) else {"canon1": f32(src["canon1"])}
            if L.parallel or L.post_only or L.pre_norm:
                d["norm1"] = vec(src["norm1"])
            else:
                d["norm1"], d["norm1b"] = float(src["norm1"]), float(src["norm1b"])
            qn, kn, vn = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
            if m.kind == "attention" and m.kv_from is not None:
                # only queries: keys and values are the source layer's cache
                if m.head_gate or m.qk_norm or m.rot_dims or m.rotate_values:
                    raise ValueError(f"layer {i}: another layer's cache with a gate, head norms or rotation is not supported")
                d["w_proj"] = mat(src["q"])
                d["off"] = {"q": 0, "k": 0, "v": 0, "g": -1}
                d["q_norm"] = d["k_norm"] = d["sink"] = None
                d["qkv_b"] = vec(src["q_b"]) if m.bias else None
                d["r1"], d["r2"] = (vec(src["r1"]), vec(src["r2"])) if m.dist_penalty else (None, None)
            elif m.kind == "attention":
                d["w_proj"] = mat(src["q"], src["k"], src["v"], src["g"]) if m.head_gate else mat(src["q"], src["k"], src["v"])
                d["off"] = {"q": 0, "k": qn, "v": qn + kn, "g": qn + kn + vn if m.head_gate else -1}
                d["qkv_b"] = vec(torch.cat([src[k].reshape(-1).float() for k in ("q_b", "k_b", "v_b")])) if m.bias else None
                # a norm without weights is the norm with unit weights
                ones = torch.ones(m.dim, dtype=torch.float32, device=dev)
                d["q_norm"] = (vec(src["q_norm"]) if "q_norm" in src else ones) if m.qk_norm else None
                d["k_norm"] = (vec(src["k_norm"]) if "k_norm" in src else ones) if m.qk_norm else None
                d["sink"] = vec(src["sink"]) if m.sink else None
                d["r1"], d["r2"] = (vec(src["r1"]), vec(src["r2"])) if m.dist_penalty else (None, None)
            elif m.kind == "mlstm":
                gn = m.heads * m.vdim
                d["w_proj"] = mat(src["q"], src["k"], src["v"], src["g"], src["i"], src["f"])
                d["off"] = {"q": 0, "k": qn, "v": 2 * qn, "g": 2 * qn + gn, "i": 2 * qn + 2 * gn,
                            "f": 2 * qn + 2 * gn + m.heads}
                d["i_b"], d["f_b"], d["out_norm"] = vec(src["i_b"]), vec(src["f_b"]), vec(src["out_norm"])
            elif m.kind == "latent_attention":
                # one projection of the mixer's input: query latent (or, without one, the queries themselves) | key/value
                # latent and rotated key part (none in a layer that reads another layer's cache) | output gate
                if m.kv_from is not None and m.q_rank:
                    raise ValueError(f"layer {i}: a query latent together with another layer's cache is not supported")
                nq = m.q_rank if m.q_rank else m.heads * (m.dim + m.rot_dims)
                parts = [src["dq"] if m.q_rank else src["q"]] + ([src["dkv"]] if m.kv_from is None else []) + \
                        ([src["g"]] if m.out_gate else [])
                d["w_proj"] = mat(*parts)
                nkv = m.kv_rank + m.rot_dims if m.kv_from is None else 0
                d["off"] = {"cq": 0, "kv": nq, "g": nq + nkv if m.out_gate else -1}
                if m.q_rank:
                    d["w_uq"] = mat(src["uq"], pad_rows=False)
                    d["q_norm"] = vec(src["dq_norm"])
                d["kv_norm"] = vec(src["dkv_norm"]) if m.kv_from is None else None
                d["sink"] = vec(src["sink"]) if m.sink else None
                d["uk"], d["uv"] = mat(src["uk"], pad_rows=False), mat(src["uv"], pad_rows=False)
                if E == BF and ops.attn_ragged_tc_supported(m.dim + m.rot_dims, m.vdim, E):
                    # steps with portions of prompts expand the cached latents to per-head keys and values with ONE GEMM
                    # over the pool rows [latent | rotated key part]: [uk; uv] with zero columns under the rotated part
                    ukv = torch.cat((src["uk"], src["uv"]), dim=0).to(E)
                    d["w_ukv"] = torch.cat((ukv, torch.zeros(ukv.shape[0], m.rot_dims, dtype=E, device=ukv.device)),
                                           dim=1).contiguous().to(dev)
            elif m.kind == "mamba2":
                inner, gn = m.heads * m.vdim, m.groups * m.state
                d["w_proj"] = mat(src["in"])
                d["off"] = {"z": 0, "x": inner, "dt": 2 * inner + 2 * gn}
                d["conv_w"], d["conv_b"] = f32(src["conv"]), vec(src["conv_b"])
                d["dt_bias"], d["a_log"], d["d_skip"] = vec(src["dt_bias"]), vec(src["A_log"]), vec(src["D"])
                d["out_norm"] = vec(src["out_norm"])
            elif m.kind == "delta":
                gd, hv = m.kv_heads * m.dim, m.heads * m.vdim
                d["w_proj"] = mat(src["q"], src["k"], src["v"], src["g"], src["b"], src["a"])
                d["off"] = {"q": 0, "k": gd, "v": 2 * gd, "g": 2 * gd + hv, "b": 2 * gd + 2 * hv, "a": 2 * gd + 2 * hv + m.heads}
                d["conv_w"] = f32(src["conv"])
                d["a_log"], d["dt_bias"], d["out_norm"] = vec(src["A_log"]), vec(src["dt_bias"]), vec(src["out_norm"])
            else:
                raise ValueError(f"layer {i}: mixer kind {m.kind!r}")
            d["wo"] = mat(src["o"], pad_rows=False)
            if L.side_dim:
                d["side_gate"], d["side_proj"] = mat(src["side_gate"], pad_rows=False), mat(src["side_proj"], pad_rows=False)
                d["side_norm"] = vec(src["side_norm"])
            if L.pre_norm:
                for k in ("shift", "ls1", "ls2", "dwa"):
                    d[k] = vec(src[k]) if k in src else None
                if d["dwa"] is not None and d["dwa"].numel() != i + 2:
                    raise ValueError(f"layer {i}: {d['dwa'].numel()} averaging weights for {i + 2} results")
                if L.ff or L.moe is not None:
                    d["norm2"] = vec(src["norm2"])
            if L.ff and L.pre_norm:
                # silu(gate) * up as the GEMM's epilogue where there are no biases and the tile's alignment holds; else
                # [gate rows | up rows] and the activation (with the biases) as a kernel of its own
                d["packed"] = E == BF and not L.ff_bias and L.ff % 128 == 0 and s.width % 8 == 0
                if d["packed"]:
                    d["w_gu"] = ops.pack_gate_up(src["gate"].to(BF), src["up"].to(BF)).to(dev)
                else:
                    d["w_gu"] = mat(src["gate"], src["up"], pad_rows=False)
                d["gu_b"] = vec(torch.cat((src["gate_b"].reshape(-1).float(), src["up_b"].reshape(-1).float()))) if L.ff_bias else None
                d["down_b"] = vec(src["down_b"]) if L.ff_bias else None
                d["w_down"] = mat(src["down"], pad_rows=False)
            elif L.ff and L.post_only:
                d["norm2"] = vec(src["norm2"])
                # the tensor-core path interleaves gate and up rows so that the clamped activation is the GEMM's epilogue;
                # other shapes: [gate rows | up rows] and the activation as a kernel of its own
                d["packed"] = E == BF and L.ff % 128 == 0 and s.width % 8 == 0
                if d["packed"]:
                    d["w_gu"] = ops.pack_gate_up(src["gate"].to(BF), src["up"].to(BF)).to(dev)
                    d["ff_act"] = torch.tensor([L.ff_limit, L.ff_alpha], dtype=torch.float32, device=dev)
                else:
                    d["w_gu"] = mat(src["gate"], src["up"])
                d["w_down"] = mat(src["down"], pad_rows=False)
            elif L.ff:
                d["norm2"], d["norm2b"] = float(src["norm2"]), float(src["norm2b"])
                d["canon2"] = f32(src["canon2"])
                # the tensor-core path interleaves gate and up rows so that silu(gate) * up is the GEMM's epilogue
                d["packed"] = E == BF and L.ff % 128 == 0 and s.width % 8 == 0
                if d["packed"]:
                    d["w_gu"] = ops.pack_gate_up(src["gate"].to(BF), src["up"].to(BF)).to(dev)
                else:
                    d["w_gu"] = torch.cat((src["gate"], src["up"]), dim=0).to(E).contiguous().to(dev)
                d["w_down"] = mat(src["down"], pad_rows=False)
            if L.moe is not None:
                # all experts as ONE gate/up matrix (per expert [gate; up], the shared expert last) and ONE down matrix
                # over the concatenated expert activations: the routing weights are applied between the two
                e = L.moe
                blocks = [x for g_, u_, _ in src["experts"] for x in ((g_, u_) if e.gated else (u_,))]
                downs = [d_ for _, _, d_ in src["experts"]]
                if e.shared_ff:
                    blocks += [src["shared"][0], src["shared"][1]] if e.gated else [src["shared"][1]]
                    downs.append(src["shared"][2])
                d["w_gu"] = mat(*blocks)
                d["w_down"] = torch.cat([x.to(E) for x in downs], dim=1).contiguous().to(dev)
                d["w_router"], d["corr"] = f32(src["router"]), vec(src["correction"])
            self.layers[i] = d

    def weight_bytes(self) -> int:
        total = self.w["embed"].numel() * self.w["embed"].element_size() + self.w["head"].numel() * self.w["head"].element_size()
        for d in self.layers.values():
            total += sum(v.numel() * v.element_size() for v in d.values() if isinstance(v, torch.Tensor))
        return total

    def unload(self) -> None:
        self._graphs.clear()
        self._sk = None
        self.w.clear()
        self.layers.clear()
        self.kv.release_all()
        self.kv.k.clear()
        self.kv.v.clear()
        self.slots.tensors.clear()
        self._ws_rows = 0
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------ sequences
    def open_sequence(self) -> int:
        """Admit a sequence: a state slot, which is also its row of the page table.  Pages come with the tokens."""
        slot = self.slots.alloc()
        self.lengths[slot] = 0
        return slot

    def close_sequence(self, slot: int) -> None:
        """Give back the sequence's pages and slot."""
        self.kv.release(slot)
        self.slots.release(slot)
        self.lengths.pop(slot, None)

    # ------------------------------------------------------------------ workspace
    def _workspace(self, rows: int) -> None:
        if rows <= self._ws_rows:
            return
        s, dev, E = self.spec, self.device, self.dtype
        rows = _ceil(rows, 64)
        mx = [L.mixer for L in s.layers]
        n_proj = max(d["w_proj"].shape[0] for d in self.layers.values())
        n_mix = max(m.heads * m.vdim for m in mx)
        n_q = max([m.heads * m.dim for m in mx if m.kind == "attention"] +
                  [m.heads * (max(m.kv_rank, m.dim) + m.rot_dims) for m in mx if m.kind == "latent_attention"] + [1])
        ff = max([max(L.moe.total_ff, L.moe.top * L.moe.ff + L.moe.shared_ff) if L.moe is not None else L.ff
                  for L in s.layers] or [0])
        n_gu = max([d["w_gu"].shape[0] for d in self.layers.values() if "w_gu" in d] or [1])
        f32 = torch.float32
        self._x = torch.empty(rows, s.width, dtype=f32, device=dev)
        self._hn = torch.empty(rows, s.width, dtype=f32, device=dev)
        self._hc = torch.empty(rows, s.width, dtype=E, device=dev)
        self._proj = torch.empty(rows * n_proj, dtype=E, device=dev)
        self._qbuf = torch.empty(rows * n_q, dtype=f32, device=dev)
        self._mix = torch.empty(rows * n_mix, dtype=E, device=dev)
        self._oscr = torch.empty(rows * n_mix, dtype=f32, device=dev)
        self._y = torch.empty(rows, s.width, dtype=E, device=dev)
        self._act = torch.empty(rows * max(ff, 1), dtype=E, device=dev)
        self._gu = torch.empty(rows * max(2 * ff, n_gu, 1), dtype=E, device=dev)
        lat = [m for m in mx if m.kind == "latent_attention"]
        if lat:
            self._cq = torch.empty(rows * max(max(m.q_rank for m in lat), 1), dtype=E, device=dev)
            self._q = torch.empty(rows * max(m.heads * (m.dim + m.rot_dims) for m in lat), dtype=E, device=dev)
            self._olat = torch.empty(rows * max(m.heads * m.kv_rank for m in lat), dtype=E, device=dev)
            # partial sums of the key splits of decode rows (rows * heads * splits <= 16 * SMs + 4 * rows * heads)
            self._apart = torch.empty((16 * self._sms + 64 * max(m.heads for m in lat)) * (max(m.kv_rank for m in lat) + 2),
                                      dtype=f32, device=dev)
        att = [m for m in mx if m.kind == "attention"]
        if att:
            self._apart_att = torch.empty((8 * self._sms + 16 * max(m.heads for m in att)) * (max(m.vdim for m in att) + 2),
                                          dtype=f32, device=dev)
        ssm = [m for m in mx if m.kind in ("mamba2", "delta")]
        if ssm:
            # fp32 outputs of a recurrent mixer's short convolution (x | B | C, or q | k | v)
            self._xbc = torch.empty(rows * max(m.heads * m.vdim + 2 * (m.groups * m.state if m.kind == "mamba2" else
                                                                         m.kv_heads * m.dim) for m in ssm), dtype=f32, device=dev)
        sides = [L.side_dim for L in s.layers if L.side_dim]
        if sides:
            self._sg = torch.empty(rows * max(sides), dtype=E, device=dev)
            self._sa = torch.empty(rows * max(sides), dtype=E, device=dev)
        if any(L.parallel or L.pre_norm for L in s.layers):
            self._he = torch.empty(rows, s.width, dtype=E, device=dev)
            self._y2 = torch.empty(rows, s.width, dtype=E, device=dev)
        if any(L.pre_norm for L in s.layers):
            self._hs = torch.empty(rows, s.width, dtype=f32, device=dev)  # normed rows before the token shift / after the last norm
        if any(L.pre_norm and L.depth_avg for L in s.layers):
            # the embedding output and every layer's result, for the averages after the layers
            self._xs = torch.empty(s.n_layers + 1, rows, s.width, dtype=f32, device=dev)
        moes = [L.moe for L in s.layers if L.moe is not None]
        if moes:
            self._wts = torch.empty(rows * max(e.experts for e in moes), dtype=f32, device=dev)
            self._idw = torch.empty(rows, dtype=f32, device=dev)
            self._sel_idx = torch.empty(rows * max(e.top for e in moes), dtype=torch.int32, device=dev)
            self._sel_w = torch.empty(rows * max(e.top for e in moes), dtype=f32, device=dev)
        if s.loop_passes:
            self._x0 = torch.empty(rows, s.width, dtype=f32, device=dev)
            self._cat = torch.empty(rows, 2 * s.width, dtype=E, device=dev)
        self._hw = torch.empty(max(self.max_batch, 8), s.width, dtype=E, device=dev)
        self._ws_rows = rows
        self._graphs.clear()  # captured graphs hold the old workspace pointers

    def _lin(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = x @ w.T: the framework's bf16 projection (tcgen05 GEMM / weight-streaming GEMV) where its alignment
        rules hold, else the CUDA-core GEMM (float32 engines, odd shapes)."""
        if self.dtype == BF and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.is_contiguous() and \
                not (x.shape[0] > 16 and (x.shape[1] % 64 or w.shape[0] % 16)):  # those would run row by row on the GEMV
            if 2 < x.shape[0] <= 128 and x.shape[1] % 64 == 0 and w.shape[0] % 16 == 0:
                # few rows (batched decode, short portions): the split-K weight stream on every SM, as the uniform
                # stacks' batched decode does
                return ops.linear_splitk(x, w, self._splitk(), out=out)
            return ops.linear(x, w, out=out)
        return ops.linear_any(x, w, out)

    def _splitk(self) -> torch.Tensor:
        """Zero-filled scratch of the split-K projections (self-resetting; calls are ordered on one stream)."""
        if getattr(self, "_sk", None) is None:
            n_max = max([self.w["head"].shape[0], self.spec.width] +
                        [v.shape[0] for d in self.layers.values() for k, v in d.items() if k.startswith("w") and
                         isinstance(v, torch.Tensor) and v.dim() == 2])
            self._sk = torch.zeros(ops.gemm_splitk_scratch_bytes(128, n_max), dtype=torch.uint8, device=self.device)
        return self._sk

    # ------------------------------------------------------------------ one step
    def step(self, batch: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None):
        """batch: [(slot, next tokens)] — every live sequence at most once; want[i]: indices into entry i's tokens
        whose logits are asked for (default: the last one of each entry).  Runs the tokens on top of what earlier
        steps left in the caches and slots and returns the logits [sum(len(want[i])), vocab] (engine dtype, device),
        rows in the order of the entries and of want."""
        s, dev, E = self.spec, self.device, self.dtype
        if want is None:
            want = [[len(t) - 1] for _, t in batch]
        rows = sum(len(t) for _, t in batch)
        if rows == 0:
            return torch.empty(0, s.vocab, dtype=E, device=dev)
        n_ent = len(batch)
        tokens: List[int] = []
        row_ent: List[int] = []
        ent: List[int] = []
        want_rows: List[int] = []
        grew = False
        seen = set()
        for i, (slot, toks) in enumerate(batch):
            if slot not in self.lengths or slot in seen or len(toks) == 0:
                raise ValueError(f"step: slot {slot} is not live, appears twice or brings no tokens")
            seen.add(slot)
            start = self.lengths[slot]
            if start + len(toks) > self.max_seq_len:
                raise ValueError(f"sequence of {start + len(toks)} tokens exceeds max_seq_len {self.max_seq_len}")
            if self.attn_layers:
                grew |= self.kv.reserve(slot, start + len(toks))
            ent += [slot, len(tokens), len(toks), start]
            want_rows += [len(tokens) + int(j) for j in want[i]]
            row_ent += [i] * len(toks)
            tokens += [int(t) for t in toks]
        if grew:
            self.kv.commit()
        self._step_pages = None
        if self.attn_layers:
            used = [p for slot, toks in batch
                    for p in self.kv.owned[slot][:(self.lengths[slot] + len(toks) + self.kv.page_size - 1) // self.kv.page_size]]
            self._step_pages = (min(used), max(used))
        # steps that hold a portion of a prompt run attention in 64-row query tiles on the tensor cores
        tiles: List[int] = []
        if any(len(t) >= self.tc_min_rows for _, t in batch):
            for i, (_, toks) in enumerate(batch):
                for q0 in range(0, len(toks), 64):
                    tiles += [i, q0]
        # one host -> device copy of the step's description: tokens | row_ent | ent | want_rows | tiles (16-byte aligned parts)
        r4, e4, w4 = _ceil(rows, 4), 4 * n_ent, _ceil(max(len(want_rows), 1), 4)
        total = 2 * r4 + e4 + w4 + len(tiles)
        if total > self._meta_cap:
            self._meta_cap = _ceil(total, 1024)
            # a ring of pinned staging buffers: the host may run ahead of the device by several steps, and a buffer
            # is written again only after the copy that read it has finished
            self._meta_ring = [(torch.zeros(self._meta_cap, dtype=torch.int32).pin_memory(), torch.cuda.Event())
                               for _ in range(4)]
            self._meta_turn = 0
            self._meta_dev = torch.zeros(self._meta_cap, dtype=torch.int32, device=dev)
            self._graphs.clear()  # captured graphs hold the old buffer's addresses
        self._meta_turn = (self._meta_turn + 1) % len(self._meta_ring)
        mh, copied = self._meta_ring[self._meta_turn]
        copied.synchronize()
        mh[:rows] = torch.tensor(tokens, dtype=torch.int32)
        mh[r4:r4 + rows] = torch.tensor(row_ent, dtype=torch.int32)
        mh[2 * r4:2 * r4 + e4] = torch.tensor(ent, dtype=torch.int32)
        if want_rows:
            mh[2 * r4 + e4:2 * r4 + e4 + len(want_rows)] = torch.tensor(want_rows, dtype=torch.int32)
        if tiles:
            mh[2 * r4 + e4 + w4:total] = torch.tensor(tiles, dtype=torch.int32)
        md = self._meta_dev
        md[:total].copy_(mh[:total], non_blocking=True)
        copied.record()
        d_tok, d_rent, d_ent = md[:rows], md[r4:r4 + rows], md[2 * r4:2 * r4 + e4]
        d_want = md[2 * r4 + e4:2 * r4 + e4 + len(want_rows)]
        d_tiles = md[2 * r4 + e4 + w4:total]

        self._workspace(rows)
        long_step = any(len(t) >= self.tc_min_rows for _, t in batch)  # a portion of a prompt is in the step
        nw = len(want_rows)
        views = (d_tok, d_rent, d_ent, d_want, d_tiles)
        # a step of single tokens (decode) has the same launches every time: the device buffers of its description sit
        # at fixed addresses per batch size, so it is captured once as a CUDA graph and replayed
        if self.use_cuda_graph and rows == n_ent and self.layer_trace is None:
            logits = self._graphed_forward(rows, n_ent, nw, views)
        else:
            logits = self._forward(rows, n_ent, nw, views, long_step, bool(tiles), None)
        for slot, toks in batch:
            self.lengths[slot] += len(toks)
        if logits is None:
            return torch.empty(0, s.vocab, dtype=E, device=dev)
        return logits[:, :s.vocab]

    def _graphed_forward(self, rows, n_ent, nw, views):
        key = (rows, nw)
        hit = self._graphs.get(key)
        if hit is None:
            # first use: run it (this also sets every kernel's attributes); the capture happens at the second use,
            # because a capture does not execute and the step must advance the caches exactly once
            self._graphs[key] = "warm"
            return self._forward(rows, n_ent, nw, views, False, False, None)
        if hit == "warm":
            out = torch.empty(max(nw, 1), self.w["head"].shape[0], dtype=self.dtype, device=self.device)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            n0 = ops.launch_count
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._forward(rows, n_ent, nw, views, False, False, out)
            self._graphs[key] = hit = (g, out, ops.launch_count - n0)
        g, out, launches = hit
        g.replay()
        ops.launch_count += launches
        return out[:nw].clone() if nw else None

    def _forward(self, rows, n_ent, nw, views, long_step, use_tiles, logits_out):
        """Every kernel of one step, in order; logits_out: where the logits go (a buffer of fixed address under capture)."""
        s, dev, E = self.spec, self.device, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        tiles = use_tiles
        W = s.width
        x, hn, hc = self._x[:rows], self._hn[:rows], self._hc[:rows]
        y = self._y[:rows]
        single = rows == n_ent and s.taps > 1 and self.layer_trace is None  # decode rows: norm + convolution fused

        def enter_sublayer(y_prev, g_post, g_next, tail, taps_w):
            """Close the previous sublayer (x += postnorm(y_prev)) and open the next one: hc = its normed and convolved
            input.  One kernel for decode rows, norm kernel + convolution (+ tail shift) otherwise."""
            if single:
                ops.postnorm_add_norm_conv_single(y_prev, x, tail, taps_w, d_ent, hc, g_post, g_next, s.eps)
                return
            if y_prev is None:
                ops.scalar_rmsnorm(x, g_next, s.eps, hn)
            else:
                ops.postnorm_add_norm(y_prev, x, g_post, s.eps, hn, g_next)
            ops.causal_conv_ragged(hn, tail, taps_w, d_rent, d_ent, hc)  # one tap: no tail, h * (1 + w)

        x0 = self._x0[:rows] if s.loop_passes else None
        # a first layer that reads the residual stream itself gets its GEMM operand from the same kernel
        first_post = s.layers and s.layers[0].post_only and E != torch.float32
        if x0 is None and any(L.pre_norm and L.depth_avg for L in s.layers):
            x0 = self._xs[0][:rows]
        ops.embedding_f32(d_tok, self.w["embed"], x, s.embed_scale, out2=x0, out_e=hc if first_post else None,
                          row_ent=d_rent if s.pos_sinusoid else None, ent=d_ent if s.pos_sinusoid else None,
                          inv_freq=self.w["pos_freq"] if s.pos_sinusoid else None)
        pt = self.kv.page_table
        y_prev, g_prev = None, 1.0
        opened = final_done = False  # pre-norm layers: the previous layer's last kernel already made this one's input / the final norm
        for li, L in enumerate(s.layers):
            P, m = self.layers[s.source(li)], L.mixer
            if L.pre_norm:
                if y_prev is not None:  # close the sequential sublayer before it
                    ops.postnorm_add_norm(y_prev, x, g_prev, s.eps)
                    y_prev = None
                nxt = s.layers[li + 1] if li + 1 < s.n_layers else None
                if nxt is None:
                    follow = ("final", self.w["final_norm"], None, None) if (s.norm_groups == 1 and nw) else (None, None, None, None)
                elif nxt.pre_norm:
                    Pn = self.layers[s.source(li + 1)]
                    follow = ("layer", Pn["norm1"], Pn["shift"], self.slots.tensors.get(("shift", li + 1)))
                else:
                    follow = (None, None, None, None)
                self._pre_norm_layer(li, L, P, rows, n_ent, views, tiles, opened, follow)
                opened, final_done = follow[0] == "layer", follow[0] == "final"
                if self.layer_trace is not None:
                    self.layer_trace.append(x.clone())
                continue
            if L.reenter is not None or L.parallel:
                if y_prev is not None:  # close the sequential sublayer before it
                    ops.postnorm_add_norm(y_prev, x, g_prev, s.eps)
                    y_prev = None
            if L.reenter is not None:
                # a pass of the loop starts from a projection of [x | embedding output] plus the pass's vector
                cat = self._cat[:rows]
                ops.concat_cast(x, x0, cat)
                self._lin(cat, self.w["loop_in"], y)
                ops.rows_bias_f32(y, self.w["loop_step"][L.reenter], x)
            if L.parallel:
                self._parallel_layer(li, L, P, rows, n_ent, views, long_step, tiles)
                if self.layer_trace is not None:
                    self.layer_trace.append(x.clone())
                continue
            if L.post_only:
                if y_prev is not None:
                    ops.postnorm_add_norm(y_prev, x, g_prev, s.eps)
                    y_prev = None
                self._post_only_layer(li, L, P, rows, n_ent, views, long_step, tiles, first=(li == 0))
                if self.layer_trace is not None:
                    self.layer_trace.append(x.clone())
                continue
            enter_sublayer(y_prev, g_prev, P["norm1"], self.slots.tensors.get(("tail1", li)), P.get("canon1"))
            n_proj = P["w_proj"].shape[0]
            proj = self._proj[:rows * n_proj].view(rows, n_proj)
            self._lin(hc, P["w_proj"], proj)
            n_mix = m.heads * m.vdim
            mix = self._mix[:rows * n_mix].view(rows, n_mix)
            off = P["off"]
            if m.kind == "attention":
                self._attention(li, m, P, proj, mix, rows, views, tiles)
            else:
                oscr = self._oscr[:rows * n_mix]
                n_tiles = d_tiles.numel() // 2
                need = ops.mlstm_parallel_scratch_floats(n_tiles, m.heads, m.dim, m.vdim) if tiles and n_tiles > n_ent else 0
                if need and need <= self.mlstm_parallel_max_floats and m.dim <= 224:
                    # some entry spans several 64-position blocks: all blocks in parallel
                    if getattr(self, "_mlstm_scr", None) is None or self._mlstm_scr.numel() < need:
                        self._mlstm_scr = torch.empty(need, dtype=torch.float32, device=dev)
                    ops.mlstm_ragged_parallel(proj, oscr, mix, d_ent, d_tiles, self._mlstm_scr, m.heads, m.dim, m.vdim,
                                              off["q"], off["k"], off["v"], off["i"], off["f"], off["g"], P["i_b"],
                                              P["f_b"], m.gate_cap, P["out_norm"], s.eps, self.slots[("S", li)],
                                              self.slots[("n", li)], self.slots[("m", li)])
                else:
                    ops.mlstm_ragged(proj, oscr, mix, d_ent, m.heads, m.dim, m.vdim, off["q"], off["k"], off["v"], off["i"],
                                     off["f"], off["g"], P["i_b"], P["f_b"], m.gate_cap, P["out_norm"], s.eps,
                                     self.slots[("S", li)], self.slots[("n", li)], self.slots[("m", li)], blocked=long_step)
            self._lin(mix, P["wo"], y)
            g_post = P["norm1b"]
            if L.ff:
                enter_sublayer(y, g_post, P["norm2"], self.slots.tensors.get(("tail2", li)), P.get("canon2"))
                act = self._act[:rows * L.ff].view(rows, L.ff)
                if P["packed"] and 2 < rows <= 128 and W % 64 == 0:
                    ops.linear_splitk_gated_silu(hc, P["w_gu"], self._splitk(), out=act)
                elif P["packed"]:
                    ops.linear_gated_silu(hc, P["w_gu"], out=act)
                else:
                    gu = self._gu[:rows * 2 * L.ff].view(rows, 2 * L.ff)
                    self._lin(hc, P["w_gu"], gu)
                    ops.silu_mul(gu, act)
                self._lin(act, P["w_down"], y)
                g_post = P["norm2b"]
            y_prev, g_prev = y, g_post
            if self.layer_trace is not None:
                # the residual stream after the layer (debugging): close the sublayer now and open the next without it
                ops.postnorm_add_norm(y, x, g_post, s.eps)
                self.layer_trace.append(x.clone())
                y_prev = None
        if s.norm_groups:
            if y_prev is not None:
                ops.postnorm_add_norm(y_prev, x, g_prev, s.eps)
            if nw and not final_done:
                ops.group_rmsnorm(x, self.w["final_norm"], s.norm_groups, s.eps, hn=hn)
        elif y_prev is None:
            ops.scalar_rmsnorm(x, self.w["final_norm"], s.eps, hn)
        else:
            ops.postnorm_add_norm(y_prev, x, g_prev, s.eps, hn, self.w["final_norm"])
        if nw == 0:
            return None
        hw = self._hw[:nw] if nw <= self._hw.shape[0] else torch.empty(nw, W, dtype=E, device=dev)
        ops.gather_cast(self._hs[:rows] if final_done else hn, d_want, hw)
        vp = self.w["head"].shape[0]
        logits = logits_out[:nw] if logits_out is not None else torch.empty(nw, vp, dtype=E, device=dev)
        self._lin(hw, self.w["head"], logits)
        return logits

    # ------------------------------------------------------------------ layers normed on their sublayers' outputs only
    def _operand(self, rows, refresh):
        """The residual stream as a GEMM operand: x itself in a float32 engine, else its copy in the element type (kept
        up to date by the kernels that change x; `refresh` makes it anew after a layer of another style)."""
        x = self._x[:rows]
        if self.dtype == torch.float32:
            return x
        hc = self._hc[:rows]
        if refresh:
            ops.postnorm_vec_add(None, x, None, self.spec.eps, he=hc)
        return hc

    def _post_only_layer(self, li, L, P, rows, n_ent, views, long_step, tiles, first):
        """x += norm1(mixer(x)); x += norm2(ff(x)); x += side_norm(side_proj(gelu(side_gate x) * token's side embedding))."""
        s, E = self.spec, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        x, y = self._x[:rows], self._y[:rows]
        he = None if E == torch.float32 else self._hc[:rows]
        prev_same = s.layers[li - 1].post_only if li > 0 else s.layers[0].reenter is None
        h = self._operand(rows, refresh=not prev_same)
        m = L.mixer
        n_proj = P["w_proj"].shape[0]
        proj = self._proj[:rows * n_proj].view(rows, n_proj)
        self._lin(h, P["w_proj"], proj)
        n_mix = m.heads * m.vdim
        mix = self._mix[:rows * n_mix].view(rows, n_mix)
        off = P["off"]
        if m.kind == "attention":
            self._attention(li, m, P, proj, mix, rows, views, tiles)
        elif m.kind == "latent_attention":
            self._latent_attention(li, m, P, proj, mix, rows, views, tiles)
        elif m.kind == "delta":
            self._delta(li, m, P, proj, mix, rows, views, long_step and self.delta_blocked)
        else:
            raise ValueError(f"layer {li}: mixer {m.kind!r} has no output-normed form")
        self._lin(mix, P["wo"], y)
        ops.postnorm_vec_add(y, x, P["norm1"], s.eps, he=he)
        if L.ff:
            act = self._act[:rows * L.ff].view(rows, L.ff)
            if P["packed"]:
                ops.linear_gated_act(h, P["w_gu"], P["ff_act"], self._splitk() if 2 < rows <= 128 and s.width % 64 == 0 else None,
                                     out=act)
            else:
                n_gu = P["w_gu"].shape[0]
                gu = self._gu[:rows * n_gu].view(rows, n_gu)
                self._lin(h, P["w_gu"], gu)
                ops.moe_act(gu, None, act, 0, 0, 0.0, ff_s=L.ff, limit_s=L.ff_limit, alpha=L.ff_alpha)
            self._lin(act, P["w_down"], y)
            ops.postnorm_vec_add(y, x, P["norm2"], s.eps, he=he)
        if L.side_dim:
            n = L.side_dim
            # the one-kernel form reads both matrices with ONE CTA per row: only where they are small enough for that
            if rows <= self.side_fused_max_rows and (2 * s.width + n) * 4 <= 48 * 1024 and \
                    2 * s.width * n * P["side_gate"].element_size() <= self.side_fused_max_bytes:
                ops.token_side(x, d_tok, self.w["side_embed"], L.side_off, P["side_gate"], P["side_proj"], P["side_norm"],
                               s.eps, he=he)
            else:
                sa = self._sa[:rows * n].view(rows, n)
                if rows <= self.side_fused_max_rows:
                    ops.token_side_gate(x, d_tok, self.w["side_embed"], L.side_off, P["side_gate"], sa)
                else:
                    sg = self._sg[:rows * n].view(rows, n)
                    self._lin(h, P["side_gate"], sg)
                    ops.token_side_act(sg, d_tok, self.w["side_embed"], L.side_off, sa)
                self._lin(sa, P["side_proj"], y)
                ops.postnorm_vec_add(y, x, P["side_norm"], s.eps, he=he)

    # ------------------------------------------------------------------ pre-norm layers with layer scale, shift and average
    def _pre_norm_layer(self, li, L, P, rows, n_ent, views, tiles, opened, follow):
        """x += ls1 * mixer(shift(norm1(x))); x += ls2 * ff(norm2(x)); X_(li+1) = x; x = sum_j dwa[j] X_j.
        Everything between two projections is ONE kernel (ops.layer_close): the scaled residual add, the average and the
        norm that follows — the feed-forward's, the next layer's (follow = ("layer", weights, shift, slot rows)) or the
        model's last one (("final", weights, ..)).  opened: the previous layer's closing kernel already wrote this mixer's
        input.  Steps of one row per entry (decode) also get the next mixer's token shift from that kernel; steps with
        portions of prompts shift the normed rows in a kernel of their own, which needs the previous ROW."""
        s, E = self.spec, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        x, hn, hc, he, y = self._x[:rows], self._hn[:rows], self._hc[:rows], self._he[:rows], self._y[:rows]
        single = rows == n_ent
        m = L.mixer

        def open_mixer(Pm, tail, y_=None, **close):
            """Closing kernel (if any work is left for it) + the norm in front of a mixer + its token shift -> hc."""
            if Pm["shift"] is None:
                ops.layer_close(x, y_, w_next=Pm["norm1"], out_e=hc, eps=s.eps, **close)
            elif single:
                ops.layer_close(x, y_, w_next=Pm["norm1"], shift=Pm["shift"], tail=tail, ent=d_ent, out_e=hc, eps=s.eps, **close)
            else:
                hs = self._hs[:rows]
                ops.layer_close(x, y_, w_next=Pm["norm1"], out_f=hs, eps=s.eps, **close)
                ops.token_shift_ragged(hs, Pm["shift"], tail, d_rent, d_ent, hc)

        if not opened:
            open_mixer(P, self.slots.tensors.get(("shift", li)))
        n_proj = P["w_proj"].shape[0]
        proj = self._proj[:rows * n_proj].view(rows, n_proj)
        self._lin(hc, P["w_proj"], proj)
        n_mix = m.heads * m.vdim
        mix = self._mix[:rows * n_mix].view(rows, n_mix)
        if m.kind != "attention":
            raise ValueError(f"layer {li}: mixer {m.kind!r} has no pre-norm form")
        self._attention(li, m, P, proj, mix, rows, views, tiles)
        self._lin(mix, P["wo"], y)
        close = {"ls": P["ls1"]}
        y_last = y
        if L.ff:
            ops.layer_close(x, y, ls=P["ls1"], w_next=P["norm2"], out_e=he, eps=s.eps)
            act = self._act[:rows * L.ff].view(rows, L.ff)
            if P["packed"] and 2 < rows <= 128 and s.width % 64 == 0:
                ops.linear_splitk_gated_silu(he, P["w_gu"], self._splitk(), out=act)
            elif P["packed"]:
                ops.linear_gated_silu(he, P["w_gu"], out=act)
            else:
                gu = self._gu[:rows * 2 * L.ff].view(rows, 2 * L.ff)
                self._lin(he, P["w_gu"], gu)
                ops.silu_mul(gu, act, bias=P["gu_b"])
            self._lin(act, P["w_down"], y)
            close = {"ls": P["ls2"], "bias": P["down_b"]}
        elif L.moe is not None:
            e = L.moe
            y_last = self._y2[:rows]
            wts = self._wts[:rows * e.experts].view(rows, e.experts)
            idw = self._idw[:rows]
            sel_idx, sel_w = self._sel_idx[:rows * e.top].view(rows, e.top), self._sel_w[:rows * e.top].view(rows, e.top)
            # the kernel that closes the mixer and norms the row also routes it
            ops.layer_close(x, y, ls=P["ls1"], w_next=P["norm2"], out_f=hn, out_e=he, eps=s.eps,
                            route=dict(w_router=P["w_router"], correction=P["corr"], wts=wts, idw=idw, sel_idx=sel_idx, sel_w=sel_w,
                                       n_real=e.experts, top=e.top, groups=e.groups, keep=e.keep, wscale=e.route_scale,
                                       renorm=e.renorm))
            if self._moe_sel_ok(e, rows):
                # decode rows of a sparse enough mixture: stream only the chosen experts' weights
                n_sel = e.top * e.ff + e.shared_ff
                ops.moe_sel(he, P["w_gu"], P["w_down"], sel_idx, sel_w, self._act[:rows * n_sel].view(rows, n_sel), y_last,
                            e.experts, e.top, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha, gated=e.gated)
            else:
                n_gu = P["w_gu"].shape[0]
                gu = self._gu[:rows * n_gu].view(rows, n_gu)
                self._lin(he, P["w_gu"], gu)
                act = self._act[:rows * e.total_ff].view(rows, e.total_ff)
                ops.moe_act(gu, wts, act, e.experts, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha, gated=e.gated)
                self._lin(act, P["w_down"], y_last)
            close = {"ls": P["ls2"]}
            if e.identity:
                close.update(idw=idw, h_in=hn)
        if P["dwa"] is not None:
            close.update(xs=self._xs, n_prev=li + 1, dwa=P["dwa"])
        kind, w_next, shift_next, tail_next = follow
        if kind == "layer":
            open_mixer({"norm1": w_next, "shift": shift_next}, tail_next, y_last, **close)
        elif kind == "final":
            ops.layer_close(x, y_last, w_next=w_next, out_f=self._hs[:rows], eps=s.eps, **close)
        else:
            ops.layer_close(x, y_last, eps=s.eps, **close)

    def _attention(self, li, m, P, proj, mix, rows, views, tiles):
        """Softmax attention over the layer's paged keys and values: prep (head norms, rotation, append), then the
        tensor-core tiles for steps with portions of prompts where the sizes have one, else the row-wise kernel."""
        s, E = self.spec, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        off, pt = P["off"], self.kv.page_table
        kc, vc = self.kv.k[self.kv_index[li]], self.kv.v[self.kv_index[li]]
        cq, sq = self._table(m.rot_base, m.rot_dims, m.rot_scaling) if m.rot_dims else (None, None)
        cv, sv = self._table(m.rot_base, m.vdim, None) if m.rotate_values else (None, None)
        qbuf = self._qbuf[:rows * m.heads * m.dim].view(rows, m.heads * m.dim)
        r1, r2 = P.get("r1"), P.get("r2")
        ops.attn_prep_append(proj, qbuf, kc, vc, d_rent, d_ent, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                             m.rot_dims, off["q"], off["k"], off["v"], P["q_norm"], P["k_norm"], s.eps,
                             cq, sq, cv, sv, bias=P.get("qkv_b"), q_only=m.kv_from is not None)
        if tiles and m.scale > 0 and ops.attn_ragged_tc_supported(m.dim, m.vdim, E):
            ops.attn_ragged_tc(qbuf, kc, vc, proj, mix, d_ent, d_tiles, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                               m.scale, chunk=m.chunk, window=m.window, sink=P["sink"], g_off=off["g"],
                               cos_v=cv, sin_v=sv, first=m.keep_first, r1=r1, r2=r2)
        else:
            # few rows (decode): every row's keys go to several CTAs, so that a long context is read by many SMs; the
            # count depends on the rows alone (a replayed graph keeps it while the contexts grow).  A row never sees more
            # keys than its block or window (plus the kept first positions): no more splits than 32-key pieces of that
            splits = max(1, min(16, (4 * self._sms) // (rows * m.heads))) if rows <= 16 else 1
            span = min([v for v in (m.chunk, m.window) if v > 0] or [0])
            if span:
                splits = max(1, min(splits, (span + m.keep_first + 31) // 32))
            ops.attn_ragged(qbuf, kc, vc, proj, mix, d_rent, d_ent, pt, m.heads, m.kv_heads, m.dim, m.vdim,
                            m.scale, chunk=m.chunk, window=m.window, sink=P["sink"], g_off=off["g"], cos_v=cv,
                            sin_v=sv, first=m.keep_first, splits=splits, part=self._apart_att if splits > 1 else None,
                            r1=r1, r2=r2)

    def _delta(self, li, m, P, proj, mix, rows, views, long_step=False):
        """Gated delta rule: short convolutions and SiLU of q | k | v (fp32), the recurrence over the state slot, then
        the per-head norm, weight and SiLU gate."""
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        off = P["off"]
        C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
        qkv = self._xbc[:rows * C].view(rows, C)
        ops.conv1d_act_ragged(proj, self.slots.tensors.get(("ctail", li)), P["conv_w"], None, d_rent, d_ent, qkv, off["q"],
                              act=1)
        o = self._oscr[:rows * m.heads * m.vdim].view(rows, m.heads * m.vdim)
        ops.delta_rule_ragged(qkv, proj, self.slots[("S", li)], o, d_ent, m.heads, m.kv_heads, m.dim, m.vdim, off["b"],
                              off["a"], P["a_log"], P["dt_bias"], m.scale, m.unit_eps, blocked=long_step)
        ops.head_rmsnorm_gate(o, proj, P["out_norm"], mix, m.heads, m.vdim, self.spec.eps, gate=1, g_off=off["g"])

    # ------------------------------------------------------------------ layers with side-by-side sublayers
    def _parallel_layer(self, li, L, P, rows, n_ent, views, long_step, tiles):
        """h = groupnorm(x); x += mixer(h + conv(h)) + feed-forward(h)."""
        s, E = self.spec, self.dtype
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        x, hn, hc, he, y = self._x[:rows], self._hn[:rows], self._hc[:rows], self._he[:rows], self._y[:rows]
        has_ff = L.moe is not None
        need_hn = has_ff  # the router and the pass-through experts read the normed row in fp32
        if rows == n_ent and s.taps > 1 and s.norm_groups <= 64:
            # decode rows: norm, input convolution and tail shift in one kernel
            ops.group_rmsnorm_conv_single(x, P["norm1"], s.norm_groups, s.eps, self.slots[("tail1", li)], P["canon1"], d_ent,
                                          hc, hn=hn if need_hn else None, he=he if has_ff else None)
        else:
            ops.group_rmsnorm(x, P["norm1"], s.norm_groups, s.eps, hn=hn, he=he if has_ff else None)
            ops.causal_conv_ragged(hn, self.slots.tensors.get(("tail1", li)), P["canon1"], d_rent, d_ent, hc)
        m = L.mixer
        n_proj = P["w_proj"].shape[0]
        proj = self._proj[:rows * n_proj].view(rows, n_proj)
        self._lin(hc, P["w_proj"], proj)
        n_mix = m.heads * m.vdim
        mix = self._mix[:rows * n_mix].view(rows, n_mix)
        if m.kind == "latent_attention":
            self._latent_attention(li, m, P, proj, mix, rows, views, tiles)
        elif m.kind == "mamba2":
            self._mamba2(li, m, P, proj, mix, rows, views, long_step)
        else:
            raise ValueError(f"layer {li}: mixer {m.kind!r} has no side-by-side form")
        self._lin(mix, P["wo"], y)
        if not has_ff:
            ops.residual_add2(x, y)
            return
        e = L.moe
        y2 = self._y2[:rows]
        wts = self._wts[:rows * e.experts].view(rows, e.experts)
        idw = self._idw[:rows]
        ops.moe_route(hn, P["w_router"], P["corr"], wts, idw, self._sel_idx[:rows * e.top].view(rows, e.top),
                      self._sel_w[:rows * e.top].view(rows, e.top), e.experts, e.top)
        if self._moe_sel_ok(e, rows):
            # decode rows of a sparse enough mixture: stream only the chosen experts' weights (and the shared expert's)
            n_sel = e.top * e.ff + e.shared_ff
            ops.moe_sel(he, P["w_gu"], P["w_down"], self._sel_idx[:rows * e.top].view(rows, e.top),
                        self._sel_w[:rows * e.top].view(rows, e.top), self._act[:rows * n_sel].view(rows, n_sel), y2,
                        e.experts, e.top, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha)
            ops.residual_add2(x, y, y2, idw if e.identity else None, hn if e.identity else None)
            return
        n_gu = P["w_gu"].shape[0]
        gu = self._gu[:rows * n_gu].view(rows, n_gu)
        self._lin(he, P["w_gu"], gu)
        act = self._act[:rows * e.total_ff].view(rows, e.total_ff)
        ops.moe_act(gu, wts, act, e.experts, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha)
        self._lin(act, P["w_down"], y2)
        ops.residual_add2(x, y, y2, idw if e.identity else None, hn if e.identity else None)

    def _moe_sel_ok(self, e, rows) -> bool:
        """Do the kernels that stream only the chosen experts' weights pay for a step of `rows` rows?  Every row streams its
        own choice, so their traffic grows with the rows while the all-experts form reads every weight once."""
        total_bytes = e.total_ff * self.spec.width * (3 if e.gated else 2) * 2
        return self.dtype == BF and rows <= self.moe_sel_max_rows and total_bytes >= self.moe_sel_min_bytes and \
            self.moe_sel_share * rows * (e.top * e.ff + e.shared_ff) <= e.total_ff and \
            ops.moe_sel_supported(self.spec.width, e.ff, e.shared_ff, e.top)

    def _latent_attention(self, li, m, P, proj, mix, rows, views, tiles=False):
        """Decode rows and short portions: attention over the cached latents themselves — the heads' key up-projections
        are folded into the queries, the value up-projections applied to the attention output (one shared key/value row
        per position).  Steps with portions of prompts (tiles): the latents of the pages in use are expanded to per-head
        keys and values by one GEMM and attention runs head by head on the tensor-core tiles."""
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        pool = self.kv.k[self.kv_index[li]]
        K, R, H, D, V = m.kv_rank, m.rot_dims, m.heads, m.dim, m.vdim
        cos_t, sin_t = self._table(m.rot_base, R, None) if R else (None, None)
        hv = m.rot_halves
        cq = self._cq[:rows * m.q_rank].view(rows, m.q_rank) if m.q_rank else None
        off = P["off"]
        if m.kv_from is None:
            ops.latent_prep(proj, cq, pool, d_rent, d_ent, self.kv.page_table, m.q_rank, K, R, off["cq"], off["kv"],
                            P.get("q_norm"), P["kv_norm"], self.spec.eps, cos_t, sin_t, halves=hv)
        if m.q_rank:
            q = self._q[:rows * H * (D + R)].view(rows, H * (D + R))
            self._lin(cq, P["w_uq"], q)
        else:
            q = proj[:, :H * (D + R)]  # the queries are the leading columns of the projection
        sink = P.get("sink")
        ps = self.kv.page_size
        if tiles and "w_ukv" in P and m.scale > 0 and self._step_pages is not None and (K + R) % 8 == 0:
            lo, hi = self._step_pages
            n = (hi - lo + 1) * ps
            need = n * H * (2 * D + R + 2 * V)
            if need <= self.latent_expand_max_elems:
                if getattr(self, "_lx", None) is None or self._lx.numel() < need:
                    self._lx = torch.empty(need, dtype=self.dtype, device=self.device)
                kvx = self._lx[:n * H * (D + V)].view(n, H * (D + V))
                kx = self._lx[n * H * (D + V):n * H * (2 * D + R + V)].view(hi - lo + 1, H, ps, D + R)
                vx = self._lx[n * H * (2 * D + R + V):need].view(hi - lo + 1, H, ps, V)
                rows_pool = pool.view(-1, K + R)[lo * ps:(hi + 1) * ps]
                self._lin(rows_pool, P["w_ukv"], kvx)
                ops.latent_expand(kvx, rows_pool, kx, vx, H, D, R, V, K, ps)
                qbuf = self._qbuf[:rows * H * (D + R)].view(rows, H * (D + R))
                ops.latent_q_absorb(q, None, qbuf, d_rent, d_ent, cos_t, sin_t, H, D, R, D, halves=hv)
                ops.attn_ragged_tc(qbuf, kx, vx, None, mix, d_ent, d_tiles, self.kv.page_table, H, H, D + R, V, m.scale,
                                   page_base=lo, sink=sink)
                if m.out_gate:
                    ops.sigmoid_gate(mix, proj, off["g"])
                return
        qbuf = self._qbuf[:rows * H * (K + R)].view(rows, H * (K + R))
        ops.latent_q_absorb(q, P["uk"], qbuf, d_rent, d_ent, cos_t, sin_t, H, D, R, K, halves=hv)
        olat = self._olat[:rows * H * K].view(rows, H * K)
        # few rows (decode): every row's keys go to several CTAs, so that a long context is read by the whole GPU; the
        # count depends on the rows alone (a replayed graph keeps it while the contexts grow)
        # (heads in fours: the shared-key/value kernel gives a CTA four heads of a row)
        splits = max(1, min(64, (4 * self._sms) // (rows * ((H + 3) // 4)))) if rows <= 16 else 1
        part = self._apart if splits > 1 else None
        ops.attn_ragged(qbuf, pool, pool, None, olat, d_rent, d_ent, self.kv.page_table, H, 1, K + R, K, m.scale,
                        ldv=K + R, splits=splits, part=part, sink=sink)
        ops.latent_v_up(olat, P["uv"], proj if m.out_gate else None, mix, H, V, K, g_off=off["g"])

    def _mamba2(self, li, m, P, proj, mix, rows, views, long_step=False):
        d_tok, d_rent, d_ent, d_want, d_tiles = views
        inner, gn = m.heads * m.vdim, m.groups * m.state
        C = inner + 2 * gn
        off = P["off"]
        xbc = self._xbc[:rows * C].view(rows, C)
        ops.conv1d_act_ragged(proj, self.slots.tensors.get(("ctail", li)), P["conv_w"], P["conv_b"], d_rent, d_ent, xbc,
                              off["x"], act=1)
        yss = self._oscr[:rows * inner].view(rows, inner)
        scr, n_tiles = None, d_tiles.numel() // 2
        if long_step and n_tiles > d_ent.numel() // 4 and 2 * (d_ent.numel() // 4) * m.heads <= self._sms:
            # some entry spans several 64-row blocks and one CTA per (entry, head) would leave most SMs idle: all blocks
            # in parallel (bounded scratch, else blocks in order; measured 0.67 vs 0.93 ms at 64 such CTAs, but 1.32 vs
            # 1.04 ms at 128, where the scratch traffic costs more than the idle SMs)
            need = ops.ssm_parallel_scratch_floats(n_tiles, m.heads, m.state, m.vdim)
            if need <= self.mlstm_parallel_max_floats:
                if getattr(self, "_ssm_scr", None) is None or self._ssm_scr.numel() < need:
                    self._ssm_scr = torch.empty(need, dtype=torch.float32, device=self.device)
                scr = self._ssm_scr
        ops.ssm_scan_ragged(xbc, proj, self.slots[("S", li)], yss, d_ent, m.heads, m.vdim, m.state, m.groups, off["dt"],
                            P["dt_bias"], P["a_log"], P["d_skip"], blocked=long_step, tiles=d_tiles if scr is not None else None,
                            scratch=scr)
        ops.gated_group_rmsnorm(yss, proj, P["out_norm"], mix, m.norm_groups, self.spec.eps, off["z"])

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_length: int, do_sample: bool = False, temperature: float = 0.8,
                 top_k: int = 50, top_p: float = 0.95, seed: int = 0, deadline: Optional[float] = None,
                 on_tokens=None, **_):
        """ShardEngine.generate's signature and behaviour (int [B, T] prompts -> int64 [B, <= max_length] on the host, greedy or
        the sampling call), run by the ragged scheduler: prompts go in portions beside the decoding rows."""
        import time as _time

        from .batching import RaggedBatcher
        from .engine import apply_eos, check_max_length

        B, T = input_ids.shape
        check_max_length(T, max_length)
        sched = RaggedBatcher(self, chunk=self.prefill_chunk or 512, temperature=temperature, top_k=top_k, top_p=top_p)
        futs = [sched.submit(input_ids[b], max_length=max_length, do_sample=do_sample, seed=seed + b,
                             timeout=None if deadline is None else max(0.0, deadline - _time.time()))
                for b in range(B)]
        n = 0
        while not all(f.done() for f in futs):
            sched.step()
            n += 1
            if on_tokens is not None and (n & 7) == 0 and B == 1:
                on_tokens(torch.cat((input_ids[0].cpu().long(), torch.tensor(futs[0].request.out, dtype=torch.int64)))[None])
        outs = [f.result() for f in futs]
        width = max(len(o) for o in outs)
        pad = self.pad_token_id if self.pad_token_id is not None else (self.eos_token_ids[0] if self.eos_token_ids else 0)
        out = torch.full((B, width), int(pad), dtype=torch.int64)
        for b, o in enumerate(outs):
            out[b, :len(o)] = o
        new = apply_eos(out[:, T:], tuple(self.eos_token_ids), self.pad_token_id)
        return torch.cat((input_ids.cpu().long(), new), dim=1)
