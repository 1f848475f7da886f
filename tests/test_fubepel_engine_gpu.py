"""The Fubepel design on the ragged engine against the plain float64 oracle (oracle/fubepel_ref.py).

Small made-up configurations with random weights.  The float32 engine must agree with the oracle to ~1e-4 of the
logits' spread at EVERY position — a key one position off at a window's edge, a lost recurrent state or convolution
history, a sink left out, another layer's cache read wrongly or a stale slot changes logits by orders of magnitude
more — whatever the schedule: whole prompts, token-by-token decoding, portions down to two tokens, mixed batches,
small page pools and reused slots.  The bfloat16 engine is held to a bf16-sized bound and to agreement between
schedules.  The prompts are ones on which the oracle itself, run in float32, stays within 5e-5 of its float64 run: with
random weights a few prompts have a position where a delta-rule head's read-out nearly cancels before its norm, and
there plain float32 arithmetic is already as far off as the bound.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import fubepel_ref as R  # noqa: E402


def latent(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, scale=0.4, base=1000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def attention(heads=4, kv_heads=2, dim=8, vdim=10, scale=0.5, size=9, keep_first=3):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": size, "keep_first": keep_first}}}


def dense(ff=40, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def config(layers, width=48, vocab=97, eps=1e-5, side=6, scale=3.0):
    out = []
    for L, mlp in layers:
        L = dict(L)
        L["mlp"] = mlp
        out.append(L)
    cfg = {"architecture": "Fubepel", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
           "layers": out}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def cfg_a():
    """latent attention, delta rule, windowed attention, latent attention on layer 0's cache, delta rule without a
    feed-forward, latent attention with a cache of its own."""
    return config([(latent(), dense()), (delta(), dense()), (attention(), dense(ff=24, limit=0.7)),
                   (latent(heads=2, dim=6, vdim=8, kv_from=0), dense()), (delta(heads=2, kv_heads=2, dim=12, vdim=16, conv=4), None),
                   (latent(heads=1, dim=4, rot_dim=6, vdim=10, kv_rank=14, scale=0.6, base=50.0), dense())])


def cfg_b():
    """other sizes: no per-layer token input, one head, a one-tap convolution (no history), a window of one position,
    more kept first positions than the window holds, a rotated part larger than the unrotated one, two layers on the
    cache of a layer that is not the first, key size 40 (two state rows per lane, partly empty), three value columns,
    odd vocabulary, a width that is no multiple of 16."""
    return config([(delta(heads=1, kv_heads=1, dim=40, vdim=3, conv=1), dense(ff=20, limit=5.0)),
                   (latent(heads=1, dim=4, rot_dim=10, vdim=6, kv_rank=12, scale=0.7), None),
                   (attention(heads=1, kv_heads=1, dim=6, vdim=4, scale=0.9, size=1, keep_first=0), dense(ff=8, limit=0.3)),
                   (latent(heads=2, dim=2, rot_dim=10, vdim=2, kv_rank=12, scale=1.0, kv_from=1), None),
                   (attention(heads=6, kv_heads=3, dim=4, vdim=6, scale=0.4, size=3, keep_first=5), None),
                   (latent(heads=3, dim=6, rot_dim=10, vdim=4, kv_rank=12, scale=0.2, kv_from=1), dense(ff=12, limit=2.0))],
                  width=40, vocab=53, side=0, scale=1.0)


def cfg_c():
    """delta-rule layers only (no paged cache at all); a per-layer token input of one channel."""
    return config([(delta(), dense()), (delta(heads=3, kv_heads=1, dim=33, vdim=17, conv=2), None),
                   (delta(heads=2, kv_heads=2, dim=4, vdim=40, conv=5), dense(ff=16, limit=1.0))], width=32, side=1)


def cfg_d():
    """attention layers only: no window at all, a window with nothing kept, a window that keeps many."""
    return config([({"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.35}}, dense()),
                   (attention(size=5, keep_first=0), None), (attention(heads=2, kv_heads=1, size=4, keep_first=11), dense())],
                  width=32, side=5)


def build(cfg, dtype, seed=0, max_batch=4, max_seq_len=256, pool=None, page_size=4, std=0.15):
    from dli_b200 import fubepel
    from dli_b200.ragged_engine import RaggedEngine

    spec = fubepel.spec_from_config(cfg)
    sd = fubepel.random_state_dict(spec, seed=seed, std=std)
    eng = RaggedEngine(spec, max_batch=max_batch, max_seq_len=max_seq_len, page_size=page_size, kv_pool_tokens=pool,
                       dtype=dtype)
    eng.load_tensors(fubepel.model_tensors(spec, sd))
    return eng, sd


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, ref):
    """Per position: RMS of the logit difference (mean removed) over the RMS spread of the reference logits."""
    d = got.double().cpu() - ref
    d = d - d.mean(-1, keepdim=True)
    spread = (ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def run_schedule(eng, toks, cuts):
    """One sequence alone, cut into portions of the given sizes (the rest token by token); logits at every position."""
    slot = eng.open_sequence()
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(eng.step([(slot, toks[at:at + n])], [list(range(n))]).float().cpu())
        at += n
    eng.close_sequence(slot)
    return torch.cat(out)


TOL32, TOL16 = 2e-4, 0.08


def close16(err):
    """bfloat16: nearly every position within the bf16-sized bound and none far from it (the output norms give every
    sublayer's rounding the same weight in the residual stream, whatever the sublayer's own scale)."""
    return bool((err < TOL16).double().mean() >= 0.9 and err.max() < 0.25)

ALL = [cfg_a, cfg_b, cfg_c, cfg_d]


@pytest.mark.parametrize("make", ALL)
def test_whole_prompt_float32_matches_oracle_at_every_position(make):
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(45, cfg["vocab"], 12)
    assert rel_err(run_schedule(eng, toks, [45]), R.forward(cfg, sd, toks)).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_residual_stream_after_every_layer(make):
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(19, cfg["vocab"], 2)
    layers = []
    R.forward(cfg, sd, toks, layers)
    eng.layer_trace = []
    run_schedule(eng, toks, [19])
    assert len(eng.layer_trace) == len(layers) == len(cfg["layers"])
    for got, ref in zip(eng.layer_trace, layers):
        assert (got.double().cpu() - ref).abs().max() < 1e-4 * ref.abs().max()


@pytest.mark.parametrize("make", ALL)
@pytest.mark.parametrize("cuts", [[], [1, 1, 2], [2, 2, 3, 5, 7, 11], [17, 2, 16, 3], [30]])
def test_portions_and_decoding_float32(make, cuts):
    """Token by token from the first token; portions of 2..; a prompt then decoding over page borders and past the
    windows (9, 5, 4, 3 and 1 positions) and the kept first positions."""
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(52, cfg["vocab"], 3)
    assert rel_err(run_schedule(eng, toks, cuts), R.forward(cfg, sd, toks)).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_d])
def test_bfloat16_engine_is_close_and_schedules_agree(make):
    cfg = make()
    eng, sd = build(cfg, torch.bfloat16)
    toks = prompt(40, cfg["vocab"], 4)
    ref = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [40])
    parts = run_schedule(eng, toks, [7, 2, 9, 3])
    assert close16(rel_err(whole, ref))
    assert close16(rel_err(parts, ref))
    assert close16(rel_err(parts, whole.double()))


def test_bfloat16_sizes_of_the_tensor_core_kernels():
    """Widths and sizes in multiples of 64 / 128: projections on the tensor-core GEMMs and the split-K weight stream,
    windowed and latent attention over portions of 16 rows and more on the tensor-core attention tiles (window and kept
    first positions inside one 64-position tile, across tiles, and tiles of kept positions far below the window), the
    row-wise kernels for the other steps; all against the oracle and against each other."""
    cfg = config([(latent(heads=4, dim=32, rot_dim=32, vdim=64, kv_rank=64, scale=0.125), dense(ff=256)),
                  (delta(heads=4, kv_heads=2, dim=64, vdim=32, conv=4), dense(ff=128)),
                  (attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=70, keep_first=5), dense(ff=128)),
                  (latent(heads=2, dim=96, rot_dim=32, vdim=128, kv_rank=64, scale=0.09, kv_from=0), None),
                  (attention(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, size=20, keep_first=70), dense(ff=128))],
                 width=128, vocab=200, side=16)
    eng, sd = build(cfg, torch.bfloat16, max_seq_len=256, page_size=16, pool=512)
    assert "w_ukv" in eng.layers[0] and "w_ukv" in eng.layers[3]
    toks = prompt(230, cfg["vocab"], 6)
    ref = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [230])
    hold = eng.open_sequence()                 # another sequence holds the first pages of the pool meanwhile
    eng.step([(hold, prompt(40, cfg["vocab"], 7))])
    parts = run_schedule(eng, toks, [70, 3, 64, 20, 50])
    eng.close_sequence(hold)
    eng.tc_min_rows = 10 ** 9
    rowwise = run_schedule(eng, toks, [230])
    for got in (whole, parts, rowwise):
        assert close16(rel_err(got, ref))
    assert close16(rel_err(whole, rowwise.double()))
    # a long portion beside a decoding sequence in one step
    eng.tc_min_rows = 16
    a, b = eng.open_sequence(), eng.open_sequence()
    eng.step([(a, toks[:150])])
    both = eng.step([(a, [toks[150]]), (b, toks[:90])], [[0], list(range(90))]).float().cpu()
    assert rel_err(both[:1], ref[150:151]).max() < 0.25 and close16(rel_err(both[1:], ref[:90]))


def test_mixed_batches_of_unequal_requests_match_each_alone():
    """Four requests of different lengths move through shared steps in portions of different sizes, some decoding
    while others are in their prompt, some skipping steps; each position equals the oracle's for that request alone."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, pool=160, max_seq_len=160)
    lens = [37, 9, 58, 1]
    reqs = [prompt(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    refs = [R.forward(cfg, sd, t) for t in reqs]
    slots = [eng.open_sequence() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    pattern = [[5, 2, 9, 1], [1, 0, 16, 0], [3, 1, 1, 0], [0, 3, 2, 0], [8, 1, 7, 0], [1, 1, 1, 0], [19, 1, 22, 0]]
    k = 0
    while any(a < n for a, n in zip(at, lens)):
        sizes = pattern[k % len(pattern)]
        k += 1
        batch, want, who = [], [], []
        for i, n in enumerate(sizes):
            n = min(n, lens[i] - at[i])
            if n > 0:
                batch.append((slots[i], reqs[i][at[i]:at[i] + n]))
                want.append(list(range(n)))
                who.append((i, n))
        if not batch:
            continue
        lg = eng.step(batch, want).float().cpu()
        o = 0
        for i, n in who:
            got[i].append(lg[o:o + n])
            o += n
            at[i] += n
    for i in range(len(reqs)):
        assert rel_err(torch.cat(got[i]), refs[i]).max() < TOL32, f"request {i}"


def test_pages_and_slots_are_used_again():
    """A pool that holds two sequences at most and two slots: six sequences pass through in turn, each against the
    oracle; a slot's previous state (delta-rule state, convolution histories, pages) must not leak into the next one."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=2, pool=64, max_seq_len=64, page_size=4)
    for t in eng.slots.tensors.values():
        t.fill_(1e4)                            # whatever a slot held before
    for r in range(3):
        ta, tb = prompt(29 + r, cfg["vocab"], 20 + r), prompt(11 + 2 * r, cfg["vocab"], 30 + r)
        ra, rb = R.forward(cfg, sd, ta), R.forward(cfg, sd, tb)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        la = [eng.step([(sa, ta[:13])], [list(range(13))])]
        both = eng.step([(sa, ta[13:]), (sb, tb)], [list(range(len(ta) - 13)), list(range(len(tb)))])
        la.append(both[:len(ta) - 13])
        assert rel_err(torch.cat(la), ra).max() < TOL32
        assert rel_err(both[len(ta) - 13:], rb).max() < TOL32
        eng.close_sequence(sb if r % 2 else sa)   # give the slots back in changing order
        eng.close_sequence(sa if r % 2 else sb)
    assert len(eng.kv.free) == eng.kv.num_pages and len(eng.slots.free) == 2


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_long_decoding_float32(make):
    """150 tokens one by one: the state is carried 150 times, pages fill and follow, windows pass over decoded tokens."""
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(150, cfg["vocab"], 11)
    assert rel_err(run_schedule(eng, toks, [3]), R.forward(cfg, sd, toks)).max() < TOL32


def test_greedy_generation_through_the_scheduler():
    """generate() -> RaggedBatcher -> step(): three prompts of one length share steps; tokens equal the oracle's greedy
    continuation (float32 engine: no near-ties at these sizes)."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=3)
    eng.prefill_chunk = 8   # prompts go in portions of at most 8 tokens per step, shared between the requests
    ids = torch.tensor([prompt(13, cfg["vocab"], 40 + i) for i in range(3)])
    out = eng.generate(ids, max_length=13 + 5)
    for b in range(3):
        assert out[b].tolist() == R.greedy(cfg, sd, ids[b].tolist(), 5)
    assert len(eng.slots.free) == 3 and len(eng.kv.free) == eng.kv.num_pages


def test_decode_steps_replayed_as_a_graph_equal_eager_steps():
    """Steps of single tokens are captured once per batch size and replayed; the logits equal the eager launches' bit
    for bit, also when the batch size changes and a sequence leaves in between."""
    cfg = cfg_a()
    outs = []
    for graph in (True, False):
        eng, sd = build(cfg, torch.float32, max_batch=3)
        eng.use_cuda_graph = graph
        seqs = [prompt(30, cfg["vocab"], 60 + i) for i in range(3)]
        slots = [eng.open_sequence() for _ in seqs]
        got = [eng.step([(slots[i], seqs[i][:9]) for i in range(3)])]
        for t in range(9, 20):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in range(3)]))
        eng.close_sequence(slots[1])
        for t in range(20, 30):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in (0, 2)]))
        outs.append(torch.cat([g.float().cpu() for g in got]))
        if graph:
            assert any(isinstance(v, tuple) for v in eng._graphs.values())
    assert torch.equal(outs[0], outs[1])


def test_delta_rule_in_blocks_of_16_rows_through_the_engine():
    """The engine's switch for portions of prompts: the block form against the oracle, in portions that end anywhere."""
    cfg = cfg_c()
    eng, sd = build(cfg, torch.float32)
    eng.delta_blocked = True
    toks = prompt(52, cfg["vocab"], 3)
    assert rel_err(run_schedule(eng, toks, [17, 2, 16, 3]), R.forward(cfg, sd, toks)).max() < TOL32


def test_per_layer_token_input_in_one_kernel_equals_its_separate_steps():
    """Few rows take the fused kernel, more rows two projections around the activation; both against the oracle."""
    cfg = cfg_a()
    toks = prompt(24, cfg["vocab"], 9)
    outs = []
    for fused_rows in (0, 10 ** 9):
        eng, sd = build(cfg, torch.float32)
        eng.side_fused_max_rows = fused_rows
        outs.append(run_schedule(eng, toks, [12, 5]))
    ref = R.forward(cfg, sd, toks)
    assert rel_err(outs[0], ref).max() < TOL32 and rel_err(outs[1], ref).max() < TOL32
