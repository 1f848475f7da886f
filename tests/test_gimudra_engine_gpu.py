"""The Gimudra design on the ragged engine against the plain float64 oracle (oracle/gimudra_ref.py).

Small made-up configurations with random weights.  The float32 engine must agree with the oracle to ~1e-4 of the
logits' spread at EVERY position — a key one position off at a block's edge, a lost previous row of the token shift, a
depth average over the wrong results, another layer's cache read wrongly, a router group left in or a stale slot changes
logits by orders of magnitude more — whatever the schedule: whole prompts, token-by-token decoding, portions down to
two tokens, mixed batches, small page pools and reused slots.  The bfloat16 engine is held to a bf16-sized bound and to
agreement between schedules.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import gimudra_ref as R  # noqa: E402


def attention(heads=4, kv_heads=2, dim=8, vdim=10, scale=0.5, size=9, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, identity=2, top=2, count=4, keep=2, ff=12, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale,
                       "groups": {"count": count, "keep": keep}}}


def config(layers, width=48, vocab=97, eps=1e-5, scale=3.0):
    out = []
    for L, mlp in layers:
        L = dict(L)
        L["mlp"] = mlp
        out.append(L)
    return {"architecture": "Gimudra", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": out}


def cfg_a():
    """dense, experts in groups, a reader of layer 1's cache with experts, a reader of layer 0's cache without a
    feed-forward, a layer with its own cache, other sizes and another block size, no groups and no pass-through outputs,
    and a reader of that one."""
    return config([(attention(), dense()), (attention(heads=6, kv_heads=2, dim=6, vdim=4, scale=0.4, size=7), moe()),
                   (attention(heads=6, kv_heads=2, dim=6, vdim=4, scale=0.3, size=7, kv_from=1), moe(experts=3, identity=1, top=3, count=2, keep=2, ff=20, scale=0.7)),
                   (attention(size=13, kv_from=0), None),
                   (attention(heads=2, kv_heads=2, dim=12, vdim=16, scale=0.3, size=5), moe(experts=5, identity=0, top=2, count=1, keep=1, ff=8, scale=1.0)),
                   (attention(heads=2, kv_heads=2, dim=12, vdim=16, scale=0.6, size=32, kv_from=4), dense(ff=24))])


def cfg_b():
    """other sizes: one head, blocks of one position and no blocks at all, one group kept of three, top == all outputs of
    the kept group, a single pass-through output, a single expert, odd vocabulary, a width that is no multiple of 16,
    three query heads per key/value head."""
    return config([(attention(heads=1, kv_heads=1, dim=6, vdim=4, scale=0.9, size=1), moe(experts=5, identity=1, top=2, count=3, keep=1, ff=8, scale=2.0)),
                   (attention(heads=3, kv_heads=1, dim=4, vdim=6, scale=0.4, size=0), dense(ff=20)),
                   (attention(heads=3, kv_heads=1, dim=4, vdim=6, scale=0.4, size=3, kv_from=1), moe(experts=1, identity=1, top=1, count=2, keep=2, ff=16, scale=1.0)),
                   (attention(heads=2, kv_heads=2, dim=2, vdim=2, scale=1.0, size=50), None)],
                  width=40, vocab=53, scale=1.0)


def cfg_c():
    """one layer; the average then runs over the embedding output and that layer's result only."""
    return config([(attention(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.35, size=6), moe(experts=4, identity=4, top=3, count=2, keep=1, ff=10))],
                  width=32)


def build(cfg, dtype, seed=0, max_batch=4, max_seq_len=256, pool=None, page_size=4, std=0.15):
    from dli_b200 import gimudra
    from dli_b200.ragged_engine import RaggedEngine

    spec = gimudra.spec_from_config(cfg)
    sd = gimudra.random_state_dict(spec, seed=seed, std=std)
    eng = RaggedEngine(spec, max_batch=max_batch, max_seq_len=max_seq_len, page_size=page_size, kv_pool_tokens=pool,
                       dtype=dtype)
    eng.load_tensors(gimudra.model_tensors(spec, sd))
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


def close16(err, flips=0):
    """bfloat16: nearly every position within the bf16-sized bound and none far from it.  flips: that many positions are
    left out of the second condition — where two experts' choice scores lie within a few thousandths of each other, bf16
    rounding upstream decides the router's choice, and the logits of that one position move by the spread itself."""
    rest = err.flatten().sort().values[:err.numel() - flips] if flips else err
    return bool((err < TOL16).double().mean() >= 0.9 and rest.max() < 0.3)


ALL = [cfg_a, cfg_b, cfg_c]


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
    for cuts in ([19], []):                    # portions take the separate shift kernel, single rows the fused one
        eng.layer_trace = []
        run_schedule(eng, toks, cuts)
        trace = eng.layer_trace
        eng.layer_trace = None
        n = len(cfg["layers"])
        assert len(layers) == n and len(trace) == n * (1 if cuts else 19)
        got = trace if cuts else [torch.cat(trace[i::n]) for i in range(n)]
        for g, ref in zip(got, layers):
            assert (g.double().cpu() - ref).abs().max() < 1e-4 * ref.abs().max()


@pytest.mark.parametrize("make", ALL)
@pytest.mark.parametrize("cuts", [[], [1, 1, 2], [2, 2, 3, 5, 7, 11], [17, 2, 16, 3], [30]])
def test_portions_and_decoding_float32(make, cuts):
    """Token by token from the first token; portions of 2..; a prompt then decoding over page borders and over the edges
    of blocks of 1, 3, 5, 6, 7, 9, 13, 32 and 50 positions."""
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(52, cfg["vocab"], 3)
    assert rel_err(run_schedule(eng, toks, cuts), R.forward(cfg, sd, toks)).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
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
    attention over portions of 16 rows and more on the tensor-core tiles (blocks inside one 64-position tile and across
    tiles, a reader of another layer's cache), the chosen-experts kernels for decode rows and the all-experts form for
    portions, the row-wise kernels for the other steps; all against the oracle and against each other."""
    cfg = config([(attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, size=70), dense(ff=256)),
                  (attention(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, size=20), moe(experts=10, identity=2, top=2, count=4, keep=2, ff=64)),
                  (attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.1, size=100, kv_from=0), moe(experts=12, identity=0, top=2, count=2, keep=1, ff=128)),
                  (attention(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, size=0, kv_from=1), dense(ff=128))],
                 width=128, vocab=200)
    eng, sd = build(cfg, torch.bfloat16, max_seq_len=256, page_size=16, pool=512, std=0.08)
    from dli_b200 import ops
    assert not eng._moe_sel_ok(eng.spec.layers[1].moe, 1)
    eng.moe_sel_min_bytes = 0                     # the engine keeps the chosen-experts kernels for large mixtures; here they run
    assert all(eng._moe_sel_ok(eng.spec.layers[i].moe, 1) and not eng._moe_sel_ok(eng.spec.layers[i].moe, 3) for i in (1, 2))
    assert all(ops.attn_ragged_tc_supported(L.mixer.dim, L.mixer.vdim, torch.bfloat16) for L in eng.spec.layers)
    toks = prompt(230, cfg["vocab"], 6)
    ref = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [230])
    hold = eng.open_sequence()                 # another sequence holds the first pages of the pool meanwhile
    eng.step([(hold, prompt(40, cfg["vocab"], 7))])
    parts = run_schedule(eng, toks, [70, 3, 64, 20, 50])
    eng.close_sequence(hold)
    eng.tc_min_rows = 10 ** 9
    eng.moe_sel_max_rows = 0
    rowwise = run_schedule(eng, toks, [230])
    for got in (whole, parts, rowwise):
        assert close16(rel_err(got, ref), flips=2)
    assert close16(rel_err(whole, rowwise.double()), flips=2)
    # a long portion beside a decoding sequence in one step
    eng.tc_min_rows = 16
    eng.moe_sel_max_rows = 8
    a, b = eng.open_sequence(), eng.open_sequence()
    eng.step([(a, toks[:150])])
    both = eng.step([(a, [toks[150]]), (b, toks[:90])], [[0], list(range(90))]).float().cpu()
    assert rel_err(both[:1], ref[150:151]).max() < 0.3 and close16(rel_err(both[1:], ref[:90]))


@pytest.mark.parametrize("dims", [(128, 64, 128, 256), (64, 128, 64, 64)])
def test_bfloat16_tensor_core_tiles_with_unequal_key_and_value_sizes(dims):
    """The tensor-core tiles whose key and value sizes differ, with a reader of layer 0's cache, in whole prompts, portions
    and token-by-token tails.  The routers' corrections are multiples of 3, so the choice never hangs on bf16 rounding
    (the weights still are the scores) and every position is held to the bound."""
    from dli_b200 import gimudra, ops
    from dli_b200.ragged_engine import RaggedEngine

    d0, v0, d2, v2 = dims
    cfg = config([(attention(heads=2, kv_heads=1, dim=d0, vdim=v0, scale=0.09, size=70), dense(ff=96)),
                  (attention(heads=2, kv_heads=1, dim=d0, vdim=v0, scale=0.09, size=33, kv_from=0), moe(experts=4, identity=0, top=2, count=2, keep=2, ff=32)),
                  (attention(heads=1, kv_heads=1, dim=d2, vdim=v2, scale=0.09, size=100), moe(experts=5, identity=1, top=2, count=3, keep=2, ff=16))],
                 width=64, vocab=200)
    spec = gimudra.spec_from_config(cfg)
    sd = gimudra.random_state_dict(spec, seed=1, std=0.15)
    for k in list(sd):
        if k.endswith("correction"):
            n = sd[k].numel()
            sd[k] = (torch.randperm(n, generator=torch.Generator().manual_seed(n)).float() * 3.0).to(sd[k].dtype)
    eng = RaggedEngine(spec, max_batch=4, max_seq_len=512, page_size=4, dtype=torch.bfloat16)
    eng.load_tensors(gimudra.model_tensors(spec, sd))
    assert all(ops.attn_ragged_tc_supported(L.mixer.dim, L.mixer.vdim, torch.bfloat16) for L in eng.spec.layers)
    toks = prompt(300, cfg["vocab"], 5)
    ref = R.forward(cfg, sd, toks)
    runs = [run_schedule(eng, toks, cuts) for cuts in ([300], [100, 3, 64, 63, 70], [17, 2, 130, 2, 100])]
    for got in runs:
        assert rel_err(got, ref).max() < TOL16
    assert rel_err(runs[1], runs[0].double()).max() < TOL16


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
    oracle; a slot's previous rows of the token shift and its pages must not leak into the next sequence."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=2, pool=64, max_seq_len=64, page_size=4)
    for t in eng.slots.tensors.values():
        t.fill_(1e4)                            # whatever a slot held before
    assert len(eng.slots.tensors) == len(cfg["layers"])
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


def test_a_lost_previous_row_would_show():
    """Shift weights of 1 in layer 0: its mixer then reads ONLY the previous position's normed row, so a row that is not
    carried from step to step (or is carried from the wrong slot) changes every logit."""
    cfg = cfg_c()
    eng, sd = build(cfg, torch.float32)
    sd["l0.shift"] = torch.ones_like(sd["l0.shift"])
    from dli_b200 import gimudra
    eng.load_tensors(gimudra.model_tensors(eng.spec, sd))
    toks = prompt(30, cfg["vocab"], 5)
    ref = R.forward(cfg, sd, toks)
    other = eng.open_sequence()                # a second live sequence whose rows lie in another slot
    eng.step([(other, prompt(6, cfg["vocab"], 8))])
    for cuts in ([30], [], [4, 2, 2, 9]):
        assert rel_err(run_schedule(eng, toks, cuts), ref).max() < TOL32
    eng.close_sequence(other)
    # the oracle itself: with the previous rows taken away the logits differ grossly
    sd0 = dict(sd)
    sd0["l0.shift"] = torch.zeros_like(sd["l0.shift"])
    assert rel_err(R.forward(cfg, sd0, toks), ref).max() > 100 * TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_long_decoding_float32(make):
    """150 tokens one by one: the shift rows are carried 150 times, pages fill and follow, blocks pass over decoded
    tokens."""
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


def test_layers_without_shift_scale_or_average_tensors_run_without_those_steps():
    cfg = cfg_b()
    eng, sd = build(cfg, torch.float32)
    from dli_b200 import gimudra
    for k in ("l0.shift", "l1.ls1", "l1.ls2", "l2.dwa", "l3.shift", "l3.ls1", "l3.dwa"):
        del sd[k]
    eng.load_tensors(gimudra.model_tensors(eng.spec, sd))
    toks = prompt(33, cfg["vocab"], 17)
    ref = R.forward(cfg, sd, toks)
    for cuts in ([33], [5, 2]):
        assert rel_err(run_schedule(eng, toks, cuts), ref).max() < TOL32
