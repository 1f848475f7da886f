#!/usr/bin/env python
"""Benchmark of the one hot path: the worker's (sharded) decoder forward.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one decode step: one new token for
every sequence of the batch, with the KV cache already holding `ctx` tokens.

N = 1 : config[2] of BASELINE.json — Llama-3-8B shape, bf16, random-init weights,
        batch 1, 2k-token context, paged KV (the north-star target).  Also reports
        the 2k-token prefill and (extra) batch-32 decode.
N > 1 : the same model split into N contiguous layer ranges (reference sharder
        formula), one stage per GPU; decode hands hidden states, head candidates and
        tokens over in per-tick mailboxes (one NCCL all-gather per tick, issued on its
        own stream under the next tick's kernels), 2(N+1) micro-batch slots of `batch`
        sequences in flight so that every stage works every tick (weak scaling: per-GPU
        batch fixed, per-GPU weights shrink).  Before timing, rank 0 checks the
        pipeline's first tokens against the single-GPU engine on the same weights and
        the run aborts on a mismatch (extra.parity_check); extra.named_config runs the
        BASELINE.json configuration that is stated for exactly N GPUs.

value  : decode tokens/s with everything resident in HBM (CUDA-graph replay).
e2e    : the same metric through the plugin call the reference's master makes
         (reference worker/app.py:254-330 `run_inference`): POST /inference on the
         drop-in Worker (werkzeug test client, no socket) with the 2k-token prompt as
         host text -> tokenise -> host->device copy -> prefill -> K decode steps ->
         device->host copy of the tokens -> decode to text -> JSON.  Decode rate =
         K / (t[request with K+1 new tokens] - t[request with 1 new token]); the whole
         request's seconds are reported beside it.
extra.hf_gpu : transformers' own generate (bf16, sdpa) on the same GPU and shape — the only
         existing GPU implementation of this path (what the reference runs with USE_GPU=1).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


from dli_b200.measure import ClockSampler, decode_step_bytes, prefill_flops  # noqa: E402


def ev_time_ms(fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


# ---------------------------------------------------------------------------------- ours, 1 GPU
def run_single(args, spec, peaks):
    from dli_b200 import ops
    from dli_b200.engine import ShardEngine

    B, ctx, K, W = args.batch, args.ctx, args.steps, args.warmup
    max_len = ctx + 2 * (K + W) + 16
    eng = ShardEngine(spec, max_batch=B, max_seq_len=max_len, page_size=args.page_size)
    eng.load_random(seed=0)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, spec.vocab, (B, ctx), generator=g, dtype=torch.int32).pin_memory()

    # ---- prefill (also fills the KV cache with `ctx` tokens per sequence) -----------------
    def do_prefill():
        eng.start_batch(B, ctx, max_len)
        ids = prompt.to("cuda", non_blocking=True).reshape(-1)
        eng.prefill(B, ctx, ids=ids)

    do_prefill()  # warm-up (function attributes, workspace)
    pf_ms = min(ev_time_ms(do_prefill) for _ in range(2))
    pf_flops = prefill_flops(spec, B, ctx)

    # ---- decode, device-resident -------------------------------------------------------------
    for _ in range(max(W, 3)):
        eng.decode_step(B)
    torch.cuda.synchronize()
    n0 = ops.launch_count
    with ClockSampler() as clk:
        ms = ev_time_ms(lambda: [eng.decode_step(B) for _ in range(K)])
    launches = ops.launch_count - n0
    ms_step = ms / K
    S_mid = ctx + max(W, 3) + K // 2
    step_bytes = decode_step_bytes(spec, spec.n_layers, True, B, S_mid)
    value = B * K / (ms / 1e3)

    # ---- decode through the plugin call (POST /inference on the drop-in worker) ---------------
    if B == 1:
        e2e = e2e_through_worker(eng, prompt[0], ctx, K)
    else:  # the worker serves one prompt per request: larger batches go through the per-step host call
        e2e = e2e_step_host(eng, B, K)

    # ---- dominant kernel: the gate/up weight-streaming projection ----------------------------
    roof = dominant_kernel_roofline(eng, spec, B, peaks)
    roof_step = {"bound": "hbm", "achieved": step_bytes / (ms_step / 1e3) / 1e9, "peak": peaks["hbm_gbs"],
                 "unit": "GB/s", "frac": step_bytes / (ms_step / 1e3) / 1e9 / peaks["hbm_gbs"],
                 "bytes_per_step": step_bytes, "frac_of_nominal_8TBps": step_bytes / (ms_step / 1e3) / 8e12}

    extra = {
        "prefill_tokens_per_s": B * ctx / (pf_ms / 1e3), "prefill_ms": pf_ms,
        "prefill_roofline": {"bound": "tensor", "achieved": pf_flops / (pf_ms / 1e3) / 1e12,
                             "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                             "frac": pf_flops / (pf_ms / 1e3) / 1e12 / peaks["bf16_tflops"]},
        "roofline_step": roof_step, "attn_splits": eng._state(B)["splits"],
        "weights_gb": eng.weight_bytes() / 1e9, "peaks": peaks["source"],
    }
    extra["env"] = {k: v for k, v in os.environ.items() if k.startswith("DLI_")}  # knobs that change the measured path
    if args.batch == 1 and not args.no_extra:
        try:
            extra["decode_b32"] = batch_decode_extra(spec, 32, ctx, min(K, 32), peaks, args.page_size, eng)
        except Exception as e:  # noqa: BLE001
            extra["decode_b32"] = {"error": str(e)[:200]}
    if not args.no_extra:
        eng_w, eng_layers = eng.w, eng.layers
        try:
            eng.w, eng.layers = {}, []
            eng.unload()  # frees KV and workspaces; the weights go with the references below
            del eng_w, eng_layers
            torch.cuda.empty_cache()
            extra["hf_gpu"] = hf_gpu_comparator(spec, ctx)
            extra["hf_gpu"]["ours_over_hf_decode"] = value / extra["hf_gpu"]["decode_tokens_per_s"]
        except Exception as e:  # noqa: BLE001
            extra["hf_gpu"] = {"error": str(e)[:300]}
    return {"value": value, "ms_per_step": ms_step, "e2e": e2e, "roofline": roof, "gpu_launches": launches,
            "clocks": clk.summary(), "extra": extra,
            "config": {"workload": f"{args.model} bf16 random-init, 1 GPU, batch {B} greedy decode at {ctx}-token context, "
                                   f"paged KV (page {args.page_size}); BASELINE.json configs[2]",
                       "batch": B, "ctx": ctx, "page_size": args.page_size, "parallelism": "1 stage",
                       "l2": f"inputs larger than L2: {step_bytes / 1e9:.2f} GB streamed per step vs 126 MB L2"}}


def e2e_step_host(eng, B, K):
    """Batch > 1: one decode step per call with HOST buffers (pinned tokens in, tokens out, sync per step)."""
    t_in = torch.zeros(B, dtype=torch.int32).pin_memory()
    t_out = torch.zeros(B, dtype=torch.int32).pin_memory()
    t_in.copy_(eng._state(B)["tokens"].cpu())
    for _ in range(3):
        eng.decode_step_host(t_in, t_out)
        t_in.copy_(t_out)

    def host_loop():
        for _ in range(K):
            eng.decode_step_host(t_in, t_out)
            t_in.copy_(t_out)

    e2e_ms = ev_time_ms(host_loop)
    return {"value": B * K / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B,
            "ms_per_step": e2e_ms / K, "api": "ShardEngine.decode_step_host"}


def e2e_through_worker(eng, prompt_row, ctx, K):
    """The reference-facing plugin call: the drop-in Worker's POST /inference (worker.py, the route the
    reference master posts to: master/dashboard/views.py:345-355, :412-421), greedy.  The engine already
    holds the weights (the load routes are not part of the per-request path); everything a request does
    — JSON, tokenising the prompt text, the host->device copy of the ids, prefill, K decode steps, the
    device->host copy of the tokens, decoding to text — is inside the timed region."""
    from werkzeug.test import Client

    from dli_b200.worker import IdTokenizer, Worker

    w = Worker(env={"MODEL_CACHE_DIR": "/nonexistent", "USE_GPU": "1", "DLI_MAX_SEQ_LEN": str(eng.max_seq_len)})
    w.loaded_models["bench"] = eng
    w.loaded_tokenizers["bench"] = IdTokenizer()
    client = Client(w)
    text = " ".join(str(int(t)) for t in prompt_row)

    def request(n_new):
        t0 = time.perf_counter()
        r = client.post("/inference", json={"model_name": "bench", "prompt": text, "max_length": ctx + n_new,
                                            "do_sample": False, "timeout": 600})
        dt = time.perf_counter() - t0
        body = r.get_json()
        if r.status_code != 200 or body.get("status") != "success":
            raise RuntimeError(f"/inference failed: {r.status_code} {body}")
        n_out = len(body["result"].split())
        if n_out != ctx + n_new:
            raise RuntimeError(f"/inference returned {n_out} tokens, expected {ctx + n_new}")
        return dt

    request(1), request(K + 1)  # warm-up: graph capture for this state, allocator
    t_first = min(request(1) for _ in range(3))
    t_full = min(request(K + 1) for _ in range(2))
    dec = max(t_full - t_first, 1e-9)
    return {"value": K / dec, "unit": UNIT, "h2d_bytes_per_step": 4.0 * ctx / K, "d2h_bytes_per_step": 4.0 * (K + 1) / K,
            "ms_per_step": dec / K * 1e3, "api": "Worker.inference (POST /inference, werkzeug test client)",
            "request_s": t_full, "request_new_tokens": K + 1, "request_tokens_per_s": (K + 1) / t_full,
            "prefill_request_s": t_first, "prompt_tokens": ctx,
            "note": "value = K decode steps / (request with K+1 new tokens - request with 1 new token), both "
                    "timed on the host clock around the HTTP handler; h2d = the int32 prompt ids amortised over K"}


def hf_gpu_comparator(spec, ctx, n_new=32):
    """transformers generate (bf16, sdpa, greedy) on this GPU at the same shape: the stock-PyTorch GPU
    comparator BASELINE.md 5 names — what the reference's worker runs with USE_GPU=1
    (reference worker/app.py:23-26,121-124,297-305) on a torch that supports the B200."""
    import gc

    import transformers

    kw = dict(vocab_size=spec.vocab, hidden_size=spec.d_model, intermediate_size=spec.d_ff,
              num_hidden_layers=spec.n_layers, num_attention_heads=spec.n_heads, num_key_value_heads=spec.n_kv_heads,
              head_dim=spec.head_dim, max_position_embeddings=max(spec.max_pos, ctx + n_new + 8), rms_norm_eps=spec.eps,
              tie_word_embeddings=spec.tie_embeddings, rope_parameters={"rope_type": "default", "rope_theta": spec.rope_theta})
    cfg = (transformers.MistralConfig(sliding_window=spec.sliding_window, **kw) if spec.sliding_window
           else transformers.LlamaConfig(**kw))
    with torch.device("cuda"):
        m = transformers.AutoModelForCausalLM.from_config(cfg, dtype=torch.bfloat16).eval()
    ids = torch.randint(0, spec.vocab, (1, ctx), generator=torch.Generator().manual_seed(1)).cuda()
    mask = torch.ones_like(ids)

    def gen(n):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.no_grad():
            m.generate(ids, attention_mask=mask, max_new_tokens=n, min_new_tokens=n, do_sample=False, pad_token_id=0)
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    gen(2)
    t1 = min(gen(1) for _ in range(2))
    t2 = min(gen(1 + n_new) for _ in range(2))
    out = {"decode_tokens_per_s": n_new / max(t2 - t1, 1e-9), "prefill_tokens_per_s": ctx / t1, "ms_per_step": (t2 - t1) / n_new * 1e3,
           "impl": f"transformers {transformers.__version__} generate, bf16, attn_implementation={m.config._attn_implementation}, "
                   f"torch {torch.__version__}", "sample": f"batch 1, {ctx}-token prompt, {n_new} decode steps"}
    del m
    gc.collect()
    torch.cuda.empty_cache()
    return out


def dominant_kernel_roofline(eng, spec, B, peaks):
    """Time the dominant decode kernel alone with CUDA events on its stream: the gated
    gate/up projection of every layer back to back (each launch reads a different
    layer's 2*d*ff*2 bytes, so nothing is L2-resident)."""
    from dli_b200 import ops

    x = torch.randn(B, spec.d_model, device="cuda").to(torch.bfloat16)
    out = torch.empty(B, spec.d_ff, device="cuda", dtype=torch.bfloat16)
    ws = [L["wgu"] for L in eng.layers]

    def loop():
        for w in ws:
            ops.linear_gated_silu(x, w, out=out)

    loop()
    ms = min(ev_time_ms(loop) for _ in range(3)) / len(ws)
    nbytes = 2 * spec.d_ff * spec.d_model * 2
    ach = nbytes / (ms / 1e3) / 1e9
    # dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of this kernel from an `ncu --set full` capture
    # (profiles/): a recorded measurement, not taken in this run — the capture's tree is named beside it
    traffic, traffic_src = None, None
    tp = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    if os.path.exists(tp):
        rec = json.load(open(tp))
        traffic = rec.get("gate_up_projection_dram_bytes_per_launch")
        traffic_src = rec.get("source")
    return {"bound": "hbm", "kernel": "gemv_kernel<M,gated> (gate/up projection)" if B <= 4 else
            "gemm_tcgen05_kernel<swap,gated> (gate/up projection)", "achieved": ach, "peak": peaks["hbm_gbs"],
            "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": traffic, "traffic_source": traffic_src,
            "bytes_per_launch": nbytes,
            "us_per_launch": ms * 1e3, "peak_source": peaks["source"]}


def batch_decode_extra(spec, B, ctx, K, peaks, page_size, old_eng):
    """Extra (not the headline): batch-32 decode at the same context."""
    from dli_b200.engine import ShardEngine

    max_len = ctx + 3 * K + 16
    eng = ShardEngine(spec, max_batch=B, max_seq_len=max_len, page_size=page_size)
    eng.w, eng.layers = old_eng.w, old_eng.layers  # share the weights already in HBM
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, spec.vocab, (B * ctx,), generator=g, dtype=torch.int32).cuda()
    eng.start_batch(B, ctx, max_len)
    pf_ms = ev_time_ms(lambda: eng.prefill(B, ctx, ids=ids))
    for _ in range(3):
        eng.decode_step(B)
    runs = [ev_time_ms(lambda: [eng.decode_step(B) for _ in range(K)]) / K for _ in range(3)]
    ms = statistics.median(runs)
    nbytes = decode_step_bytes(spec, spec.n_layers, True, B, ctx + 3 + 3 * K // 2)
    out = {"tokens_per_s": B / (ms / 1e3), "ms_per_step": ms, "ms_per_step_runs": runs,
           "hbm_frac": nbytes / (ms / 1e3) / 1e9 / peaks["hbm_gbs"],
           "bytes_per_step": nbytes, "prefill_tokens_per_s": B * ctx / (pf_ms / 1e3),
           "prefill_tensor_frac": prefill_flops(spec, B, ctx) / (pf_ms / 1e3) / 1e12 / peaks["bf16_tflops_sustained"]}
    eng.w, eng.layers = {}, []
    eng.unload()
    return out


# ---------------------------------------------------------------------------------- CPU baseline
def _use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 for multi-process launches; the CPU arm is meant to use
    every host core this process may run on."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if os.environ.get("OMP_NUM_THREADS") and torch.get_num_threads() < n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_baseline(spec, args, new_tokens=4, prompt_len=16):
    from oracle import ref_worker_port as P

    _use_all_host_threads()
    t0 = time.time()
    r = P.time_cpu_decode(spec, prompt_len, new_tokens, greedy=True, warmup_tokens=0)
    out = {"value": r["decode_tok_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
           "sample": r["sample"] + f" (transformers generate, the reference's worker/app.py path with USE_GPU=0); "
                                   f"host cpu_count={os.cpu_count()}", "wall_s": time.time() - t0,
           "prefill_tok_s": r["prefill_tok_s"]}
    try:
        out["configs0"] = cpu_configs0()
    except Exception as e:  # noqa: BLE001
        out["configs0"] = {"error": str(e)[:200]}
    return out


def cpu_configs0():
    """BASELINE.json configs[0]: GPT-2 small (124M) random-init, fp32 (the reference's default load dtype,
    worker/app.py:121), USE_GPU=0, 32-token prompt -> 64 new tokens (max_length 96) through the port of the
    reference's /inference body — greedy (the parity mode) and with the reference's own sampling call."""
    from dli_b200.engine import NAMED_SPECS
    from oracle import ref_worker_port as P

    spec = NAMED_SPECS["gpt2"]
    model = P.build_cpu_model(spec, dtype=torch.float32)
    greedy = P.time_cpu_decode(spec, 32, 64, dtype=torch.float32, greedy=True, model=model, warmup_tokens=1)
    sampled = P.time_cpu_decode(spec, 32, 64, dtype=torch.float32, greedy=False, model=model, warmup_tokens=0)
    return {"workload": "GPT-2 small fp32 random-init, 1 worker, 1 shard, USE_GPU=0, 32-token prompt -> 64 tokens",
            "cores": greedy["threads"], "kind": "port",
            "greedy": {"request_s": greedy["t_total_s"], "tokens_per_s": 64 / greedy["t_total_s"],
                       "decode_tokens_per_s": greedy["decode_tok_s"]},
            "reference_sampling": {"request_s": sampled["t_total_s"], "tokens_per_s": 64 / sampled["t_total_s"],
                                   "decode_tokens_per_s": sampled["decode_tok_s"]}}


def run_reference(args, spec):
    """--impl reference: the reference's CPU path (port, see oracle/ref_worker_port.py),
    all host threads, each step = one decoded token at the product arm's context (batch 1, `--ctx` tokens), decode
    rate = K tokens / (t[K+1 new tokens] - t[1 new token])."""
    from oracle import ref_worker_port as P

    _use_all_host_threads()
    model = P.build_cpu_model(spec)
    tok = P.IdTokenizer()
    K, W = min(args.steps, 64), min(args.warmup, 2)  # bounded: ~0.12 s per token on the box's 16 cores
    # the product arm's context (DLI_REF_CTX bounds it: the prompt pass of an 8B model costs the host cores ~10-20 s
    # per call and the arm makes two of them)
    prompt_len = max(1, min(int(os.environ.get("DLI_REF_CTX", args.ctx)), spec.max_pos - K - 2))
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, spec.vocab, (prompt_len,), generator=g)
    prompt = " ".join(str(int(i)) for i in ids)
    if W:  # warm-up on a short prompt: thread pool, allocator, first-call costs
        short = " ".join(str(int(i)) for i in ids[:16])
        P.run_inference_port(model, tok, short, min(16, prompt_len) + 1 + W, timeout=1e9, greedy=True)
    t0 = time.time()
    P.run_inference_port(model, tok, prompt, prompt_len + 1, timeout=1e9, greedy=True)
    t_pf = time.time() - t0
    t0 = time.time()
    P.run_inference_port(model, tok, prompt, prompt_len + 1 + K, timeout=1e9, greedy=True)
    dt = max(time.time() - t0 - t_pf, 1e-9)
    v = K / dt
    sample = (f"{args.model} bf16 on CPU via transformers generate (reference worker/app.py path, USE_GPU=0), greedy; "
              f"bounded sample: batch 1, {prompt_len}-token prompt, {K} decoded tokens (prefill time subtracted); "
              f"host cpu_count={os.cpu_count()}")
    return {"metric": METRIC, "value": v, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": K,
            "warmup": W, "ms_per_step": dt / K * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.model} bf16 random-init, batch 1 greedy decode at {prompt_len}-token context "
                                   f"(CPU, {K} steps)", "batch": 1, "ctx": prompt_len},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ---------------------------------------------------------------------------------- main
# ---------------------------------------------------------------------------------- layer-by-layer family
HYBRID_SIZES = {
    # name: (width, heads, kv heads, head size, feed-forward, layers, vocab)
    "1b": (2048, 16, 4, 128, 8192, 4, 32000),
    "8b": (4096, 32, 8, 128, 14336, 4, 32000),
}


def hybrid_config(width, heads, kv, hd, ff, layers, vocab, chunk):
    """Layers alternate attention and mLSTM mixers, every one with a feed-forward: the Sokevik design at the sizes of
    a Llama layer (same width, heads, head size and feed-forward size as the uniform stack it is compared with)."""
    att = {"type": "attention", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": heads, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": chunk},
                     "rot": {"base": 500000.0, "dims": hd, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    rec = {"type": "mlstm", "mlp": {"kind": "dense", "ff": ff},
           "mixer": {"heads": heads // 2, "dim": hd, "vdim": 2 * hd, "gate_cap": 15.0}}
    return {"architecture": "Sokevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "layers": [att if i % 2 == 0 else rec for i in range(layers)]}


def run_hybrid_compare(args, peaks):
    """Prefill and decode throughput of the layer-by-layer family (RaggedEngine) beside the uniform Llama stack
    (ShardEngine) at equal layer sizes, random weights, plus the time of each kind of kernel per step (CUDA events
    around eager steps).  One JSON line; the default workload of this file is untouched."""
    from dli_b200 import ops, sokevik
    from dli_b200.engine import ModelSpec, ShardEngine
    from dli_b200.ragged_engine import RaggedEngine

    T, K, W = args.ctx, args.steps, args.warmup
    out = {"metric": "hybrid_vs_uniform", "unit": "tokens/s", "ctx": T, "steps": K, "warmup": W, "dtype": "bf16",
           "data": "synthetic", "peaks": peaks, "sizes": {}}
    names = args.hybrid_sizes.split(",")
    if len(names) > 1:
        # one process per size: a size measured after another one in the same process inherits its allocator and
        # graph-pool state (the batch-8 decode of the second size came out up to 10x slower that way)
        import subprocess
        for name in names:
            cmd = [sys.executable, os.path.abspath(__file__), "--compare-hybrid", "--hybrid-sizes", name, "--steps", str(K),
                   "--warmup", str(W), "--ctx", str(T), "--batch", str(args.batch), "--page-size", str(args.page_size)]
            p = subprocess.run(cmd, capture_output=True, text=True, check=True)
            out["sizes"].update(json.loads(p.stdout.strip().splitlines()[-1])["sizes"])
        return out
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > L2: written between timed prefills
    for name in names:
        width, heads, kv, hd, ff, layers, vocab = HYBRID_SIZES[name]
        res = {}
        # ---- the new family
        cfg = hybrid_config(width, heads, kv, hd, ff, layers, vocab, chunk=T)
        spec = sokevik.spec_from_config(cfg)
        eng = RaggedEngine(spec, max_batch=max(args.batch, 8), max_seq_len=T + K + W + 64, page_size=args.page_size)
        eng.load_tensors(sokevik.model_tensors(spec, sokevik.random_state_dict(spec, seed=1, std=0.02, device="cuda")))
        g = torch.Generator().manual_seed(0)
        prompt = torch.randint(0, vocab, (T,), generator=g).tolist()

        def prefill_once():
            s = eng.open_sequence()
            eng.step([(s, prompt)])
            return s

        for _ in range(2):
            eng.close_sequence(prefill_once())
        times = []
        for _ in range(3):
            flush.fill_(1)
            slot = [None]
            times.append(ev_time_ms(lambda: slot.__setitem__(0, prefill_once())))
            eng.close_sequence(slot[0])
        res["hybrid_prefill_tok_s"] = round(T / (statistics.median(times) / 1e3), 1)
        for B in sorted({1, args.batch if args.batch > 1 else 8}):
            slots = []
            for b in range(B):
                slots.append(prefill_once())
            step = lambda: eng.step([(s, [7]) for s in slots])  # noqa: E731
            for _ in range(W):
                step()
            n0 = ops.launch_count
            ms = ev_time_ms(lambda: [step() for _ in range(K)])
            res[f"hybrid_decode_b{B}_tok_s"] = round(B * K / (ms / 1e3), 1)
            res[f"hybrid_decode_b{B}_launches_per_step"] = (ops.launch_count - n0) // K
            for s in slots:
                eng.close_sequence(s)
        res["hybrid_weight_gb"] = round(eng.weight_bytes() / 1e9, 3)
        res["kernels"] = hybrid_kernel_times(eng, spec, T, peaks)
        eng.unload()
        del eng
        torch.cuda.empty_cache()
        # ---- the uniform stack at the same sizes
        lspec = ModelSpec("llama", layers, width, heads, kv, hd, ff, vocab, 1e-6, 500000.0, 0, T + K + W + 64)
        le = ShardEngine(lspec, max_batch=max(args.batch, 8), max_seq_len=T + K + W + 64, page_size=args.page_size)
        le.load_random(seed=1)
        ids = torch.tensor(prompt, dtype=torch.int32, device="cuda")
        le.start_batch(1, T, T + K + W + 8)
        for _ in range(2):
            le.prefill(1, T, ids=ids)
        times = []
        for _ in range(3):
            flush.fill_(1)
            times.append(ev_time_ms(lambda: le.prefill(1, T, ids=ids)))
        res["uniform_prefill_tok_s"] = round(T / (statistics.median(times) / 1e3), 1)
        for B in sorted({1, args.batch if args.batch > 1 else 8}):
            le.start_batch(B, T, T + K + W + 8)
            le.prefill(B, T, ids=ids.repeat(B))
            for _ in range(W):
                le.decode_step(B)
            ms = ev_time_ms(lambda: [le.decode_step(B) for _ in range(K)])
            res[f"uniform_decode_b{B}_tok_s"] = round(B * K / (ms / 1e3), 1)
        res["uniform_weight_gb"] = round(le.weight_bytes() / 1e9, 3)
        le.unload()
        del le
        torch.cuda.empty_cache()
        out["sizes"][name] = res
    return out


# ---------------------------------------------------------------------------------- Togalorn beside Sokevik
def togalorn_config(width, heads, kv, hd, ff, layers, vocab):
    """The Togalorn design at the sizes of a Llama layer: layers alternate state-space and latent-attention mixers (the
    same head count and head size as the attention it is compared with: 64 unrotated + 64 rotated key dims, value
    size hd, a 512-wide cached latent), every layer with a mixture of 8 experts of size ff/4 (2 per token) beside one
    shared expert of size ff/2, so that a token uses as many feed-forward weights as the dense layer it is compared
    with; the two layers run twice (a loop of two passes)."""
    lat = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": hd // 2, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 512, "q_rank": width // 2,
                     "scale": hd ** -0.5, "rot": {"base": 500000.0, "dims": hd // 2}}}
    ssm = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1,
                                       "conv": 4}}
    mlp = {"kind": "moe", "expert": {"ff": ff // 4, "limit": 7.0}, "router": {"experts": 8, "identity": 1, "top": 2},
           "shared": {"ff": ff // 2, "limit": 7.0}}
    return {"architecture": "Togalorn", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6, "groups": 4}, "canon": {"taps": 4}, "loop": {"start": 0, "stop": 2, "times": layers // 2},
            "layers": [dict(ssm, mlp=mlp), dict(lat, mlp=mlp)]}


def ragged_throughput(eng, vocab, T, K, W, batch, tag, flush):
    """Prefill (one T-token portion, L2 flushed before) and decode (batch 1 and `batch`, context T) tokens/s of a
    RaggedEngine, CUDA events."""
    from dli_b200 import ops

    res = {}
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, vocab, (T,), generator=g).tolist()

    def prefill_once():
        s = eng.open_sequence()
        eng.step([(s, prompt)])
        return s

    for _ in range(2):
        eng.close_sequence(prefill_once())
    times = []
    for _ in range(3):
        flush.fill_(1)
        slot = [None]
        times.append(ev_time_ms(lambda: slot.__setitem__(0, prefill_once())))
        eng.close_sequence(slot[0])
    res[f"{tag}_prefill_tok_s"] = round(T / (statistics.median(times) / 1e3), 1)
    res[f"{tag}_prefill_ms"] = round(statistics.median(times), 3)
    for B in sorted({1, batch if batch > 1 else 8}):
        slots = [prefill_once() for _ in range(B)]
        step = lambda: eng.step([(s, [7]) for s in slots])  # noqa: E731
        for _ in range(W):
            step()
        n0 = ops.launch_count
        ms = ev_time_ms(lambda: [step() for _ in range(K)])
        res[f"{tag}_decode_b{B}_tok_s"] = round(B * K / (ms / 1e3), 1)
        res[f"{tag}_decode_b{B}_launches_per_step"] = (ops.launch_count - n0) // K
        for s in slots:
            eng.close_sequence(s)
    res[f"{tag}_weight_gb"] = round(eng.weight_bytes() / 1e9, 3)
    return res


def run_togalorn_compare(args, peaks):
    """Prefill and decode throughput of the Togalorn design beside the framework's closest model, the Sokevik design
    (both on RaggedEngine), at equal layer sizes and depth, random weights, plus each kernel of the new mechanisms
    alone against its roofline.  One JSON line; the default workload of this file is untouched."""
    from dli_b200 import sokevik, togalorn
    from dli_b200.ragged_engine import RaggedEngine

    T, K, W = args.ctx, args.steps, args.warmup
    out = {"metric": "togalorn_vs_sokevik", "unit": "tokens/s", "ctx": T, "steps": K, "warmup": W, "dtype": "bf16",
           "data": "synthetic", "peaks": peaks, "sizes": {}}
    names = args.hybrid_sizes.split(",")
    if len(names) > 1:
        import subprocess
        for name in names:
            cmd = [sys.executable, os.path.abspath(__file__), "--compare-togalorn", "--hybrid-sizes", name, "--steps", str(K),
                   "--warmup", str(W), "--ctx", str(T), "--batch", str(args.batch), "--page-size", str(args.page_size)]
            p = subprocess.run(cmd, capture_output=True, text=True, check=True)
            out["sizes"].update(json.loads(p.stdout.strip().splitlines()[-1])["sizes"])
        return out
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in names:
        width, heads, kv, hd, ff, layers, vocab = HYBRID_SIZES[name]
        mods = ((togalorn, togalorn_config(width, heads, kv, hd, ff, layers, vocab), "togalorn"),
                (sokevik, hybrid_config(width, heads, kv, hd, ff, layers, vocab, chunk=T), "sokevik"))
        res = {}
        for mod, cfg, tag in mods:
            spec = mod.spec_from_config(cfg)
            eng = RaggedEngine(spec, max_batch=max(args.batch, 8), max_seq_len=T + K + W + 64, page_size=args.page_size)
            eng.load_tensors(mod.model_tensors(spec, mod.random_state_dict(spec, seed=1, std=0.02, device="cuda")))
            res.update(ragged_throughput(eng, vocab, T, K, W, args.batch, tag, flush))
            res[f"{tag}_kernels"] = togalorn_kernel_times(eng, spec, T, peaks) if tag == "togalorn" else \
                hybrid_kernel_times(eng, spec, T, peaks)
            eng.unload()
            del eng
            torch.cuda.empty_cache()
        out["sizes"][name] = res
    return out


def togalorn_kernel_times(eng, spec, T, peaks):
    """Each kernel of the Togalorn mechanisms alone at the step sizes of the comparison: a T-token portion (prefill) and
    one token after T (decode), against its algorithmic HBM bytes or FLOPs and the measured peaks."""
    from dli_b200 import ops

    dev, E, W = eng.device, eng.dtype, spec.width
    li_a = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "latent_attention")
    li_s = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "mamba2")
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    res = {}

    def timeit(fn, n=5, reps=10):
        fn()
        return statistics.median(ev_time_ms(lambda: [fn() for _ in range(reps)]) for _ in range(n)) / reps

    def put(key, ms, byt=None, flops=None, fp32=None):
        d = {"ms": round(ms, 4)}
        if byt is not None:
            d["of_hbm"] = round(byt / (ms / 1e3) / hbm, 3)
        if flops is not None:
            d["of_bf16_peak"] = round(flops / (ms / 1e3) / tc, 4)
        if fp32 is not None:
            d["tflops_fp32"] = round(fp32 / (ms / 1e3) / 1e12, 3)
        res[key] = d

    slot = eng.open_sequence()
    eng.kv.reserve(slot, T + 1)
    eng.kv.commit()
    eb = 2
    for tag, rows, start in (("prefill", T, 0), ("decode", 1, T)):
        eng._workspace(rows)
        row_ent = torch.zeros(rows, dtype=torch.int32, device=dev)
        ent = torch.tensor([slot, 0, rows, start], dtype=torch.int32, device=dev)
        tiles = torch.tensor([[0, q0] for q0 in range(0, rows, 64)], dtype=torch.int32, device=dev)
        views = (row_ent, row_ent, ent, row_ent, tiles)
        eng._step_pages = (min(eng.kv.owned[slot]), max(eng.kv.owned[slot]))
        x = torch.randn(rows, W, device=dev)
        hn, he = torch.empty_like(x), torch.empty(rows, W, dtype=E, device=dev)
        y1 = torch.randn(rows, W, device=dev).to(E)
        P = eng.layers[li_a]
        put(f"{tag}_group_rmsnorm", timeit(lambda: ops.group_rmsnorm(x, P["norm1"], spec.norm_groups, 1e-6, hn=hn, he=he)),
            byt=rows * W * (4 + 4 + eb))
        idw = torch.rand(rows, device=dev)
        put(f"{tag}_residual_add2", timeit(lambda: ops.residual_add2(x, y1, y1, idw, hn)), byt=rows * W * (8 + 2 * eb + 4))
        # latent attention: everything between the input projection and the output projection
        m = spec.layers[li_a].mixer
        proj = (0.5 * torch.randn(rows, P["w_proj"].shape[0], device=dev)).to(E)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        ms = timeit(lambda: eng._latent_attention(li_a, m, P, proj, mix, rows, views, rows > 1), n=3, reps=3)
        if rows > 1:
            fl = 2 * (rows * rows // 2) * m.heads * (m.dim + m.rot_dims + m.vdim) + \
                2 * rows * (m.q_rank * m.heads * (m.dim + m.rot_dims) + m.kv_rank * m.heads * (m.dim + m.vdim))
            put(f"{tag}_latent_attention_all", ms, flops=fl)
        else:
            byt = (start + 1) * (m.kv_rank + m.rot_dims) * eb + (P["w_uq"].numel() + P["uk"].numel() + P["uv"].numel()) * eb
            put(f"{tag}_latent_attention_all", ms, byt=byt)
        # state-space mixer: convolution, scan, gated norm
        m, P = spec.layers[li_s].mixer, eng.layers[li_s]
        inner, gn = m.heads * m.vdim, m.groups * m.state
        C = inner + 2 * gn
        proj = (0.5 * torch.randn(rows, P["w_proj"].shape[0], device=dev)).to(E)
        xbc = torch.empty(rows, C, device=dev)
        yss = torch.empty(rows, inner, device=dev)
        mix = torch.empty(rows, inner, dtype=E, device=dev)
        off = P["off"]
        put(f"{tag}_ssm_conv", timeit(lambda: ops.conv1d_act_ragged(proj, eng.slots[("ctail", li_s)], P["conv_w"], P["conv_b"],
                                                                    row_ent, ent, xbc, off["x"])), byt=rows * C * (eb + 4))
        ms = timeit(lambda: ops.ssm_scan_ragged(xbc, proj, eng.slots[("S", li_s)], yss, ent, m.heads, m.vdim, m.state,
                                                m.groups, off["dt"], P["dt_bias"], P["a_log"], P["d_skip"], blocked=rows > 1),
                    n=3, reps=3)
        if rows > 1:
            # FMAs counted as 2: per 64-row block and head C.B^T (64*64*N), G.x (64*64*V), C.S and the state update (2*64*N*V)
            bl_flops = 2 * rows * m.heads * (64 * m.state + 64 * m.vdim + 2 * m.state * m.vdim)
            put(f"{tag}_ssm_scan_blocks_in_order", ms, fp32=bl_flops)
            scr = torch.empty(ops.ssm_parallel_scratch_floats(tiles.shape[0], m.heads, m.state, m.vdim), device=dev)
            ms = timeit(lambda: ops.ssm_scan_ragged(xbc, proj, eng.slots[("S", li_s)], yss, ent, m.heads, m.vdim, m.state,
                                                    m.groups, off["dt"], P["dt_bias"], P["a_log"], P["d_skip"], blocked=True,
                                                    tiles=tiles, scratch=scr), n=3, reps=3)
            put(f"{tag}_ssm_scan_blocks_parallel", ms, fp32=bl_flops)
            ms = timeit(lambda: ops.ssm_scan_ragged(xbc, proj, eng.slots[("S", li_s)], yss, ent, m.heads, m.vdim, m.state,
                                                    m.groups, off["dt"], P["dt_bias"], P["a_log"], P["d_skip"]), n=2, reps=1)
            put(f"{tag}_ssm_scan_token_by_token", ms, fp32=rows * m.heads * m.state * m.vdim * 5)
        else:
            put(f"{tag}_ssm_scan", ms, byt=2 * m.heads * m.state * m.vdim * 4)
        put(f"{tag}_ssm_gated_norm", timeit(lambda: ops.gated_group_rmsnorm(yss, proj, P["out_norm"], mix, m.norm_groups, 1e-6,
                                                                            off["z"])), byt=rows * inner * (4 + 2 * eb))
        # mixture of experts: router, the activation between the two projections, the projections themselves
        e = spec.layers[li_s].moe
        wts, idw = torch.empty(rows, e.experts, device=dev), torch.empty(rows, device=dev)
        si = torch.empty(rows, e.top, dtype=torch.int32, device=dev)
        sw = torch.empty(rows, e.top, device=dev)
        put(f"{tag}_moe_route", timeit(lambda: ops.moe_route(hn, P["w_router"], P["corr"], wts, idw, si, sw, e.experts, e.top)),
            byt=rows * W * 4 + P["w_router"].numel() * 4)
        gu = torch.empty(rows, P["w_gu"].shape[0], dtype=E, device=dev)
        act = torch.empty(rows, e.total_ff, dtype=E, device=dev)
        y2 = torch.empty(rows, W, dtype=E, device=dev)
        ms_gu = timeit(lambda: eng._lin(he, P["w_gu"], gu), n=3, reps=3)
        ms_act = timeit(lambda: ops.moe_act(gu, wts, act, e.experts, e.ff, e.limit, e.shared_ff, e.shared_limit, e.alpha))
        ms_dn = timeit(lambda: eng._lin(act, P["w_down"], y2), n=3, reps=3)
        put(f"{tag}_moe_act", ms_act, byt=rows * e.total_ff * 3 * eb)
        if rows > 1:
            used = 2 * rows * 3 * W * (e.top * e.ff + e.shared_ff)      # FLOPs of the experts a token uses
            put(f"{tag}_moe_projections", ms_gu + ms_dn, flops=used)
            res[f"{tag}_moe_projections"]["of_bf16_peak_all_experts"] = round(2 * rows * 3 * W * e.total_ff / ((ms_gu + ms_dn) / 1e3) / tc, 4)
        else:
            put(f"{tag}_moe_projections_all_experts", ms_gu + ms_dn, byt=3 * W * e.total_ff * eb)
            if ops.moe_sel_supported(W, e.ff, e.shared_ff, e.top):
                act_sel = torch.empty(rows, e.top * e.ff + e.shared_ff, dtype=E, device=dev)
                ms = timeit(lambda: ops.moe_sel(he, P["w_gu"], P["w_down"], si, sw, act_sel, y2, e.experts, e.top, e.ff, e.limit,
                                                e.shared_ff, e.shared_limit, e.alpha))
                put(f"{tag}_moe_chosen_experts", ms, byt=3 * W * (e.top * e.ff + e.shared_ff) * eb)
    eng.close_sequence(slot)
    return res



# ---------------------------------------------------------------------------------- Fubepel beside Sokevik
def fubepel_config(width, heads, kv, hd, ff, layers, vocab, window=1024):
    """The Fubepel design at the sizes of a Llama layer: latent attention (64 + 64 key dims per head, value size hd, a
    512-wide cached latent), a gated delta-rule layer (heads/2 value heads of 2 hd over heads/2 query/key heads of hd:
    the matrix memory of the mLSTM layer it is compared with), windowed attention that keeps 4 first tokens, and a latent
    attention layer on the first layer's cache; every layer with the dense feed-forward and a 256-wide token input."""
    lat = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": hd // 2, "rot_dim": hd // 2, "vdim": hd, "kv_rank": 512, "scale": hd ** -0.5,
                     "rot": {"base": 500000.0, "dims": hd // 2}}}
    dlt = {"type": "delta", "mixer": {"heads": heads // 2, "kv_heads": heads // 2, "dim": hd, "vdim": 2 * hd, "conv": 4}}
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                                          "mask": {"size": window, "keep_first": 4}}}
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    order = [lat, dlt, att, dict(lat, mixer=dict(lat["mixer"], kv_from=0))]
    return {"architecture": "Fubepel", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "token_side": {"dim": 256}, "layers": [dict(order[i % 4], mlp=mlp) for i in range(layers)]}


def run_fubepel_compare(args, peaks):
    """Prefill and decode throughput of the Fubepel design beside the framework's closest model, the Sokevik design
    (both on RaggedEngine: attention beside a matrix-memory recurrent layer, dense feed-forwards), at equal layer sizes
    and depth, random weights, plus each kernel of the new mechanisms alone against its roofline.  One JSON line; the
    default workload of this file is untouched."""
    from dli_b200 import fubepel, sokevik
    from dli_b200.ragged_engine import RaggedEngine

    T, K, W = args.ctx, args.steps, args.warmup
    out = {"metric": "fubepel_vs_sokevik", "unit": "tokens/s", "ctx": T, "steps": K, "warmup": W, "dtype": "bf16",
           "data": "synthetic", "peaks": peaks, "sizes": {}}
    names = args.hybrid_sizes.split(",")
    if len(names) > 1:
        import subprocess
        for name in names:
            cmd = [sys.executable, os.path.abspath(__file__), "--compare-fubepel", "--hybrid-sizes", name, "--steps", str(K),
                   "--warmup", str(W), "--ctx", str(T), "--batch", str(args.batch), "--page-size", str(args.page_size)]
            p = subprocess.run(cmd, capture_output=True, text=True, check=True)
            out["sizes"].update(json.loads(p.stdout.strip().splitlines()[-1])["sizes"])
        return out
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in names:
        width, heads, kv, hd, ff, layers, vocab = HYBRID_SIZES[name]
        mods = ((fubepel, fubepel_config(width, heads, kv, hd, ff, layers, vocab), "fubepel"),
                (sokevik, hybrid_config(width, heads, kv, hd, ff, layers, vocab, chunk=T), "sokevik"))
        res = {}
        for mod, cfg, tag in mods:
            spec = mod.spec_from_config(cfg)
            eng = RaggedEngine(spec, max_batch=max(args.batch, 8), max_seq_len=T + K + W + 64, page_size=args.page_size)
            eng.load_tensors(mod.model_tensors(spec, mod.random_state_dict(spec, seed=1, std=0.02, device="cuda")))
            res.update(ragged_throughput(eng, vocab, T, K, W, args.batch, tag, flush))
            res[f"{tag}_kernels"] = fubepel_kernel_times(eng, spec, T, peaks) if tag == "fubepel" else \
                hybrid_kernel_times(eng, spec, T, peaks)
            eng.unload()
            del eng
            torch.cuda.empty_cache()
        out["sizes"][name] = res
    return out


def fubepel_kernel_times(eng, spec, T, peaks):
    """Each kernel of the Fubepel mechanisms alone at the step sizes of the comparison: a T-token portion (prefill) and
    one token after T (decode), against its algorithmic HBM bytes or FLOPs and the measured peaks."""
    from dli_b200 import ops

    dev, E, W = eng.device, eng.dtype, spec.width
    li_l = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "latent_attention" and L.mixer.kv_from is None)
    li_d = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "delta")
    li_a = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "attention")
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    res = {}

    def timeit(fn, n=5, reps=10):
        fn()
        return statistics.median(ev_time_ms(lambda: [fn() for _ in range(reps)]) for _ in range(n)) / reps

    def put(key, ms, byt=None, flops=None, fp32=None):
        d = {"ms": round(ms, 4)}
        if byt is not None:
            d["of_hbm"] = round(byt / (ms / 1e3) / hbm, 3)
        if flops is not None:
            d["of_bf16_peak"] = round(flops / (ms / 1e3) / tc, 4)
        if fp32 is not None:
            d["tflops_fp32"] = round(fp32 / (ms / 1e3) / 1e12, 3)
        res[key] = d

    slot = eng.open_sequence()
    eng.kv.reserve(slot, T + 1)
    eng.kv.commit()
    eb = 2
    for tag, rows, start in (("prefill", T, 0), ("decode", 1, T)):
        eng._workspace(rows)
        row_ent = torch.zeros(rows, dtype=torch.int32, device=dev)
        ent = torch.tensor([slot, 0, rows, start], dtype=torch.int32, device=dev)
        tiles = torch.tensor([[0, q0] for q0 in range(0, rows, 64)], dtype=torch.int32, device=dev)
        views = (row_ent, row_ent, ent, row_ent, tiles)
        eng._step_pages = (min(eng.kv.owned[slot]), max(eng.kv.owned[slot]))
        x = torch.randn(rows, W, device=dev)
        he = torch.empty(rows, W, dtype=E, device=dev)
        y1 = torch.randn(rows, W, device=dev).to(E)
        P = eng.layers[li_l]
        put(f"{tag}_postnorm_vec_add", timeit(lambda: ops.postnorm_vec_add(y1, x, P["norm1"], 1e-6, he=he)),
            byt=rows * W * (eb + 8 + eb))
        # per-layer token input
        L = spec.layers[li_l]
        n = L.side_dim
        tok = torch.randint(0, spec.vocab, (rows,), dtype=torch.int32, device=dev)
        if rows <= eng.side_fused_max_rows and 2 * W * n * eb <= eng.side_fused_max_bytes:
            put(f"{tag}_token_side", timeit(lambda: ops.token_side(x, tok, eng.w["side_embed"], L.side_off, P["side_gate"],
                                                                   P["side_proj"], P["side_norm"], 1e-6, he=he)),
                byt=2 * W * n * eb)
        else:
            sg, sa = torch.empty(rows, n, dtype=E, device=dev), torch.empty(rows, n, dtype=E, device=dev)

            def side():
                eng._lin(he, P["side_gate"], sg)
                ops.token_side_act(sg, tok, eng.w["side_embed"], L.side_off, sa)
                eng._lin(sa, P["side_proj"], y1)
                ops.postnorm_vec_add(y1, x, P["side_norm"], 1e-6, he=he)
            put(f"{tag}_token_side_all", timeit(side, n=3, reps=3), flops=4 * rows * W * n)
        # latent attention: everything between the input projection and the output projection
        m = spec.layers[li_l].mixer
        proj = (0.5 * torch.randn(rows, P["w_proj"].shape[0], device=dev)).to(E)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        ms = timeit(lambda: eng._latent_attention(li_l, m, P, proj, mix, rows, views, rows > 1), n=3, reps=3)
        if rows > 1:
            fl = 2 * (rows * rows // 2) * m.heads * (m.dim + m.rot_dims + m.vdim) + 2 * rows * m.kv_rank * m.heads * (m.dim + m.vdim)
            put(f"{tag}_latent_attention_all", ms, flops=fl)
        else:
            put(f"{tag}_latent_attention_all", ms, byt=(start + 1) * (m.kv_rank + m.rot_dims) * eb + (P["uk"].numel() + P["uv"].numel()) * eb)
        # windowed attention with kept first tokens
        m, P = spec.layers[li_a].mixer, eng.layers[li_a]
        proj = (0.5 * torch.randn(rows, P["w_proj"].shape[0], device=dev)).to(E)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        ms = timeit(lambda: eng._attention(li_a, m, P, proj, mix, rows, views, rows > 1), n=3, reps=3)
        span = min(m.window, start + rows) if m.window else start + rows
        if rows > 1:
            pairs = sum(min(t + 1, m.window) if m.window else t + 1 for t in range(rows))
            put(f"{tag}_window_attention_all", ms, flops=2 * pairs * m.heads * (m.dim + m.vdim))
        else:
            put(f"{tag}_window_attention_all", ms, byt=span * m.kv_heads * (m.dim + m.vdim) * eb)
        # gated delta rule: convolution, recurrence, head norm and gate
        m, P = spec.layers[li_d].mixer, eng.layers[li_d]
        C = 2 * m.kv_heads * m.dim + m.heads * m.vdim
        proj = (0.5 * torch.randn(rows, P["w_proj"].shape[0], device=dev)).to(E)
        qkv = torch.empty(rows, C, device=dev)
        o = torch.empty(rows, m.heads * m.vdim, device=dev)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        off = P["off"]
        put(f"{tag}_delta_conv", timeit(lambda: ops.conv1d_act_ragged(proj, eng.slots[("ctail", li_d)], P["conv_w"], None, row_ent,
                                                                      ent, qkv, off["q"])), byt=rows * C * (eb + 4))
        ms = timeit(lambda: ops.delta_rule_ragged(qkv, proj, eng.slots[("S", li_d)], o, ent, m.heads, m.kv_heads, m.dim, m.vdim,
                                                  off["b"], off["a"], P["a_log"], P["dt_bias"], m.scale, m.unit_eps, blocked=rows > 1), n=3, reps=3)
        if rows > 1:
            put(f"{tag}_delta_rule_blocks", ms, fp32=rows * m.heads * m.dim * m.vdim * 6)   # three multiply-adds per state entry and token
            ms = timeit(lambda: ops.delta_rule_ragged(qkv, proj, eng.slots[("S", li_d)], o, ent, m.heads, m.kv_heads, m.dim, m.vdim,
                                                      off["b"], off["a"], P["a_log"], P["dt_bias"], m.scale, m.unit_eps), n=2, reps=2)
            put(f"{tag}_delta_rule_row_by_row", ms, fp32=rows * m.heads * m.dim * m.vdim * 6)
        else:
            put(f"{tag}_delta_rule", ms, byt=2 * m.heads * m.dim * m.vdim * 4)
        put(f"{tag}_delta_head_norm_gate", timeit(lambda: ops.head_rmsnorm_gate(o, proj, P["out_norm"], mix, m.heads, m.vdim, 1e-6,
                                                                                gate=1, g_off=off["g"])),
            byt=rows * m.heads * m.vdim * (4 + 2 * eb))
        # feed-forward: gate/up projection with the clamped activation in its epilogue, beside the two-kernel form
        L, P = spec.layers[li_d], eng.layers[li_d]
        act = torch.empty(rows, L.ff, dtype=E, device=dev)
        if P["packed"]:
            sk = eng._splitk() if 2 < rows <= 128 else None
            ms = timeit(lambda: ops.linear_gated_act(he, P["w_gu"], P["ff_act"], sk, out=act), n=3, reps=3)
            if rows > 1:
                put(f"{tag}_ff_gate_up_act", ms, flops=4 * rows * W * L.ff)
            else:
                put(f"{tag}_ff_gate_up_act", ms, byt=2 * W * L.ff * eb)
    eng.close_sequence(slot)
    return res


# ---------------------------------------------------------------------------------- Gimudra beside Togalorn and Sokevik
def gimudra_config(width, heads, kv, hd, ff, layers, vocab, block=512):
    """The Gimudra design at the sizes of a Llama layer: attention inside blocks of `block` positions with the Llama
    layer's head counts and head size; layer 0 with the dense feed-forward and a cache of its own, layer 1 with a cache
    of its own, the later layers on layer 1's cache; layers 1.. with a mixture of 14 squared-ReLU experts of size ff/4
    plus 2 pass-through outputs in 4 groups of which 2 are kept, 4 outputs per token."""
    mix = {"heads": heads, "kv_heads": kv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": block}}
    moe = {"kind": "moe", "expert": {"ff": ff // 4},
           "router": {"experts": 14, "identity": 2, "top": 4, "scale": 1.5, "groups": {"count": 4, "keep": 2}}}
    out = []
    for i in range(layers):
        out.append({"type": "attention", "mixer": dict(mix, kv_from=1) if i >= 2 else dict(mix),
                    "mlp": {"kind": "dense", "ff": ff} if i == 0 else moe})
    return {"architecture": "Gimudra", "vocab": vocab, "width": width, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
            "layers": out}


def run_gimudra_compare(args, peaks):
    """Prefill and decode throughput of the Gimudra design beside the framework's closest models on RaggedEngine — the
    Togalorn design (mixture of experts with pass-through outputs, attention with a cache) and the Sokevik design (the
    same attention kernels under a block mask, dense feed-forward) — at equal layer sizes and depth, random weights, plus
    each kernel of the new mechanisms alone against its roofline.  One JSON line; the default workload of this file is
    untouched."""
    from dli_b200 import gimudra, sokevik, togalorn
    from dli_b200.ragged_engine import RaggedEngine

    T, K, W = args.ctx, args.steps, args.warmup
    out = {"metric": "gimudra_vs_togalorn_sokevik", "unit": "tokens/s", "ctx": T, "steps": K, "warmup": W, "dtype": "bf16",
           "data": "synthetic", "peaks": peaks, "sizes": {}}
    names = args.hybrid_sizes.split(",")
    if len(names) > 1:
        import subprocess
        for name in names:
            cmd = [sys.executable, os.path.abspath(__file__), "--compare-gimudra", "--hybrid-sizes", name, "--steps", str(K),
                   "--warmup", str(W), "--ctx", str(T), "--batch", str(args.batch), "--page-size", str(args.page_size)]
            p = subprocess.run(cmd, capture_output=True, text=True, check=True)
            out["sizes"].update(json.loads(p.stdout.strip().splitlines()[-1])["sizes"])
        return out
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name in names:
        width, heads, kv, hd, ff, layers, vocab = HYBRID_SIZES[name]
        mods = ((gimudra, gimudra_config(width, heads, kv, hd, ff, layers, vocab), "gimudra"),
                (togalorn, togalorn_config(width, heads, kv, hd, ff, layers, vocab), "togalorn"),
                (sokevik, hybrid_config(width, heads, kv, hd, ff, layers, vocab, chunk=512), "sokevik"))
        res = {}
        for mod, cfg, tag in mods:
            spec = mod.spec_from_config(cfg)
            eng = RaggedEngine(spec, max_batch=max(args.batch, 8), max_seq_len=T + K + W + 64, page_size=args.page_size)
            eng.load_tensors(mod.model_tensors(spec, mod.random_state_dict(spec, seed=1, std=0.02, device="cuda")))
            res.update(ragged_throughput(eng, vocab, T, K, W, args.batch, tag, flush))
            res[f"{tag}_kernels"] = {"gimudra": gimudra_kernel_times, "togalorn": togalorn_kernel_times,
                                     "sokevik": hybrid_kernel_times}[tag](eng, spec, T, peaks)
            eng.unload()
            del eng
            torch.cuda.empty_cache()
        out["sizes"][name] = res
    return out


def gimudra_kernel_times(eng, spec, T, peaks):
    """Each kernel of the Gimudra mechanisms alone at the step sizes of the comparison: a T-token portion (prefill) and
    the prompt's last token alone (decode), against its algorithmic HBM bytes or FLOPs and the measured peaks."""
    from dli_b200 import ops

    dev, E, W = eng.device, eng.dtype, spec.width
    li_d = next(i for i, L in enumerate(spec.layers) if L.ff)
    li_m = next(i for i, L in enumerate(spec.layers) if L.moe is not None)
    n_last = spec.n_layers
    hbm, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    res = {}

    def timeit(fn, n=5, reps=10):
        fn()
        return statistics.median(ev_time_ms(lambda: [fn() for _ in range(reps)]) for _ in range(n)) / reps

    def put(key, ms, byt=None, flops=None):
        d = {"ms": round(ms, 4)}
        if byt is not None:
            d["of_hbm"] = round(byt / (ms / 1e3) / hbm, 3)
        if flops is not None:
            d["of_bf16_peak"] = round(flops / (ms / 1e3) / tc, 4)
        res[key] = d

    slot = eng.open_sequence()
    eng.kv.reserve(slot, T + 1)
    eng.kv.commit()
    eb = 2
    for tag, rows, start in (("prefill", T, 0), ("decode", 1, T - 1)):  # the decode row sees a whole block of keys
        eng._workspace(rows)
        row_ent = torch.zeros(rows, dtype=torch.int32, device=dev)
        ent = torch.tensor([slot, 0, rows, start], dtype=torch.int32, device=dev)
        x = torch.randn(rows, W, device=dev)
        hn, he = torch.empty_like(x), torch.empty(rows, W, dtype=E, device=dev)
        y1 = torch.randn(rows, W, device=dev).to(E)
        idw = torch.rand(rows, device=dev)
        Pm, Pd = eng.layers[li_m], eng.layers[li_d]
        # between the output projection and the feed-forward: x += ls1 * y, norm2 -> fp32 (router) and bf16 (projections)
        put(f"{tag}_close_mixer_norm", timeit(lambda: ops.layer_close(x, y1, ls=Pm["ls1"], w_next=Pm["norm2"], out_f=hn, out_e=he,
                                                                      eps=1e-6)), byt=rows * W * (eb + 8 + 4 + eb))
        # the same kernel with the router of the mixture that follows (what the engine launches in front of the experts)
        e = spec.layers[li_m].moe
        wts = torch.empty(rows, e.experts, device=dev)
        si = torch.empty(rows, e.top, dtype=torch.int32, device=dev)
        sw = torch.empty(rows, e.top, device=dev)
        route = dict(w_router=Pm["w_router"], correction=Pm["corr"], wts=wts, idw=idw, sel_idx=si, sel_w=sw, n_real=e.experts,
                     top=e.top, groups=e.groups, keep=e.keep, wscale=e.route_scale, renorm=False)
        put(f"{tag}_close_mixer_norm_route", timeit(lambda: ops.layer_close(x, y1, ls=Pm["ls1"], w_next=Pm["norm2"], out_f=hn,
                                                                            out_e=he, eps=1e-6, route=route)),
            byt=rows * W * (eb + 8 + 4 + eb) + Pm["w_router"].numel() * 4)
        # after the last layer's feed-forward: x += ls2 * (y + share * h), store the result, average over all results, norm
        Pl = eng.layers[n_last - 1]
        xs = eng._xs
        put(f"{tag}_close_layer_average_norm",
            timeit(lambda: ops.layer_close(x, y1, idw=idw, h_in=hn, ls=Pl["ls2"], xs=xs, n_prev=n_last, dwa=Pl["dwa"],
                                           w_next=eng.w["final_norm"], out_e=he, eps=1e-6)),
            byt=rows * W * (eb + 8 + 4 + 4 * n_last + 4 + eb))
        if rows > 1:
            put(f"{tag}_token_shift", timeit(lambda: ops.token_shift_ragged(hn, Pm["shift"], eng.slots[("shift", li_m)], row_ent,
                                                                            ent, he)), byt=rows * W * (4 + eb))
        else:
            put(f"{tag}_close_layer_average_norm_shift",
                timeit(lambda: ops.layer_close(x, y1, idw=idw, h_in=hn, ls=Pl["ls2"], xs=xs, n_prev=n_last - 1,
                                               dwa=eng.layers[n_last - 2]["dwa"], w_next=Pl["norm1"], shift=Pl["shift"],
                                               tail=eng.slots[("shift", n_last - 1)], ent=ent, out_e=he, eps=1e-6)),
                byt=rows * W * (eb + 8 + 4 + 4 * (n_last - 1) + 4 + eb + 8))
        # attention with the distance penalty (own cache: prep appends keys and values)
        m = spec.layers[li_m].mixer
        n_proj = Pm["w_proj"].shape[0]
        proj = (0.5 * torch.randn(rows, n_proj, device=dev)).to(E)
        qbuf = torch.empty(rows, m.heads * m.dim, device=dev)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        kc, vc = eng.kv.k[eng.kv_index[li_m]], eng.kv.v[eng.kv_index[li_m]]
        off = Pm["off"]
        put(f"{tag}_attn_prep", timeit(lambda: ops.attn_prep_append(proj, qbuf, kc, vc, row_ent, ent, eng.kv.page_table, m.heads,
                                                                     m.kv_heads, m.dim, m.vdim, 0, off["q"], off["k"], off["v"],
                                                                     None, None, 1e-6, None, None, None, None, bias=Pm["qkv_b"])))
        blk = m.chunk if m.chunk else T
        for pen in (True, False):
            r1, r2 = (Pm["r1"], Pm["r2"]) if pen else (None, None)
            key = f"{tag}_attn" + ("" if pen else "_without_penalty")
            if rows > 1 and ops.attn_ragged_tc_supported(m.dim, m.vdim, E):
                tiles = torch.tensor([[0, q0] for q0 in range(0, rows, 64)], dtype=torch.int32, device=dev)
                ms = timeit(lambda: ops.attn_ragged_tc(qbuf, kc, vc, None, mix, ent, tiles, eng.kv.page_table, m.heads, m.kv_heads,
                                                       m.dim, m.vdim, m.scale, chunk=m.chunk, r1=r1, r2=r2))
                put(key, ms, flops=2 * (rows * blk // 2) * m.heads * (m.dim + m.vdim))
            else:
                splits = max(1, min(16, (4 * eng._sms) // (rows * m.heads), (blk + 31) // 32))
                ms = timeit(lambda: ops.attn_ragged(qbuf, kc, vc, None, mix, row_ent, ent, eng.kv.page_table, m.heads, m.kv_heads,
                                                    m.dim, m.vdim, m.scale, chunk=m.chunk, splits=splits,
                                                    part=eng._apart_att if splits > 1 else None, r1=r1, r2=r2))
                put(key, ms, byt=(start % blk + 1) * m.kv_heads * (m.dim + m.vdim) * eb)
        # dense feed-forward with biases: the activation between the projections
        F = spec.layers[li_d].ff
        gu = (0.5 * torch.randn(rows, 2 * F, device=dev)).to(E)
        act = torch.empty(rows, F, dtype=E, device=dev)
        put(f"{tag}_ff_bias_silu_mul", timeit(lambda: ops.silu_mul(gu, act, bias=Pd["gu_b"])), byt=rows * F * 3 * eb)
        # mixture of experts: router with groups, activation, projections
        put(f"{tag}_moe_route", timeit(lambda: ops.moe_route(hn, Pm["w_router"], Pm["corr"], wts, idw, si, sw, e.experts, e.top,
                                                             groups=e.groups, keep=e.keep, wscale=e.route_scale, renorm=False)),
            byt=rows * W * 4 + Pm["w_router"].numel() * 4)
        gu = torch.empty(rows, Pm["w_gu"].shape[0], dtype=E, device=dev)
        act = torch.empty(rows, e.total_ff, dtype=E, device=dev)
        y2 = torch.empty(rows, W, dtype=E, device=dev)
        ms_gu = timeit(lambda: eng._lin(he, Pm["w_gu"], gu), n=3, reps=3)
        ms_act = timeit(lambda: ops.moe_act(gu, wts, act, e.experts, e.ff, 0.0, gated=False))
        ms_dn = timeit(lambda: eng._lin(act, Pm["w_down"], y2), n=3, reps=3)
        put(f"{tag}_moe_act", ms_act, byt=rows * (e.total_ff + e.top * e.ff) * eb)  # written: all experts; read: the chosen ones
        if rows > 1:
            put(f"{tag}_moe_projections", ms_gu + ms_dn, flops=2 * rows * 2 * W * e.top * e.ff)
            res[f"{tag}_moe_projections"]["of_bf16_peak_all_experts"] = round(2 * rows * 2 * W * e.total_ff / ((ms_gu + ms_dn) / 1e3) / tc, 4)
        else:
            put(f"{tag}_moe_projections_all_experts", ms_gu + ms_dn, byt=2 * W * e.total_ff * eb)
            if ops.moe_sel_supported(W, e.ff, 0, e.top):
                act_sel = torch.empty(rows, e.top * e.ff, dtype=E, device=dev)
                ms = timeit(lambda: ops.moe_sel(he, Pm["w_gu"], Pm["w_down"], si, sw, act_sel, y2, e.experts, e.top, e.ff, 0.0,
                                                gated=False))
                put(f"{tag}_moe_chosen_experts", ms, byt=2 * W * e.top * e.ff * eb)
    eng.close_sequence(slot)
    return res



def hybrid_kernel_times(eng, spec, T, peaks):
    """Each kernel of the ragged path alone at the step sizes of the comparison: a T-token portion (prefill) and one
    token after T (decode), against its algorithmic HBM bytes (or FLOPs) and the measured peaks."""
    from dli_b200 import ops

    dev, E = eng.device, eng.dtype
    W = spec.width
    att = next(L.mixer for L in spec.layers if L.mixer.kind == "attention")
    rec = next(L.mixer for L in spec.layers if L.mixer.kind == "mlstm")
    li_a = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "attention")
    li_r = next(i for i, L in enumerate(spec.layers) if L.mixer.kind == "mlstm")
    slot = eng.open_sequence()
    eng.kv.reserve(slot, T + 1)
    eng.kv.commit()
    hbm = peaks["hbm_gbs"] * 1e9
    res = {}

    def timeit(fn, n=5, reps=10):
        """ms per call: `reps` back-to-back launches per event bracket, so that a short kernel is not timed as one
        launch latency (the convolution and the recurrence advance their state; any state is as good as another)."""
        fn()
        return statistics.median(ev_time_ms(lambda: [fn() for _ in range(reps)]) for _ in range(n)) / reps

    for tag, rows, start in (("prefill", T, 0), ("decode", 1, T - 1)):  # the decode row sees a whole block of keys
        row_ent = torch.zeros(rows, dtype=torch.int32, device=dev)
        ent = torch.tensor([slot, 0, rows, start], dtype=torch.int32, device=dev)
        x = torch.randn(rows, W, device=dev)
        hn, hc = torch.empty_like(x), torch.empty(rows, W, dtype=E, device=dev)
        y = torch.randn(rows, W, device=dev).to(E)
        P = eng.layers[li_a]
        ms = timeit(lambda: ops.postnorm_add_norm(y, x, 1.0, 1e-6, hn, 1.0))
        res[f"{tag}_postnorm_add_norm"] = {"ms": round(ms, 4), "of_hbm": round(rows * W * (2 + 4 + 4 + 4) / (ms / 1e3) / hbm, 3)}
        ms = timeit(lambda: ops.causal_conv_ragged(hn, eng.slots[("tail1", li_a)], P["canon1"], row_ent, ent, hc))
        res[f"{tag}_conv"] = {"ms": round(ms, 4), "of_hbm": round(rows * W * (4 + 2) / (ms / 1e3) / hbm, 3)}
        # attention
        m = att
        n_proj = P["w_proj"].shape[0]
        proj = (0.5 * torch.randn(rows, n_proj, device=dev)).to(E)
        qbuf = torch.empty(rows, m.heads * m.dim, device=dev)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        kc, vc = eng.kv.k[eng.kv_index[li_a]], eng.kv.v[eng.kv_index[li_a]]
        cq, sq = eng._table(m.rot_base, m.rot_dims, m.rot_scaling)
        cv, sv = eng._table(m.rot_base, m.vdim, None)
        off = P["off"]
        prep = lambda: ops.attn_prep_append(proj, qbuf, kc, vc, row_ent, ent, eng.kv.page_table, m.heads, m.kv_heads,  # noqa: E731
                                            m.dim, m.vdim, m.rot_dims, off["q"], off["k"], off["v"], P["q_norm"],
                                            P["k_norm"], 1e-6, cq, sq, cv, sv)
        run = lambda: ops.attn_ragged(qbuf, kc, vc, proj, mix, row_ent, ent, eng.kv.page_table, m.heads, m.kv_heads,  # noqa: E731
                                      m.dim, m.vdim, m.scale, chunk=m.chunk, sink=P["sink"], g_off=off["g"], cos_v=cv, sin_v=sv)
        ms = timeit(prep)
        res[f"{tag}_attn_prep"] = {"ms": round(ms, 4)}
        if rows > 1 and ops.attn_ragged_tc_supported(m.dim, m.vdim, E):
            tiles = torch.tensor([[0, q0] for q0 in range(0, rows, 64)], dtype=torch.int32, device=dev)
            run = lambda: ops.attn_ragged_tc(qbuf, kc, vc, proj, mix, ent, tiles, eng.kv.page_table, m.heads, m.kv_heads,  # noqa: E731
                                             m.dim, m.vdim, m.scale, chunk=m.chunk, sink=P["sink"], g_off=off["g"], cos_v=cv, sin_v=sv)
        ms = timeit(run)
        if rows == 1:
            byt = ((start % m.chunk if m.chunk else start) + 1) * m.kv_heads * (m.dim + m.vdim) * 2  # visible keys only
            res[f"{tag}_attn"] = {"ms": round(ms, 4), "of_hbm": round(byt / (ms / 1e3) / hbm, 3)}
        else:
            fl = 2 * (rows * (min(rows, m.chunk) if m.chunk else rows) // 2) * m.heads * (m.dim + m.vdim)  # visible pairs only
            res[f"{tag}_attn"] = {"ms": round(ms, 4), "of_bf16_peak": round(fl / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        # recurrent layer
        m, P = rec, eng.layers[li_r]
        n_proj = P["w_proj"].shape[0]
        proj = (0.5 * torch.randn(rows, n_proj, device=dev)).to(E)
        mix = torch.empty(rows, m.heads * m.vdim, dtype=E, device=dev)
        oscr = torch.empty(rows * m.heads * m.vdim, device=dev)
        off = P["off"]
        if rows > 64:
            rtiles = torch.tensor([[0, q0] for q0 in range(0, rows, 64)], dtype=torch.int32, device=dev)
            scr = torch.empty(ops.mlstm_parallel_scratch_floats(rtiles.shape[0], m.heads, m.dim, m.vdim), device=dev)
            ms = timeit(lambda: ops.mlstm_ragged_parallel(proj, oscr, mix, ent, rtiles, scr, m.heads, m.dim, m.vdim, off["q"],
                                                          off["k"], off["v"], off["i"], off["f"], off["g"], P["i_b"],
                                                          P["f_b"], m.gate_cap, P["out_norm"], 1e-6, eng.slots[("S", li_r)],
                                                          eng.slots[("n", li_r)], eng.slots[("m", li_r)]))
            fl = rows * m.heads * (m.dim * m.vdim * 4 + 64 * (m.dim + m.vdim))  # state move + read-out, FMAs counted as 2
            res[f"{tag}_mlstm_blocks_parallel"] = {"ms": round(ms, 4), "tflops_fp32": round(fl / (ms / 1e3) / 1e12, 3)}
        ms = timeit(lambda: ops.mlstm_ragged(proj, oscr, mix, ent, m.heads, m.dim, m.vdim, off["q"], off["k"], off["v"],
                                             off["i"], off["f"], off["g"], P["i_b"], P["f_b"], m.gate_cap, P["out_norm"],
                                             1e-6, eng.slots[("S", li_r)], eng.slots[("n", li_r)], eng.slots[("m", li_r)],
                                             blocked=rows > 1))
        state = m.heads * m.dim * m.vdim * 4
        if rows == 1:
            res[f"{tag}_mlstm"] = {"ms": round(ms, 4), "of_hbm": round(2 * state / (ms / 1e3) / hbm, 3)}
        else:
            fl = rows * m.heads * m.dim * m.vdim * 4
            res[f"{tag}_mlstm"] = {"ms": round(ms, 4), "state_update_tflops": round(fl / (ms / 1e3) / 1e12, 3)}
    eng.close_sequence(slot)
    # the like kernels of the uniform stack at the same sizes (bf16 residual, rotate-half RoPE, plain softmax)
    H, KV, hd = att.heads, att.kv_heads, att.dim
    if att.dim == att.vdim and hd in (64, 128):
        qkv = (0.5 * torch.randn(T, (H + 2 * KV) * hd, device=dev)).to(torch.bfloat16)
        o = torch.empty(T, H * hd, dtype=torch.bfloat16, device=dev)
        ms = timeit(lambda: ops.attn_prefill(qkv, o, 1, T, H, KV, hd, hd ** -0.5))
        fl = 2 * (T * T // 2) * H * 2 * hd
        res["uniform_prefill_attn"] = {"ms": round(ms, 4), "of_bf16_peak": round(fl / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        ms = timeit(lambda: ops.attn_prefill(qkv, o, 1, T, H, KV, hd, hd ** -0.5, tensor_core=False))
        res["uniform_prefill_attn_mma_sync"] = {"ms": round(ms, 4), "of_bf16_peak": round(fl / (ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
        ps = eng.kv.page_size
        n_pages = (T + 1 + ps - 1) // ps
        kc = torch.randn(n_pages, KV, ps, hd, device=dev).to(torch.bfloat16)
        vc = torch.randn(n_pages, KV, ps, hd, device=dev).to(torch.bfloat16)
        ptab = torch.arange(n_pages, dtype=torch.int32, device=dev)[None].contiguous()
        lens = torch.tensor([T + 1], dtype=torch.int32, device=dev)
        q1 = qkv[:1].contiguous()
        o1 = torch.empty(1, H * hd, dtype=torch.bfloat16, device=dev)
        splits = 8
        scratch = torch.empty(max(ops.attn_decode_scratch_bytes(1, H, hd, splits) // 4, 1), dtype=torch.float32, device=dev)
        ms = timeit(lambda: ops.paged_attn_decode(q1, q1.stride(0), kc, vc, ptab, lens, o1, H, KV, hd, hd ** -0.5,
                                                  num_splits=splits, scratch=scratch))
        byt = (T + 1) * KV * 2 * hd * 2
        res["uniform_decode_attn"] = {"ms": round(ms, 4), "of_hbm": round(byt / (ms / 1e3) / hbm, 3)}
    xb = torch.randn(T, W, device=dev).to(torch.bfloat16)
    wb = torch.ones(W, dtype=torch.bfloat16, device=dev)
    ob = torch.empty_like(xb)
    ms = timeit(lambda: ops.add_rmsnorm(xb, wb, 1e-6, residual=xb, resid_out=ob, out=ob))
    res["uniform_prefill_add_rmsnorm"] = {"ms": round(ms, 4), "of_hbm": round(T * W * 2 * 4 / (ms / 1e3) / hbm, 3)}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--compare-hybrid", action="store_true",
                    help="instead of the default workload: the layer-by-layer family beside the uniform stack at equal sizes")
    ap.add_argument("--compare-togalorn", action="store_true",
                    help="instead of the default workload: the Togalorn design beside the Sokevik design at equal sizes")
    ap.add_argument("--compare-fubepel", action="store_true",
                    help="instead of the default workload: the Fubepel design beside the Sokevik design at equal sizes")
    ap.add_argument("--compare-gimudra", action="store_true",
                    help="prefill / decode throughput of the Gimudra design beside the Togalorn and Sokevik designs at equal sizes")
    ap.add_argument("--hybrid-sizes", default="1b,8b")
    args = ap.parse_args()

    from dli_b200.engine import NAMED_SPECS

    spec = NAMED_SPECS[args.model]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args, spec)), flush=True)
        return

    peaks = measured_peaks()
    if args.compare_hybrid:
        if rank == 0:
            print(json.dumps(run_hybrid_compare(args, peaks)), flush=True)
        return
    if args.compare_togalorn:
        if rank == 0:
            print(json.dumps(run_togalorn_compare(args, peaks)), flush=True)
        return
    if args.compare_fubepel:
        if rank == 0:
            print(json.dumps(run_fubepel_compare(args, peaks)), flush=True)
        return
    if args.compare_gimudra:
        if rank == 0:
            print(json.dumps(run_gimudra_compare(args, peaks)), flush=True)
        return
    if world > 1 or args.gpus > 1:
        from dli_b200.pipeline import run_pipeline_bench

        import torch.distributed as dist

        try:
            res = run_pipeline_bench(args, spec, peaks)
        finally:
            if dist.is_initialized():
                dist.destroy_process_group()
        if rank != 0:
            return
    else:
        res = run_single(args, spec, peaks)
    line = {"metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": res["config"],
            "e2e": res["e2e"], "roofline": res["roofline"], "gpu_launches": res["gpu_launches"],
            "clocks": res["clocks"], "extra": res.get("extra", {})}
    if args.gpus == 1 and not args.no_cpu_baseline:
        try:
            line["cpu_baseline"] = cpu_baseline(spec, args)
        except Exception as e:  # noqa: BLE001
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"failed: {str(e)[:200]}"}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
