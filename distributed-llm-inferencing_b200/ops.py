"""Thin torch-tensor front end over the C-ABI (include/dli.h).

torch is used only for device memory and streams; every function passes raw
device pointers to the hand-written kernels and enqueues on torch's current
stream.  Tensors must be CUDA, contiguous where noted, bf16 unless stated.
"""
from __future__ import annotations

import os as _os

import torch

from . import _lib
from ._lib import EPI_BIAS, EPI_GELU_NEW, EPI_NONE, EPI_RESIDUAL  # noqa: F401

# number of kernels this process has launched through the C-ABI (bench.py's gpu_launches)
launch_count = 0


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _req(t, dtype=torch.bfloat16):
    if t is None:
        return
    if not t.is_cuda:
        raise ValueError("dli ops need CUDA tensors (there is no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")


def sm_count() -> int:
    n = _lib.load().dli_sm_count()
    if n <= 0:
        _lib.check("dli_sm_count", n)
    return n


def embedding(ids, table, out=None, positions=None, pos_table=None):
    """ids int32 [rows]; table [V, d] -> [rows, d]."""
    global launch_count
    _req(ids, torch.int32), _req(table), _req(pos_table), _req(positions, torch.int32)
    rows, (vocab, d) = ids.numel(), table.shape
    if out is None:
        out = torch.empty(rows, d, dtype=torch.bfloat16, device=table.device)
    _lib.check("dli_embedding_bf16", _lib.load().dli_embedding_bf16(
        _p(ids), _p(positions), _p(table), _p(pos_table), _p(out), rows, d, vocab, _stream()))
    launch_count += 1
    return out


def add_rmsnorm(x, weight, eps, residual=None, resid_out=None, out=None):
    """y = rmsnorm(residual + x) * weight; optionally writes h = residual + x."""
    global launch_count
    _req(x), _req(weight), _req(residual), _req(resid_out)
    rows, d = x.shape
    if out is None:
        out = torch.empty_like(x)
    _lib.check("dli_add_rmsnorm_bf16", _lib.load().dli_add_rmsnorm_bf16(
        _p(x), _p(residual), _p(weight), _p(resid_out), _p(out), rows, d, float(eps), _stream()))
    launch_count += 1
    return out


def add_layernorm(x, weight, bias, eps, residual=None, resid_out=None, out=None):
    global launch_count
    _req(x), _req(weight), _req(bias), _req(residual), _req(resid_out)
    rows, d = x.shape
    if out is None:
        out = torch.empty_like(x)
    _lib.check("dli_add_layernorm_bf16", _lib.load().dli_add_layernorm_bf16(
        _p(x), _p(residual), _p(weight), _p(bias), _p(resid_out), _p(out), rows, d, float(eps), _stream()))
    launch_count += 1
    return out


def rope_kv_append(qkv, cos, sin, positions, seq_ids, page_table, k_cache, v_cache, H, KV, hd):
    """Rotate q,k of packed qkv [rows,(H+2KV)*hd] in place and append k,v to the paged cache."""
    global launch_count
    _req(qkv), _req(cos), _req(sin), _req(k_cache), _req(v_cache)
    _req(positions, torch.int32), _req(seq_ids, torch.int32), _req(page_table, torch.int32)
    rows = qkv.shape[0]
    page_size = k_cache.shape[2]
    _lib.check("dli_rope_kv_append_bf16", _lib.load().dli_rope_kv_append_bf16(
        _p(qkv), _p(cos), _p(sin), _p(positions), _p(seq_ids), _p(page_table), page_table.shape[1],
        _p(k_cache), _p(v_cache), rows, H, KV, hd, page_size, _stream()))
    launch_count += 1


def qkv_rope_append_supported(rows, K, H, KV, hd, bias) -> bool:
    """Can the qkv projection of this prompt pass run as ONE kernel with RoPE and the cache append in its epilogue?"""
    return rows > 128 and hd == 128 and H % 2 == 0 and KV % 2 == 0 and K % 64 == 0 and bias is None


def linear_qkv_rope_append(x, w_qkv, qkv, cos, sin, positions, seq_ids, page_table, k_cache, v_cache, H, KV, hd):
    """qkv = x @ w_qkv.T with q, k rotated and k, v appended to the paged cache in the GEMM's epilogue (a prompt pass;
    the same bits as linear() followed by rope_kv_append())."""
    global launch_count
    _req(x), _req(w_qkv), _req(qkv), _req(cos), _req(sin), _req(k_cache), _req(v_cache)
    _req(positions, torch.int32), _req(seq_ids, torch.int32), _req(page_table, torch.int32)
    M, K = x.shape
    if w_qkv.shape != ((H + 2 * KV) * hd, K) or qkv.shape != (M, (H + 2 * KV) * hd):
        raise ValueError("linear_qkv_rope_append: shapes do not match H, KV, hd")
    _lib.check("dli_gemm_qkv_rope_append_bf16", _lib.load().dli_gemm_qkv_rope_append_bf16(
        _p(x), _p(w_qkv), _p(qkv), M, K, _p(cos), _p(sin), _p(positions), _p(seq_ids), _p(page_table),
        page_table.shape[1], _p(k_cache), _p(v_cache), H, KV, hd, k_cache.shape[2], _stream()))
    launch_count += 1
    return qkv


def attn_decode_scratch_bytes(B, H, hd, num_splits) -> int:
    return int(_lib.load().dli_paged_attn_decode_scratch_bytes(B, H, hd, num_splits))


def paged_attn_decode(q, q_stride, k_cache, v_cache, page_table, seq_lens, out, H, KV, hd,
                      scale, num_splits=1, scratch=None, window=0):
    """q: tensor whose row b starts at q.data_ptr() + b*q_stride elements."""
    global launch_count
    _req(k_cache), _req(v_cache), _req(out)
    _req(page_table, torch.int32), _req(seq_lens, torch.int32)
    B = seq_lens.numel()
    page_size = k_cache.shape[2]
    sbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _lib.check("dli_paged_attn_decode_bf16", _lib.load().dli_paged_attn_decode_bf16(
        _p(q), q_stride, _p(k_cache), _p(v_cache), _p(page_table), page_table.shape[1], _p(seq_lens),
        _p(out), _p(scratch), sbytes, B, H, KV, hd, page_size, num_splits, float(scale), window,
        _stream()))
    launch_count += 2 if num_splits > 1 else 1
    return out


def attn_prefill(qkv, out, B, T, H, KV, hd, scale, window=0, tensor_core=None):
    """Causal prefill attention.  head_dim 128 runs on tcgen05 (dli_attn_prefill_tc_bf16) unless
    tensor_core=False or DLI_PREFILL_ATTN=mma; head_dim 64 uses the mma.sync kernel."""
    global launch_count
    _req(qkv), _req(out)
    if tensor_core is None:
        tensor_core = hd == 128 and _os.environ.get("DLI_PREFILL_ATTN", "tc") != "mma"
    if tensor_core:
        _lib.check("dli_attn_prefill_tc_bf16", _lib.load().dli_attn_prefill_tc_bf16(
            _p(qkv), _p(out), B, T, H, KV, hd, float(scale), window, _stream()))
        launch_count += 1
        return out
    _lib.check("dli_attn_prefill_bf16", _lib.load().dli_attn_prefill_bf16(
        _p(qkv), _p(out), B, T, H, KV, hd, float(scale), window, _stream()))
    launch_count += 1
    return out


def attn_prefill_paged(qkv, out, k_cache, v_cache, page_table, B, T, prefix, H, KV, hd, scale, window=0):
    """Causal attention of a prompt chunk (positions prefix..prefix+T-1) against the paged cache
    (chunked prefill); page_table holds the rows of the B sequences of this call."""
    global launch_count
    _req(qkv), _req(out), _req(k_cache), _req(v_cache), _req(page_table, torch.int32)
    _lib.check("dli_attn_prefill_paged_bf16", _lib.load().dli_attn_prefill_paged_bf16(
        _p(qkv), _p(out), _p(k_cache), _p(v_cache), _p(page_table), page_table.shape[1], k_cache.shape[0], B, T, prefix,
        H, KV, hd, k_cache.shape[2], float(scale), window, _stream()))
    launch_count += 1
    return out


def _linear(fn_name, x, w, bias, residual, out, epilogue):
    global launch_count
    _req(x), _req(w), _req(bias), _req(residual), _req(out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"linear: x is [{M},{K}] but w is {tuple(w.shape)}")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    epi = epilogue | (EPI_BIAS if bias is not None else 0) | (EPI_RESIDUAL if residual is not None else 0)
    fn = getattr(_lib.load(), fn_name)
    _lib.check(fn_name, fn(_p(x), _p(w), _p(bias), _p(residual), _p(out), M, N, K, epi, _stream()))
    launch_count += (M + 3) // 4 if fn_name == "dli_gemv_bf16" else 1
    return out


def linear(x, w, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    """y = epi(x @ w.T); CUDA-core GEMV for M <= 2, tcgen05 GEMM otherwise."""
    return _linear("dli_linear_bf16", x, w, bias, residual, out, epilogue)


def gemv(x, w, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    return _linear("dli_gemv_bf16", x, w, bias, residual, out, epilogue)


def gemv_mma(x, w, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    """Weight stream with mma.sync for 3..16 rows (dli_gemv_mma_bf16)."""
    return _linear("dli_gemv_mma_bf16", x, w, bias, residual, out, epilogue)


def gemm(x, w, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    return _linear("dli_gemm_bf16", x, w, bias, residual, out, epilogue)


def _gated(fn_name, x, w_gu, out):
    global launch_count
    _req(x), _req(w_gu), _req(out)
    M, K = x.shape
    F = w_gu.shape[0] // 2
    if out is None:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
    fn = getattr(_lib.load(), fn_name)
    _lib.check(fn_name, fn(_p(x), _p(w_gu), _p(out), M, F, K, _stream()))
    launch_count += (M + 3) // 4 if fn_name == "dli_gemv_gated_silu_bf16" else 1
    return out


def linear_gated_silu(x, w_gu, out=None):
    """silu(x @ Wg.T) * (x @ Wu.T) with w_gu = pack_gate_up(Wg, Wu)."""
    return _gated("dli_linear_gated_silu_bf16", x, w_gu, out)


def gemv_gated_silu(x, w_gu, out=None):
    return _gated("dli_gemv_gated_silu_bf16", x, w_gu, out)


def gemv_mma_gated_silu(x, w_gu, out=None):
    return _gated("dli_gemv_mma_gated_silu_bf16", x, w_gu, out)


def gemm_gated_silu(x, w_gu, out=None):
    return _gated("dli_gemm_gated_silu_bf16", x, w_gu, out)


def linear_gated_act(x, w_gu, act, scratch=None, out=None):
    """min(g, l) * sigmoid(a min(g, l)) * (clamp(u, -l, l) + 1) with g = x @ Wg.T, u = x @ Wu.T as the projection's epilogue;
    w_gu = pack_gate_up(Wg, Wu), act float32 [2] = (l, a) on the device; scratch: the split-K buffer (3..128 rows)."""
    global launch_count
    _req(x), _req(w_gu), _req(out), _req(act, torch.float32)
    M, K = x.shape
    F = w_gu.shape[0] // 2
    if out is None:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
    _lib.check("dli_linear_gated_act_bf16", _lib.load().dli_linear_gated_act_bf16(
        _p(x), _p(w_gu), _p(out), M, F, K, _p(act), _p(scratch), _bytes(scratch), _stream()))
    launch_count += (M + 3) // 4 if (M <= 2 or K % 64) else 1
    return out


def pack_gate_up(w_gate, w_up):
    """Interleave gate and up rows in blocks of 128 (layout dli.h documents)."""
    F, K = w_gate.shape
    if F % 128 != 0:
        raise ValueError("intermediate size must be a multiple of 128")
    g = w_gate.reshape(F // 128, 128, K)
    u = w_up.reshape(F // 128, 128, K)
    return torch.stack((g, u), dim=1).reshape(2 * F, K).contiguous()


def argmax(logits, out=None):
    """logits bf16 [B, V] (row stride may exceed V) -> int32 [B]."""
    global launch_count
    if logits.dtype != torch.bfloat16 or not logits.is_cuda or logits.stride(1) != 1:
        raise ValueError("argmax needs a CUDA bf16 tensor with unit inner stride")
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _lib.check("dli_argmax_bf16", _lib.load().dli_argmax_bf16(
        _p(logits), logits.stride(0), _p(out), B, V, _stream()))
    launch_count += 1
    return out


def decode_advance(tokens, token_log, positions, seq_lens, step):
    """Log sampled tokens and advance positions / lengths / step counter on device."""
    global launch_count
    for t in (tokens, token_log, positions, seq_lens, step):
        _req(t, torch.int32)
    B = tokens.numel()
    cap = 0 if token_log is None else token_log.numel() // max(B, 1)
    _lib.check("dli_decode_advance", _lib.load().dli_decode_advance(
        _p(tokens), _p(token_log), _p(positions), _p(seq_lens), _p(step), B, cap, _stream()))
    launch_count += 1


def set_pdl(enable: bool) -> bool:
    """Programmatic dependent launch for all subsequent kernel launches; returns the old setting."""
    return bool(_lib.load().dli_set_pdl(1 if enable else 0))


def _bytes(t):
    return 0 if t is None else t.numel() * t.element_size()


def paged_attn_decode_fused(qkv, cos, sin, k_cache, v_cache, page_table, seq_lens, out, H, KV, hd, scale,
                            num_splits=1, scratch=None, window=0, prefetch_a=None, prefetch_b=None):
    """RoPE + KV append of the new token + split-KV decode attention in one kernel (+ merge)."""
    global launch_count
    _req(qkv), _req(cos), _req(sin), _req(k_cache), _req(v_cache), _req(out)
    _req(page_table, torch.int32), _req(seq_lens, torch.int32)
    B = seq_lens.numel()
    page_size = k_cache.shape[2]
    sbytes = 0 if scratch is None else scratch.numel() * scratch.element_size()
    _lib.check("dli_paged_attn_decode_fused_bf16", _lib.load().dli_paged_attn_decode_fused_bf16(
        _p(qkv), qkv.shape[1], _p(cos), _p(sin), _p(k_cache), _p(v_cache), _p(page_table), page_table.shape[1],
        _p(seq_lens), _p(out), _p(scratch), sbytes, B, H, KV, hd, page_size, num_splits, float(scale), window,
        _p(prefetch_a), _bytes(prefetch_a), _p(prefetch_b), _bytes(prefetch_b), _stream()))
    launch_count += 2 if (num_splits > 1 and scratch is not None) else 1  # cluster merge: one kernel
    return out


def rmsnorm_linear(h, ln_w, eps, w, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    """epi(rmsnorm(h) * ln_w @ w.T) in one weight-streaming kernel (decode, M <= 4 per pass)."""
    global launch_count
    _req(h), _req(ln_w), _req(w), _req(bias), _req(residual), _req(out)
    M, K = h.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=h.device)
    epi = epilogue | (EPI_BIAS if bias is not None else 0) | (EPI_RESIDUAL if residual is not None else 0)
    _lib.check("dli_rmsnorm_gemv_bf16", _lib.load().dli_rmsnorm_gemv_bf16(
        _p(h), _p(ln_w), float(eps), _p(w), _p(bias), _p(residual), _p(out), M, N, K, epi, _stream()))
    launch_count += (M + 3) // 4
    return out


def rmsnorm_linear_gated_silu(h, ln_w, eps, w_gu, out=None):
    global launch_count
    _req(h), _req(ln_w), _req(w_gu), _req(out)
    M, K = h.shape
    F = w_gu.shape[0] // 2
    if out is None:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=h.device)
    _lib.check("dli_rmsnorm_gemv_gated_silu_bf16", _lib.load().dli_rmsnorm_gemv_gated_silu_bf16(
        _p(h), _p(ln_w), float(eps), _p(w_gu), _p(out), M, F, K, _stream()))
    launch_count += (M + 3) // 4
    return out


def gemm_splitk_scratch_bytes(M, N) -> int:
    return int(_lib.load().dli_gemm_splitk_scratch_bytes(M, N))


def linear_splitk(x, w, scratch, bias=None, residual=None, out=None, epilogue=EPI_NONE):
    """Batched-decode projection (4 < M <= 128): split-K tcgen05 weight stream.  `scratch` is a
    zero-initialised uint8/float tensor of gemm_splitk_scratch_bytes(M, N) bytes."""
    global launch_count
    _req(x), _req(w), _req(bias), _req(residual), _req(out)
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    epi = epilogue | (EPI_BIAS if bias is not None else 0) | (EPI_RESIDUAL if residual is not None else 0)
    _lib.check("dli_gemm_splitk_bf16", _lib.load().dli_gemm_splitk_bf16(
        _p(x), _p(w), _p(bias), _p(residual), _p(out), M, N, K, epi, _p(scratch), _bytes(scratch), _stream()))
    launch_count += 1
    return out


def linear_splitk_gated_silu(x, w_gu, scratch, out=None):
    global launch_count
    _req(x), _req(w_gu), _req(out)
    M, K = x.shape
    F = w_gu.shape[0] // 2
    if out is None:
        out = torch.empty(M, F, dtype=torch.bfloat16, device=x.device)
    _lib.check("dli_gemm_splitk_gated_silu_bf16", _lib.load().dli_gemm_splitk_gated_silu_bf16(
        _p(x), _p(w_gu), _p(out), M, F, K, _p(scratch), _bytes(scratch), _stream()))
    launch_count += 1
    return out


def sample(logits, out=None, temperature=0.8, top_k=50, top_p=0.95, seed=None, step=None, debug_cap=0):
    """Temperature -> top-k -> top-p -> multinomial on bf16 logits [B, V].
    seed: int64 device tensor [1]; step: int32 device tensor [1] (both optional).
    debug_cap > 0 additionally returns (probs [B, cap] fp32, ids [B, cap] int32) of the kept set."""
    global launch_count
    if logits.dtype != torch.bfloat16 or not logits.is_cuda or logits.stride(1) != 1:
        raise ValueError("sample needs a CUDA bf16 tensor with unit inner stride")
    _req(seed, torch.int64), _req(step, torch.int32)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    probs = ids = None
    if debug_cap:
        probs = torch.empty(B, debug_cap, dtype=torch.float32, device=logits.device)
        ids = torch.empty(B, debug_cap, dtype=torch.int32, device=logits.device)
    _lib.check("dli_sample_bf16", _lib.load().dli_sample_bf16(
        _p(logits), logits.stride(0), _p(out), B, V, float(temperature), int(top_k), float(top_p), _p(seed), _p(step),
        _p(probs), _p(ids), int(debug_cap), _stream()))
    launch_count += 1
    return (out, probs, ids) if debug_cap else out


def sample_rows(logits, out, seeds, steps, row_mask=None, temperature=0.8, top_k=50, top_p=0.95):
    """sample() for rows of different requests: per-row seeds (int64 [B]) and steps (int32 [B]); rows whose
    row_mask (int32 [B]) is 0 keep the token already in `out`."""
    global launch_count
    if logits.dtype != torch.bfloat16 or not logits.is_cuda or logits.stride(1) != 1:
        raise ValueError("sample_rows needs a CUDA bf16 tensor with unit inner stride")
    _req(seeds, torch.int64), _req(steps, torch.int32), _req(row_mask, torch.int32), _req(out, torch.int32)
    B, V = logits.shape
    _lib.check("dli_sample_rows_bf16", _lib.load().dli_sample_rows_bf16(
        _p(logits), logits.stride(0), _p(out), B, V, float(temperature), int(top_k), float(top_p), _p(seeds), _p(steps),
        _p(row_mask), _stream()))
    launch_count += 1
    return out


def argmax_candidate(logits, idx_offset, cand):
    """Best (logit, idx_offset + index) of each row of a logits slice -> cand [B, 2] float32."""
    global launch_count
    _req(cand, torch.float32)
    B, V = logits.shape
    _lib.check("dli_argmax_candidate_bf16", _lib.load().dli_argmax_candidate_bf16(
        _p(logits), logits.stride(0), int(idx_offset), _p(cand), B, V, _stream()))
    launch_count += 1
    return cand


def argmax_merge(cands, out):
    """cands [n, B, 2] float32 (per-slice candidates) -> out int32 [B]: the global greedy token."""
    global launch_count
    _req(cands, torch.float32), _req(out, torch.int32)
    n, B = cands.shape[0], cands.shape[1]
    _lib.check("dli_argmax_merge", _lib.load().dli_argmax_merge(_p(cands), n, B, _p(out), _stream()))
    launch_count += 1
    return out


def argmax_merge_strided(cands_ptr: int, n: int, B: int, n_stride: int, out):
    """argmax_merge over n candidate sets [B, 2] float32 that start n_stride floats apart (raw device pointer:
    the sets sit inside the pipeline's mailboxes)."""
    global launch_count
    _req(out, torch.int32)
    _lib.check("dli_argmax_merge_strided", _lib.load().dli_argmax_merge_strided(cands_ptr, n, B, n_stride, _p(out), _stream()))
    launch_count += 1
    return out


def gemv_argmax_scratch_bytes(M) -> int:
    return int(_lib.load().dli_gemv_argmax_scratch_bytes(M))


def linear_argmax(h, w, logits, scratch, tokens=None, cand=None, ln_w=None, eps=0.0, idx_offset=0):
    """lm_head for <= 4 rows with the greedy choice fused into the weight stream: logits = (rmsnorm(h) * ln_w
    if ln_w is given else h) @ w.T, and tokens[m] = idx_offset + argmax (or `cand` [M, 2] float32 = (best logit,
    idx_offset + index) for one vocabulary slice).  `scratch`: gemv_argmax_scratch_bytes(M) bytes."""
    global launch_count
    _req(h), _req(w), _req(logits), _req(ln_w), _req(tokens, torch.int32), _req(cand, torch.float32)
    M, K = h.shape
    N = w.shape[0]
    _lib.check("dli_gemv_argmax_bf16", _lib.load().dli_gemv_argmax_bf16(
        _p(h), _p(ln_w), float(eps), _p(w), _p(logits), M, N, K, int(idx_offset), _p(tokens), _p(cand), _p(scratch),
        _bytes(scratch), _stream()))
    launch_count += 2
    return tokens if tokens is not None else cand


# ---------------------------------------------------------------------------------------------------------------
# Ragged steps with an fp32 residual stream (ragged_rows.cu, attn_ragged.cu, mlstm.cu).  `dt` (0 = bf16, 1 = float)
# is the element type of weights, activations and caches; the wrappers take it from the tensors.
def _dt(t) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise ValueError(f"element type {t.dtype}: bf16 or float32")


def _call(name, n_launch, *args):
    global launch_count
    _lib.check(name, getattr(_lib.load(), name)(*args))
    launch_count += n_launch


def _f32(*ts):
    for t in ts:
        _req(t, torch.float32)


def _i32(*ts):
    for t in ts:
        _req(t, torch.int32)


def embedding_f32(ids, table, out, scale: float = 1.0, out2=None, out_e=None, row_ent=None, ent=None, inv_freq=None):
    """ids int32 [rows]; table [V, d] bf16 / float -> out float32 [rows, d] = table[ids] * scale (out2: a second copy;
    out_e: a copy in the table's element type).  inv_freq float32 [ceil(d/2)] with row_ent / ent: plus the sinusoidal
    position vector (sin(p f_i) at channel 2i, cos(p f_i) at 2i+1)."""
    _i32(ids, row_ent, ent), _req(table, table.dtype), _f32(out, out2, inv_freq), _req(out_e, table.dtype)
    if inv_freq is not None and inv_freq.numel() < (table.shape[1] + 1) // 2:
        raise ValueError("embedding_f32: one frequency per pair of channels")
    _call("dli_embedding_f32", 1, _p(ids), _p(table), _p(out), _p(out2), _p(out_e), ids.numel(), table.shape[1],
          table.shape[0], float(scale), _dt(table), _p(row_ent), _p(ent), _p(inv_freq), _stream())
    return out


def group_rmsnorm(x, w, groups: int, eps: float, hn=None, he=None):
    """RMS norm of x float32 [rows, d] in `groups` equal parts, times w float32 [d] -> hn (float32) and / or he
    (bf16 / float32)."""
    _f32(x, w, hn)
    if he is not None:
        _req(he, he.dtype)
    _call("dli_group_rmsnorm", 1, _p(x), _p(w), _p(hn), _p(he), x.shape[0], x.shape[1], int(groups), float(eps),
          _dt(he) if he is not None else 1, _stream())


def group_rmsnorm_conv_single(x, w, groups, eps, tail, conv_w, ent, hc, hn=None, he=None):
    """Decode rows (one per entry): group_rmsnorm (-> hn, he) and causal_conv_ragged of the normed row (-> hc, the slot's
    tail shifted) as one kernel."""
    _f32(x, w, hn, tail, conv_w), _i32(ent), _req(hc, hc.dtype), _req(he, hc.dtype)
    _call("dli_group_rmsnorm_conv_single", 1, _p(x), _p(w), _p(hn), _p(he), _p(tail), _p(conv_w), _p(ent), _p(hc),
          x.shape[0], x.shape[1], int(groups), float(eps), conv_w.shape[1], _dt(hc), _stream())


def residual_add2(x, y1, y2=None, a=None, h=None):
    """x += y1 + y2 + a[:, None] * h (x, a, h float32; y1, y2 in one element type)."""
    _f32(x, a, h), _req(y1, y1.dtype), _req(y2, y1.dtype)
    _call("dli_residual_add2", 1, _p(x), _p(y1), _p(y2), _p(a), _p(h), x.shape[0], x.shape[1], _dt(y1), _stream())
    return x


def concat_cast(a, b, out):
    """out [rows, 2d] = [a | b] (a, b float32) in out's element type."""
    _f32(a, b), _req(out, out.dtype)
    _call("dli_concat_cast", 1, _p(a), _p(b), _p(out), a.shape[0], a.shape[1], _dt(out), _stream())
    return out


def rows_bias_f32(y, bias, x):
    """x = y + bias (x, bias float32)."""
    _req(y, y.dtype), _f32(bias, x)
    _call("dli_rows_bias_f32", 1, _p(y), _p(bias), _p(x), x.shape[0], x.shape[1], _dt(y), _stream())
    return x


def scalar_rmsnorm(x, g: float, eps: float, out):
    """out = x / sqrt(mean(x^2) + eps) * g (one weight per norm); x, out float32 [rows, d]."""
    _f32(x, out)
    _call("dli_scalar_rmsnorm_f32", 1, _p(x), _p(out), x.shape[0], x.shape[1], float(eps), float(g), _stream())
    return out


def postnorm_add_norm(y, x, g_post: float, eps: float, hn=None, g_next: float = 1.0):
    """x += y / rms(y) * g_post (x float32, in place); hn = x / rms(x) * g_next when hn is given."""
    _req(y, y.dtype), _f32(x, hn)
    _call("dli_postnorm_add_norm", 1, _p(y), _p(x), _p(hn), x.shape[0], x.shape[1], float(eps), float(g_post),
          float(g_next), _dt(y), _stream())
    return x


def causal_conv_ragged(h, tail, w, row_ent, ent, out):
    """out = h + conv(h) over time per channel (w float32 [d, taps]); tail float32 [slots, taps-1, d] is advanced."""
    _f32(h, tail, w), _i32(row_ent, ent), _req(out, out.dtype)
    taps = w.shape[1]
    single = h.shape[0] == ent.numel() // 4  # one row per entry: convolution and tail shift are one kernel
    _call("dli_causal_conv_ragged", 2 if (taps > 1 and not single) else 1, _p(h), _p(tail), _p(w), _p(row_ent), _p(ent), _p(out),
          h.shape[0], ent.numel() // 4, h.shape[1], taps, _dt(out), _stream())
    return out


def gather_cast(src, rows, out):
    """out[i] = src[rows[i]] cast to out's element type; src float32 [n, d]."""
    _f32(src), _i32(rows), _req(out, out.dtype)
    _call("dli_gather_cast", 1, _p(src), _p(rows), _p(out), rows.numel(), src.shape[1], _dt(out), _stream())
    return out


def linear_any(x, w, out):
    """out = x @ w.T on the CUDA cores (fp32 accumulation; true fp32 for float operands).  Any shape; x and out
    may be row-strided views."""
    if x.dtype != w.dtype or out.dtype != w.dtype or not w.is_contiguous() or x.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("linear_any: one element type, unit inner strides")
    M, K = x.shape
    _call("dli_linear_any", 1, _p(x), _p(w), _p(out), M, w.shape[0], K, x.stride(0), out.stride(0), _dt(w), _stream())
    return out


def silu_mul(gu, out, bias=None):
    """out[m, f] = silu(gu[m, f] + b[f]) * (gu[m, F + f] + b[F + f]); bias float32 [2F] or None."""
    _req(gu, gu.dtype), _req(out, gu.dtype), _f32(bias)
    _call("dli_silu_mul", 1, _p(gu), _p(out), gu.shape[0], out.shape[1], gu.shape[1], _dt(gu), _p(bias), _stream())
    return out


def attn_prep_append(proj, qbuf, k_cache, v_cache, row_ent, ent, page_table, H, G, D, V, rd, q_off, k_off, v_off,
                     q_norm, k_norm, eps, cos_qk, sin_qk, cos_v, sin_v, bias=None, q_only=False):
    """q/k head norms, rotation and value rotation of a ragged step; q -> qbuf (float32), k / v -> the paged caches.
    bias float32 (indexed like proj's columns) is added first; q_only: no keys or values are made or appended (the caches
    are only asked for their page size)."""
    _req(proj, proj.dtype), _req(k_cache, proj.dtype), _req(v_cache, proj.dtype)
    _f32(qbuf, q_norm, k_norm, cos_qk, sin_qk, cos_v, sin_v, bias), _i32(row_ent, ent, page_table)
    tl = cos_qk.shape[0] if cos_qk is not None else (cos_v.shape[0] if cos_v is not None else 0)
    _call("dli_attn_prep_append", 1, _p(proj), _p(qbuf), _p(k_cache), _p(v_cache), _p(row_ent), _p(ent), _p(page_table),
          page_table.shape[1], k_cache.shape[2], proj.shape[0], H, G, D, V, rd, proj.shape[1], q_off, k_off, v_off,
          _p(q_norm), _p(k_norm), float(eps), _p(cos_qk), _p(sin_qk), _p(cos_v), _p(sin_v), tl, _dt(proj), _p(bias),
          1 if q_only else 0, _stream())


def attn_ragged(qbuf, k_cache, v_cache, proj, out, row_ent, ent, page_table, H, G, D, V, scale, chunk=0, window=0,
                sink=None, g_off=-1, cos_v=None, sin_v=None, ldv=0, splits=1, part=None, first=0, r1=None, r2=None):
    """Chunk- / window-masked attention with an optional sink and output gate over the paged cache -> out [rows, H*V].
    r1, r2 float32 [H]: the distance penalty r1 ln(1 + r2 (i - j)) on the scaled scores.
    first: positions below it stay visible whatever the chunk or window says.
    ldv: elements between value rows (0 = V); v_cache may be k_cache itself (values = leading part of the keys).
    splits > 1: every row's keys are dealt to that many CTAs; part: float32 scratch of rows * H * splits * (V + 2)."""
    _f32(qbuf, sink, cos_v, sin_v, part, r1, r2), _i32(row_ent, ent, page_table), _req(out, k_cache.dtype), _req(proj, k_cache.dtype)
    if splits > 1 and part.numel() < qbuf.shape[0] * H * splits * (V + 2):
        raise ValueError("attn_ragged: scratch too small for the key splits")
    _call("dli_attn_ragged", 2 if splits > 1 else 1, _p(qbuf), _p(k_cache), _p(v_cache), _p(proj), _p(out), _p(row_ent), _p(ent),
          _p(page_table), page_table.shape[1], k_cache.shape[2], qbuf.shape[0], H, G, D, V, float(scale), int(chunk),
          int(window), int(first), _p(sink), proj.shape[1] if proj is not None else 0, g_off, _p(cos_v), _p(sin_v), int(ldv),
          int(splits), _p(part), _dt(k_cache), _p(r1), _p(r2), _stream())
    return out


def attn_ragged_tc_supported(D, V, dtype) -> bool:
    return dtype == torch.bfloat16 and bool(_lib.load().dli_attn_ragged_tc_supported(int(D), int(V), 0))


def attn_ragged_tc(qbuf, k_cache, v_cache, proj, out, ent, tiles, page_table, H, G, D, V, scale, chunk=0, window=0,
                   sink=None, g_off=-1, cos_v=None, sin_v=None, page_base=0, first=0, r1=None, r2=None):
    """attn_ragged for steps with portions of prompts, on the tensor cores: tiles int32 [n_tiles, 2] = (entry, first
    row of the 64-row query tile within the entry).  page_base: k_cache / v_cache hold pages page_base.. of the pool only
    (the pages the step's sequences use must all lie in that range)."""
    _f32(qbuf, sink, cos_v, sin_v, r1, r2), _i32(ent, tiles, page_table), _req(out), _req(proj), _req(k_cache), _req(v_cache)
    kb = page_base * k_cache.stride(0) * k_cache.element_size()
    vb = page_base * v_cache.stride(0) * v_cache.element_size()
    _call("dli_attn_ragged_tc", 1, _p(qbuf), _p(k_cache) - kb, _p(v_cache) - vb, _p(proj), _p(out), _p(ent), _p(tiles),
          tiles.numel() // 2, _p(page_table), page_table.shape[1], k_cache.shape[2], H, G, D, V, float(scale), int(chunk),
          int(window), int(first), _p(sink), proj.shape[1] if proj is not None else 0, g_off, _p(cos_v), _p(sin_v), _p(r1),
          _p(r2), _stream())
    return out


def mlstm_ragged(proj, o_scratch, out, ent, H, D, V, q_off, k_off, v_off, i_off, f_off, g_off, i_bias, f_bias, cap,
                 out_w, eps, S, n, m, blocked=False):
    """Matrix-memory recurrence over the rows of every entry + head norm, weight and output gate -> out [rows, H*V]."""
    _req(proj, proj.dtype), _req(out, proj.dtype), _f32(o_scratch, i_bias, f_bias, out_w, S, n, m), _i32(ent)
    _call("dli_mlstm_ragged", 2, _p(proj), _p(o_scratch), _p(out), _p(ent), ent.numel() // 4, proj.shape[0], H, D, V,
          proj.shape[1], q_off, k_off, v_off, i_off, f_off, g_off, _p(i_bias), _p(f_bias), float(cap), _p(out_w),
          float(eps), _p(S), _p(n), _p(m), int(bool(blocked)), _dt(proj), _stream())
    return out


def mlstm_parallel_scratch_floats(n_tiles, H, D, V) -> int:
    return int(_lib.load().dli_mlstm_parallel_scratch_floats(int(n_tiles), int(H), int(D), int(V)))


def mlstm_ragged_parallel(proj, o_scratch, out, ent, tiles, scratch, H, D, V, q_off, k_off, v_off, i_off, f_off, g_off,
                          i_bias, f_bias, cap, out_w, eps, S, n, m):
    """mlstm_ragged for steps with long portions: the 64-position blocks of every entry run in parallel (local state
    contributions, an ordered elementwise carry, read-outs).  tiles int32 [n_tiles, 2] = (entry, first row of the block
    within the entry), blocks of an entry consecutive; scratch: mlstm_parallel_scratch_floats(...) float32."""
    _req(proj, proj.dtype), _req(out, proj.dtype), _f32(o_scratch, i_bias, f_bias, out_w, S, n, m, scratch), _i32(ent, tiles)
    n_tiles = tiles.numel() // 2
    if scratch.numel() < mlstm_parallel_scratch_floats(n_tiles, H, D, V):
        raise ValueError("mlstm_ragged_parallel: scratch too small")
    _call("dli_mlstm_ragged_parallel", 4, _p(proj), _p(o_scratch), _p(out), _p(ent), ent.numel() // 4, _p(tiles), n_tiles,
          _p(scratch), proj.shape[0], H, D, V, proj.shape[1], q_off, k_off, v_off, i_off, f_off, g_off, _p(i_bias),
          _p(f_bias), float(cap), _p(out_w), float(eps), _p(S), _p(n), _p(m), _dt(proj), _stream())
    return out


def postnorm_add_norm_conv_single(y, x, tail, w, ent, out, g_post: float, g_next: float, eps: float):
    """Decode rows (one per entry): x += y / rms(y) * g_post (skipped when y is None), h = x / rms(x) * g_next,
    out = h + conv(h) with the slot's tail shifted — postnorm_add_norm and the next sublayer's causal_conv_ragged
    as one kernel."""
    _f32(x, tail, w), _i32(ent), _req(out, out.dtype)
    if y is not None:
        _req(y, out.dtype)
    _call("dli_postnorm_add_norm_conv_single", 1, _p(y), _p(x), _p(tail), _p(w), _p(ent), _p(out), x.shape[0], x.shape[1],
          w.shape[1], float(eps), float(g_post), float(g_next), _dt(out), _stream())
    return out


# ---------------------------------------------------------------------------------------------------------------
# Latent attention, state-space mixer, mixture of experts (latent_attn.cu, mamba2.cu, moe.cu)
def latent_prep(proj, cq, pool, row_ent, ent, page_table, Q, K, R, q_off, kv_off, q_norm, kv_norm, eps, cos_t, sin_t,
                halves=False):
    """Query latent (normed) -> cq [rows, Q] (Q == 0: none); key/value latent (normed) and the rotated shared key part
    -> the pool [pages, 1, page_size, K + R].  halves: rotation pairs (i, i + R/2) instead of (2i, 2i+1)."""
    _req(proj, proj.dtype), _req(cq, proj.dtype), _req(pool, proj.dtype)
    _f32(q_norm, kv_norm, cos_t, sin_t), _i32(row_ent, ent, page_table)
    _call("dli_latent_prep", 1, _p(proj), _p(cq), _p(pool), _p(row_ent), _p(ent), _p(page_table), page_table.shape[1],
          pool.shape[2], proj.shape[0], Q, K, R, proj.shape[1], q_off, kv_off, _p(q_norm), _p(kv_norm), float(eps),
          _p(cos_t), _p(sin_t), cos_t.shape[0] if cos_t is not None else 0, int(bool(halves)), _dt(proj), _stream())


def latent_q_absorb(q, uk, qbuf, row_ent, ent, cos_t, sin_t, H, D, R, K, halves=False):
    """q [rows, H*(D+R)] (or the leading columns of a wider row-major matrix), uk [H*D, K] -> qbuf float32
    [rows, H*(K+R)] = per head [uk[h]^T q_n | rot(q_r)]; uk None (K == D): [q_n | rot(q_r)]."""
    if q.stride(1) != 1 or not q.is_cuda:
        raise ValueError("latent_q_absorb: q needs unit inner stride on the device")
    _req(uk, q.dtype), _f32(qbuf, cos_t, sin_t), _i32(row_ent, ent)
    _call("dli_latent_q_absorb", 1, _p(q), _p(uk), _p(qbuf), _p(row_ent), _p(ent), _p(cos_t), _p(sin_t), q.shape[0], H, D,
          R, K, int(bool(halves)), q.stride(0), _dt(q), _stream())
    return qbuf


def latent_v_up(o, uv, proj, out, H, V, K, g_off=-1):
    """o [rows, H*K], uv [H*V, K] -> out [rows, H*V] = (uv[h] o[h]) * sigmoid(proj[:, g_off + h*V + v])."""
    _req(o, o.dtype), _req(uv, o.dtype), _req(out, o.dtype), _req(proj, o.dtype)
    _call("dli_latent_v_up", 1, _p(o), _p(uv), _p(proj), _p(out), o.shape[0], H, V, K,
          proj.shape[1] if proj is not None else 0, g_off, _dt(o), _stream())
    return out


def latent_expand(kv, pool_rows, kx, vx, H, D, R, V, K, page_size):
    """kv [n, H*D + H*V] (up-projections of n consecutive pool rows) and those rows [n, K+R] -> per-head key and
    value pools kx [n/page_size, H, page_size, D+R], vx [n/page_size, H, page_size, V]."""
    _req(kv, kv.dtype), _req(pool_rows, kv.dtype), _req(kx, kv.dtype), _req(vx, kv.dtype)
    _call("dli_latent_expand", 1, _p(kv), _p(pool_rows), _p(kx), _p(vx), kv.shape[0], H, D, R, V, K, page_size, _dt(kv),
          _stream())


def sigmoid_gate(out, proj, g_off):
    """out[row, c] *= sigmoid(proj[row, g_off + c])."""
    _req(out, out.dtype), _req(proj, out.dtype)
    _call("dli_sigmoid_gate", 1, _p(out), _p(proj), out.shape[0], out.shape[1], proj.shape[1], g_off, _dt(out), _stream())
    return out


def conv1d_act_ragged(proj, tail, w, bias, row_ent, ent, out, off, act=1):
    """Causal per-channel convolution (+ bias, SiLU) over columns [off, off + C) of proj -> out float32 [rows, C]; the
    slots' histories tail float32 [slots, taps-1, C] are advanced."""
    _req(proj, proj.dtype), _f32(tail, w, bias, out), _i32(row_ent, ent)
    C, taps = w.shape
    _call("dli_conv1d_act_ragged", 2 if (taps > 1 and proj.shape[0] != ent.numel() // 4) else 1, _p(proj), _p(tail), _p(w), _p(bias), _p(row_ent), _p(ent), _p(out),
          proj.shape[0], ent.numel() // 4, C, taps, proj.shape[1], off, int(act), _dt(proj), _stream())
    return out


def ssm_parallel_scratch_floats(n_tiles, H, N, V) -> int:
    return int(_lib.load().dli_ssm_parallel_scratch_floats(int(n_tiles), int(H), int(N), int(V)))


def ssm_scan_ragged(xbc, proj, S, y, ent, H, V, N, G, dt_off, dt_bias, a_log, d_skip, blocked=False, tiles=None,
                    scratch=None):
    """The state-space recurrence over the rows of every entry; S float32 [slots, H, N, V] is advanced; y float32
    [rows, H*V].  blocked: 64 rows at a time (steps with portions of prompts); with tiles int32 [n_tiles, 2] = (entry,
    first row of the block within the entry) and scratch of ssm_parallel_scratch_floats(...) floats the blocks of an
    entry run in parallel."""
    _f32(xbc, S, y, dt_bias, a_log, d_skip, scratch), _req(proj, proj.dtype), _i32(ent, tiles)
    n_ent = ent.numel() // 4
    n_tiles = tiles.numel() // 2 if tiles is not None else 0
    par = bool(blocked) and tiles is not None and scratch is not None and n_tiles > n_ent
    if par and scratch.numel() < ssm_parallel_scratch_floats(n_tiles, H, N, V):
        raise ValueError("ssm_scan_ragged: scratch too small")
    _call("dli_ssm_scan_ragged", 3 if par else 1, _p(xbc), _p(proj), _p(S), _p(y), _p(ent), n_ent, H, V, N, G, proj.shape[1],
          dt_off, _p(dt_bias), _p(a_log), _p(d_skip), int(bool(blocked)), _p(tiles) if par else None, n_tiles if par else 0,
          _p(scratch) if par else None, _dt(proj), _stream())
    return y


def gated_group_rmsnorm(y, proj, w, out, groups, eps, z_off):
    """out = groupnorm(y * silu(proj[:, z_off : z_off + d])) * w."""
    _f32(y, w), _req(proj, proj.dtype), _req(out, proj.dtype)
    _call("dli_gated_group_rmsnorm", 1, _p(y), _p(proj), _p(w), _p(out), y.shape[0], y.shape[1], int(groups), float(eps),
          proj.shape[1], z_off, _dt(proj), _stream())
    return out


def moe_route(h, w_router, correction, wts, idw, sel_idx, sel_w, n_real, top, groups=1, keep=1, wscale=1.0, renorm=True):
    """Router of a mixture of experts on float32 rows: dense weights wts [rows, n_real], pass-through weight idw [rows],
    the choice sel_idx / sel_w [rows, top].  groups > 1: only outputs of the `keep` best of that many equal groups can be
    chosen; renorm False: the weights are the scores themselves; both times wscale."""
    _f32(h, w_router, correction, wts, idw, sel_w), _i32(sel_idx)
    _call("dli_moe_route", 1, _p(h), _p(w_router), _p(correction), _p(wts), _p(idw), _p(sel_idx), _p(sel_w), h.shape[0],
          h.shape[1], w_router.shape[0], int(n_real), int(top), int(groups), int(keep), float(wscale), 1 if renorm else 0,
          _stream())


def moe_act(gu, wts, act, n_exp, ff, limit, ff_s=0, limit_s=0.0, alpha=1.702, gated=True):
    """Activation of all experts' stacked projections, times the routing weights: the clamped gated form on [gate; up] rows,
    or (gated False) max(u, 0)^2 on up rows alone."""
    _req(gu, gu.dtype), _req(act, gu.dtype), _f32(wts)
    _call("dli_moe_act", 1, _p(gu), _p(wts), _p(act), gu.shape[0], int(n_exp), int(ff), float(limit), int(ff_s),
          float(limit_s), float(alpha), gu.shape[1], _dt(gu), 0 if gated else 1, _stream())
    return act


def moe_sel_supported(d, ff, ff_s, top) -> bool:
    return bool(_lib.load().dli_moe_sel_supported(int(d), int(ff), int(ff_s), int(top)))


def moe_sel(x, w_gu, w_down, sel_idx, sel_w, act_sel, y, n_exp, top, ff, limit, ff_s=0, limit_s=0.0, alpha=1.702, gated=True):
    """Few rows (decode): the chosen experts' and the shared expert's weights only -> y [rows, d] (bf16)."""
    _req(x), _req(w_gu), _req(w_down), _req(act_sel), _req(y), _i32(sel_idx), _f32(sel_w)
    _call("dli_moe_sel_bf16", 2, _p(x), _p(w_gu), _p(w_down), _p(sel_idx), _p(sel_w), _p(act_sel), _p(y), x.shape[0],
          x.shape[1], int(n_exp), int(top), int(ff), float(limit), int(ff_s), float(limit_s), float(alpha), 0 if gated else 1,
          _stream())
    return y


# ---------------------------------------------------------------------------------------------------------------
# Pre-norm layers with layer scale, token shift and depth average (prenorm_rows.cu)
def layer_close(x, y=None, bias=None, idw=None, h_in=None, ls=None, xs=None, n_prev=0, dwa=None, w_next=None, shift=None,
                tail=None, ent=None, out_f=None, out_e=None, eps: float = 1e-6, route=None):
    """x += ls * (y + bias + idw[:, None] * h_in) (x float32 in place; y in the element type); with dwa (float32 [n_prev + 1])
    the result is stored as xs[n_prev] and x becomes sum_j dwa[j] * xs[j] (xs float32 [n, rows_cap, d]); with w_next the
    normed x goes to out_f (float32) / out_e (element type); shift (steps of one row per entry): the normed row is mixed
    with the slot's stored row (tail float32 [slots, d]), which it replaces.  route: moe_route's arguments after h as a
    dict (w_router, correction, wts, idw, sel_idx, sel_w, n_real, top, groups, keep, wscale, renorm) — the router then runs on
    the rows of out_f in the same kernel."""
    _f32(x, bias, idw, h_in, ls, xs, dwa, w_next, shift, tail, out_f), _i32(ent)
    r = route or {}
    if route is not None:
        _f32(r["w_router"], r.get("correction"), r["wts"], r["idw"], r["sel_w"]), _i32(r["sel_idx"])
        if out_f is None or r["w_router"].shape[1] != x.shape[1]:
            raise ValueError("layer_close: the router reads the float32 normed rows")
    for t in (y, out_e):
        if t is not None:
            _req(t, t.dtype)
    ref = y if y is not None else out_e
    if dwa is not None and (xs is None or xs.shape[0] <= n_prev or dwa.numel() < n_prev + 1):
        raise ValueError("layer_close: the depth average needs n_prev + 1 weights and stored results")
    _call("dli_layer_close", 1, _p(y), _p(bias), _p(idw), _p(h_in), _p(ls), _p(x), _p(xs), xs.stride(0) if xs is not None else 0,
          int(n_prev), _p(dwa), _p(w_next), _p(shift), _p(tail), _p(ent), _p(out_f), _p(out_e), x.shape[0], x.shape[1],
          float(eps), _dt(ref) if ref is not None else 1, _p(r.get("w_router")), _p(r.get("correction")), _p(r.get("wts")),
          _p(r.get("idw")), _p(r.get("sel_idx")), _p(r.get("sel_w")), r["w_router"].shape[0] if route is not None else 0,
          int(r.get("n_real", 0)), int(r.get("top", 0)), int(r.get("groups", 1)), int(r.get("keep", 1)),
          float(r.get("wscale", 1.0)), 1 if r.get("renorm", True) else 0, _stream())
    return x


def token_shift_ragged(h, shift, tail, row_ent, ent, out):
    """out = h + (previous row - h) * shift per channel; h float32 [rows, d] normed rows; an entry's first row takes the
    slot's stored row (zeros at position 0) and stores the entry's last row in its place."""
    _f32(h, shift, tail), _i32(row_ent, ent), _req(out, out.dtype)
    _call("dli_token_shift_ragged", 1, _p(h), _p(shift), _p(tail), _p(row_ent), _p(ent), _p(out), h.shape[0], h.shape[1],
          _dt(out), _stream())
    return out


# ---------------------------------------------------------------------------------------------------------------
# Layers normed on their sublayers' outputs only, per-layer token input, gated delta rule (ragged_rows.cu, delta_rule.cu)
def postnorm_vec_add(y, x, w, eps: float, he=None):
    """x += y / rms(y) * w (x float32 in place, w float32 [d]; y None: x stays); he = x in its element type when given."""
    _f32(x, w)
    for t in (y, he):
        if t is not None:
            _req(t, t.dtype)
    ref = y if y is not None else he
    _call("dli_postnorm_vec_add", 1, _p(y), _p(x), _p(w), _p(he), x.shape[0], x.shape[1], float(eps), _dt(ref), _stream())
    return x


def token_side_act(s, ids, table, off: int, out):
    """out [rows, n] = gelu_tanh(s) * table[ids, off : off + n]."""
    _req(s, s.dtype), _req(table, s.dtype), _req(out, s.dtype), _i32(ids)
    _call("dli_token_side_act", 1, _p(s), _p(ids), _p(table), _p(out), s.shape[0], s.shape[1], table.shape[1], int(off),
          table.shape[0], _dt(s), _stream())
    return out


def token_side_gate(x, ids, table, off: int, w_gate, out):
    """Few rows: out [rows, n] = gelu_tanh(x @ w_gate.T) * table[ids, off : off + n] in one kernel (x float32)."""
    _f32(x), _i32(ids), _req(table, table.dtype), _req(w_gate, table.dtype), _req(out, table.dtype)
    _call("dli_token_side_gate", 1, _p(x), _p(ids), _p(table), _p(w_gate), _p(out), x.shape[0], x.shape[1], w_gate.shape[0],
          table.shape[1], int(off), table.shape[0], _dt(table), _stream())
    return out


def token_side(x, ids, table, off: int, w_gate, w_proj, w, eps: float, he=None):
    """Few rows: x += rmsnorm(w_proj (gelu_tanh(w_gate x) * table[ids, off : off + n])) * w in one kernel; he = x."""
    _f32(x, w), _i32(ids), _req(table, table.dtype), _req(w_gate, table.dtype), _req(w_proj, table.dtype)
    if he is not None:
        _req(he, table.dtype)
    _call("dli_token_side", 1, _p(x), _p(ids), _p(table), _p(w_gate), _p(w_proj), _p(w), _p(he), x.shape[0], x.shape[1],
          w_gate.shape[0], table.shape[1], int(off), table.shape[0], float(eps), _dt(table), _stream())
    return x


def delta_rule_ragged(qkv, proj, St, o, ent, H, G, D, V, b_off, a_off, a_log, dt_bias, q_scale, unit_eps=1e-6, blocked=False):
    """Gated delta rule over the rows of every entry.  qkv float32 [rows, 2*G*D + H*V] = q | k | v; St float32
    [slots, H, V, D] (the transposed state) is advanced; o float32 [rows, H*V].  blocked: 16 rows at a time (steps with portions
    of prompts)."""
    _f32(qkv, St, o, a_log, dt_bias), _req(proj, proj.dtype), _i32(ent)
    _call("dli_delta_rule_ragged", 1, _p(qkv), _p(proj), _p(St), _p(o), _p(ent), ent.numel() // 4, H, G, D, V, qkv.shape[1],
          proj.shape[1], b_off, a_off, _p(a_log), _p(dt_bias), float(q_scale), float(unit_eps), int(bool(blocked)), _dt(proj), _stream())
    return o


def head_rmsnorm_gate(o, proj, w, out, H, V, eps, gate=1, g_off=0):
    """out [rows, H*V] = o / rms_head(o) * w * act(proj[:, g_off + h*V + v]); w float32 [V] (shared) or [H*V];
    gate 0 none, 1 SiLU, 2 sigmoid."""
    _f32(o, w), _req(out, out.dtype)
    if proj is not None:
        _req(proj, out.dtype)
    _call("dli_head_rmsnorm_gate", 1, _p(o), _p(proj), _p(w), _p(out), o.shape[0], H, V, float(eps),
          int(w.numel() == H * V and H > 1), int(gate), proj.shape[1] if proj is not None else 0, int(g_off), _dt(out), _stream())
    return out
