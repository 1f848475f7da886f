"""Model registry: which engine serves a model directory.

config.json decides: `model_type` llama / mistral / gpt2 -> engine.ShardEngine (uniform stacks, Hugging Face tensor
names); `architecture` Sokevik, Togalorn, Fubepel or Gimudra -> ragged_engine.RaggedEngine with the layer list that sokevik.py /
togalorn.py / fubepel.py / gimudra.py read from the configuration.  The worker, the trace replayer (bin/trace_run) and bench.py all come
through here.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch


def read_config(path: str) -> dict:
    with open(os.path.join(path, "config.json")) as f:
        return json.load(f)


# designs described layer by layer, served by RaggedEngine: architecture -> module with spec_from_config,
# model_tensors and random_state_dict
LAYERWISE = {"Sokevik": "sokevik", "Togalorn": "togalorn", "Fubepel": "fubepel", "Gimudra": "gimudra"}


def family(cfg: dict) -> str:
    if cfg.get("architecture") in LAYERWISE:
        return LAYERWISE[cfg["architecture"]]
    if cfg.get("model_type") in ("llama", "mistral", "gpt2"):
        return "uniform"
    raise ValueError(f"unsupported model: model_type {cfg.get('model_type')!r}, architecture {cfg.get('architecture')!r} "
                     f"(llama, mistral, gpt2, {', '.join(LAYERWISE)})")


def definition(cfg: dict):
    """The module that defines a layer-by-layer design, None for the uniform stacks."""
    fam = family(cfg)
    if fam == "uniform":
        return None
    import importlib
    return importlib.import_module("." + fam, __package__)


def supports_float32(cfg: dict) -> bool:
    """RaggedEngine has a true-fp32 mode; the uniform-stack engine is bf16 only."""
    return family(cfg) != "uniform"


def spec_from_config(cfg: dict):
    mod = definition(cfg)
    if mod is not None:
        return mod.spec_from_config(cfg)
    from .engine import ModelSpec
    return ModelSpec.from_hf_config(cfg)


def read_all_tensors(path: str) -> Dict[str, torch.Tensor]:
    from .sharding import _tensor_files
    out: Dict[str, torch.Tensor] = {}
    for f in _tensor_files(path):
        if f.endswith(".safetensors"):
            from safetensors import safe_open

            with safe_open(f, framework="pt", device="cpu") as sf:
                for name in sf.keys():
                    out[name] = sf.get_tensor(name)
        else:
            out.update(torch.load(f, map_location="cpu", weights_only=True))
    return out


def load_engine(path: str, device: str = "cuda:0", max_batch: int = 1, max_seq_len: int = 4096,
                kv_pool_tokens: Optional[int] = None, dtype=torch.bfloat16):
    """A full-range engine with the directory's weights loaded."""
    cfg = read_config(path)
    spec = spec_from_config(cfg)
    mod = definition(cfg)
    if mod is not None:
        from .ragged_engine import RaggedEngine

        eng = RaggedEngine(spec, device=device, max_batch=max_batch, max_seq_len=max_seq_len,
                           kv_pool_tokens=kv_pool_tokens, dtype=dtype)
        eng.load_tensors(mod.model_tensors(spec, read_all_tensors(path)))
        return eng
    if dtype != torch.bfloat16:
        raise ValueError("the uniform-stack engine runs in bfloat16 only")
    from .engine import ShardEngine
    from .sharding import load_hf_state_dict

    eng = ShardEngine(spec, device=device, max_batch=max_batch, max_seq_len=min(max_seq_len, spec.max_pos),
                      kv_pool_tokens=kv_pool_tokens)
    eng.load_state_dict(load_hf_state_dict(path, 0, None, spec.n_layers))
    return eng
