"""Model registry: which native engine runs a model directory, chosen from its config.json.

Two engines exist.  `NativeShard` (libxotb200.so) runs Llama-style and Mixtral shards through one persistent kernel; its config
is the Hugging Face one (`model_type`, `num_hidden_layers`, ...).  `LayeredShard` (libxotb200_lm.so) runs models given as a list
of layers with different token mixers; its config names the family in `architecture`.  Everything above the native object — the
`InferenceEngine`, the Cheetah service, the schedulers, the trace replayer — asks this module and never names a class itself.

`model_summary` gives the few numbers the callers need whatever the config's dialect is (depth, vocabulary, width, context)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

NO_CONTEXT_LIMIT = 1 << 30     # families without a trained context length (rotations are computed from the position, no table)


def load_model_config(model_dir) -> dict:
  with open(Path(model_dir) / "config.json", "r") as f:
    return json.load(f)


def is_layered(config: dict) -> bool:
  from .layered import LAYERED_FAMILIES
  return config.get("architecture") in LAYERED_FAMILIES


def model_summary(config: dict) -> dict:
  """{"n_layers", "vocab", "width", "max_positions", "engine"} of a config in either dialect"""
  if is_layered(config):
    from .layered import LAYERED_FAMILIES
    g = LAYERED_FAMILIES[config["architecture"]][1](config)
    return {"n_layers": len(config["layers"]), "vocab": g["vocab"], "width": g["width"],
            "max_positions": g.get("max_positions") or NO_CONTEXT_LIMIT, "engine": "layered"}
  if "num_hidden_layers" in config:
    return {"n_layers": int(config["num_hidden_layers"]), "vocab": int(config["vocab_size"]), "width": int(config["hidden_size"]),
            "max_positions": int(config.get("max_position_embeddings", NO_CONTEXT_LIMIT)), "engine": "shard"}
  raise ValueError(f"config.json describes no model family known here (architecture={config.get('architecture')!r}, "
                   f"model_type={config.get('model_type')!r})")


def make_native(config: dict, device: int = 0, dtype: Optional[str] = None):
  """the native engine object for a config; `dtype` None = the dtype the family is served in"""
  if is_layered(config):
    from .layered import LayeredShard
    return LayeredShard(config, device, dtype or "bfloat16")
  if "num_hidden_layers" in config:
    if dtype not in (None, "bfloat16", "float16"):
      raise ValueError(f"the shard engine runs 16-bit weights (bfloat16 / float16 as the checkpoint says), not {dtype}")
    from .native import NativeShard
    return NativeShard(config, device)
  model_summary(config)   # raises with the reason
