"""Helpers of the layered-engine tests: small Zokuvik configurations, the bridge from the oracle's random weights to a
`LayeredShard`, schedules (whole / portions / token by token) and the error measure."""
from __future__ import annotations

import copy
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from tests import zokuvik_oracle as zo


def attn(kind="latent_attention", heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, q_rank=10, base=100.0, scale=None, window=None, ff=40):
  m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "rot": {"base": base, "dims": rot_dim},
       "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
  if kind == "latent_attention":
    m["q_rank"] = q_rank
  else:
    m["mask"] = {"size": int(window if window is not None else 5)}
  return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads=2, dim=8, decay_rank=4, ff=0):
  return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank},
          "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers: List[dict], width=48, vocab=80, groups=3, eps=1e-5) -> dict:
  return {"architecture": "Zokuvik", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups}, "layers": copy.deepcopy(layers)}


def public_config(cfg: dict) -> dict:
  """the config as a model directory would hold it: the oracle's private 'decay_rank' is not a key of the family (the engine
  reads that size from the tensor's shape)"""
  c = copy.deepcopy(cfg)
  for layer in c["layers"]:
    layer["mixer"].pop("decay_rank", None)
  return c


def bf16_bits(t: torch.Tensor) -> np.ndarray:
  a = t.detach().to(torch.float32).contiguous().numpy().view(np.uint32)
  assert not (a & 0xFFFF).any(), "weights must be bf16-representable"
  return (a >> 16).astype(np.uint16)


def make_engine(cfg: dict, weights: Dict[str, torch.Tensor], dtype: str, max_tokens=512, max_requests=4, page_size=8, start=0, end=None):
  from xotorch_b200.models import make_native
  n = make_native(public_config(cfg), 0, dtype)
  shapes = {k: tuple(v.shape) for k, v in weights.items()}
  n.set_shard(start, len(cfg["layers"]) - 1 if end is None else end, shapes)
  for name, t in weights.items():
    n.load_tensor(name, bf16_bits(t))
  n.check_loaded()
  n.begin_pool(max_tokens, max_requests, page_size)
  return n


def oracle_logits(cfg, weights, tokens, dtype=torch.float64):
  lg, trail = zo.forward(cfg, weights, tokens, dtype)
  return lg.double().numpy(), [t.double().numpy() for t in trail]


def row_err(got: np.ndarray, ref: np.ndarray) -> float:
  """largest per-row error: rms of the difference (its mean taken off) over the rms of the reference row (its mean taken off)"""
  d = got.astype(np.float64) - ref
  d = d - d.mean(axis=-1, keepdims=True)
  r = ref - ref.mean(axis=-1, keepdims=True)
  return float((np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean(-1) + 1e-30)).max())


TOL = {"float32": 2e-4, "bfloat16": 0.08}


def run_cut(native, slot: int, tokens: Sequence[int], cuts: Sequence[int]) -> np.ndarray:
  """feed `tokens` to one slot in portions of the given sizes (the last size repeats); logits of every row"""
  toks = np.asarray(tokens, dtype=np.int32)
  out, at, i = [], 0, 0
  while at < toks.size:
    n = min(int(cuts[min(i, len(cuts) - 1)]), toks.size - at)
    lg, _ = native.step([slot], [toks[at:at + n]], want=list(range(n)))
    out.append(lg)
    at += n
    i += 1
  return np.concatenate(out, axis=0)


def rand_tokens(vocab: int, n: int, seed: int) -> np.ndarray:
  return np.random.default_rng(seed).integers(0, vocab, size=n).astype(np.int32)
