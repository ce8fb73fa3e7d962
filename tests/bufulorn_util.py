"""Helpers of the Bufulorn tests: small configurations of the family (layers of attention / gated delta rule with dense or
mixture-of-experts feed-forwards) and the oracle's logits.  Engines, schedules and the error measure come from layered_util."""
from __future__ import annotations

import copy
from typing import List, Optional

import torch

from tests import bufulorn_oracle as bo


def dense(ff=40):
  return {"kind": "dense", "ff": ff}


def moe(experts=8, top=2, groups=(4, 2), ff=12):
  r = {"experts": experts, "top": top}
  if groups:
    r["groups"] = {"count": groups[0], "keep": groups[1]}
  return {"kind": "moe", "router": r, "expert": {"ff": ff}}


def attention(heads=4, kv_heads=2, dim=8, vdim=12, scale=None, softcap: Optional[float] = 30.0, chunk: Optional[int] = 16, kv_from=None, mlp=None):
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
  if softcap:
    m["softcap"] = float(softcap)
  if chunk:
    m["mask"] = {"size": int(chunk)}
  if kv_from is not None:
    m["kv_from"] = int(kv_from)
  return {"type": "attention", "mixer": m, "mlp": mlp}


def delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=4, mlp=None):
  return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def config(layers: List[dict], width=48, vocab=80, max_positions=512, eps=1e-5) -> dict:
  return {"architecture": "Bufulorn", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps},
          "layers": copy.deepcopy(layers)}


def oracle_logits(cfg, weights, tokens, dtype=torch.float64):
  lg, trail = bo.forward(cfg, weights, tokens, dtype)
  return lg.double().numpy(), [t.double().numpy() for t in trail]
