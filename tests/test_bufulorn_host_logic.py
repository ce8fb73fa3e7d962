"""Bufulorn without a GPU: config.json -> layer table of the layered engine, the registry, and self-checks of the plain oracle
(recurrences carried over portions, routing rules, mask edges) that the GPU tests lean on."""
import math

import numpy as np
import pytest
import torch

from tests import bufulorn_oracle as bo
from tests.bufulorn_util import attention, config, delta, dense, moe
from xotorch_b200 import _lib
from xotorch_b200.layered import LAYERED_FAMILIES, bufulorn_globals, bufulorn_layers
from xotorch_b200.models import is_layered, model_summary


def test_config_to_layer_table():
  cfg = config([attention(heads=6, kv_heads=2, dim=8, vdim=12, chunk=16, softcap=30.0, mlp=moe(8, 2, (4, 3), 12)),
                attention(heads=6, kv_heads=2, dim=8, vdim=12, chunk=None, softcap=None, kv_from=0, mlp=dense(40)),
                delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, mlp=None)], width=48, vocab=80, max_positions=99)
  a, b, d = bufulorn_layers(cfg, {})
  assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.chunk, a.kv_from, a.out_gate) == (_lib.LM_MIX_ATTENTION, 6, 2, 8, 12, 16, -1, 2)
  assert (a.qk_norm, a.proj_bias, a.dist_bias, a.window) == (1, 1, 1, 0) and a.softcap == 30.0
  assert (a.ff_kind, a.experts, a.top, a.groups, a.groups_keep, a.expert_ff, a.ff) == (_lib.LM_FF_MOE, 8, 2, 4, 3, 12, 0)
  assert (b.kv_from, b.chunk, b.softcap, b.ff_kind, b.ff) == (0, 0, 0.0, _lib.LM_FF_XIELU, 40)
  assert (d.mixer, d.heads, d.kv_heads, d.dim, d.vdim, d.conv_taps, d.ff) == (_lib.LM_MIX_GATED_DELTA, 4, 2, 8, 6, 3, 0)
  assert bufulorn_globals(cfg) == {"width": 48, "vocab": 80, "norm_groups": 1, "norm_eps": 1e-5, "block": _lib.LM_BLOCK_POST_LN, "max_positions": 99}
  assert is_layered(cfg) and model_summary(cfg) == {"n_layers": 3, "vocab": 80, "width": 48, "max_positions": 99, "engine": "layered"}
  assert "Bufulorn" in LAYERED_FAMILIES
  cfg["layers"][2]["type"] = "something_else"
  with pytest.raises(ValueError, match="something_else"):
    bufulorn_layers(cfg, {})
  cfg["layers"][2]["type"] = "delta"
  cfg["layers"][1]["mlp"]["kind"] = "sparse"
  with pytest.raises(ValueError, match="sparse"):
    bufulorn_layers(cfg, {})


def test_c_structs_mirror_the_header():
  """every field of the two structs in include/xotb200_lm.h, in order"""
  import re
  from pathlib import Path
  src = (Path(__file__).resolve().parent.parent / "include" / "xotb200_lm.h").read_text()
  for name, cls in (("xotb200_lm_layer", _lib.LmLayer), ("xotb200_lm_cfg", _lib.LmCfg)):
    body = re.search(r"typedef struct " + name + r" \{(.*?)\} " + name + ";", src, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"\b(?:int32_t|float)\s+(\w+)\s*;", body)
    assert fields == [f for f, _ in cls._fields_]


# ---- the oracle against itself -------------------------------------------------------------------------------------------------
def test_oracle_delta_rule_carries_its_state_over_portions():
  cfg = config([delta(heads=4, kv_heads=2, dim=8, vdim=6, conv=4)])
  W = {k: v.double() for k, v in bo.random_weights(cfg, 1).items()}
  m, Wm = cfg["layers"][0]["mixer"], bo.sub(W, "l0.mix.")
  h = torch.randn(23, 48, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
  whole, _ = bo.gated_delta(h, Wm, m, 1e-5)
  parts, st = [], None
  for lo, hi in ((0, 1), (1, 3), (3, 4), (4, 15), (15, 23)):
    y, st = bo.gated_delta(h[lo:hi], Wm, m, 1e-5, st)
    parts.append(y)
  assert torch.allclose(torch.cat(parts), whole, atol=1e-12)


def test_oracle_short_conv_weighs_the_current_token_last():
  x = torch.arange(1.0, 6.0).reshape(5, 1)
  y, tail = bo.short_conv(x, torch.tensor([[100.0, 10.0, 1.0]]))
  assert y.reshape(-1).tolist() == [1.0, 12.0, 123.0, 234.0, 345.0] and tail.reshape(-1).tolist() == [4.0, 5.0]


def test_oracle_block_mask_edges():
  v = bo.chunk_visible(10, 4)
  assert v[3, 0] and v[3, 3] and not v[4, 3] and v[4, 4] and v[7, 4] and not v[8, 7] and not v[2, 3]
  assert bo.chunk_visible(5, None)[4, 0]


def test_oracle_routing_rules():
  r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}
  # logits chosen so that the scores order as e5 > e4 > e0 > e2 > ...: groups (0,1) (2,3) (4,5) score e0, e2, e5 -> group 1 is dropped
  z = torch.tensor([[2.0, -1.0, 1.5, 1.4, 2.5, 3.0]])
  idx, wt = bo.route(torch.ones(1, 6), torch.zeros(6, 6), r)                 # uniform scores: any valid choice, weights 1/6
  assert torch.allclose(wt, torch.full((1, 2), 1 / 6))
  h = torch.ones(1, 1)
  idx, wt = bo.route(h, z.T.contiguous(), r)
  s = torch.softmax(z, -1)
  assert sorted(idx[0].tolist()) == [4, 5] and torch.allclose(wt.sum(), s[0, 4] + s[0, 5])
  r = {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}}
  idx, wt = bo.route(h, z.T.contiguous(), r)
  assert sorted(idx[0].tolist()) == [0, 4, 5], "e2 and e3 belong to the dropped group although they beat e1"
  assert float(wt.sum()) < 1.0, "weights are the raw scores, not renormalised"


def test_oracle_activation_is_continuous_and_matches_its_formula():
  p, q = torch.tensor(0.3), torch.tensor(-0.2)
  z = torch.tensor([-2.0, -1e-6, 0.0, 1e-6, 1.5])
  y = bo.xielu(z, p, q)
  sp = lambda t: math.log1p(math.exp(float(t)))
  assert abs(float(y[4]) - (sp(p) * 2.25 + 0.75)) < 1e-6
  assert abs(float(y[0]) - ((0.5 + sp(q)) * (math.exp(-2.0) - 1 + 2.0) - 1.0)) < 1e-6
  assert abs(float(y[1])) < 1e-5 and float(y[2]) == 0.0 and abs(float(y[3])) < 1e-5


def test_batch_scheduler_refuses_requests_beyond_the_position_table():
  from tests.test_layered_host_logic import FakeLayered, fake_generate
  from xotorch_b200.scheduler import ContinuousBatch
  n = FakeLayered()
  n.max_positions = 20
  s = ContinuousBatch(n, max_requests=2, max_tokens=64, page_size=8)
  with pytest.raises(ValueError, match="positions"):
    s.submit("long", list(range(1, 16)), 7)           # 15 + 7 - 1 = 21 tokens would be held
  s.submit("fits", list(range(1, 16)), 6)             # 20 tokens held: the last generated token is never fed back
  assert s.run_until_idle()["fits"] == fake_generate(list(range(1, 16)), 6)
