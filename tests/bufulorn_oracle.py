"""Plain, slow restatement of the Bufulorn design in torch (fp32 or fp64, CPU): one function per mechanism, whole sequences at
once, token-by-token recurrences, no cache, no batching.  The product path (the layered-model kernels of libxotb200_lm) shares
no code with this file; the tests compare the two on small random models.

Notation: T tokens, D width, H query (or value) heads, G key/value heads, dk query/key size, dv value size per head."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# ---- norms and activations -------------------------------------------------------------------------------------------------
def rms_unit(x: Tensor, eps: float) -> Tensor:
  return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: Tensor, w: Tensor, b: Tensor, eps: float) -> Tensor:
  mu = x.mean(dim=-1, keepdim=True)
  var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
  return (x - mu) / torch.sqrt(var + eps) * w + b


def xielu(z: Tensor, p: Tensor, q: Tensor) -> Tensor:
  """two-sided activation with learned curvatures: a parabola on the right, a saturating exponential on the left"""
  right = F.softplus(p) * z * z + 0.5 * z
  left = (0.5 + F.softplus(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z
  return torch.where(z > 0, right, left)


# ---- attention -------------------------------------------------------------------------------------------------------------
def chunk_visible(T: int, size: Optional[int]) -> Tensor:
  """[T, T] bool: query i sees key j iff j <= i and both lie in the same block of `size` positions (counted from 0)"""
  i = torch.arange(T)[:, None]
  j = torch.arange(T)[None, :]
  m = j <= i
  if size:
    m = m & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
  return m


def attention_keys_values(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float) -> Tuple[Tensor, Tensor]:
  """what an attention layer's cache holds: keys after their per-head norm [T, G, dk] and values [T, G, dv]"""
  T = h.shape[0]
  G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
  k = (h @ W["k"].T + W["k.b"]).reshape(T, G, dk)
  v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
  return rms_unit(k, eps) * W["k.norm"], v


def attention(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float, kv: Optional[Tuple[Tensor, Tensor]] = None) -> Tensor:
  """Grouped-query attention without rotation: normed queries and keys, soft-capped scores, a logarithmic distance penalty per
  head, block-local causal mask, softmax, element-wise sigmoid gate on the concatenated heads.  `kv`: keys/values of another
  layer (this layer then has no key/value tensors)."""
  T = h.shape[0]
  H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  q = rms_unit((h @ W["q"].T + W["q.b"]).reshape(T, H, dk), eps) * W["q.norm"]
  k, v = kv if kv is not None else attention_keys_values(h, W, m, eps)
  rep = H // G
  k = k.repeat_interleave(rep, dim=1)                            # query head a reads key/value head a // rep
  v = v.repeat_interleave(rep, dim=1)
  s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
  cap = m.get("softcap")
  if cap:
    s = cap * torch.tanh(s / cap)
  dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(s.dtype)      # i - j where visible
  s = s - W["r1"][:, None, None] * torch.log1p(W["r2"][:, None, None] * dist[None])
  size = m["mask"]["size"] if m.get("mask") else None
  s = s.masked_fill(~chunk_visible(T, size)[None], float("-inf"))
  p = torch.softmax(s, dim=-1)
  o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
  o = o * torch.sigmoid(h @ W["g"].T)
  return o @ W["o"].T


# ---- gated delta rule ------------------------------------------------------------------------------------------------------
def short_conv(x: Tensor, w: Tensor, before: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
  """causal per-channel filter over time.  x [T, C], w [C, taps] (last column weighs the current token), `before` [taps-1, C] the
  inputs that came earlier (zeros at the start).  Returns (filtered [T, C], the last taps-1 inputs)."""
  T, C = x.shape
  taps = w.shape[1]
  past = torch.zeros(taps - 1, C, dtype=x.dtype) if before is None else before
  ext = torch.cat([past, x], dim=0)                              # ext[t + taps - 1] = x[t]
  y = torch.zeros_like(x)
  for i in range(taps):
    y = y + ext[i:i + T] * w[:, i]
  return y, ext[T:]


def unit_vector(x: Tensor) -> Tensor:
  return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float, state=None):
  """Delta rule with one scalar decay per head, token by token.  state = (S [H, dk, dv], conv inputs of q, k, v) or None.
  Returns (mixer output [T, D], new state)."""
  T = h.shape[0]
  H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
  S, cq, ck, cv = state if state is not None else (torch.zeros(H, dk, dv, dtype=h.dtype), None, None, None)
  q, cq = short_conv(h @ W["q"].T, W["q.conv"], cq)
  k, ck = short_conv(h @ W["k"].T, W["k.conv"], ck)
  v, cv = short_conv(h @ W["v"].T, W["v.conv"], cv)
  q, k, v = F.silu(q), F.silu(k), F.silu(v)
  q = unit_vector(q.reshape(T, G, dk)) * dk ** -0.5
  k = unit_vector(k.reshape(T, G, dk))
  rep = H // G
  q = q.repeat_interleave(rep, dim=1)
  k = k.repeat_interleave(rep, dim=1)
  v = v.reshape(T, H, dv)
  beta = torch.sigmoid(h @ W["b"].T)                             # [T, H]
  decay = torch.exp(-torch.exp(W["A_log"]) * F.softplus(h @ W["a"].T + W["dt_bias"]))
  out = torch.empty(T, H, dv, dtype=h.dtype)
  S = S.clone()
  for t in range(T):
    S = decay[t][:, None, None] * S
    u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
    S = S + k[t][:, :, None] * u[:, None, :]
    out[t] = torch.einsum("hkv,hk->hv", S, q[t])
  o = (rms_unit(out, eps) * W["norm"]).reshape(T, H * dv) * F.silu(h @ W["g"].T)
  return o @ W["o"].T, (S, cq, ck, cv)


# ---- feed-forward ----------------------------------------------------------------------------------------------------------
def dense_ff(h: Tensor, W: Dict[str, Tensor]) -> Tensor:
  return xielu(h @ W["up"].T, W["act"][0], W["act"][1]) @ W["down"].T


def route(h: Tensor, w_router: Tensor, r: dict) -> Tuple[Tensor, Tensor]:
  """chosen experts [T, top] and their weights: softmax over all experts, only experts of the `keep` best groups (a group's
  score is its best expert's) may be chosen, weights are the raw scores"""
  E, top = r["experts"], r["top"]
  s = torch.softmax(h @ w_router.T, dim=-1)
  allowed = torch.ones_like(s, dtype=torch.bool)
  gr = r.get("groups")
  if gr and gr["count"] > 1:
    n, keep = gr["count"], gr["keep"]
    best = s.reshape(-1, n, E // n).max(dim=-1).values            # [T, n]
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    allowed = kept.repeat_interleave(E // n, dim=1)
  idx = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
  return idx, s.gather(1, idx)


def moe_ff(h: Tensor, W: Dict[str, Tensor], mlp: dict) -> Tensor:
  idx, wt = route(h, W["router"], mlp["router"])
  out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
  for e in range(mlp["router"]["experts"]):                      # expert by expert: the rows that chose it, with their weight for it
    rows, slot = (idx == e).nonzero(as_tuple=True)
    if rows.numel():
      x = h[rows]
      a = F.silu(x @ W[f"e{e}.gate"].T) * (x @ W[f"e{e}.up"].T)
      out[rows] += wt[rows, slot].to(h.dtype)[:, None] * (a @ W[f"e{e}.down"].T)
  return out


# ---- the model -------------------------------------------------------------------------------------------------------------
def sub(weights: Dict[str, Tensor], prefix: str) -> Dict[str, Tensor]:
  return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float32) -> Tuple[Tensor, List[Tensor]]:
  """logits [T, vocab] of one whole sequence and the residual stream after every layer"""
  Wt = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
  eps = cfg["norm"]["eps"]
  tok = torch.as_tensor(tokens, dtype=torch.long)
  x = Wt["embed"][tok] + Wt["pos"][: tok.numel()]
  trail, kvs = [], {}
  for i, layer in enumerate(cfg["layers"]):
    p, m = f"l{i}.", layer["mixer"]
    W = sub(Wt, p + "mix.")
    if layer["type"] == "attention":
      src = m.get("kv_from")
      if src is None:
        kvs[i] = attention_keys_values(x, W, m, eps)
      y = attention(x, W, m, eps, kvs[i if src is None else src])
    elif layer["type"] == "delta":
      y = gated_delta(x, W, m, eps)[0]
    else:
      raise ValueError(layer["type"])
    x = x + layer_norm(y, Wt[p + "norm1"], Wt[p + "norm1.b"], eps)
    mlp = layer.get("mlp")
    if mlp is not None:
      y = dense_ff(x, sub(Wt, p + "mlp.")) if mlp["kind"] == "dense" else moe_ff(x, sub(Wt, p + "mlp."), mlp)
      x = x + layer_norm(y, Wt[p + "norm2"], Wt[p + "norm2.b"], eps)
    trail.append(x)
  x = layer_norm(x, Wt["final.norm"], Wt["final.norm.b"], eps)
  return x @ Wt["head"].T, trail


# ---- small random models ---------------------------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
  D, V = cfg["width"], cfg["vocab"]
  out: Dict[str, Tuple[int, ...]] = {"embed": (V, D), "pos": (cfg["max_positions"], D), "final.norm": (D,), "final.norm.b": (D,), "head": (V, D)}
  for i, layer in enumerate(cfg["layers"]):
    p, m = f"l{i}.", layer["mixer"]
    out[p + "norm1"] = out[p + "norm1.b"] = (D,)
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    if layer["type"] == "attention":
      out[p + "mix.q"], out[p + "mix.q.b"], out[p + "mix.q.norm"] = (H * dk, D), (H * dk,), (dk,)
      if m.get("kv_from") is None:
        out[p + "mix.k"], out[p + "mix.k.b"], out[p + "mix.k.norm"] = (G * dk, D), (G * dk,), (dk,)
        out[p + "mix.v"], out[p + "mix.v.b"] = (G * dv, D), (G * dv,)
      out[p + "mix.r1"] = out[p + "mix.r2"] = (H,)
      out[p + "mix.g"], out[p + "mix.o"] = (H * dv, D), (D, H * dv)
    else:
      for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
        out[p + "mix." + n], out[p + "mix." + n + ".conv"] = (c, D), (c, m["conv"])
      out[p + "mix.b"] = out[p + "mix.a"] = (H, D)
      out[p + "mix.A_log"] = out[p + "mix.dt_bias"] = (H,)
      out[p + "mix.norm"] = (dv,)
      out[p + "mix.g"], out[p + "mix.o"] = (H * dv, D), (D, H * dv)
    mlp = layer.get("mlp")
    if mlp is not None:
      out[p + "norm2"] = out[p + "norm2.b"] = (D,)
      if mlp["kind"] == "dense":
        out[p + "mlp.up"], out[p + "mlp.down"], out[p + "mlp.act"] = (mlp["ff"], D), (D, mlp["ff"]), (2,)
      else:
        out[p + "mlp.router"] = (mlp["router"]["experts"], D)
        for e in range(mlp["router"]["experts"]):
          out[p + f"mlp.e{e}.gate"] = out[p + f"mlp.e{e}.up"] = (mlp["expert"]["ff"], D)
          out[p + f"mlp.e{e}.down"] = (D, mlp["expert"]["ff"])
  return out


def random_weights(cfg: dict, seed: int, gain: float = 1.0) -> Dict[str, Tensor]:
  """bf16-representable random weights (so a 16-bit engine and this oracle start from identical numbers)"""
  g = torch.Generator().manual_seed(seed)
  out = {}
  for name, shape in tensor_shapes(cfg).items():
    if name.endswith(".conv"):
      t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
    elif name.endswith("router"):
      t = 3.0 * torch.randn(shape, generator=g) / math.sqrt(shape[1])     # spread scores: no near-ties between experts
    elif len(shape) == 1:
      if name.endswith("r1"): t = 0.3 * torch.rand(shape, generator=g)
      elif name.endswith("r2"): t = 0.5 + torch.rand(shape, generator=g)
      elif name.endswith("A_log"): t = torch.log(0.5 + 2.0 * torch.rand(shape, generator=g))
      elif name.endswith("norm"): t = 1.0 + 0.2 * torch.randn(shape, generator=g)
      else: t = 0.3 * torch.randn(shape, generator=g)
    elif name == "embed":
      t = torch.randn(shape, generator=g)
    elif name == "pos":
      t = 0.5 * torch.randn(shape, generator=g)
    else:
      t = gain * torch.randn(shape, generator=g) / math.sqrt(shape[1])
    out[name] = t.to(torch.bfloat16).to(torch.float32)
  return out
