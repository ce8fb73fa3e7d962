"""Plain, slow restatement of the Zokuvik design in torch (fp32 or fp64, CPU): one function per mechanism, whole sequences at
once, no cache, no batching.  The product path (libxotb200's layered-model kernels) shares no code with this file; the tests
compare the two on small random models.

Notation: T tokens, D width, H heads, dn / dr unrotated / rotated query-key sizes, dv value size, R latent rank."""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

Tensor = torch.Tensor


def rms(x: Tensor, eps: float) -> Tensor:
  return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_norm(x: Tensor, w: Tensor, eps: float) -> Tensor:
  return rms(x, eps) * w


def grouped_norm(x: Tensor, w: Tensor, groups: int, eps: float) -> Tensor:
  """every one of `groups` consecutive equal parts of the vector is scaled by its own root mean square"""
  T, D = x.shape
  return (rms(x.reshape(T, groups, D // groups), eps).reshape(T, D)) * w


def rotate(x: Tensor, pos: Tensor, base: float, dims: int, layout: str) -> Tensor:
  """x [T, ..., d]: the first `dims` entries of the last axis are turned by pos * base^(-2i/dims); pairs are (2i, 2i+1)
  ('interleaved') or (i, i + dims/2) ('half')."""
  half = dims // 2
  i = torch.arange(half, dtype=torch.float64)
  f = (float(base) ** (-2.0 * i / dims)).to(torch.float32 if x.dtype != torch.float64 else torch.float64)
  ang = pos.to(f.dtype)[:, None] * f[None, :]                    # [T, half]
  shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
  c, s = torch.cos(ang).reshape(shape).to(x.dtype), torch.sin(ang).reshape(shape).to(x.dtype)
  out = x.clone()
  if layout == "interleaved":
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
  elif layout == "half":
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
  else:
    raise ValueError(layout)
  return out


def visible(T: int, window: Optional[int]) -> Tensor:
  """[T, T] bool: query i sees key j iff j <= i and (no window or i - j < window)"""
  i = torch.arange(T)[:, None]
  j = torch.arange(T)[None, :]
  m = j <= i
  if window is not None:
    m = m & (i - j < window)
  return m


def latent_attention(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float, *, q_latent: bool, layout: str, gated: bool) -> Tensor:
  """Attention whose keys and values are expanded from one normed latent per token plus one rotated key part shared by all
  heads.  W holds the mixer's tensors by their short names ('dq', 'dq.norm', 'uq' | 'q', 'dkv', 'dkv.norm', 'uk', 'uv', 'g', 'o')."""
  T = h.shape[0]
  H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
  pos = torch.arange(T)
  if q_latent:
    q = plain_norm(h @ W["dq"].T, W["dq.norm"], eps) @ W["uq"].T
  else:
    q = h @ W["q"].T
  q = q.reshape(T, H, dn + dr)
  qn, qr = q[..., :dn], q[..., dn:]
  ckv = h @ W["dkv"].T
  c = plain_norm(ckv[:, :R], W["dkv.norm"], eps)
  kr = ckv[:, R:]                                                # [T, dr], not normed, one per token
  base, dims = m["rot"]["base"], m["rot"]["dims"]
  qr = rotate(qr, pos, base, dims, layout)
  kr = rotate(kr, pos, base, dims, layout)
  kn = (c @ W["uk"].T).reshape(T, H, dn)
  v = (c @ W["uv"].T).reshape(T, H, dv)
  s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
  window = m["mask"]["size"] if m.get("mask") else None
  s = s.masked_fill(~visible(T, window)[None], float("-inf"))
  p = torch.softmax(s, dim=-1)
  o = torch.einsum("hij,jhd->ihd", p, v)                         # [T, H, dv]
  if gated:
    o = o * torch.sigmoid(h @ W["g"].T)[:, :, None]
  return o.reshape(T, H * dv) @ W["o"].T


def general_delta(h: Tensor, W: Dict[str, Tensor], m: dict, eps: float, state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
  """Generalised delta rule, token by token.  state [H, d(key), d(value)]; returns (mixer output [T, D], final state)."""
  T = h.shape[0]
  H, d = m["heads"], m["dim"]
  r = (h @ W["r"].T).reshape(T, H, d)
  k = (h @ W["k"].T).reshape(T, H, d)
  v = (h @ W["v"].T).reshape(T, H, d)
  w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W["w1"].T) @ W["w2"].T + W["w0"])).reshape(T, H, d)
  a = torch.sigmoid(h @ W["a"].T + W["a.b"]).reshape(T, H, d)
  u = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
  S = torch.zeros(H, d, d, dtype=h.dtype) if state is None else state.clone()
  out = torch.empty(T, H, d, dtype=h.dtype)
  for t in range(T):
    uS = torch.einsum("hk,hkv->hv", u[t], S)                     # reads the old state
    S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
    out[t] = torch.einsum("hkv,hk->hv", S, r[t])
  o = rms(out, eps).reshape(T, H * d) * W["norm"]
  o = o * torch.sigmoid(h @ W["g"].T)
  return o @ W["o"].T, S


def relu2_mlp(h: Tensor, W: Dict[str, Tensor]) -> Tensor:
  return (torch.relu(h @ W["up"].T) ** 2) @ W["down"].T


def sub(weights: Dict[str, Tensor], prefix: str) -> Dict[str, Tensor]:
  return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(kind: str, h: Tensor, W: Dict[str, Tensor], m: dict, eps: float) -> Tensor:
  if kind == "latent_attention":
    return latent_attention(h, W, m, eps, q_latent=True, layout="interleaved", gated=True)
  if kind == "latent_attention_2":
    return latent_attention(h, W, m, eps, q_latent=False, layout="half", gated=False)
  if kind == "general_delta":
    return general_delta(h, W, m, eps)[0]
  raise ValueError(kind)


def forward(cfg: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float32) -> Tuple[Tensor, List[Tensor]]:
  """logits [T, vocab] of one whole sequence and the residual stream after every layer"""
  Wt = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
  eps, G = cfg["norm"]["eps"], cfg["norm"]["groups"]
  x = Wt["embed"][torch.as_tensor(tokens, dtype=torch.long)]
  trail = []
  for i, layer in enumerate(cfg["layers"]):
    p = f"l{i}."
    y = mixer(layer["type"], grouped_norm(x, Wt[p + "norm1"], G, eps), sub(Wt, p + "mix."), layer["mixer"], eps)
    x = x + grouped_norm(y, Wt[p + "norm1b"], G, eps)
    if layer.get("mlp") is not None:
      y = relu2_mlp(grouped_norm(x, Wt[p + "norm2"], G, eps), sub(Wt, p + "mlp."))
      x = x + grouped_norm(y, Wt[p + "norm2b"], G, eps)
    trail.append(x)
  x = grouped_norm(x, Wt["final.norm"], G, eps)
  return x @ Wt["head"].T, trail


# ---- small random models -------------------------------------------------------------------------------------------------
def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
  D, V = cfg["width"], cfg["vocab"]
  out: Dict[str, Tuple[int, ...]] = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
  for i, layer in enumerate(cfg["layers"]):
    p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
    out[p + "norm1"] = out[p + "norm1b"] = (D,)
    if kind in ("latent_attention", "latent_attention_2"):
      H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
      if kind == "latent_attention":
        out[p + "mix.dq"] = (m["q_rank"], D)
        out[p + "mix.dq.norm"] = (m["q_rank"],)
        out[p + "mix.uq"] = (H * (dn + dr), m["q_rank"])
        out[p + "mix.g"] = (H, D)
      else:
        out[p + "mix.q"] = (H * (dn + dr), D)
      out[p + "mix.dkv"] = (R + dr, D)
      out[p + "mix.dkv.norm"] = (R,)
      out[p + "mix.uk"] = (H * dn, R)
      out[p + "mix.uv"] = (H * dv, R)
      out[p + "mix.o"] = (D, H * dv)
    else:
      H, d = m["heads"], m["dim"]
      for n in ("r", "k", "v", "g", "a"):
        out[p + "mix." + n] = (H * d, D)
      out[p + "mix.a.b"] = out[p + "mix.w0"] = out[p + "mix.norm"] = (H * d,)
      out[p + "mix.w1"] = (m.get("decay_rank", 8), D)
      out[p + "mix.w2"] = (H * d, m.get("decay_rank", 8))
      out[p + "mix.o"] = (D, H * d)
    if layer.get("mlp") is not None:
      out[p + "norm2"] = out[p + "norm2b"] = (D,)
      out[p + "mlp.up"] = (layer["mlp"]["ff"], D)
      out[p + "mlp.down"] = (D, layer["mlp"]["ff"])
  return out


def random_weights(cfg: dict, seed: int, gain: float = 1.0) -> Dict[str, Tensor]:
  """bf16-representable random weights (so a 16-bit engine and this oracle start from identical numbers)"""
  g = torch.Generator().manual_seed(seed)
  out = {}
  for name, shape in tensor_shapes(cfg).items():
    if len(shape) == 1:
      t = 1.0 + 0.2 * torch.randn(shape, generator=g) if "norm" in name else 0.5 * torch.randn(shape, generator=g)
    elif name == "embed":
      t = torch.randn(shape, generator=g)
    else:
      t = gain * torch.randn(shape, generator=g) / math.sqrt(shape[1])
    out[name] = t.to(torch.bfloat16).to(torch.float32)
  return out
