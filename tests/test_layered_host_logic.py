"""Host side of the layered engine without a GPU: config -> layer table, the model registry, the request table, the trace
replayer and the batch scheduler, driven over a stand-in for the native object (it keeps per-slot token lists and answers with a
function of everything a slot has seen, so a lost, mixed-up or stale slot changes the answer)."""
import io
import json

import numpy as np
import pytest

from tests.layered_util import attn, config, delta, public_config
from xotorch_b200 import _lib
from xotorch_b200.layered import RequestSlots, zokuvik_globals, zokuvik_layers
from xotorch_b200.models import is_layered, model_summary


class FakeLayered:
  """LayeredShard's request-state surface on the host: the 'logits' of a row are one-hot at (sum of the slot's tokens so far
  + 7 * its length) % vocab"""
  is_first = is_last = True

  def __init__(self, vocab=50):
    self.vocab, self.n_slots, self.page, self.pages_total = vocab, 0, 8, 0
    self.seen, self.steps = {}, []

  def begin_pool(self, max_tokens, max_requests, page_size=8):
    self.n_slots, self.page = max_requests, page_size or 64
    self.pages_total = -(-max_tokens // self.page) + max_requests
    self.seen = {i: [] for i in range(max_requests)}

  def clear_request(self, slot): self.seen[slot] = []
  def request_len(self, slot): return len(self.seen[slot])

  def cache_stats(self):
    used = sum(-(-len(v) // self.page) for v in self.seen.values())
    return {"pages_total": self.pages_total, "pages_free": self.pages_total - used, "page_size": self.page}

  def step(self, slots, rows, want=None, logits=True, argmax=True):
    assert len(set(slots)) == len(slots)
    self.steps.append([len(r) for r in rows])
    per_row = []
    for s, r in zip(slots, rows):
      for t in np.asarray(r).reshape(-1):
        self.seen[s].append(int(t))
        per_row.append((sum(self.seen[s]) + 7 * len(self.seen[s])) % self.vocab)
    assert self.cache_stats()["pages_free"] >= 0, "the scheduler overcommitted the page pool"
    if want is None:
      want = np.cumsum([len(r) for r in rows]) - 1
    ids = np.array([per_row[w] for w in want], dtype=np.int32)
    lg = np.zeros((len(ids), self.vocab), dtype=np.float32)
    lg[np.arange(len(ids)), ids] = 1.0
    return (lg if logits else None), (ids if argmax else None)

  def close(self): pass


def fake_generate(prompt, n, vocab=50):
  seq, out = [int(t) for t in prompt], []
  for _ in range(n):
    out.append((sum(seq) + 7 * len(seq)) % vocab)
    seq.append(out[-1])
  return out


def test_config_to_layer_table():
  cfg = public_config(config([attn("latent_attention", q_rank=10, base=777.0), attn("latent_attention_2", window=9, ff=0), delta(heads=2, dim=8)]))
  specs = zokuvik_layers(cfg, {"l2.mix.w1": (5, 48)})
  a, b, d = specs
  assert (a.mixer, a.q_rank, a.rot_layout, a.out_gate, a.window, a.ff) == (_lib.LM_MIX_LATENT_ATTN, 10, _lib.LM_ROT_INTERLEAVED, 1, 0, 40)
  assert a.rot_base == 777.0 and abs(a.scale - cfg["layers"][0]["mixer"]["scale"]) < 1e-12
  assert (b.q_rank, b.rot_layout, b.out_gate, b.window, b.ff) == (0, _lib.LM_ROT_HALF, 0, 9, 0)
  assert (d.mixer, d.heads, d.dim, d.vdim, d.low_rank, d.ff) == (_lib.LM_MIX_DELTA_RULE, 2, 8, 8, 5, 0)
  assert zokuvik_globals(cfg) == {"width": 48, "vocab": 80, "norm_groups": 3, "norm_eps": 1e-5}
  with pytest.raises(ValueError, match="w1"):
    zokuvik_layers(cfg, {})
  cfg["layers"][0]["type"] = "something_else"
  with pytest.raises(ValueError, match="something_else"):
    zokuvik_layers(cfg, {"l2.mix.w1": (5, 48)})


def test_registry_tells_the_engines_apart():
  z = public_config(config([delta()]))
  assert is_layered(z) and model_summary(z)["engine"] == "layered" and model_summary(z)["n_layers"] == 1
  hf = {"model_type": "llama", "num_hidden_layers": 4, "vocab_size": 100, "hidden_size": 64, "max_position_embeddings": 128}
  assert not is_layered(hf) and model_summary(hf) == {"n_layers": 4, "vocab": 100, "width": 64, "max_positions": 128, "engine": "shard"}
  with pytest.raises(ValueError):
    model_summary({"architecture": "Unknown"})


def test_request_table_reuses_slots_and_clears_them():
  n = FakeLayered()
  n.begin_pool(64, 2)
  t = RequestSlots(n)
  assert t.acquire("a") == 0 and t.acquire("b") == 1 and t.acquire("a") == 0
  with pytest.raises(RuntimeError):
    t.acquire("c")
  n.step([0], [[1, 2, 3]])
  t.release("a")
  assert n.request_len(0) == 0 and t.acquire("c") == 0 and "a" not in t and len(t) == 2


def test_trace_replay_over_the_request_table(tmp_path, monkeypatch):
  from xotorch_b200 import trace_replay as tr
  fake = FakeLayered(vocab=11)
  fake.load_dir = lambda d: None
  monkeypatch.setattr(tr, "load_model_config", lambda d: public_config(config([delta()], vocab=11)))
  monkeypatch.setattr(tr, "make_native", lambda cfg, dev, dtype: fake)
  steps = [
    {"step": 0, "entries": [{"id": "x", "tokens": [1, 2, 3], "want": [0, 2]}, {"id": "y", "tokens": [4], "want": []}], "end": []},
    {"step": 1, "entries": [{"id": "x", "tokens": [5], "want": []}, {"id": "y", "tokens": [6], "want": []}], "end": ["x"]},
    {"step": 2, "entries": [{"id": "y", "tokens": [7], "want": [0]}, {"id": "z", "tokens": [8, 9], "want": [1]}], "end": ["y", "z"]},
  ]
  monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
  out = io.StringIO()
  monkeypatch.setattr("sys.stdout", out)
  assert tr.main(["--model", "m", "--out", str(tmp_path), "--max-tokens", "32"]) == 0
  assert out.getvalue().split() == ["done", "0", "done", "1", "done", "2"]
  a = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, 11)
  assert a.argmax(1).tolist() == [(1 + 7) % 11, (6 + 21) % 11]
  assert not (tmp_path / "1.f32").exists()
  c = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(2, 11)
  # y continues its own history; z reuses x's slot, which must have been emptied
  assert c.argmax(1).tolist() == [(4 + 6 + 7 + 21) % 11, (8 + 9 + 14) % 11]


@pytest.mark.parametrize("budget,max_requests", [(1000, 4), (5, 2), (1, 1)])
def test_batch_scheduler_admission_budget_and_streams(budget, max_requests):
  from xotorch_b200.scheduler import ContinuousBatch
  n = FakeLayered()
  events = []
  s = ContinuousBatch(n, max_requests=max_requests, max_tokens=96, page_size=8, token_budget=budget,
                      on_token=lambda rid, toks, fin: events.append((rid, toks[0], fin)))
  rng = np.random.default_rng(0)
  reqs = [(f"q{i}", rng.integers(0, 50, size=L), g) for i, (L, g) in enumerate([(9, 5), (1, 7), (30, 2), (4, 1), (12, 9)])]
  for rid, p, g in reqs:
    s.submit(rid, p, g)
  out = s.run_until_idle()
  for rid, p, g in reqs:
    assert out[rid] == fake_generate(p, g), rid
    assert [e[1] for e in events if e[0] == rid] == out[rid] and [e[2] for e in events if e[0] == rid][-1] is True
  assert all(sum(st) <= budget for st in n.steps)
  assert n.cache_stats()["pages_free"] == n.pages_total and s.reserved_pages == 0
  with pytest.raises(ValueError):
    s.submit("big", np.zeros(90, dtype=np.int32), 10)


def test_batch_scheduler_stops_at_eos():
  from xotorch_b200.scheduler import ContinuousBatch
  n = FakeLayered()
  s = ContinuousBatch(n, max_requests=2, max_tokens=64, page_size=8)
  p = np.array([3, 4], dtype=np.int32)
  full = fake_generate(p, 10)
  s.submit("e", p, 10, eos_token_id=full[3])
  assert s.run_until_idle()["e"] == full[:full.index(full[3]) + 1]
