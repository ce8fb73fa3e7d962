"""The layered engine (libxotb200_lm.so) against the plain oracle (tests/zokuvik_oracle.py) on small random models (-m gpu).
The float32 engine is held to the oracle in float64 tightly, the bfloat16 engine loosely; every test asks for the logits of
EVERY row unless it says otherwise, so a wrong key, position or state at any place shows."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from tests import zokuvik_oracle as zo
from tests.layered_util import (TOL, attn, config, delta, make_engine, oracle_logits, public_config, rand_tokens, row_err, run_cut)

DTYPES = ["float32", "bfloat16"]

MIXED = [attn("latent_attention"), attn("latent_attention_2", heads=2, dim=6, rot_dim=6, vdim=5, kv_rank=9, window=7, base=10.0),
         delta(heads=2, dim=8), attn("latent_attention", heads=5, dim=4, rot_dim=2, vdim=4, kv_rank=33, q_rank=7, ff=0),
         delta(heads=3, dim=12, decay_rank=3, ff=24)]


def check(native, cfg, W, tokens, cuts, dtype, slot=0, tol=None):
  ref, _ = oracle_logits(cfg, W, tokens)
  got = run_cut(native, slot, tokens, cuts)
  e = row_err(got, ref)
  assert e < (tol or TOL[dtype]), f"{dtype}: rows differ from the oracle, worst relative error {e:.3e}"
  return got


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
SINGLE = {
  "latent_q_latent_gate": [attn("latent_attention", ff=0)],
  "latent_window_half": [attn("latent_attention_2", window=4, ff=0)],
  "latent_window_1": [attn("latent_attention_2", window=1, ff=0)],
  "latent_odd_sizes": [attn("latent_attention", heads=7, dim=5, rot_dim=6, vdim=3, kv_rank=37, q_rank=11, ff=0)],
  "latent_wide_rank": [attn("latent_attention_2", heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=130, window=50, ff=0)],
  "latent_one_head": [attn("latent_attention", heads=1, dim=12, rot_dim=4, vdim=20, kv_rank=24, q_rank=6, ff=0)],
  "latent_rank_260": [attn("latent_attention", heads=3, dim=8, rot_dim=8, vdim=8, kv_rank=260, q_rank=16, ff=0)],
  "latent_many_heads": [attn("latent_attention_2", heads=40, dim=4, rot_dim=4, vdim=4, kv_rank=16, window=11, ff=0)],
  "delta": [delta()],
  "delta_one_head_wide": [delta(heads=1, dim=40, decay_rank=1)],
  "delta_dim_20": [delta(heads=3, dim=20, decay_rank=5)],
  "feed_forward": [attn("latent_attention_2", window=3, ff=50)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_layer_models(name, dtype):
  groups = 1 if "odd" in name else 3
  cfg = config(SINGLE[name], width=36 if "odd" in name else 48, groups=groups)
  W = zo.random_weights(cfg, 11)
  n = make_engine(cfg, W, dtype)
  toks = rand_tokens(cfg["vocab"], 41, 3)
  n.set_trace(True)
  ref, trail = oracle_logits(cfg, W, toks)
  got, _ = n.step([0], [toks], want=list(range(len(toks))))
  x = n.read_trace(len(toks))[0]
  scale = np.abs(trail[0]).max()
  assert np.abs(x - trail[0]).max() / scale < (1e-5 if dtype == "float32" else 0.03), "residual stream after the layer differs"
  assert row_err(got, ref) < TOL[dtype]
  cut = run_cut(n, 1, toks, [7, 5, 1])               # short portions and single rows: the few-rows kernels of the same mechanism
  assert row_err(cut, ref) < TOL[dtype]
  n.close()


def test_rotation_of_a_leading_part_only():
  """rot.dims smaller than rot_dim: the remaining entries of the rotated part pass unchanged"""
  layer = attn("latent_attention", rot_dim=8, ff=0)
  layer["mixer"]["rot"]["dims"] = 4
  cfg = config([layer, attn("latent_attention_2", rot_dim=6, window=9, ff=0)])
  cfg["layers"][1]["mixer"]["rot"]["dims"] = 2
  W = zo.random_weights(cfg, 5)
  n = make_engine(cfg, W, "float32")
  check(n, cfg, W, rand_tokens(cfg["vocab"], 30, 1), [30], "float32")
  n.close()


# ---- prefill / decoding / portions -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[1], [2], [3], [17, 1], [5, 2, 9, 1], [64]])
def test_portions_equal_the_whole_prompt(cuts, dtype):
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 2)
  n = make_engine(cfg, W, dtype, page_size=4)
  toks = rand_tokens(cfg["vocab"], 37, 8)
  got = check(n, cfg, W, toks, cuts, dtype)
  n.clear_request(0)
  whole = run_cut(n, 0, toks, [len(toks)])
  # the engine against itself: cutting the prompt changes rounding only
  assert row_err(got, whole.astype(np.float64)) < (2e-5 if dtype == "float32" else 0.05)
  n.close()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
  cfg = config([attn("latent_attention_2", window=33), delta(heads=2, dim=16), attn("latent_attention")], width=32, groups=2)
  W = zo.random_weights(cfg, 21)
  n = make_engine(cfg, W, dtype, max_tokens=400, page_size=16)
  check(n, cfg, W, rand_tokens(cfg["vocab"], 300, 4), [6, 1], dtype)
  n.close()


def test_first_tokens_of_a_sequence():
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 9)
  n = make_engine(cfg, W, "float32")
  for length in (1, 2, 3):
    n.clear_request(0)
    check(n, cfg, W, rand_tokens(cfg["vocab"], length, length), [1], "float32")
  n.close()


# ---- batches ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_equal_each_alone(dtype):
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 4)
  n = make_engine(cfg, W, dtype, max_tokens=256, max_requests=5, page_size=4)
  lens = [1, 13, 30, 2, 8]
  seqs = [rand_tokens(cfg["vocab"], L + 6, 50 + i) for i, L in enumerate(lens)]
  refs = [oracle_logits(cfg, W, s)[0] for s in seqs]
  slots = [3, 0, 4, 1, 2]
  # prompts together (all rows wanted), then six decoding steps together, the shortest requests leaving early
  rows = [s[:L] for s, L in zip(seqs, lens)]
  lg, _ = n.step(slots, rows, want=list(range(sum(lens))))
  at = 0
  for i, L in enumerate(lens):
    assert row_err(lg[at:at + L], refs[i][:L]) < TOL[dtype], f"prompt of request {i}"
    at += L
  live = list(range(len(lens)))
  for t in range(6):
    if t == 2:
      live.remove(0)
      n.clear_request(slots[0])
    if t == 4:
      live.remove(3)
      n.clear_request(slots[3])
    lg, am = n.step([slots[i] for i in live], [seqs[i][lens[i] + t:lens[i] + t + 1] for i in live])
    for k, i in enumerate(live):
      assert row_err(lg[k:k + 1], refs[i][lens[i] + t:lens[i] + t + 1]) < TOL[dtype], f"request {i}, decoded token {t}"
      assert am[k] == int(np.argmax(lg[k]))
  n.close()


def test_mixed_batch_of_portions_and_decoded_rows():
  """one step may bring a prompt portion for one request and a single row for another"""
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 6)
  n = make_engine(cfg, W, "float32", page_size=4)
  a, b = rand_tokens(cfg["vocab"], 20, 1), rand_tokens(cfg["vocab"], 26, 2)
  ra, rb = oracle_logits(cfg, W, a)[0], oracle_logits(cfg, W, b)[0]
  n.step([0], [a[:15]])
  lg, _ = n.step([0, 1], [a[15:16], b[:11]], want=list(range(12)))
  assert row_err(lg[:1], ra[15:16]) < TOL["float32"] and row_err(lg[1:], rb[:11]) < TOL["float32"]
  lg, _ = n.step([1, 0], [b[11:26], a[16:17]], want=list(range(16)))
  assert row_err(lg[:15], rb[11:26]) < TOL["float32"] and row_err(lg[15:], ra[16:17]) < TOL["float32"]
  n.close()


# ---- pages and slots that are given back and used again ---------------------------------------------------------------------
def test_freed_pages_and_slots_are_clean_for_the_next_request():
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 13)
  n = make_engine(cfg, W, "float32", max_tokens=64, max_requests=2, page_size=4)
  total = n.cache_stats()["pages_total"]
  a, b, c = (rand_tokens(cfg["vocab"], L, s) for L, s in ((29, 1), (18, 2), (31, 3)))
  check(n, cfg, W, a, [9, 1], "float32", slot=0)
  check(n, cfg, W, b, [18], "float32", slot=1)
  assert n.cache_stats()["pages_free"] == total - 8 - 5
  n.clear_request(0)                                  # a's pages (and its recurrent state) go back ...
  assert n.cache_stats()["pages_free"] == total - 5 and n.request_len(0) == 0
  check(n, cfg, W, c, [5, 3, 1], "float32", slot=0)   # ... and c gets them, in another order, next to the live b
  lg, _ = n.step([1], [a[:3]], want=[0, 1, 2])        # b goes on undisturbed
  ref = oracle_logits(cfg, W, np.concatenate([b, a[:3]]))[0]
  assert row_err(lg, ref[18:]) < TOL["float32"]
  n.clear_request(0)
  n.clear_request(1)
  assert n.cache_stats()["pages_free"] == total
  with pytest.raises(Exception, match="cache"):       # a request larger than the pool is refused and changes nothing
    n.step([0], [rand_tokens(cfg["vocab"], 200, 1)])
  assert n.cache_stats()["pages_free"] == total and n.request_len(0) == 0
  n.close()


# ---- keys that must (not) be seen: made to stand out -------------------------------------------------------------------------
def needle(cfg, W, seq, pos, vocab):
  """the token that, put at `pos`, moves the last row's logits the most (searched with the oracle), and by how much"""
  base = oracle_logits(cfg, W, seq, torch.float32)[0][-1]
  best, gain = 0, -1.0
  for t in range(vocab):
    if t == seq[pos]:
      continue
    s = seq.copy()
    s[pos] = t
    d = np.abs(oracle_logits(cfg, W, s, torch.float32)[0][-1] - base).max()
    if d > gain:
      best, gain = t, d
  return best, gain


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_and_far_keys(decode, dtype):
  """sharp attention (large score scale): one key takes nearly all the weight.  A far key under the causal mixer, the oldest key
  inside a window and the newest key outside it are each made that key; reading one key too many or too few moves the logits by
  far more than the tolerance."""
  V, n_tok, window = 40, 150, 23
  last = n_tok - 1
  cases = [("far", attn("latent_attention", heads=2, ff=0, scale=8.0), 3, None),
           ("page_border", attn("latent_attention", heads=2, ff=0, scale=8.0), 64, None),
           ("window_in", attn("latent_attention_2", heads=2, ff=0, scale=8.0, window=window), last - window + 1, None),
           ("window_out", attn("latent_attention_2", heads=2, ff=0, scale=8.0, window=window), last - window, window + 1)]
  for name, layer, pos, search_window in cases:
    cfg = config([layer], vocab=V, width=32, groups=2)
    W = zo.random_weights(cfg, 17)
    seq = rand_tokens(V, n_tok, 5)
    scfg = config([layer], vocab=V, width=32, groups=2)
    if search_window:
      scfg["layers"][0]["mixer"]["mask"]["size"] = search_window   # the token that WOULD dominate if it were seen
    tok, gain = needle(scfg, W, seq, pos, V)
    assert gain > 0.5, f"{name}: the made-up key does not stand out ({gain})"
    seq[pos] = tok
    ref = oracle_logits(cfg, W, seq)[0]
    n = make_engine(cfg, W, dtype, max_tokens=256, page_size=64 if name == "page_border" else 16)
    got = run_cut(n, 0, seq, [n_tok - 40, 1] if decode else [n_tok])
    # scores eight times sharper than usual magnify the 16-bit rounding of the scores too; a misread key costs 0.5 and more
    tol = TOL[dtype] * (3 if dtype == "bfloat16" else 1)
    e = row_err(got[-1:], ref[-1:])
    assert e < tol, f"{name} ({'decoded' if decode else 'prompt'}): {e:.3e}"
    assert row_err(got, ref) < tol
    n.close()


# ---- several shards ----------------------------------------------------------------------------------------------------------
def test_two_shards_hand_over_the_residual_stream():
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 31)
  a = make_engine(cfg, W, "float32", start=0, end=1)
  b = make_engine(cfg, W, "float32", start=2, end=4)
  toks = rand_tokens(cfg["vocab"], 19, 7)
  ref = oracle_logits(cfg, W, toks)[0]
  hid = a.step([0], [toks[:12]])
  lg, _ = b.step([0], [hid], want=list(range(12)))
  assert row_err(lg, ref[:12]) < TOL["float32"]
  hid = a.step([0], [toks[12:]])
  lg, _ = b.step([0], [hid], want=list(range(7)))
  assert row_err(lg, ref[12:]) < TOL["float32"]
  a.close()
  b.close()


# ---- the loader ---------------------------------------------------------------------------------------------------------------
def write_model_dir(path, cfg, W):
  import json
  import struct
  from tests.layered_util import bf16_bits
  hdr, blobs, at = {}, [], 0
  for k, t in W.items():
    raw = bf16_bits(t).tobytes()
    hdr[k] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
    blobs.append(raw)
    at += len(raw)
  h = json.dumps(hdr).encode()
  with open(path / "model.safetensors", "wb") as f:
    f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))
  with open(path / "config.json", "w") as f:
    json.dump(public_config(cfg), f)


def test_model_directory_loader_is_strict(tmp_path):
  from xotorch_b200.models import load_model_config, make_native
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 3)
  write_model_dir(tmp_path, cfg, W)
  n = make_native(load_model_config(tmp_path), 0, "float32")
  n.load_dir(tmp_path)
  n.begin_pool(64, 1, 8)
  toks = rand_tokens(cfg["vocab"], 12, 1)
  check(n, cfg, W, toks, [12], "float32")
  n.close()
  bad = dict(W)
  del bad["l2.mix.w0"]
  write_model_dir(tmp_path, cfg, bad)
  with pytest.raises(Exception, match="l2.mix.w0"):
    make_native(load_model_config(tmp_path), 0, "float32").load_dir(tmp_path)
  bad = dict(W)
  bad["l0.mix.extra"] = torch.zeros(2, 2)
  write_model_dir(tmp_path, cfg, bad)
  with pytest.raises(Exception, match="l0.mix.extra"):
    make_native(load_model_config(tmp_path), 0, "float32").load_dir(tmp_path)


# ---- generation through the scheduler ---------------------------------------------------------------------------------------------
def oracle_greedy(cfg, W, prompt, n_new):
  """greedy ids and, per step, the gap between the two largest logits"""
  seq, ids, gaps = list(prompt), [], []
  for _ in range(n_new):
    lg = oracle_logits(cfg, W, np.array(seq))[0][-1]
    top = np.sort(lg)[-2:]
    ids.append(int(np.argmax(lg)))
    gaps.append(float(top[1] - top[0]))
    seq.append(ids[-1])
  return ids, gaps


@pytest.mark.parametrize("dtype,budget", [("float32", 2048), ("bfloat16", 7)])
def test_greedy_generation_through_the_batch_scheduler(dtype, budget):
  from xotorch_b200.scheduler import ContinuousBatch
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 8)
  n = make_engine(cfg, W, dtype)
  events = []
  sched = ContinuousBatch(n, max_requests=3, max_tokens=160, page_size=8, token_budget=budget,
                          on_token=lambda rid, toks, fin: events.append((rid, list(toks), fin)))
  reqs = [(f"r{i}", rand_tokens(cfg["vocab"], L, 70 + i), g) for i, (L, g) in enumerate([(5, 9), (17, 4), (1, 12), (26, 6), (3, 1)])]
  for rid, p, g in reqs[:3]:
    sched.submit(rid, p, g)
  sched.step()
  for rid, p, g in reqs[3:]:
    sched.submit(rid, p, g)                           # joins while others are running
  out = sched.run_until_idle()
  for rid, p, g in reqs:
    ids, gaps = oracle_greedy(cfg, W, p, g)
    assert len(out[rid]) == g
    if out[rid] != ids:                               # after a near tie the continuations differ legitimately
      d = next(i for i in range(g) if out[rid][i] != ids[i])
      assert gaps[d] < (1e-3 if dtype == "float32" else 0.15), f"{rid}: ids leave the oracle's at step {d} with a clear gap {gaps[d]}"
    assert [e[1][0] for e in events if e[0] == rid] == out[rid]
    assert [e[2] for e in events if e[0] == rid] == [False] * (g - 1) + [True]
  st = n.cache_stats()
  assert st["pages_free"] == st["pages_total"], "finished requests must give their pages back"
  n.close()


# ---- the tensor-core products ------------------------------------------------------------------------------------------------------
def test_tensor_core_products_equal_the_fma_tiles():
  """sizes that TMA can describe (multiples of 8): prompts run their products on tcgen05, decoding on the one-warp-per-output
  kernel; both must agree with the fp32-FMA tiles on the same 16-bit operands, and with the oracle"""
  layers = [attn("latent_attention", heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=24, ff=72),
            attn("latent_attention_2", heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, window=70, ff=200),
            delta(heads=2, dim=16, decay_rank=8, ff=0)]
  cfg = config(layers, width=64, vocab=136, groups=4)
  W = zo.random_weights(cfg, 12)
  n = make_engine(cfg, W, "bfloat16", max_tokens=700, page_size=32)
  toks = rand_tokens(cfg["vocab"], 300, 9)      # 300 rows: two full 128-row tiles and a ragged one
  ref = oracle_logits(cfg, W, toks)[0]
  before = n.tensor_core_launches()
  tc = run_cut(n, 0, toks, [300])
  used = n.tensor_core_launches() - before
  assert used == 17, f"{used} of the prompt's 17 products ran on the tensor cores"
  n.set_gemm_mode(1)
  fma = run_cut(n, 1, toks, [300])
  assert n.tensor_core_launches() - before == used
  assert row_err(tc, ref) < TOL["bfloat16"] and row_err(fma, ref) < TOL["bfloat16"]
  assert row_err(tc, fma.astype(np.float64)) < 0.02, "same operands, fp32 accumulation in both: only the summation order differs"
  n.set_gemm_mode(2)                            # tensor cores also for a handful of rows
  few = run_cut(n, 2, toks[:40], [5, 1])
  assert row_err(few, ref[:40]) < TOL["bfloat16"]
  n.close()


# ---- prompt attention in the expanded form -----------------------------------------------------------------------------------------
@pytest.mark.parametrize("sizes", ["aligned", "odd"])
def test_expanded_prompt_attention_equals_the_absorbed_kernel(sizes):
  """bf16: a request that brings 16 rows or more has its keys and values expanded and runs the tensor-core streaming-softmax
  kernel; fewer rows run the absorbed kernel over the latent rows.  Same design, two kernels: they agree with each other and
  with the oracle — across 64-row tiles, second portions that start inside a window, gated and windowed mixers, in one batch
  with short requests."""
  if sizes == "aligned":
    layers = [attn("latent_attention", heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=24, ff=0),
              attn("latent_attention_2", heads=2, dim=32, rot_dim=16, vdim=72, kv_rank=64, window=70, ff=64)]
  else:
    layers = [attn("latent_attention", heads=3, dim=10, rot_dim=6, vdim=5, kv_rank=21, q_rank=9, ff=0),
              attn("latent_attention_2", heads=5, dim=7, rot_dim=4, vdim=9, kv_rank=12, window=37, ff=20)]
  cfg = config(layers, width=64 if sizes == "aligned" else 40, vocab=90, groups=4)
  W = zo.random_weights(cfg, 14)
  n = make_engine(cfg, W, "bfloat16", max_tokens=1200, max_requests=4, page_size=16)
  a, b, c = rand_tokens(90, 333, 1), rand_tokens(90, 150, 2), rand_tokens(90, 9, 3)
  ra, rb, rc = (oracle_logits(cfg, W, t)[0] for t in (a, b, c))
  before = n.prompt_attention_launches()
  # step 1: a's first 200 rows, all of b and all of c (short: absorbed) in one batch;  step 2: the rest of a (133 rows, starts at 200)
  lg1, _ = n.step([0, 1, 2], [a[:200], b, c], want=list(range(200 + 150 + 9)))
  lg2, _ = n.step([0], [a[200:]], want=list(range(133)))
  assert n.prompt_attention_launches() - before == 4
  got_a = np.concatenate([lg1[:200], lg2])
  for got, ref, who in ((got_a, ra, "a"), (lg1[200:350], rb, "b"), (lg1[350:], rc, "c")):
    assert row_err(got, ref) < TOL["bfloat16"], who
  n.set_attention_mode(1)
  n.clear_request(0)
  absorbed = run_cut(n, 0, a, [200, 133])
  assert n.prompt_attention_launches() - before == 4
  assert row_err(got_a, absorbed.astype(np.float64)) < 0.03
  n.close()


# ---- decode steps replayed from CUDA graphs ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_graph_replay_of_decode_steps_changes_nothing(dtype):
  """a decode step is captured the second time its shape is seen and replayed afterwards; lengths, pages, slots and wanted rows
  live in device arrays that every replay refreshes — so the logits equal those of plain launches bit for bit, across page
  borders, across the 256-token length bucket, and when a request leaves the batch"""
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 19)
  seqs = [rand_tokens(cfg["vocab"], 300, 40 + i) for i in range(3)]
  starts = [240, 3, 17]

  def run(graphs):
    n = make_engine(cfg, W, dtype, max_tokens=1000, max_requests=3, page_size=8)
    n.set_graphs(graphs)
    n.step([0, 1, 2], [s[:k] for s, k in zip(seqs, starts)])
    out, live = [], [0, 1, 2]
    for t in range(40):
      if t == 25:
        live = [0, 2]
        n.clear_request(1)
      lg, _ = n.step(live, [seqs[i][starts[i] + t:starts[i] + t + 1] for i in live])
      out.append(lg)
    replays = n.graph_replays()
    n.close()
    return out, replays

  plain, r0 = run(False)
  replayed, r1 = run(True)
  assert r0 == 0 and r1 >= 30
  for a, b in zip(plain, replayed):
    assert np.array_equal(a, b)
  ref = oracle_logits(cfg, W, seqs[0][:280])[0]
  got = np.stack([x[0] for x in replayed])
  assert row_err(got, ref[240:280]) < TOL[dtype]


def test_command_line_generates_from_a_model_directory(tmp_path, capsys):
  """`xotorch_b200.cli generate` on a layered model directory: registry -> loader -> batch scheduler -> greedy ids"""
  import json
  from xotorch_b200.cli import main
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 8)
  write_model_dir(tmp_path, cfg, W)
  prompts = [rand_tokens(cfg["vocab"], 6, 1), rand_tokens(cfg["vocab"], 11, 2)]
  arg = ";".join(",".join(str(int(t)) for t in p) for p in prompts)
  assert main(["generate", "--model", str(tmp_path), "--prompt-ids", arg, "--max-tokens", "5", "--dtype", "float32"]) == 0
  lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
  for p, line in zip(prompts, lines):
    ids, gaps = oracle_greedy(cfg, W, p, 5)
    if line["ids"] != ids:
      d = next(i for i in range(5) if line["ids"][i] != ids[i])
      assert gaps[d] < 1e-3


def test_wide_values_keep_all_attention_on_the_absorbed_kernel():
  """a value size beyond what the expanded kernel's tiles hold: prompts of any length still come out right (absorbed form)"""
  cfg = config([attn("latent_attention", heads=2, dim=8, rot_dim=8, vdim=136, kv_rank=16, q_rank=8, ff=0)], width=32, groups=2)
  W = zo.random_weights(cfg, 23)
  n = make_engine(cfg, W, "bfloat16")
  check(n, cfg, W, rand_tokens(cfg["vocab"], 70, 2), [40, 30], "bfloat16")
  assert n.prompt_attention_launches() == 0
  n.close()


def test_inference_engine_serves_a_layered_model_directory(tmp_path):
  """`B200ShardInferenceEngine` (the reference's engine interface) on a layered model split over two shards, two request ids
  interleaved: ensure_shard -> registry -> LayeredShard, the position protocol of infer_tensor, sample(temp 0)"""
  import asyncio
  from xotorch_b200.inference.b200_engine import B200ShardInferenceEngine, LocalDirDownloader
  from xotorch_b200.inference.shard import Shard
  cfg = config(MIXED)
  W = zo.random_weights(cfg, 27)
  write_model_dir(tmp_path, cfg, W)
  n = len(cfg["layers"])
  first, last = Shard("m", 0, 1, n), Shard("m", 2, n - 1, n)
  prompts = {"a": rand_tokens(cfg["vocab"], 9, 1), "b": rand_tokens(cfg["vocab"], 21, 2)}

  async def run():
    e1 = B200ShardInferenceEngine(LocalDirDownloader({"m": tmp_path}), device=0, max_concurrent_requests=2, max_total_len=64)
    e2 = B200ShardInferenceEngine(LocalDirDownloader({"m": tmp_path}), device=0, max_concurrent_requests=2, max_total_len=64)
    out, state, data = {r: [] for r in prompts}, {r: None for r in prompts}, {r: p.reshape(1, -1).astype(np.int64) for r, p in prompts.items()}
    for _ in range(4):
      for r in prompts:                               # the two requests take turns, token by token
        hid, st = await e1.infer_tensor(r, first, data[r], state[r])
        assert hid.ndim == 3 and hid.shape[2] == cfg["width"]
        logits, st2 = await e2.infer_tensor(r, last, hid, state[r])
        tok = await e2.sample(logits, temp=0.0)
        out[r].append(int(tok[0, 0]))
        state[r] = st2
        data[r] = tok.reshape(1, 1).astype(np.int64)
    return out

  out = asyncio.run(run())
  for r, p in prompts.items():
    ids, gaps = oracle_greedy(cfg, W, p, 4)
    if out[r] != ids:
      d = next(i for i in range(4) if out[r][i] != ids[i])
      assert gaps[d] < 0.15, f"{r}: ids leave the oracle's at step {d} with a clear gap"
