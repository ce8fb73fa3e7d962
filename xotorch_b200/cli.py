"""Command line of xotorch_b200.

  python -m xotorch_b200.cli generate --model DIR (--prompt TEXT | --prompt-ids 1,2,3) [--max-tokens N] [--temp T] [--top-k K]
  python -m xotorch_b200.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (= bin/trace_run)
  python -m xotorch_b200.cli info     --model DIR

`generate` picks the native engine from the model's config.json (xotorch_b200/models.py): a layered model runs through the
packed-batch scheduler (`ContinuousBatch`), a Llama / Mixtral checkpoint through the device-resident ring (`LocalRing`, greedy).
Several `--prompt-ids` (separated by ';') are served together."""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

from .models import load_model_config, make_native, model_summary


def _prompts(a, tokenizer):
  if a.prompt_ids:
    return [np.array([int(x) for x in part.replace(",", " ").split()], dtype=np.int32) for part in a.prompt_ids.split(";") if part.strip()]
  return [np.asarray(tokenizer.encode(a.prompt), dtype=np.int32).reshape(-1)]


def cmd_generate(a) -> int:
  from .inference.tokenizers import resolve_local_tokenizer
  cfg = load_model_config(a.model)
  info = model_summary(cfg)
  tok = resolve_local_tokenizer(a.model, info["vocab"])
  prompts = _prompts(a, tok)
  eos = getattr(tok, "eos_token_id", None)
  eos = None if eos is None or eos < 0 else int(eos)
  if info["engine"] == "layered":
    from .scheduler import ContinuousBatch
    native = make_native(cfg, a.device, a.dtype)
    native.load_dir(a.model)
    total = sum(len(p) + a.max_tokens for p in prompts)
    sched = ContinuousBatch(native, max_requests=min(len(prompts), 64), max_tokens=max(total, 64), temp=a.temp, top_k=a.top_k, seed=a.seed)
    for i, p in enumerate(prompts):
      sched.submit(f"request-{i}", p, a.max_tokens, eos)
    out = sched.run_until_idle()
    ids = [out[f"request-{i}"] for i in range(len(prompts))]
    native.close()
  else:
    if a.temp > 0:
      raise SystemExit("the device-resident ring generates greedily; sampling with a temperature goes through B200ShardInferenceEngine.sample")
    from .ring import LocalRing
    native = make_native(cfg, a.device)
    native.load_dir(a.model, 0, info["n_layers"] - 1)
    ring = LocalRing([native])
    ids = [ring.generate(p.reshape(1, -1), a.max_tokens)[0].tolist() for p in prompts]
    ring.close()
  for i, seq in enumerate(ids):
    print(json.dumps({"request": i, "ids": [int(t) for t in seq], "text": tok.decode(seq)}))
  return 0


def cmd_info(a) -> int:
  cfg = load_model_config(a.model)
  print(json.dumps(model_summary(cfg)))
  return 0


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(prog="xotorch_b200")
  sub = ap.add_subparsers(dest="cmd", required=True)
  g = sub.add_parser("generate", help="generate from a local model directory")
  g.add_argument("--model", required=True)
  g.add_argument("--prompt", default="")
  g.add_argument("--prompt-ids", default="", help="token ids, comma or space separated; ';' between requests")
  g.add_argument("--max-tokens", type=int, default=32)
  g.add_argument("--temp", type=float, default=0.0)
  g.add_argument("--top-k", type=int, default=35)
  g.add_argument("--seed", type=int, default=1234)
  g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="layered models: serving kernels or everything in 32-bit")
  g.add_argument("--device", type=int, default=0)
  g.set_defaults(fn=cmd_generate)
  i = sub.add_parser("info", help="which engine runs a model directory, and its sizes")
  i.add_argument("--model", required=True)
  i.set_defaults(fn=cmd_info)
  t = sub.add_parser("trace", help="replay a token trace from standard input (see xotorch_b200/trace_replay.py)", add_help=False)
  t.set_defaults(fn=None)
  if argv is None:
    argv = sys.argv[1:]
  if argv and argv[0] == "trace":
    from .trace_replay import main as trace_main
    return trace_main(argv[1:])
  a = ap.parse_args(argv)
  if a.cmd == "generate" and not (a.prompt or a.prompt_ids):
    ap.error("generate needs --prompt or --prompt-ids")
  return a.fn(a)


if __name__ == "__main__":
  sys.exit(main())
