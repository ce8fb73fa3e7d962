"""Replay of a token trace through a model: given token ids go in step by step, logits come out; nothing is sampled.

A trace is a stream of JSON lines on standard input, one step each:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["b"]}

`entries` brings every participating request its next tokens (a whole prompt, a portion of one, or a single decoded token) and
names in `want` the places among them whose logits are asked for; `end` lists requests that are over after the step.  All entries
of a step run as ONE batch of the native engine (`LayeredShard.step`: packed rows, paged cache, per-request state); a request
keeps its slot from its first step until it is ended, then the slot's pages and state go back to the pool.  For a step that wants
something, `<out>/<step>.f32` receives the logits as little-endian float32 [wanted, vocab] in the order of the entries; after
every step the line `done <step>` is printed.

The replayer owns no model code: the engine comes from the model registry (xotorch_b200/models.py), the request table is the one
the scheduler uses (`RequestSlots`)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Optional

import numpy as np

from .layered import RequestSlots
from .models import load_model_config, make_native, model_summary

EXIT_NO_FLOAT32 = 3


class TraceReplayer:
  def __init__(self, model_dir, dtype: str, out_dir, max_tokens: int, device: int = 0, max_requests: Optional[int] = None):
    cfg = load_model_config(model_dir)
    if model_summary(cfg)["engine"] != "layered":
      raise NotImplementedError("trace replay drives the batched step of the layered engine; the shard engine serves one row "
                                "batch per request (use B200ShardInferenceEngine / ContinuousRing for those models)")
    self.native = make_native(cfg, device, dtype)
    self.native.load_dir(model_dir)
    # every live request holds at least one token, so max_tokens also bounds the requests; the table is kept moderate
    n_req = int(max_requests) if max_requests else max(1, min(int(max_tokens), 256))
    self.native.begin_pool(int(max_tokens), n_req)
    self.slots = RequestSlots(self.native)
    self.out_dir = Path(out_dir)
    self.out_dir.mkdir(parents=True, exist_ok=True)

  def run_step(self, step: dict) -> int:
    entries = step.get("entries", [])
    slots, rows, want = [], [], []
    base = 0
    for en in entries:
      slots.append(self.slots.acquire(en["id"]))
      toks = np.asarray(en["tokens"], dtype=np.int32).reshape(-1)
      rows.append(toks)
      want += [base + int(w) for w in en.get("want", [])]
      base += toks.size
    if entries:
      logits, _ = self.native.step(slots, rows, want=want, logits=True, argmax=False)
      if want:
        tmp = self.out_dir / f".{int(step['step'])}.part"
        np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
        os.replace(tmp, self.out_dir / f"{int(step['step'])}.f32")
    for rid in step.get("end", []):
      self.slots.release(rid)
    return len(want)

  def close(self):
    self.native.close()


def main(argv=None) -> int:
  ap = argparse.ArgumentParser(prog="trace_run", description="replay a token trace (JSON lines on stdin) through a model and write logits")
  ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
  ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                  help="bfloat16: the serving kernels; float32: everything in true 32-bit")
  ap.add_argument("--out", required=True, help="folder for <step>.f32")
  ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens that live requests hold at any time (sizes the cache)")
  ap.add_argument("--max-requests", type=int, default=0, help="most live requests (default: derived from --max-tokens)")
  ap.add_argument("--device", type=int, default=0)
  a = ap.parse_args(argv)
  rp = TraceReplayer(a.model, a.dtype, a.out, a.max_tokens, a.device, a.max_requests or None)
  try:
    for line in sys.stdin:
      line = line.strip()
      if not line:
        continue
      step = json.loads(line)
      rp.run_step(step)
      sys.stdout.write(f"done {int(step['step'])}\n")
      sys.stdout.flush()
  finally:
    rp.close()
  return 0


if __name__ == "__main__":
  sys.exit(main())
