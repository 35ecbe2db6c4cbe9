"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
``load_model`` and ``Engine.step``, the ones generation uses.  Input: one JSON object per line on
standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request's next tokens and the places among them whose logits are wanted;
``end`` names requests that are finished after the step.  For a step with wanted places the
logits are written to ``<out>/<step>.f32`` as little-endian float32 ``[wanted, vocab]``, in the
order of the entries and of ``want``.  After every step the line ``done <step>`` is printed and
flushed.  The reference has only tests that dump logits token by token
(tests/Daisi.Llogos.Tests/Chat/LogitDumpTest.cs:36-96); this program is the library's own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

from .engine.engine import Engine
from .weights.loader import load_model

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=sorted(_DTYPES))
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each request rounded up to 64")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--no-graphs", action="store_true", help="do not replay decode steps as CUDA graphs")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    os.makedirs(args.out, exist_ok=True)

    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = load_model(args.model, dtype=_DTYPES[args.dtype], device=args.device)
    pages = (args.max_tokens + 63) // 64
    # the longest single request: what the cache holds, or the model's position limit where that is less
    engine = Engine(model, max_tokens=pages * 64, use_graphs=not args.no_graphs)
    print(f"[trace_run] ready: cache of {pages} pages of 64 tokens ({engine.cache.bytes() / 2**20:.1f} MiB)",
          file=sys.stderr, flush=True)

    slot_of = {}
    for line_no, line in enumerate(sys.stdin, 1):
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = rec.get("entries", [])
            ended = rec.get("end", [])
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            print(f"[trace_run] line {line_no}: not a step record ({e})", file=sys.stderr, flush=True)
            return 2
        batch, want = [], []
        for e in entries:
            rid = e["id"]
            if rid not in slot_of:
                slot_of[rid] = engine.open()
            batch.append((slot_of[rid], e["tokens"]))
            want.append(list(e.get("want", [])))
        if batch:
            logits = engine.step(batch, want)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in ended:
            slot = slot_of.pop(rid, None)
            if slot is not None:
                engine.close(slot)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
