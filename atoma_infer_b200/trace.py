"""Trace replay: feeds given token ids through a model step by step and writes the logits asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` = per request its next tokens and the places among them whose logits are wanted; all entries of
a step run as ONE batch (portions of prompts beside single tokens); `end` = requests that are over after
the step (their pages and state slot are given back).  For a step that wants something the logits are
written to DIR/<step>.f32 (little-endian float32 [wanted, vocab], in the order of the entries and their
wanted places); after every step a line `done <step>` is printed.  Nothing is sampled.

The replay drives the serving engine itself (engine.Engine.step_forced -> scheduler.plan_forced ->
cache manager -> the model's executor): the page pool is sized for --max-tokens and there are four
state slots, so pages and slots are reused as requests end.  The shared library is built on first use.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-live", type=int, default=4)
    a = ap.parse_args(argv)

    from . import _lib
    _lib.ensure_built()
    import numpy as np
    import torch

    from .engine import Engine

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device", file=sys.stderr)
        return 1
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    engine = Engine.from_model_dir(a.model, dtype=dtype, device="cuda:0", max_tokens=a.max_tokens, block_size=a.block_size,
                                   max_live_requests=a.max_live)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        n = msg["step"]
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in msg.get("entries", []) if e.get("tokens")]
        if entries:
            out = engine.step_forced(entries, msg.get("end", []))
            if out.logits is not None and out.logits.shape[0] > 0:
                arr = out.logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                with open(os.path.join(a.out, f"{n}.f32"), "wb") as f:
                    f.write(np.ascontiguousarray(arr).tobytes())
            else:
                torch.cuda.synchronize()
        else:
            for seq_id in msg.get("end", []):
                if seq_id in engine.sequences:
                    engine.finish_request(seq_id)
        sys.stdout.write(f"done {n}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
