"""Command line of the serving engine.

    python -m atoma_infer_b200 generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] [--max-new-tokens N]
                                        [--dtype bfloat16|float32] [--max-tokens N] [--max-live N] [--block-size N]
    python -m atoma_infer_b200 trace    --model DIR --dtype ... --out DIR --max-tokens N      (same as bin/trace_run)
    python -m atoma_infer_b200 models                                                         (registered architectures)

`generate` loads the model named by DIR/config.json through the model registry, runs the prompts (token ids; the
library has no tokenizer) through the scheduler with continuous batching and greedy sampling, and prints one JSON
line per prompt: {"prompt": [...], "generated": [...]}."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "trace":
        from .trace import main as trace_main
        return trace_main(rest)
    if cmd == "models":
        from . import models
        print("\n".join(sorted(models.MODEL_REGISTRY)))
        return 0
    if cmd != "generate":
        print(f"unknown command {cmd!r}\n{__doc__}", file=sys.stderr)
        return 2
    ap = argparse.ArgumentParser(prog="atoma_infer_b200 generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for more prompts")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-tokens", type=int, default=8192, help="tokens the page pool holds")
    ap.add_argument("--max-live", type=int, default=4, help="requests live at a time (state slots)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--stop-token-id", type=int, action="append", default=[])
    a = ap.parse_args(rest)
    from . import _lib
    _lib.ensure_built()
    import torch

    from .engine import Engine
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    eng = Engine.from_model_dir(a.model, dtype=dtype, device="cuda:0", max_tokens=a.max_tokens, block_size=a.block_size,
                                max_live_requests=a.max_live)
    for p, g in zip(prompts, eng.generate(prompts, a.max_new_tokens, tuple(a.stop_token_id))):
        print(json.dumps({"prompt": p, "generated": g}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
