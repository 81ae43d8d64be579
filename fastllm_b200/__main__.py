"""Command line of the package.

    python -m fastllm_b200 generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] [--max-tokens N] [--temperature T]
                                    [--dtype bf16|f32] [--max-batch B] [--prefill-chunk C] [--eos ID]
    python -m fastllm_b200 trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (same as bin/trace_run)

`generate` loads the model the registry picks for DIR/config.json and continues every prompt (token ids in, token ids out: the
tokenizer stays with the server above this library) through the continuous batcher; one JSON line per prompt.
"""
from __future__ import annotations

import argparse
import json
import sys


def _generate(argv) -> int:
    ap = argparse.ArgumentParser(prog="python -m fastllm_b200 generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for several prompts")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--max-batch", type=int, default=4)
    ap.add_argument("--prefill-chunk", type=int, default=None)
    ap.add_argument("--eos", type=int, default=None)
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)
    from . import build
    build.build_library()
    from . import models
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    model, _ = models.load_model(a.model, a.dtype, a.device)
    batcher = models.ContinuousBatcher(model, max_batch=a.max_batch, eos_token_id=a.eos, prefill_chunk=a.prefill_chunk)
    for p, ids in zip(prompts, batcher.generate(prompts, a.max_tokens, a.temperature)):
        print(json.dumps({"prompt": p, "generated": [int(t) for t in ids]}))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    if argv[0] == "generate":
        return _generate(argv[1:])
    if argv[0] == "trace":
        from . import trace_runner
        return trace_runner.main(argv[1:])
    print(f"unknown command {argv[0]!r}\n{__doc__}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
