"""Replays a token trace through a model, step by step, and writes the logits that the trace asks for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

It samples nothing: every step names, per request, the next tokens to feed and the places among them whose logits are wanted.
The engine underneath is the library's own: the registry picks the model class from config.json, the weights go through the
ordinary loader, requests live in sequence slots of a pooled device cache (pages handed out on demand, given back when a request
ends), and every step is ONE mixed-batch forward (DeviceCache.forward_ragged) -- portions of prompts beside single decoded tokens.

Input: one JSON object per line on standard input,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
Output: for a step that wants something, DIR/<step>.f32 (little-endian f32 [wanted places, vocab], in the order of the entries and
of their 'want' lists); after every step a line 'done <step>' on standard output.  Exit code 0 at end of input.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

MAX_LIVE = 4          # requests alive at the same time (sequence slots of the cache)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the live requests hold at most (each rounded up to a page)")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)

    from . import build
    build.build_library()               # compiles on the first call of a fresh checkout; a no-op afterwards
    from . import models

    model, _ = models.load_model(a.model, "f32" if a.dtype == "float32" else "bf16", a.device)
    if not hasattr(model, "new_device_cache"):
        print("trace_run: this model family has no mixed-batch step function", file=sys.stderr)
        return 4
    page = 64
    pool = max(page, (a.max_tokens + page - 1) // page * page)
    cache = model.new_device_cache(max_batch=MAX_LIVE, max_seq=pool, pool_tokens=pool)
    os.makedirs(a.out, exist_ok=True)
    slot_of: dict = {}
    free = list(range(MAX_LIVE))[::-1]
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        slots, toks, want = [], [], []
        for e in step.get("entries", []):
            if e["id"] not in slot_of:
                if not free:
                    raise RuntimeError("more live requests than sequence slots")
                slot_of[e["id"]] = free.pop()
            if not e.get("tokens"):
                continue                # admitted, nothing to feed in this step
            slots.append(slot_of[e["id"]])
            toks.append(e["tokens"])
            want.append(e.get("want", []))
        if slots:
            logits = cache.forward_ragged(slots, toks, want)
            if logits.shape[0] > 0:
                tmp = os.path.join(a.out, ".%d.f32.part" % step["step"])
                np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
                os.replace(tmp, os.path.join(a.out, "%d.f32" % step["step"]))
        for rid in step.get("end", []):
            if rid in slot_of:
                s = slot_of.pop(rid)
                cache.slot_reset(s)
                free.append(s)
        sys.stdout.write("done %d\n" % step["step"])
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
