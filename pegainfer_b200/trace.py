"""Replay a trace of engine steps and write the logits that were asked for.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Every entry carries a request's next tokens (a request is admitted at its first entry), ``want`` the offsets among them whose
logits are written, ``end`` the requests that are finished after the step.  All entries of a step run as one batch through
the engine (``pegainfer_b200.engine.Engine`` over the model class ``config.json`` names).  For a step with wanted rows the
logits go to ``<out>/<step>.f32`` as little-endian fp32 [rows, vocab]; after every step a line ``done <step>`` is printed.
Nothing is sampled.  The cache pool holds ``--max-tokens`` tokens and there are four request slots.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-requests", type=int, default=4)
    a = ap.parse_args(argv)

    from .registry import FLOAT32_CAPABLE, architecture_of
    arch = architecture_of(a.model)
    if a.dtype == "float32" and arch not in FLOAT32_CAPABLE:
        print(f"{arch} has no float32 path", file=sys.stderr)
        return 3
    from . import build
    build.build(parts=build.PARTS_OF.get(arch))
    from .engine import Engine
    from .registry import load_model
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_requests=a.max_requests)
    if not hasattr(model, "step"):
        print(f"{arch} has no ragged step to replay a trace with", file=sys.stderr)
        return 3
    eng = Engine(model)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        s = json.loads(line)
        logits = eng.step([(e["id"], e["tokens"], e.get("want", [])) for e in s["entries"]], s.get("end", []))
        if logits.shape[0]:
            tmp = os.path.join(a.out, f".{s['step']}.part")
            with open(tmp, "wb") as f:
                f.write(logits.numpy().astype("<f4").tobytes())
            os.replace(tmp, os.path.join(a.out, f"{s['step']}.f32"))
        print(f"done {s['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
