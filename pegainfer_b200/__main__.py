"""Command line of the package.

    python -m pegainfer_b200 build                      # compile the CUDA libraries in-tree
    python -m pegainfer_b200 generate --model DIR --prompt 5,17,3 [--prompt 9,9] [--max-new 16] [--dtype bfloat16|float32]
    python -m pegainfer_b200 trace --model DIR --dtype ... --out DIR --max-tokens N < steps.jsonl   (see pegainfer_b200/trace.py)

``generate`` loads the checkpoint with the class its ``config.json`` names and continues every prompt (token ids) greedily;
models with a ragged step run all prompts through the continuous-batching scheduler, the others one after another.
"""
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
    if cmd == "build":
        from . import build
        build.build(force="--force" in rest, verbose=True)
        return 0
    if cmd == "trace":
        from . import trace
        return trace.main(rest)
    if cmd != "generate":
        print(f"unknown command {cmd!r}\n{__doc__}", file=sys.stderr)
        return 2
    ap = argparse.ArgumentParser(prog="pegainfer_b200 generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for several requests")
    ap.add_argument("--max-new", type=int, default=16)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--max-live", type=int, default=4)
    ap.add_argument("--token-budget", type=int, default=256)
    a = ap.parse_args(rest)
    from . import build
    from .registry import architecture_of, load_model
    build.build(parts=build.PARTS_OF.get(architecture_of(a.model)))
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt]
    model = load_model(a.model, a.dtype, max_requests=a.max_live)
    if hasattr(model, "step"):
        from .engine import Engine
        outs = Engine(model).generate(prompts, a.max_new, max_live=a.max_live, token_budget=a.token_budget)
    else:
        outs = [model.generate(p, a.max_new)[0] for p in prompts]
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt": p, "generated": o}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
