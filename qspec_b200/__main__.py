"""Command line of the framework.

    python -m qspec_b200 models                                   architectures the registry knows
    python -m qspec_b200 generate --model DIR --prompt 5,17,3 [--prompt ...] [--max-new-tokens N] [--dtype bfloat16]
    python -m qspec_b200 trace --model DIR --dtype ... --out DIR  replay recorded steps (qspec_b200/trace.py)
    python -m qspec_b200 build [--seq]                            compile the kernel libraries

`generate` takes prompts as comma-separated token ids (the framework has no tokenizer), runs them through the
continuous-batching scheduler with greedy sampling and prints one JSON line per prompt.
"""
from __future__ import annotations

import argparse
import json
import sys


def _generate(argv) -> int:
    ap = argparse.ArgumentParser(prog="python -m qspec_b200 generate")
    ap.add_argument("--model", required=True, help="folder with config.json (and weights)")
    ap.add_argument("--dtype", default=None, help="bfloat16 | float32 | float16 (default: the model's serving type)")
    ap.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for several prompts")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--eos", type=int, default=None)
    ap.add_argument("--slots", type=int, default=8)
    ap.add_argument("--step-tokens", type=int, default=2048)
    ap.add_argument("--prefill-portion", type=int, default=None, help="most prompt tokens of one request per step")
    args = ap.parse_args(argv)
    from . import registry
    from .build import build_library, build_seq_library
    arch = registry.architecture_of(registry.read_config(args.model))
    build_seq_library()
    if arch not in registry.SEQUENCE_DESIGNS:
        build_library()
    from .scheduler import Scheduler
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt]
    # models whose cache grows with the sequence size it for the longest request
    model = registry.load_model(args.model, dtype=args.dtype, n_slots=args.slots, max_step_tokens=args.step_tokens,
                                max_seq_tokens=max(len(p) for p in prompts) + args.max_new_tokens)
    outs = Scheduler(model, prefill_portion=args.prefill_portion).generate(prompts, args.max_new_tokens, eos=args.eos)
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt": p, "tokens": o}))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "models":
        from . import registry
        print("\n".join(registry.architectures()))
        return 0
    if cmd == "generate":
        return _generate(rest)
    if cmd == "trace":
        from .trace import main as trace_main
        return trace_main(rest)
    if cmd == "build":
        from .build import build_library, build_seq_library
        print(build_seq_library(force="--force" in rest, verbose=True) if "--seq" in rest
              else build_library(force="--force" in rest, verbose=True))
        return 0
    print(f"unknown command {cmd!r}\n{__doc__}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
