"""Command line: ``python -m lite_llama_b200 <command>``.

    generate  --model DIR [--dtype bfloat16] --prompt 1,2,3 [--prompt ...] --max-new-tokens N
              greedy continuation of token-id prompts through the engine (no tokenizer ships with the package)
    trace     --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (steps on standard input)
    build     compile the in-tree CUDA library
    archs     list the registered architectures
"""

from __future__ import annotations

import argparse
import json
import sys


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="lite_llama_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--model", required=True)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    g.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeatable")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--max-tokens", type=int, default=8192, help="rows of the KV pool")
    g.add_argument("--max-requests", type=int, default=4)
    g.add_argument("--max-step-tokens", type=int, default=2048)
    t = sub.add_parser("trace")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--max-requests", type=int, default=4)
    sub.add_parser("build")
    sub.add_parser("archs")
    a = ap.parse_args(argv)
    if a.cmd == "archs":
        from .executor import registry

        print("\n".join(registry.names()))
        return 0
    from .build import LAYERED_SOURCES, build

    if a.cmd == "build":
        build(verbose=True)
        return 0
    from .executor.registry import architecture_of

    build(verbose=False, sources=architecture_of(a.model)[0].sources or LAYERED_SOURCES)    # what this family launches
    if a.cmd == "trace":
        from .trace import replay

        return replay(a.model, a.dtype, a.out, a.max_tokens, a.max_requests)
    from .engine import Engine
    from .executor import ModelRunner
    from .trace import DTYPES

    runner = ModelRunner.from_checkpoint(a.model, dtype=DTYPES[a.dtype], max_tokens=a.max_tokens,
                                         max_requests=a.max_requests)
    engine = Engine(runner, max_step_tokens=a.max_step_tokens)
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt]
    for p, out in zip(prompts, engine.generate(prompts, a.max_new_tokens)):
        print(json.dumps({"prompt": p, "tokens": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
