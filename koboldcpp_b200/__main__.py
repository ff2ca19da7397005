"""Command line: `python -m koboldcpp_b200 generate --model DIR --prompt 5,17,3 [--prompt ...] --max-new-tokens 32`.

Prompts and outputs are token ids (tokenisers are outside this package).  One JSON line per request is printed.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="koboldcpp_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate token ids from prompts of token ids")
    g.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--n-ctx", type=int, default=0, help="cache cells (default: what the prompts need)")
    a = ap.parse_args(argv)

    from . import build as _build
    _build.build()
    from .engine import Engine, Request, Sampler
    from .models import load_model

    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt]
    need = sum(len(p) + a.max_new_tokens for p in prompts)
    model = load_model(a.model, dtype=a.dtype, n_ctx=a.n_ctx or need, n_seq_max=len(prompts), max_batch=min(max(need, 1), 4096))
    reqs = [Request(p, a.max_new_tokens, Sampler(a.temperature, a.top_k, a.top_p, a.seed + i)) for i, p in enumerate(prompts)]
    for p, out in zip(prompts, Engine(model).generate(reqs)):
        print(json.dumps({"prompt": p, "tokens": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
