"""``redline_generate``: token ids in, one JSON line per request out
(reference: apps/redline_generate.cpp)."""

from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional

from .cli_common import add_engine_options, engine_options, parse_id_list, resolve_model


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="redline_generate", description=__doc__)
    add_engine_options(ap)
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS", help="comma-separated ids; repeatable")
    ap.add_argument("--prompts-json", help="file with a JSON list of id lists")
    ap.add_argument("--score-ids", help="print log p(ids[i] | ids[:i]) instead of generating")
    ap.add_argument("--max-new-tokens", type=int, default=128)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0, help="request i samples with seed + i")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--stop-token-ids", default="", help="comma-separated extra stop ids")
    args = ap.parse_args(argv)
    try:
        prompts = [parse_id_list(s) for s in args.prompt_ids]
        if args.prompts_json:
            with open(args.prompts_json) as f:
                prompts += [[int(t) for t in p] for p in json.load(f)]
        model = resolve_model(args)
        from ..engine.engine import Engine
        # a command-line run does not need the whole GPU
        engine = Engine(model, **engine_options(args, default_utilization=0.5))
        if args.score_ids:
            print(json.dumps({"logprobs": engine.score(parse_id_list(args.score_ids))}))
            return 0
        if not prompts:
            raise ValueError("no prompts given (--prompt-ids or --prompts-json)")
        outs = engine.generate(prompts, args.max_new_tokens, args.temperature, args.top_k, args.top_p,
                               args.seed, args.ignore_eos, parse_id_list(args.stop_token_ids))
        for o in outs:
            print(json.dumps({"id": o["id"], "output_ids": o["output_ids"], "logprobs": o["logprobs"],
                              "finish_reason": o["finish_reason"], "ttft_ms": o["ttft_s"] * 1e3,
                              "e2e_ms": o["e2e_s"] * 1e3}))
    except Exception as e:  # noqa: BLE001 - a command-line program reports and exits 1
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0
