"""``redline_bench``: runs workloads and writes a JSON report per workload
(reference: apps/redline_bench.cpp:31-98)."""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

from .cli_common import add_engine_options, engine_options, parse_id_list, resolve_model


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="redline_bench", description=__doc__)
    add_engine_options(ap)
    ap.add_argument("--workload", action="append", default=[], metavar="FILE")
    ap.add_argument("--synthetic", action="append", default=[], metavar="N,IN,OUT")
    ap.add_argument("--out", help="report file")
    ap.add_argument("--out-dir", help="report folder (one file per workload)")
    ap.add_argument("--online", action="store_true", help="honour workload arrival times")
    ap.add_argument("--warmup", type=int, default=2, help="warm-up requests")
    ap.add_argument("--per-request", action="store_true", help="include per-request metrics")
    ap.add_argument("--trace-out", help="step-by-step trace file")
    ap.add_argument("--profile-ops", action="store_true",
                    help="per-op GPU time breakdown with roofline fractions (runs eagerly; skews throughput)")
    ap.add_argument("--tag", default="redline_b200", help="label stored in the report")
    args = ap.parse_args(argv)
    try:
        if not args.workload and not args.synthetic:
            raise ValueError("give --workload or --synthetic")
        from ..engine.engine import Engine
        from .harness import (BenchOptions, format_report_summary, load_workload, run_benchmark,
                              synthetic_workload)
        engine = Engine(resolve_model(args), **engine_options(args))
        workloads = [(os.path.splitext(os.path.basename(f))[0], load_workload(f, engine.vocab_size))
                     for f in args.workload]
        for s in args.synthetic:
            v = parse_id_list(s)
            if len(v) != 3:
                raise ValueError("--synthetic expects N,IN,OUT")
            w = synthetic_workload(v[0], v[1], v[2], engine.vocab_size)
            workloads.append((w.name, w))
        peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                             "MEASURED_PEAKS.json")
        hbm = tflops = 0.0
        if os.path.exists(peaks):
            with open(peaks) as f:
                pk = json.load(f)
            hbm, tflops = float(pk.get("hbm_gbs", 0.0)), float(pk.get("bf16_tflops", 0.0))
        if args.out_dir:
            os.makedirs(args.out_dir, exist_ok=True)
        reports = []
        for name, w in workloads:
            opts = BenchOptions(online=args.online, warmup_requests=args.warmup, keep_per_request=args.per_request,
                                hbm_gbs=hbm, bf16_tflops=tflops, profile_ops=args.profile_ops)
            if args.trace_out:
                opts.trace_path = args.trace_out if len(workloads) == 1 else \
                    args.trace_out.replace(".json", "") + f"__{name}.json"
            rep = run_benchmark(engine, w, opts)
            rep["tag"], rep["system"] = args.tag, "redline_b200"
            print(format_report_summary(rep), file=sys.stderr)
            if args.profile_ops:
                from ..engine.profiler import format_op_profile
                print(format_op_profile(rep["op_profile"]), file=sys.stderr, end="")
            if args.out_dir:
                with open(os.path.join(args.out_dir, f"{args.tag}__{name}.json"), "w") as f:
                    json.dump(rep, f, indent=1)
            reports.append(rep)
        if args.out:
            with open(args.out, "w") as f:
                json.dump(reports[0] if len(reports) == 1 else reports, f, indent=1)
    except Exception as e:  # noqa: BLE001 - a command-line program reports and exits 1
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0
