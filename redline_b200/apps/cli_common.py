"""Options shared by the command-line programs, with the reference's flag names
(apps/cli_common.cpp:68-118), minus quantisation and speculation, plus --dtype and
the random-weights mode (--random-weights CONFIG.json --seed S writes a model folder
and runs from it)."""

from __future__ import annotations

import argparse
import json
import os
import tempfile
from typing import Any, Dict, List


def add_engine_options(ap: argparse.ArgumentParser) -> None:
    g = ap.add_argument_group("engine options")
    g.add_argument("--model", help="model folder (config.json, model.safetensors)")
    g.add_argument("--random-weights", metavar="CONFIG", help="config.json to draw random weights for "
                   "(written as a model folder under --model, or a temporary folder)")
    g.add_argument("--weights-seed", type=int, default=0, help="seed of --random-weights")
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--max-seqs", type=int, default=32, help="max concurrent sequences (default 32)")
    g.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget per step / prefill chunk")
    g.add_argument("--max-seq-len", type=int, default=4096, help="max prompt + output length")
    g.add_argument("--max-logit-rows", type=int, default=0)
    g.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    g.add_argument("--kv-cache-tokens", type=int, default=0, help="cache capacity in tokens (default: from memory)")
    g.add_argument("--gpu-memory-utilization", type=float, default=None, help="device memory fraction to use")
    g.add_argument("--no-cuda-graphs", action="store_true", help="disable CUDA graph replay for decode")
    g.add_argument("--no-async", action="store_true", help="disable asynchronous (pipelined) scheduling")
    g.add_argument("--no-mixed-batches", action="store_true", help="do not mix prefill chunks with decode tokens")
    g.add_argument("--nvtx-layers", action="store_true", help="emit one NVTX range per step and per layer call")
    g.add_argument("--track-memory", action="store_true", help="sample device memory every step (peak in the report)")
    g.add_argument("--device", type=int, default=0, help="CUDA device")


def engine_options(args: argparse.Namespace, default_utilization: float = 0.9) -> Dict[str, Any]:
    util = args.gpu_memory_utilization if args.gpu_memory_utilization is not None else default_utilization
    return dict(
        dtype=args.dtype, max_seqs=args.max_seqs, max_batched_tokens=args.max_batched_tokens,
        max_seq_len=args.max_seq_len, max_logit_rows=args.max_logit_rows, block_size=args.block_size,
        kv_cache_tokens=args.kv_cache_tokens, gpu_memory_utilization=util,
        cuda_graphs=not args.no_cuda_graphs, async_scheduling=not args.no_async,
        mix_prefill_decode=not args.no_mixed_batches, nvtx_layers=args.nvtx_layers,
        track_memory=args.track_memory, device=args.device)


def resolve_model(args: argparse.Namespace) -> str:
    """The model folder to run from; draws random weights into it first when asked."""
    if args.random_weights:
        from ..config.registry import config_from_dict
        from ..weights.random_init import write_random_model
        with open(args.random_weights) as f:
            config = config_from_dict(json.load(f))
        target = args.model or tempfile.mkdtemp(prefix="redline_random_")
        write_random_model(target, config, seed=args.weights_seed)
        return target
    if not args.model:
        raise SystemExit("error: --model is required (or --random-weights CONFIG)")
    return args.model


def parse_id_list(s: str) -> List[int]:
    return [int(t) for t in s.split(",") if t.strip()]
