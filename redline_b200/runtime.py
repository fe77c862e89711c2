"""Python entry point in the reference's manner (python/redline/runtime.py:43-145):

    from redline_b200.runtime import Engine
    engine = Engine("model_dir", max_seqs=8, kv_cache_tokens=4096)
    outs = engine.generate([[1, 2, 3]], max_new_tokens=32, temperature=0.8, seed=1)

Options carry the names of the command-line flags: ``max_seqs``, ``max_batched_tokens``,
``max_seq_len``, ``max_logit_rows``, ``block_size``, ``kv_cache_tokens``,
``gpu_memory_utilization``, ``cuda_graphs``, ``async_scheduling``, ``mix_prefill_decode``,
``device``, plus ``dtype``.  ``CliEngine`` runs ``bin/redline_generate`` in a
subprocess with the same interface; ``load_engine`` returns the in-process engine.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from typing import Any, Dict, List, Sequence

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Engine:
    """In-process engine."""

    def __init__(self, model: str, **options: Any):
        from .engine.engine import Engine as _Engine
        self._engine = _Engine(model, **{k: v for k, v in options.items() if v is not None})

    @property
    def vocab_size(self) -> int:
        return self._engine.vocab_size

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 0, ignore_eos: bool = False,
                 stop_token_ids: Sequence[int] = ()) -> List[Dict[str, Any]]:
        """One dict per prompt: id, prompt_ids, output_ids, logprobs, finish_reason, ttft_s,
        e2e_s, token_times.  Request i samples with seed + i."""
        return self._engine.generate([list(p) for p in prompts], max_new_tokens, temperature, top_k, top_p,
                                     seed, ignore_eos, list(stop_token_ids))

    def score(self, tokens: Sequence[int]) -> List[float]:
        """log p(tokens[i] | tokens[:i]) for i = 1 .. len(tokens) - 1."""
        return self._engine.score(list(tokens))

    def benchmark(self, workload: Dict[str, Any], online: bool = False, warmup: int = 2) -> Dict[str, Any]:
        from .apps.harness import BenchOptions, parse_workload, run_benchmark
        return run_benchmark(self._engine, parse_workload(workload, self.vocab_size),
                             BenchOptions(online=online, warmup_requests=warmup))

    def memory_report(self) -> Dict[str, Any]:
        return self._engine.memory_report()

    def describe(self) -> Dict[str, Any]:
        return self._engine.describe()


class CliEngine:
    """Subprocess fallback around ``bin/redline_generate`` (one engine per call)."""

    NEGATED = {"cuda_graphs": "--no-cuda-graphs", "async_scheduling": "--no-async",
               "mix_prefill_decode": "--no-mixed-batches"}

    def __init__(self, model: str, **options: Any):
        self.model = model
        self.flags: List[str] = []
        for k, v in options.items():
            if v is None:
                continue
            if k in self.NEGATED:
                if v is False:
                    self.flags.append(self.NEGATED[k])
                continue
            flag = "--" + k.replace("_", "-")
            if isinstance(v, bool):
                if v:
                    self.flags.append(flag)
                continue
            self.flags += [flag, str(v)]
        self.binary = os.path.join(ROOT, "bin", "redline_generate")

    def _run(self, extra: List[str]) -> List[Dict[str, Any]]:
        out = subprocess.run([sys.executable, self.binary, "--model", self.model, *self.flags, *extra],
                             check=True, capture_output=True, text=True)
        return [json.loads(line) for line in out.stdout.splitlines() if line.strip().startswith("{")]

    def generate(self, prompts, max_new_tokens=128, temperature=0.0, top_k=0, top_p=1.0, seed=0,
                 ignore_eos=False, stop_token_ids=()) -> List[Dict[str, Any]]:
        with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
            json.dump([list(p) for p in prompts], f)
            path = f.name
        try:
            args = ["--prompts-json", path, "--max-new-tokens", str(max_new_tokens), "--temperature",
                    str(temperature), "--top-k", str(top_k), "--top-p", str(top_p), "--seed", str(seed)]
            if ignore_eos:
                args.append("--ignore-eos")
            if stop_token_ids:
                args += ["--stop-token-ids", ",".join(map(str, stop_token_ids))]
            return self._run(args)
        finally:
            os.unlink(path)

    def score(self, tokens: Sequence[int]) -> List[float]:
        return self._run(["--score-ids", ",".join(map(str, tokens))])[0]["logprobs"]


def load_engine(model: str, **options: Any) -> Engine:
    return Engine(model, **options)
