"""Python entry point in the reference's manner (python/redline/runtime.py:43-145):

    from redline_b200.runtime import Engine
    engine = Engine("model_dir", max_seqs=8, kv_cache_tokens=4096)
    outs = engine.generate([[1, 2, 3]], max_new_tokens=32, temperature=0.8, seed=1)

Options carry the names of the command-line flags: ``max_seqs``, ``max_batched_tokens``,
``max_seq_len``, ``max_logit_rows``, ``block_size``, ``kv_cache_tokens``,
``gpu_memory_utilization``, ``cuda_graphs``, ``async_scheduling``, ``mix_prefill_decode``,
``device``, plus ``dtype``.  The reference also has a subprocess engine around its
compiled programs for installs without the extension module; this package is
importable wherever its programs run, so ``load_engine`` always returns the in-process engine.
"""

from __future__ import annotations

from typing import Any, Dict, List, Sequence


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


def load_engine(model: str, **options: Any) -> Engine:
    """The engine for a model folder (reference: python/redline/runtime.py:143-145, which
    chooses between its extension module and its subprocess engine; here there is one)."""
    return Engine(model, **options)
