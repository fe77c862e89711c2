"""The session behind ``bin/trace_run``: an ``Engine`` sized for the trace, driven
through ``Engine.step_tokens`` (no scheduler, no sampler)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np

MAX_LIVE_REQUESTS = 8          # the trace format allows up to four live requests
MAX_STEP_TOKENS = 8192         # larger steps are run as several batches
MAX_LOGITS_BYTES = 1 << 30


class ReplaySession:
    def __init__(self, model: str, dtype: str, max_tokens: int, block_size: int = 16):
        from ..config.registry import load_config
        from ..engine.engine import Engine

        if max_tokens <= 0:
            raise ValueError("--max-tokens must be positive")
        config = load_config(model)
        pool = (max_tokens + 63) // 64 * 64
        rows = max(64, min(MAX_STEP_TOKENS, MAX_LOGITS_BYTES // (4 * config.vocab_size)))
        self.engine = Engine(
            model, dtype=dtype, kv_cache_tokens=pool, max_seq_len=max(pool, 64),
            max_num_seqs=MAX_LIVE_REQUESTS, max_num_batched_tokens=max(min(pool, MAX_STEP_TOKENS), 64),
            max_logit_rows=rows, block_size=block_size, cuda_graphs=False, async_scheduling=False)

    def run_step(self, entries: Sequence[Dict[str, Any]], end: Sequence[Any]) -> Optional[np.ndarray]:
        """Runs one step; returns the float32 logits [wanted, vocab] or None if nothing was wanted."""
        batch = [(e["id"], e.get("tokens", []), e.get("want", [])) for e in entries]
        wanted = sum(len(w) for _, _, w in batch)
        out = None
        if any(len(t) for _, t, _ in batch):
            logits = self.engine.step_tokens(batch)
            if wanted:
                out = logits.cpu().numpy().astype("<f4", copy=False)
        self.engine.runner.check_status()
        for key in end:
            if self.engine.runner.cache.is_open(key):
                self.engine.close_request(key)
        return out
