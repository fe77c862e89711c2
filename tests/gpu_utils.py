"""Helpers of the GPU tests: model folders in a temporary place, engines over them,
the oracle's logits, and the error measures with the tolerances the tests use."""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

import plain_llama as P

# Tolerances (never widened to make a test pass; a failure means a fault to find).
#   float32 engine vs the double-precision oracle: the reference's own bound for its
#   exporter test, max |diff| / max |ref| < 1e-4 (tests/python/test_convert.py:77).
#   bfloat16 engine vs the oracle that rounds what a 16-bit engine stores: only the
#   order of sums differs, which flips roundings here and there: 3e-2 of max |ref|.
#   bfloat16 engine vs the unrounded oracle: the reference's bounds for its fp16 engine,
#   mean |diff| < 0.03 and max < 0.3 of log-probabilities (tests/cuda/test_engine.cpp:121).
F32_REL = 1e-4
BF16_REL_ROUNDED = 3e-2


def rel_max(a: np.ndarray, ref: np.ndarray) -> float:
    return float(np.abs(a - ref).max() / (np.abs(ref).max() + 1e-30))


def make_model(tmp, cfg_json: dict, seed: int, sharpen: float = 6.0,
               store: torch.dtype = torch.bfloat16, patch=None) -> Tuple[str, Dict[str, torch.Tensor]]:
    """Writes a model folder with the tests' seeded weights; returns (folder, weights as float32)."""
    w = P.random_weights(cfg_json, seed, sharpen)
    if patch is not None:
        patch(w)
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    d = os.path.join(str(tmp), f"model_{seed}_{abs(hash(str(cfg_json))) % 10**8}")
    P.write_model_dir(d, cfg_json, {k: v.to(store) for k, v in w.items()})
    return d, w


def oracle_logits(cfg_json: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                  rounded: Optional[torch.dtype] = None, pc: Optional[P.PlainConfig] = None) -> np.ndarray:
    pc = pc or P.plain_config(cfg_json)
    P.STORE_DTYPE = rounded
    try:
        return P.forward(pc, w, list(tokens)).numpy()
    finally:
        P.STORE_DTYPE = None


def engine_for(model_dir: str, dtype: str, **kw):
    from redline_b200.engine.engine import Engine
    opts = dict(dtype=dtype, kv_cache_tokens=512, max_seq_len=512, max_num_seqs=4,
                max_num_batched_tokens=256, max_logit_rows=256, cuda_graphs=False, async_scheduling=False)
    opts.update(kw)
    return Engine(model_dir, **opts)


def check_logits(got: np.ndarray, cfg_json: dict, w, tokens: Sequence[int], dtype: str, rows=None, pc=None):
    """Compares engine logits for ``rows`` (default: all positions) of ``tokens`` with the oracle."""
    rows = list(range(len(tokens))) if rows is None else list(rows)
    if dtype == "float32":
        ref = oracle_logits(cfg_json, w, tokens, pc=pc)[rows]
        err = rel_max(got, ref)
        assert err < F32_REL, f"float32 logits differ: rel-max {err:.3e} (first bad row " \
                              f"{rows[int(np.abs(got - ref).max(axis=1).argmax())]})"
    else:
        ref = oracle_logits(cfg_json, w, tokens, rounded=torch.bfloat16, pc=pc)[rows]
        err = rel_max(got, ref)
        assert err < BF16_REL_ROUNDED, f"bfloat16 logits differ: rel-max {err:.3e} (worst row " \
                                       f"{rows[int(np.abs(got - ref).max(axis=1).argmax())]})"
    return err


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    return np.random.RandomState(seed).randint(0, vocab, size=n).tolist()
