"""The step function: runs one batch of (request, its next tokens) from the cache
and returns float32 logits at the wanted places.

``ModelRunner`` owns the model, the cache manager with its device memory, the batch
builder and the sampler.  ``run`` takes segments cut anywhere (portions of prompts
beside single decoded tokens), runs only those tokens, and leaves their keys and
values in the cache for later steps.  The scheduler-driven engine and the trace
replay program both drive this one function (reference: Engine::launch_step and
forward_and_sample, src/cuda/engine/engine.cpp:280-295,420-483).
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager, GroupInfo, RequestCache
from ..cache.storage import CacheStorage, StateStorage, bytes_per_page
from ..config.engine_config import EngineConfig
from ..config.model_config import ModelConfig
from ..config.registry import load_config, model_spec
from ..ops import kernels
from ..parts.base import Runtime
from ..parts.spec import ModelSpec
from ..sampling.sampler import Sampler
from ..weights.safetensors_io import CheckpointReader
from .batch import BatchBuilder, Segment, StepContext
from .model import DecoderModel

GRAPH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 160, 192, 256, 384, 512)
GRAPH_MAX_ROWS = 1024          # no graph is captured for more rows than this
STATUS_MESSAGES = {1: "a token id outside the vocabulary", 2: "a position beyond the rotary table",
                   4: "a cache slot beyond the pool"}


class EngineError(RuntimeError):
    pass


def require_cuda(device_index: int) -> torch.device:
    if not torch.cuda.is_available():
        raise EngineError("redline_b200 needs a CUDA device (B200, sm_100a); there is no CPU fallback")
    return torch.device("cuda", device_index)


def pin_library_products() -> None:
    """The library's matrix products (the bfloat16 products of more than 16 rows) must keep what the
    package's own kernels promise: float32 accumulation all the way, also across the parts of a split
    k dimension (torch's default lets cuBLAS reduce those parts in bfloat16), and no TF32 anywhere."""
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


class ModelRunner:
    def __init__(self, cfg: EngineConfig, model_config: Optional[ModelConfig] = None,
                 spec: Optional[ModelSpec] = None):
        cfg.validate()
        self.cfg = cfg
        self.device = require_cuda(cfg.device)
        torch.cuda.set_device(self.device)
        pin_library_products()
        self.model_config = model_config or load_config(cfg.model)
        self.spec = spec or model_spec(self.model_config)
        self.dtype = cfg.torch_dtype
        self.max_seq_len = cfg.max_seq_len
        self.rt = Runtime(device=self.device, dtype=self.dtype, max_tokens=cfg.max_num_batched_tokens,
                          max_seqs=cfg.max_num_seqs, max_seq_len=cfg.max_seq_len, page_size=cfg.block_size)
        self.model = DecoderModel(self.spec, self.rt)
        self.model.load_weights(CheckpointReader(cfg.model))
        self.vocab_size = self.spec.vocab_size

        self.max_rows = cfg.logit_rows
        self.logits = torch.zeros((self.max_rows, self.vocab_size), dtype=torch.float32, device=self.device)
        self.sampler = Sampler(self.max_rows, self.device)

        self.groups: List[GroupInfo] = self.model.cache_groups()
        pages = self._size_cache()
        self.cache = CacheManager(self.groups, pages, cfg.block_size, num_state_slots=cfg.max_num_seqs)
        self.storage = CacheStorage(self.groups, pages, cfg.block_size, self.dtype, self.device)
        self.states = StateStorage(self.model.state_specs(), cfg.max_num_seqs, self.device)
        if self.states.pools:   # a fresh request starts from zero state
            self.cache.on_open = lambda rc: self.states.reset_slot(rc.state_slot)
        tiling = self.model.tiling()
        self.builder = BatchBuilder(self.cache, cfg.max_num_batched_tokens, cfg.max_num_seqs, self.max_rows,
                                    cfg.max_seq_len, self.device, **({} if tiling is None else
                                                                      {"tile_rows": tiling[0], "partition": tiling[1]}))
        order = self.spec.order
        self._caches = []
        for i, call in enumerate(order):
            if self.model.blocks[call.layer].mixer.cache_spec() is None:
                self._caches.append(None)
            elif call.cache_of is None:
                self._caches.append(self.storage.of_owner(i, True))
            else:
                self._caches.append(self.storage.of_owner(call.cache_of, False))
        self._states = [self.states.of_call(i) for i in range(len(order))]
        self.model.nvtx_layers = cfg.nvtx_layers
        self.profiler = None                       # engine.profiler.OpProfiler while per-op profiling is on
        # one graph per padded size and per answer of the mixers to "which kernel for the single tokens", and
        # one per shape of a full prompt portion (see _chunk_key)
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._graph_kernels: Dict[tuple, int] = {}   # kernels of this package in each graph
        self.num_kernel_launches = 0               # kernels of this package run by steps so far
        self.num_graph_steps = 0
        self.num_eager_steps = 0

    # ---------------------------------------------------------------- sizing
    def _size_cache(self) -> List[int]:
        cfg = self.cfg
        ps = cfg.block_size
        elem = torch.empty((), dtype=self.dtype).element_size()
        per_page = bytes_per_page(self.groups, ps, elem)
        need_one = (cfg.max_seq_len + ps - 1) // ps
        if cfg.kv_cache_tokens > 0:
            n = (cfg.kv_cache_tokens + ps - 1) // ps
        else:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = int(cfg.gpu_memory_utilization * total) - (total - free) - (1 << 30)
            n = max(budget, 0) // max(sum(per_page), 1)
            n = min(n, cfg.max_num_seqs * need_one)
            if n < need_one:
                raise EngineError(f"the memory budget holds {n} pages; one sequence of max_seq_len="
                                  f"{cfg.max_seq_len} needs {need_one}")
        return [n + 1 for _ in self.groups]   # + the reserved page 0

    # -------------------------------------------------------------- requests
    def open(self, key: object) -> RequestCache:
        return self.cache.open(key)

    def close(self, key: object) -> None:
        self.cache.close(key)

    # ------------------------------------------------------------------ step
    def run(self, segments: Sequence[Segment], sample: bool = False, allow_graph: bool = True
            ) -> Tuple[torch.Tensor, StepContext]:
        """Runs the segments as one batch.  Pages for every position touched must have
        been reserved.  Returns (logits[:R], ctx); with ``sample`` the sampler's
        ``tokens[:R]`` / ``logprobs[:R]`` are filled too.  A segment with ``src_row`` >= 0
        takes its token from that row of the sampler's tokens as the previous step left them."""
        profiling = self.profiler is not None          # (a graph cannot be cut into ops: profiled steps are eager)
        graphs = allow_graph and self.cfg.cuda_graphs and sample and not profiling
        bucket = self._graph_bucket(segments) if graphs else 0
        chunk = self._chunk_key(segments) if (graphs and not bucket) else None
        ctx = self.builder.build(segments, pad_to=bucket)
        if profiling:
            single = sum(1 for s in segments if len(s.tokens) == 1)
            ctx.profiler = self.profiler
            self.profiler.begin("decode" if single == len(segments) else ("prefill" if single == 0 else "mixed"))
        if bucket or chunk is not None:
            key = (bucket, self.model.decode_variants(ctx)) if bucket else chunk
            g = self._graphs.get(key)
            if g is None:
                g = self._capture(key, ctx)
            else:
                g.replay()
            self.num_graph_steps += 1
            self.num_kernel_launches += self._graph_kernels[key]
        else:
            before = kernels.LAUNCHES
            self._forward(ctx, sample, ctx.has_src)
            self.num_eager_steps += 1
            self.num_kernel_launches += kernels.LAUNCHES - before
            if profiling:
                self.profiler.end()
        return self.logits[:ctx.R], ctx

    def _forward(self, ctx: StepContext, sample: bool, resolve: bool) -> None:
        if resolve:
            kernels.resolve_ids(ctx.token_ids, ctx.token_src, self.sampler.tokens, ctx.T)
        self.model.forward(ctx, self._caches, self._states, self.logits)
        if sample and ctx.R > 0:
            self.sampler.sample(self.logits, ctx)
            if ctx.profiler is not None:
                ctx.profiler.mark("sample", ctx.R * self.vocab_size * 4.0, 0.0)

    def _graph_bucket(self, segments: Sequence[Segment]) -> int:
        """The padded size at which this step is replayed as a CUDA graph, or 0 for an eager step.
        A model whose mixers keep per-request state always steps eagerly: a graph's padding rows would
        need a state slot of their own, and capturing runs the step more than once, which a state that
        is updated in place does not survive."""
        if self.states.pools:
            return 0
        n = len(segments)
        for s in segments:
            if len(s.tokens) != 1 or len(s.want) != 1:
                return 0
        for b in GRAPH_BUCKETS:
            if n <= b <= self.cfg.max_num_seqs:
                return b
        # more sequences than the largest bucket within the limit: the limit itself is the last bucket
        return self.cfg.max_num_seqs if n <= self.cfg.max_num_seqs <= GRAPH_MAX_ROWS else 0

    def _chunk_key(self, segments: Sequence[Segment]) -> Optional[tuple]:
        """The key of the CUDA graph of a step that is ONE full portion of a prompt (as many tokens as a step
        takes, which is what every step but the last of a long prompt is, and the whole step of a prompt of
        exactly that length), or None.  Such steps all launch the same kernels with the same arguments: where
        the portion starts, its pages and the wanted row are in the step's metadata on the device."""
        if len(segments) != 1 or self.states.pools:
            return None
        s = segments[0]
        n = len(s.tokens)
        if n != self.cfg.max_num_batched_tokens or n < 128 or s.src_row >= 0 or len(s.want) > 1:
            return None
        return ("portion", n, len(s.want))

    def _capture(self, key: tuple, ctx: StepContext) -> torch.cuda.CUDAGraph:
        # The graph always resolves device-fed ids (token_src is -1 where there are none),
        # so one graph serves steps with and without them.  The step runs once eagerly
        # (compiles kernels, sizes workspaces), is captured, and the first replay runs it
        # again: every kernel of a step gives the same result when repeated.
        fed = self.sampler.tokens.clone()       # the warm-up run overwrites what the step reads
        self._forward(ctx, True, True)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        before = kernels.LAUNCHES
        with torch.cuda.graph(g):
            self._forward(ctx, True, True)
        self._graph_kernels[key] = kernels.LAUNCHES - before
        self._graphs[key] = g
        self.sampler.tokens.copy_(fed)
        g.replay()
        return g

    def check_status(self) -> None:
        """Raises if a kernel flagged bad input since the last check (synchronises)."""
        code = int(self.builder.status.item())
        tc = kernels.tc_status(self.device)
        tc_code = int(tc.item())
        if code or tc_code:
            self.builder.status.zero_()
            tc.zero_()
            what = [m for bit, m in STATUS_MESSAGES.items() if code & bit]
            if tc_code & 1:
                what.append("a wait inside the tcgen05 matrix product that ran out")
            if tc_code & 4:
                what.append("a wait inside the tcgen05 attention that ran out")
            if tc_code & 8:
                what.append("a wait inside the tcgen05 product for few rows that ran out")
            raise EngineError("a kernel met " + " and ".join(what))

    def set_op_profiling(self, on: bool) -> None:
        """Per-op device times of every step from now on (steps then run eagerly), or off."""
        from .profiler import OpProfiler
        if on and self.profiler is None:
            self.profiler = OpProfiler()
        elif not on:
            self.profiler = None

    def memory_report(self) -> Dict[str, int]:
        return {
            "weights": self.model.weight_bytes(),
            "kv_cache": self.storage.nbytes(),
            "state": self.states.nbytes(),
            "activations": self.rt.workspace.nbytes() + self.logits.numel() * 4,
            "metadata": self.builder.capacity_words * 4,
        }
