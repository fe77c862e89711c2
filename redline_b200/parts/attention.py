"""Grouped-query causal attention over the paged cache.

q, k, v come from one fused projection [q | k | v]; q and k are rotated by the
position encoding in the kernel that writes k and v into the cache; sequences that
bring one token go to the split-K decode kernel, longer portions to the tiled
prefill kernel; then the output projection.  Query head h reads kv head h // G, the
scale is 1 / sqrt(head_dim) unless given, a window w > 0 keeps only the last w keys
(reference: src/cuda/model/llama.cpp:116-131, src/cuda/kernels/attention.cu).
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import LayerCache, Mixer, build_part, norm_handover, op_mark, register
from .spec import CacheSpec, PartSpec, TensorSpec


@dataclass(frozen=True)
class AttentionParams:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: PartSpec
    bias: bool = False          # q, k, v projections have biases
    out_bias: bool = False
    window: int = 0             # 0: every earlier key
    scale: Optional[float] = None


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        if p.num_heads % p.num_kv_heads != 0:
            raise ValueError(f"num_heads {p.num_heads} is no multiple of num_kv_heads {p.num_kv_heads}")
        if p.head_dim % 16 != 0 or not 16 <= p.head_dim <= kernels.MAX_HEAD_DIM:
            raise ValueError(f"attention kernels take head sizes that are multiples of 16 up to "
                             f"{kernels.MAX_HEAD_DIM}; got head_dim={p.head_dim}")
        self.position = build_part("position", p.position, rt)
        self.scale = p.scale if p.scale is not None else 1.0 / math.sqrt(p.head_dim)
        self.q_size = p.num_heads * p.head_dim
        self.kv_size = p.num_kv_heads * p.head_dim
        self.qkv_size = self.q_size + 2 * self.kv_size

    def cache_spec(self) -> CacheSpec:
        p = self.params
        return CacheSpec.keys_values("window" if p.window > 0 else "full", p.num_kv_heads, p.head_dim, p.window)

    def tiling(self):
        return kernels.PREFILL_TILE_ROWS, kernels.DECODE_PARTITION

    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        t = {
            "q": TensorSpec((self.q_size, p.hidden_size)),
            "k": TensorSpec((self.kv_size, p.hidden_size)),
            "v": TensorSpec((self.kv_size, p.hidden_size)),
            "o": TensorSpec((p.hidden_size, self.q_size)),
            "q_bias": TensorSpec((self.q_size,), optional=not p.bias),
            "k_bias": TensorSpec((self.kv_size,), optional=not p.bias),
            "v_bias": TensorSpec((self.kv_size,), optional=not p.bias),
            "o_bias": TensorSpec((p.hidden_size,), optional=not p.out_bias),
        }
        return t

    def fused(self) -> Dict[str, list]:
        return {"qkv": ["q", "k", "v"]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if "qkv" in tensors:                       # the loader has laid q, k and v one after another
            self.w_qkv = tensors["qkv"]
        else:
            q, k, v = tensors["q"], tensors["k"], tensors["v"]
            dt = torch.float32 if torch.float32 in (q.dtype, k.dtype, v.dtype) else q.dtype
            self.w_qkv = torch.cat([q.to(dt), k.to(dt), v.to(dt)], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.b_qkv = None
        if all(n in tensors for n in ("q_bias", "k_bias", "v_bias")):
            self.b_qkv = torch.cat([tensors[n].float() for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
        elif any(n in tensors for n in ("q_bias", "k_bias", "v_bias")):
            raise ValueError("attention: q, k and v biases must come together")
        self.b_o = tensors.get("o_bias")

    def nbytes(self) -> int:
        n = self.w_qkv.numel() * self.w_qkv.element_size() + self.w_o.numel() * self.w_o.element_size()
        return n + self.position.nbytes()

    def forward(self, x, ctx, cache: Optional[LayerCache], state=None) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        qkv = rt.workspace.get("attn.qkv", (rt.max_tokens, self.qkv_size), rt.dtype)[:T]
        linear(x, self.w_qkv, qkv)
        op_mark(ctx, "qkv_proj", self.w_qkv, T)
        attn = self._attend(qkv, ctx, cache)
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(attn, self.w_o, out)
        if self.b_o is not None:
            kernels.add_bias(out, self.b_o)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out

    def forward_into(self, residual, norm, ctx, cache: Optional[LayerCache], state=None) -> bool:
        rt = self.rt
        T = ctx.T
        rms = norm.rms_params()
        if rms is None or self.b_o is not None or rt.dtype != torch.bfloat16:
            return False
        if kernels.skinny_ok(T, self.w_qkv, rt.dtype) and kernels.skinny_ok(T, self.w_o, rt.dtype):
            return self._into_skinny(residual, rms, ctx, cache)
        if kernels.mid_rows(T, self.w_qkv, self.w_o):
            return self._into_mid(residual, rms, ctx, cache)
        return False

    def _into_skinny(self, residual, rms, ctx, cache) -> bool:
        """At most 16 rows: products that stream the weights through CUDA cores."""
        rt = self.rt
        T = ctx.T
        qkv = rt.workspace.get("attn.qkv", (rt.max_tokens, self.qkv_size), rt.dtype)[:T]
        small = T <= kernels.SKINNY_UNSTAGED_ROWS
        hand = ctx.hand_in if small else None
        if hand is not None:
            # the part before left the norm half done: its xw, and the row scales in this product
            kernels.gemm_skinny(self.w_qkv, qkv, kernels.EPI_BF16, T, x=hand.xw[:T], hand_in=hand.sums, eps=rms[1])
        elif small:
            # (see SwiGLUMLP.forward_into: a norm kernel of its own and a product without staging)
            xn = rt.workspace.get("attn.xn", (kernels.SKINNY_UNSTAGED_ROWS, self.params.hidden_size), rt.dtype)[:T]
            kernels.add_rmsnorm(residual, None, rms[0], xn, rms[1], rows=T)
            kernels.gemm_skinny(self.w_qkv, qkv, kernels.EPI_BF16, T, x=xn)
        else:
            kernels.gemm_skinny(self.w_qkv, qkv, kernels.EPI_BF16, T, residual=residual, norm_w=rms[0], eps=rms[1])
        op_mark(ctx, "norm+qkv_proj", self.w_qkv, T)
        attn = self._attend(qkv, ctx, cache)
        out = norm_handover(self, "attn", ctx, residual.shape[1], kernels.SKINNY_UNSTAGED_ROWS) if small else None
        kernels.gemm_skinny(self.w_o, residual, kernels.EPI_ADD_RESIDUAL, T, x=attn,
                            hand_out=None if out is None else (out.norm.rms_params()[0], out.xw, out.sums))
        op_mark(ctx, "o_proj+add", self.w_o, T)
        ctx.hand_out = out
        return True

    def _into_mid(self, residual, rms, ctx, cache) -> bool:
        """17 to 64 rows: tcgen05 products with the weights as the wide operand; the add to the stream
        in the second one's epilogue, the norms handed from product to product."""
        rt = self.rt
        T = ctx.T
        qkv = rt.workspace.get("attn.qkv", (rt.max_tokens, self.qkv_size), rt.dtype)[:T]
        hand = ctx.hand_in
        if hand is not None and hand.xw.shape[0] >= T:
            kernels.gemm_mid(hand.xw[:T], self.w_qkv, qkv, kernels.EPI_BF16, hand_in=hand.sums, eps=rms[1])
        else:
            xn = rt.workspace.get("attn.xn_mid", (kernels.MID_MAX_ROWS, self.params.hidden_size), rt.dtype)[:T]
            kernels.add_rmsnorm(residual, None, rms[0], xn, rms[1], rows=T)
            kernels.gemm_mid(xn, self.w_qkv, qkv, kernels.EPI_BF16)
        op_mark(ctx, "norm+qkv_proj", self.w_qkv, T)
        attn = self._attend(qkv, ctx, cache)
        out = norm_handover(self, "attn.mid", ctx, residual.shape[1], kernels.MID_MAX_ROWS, tile=128)
        kernels.gemm_mid(attn, self.w_o, None, kernels.EPI_ADD_RESIDUAL, residual=residual,
                         hand_out=None if out is None else (out.norm.rms_params()[0], out.xw, out.sums))
        op_mark(ctx, "o_proj+add", self.w_o, T)
        ctx.hand_out = out
        return True

    def decode_variant(self, ctx) -> int:
        """4 where the decode kernel of one cluster per (sequence, kv head) is expected to be the fastest (few
        sequences of similar length), else 0 (the kernels choose among themselves)."""
        p, rt = self.params, self.rt
        if rt.dtype != torch.bfloat16 or ctx.num_decode <= 0 or os.environ.get("REDLINE_DECODE_ROWS", "1") == "0":
            return 0
        # (the layers of a model mostly ask the same question: the step's context keeps the answers)
        memo = ctx.__dict__.setdefault("_decode_variants", {})
        key = (p.num_kv_heads, p.head_dim, p.window)
        if key not in memo:
            memo[key] = 4 if kernels.attn_decode_rows_pays(ctx.num_decode, p.num_kv_heads, p.head_dim,
                                                           ctx.decode_max_ctx, ctx.decode_sum_ctx, p.window,
                                                           rt.device) else 0
        return memo[key]

    def _counters(self, max_items: int) -> torch.Tensor:
        """Arrival counters of the decode kernel's fused merge: zero between launches."""
        c = getattr(self, "_cnt", None)
        if c is None or c.numel() < max_items * self.params.num_kv_heads:
            c = torch.zeros(max_items * self.params.num_kv_heads, dtype=torch.int32, device=self.rt.device)
            self._cnt = c
        return c

    def _attend(self, qkv, ctx, cache: LayerCache) -> torch.Tensor:
        """Bias, position encoding, cache write and attention on the projected [q | k | v]."""
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        if self.b_qkv is not None:
            kernels.add_bias(qkv, self.b_qkv)
        tables = self.position.rotary_tables()
        g = ctx.groups[cache.group]
        attn = ws.get("attn.out", (rt.max_tokens, self.q_size), rt.dtype)[:T]
        part_o = part_ml = None
        variant = self.decode_variant(ctx) if ctx.num_decode > 0 else 0
        if ctx.num_decode > 0:
            part_o = ws.get("attn.part_o", (ctx.max_items * p.num_heads * ctx.parts_capacity * p.head_dim,),
                            torch.float32)
            part_ml = ws.get("attn.part_ml", (ctx.max_items * p.num_heads * ctx.parts_capacity * 2,),
                             torch.float32)
            # a step of single tokens only, on a tensor-core kernel: that kernel rotates q and k itself and
            # writes the tokens' k and v into the cache, which saves the kernel that does so otherwise
            if (tables is not None and cache.write and ctx.num_decode == T and ctx.num_tiles == 0
                    and kernels.attn_decode_rope_ok(qkv, self.qkv_size, cache.k, cache.v, part_o,
                                                    self._counters(ctx.max_items), attn, ctx.decode_parts,
                                                    ctx.num_decode, p.num_heads, p.num_kv_heads, p.head_dim,
                                                    rt.page_size, self.q_size, self.q_size + self.kv_size)):
                kernels.attn_decode_rope(qkv, self.qkv_size, cache.k, cache.v, g.block_table, ctx.decode_info,
                                         part_o, part_ml, ctx.decode_parts, self._counters(ctx.max_items), attn,
                                         ctx.num_decode, p.num_heads, p.num_kv_heads, p.head_dim, rt.page_size,
                                         p.window, self.scale, tables[0], tables[1], self.q_size,
                                         self.q_size + self.kv_size, ctx.status, impl=variant)
                self._mark_attention(ctx, "rope+kv_write+attention_decode", "decode")
                return attn
        if tables is None:
            self.position.apply(qkv, p.num_heads, p.num_kv_heads, p.head_dim, ctx)
        cos, sin = tables if tables is not None else (None, None)
        kernels.rope_kv_write(qkv, ctx.positions, g.slots if cache.write else None, cos, sin, cache.k, cache.v,
                              p.num_heads, p.num_kv_heads, p.head_dim, rt.page_size, ctx.status, tokens=T)
        if ctx.profiler is not None:
            elem = qkv.element_size()
            ctx.profiler.mark("rope+kv_write", T * (2.0 * (self.q_size + self.kv_size) + 3.0 * self.kv_size) * elem, 0.0)
        if ctx.num_decode > 0:
            kernels.attn_decode(qkv, self.qkv_size, cache.k, cache.v, g.block_table, ctx.decode_info,
                                part_o, part_ml, ctx.decode_parts, self._counters(ctx.max_items), attn,
                                ctx.num_decode, p.num_heads, p.num_kv_heads, p.head_dim, rt.page_size,
                                p.window, self.scale, impl=variant)
            self._mark_attention(ctx, "attention_decode", "decode")
        if ctx.num_tiles > 0:
            kernels.attn_prefill(qkv, self.qkv_size, cache.k, cache.v, g.block_table, ctx.tile_seq,
                                 ctx.tile_tok, ctx.tile_rows, ctx.positions, attn, ctx.num_tiles, p.num_heads,
                                 p.num_kv_heads, p.head_dim, rt.page_size, p.window, self.scale)
            self._mark_attention(ctx, "attention_prefill", "prefill")
        return attn

    def _mark_attention(self, ctx, op: str, which: str) -> None:
        if ctx.profiler is None:
            return
        from ..engine.profiler import attention_work
        p = self.params
        elem = 2 if self.rt.dtype == torch.bfloat16 else 4
        nbytes, flops = attention_work(ctx.host, p.num_heads, p.num_kv_heads, p.head_dim, p.window, elem)[which]
        ctx.profiler.mark(op, nbytes, flops)
