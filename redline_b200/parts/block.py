"""Pre-norm residual block: h += mixer(norm(h)); h += ffn(norm(h)), the residual
stream h in float32 (reference: src/cuda/model/llama.cpp:116-139)."""

from __future__ import annotations

from .base import Block, register


@register("block", "prenorm")
class PreNormBlock(Block):
    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        self.mixer_norm.add_norm(residual, pending, x, rows=T)
        a = self.mixer.forward(x, ctx, cache, state)
        self.ffn_norm.add_norm(residual, a, x, rows=T)
        return self.ffn.forward(x, ctx)
