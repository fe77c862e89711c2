"""Pre-norm residual block: h += mixer(norm(h)); h += ffn(norm(h)), the residual
stream h in float32 (reference: src/cuda/model/llama.cpp:116-139)."""

from __future__ import annotations

from .base import Block, register


@register("block", "prenorm")
class PreNormBlock(Block):
    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        x = None
        # small batches: the mixer and the feed-forward may fuse the norm into their first
        # kernel and the residual add into their last (nothing is then left pending)
        if pending is None and self.mixer.forward_into(residual, self.mixer_norm, ctx, cache, state):
            a = None
        else:
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
            self.mixer_norm.add_norm(residual, pending, x, rows=T)
            a = self.mixer.forward(x, ctx, cache, state)
        if a is None and self.ffn.forward_into(residual, self.ffn_norm, ctx):
            return None
        if x is None:
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        self.ffn_norm.add_norm(residual, a, x, rows=T)
        return self.ffn.forward(x, ctx)
