"""Pre-norm residual block: h += mixer(norm(h)); h += ffn(norm(h)), the residual
stream h in float32 (reference: src/cuda/model/llama.cpp:116-139).  A layer without a
feed-forward stops after the first half."""

from __future__ import annotations

from .base import Block, op_mark, register


@register("block", "prenorm")
class PreNormBlock(Block):
    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _fused(ctx, hand, norm, next_norm, call):
        """Runs a part's fused form with the hand-over fields of the context set for it; returns
        (taken, what the part left for ``next_norm``)."""
        ctx.hand_in = hand if (hand is not None and hand.norm is norm) else None
        ctx.next_norm, ctx.hand_out = next_norm, None
        try:
            taken = call()
            left = ctx.hand_out if taken else None
        finally:
            ctx.hand_in = ctx.hand_out = ctx.next_norm = None
        return taken, (left if (left is not None and left.norm is next_norm) else None)

    def forward(self, residual, pending, ctx, cache, state):
        rt = self.rt
        T = ctx.T
        x = None
        hand, ctx.block_hand = ctx.block_hand, None       # from the block before, for this block's first norm
        # small batches: the mixer and the feed-forward may fuse the norm into their first
        # kernel and the residual add into their last (nothing is then left pending)
        taken = False
        if pending is None:
            taken, hand = self._fused(ctx, hand, self.mixer_norm,
                                      self.ffn_norm if self.ffn is not None else ctx.block_next_norm,
                                      lambda: self.mixer.forward_into(residual, self.mixer_norm, ctx, cache, state))
        if taken:
            a = None
        else:
            hand = None
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
            self.mixer_norm.add_norm(residual, pending, x, rows=T)
            op_mark(ctx, "add+rmsnorm", nbytes=self._norm_bytes(residual, pending, x))
            a = self.mixer.forward(x, ctx, cache, state)
        if self.ffn is None:               # a layer with a mixer only: its output is what is left to add
            ctx.block_hand = hand if a is None else None
            return a
        if a is None:
            taken, hand = self._fused(ctx, hand, self.ffn_norm, ctx.block_next_norm,
                                      lambda: self.ffn.forward_into(residual, self.ffn_norm, ctx))
            if taken:
                ctx.block_hand = hand
                return None
        if x is None:
            x = rt.workspace.get("block.normed", (rt.max_tokens, residual.shape[1]), rt.dtype)[:T]
        self.ffn_norm.add_norm(residual, a, x, rows=T)
        op_mark(ctx, "add+rmsnorm", nbytes=self._norm_bytes(residual, a, x))
        return self.ffn.forward(x, ctx)

    @staticmethod
    def _norm_bytes(residual, delta, out) -> float:
        """The stream read (and written back when something is added), the addend read, the normed rows written."""
        n = residual.numel() * residual.element_size() * (2 if delta is not None else 1)
        n += out.numel() * out.element_size()
        if delta is not None:
            n += delta.numel() * delta.element_size()
        return float(n)
