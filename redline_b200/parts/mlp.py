"""SiLU-gated feed-forward: down(silu(gate(x)) * up(x)), gate and up fused into one
projection [gate | up] (reference: src/cuda/model/llama.cpp:134-136,
src/cuda/kernels/elementwise.cu:66-82)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..ops import kernels
from ..ops.linear import linear
from .base import FeedForward, norm_handover, op_mark, register
from .spec import TensorSpec


# From this many rows on the fused tcgen05 kernel beats the library product followed by the
# activation kernel (measured at 512 and 2048 rows; at 64 rows the library product is ahead).
TC_MIN_ROWS = 128


@dataclass(frozen=True)
class GatedMLPParams:
    hidden_size: int
    intermediate_size: int
    bias: bool = False


@register("ffn", "swiglu_mlp")
class SwiGLUMLP(FeedForward):
    def tensors(self) -> Dict[str, TensorSpec]:
        p = self.params
        return {
            "gate": TensorSpec((p.intermediate_size, p.hidden_size)),
            "up": TensorSpec((p.intermediate_size, p.hidden_size)),
            "down": TensorSpec((p.hidden_size, p.intermediate_size)),
            "gate_bias": TensorSpec((p.intermediate_size,), optional=not p.bias),
            "up_bias": TensorSpec((p.intermediate_size,), optional=not p.bias),
            "down_bias": TensorSpec((p.hidden_size,), optional=not p.bias),
        }

    def fused(self) -> Dict[str, list]:
        return {"gate_up": ["gate", "up"]}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if "gate_up" in tensors:                   # the loader has laid gate and up one after another
            self.w_gate_up = tensors["gate_up"]
        else:
            g, u = tensors["gate"], tensors["up"]
            dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
            self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = tensors["down"]
        self.b_gate_up = None
        if "gate_bias" in tensors and "up_bias" in tensors:
            self.b_gate_up = torch.cat([tensors["gate_bias"].float(), tensors["up_bias"].float()]).contiguous()
        self.b_down = tensors.get("down_bias")

    def nbytes(self) -> int:
        return (self.w_gate_up.numel() * self.w_gate_up.element_size()
                + self.w_down.numel() * self.w_down.element_size())

    def forward(self, x, ctx) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        ws = rt.workspace
        act = ws.get("ffn.act", (rt.max_tokens, p.intermediate_size), rt.dtype)[:T]
        if T >= TC_MIN_ROWS and self.b_gate_up is None and kernels.gemm_tc_ok(x, self.w_gate_up):
            # prompt portions: gate/up product and the gated activation in one tcgen05 kernel
            kernels.gemm_tc(x, self.w_gate_up, act, kernels.EPI_SWIGLU)
        else:
            gu = ws.get("ffn.gate_up", (rt.max_tokens, 2 * p.intermediate_size), rt.dtype)[:T]
            linear(x, self.w_gate_up, gu)
            if self.b_gate_up is not None:
                kernels.add_bias(gu, self.b_gate_up)
            kernels.swiglu(gu, act)
        op_mark(ctx, "gate_up+swiglu", self.w_gate_up, T)
        out = ws.get("ffn.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(act, self.w_down, out)
        if self.b_down is not None:
            kernels.add_bias(out, self.b_down)
        op_mark(ctx, "down_proj", self.w_down, T)
        return out

    def forward_into(self, residual, norm, ctx) -> bool:
        rt = self.rt
        T = ctx.T
        rms = norm.rms_params()
        if rms is None or self.b_gate_up is not None or self.b_down is not None or rt.dtype != torch.bfloat16:
            return False
        if kernels.skinny_ok(T, self.w_gate_up, rt.dtype) and kernels.skinny_ok(T, self.w_down, rt.dtype):
            return self._into_skinny(residual, rms, ctx)
        if kernels.mid_rows(T, self.w_gate_up, self.w_down):
            return self._into_mid(residual, rms, ctx)
        return False

    def _into_skinny(self, residual, rms, ctx) -> bool:
        """At most 16 rows: products that stream the weights through CUDA cores."""
        p, rt = self.params, self.rt
        T = ctx.T
        act = rt.workspace.get("ffn.act", (rt.max_tokens, p.intermediate_size), rt.dtype)[:T]
        small = T <= kernels.SKINNY_UNSTAGED_ROWS
        hand = ctx.hand_in if small else None
        if hand is not None:
            # the part before left the norm half done: its xw, and the row scales in this product
            kernels.gemm_skinny(self.w_gate_up, act, kernels.EPI_SWIGLU, T, x=hand.xw[:T], hand_in=hand.sums,
                                eps=rms[1])
        elif small:
            # up to 8 rows: the product takes bfloat16 activations straight from global memory (no staging,
            # no barriers in its k loop), which is worth a norm kernel of its own (measured: 2 % of the step)
            xn = rt.workspace.get("ffn.xn", (kernels.SKINNY_UNSTAGED_ROWS, p.hidden_size), rt.dtype)[:T]
            kernels.add_rmsnorm(residual, None, rms[0], xn, rms[1], rows=T)
            kernels.gemm_skinny(self.w_gate_up, act, kernels.EPI_SWIGLU, T, x=xn)
        else:
            kernels.gemm_skinny(self.w_gate_up, act, kernels.EPI_SWIGLU, T, residual=residual, norm_w=rms[0],
                                eps=rms[1])
        op_mark(ctx, "norm+gate_up+swiglu", self.w_gate_up, T)
        out = norm_handover(self, "ffn", ctx, residual.shape[1], kernels.SKINNY_UNSTAGED_ROWS) if small else None
        kernels.gemm_skinny(self.w_down, residual, kernels.EPI_ADD_RESIDUAL, T, x=act,
                            hand_out=None if out is None else (out.norm.rms_params()[0], out.xw, out.sums))
        op_mark(ctx, "down_proj+add", self.w_down, T)
        ctx.hand_out = out
        return True

    def _into_mid(self, residual, rms, ctx) -> bool:
        """17 to 64 rows: tcgen05 products with the weights as the wide operand; the gated activation in
        the first one's epilogue, the add to the stream in the second one's, the norms handed over."""
        p, rt = self.params, self.rt
        T = ctx.T
        act = rt.workspace.get("ffn.act", (rt.max_tokens, p.intermediate_size), rt.dtype)[:T]
        hand = ctx.hand_in
        if hand is not None and hand.xw.shape[0] >= T:
            kernels.gemm_mid(hand.xw[:T], self.w_gate_up, act, kernels.EPI_SWIGLU, hand_in=hand.sums, eps=rms[1])
        else:
            xn = rt.workspace.get("ffn.xn_mid", (kernels.MID_MAX_ROWS, p.hidden_size), rt.dtype)[:T]
            kernels.add_rmsnorm(residual, None, rms[0], xn, rms[1], rows=T)
            kernels.gemm_mid(xn, self.w_gate_up, act, kernels.EPI_SWIGLU)
        op_mark(ctx, "norm+gate_up+swiglu", self.w_gate_up, T)
        out = norm_handover(self, "ffn.mid", ctx, residual.shape[1], kernels.MID_MAX_ROWS, tile=128)
        kernels.gemm_mid(act, self.w_down, None, kernels.EPI_ADD_RESIDUAL, residual=residual,
                         hand_out=None if out is None else (out.norm.rms_params()[0], out.xw, out.sums))
        op_mark(ctx, "down_proj+add", self.w_down, T)
        ctx.hand_out = out
        return True
