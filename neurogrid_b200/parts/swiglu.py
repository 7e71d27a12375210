"""Gated feed-forward: down( act(gate x) * up x ), act = silu (SwiGLU) or the tanh form of gelu."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("ffn", "swiglu")
class SwiGLU:
    """Reference: gpu/engine/conv_layer.cu:334-338, gpu/engine/layer.cu:1751-1761 (two GEMMs,
    SiLU, multiply, GEMM).  Gate and up weights are stacked at bind time so that one product
    feeds the gate kernel."""

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w_gate_up = self.w_down = None

    def _name(self, role):
        return self.spec.names[role] + getattr(self.spec, "weight_suffix", ".weight")

    def tensors(self):
        s = self.spec
        return {self._name("gate"): TensorDecl((s.intermediate, s.hidden)),
                self._name("up"): TensorDecl((s.intermediate, s.hidden)),
                self._name("down"): TensorDecl((s.hidden, s.intermediate))}

    def bind(self, t):
        kw = dict(device=self.device, dtype=self.dtype)
        self.w_gate_up = torch.cat([t[self._name("gate")].to(**kw), t[self._name("up")].to(**kw)]).contiguous()
        self.w_down = t[self._name("down")].to(**kw).contiguous()

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("elementwise", None)]

    def forward(self, x, ctx):
        s = self.spec
        act = ctx.ws.buf("ffn_act", x.shape[0], s.intermediate, self.dtype)
        self.gated(x, ctx, act)
        return ops.linear_to_residual(act, self.w_down, None, ctx.ws, "ffn_out", residual=ctx.residual)

    # For a block arrangement that ends mixer and feed-forward with ONE product: the gated activations go into a
    # block of columns of the caller's buffer, and the caller multiplies by ``out_weight()``.
    def inner_width(self):
        return self.spec.intermediate

    def out_weight(self):
        return self.w_down, None

    def drop_out_weight(self):
        """The caller keeps a stacked copy of the output matrix and will not call ``forward``."""
        self.w_down = None

    def gated(self, x, ctx, act):
        """act[N, intermediate] (may be a block of columns of a wider buffer) = act(gate x) * (up x)."""
        s = self.spec
        activation = getattr(s, "activation", "silu")
        if ops.gemm_sm100_ok(x, self.w_gate_up):
            ops.gemm_swiglu_sm100(x, self.w_gate_up, act, activation=activation)    # the gate rides in the epilogue
        else:
            gu = ctx.ws.buf("ffn_gate_up", x.shape[0], 2 * s.intermediate, self.dtype)
            ops.linear(x, self.w_gate_up, None, gu)
            ops.swiglu(gu, act, activation)
