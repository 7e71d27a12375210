"""The input convolution of a sublayer, and the per-layer token input: the small parts of a block."""
from __future__ import annotations

import torch

from ..cache.manager import SlotNeed
from ..csrc import ops
from ..weights.decl import TensorDecl


class InputConv:
    """u -> u + conv(u): a causal convolution over time on each channel, taps [width, L] without a bias, tap
    L-1 on the current token.  State per request: its last L-1 inputs (float32; zero at admission)."""

    graph_safe = True

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.weight = None

    def tensors(self):
        return {"": TensorDecl((self.spec.hidden, self.spec.taps), "conv")}

    def bind(self, t):
        w = t[""].to(device=self.device, dtype=torch.float32)
        if self.spec.taps == 1:              # a single tap sees the current token only: the kernel's two taps, the older one zero
            w = torch.cat([torch.zeros_like(w), w], dim=1)
        self.weight = w.contiguous()

    def cache_need(self):
        return SlotNeed((max(self.spec.taps, 2) - 1, self.spec.hidden))

    def kernels(self):
        return [("input_conv", None)]

    def forward(self, u, ctx, cache, out):
        ops.input_conv(u, self.weight, cache.state, out, ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.n_entries, ctx.max_q)
        return out


class TokenSide:
    """x += rmsnorm(W_proj (gelu_tanh(W_gate x) * e)) * w, with e the layer's columns of a table indexed by the
    row's token; applied to the complete residual stream, in float32."""

    graph_safe = True

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.table = self.w_gate = self.w_proj = self.w_norm = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        return {n["gate"]: TensorDecl((s.dim, s.hidden)), n["proj"]: TensorDecl((s.hidden, s.dim)),
                n["norm"]: TensorDecl((s.hidden,), "norm")}

    def shared_tensors(self):
        s = self.spec
        return {s.table_name: TensorDecl((s.vocab_size, s.table_width))}

    def bind(self, t):
        n = self.spec.names
        f32 = dict(device=self.device, dtype=torch.float32)
        self.w_gate = t[n["gate"]].to(**f32).contiguous()
        self.w_proj = t[n["proj"]].to(**f32).t().contiguous()          # [dim, hidden]: the kernel reads both matrices along hidden
        self.w_norm = t[n["norm"]].to(**f32).contiguous()

    def bind_shared(self, weights):
        s = self.spec
        self.table = weights[s.table_name][:, s.offset:s.offset + s.dim].to(device=self.device,
                                                                            dtype=torch.float32).contiguous()

    def kernels(self):
        return [("token_side", None)]

    def forward(self, h, ctx):
        s = self.spec
        need = ops.token_side_scratch(h.shape[0], s.hidden, s.dim)
        scratch = ctx.ws.flat("side_scratch", need, torch.float32,
                              reserve=ops.token_side_scratch(127, s.hidden, s.dim)) if need else None
        ops.token_side(h, ctx.tokens, self.table, self.w_gate, self.w_proj, self.w_norm, ctx.row_entry,
                       s.eps, ctx.status, scratch)
