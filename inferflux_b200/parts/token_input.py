"""What a layer adds to the residual stream from the step's token ids.

    gated_table     e = side[token, first_column : first_column + dim]        (a table shared by all layers)
                    y = W_proj (gelu_tanh(W_gate x) * e)
                    delta = scale * y / rms(y) * norm                         (joins x as a normed delta)

The table belongs to the embedding part, which leaves it in `ctx.side_table` for the step; the gate reads the
residual stream in the run's dtype, the norm of y is float32 like every norm.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import NormedDelta, TokenInput, WeightBuffers, register_part


@register_part("token_input", "gated_table")
class GatedTableInput(TokenInput):
    """params: hidden_size, dim (columns of the table this layer reads), first_column, eps, scale (the normed
    delta is multiplied by it; default 1), names (tensor names of gate, proj, norm)."""

    _NAMES = {"gate": "gate", "proj": "proj", "norm": "norm"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.dim = int(p["dim"])
        self.first_column = int(p.get("first_column", 0))
        self.eps = float(p["eps"])
        self.scale = float(p.get("scale", 1.0))
        if self.hidden <= 0 or self.dim <= 0 or self.first_column < 0:
            raise ValueError("gated_table: sizes must be positive")
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_gate = self.w_proj = self.norm_weight = None

    def param_specs(self):
        n = self.names
        return {n["gate"]: TensorSpec((self.dim, self.hidden)), n["proj"]: TensorSpec((self.hidden, self.dim)),
                n["norm"]: TensorSpec((self.hidden,), init="ones")}

    def load(self, tensors, dtype, device):
        n = self.names
        self.buffers = buf = WeightBuffers(device, {"gate": ((self.dim, self.hidden), dtype),
                                                    "proj": ((self.hidden, self.dim), dtype),
                                                    "norm": ((self.hidden,), torch.float32)})
        buf["gate"].copy_(tensors[n["gate"]])
        buf["proj"].copy_(tensors[n["proj"]])
        buf["norm"].copy_(tensors[n["norm"]].to(torch.float32) * self.scale)      # the kernels multiply by this
        self.w_gate, self.w_proj, self.norm_weight = buf["gate"], buf["proj"], buf["norm"]

    def forward(self, x, ctx, rows=None):
        """`rows`: x in the run's dtype if the caller has it already."""
        k = ctx.kernels
        table = getattr(ctx, "side_table", None)
        if table is None or self.first_column + self.dim > table.shape[1]:
            raise ValueError("gated_table: the model's embedding brings no table with this layer's columns")
        if rows is None:
            rows = k.cast_rows(x, ctx.dtype)
        z = k.linear(rows, self.w_gate)                                                  # [T, dim]
        g = k.gelu_mul_table(z, table, ctx.token_ids, self.first_column)              # gelu(z) * e
        return NormedDelta(k.linear(g, self.w_proj, allow_partial=True), self.norm_weight, self.eps)
