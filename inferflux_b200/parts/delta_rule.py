"""A mixer that keeps, per head, a matrix of state (key channels x value channels) which every token decays,
partly erases along its own key, and writes to:

    r, k, v = W_r h, W_k h, W_v h                                  (heads x dim each)
    decay   = exp(-exp(-1/2) sigmoid(W_w2 tanh(W_w1 h) + w0))       per head and key channel, in (0.545, 1)
    a       = sigmoid(W_a h + b_a)                                 how much is erased, per head and key channel
    u       = k / sqrt(sum k^2 + 1e-6)                             the unit key of each head
    S       = diag(decay) S - (a * u) (u^T S) + k v^T              both products of the old S
    out     = S^T r                                                of the new S
    y       = W_o ((out / rms(out) per head) * norm * sigmoid(W_g h))

S (float32) is the request's state: a slot of fixed size, whatever the length, zeroed when a request is admitted.
The projections take h in the run's dtype and hand their results to the recurrence in float32, where the decay,
both sigmoids, the unit key, the state, the per-head norm and the gate are float32 too.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, WeightBuffers, register_part

_STACKED = ("r", "k", "v", "g", "a")


@register_part("mixer", "delta_rule")
class DeltaRule(Mixer):
    """params: hidden_size, num_heads, head_dim, decay_rank (None: the file's `w1` says; random weights then use
    16 or a quarter of the width, whichever is smaller), norm_eps (of the per-head norm of the output),
    names (tensor names of r, k, v, g, a, a_bias, w1, w2, w0, norm, o)."""

    _NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2", "w0": "w0",
              "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        if self.hidden <= 0 or self.heads <= 0 or self.dim <= 0:
            raise ValueError("delta_rule: sizes must be positive")
        if self.dim > 256:
            raise ValueError(f"delta_rule: a head size of {self.dim} is beyond the kernel's 256")
        self.rank = None if p.get("decay_rank") is None else int(p["decay_rank"])
        self.eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_stack = self.w1 = self.w2 = self.w_o = self.w0 = self.a_bias = self.norm_w = None

    # ---------------------------------------------------------------- declarations
    def state_spec(self):
        return StateSpec((self.heads * self.dim * self.dim,), torch.float32)

    def param_specs(self):
        n, HD, C = self.names, self.heads * self.dim, self.hidden
        rank = -1 if self.rank is None else self.rank
        made = self.rank if self.rank is not None else max(1, min(16, C // 4))
        specs = {n[s]: TensorSpec((HD, C)) for s in _STACKED}
        specs[n["a_bias"]] = TensorSpec((HD,), init="zeros")
        specs[n["w1"]] = TensorSpec((rank, C), made_shape=(made, C))
        specs[n["w2"]] = TensorSpec((HD, rank), made_shape=(HD, made))
        specs[n["w0"]] = TensorSpec((HD,), init="zeros")
        specs[n["norm"]] = TensorSpec((HD,), init="ones")
        specs[n["o"]] = TensorSpec((C, HD))
        return specs

    def load(self, tensors, dtype, device):
        n, HD, C = self.names, self.heads * self.dim, self.hidden
        rank = int(tensors[n["w1"]].shape[0])
        if tensors[n["w2"]].shape[1] != rank:
            raise ValueError(f"delta_rule: the decay's two matrices meet at {rank} and {tensors[n['w2']].shape[1]}")
        self.buffers = buf = WeightBuffers(device, {
            "stack": ((len(_STACKED) * HD, C), dtype),          # the five projections one below the other: one product
            "w1": ((rank, C), dtype), "w2": ((HD, rank), dtype), "o": ((C, HD), dtype),
            "w0": ((HD,), torch.float32), "a_bias": ((HD,), torch.float32), "norm": ((HD,), torch.float32)})
        for i, s in enumerate(_STACKED):
            buf["stack"][i * HD:(i + 1) * HD].copy_(tensors[n[s]])
        for s in ("w1", "w2", "o", "w0", "a_bias", "norm"):
            buf[s].copy_(tensors[n[s]])
        self.w_stack, self.w1, self.w2, self.w_o = buf["stack"], buf["w1"], buf["w2"], buf["o"]
        self.w0, self.a_bias, self.norm_w = buf["w0"], buf["a_bias"], buf["norm"]
        self.rank = rank

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        f32 = torch.float32
        HD = self.heads * self.dim
        proj = k.materialize(k.linear(h, self.w_stack, out_dtype=f32, allow_partial=True))   # [T, 5 heads dim]: r k v g a
        low = k.tanh(k.linear(h, self.w1))                                                    # [T, rank]
        w_raw = k.linear(low, self.w2, out_dtype=f32)                                         # [T, heads dim]
        y = k.delta_rule_scan(proj, w_raw, self.w0, self.a_bias, self.norm_w, self.eps, self.heads, self.dim,
                              cache.state, ctx, ctx.dtype)                                    # [T, heads dim]
        return k.linear(y, self.w_o, allow_partial=True)
