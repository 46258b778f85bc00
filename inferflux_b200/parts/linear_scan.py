"""Two mixers that keep, per head, a matrix of state S (key channels x value channels) which every token decays and
writes to, S <- diag(w_t) S + k_t v_t^T, and reads with the new S, o_t = S^T q_t.  Both run on the same scan kernel
(`ctx.kernels.decay_scan`), which turns the raw decay inputs into decays itself, in float32.

`decayed_linear_attention`: a decay per key channel from a low-rank projection,

    q = W_q h / sqrt(key_dim),  k = W_k h,  v = W_v h          (heads x key_dim, heads x key_dim, heads x value_dim)
    w = sigmoid(W_a2 (W_a1 h) + b)^(1/tau)                      per head and key channel
    y = W_o ((o / rms(o) per head) * norm * silu(W_g h))       norm: one weight per value channel, shared by the heads

`state_space`: a decay per head from a step size, keys and queries shared by the heads of a group,

    [z | x | B | C | dt] = W_in h;   x, B, C <- silu(conv(x, B, C) + b_conv)   (causal, per channel, over time)
    dt = softplus(dt + dt_bias),  w = exp(-exp(A_log) dt),  k = dt B,  q = C,  v = x       o += D x
    y = W_o (groupnorm(o * silu(z)) * norm)                     the gate in front of the norm, the norm over equal parts

S (float32) and the convolution's last taps - 1 input rows are the request's state: a slot of fixed size, whatever the
length, zeroed when a request is admitted.  The projections take h in the run's dtype and hand their results over
in float32; the decays, the step size, the state, the norms and the gates are float32.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .attention import materialized_rows
from .base import Mixer, StateSpec, WeightBuffers, register_part


@register_part("mixer", "decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, tau, norm_eps, decay_rank (None: the file's `a1` says;
    random weights then use 16 or a quarter of the width, whichever is smaller), names (tensor names of q, k, v, g,
    a1, a2, a2_bias, norm, o)."""

    _NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "a1": "a1", "a2": "a2", "a2_bias": "a2.b", "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dk = int(p["key_dim"])
        self.dv = int(p["value_dim"])
        self.tau = float(p["tau"])
        if min(self.hidden, self.heads, self.dk, self.dv) <= 0 or not self.tau > 0:
            raise ValueError("decayed_linear_attention: sizes and tau must be positive")
        if self.dk > 512:
            raise ValueError(f"decayed_linear_attention: a key size of {self.dk} is beyond the kernel's 512")
        self.rank = None if p.get("decay_rank") is None else int(p["decay_rank"])
        self.eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_stack = self.w_a1 = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None

    def state_spec(self):
        """S of every head as [head, value channel, key channel]."""
        return StateSpec((self.heads * self.dk * self.dv,), torch.float32)

    def param_specs(self):
        n, K, V, C = self.names, self.heads * self.dk, self.heads * self.dv, self.hidden
        rank = -1 if self.rank is None else self.rank
        made = self.rank if self.rank is not None else max(1, min(16, C // 4))
        return {n["q"]: TensorSpec((K, C)), n["k"]: TensorSpec((K, C)), n["v"]: TensorSpec((V, C)), n["g"]: TensorSpec((V, C)),
                n["a1"]: TensorSpec((rank, C), made_shape=(made, C)), n["a2"]: TensorSpec((K, rank), made_shape=(K, made)),
                n["a2_bias"]: TensorSpec((K,), init="zeros"), n["norm"]: TensorSpec((self.dv,), init="ones"),
                n["o"]: TensorSpec((C, V))}

    def load(self, tensors, dtype, device):
        n, K, V, C = self.names, self.heads * self.dk, self.heads * self.dv, self.hidden
        rank = int(tensors[n["a1"]].shape[0])
        if tensors[n["a2"]].shape[1] != rank:
            raise ValueError(f"decayed_linear_attention: the decay's two matrices meet at {rank} and {tensors[n['a2']].shape[1]}")
        self.buffers = buf = WeightBuffers(device, {
            "stack": ((2 * K + 2 * V, C), dtype),              # q, k, v, g one below the other: one product
            "a1": ((rank, C), dtype), "a2": ((K, rank), dtype), "o": ((C, V), dtype),
            "a2_bias": ((K,), torch.float32), "norm": ((self.dv,), torch.float32)})
        at = 0
        for s, rows in (("q", K), ("k", K), ("v", V), ("g", V)):
            buf["stack"][at:at + rows].copy_(tensors[n[s]])
            at += rows
        for s in ("a1", "a2", "o", "a2_bias", "norm"):
            buf[s].copy_(tensors[n[s]])
        self.w_stack, self.w_a1, self.w_a2, self.w_o = buf["stack"], buf["a1"], buf["a2"], buf["o"]
        self.b_a2, self.norm_w = buf["a2_bias"], buf["norm"]
        self.rank = rank

    def forward(self, h, ctx, cache):
        k = ctx.kernels
        f32 = torch.float32
        K, V = self.heads * self.dk, self.heads * self.dv
        h = materialized_rows(k, h)
        proj = k.materialize(k.linear(h, self.w_stack, out_dtype=f32, allow_partial=True))      # [T, 2K + 2V]: q k v g
        raw = k.linear(k.linear(h, self.w_a1), self.w_a2, bias=self.b_a2, out_dtype=f32)         # [T, K]
        o = k.decay_scan(proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V], raw, cache.state, ctx,
                         heads=self.heads, groups=self.heads, dk=self.dk, dv=self.dv, decay="sigmoid_root", tau=self.tau,
                         q_scale=self.dk ** -0.5)                                                # [T, V] float32
        y = k.gated_groupnorm(o, proj[:, 2 * K + V:], self.norm_w, self.eps, groups=self.heads, gate_first=False,
                              out_dtype=ctx.dtype)
        return k.linear(y, self.w_o, out_dtype=f32)


@register_part("mixer", "state_space")
class StateSpace(Mixer):
    """params: hidden_size, num_heads, value_dim, state_dim, groups, norm_groups, conv_taps, norm_eps,
    names (tensor names of in, conv, conv_bias, dt_bias, A_log, D, norm, o)."""

    _NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
              "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dv = int(p["value_dim"])
        self.n = int(p["state_dim"])
        self.groups = int(p["groups"])
        self.norm_groups = int(p.get("norm_groups", 1))
        self.taps = int(p["conv_taps"])
        if min(self.hidden, self.heads, self.dv, self.n, self.groups, self.norm_groups, self.taps) <= 0:
            raise ValueError("state_space: sizes must be positive")
        if self.heads % self.groups or (self.heads * self.dv) % self.norm_groups:
            raise ValueError("state_space: groups must divide the heads, norm_groups the inner size")
        if self.n > 512 or self.taps > 16:
            raise ValueError("state_space: a state of more than 512 or more than 16 taps is beyond the kernels")
        self.inner = self.heads * self.dv
        self.conv_channels = self.inner + 2 * self.groups * self.n
        self.eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})

    def state_spec(self):
        """[the convolution's last taps - 1 input rows, then S of every head as [head, value channel, key channel]]."""
        return StateSpec(((self.taps - 1) * self.conv_channels + self.heads * self.n * self.dv,), torch.float32)

    def param_specs(self):
        n, C = self.names, self.hidden
        return {n["in"]: TensorSpec((self.inner + self.conv_channels + self.heads, C)),
                n["conv"]: TensorSpec((self.conv_channels, self.taps)), n["conv_bias"]: TensorSpec((self.conv_channels,), init="zeros"),
                n["dt_bias"]: TensorSpec((self.heads,), init="zeros"), n["A_log"]: TensorSpec((self.heads,), init="zeros"),
                n["D"]: TensorSpec((self.heads,), init="ones"), n["norm"]: TensorSpec((self.inner,), init="ones"),
                n["o"]: TensorSpec((C, self.inner))}

    def load(self, tensors, dtype, device):
        n, C, f32 = self.names, self.hidden, torch.float32
        self.buffers = buf = WeightBuffers(device, {
            "in": ((self.inner + self.conv_channels + self.heads, C), dtype), "o": ((C, self.inner), dtype),
            "conv": ((self.conv_channels, self.taps), f32), "conv_bias": ((self.conv_channels,), f32),
            "dt_bias": ((self.heads,), f32), "A_log": ((self.heads,), f32), "D": ((self.heads,), f32),
            "norm": ((self.inner,), f32)})
        for s in buf.views:
            buf[s].copy_(tensors[n[s]])
        self.w_in, self.w_o = buf["in"], buf["o"]

    def forward(self, h, ctx, cache):
        k = ctx.kernels
        f32, buf = torch.float32, self.buffers
        inner, gn = self.inner, self.groups * self.n
        rows = (self.taps - 1) * self.conv_channels
        zx = k.materialize(k.linear(materialized_rows(k, h), self.w_in, out_dtype=f32, allow_partial=True))   # [T, z | x B C | dt]
        conv_state = None if self.taps < 2 else cache.state[:, :rows].unflatten(1, (1, self.taps - 1, self.conv_channels))
        xbc = k.short_conv(zx, buf["conv"], self.taps, conv_state, 0, ctx, add_input=False, bias=buf["conv_bias"],
                           act="silu", columns=(inner, self.conv_channels))                                      # [T, x | B | C]
        o = k.decay_scan(xbc[:, inner + gn:], xbc[:, inner:inner + gn], xbc[:, :inner], zx[:, inner + self.conv_channels:],
                         cache.state[:, rows:], ctx, heads=self.heads, groups=self.groups, dk=self.n, dv=self.dv,
                         decay="softplus_step", step_bias=buf["dt_bias"], log_rate=buf["A_log"], skip=buf["D"])
        y = k.gated_groupnorm(o, zx[:, :inner], buf["norm"], self.eps, groups=self.norm_groups, gate_first=True,
                              out_dtype=ctx.dtype)
        return k.linear(y, self.w_o, out_dtype=f32)
