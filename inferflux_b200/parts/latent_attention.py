"""Attention whose keys and values are made, for all heads, from one low-rank latent per token.

    q_h = Wq_h x                      c = rmsnorm(Wdkv x) * g          (the latent, `kv_rank` numbers)
    k_h = Wuk_h c,  v_h = Wuv_h c     score = scale * q_h . k_h        no position encoding
    weights = softmax over the window, with exp(sink_h) added to the denominator (optional)
    y = Wo [o_1; ...; o_H]

Only c is cached: one plane of one head of size kv_rank per token, in pages through the same
block tables as every other cache.  The kernels never make k or v: the query head is carried
into latent space (Wuk_h^T q_h), the weighted sum runs over cached latents, and Wuv_h is applied
to that sum.  Query and latent projections are stacked at load so that one product makes both.

Options: queries through a normed latent of their own (`q_rank`: q = Wuq rmsnorm(Wdq x) * g_q), and a
rotated part (`rot_dim` > 0 with a `position` part): every query head has rot_dim more elements behind its
qk_dim plain ones, Wdkv has rot_dim more rows behind the latent's, which are not normed and are one key part
that all heads share; both are turned by the token's position, and

    score = scale * (q_plain . k_plain + q_turned . k_turned)

The cached row is then [c; k_turned] (kv_rank + rot_dim numbers), and a query in latent space
[Wuk_h^T q_plain; q_turned] meets it in one dot product.
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from ..config.plan import PartSpec
from .base import KVCacheSpec, Mixer, WeightBuffers, build_part, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """params: hidden_size, num_heads, qk_dim, v_dim, kv_rank, window (None or int), scale (None for
    1/sqrt(qk_dim)), latent_norm_eps, sink (whether heads have a learned sink), q_rank (None: queries straight
    from the input), rot_dim (default 0) with position (a PartSpec of a position encoding that turns those
    elements), names (tensor names of q, dkv, dkv_norm, uk, uv, sink, o, dq, dq_norm, uq; default: those words
    with `_` as `.`)."""

    _NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "sink": "sink", "o": "o",
              "dq": "dq", "dq_norm": "dq.norm", "uq": "uq"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dk = int(p["qk_dim"])
        self.dv = int(p["v_dim"])
        self.rank = int(p["kv_rank"])
        for name in ("hidden", "heads", "dk", "dv", "rank"):
            if getattr(self, name) <= 0:
                raise ValueError(f"latent_attention: {name} must be positive, got {getattr(self, name)}")
        self.q_rank = None if p.get("q_rank") is None else int(p["q_rank"])
        self.rot = int(p.get("rot_dim") or 0)
        self.position = None
        if self.rot:
            position = p.get("position")
            if not isinstance(position, PartSpec):
                raise ValueError("latent_attention: a rotated part needs a position encoding")
            self.position = build_part("position", position)
        if self.rank + self.rot > 1024:
            raise ValueError(f"latent_attention: a cached row of {self.rank + self.rot} is beyond the kernels' 1024")
        if (self.q_rank is not None and self.q_rank <= 0) or self.rot < 0:
            raise ValueError("latent_attention: q_rank must be positive and rot_dim not negative")
        self.window = None if p.get("window") is None else int(p["window"])
        if self.window is not None and self.window <= 0:
            raise ValueError(f"latent_attention: window must be positive, got {self.window}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.dk)
        self.eps = float(p.get("latent_norm_eps", 1e-6))
        self.has_sink = bool(p.get("sink", False))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_q_dkv = self.w_uk = self.w_uv = self.w_o = self.latent_norm = self.sinks = None

    # ---------------------------------------------------------------- declarations
    def cache_spec(self):
        return KVCacheSpec(1, self.rank + self.rot, self.window, planes=1)

    def param_specs(self):
        n, H = self.names, self.heads
        dq = self.dk + self.rot
        specs = {n["q"]: TensorSpec((H * dq, self.hidden))} if self.q_rank is None else {
            n["dq"]: TensorSpec((self.q_rank, self.hidden)), n["dq_norm"]: TensorSpec((self.q_rank,), init="ones"),
            n["uq"]: TensorSpec((H * dq, self.q_rank))}
        specs.update({
            n["dkv"]: TensorSpec((self.rank + self.rot, self.hidden)),
            n["dkv_norm"]: TensorSpec((self.rank,), init="ones"),
            n["uk"]: TensorSpec((H * self.dk, self.rank)),
            n["uv"]: TensorSpec((H * self.dv, self.rank)),
            n["o"]: TensorSpec((self.hidden, H * self.dv)),
        })
        if self.has_sink:
            specs[n["sink"]] = TensorSpec((H,), init="zeros")
        return specs

    def load(self, tensors, dtype, device):
        n, H = self.names, self.heads
        q = H * (self.dk + self.rot) if self.q_rank is None else self.q_rank      # rows in front of the latent's
        layout = {
            "w_q_dkv": ((q + self.rank + self.rot, self.hidden), dtype), "w_uk": ((H * self.dk, self.rank), dtype),
            "w_uv": ((H * self.dv, self.rank), dtype), "w_o": ((self.hidden, H * self.dv), dtype),
            "latent_norm": ((self.rank,), torch.float32), "sinks": ((H,), torch.float32)}
        if self.q_rank is not None:
            layout.update({"w_uq": ((H * (self.dk + self.rot), self.q_rank), dtype), "q_norm": ((self.q_rank,), torch.float32)})
        self.buffers = buf = WeightBuffers(device, layout)
        buf["w_q_dkv"][:q].copy_(tensors[n["q"] if self.q_rank is None else n["dq"]])
        buf["w_q_dkv"][q:].copy_(tensors[n["dkv"]])
        self.w_uq = self.q_norm = None
        if self.q_rank is not None:
            buf["w_uq"].copy_(tensors[n["uq"]])
            buf["q_norm"].copy_(tensors[n["dq_norm"]])
            self.w_uq, self.q_norm = buf["w_uq"], buf["q_norm"]
        buf["w_uk"].copy_(tensors[n["uk"]])
        buf["w_uv"].copy_(tensors[n["uv"]])
        buf["w_o"].copy_(tensors[n["o"]])
        buf["latent_norm"].copy_(tensors[n["dkv_norm"]])
        if self.has_sink:
            buf["sinks"].copy_(tensors[n["sink"]])
        self.w_q_dkv, self.w_uk, self.w_uv, self.w_o = buf["w_q_dkv"], buf["w_uk"], buf["w_uv"], buf["w_o"]
        self.latent_norm = buf["latent_norm"]
        self.sinks = buf["sinks"] if self.has_sink else None

    def step_sections(self, ctx):
        """The work lists of the kernel table's latent attention kernels, if it has any."""
        make = getattr(ctx.kernels, "latent_attention_sections", None)
        return make(ctx) if make is not None else {}

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        if self.q_rank is not None or self.rot:
            return self._forward_with_options(h, ctx, cache)
        q_dkv = k.materialize(k.linear(h, self.w_q_dkv, allow_partial=True))   # [T, H dk + rank]
        k.latent_norm_append(q_dkv, self.heads * self.dk, self.rank, self.latent_norm, self.eps, ctx, cache)
        a = k.latent_attention(q_dkv, self.w_uk, self.w_uv, self.sinks, self.heads, self.dk, self.dv, self.rank,
                               self.window, self.scale, ctx, cache)         # [T, H dv]
        return k.linear(a, self.w_o, allow_partial=True)

    def _forward_with_options(self, h, ctx, cache):
        k = ctx.kernels
        H, dq = self.heads, self.dk + self.rot
        down = k.materialize(k.linear(h, self.w_q_dkv, allow_partial=True))    # [T, (q_rank or H dq) + rank + rot]
        col0 = self.q_rank if self.q_rank is not None else H * dq              # where the latent's columns begin
        if self.q_rank is not None:
            cq = k.rmsnorm_columns(down, 0, self.q_rank, self.q_norm, self.eps)    # the queries' normed latent
            q = k.linear(cq, self.w_uq)                                            # [T, H dq]
        else:
            q = down
        rotary = self.position.rotary(ctx.device) if self.position is not None else None
        # norms the latent, turns the shared key part and every query head's last `rot` elements, stores [c; k_turned]
        q = k.latent_rope_append(down, col0, self.rank, self.rot, self.latent_norm, self.eps, q, H, self.dk, rotary, ctx, cache,
                                 vdim=self.dv)
        a = k.latent_attention(q, self.w_uk, self.w_uv, self.sinks, H, self.dk, self.dv, self.rank, self.window,
                               self.scale, ctx, cache, rot=self.rot)            # [T, H dv]
        return k.linear(a, self.w_o, allow_partial=True)
