"""A feed-forward made of many small experts of which every token uses a few.

    z = W_router h (float32)      scores = softmax(z) over all router outputs
    chosen = the `top` outputs with the largest scores + correction        (the correction only steers the choice)
    y = sum over the chosen of score * expert(h)                           (scores as they are, not renormalised)

An expert is W_down act(W_up h) with act = relu^2 and no biases.  The last `identity` router outputs have no
weights: such an expert hands h on unchanged.  Expert weights are stacked at load, [experts, ff, width] and
[experts, width, ff], so that the kernels find an expert by its number.

Options.  `routing` = `softmax_of_chosen`: the `top` largest logits are chosen and the weights are the softmax over
those alone.  `activation` = `clamped_glu`: an expert has a gate matrix too (stacked as [experts, 2 ff, width], an
expert's gate rows above its up rows) and, with g = min(W_gate h, limit) and u = clamp(W_up h, -limit, limit),
makes W_down (g sigmoid(1.702 g) (u + 1)); `silu_glu`: the same stack, W_down (silu(W_gate h) * W_up h), nothing cut.
`routing` = `sigmoid_normalized`: scores = sigmoid(z), the `top` largest are chosen, and the weights are their scores
divided by (their sum + `weight_floor`).  `shared`: a feed-forward that every token uses; the block adds its output
beside the mixture's (forward then returns the pair).
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import FeedForward, WeightBuffers, build_part, register_part


@register_part("ffn", "moe")
class MixtureOfExperts(FeedForward):
    """params: hidden_size, expert_size (ff of an expert), num_experts, num_identity (default 0), top,
    activation (`relu2` or `clamped_glu` with `limit`), routing (`softmax_of_all`, the default, or
    `softmax_of_chosen`), correction (whether a selection bias tensor exists; default True),
    names (tensor names of router, correction, and the patterns `gate` / `up` / `down` with {e} for the expert's number)."""

    _NAMES = {"router": "router", "correction": "correction", "up": "e{e}.up", "down": "e{e}.down", "gate": "e{e}.gate"}
    GLU_SLOPE = 1.702                 # the sigmoid's slope in the gated activation

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.ff = int(p["expert_size"])
        self.experts = int(p["num_experts"])
        self.identity = int(p.get("num_identity", 0))
        self.top = int(p["top"])
        self.activation = str(p.get("activation", "relu2"))
        if self.activation not in ("relu2", "clamped_glu", "silu_glu"):
            raise ValueError(f"moe: unknown activation {self.activation!r} (known: relu2, clamped_glu, silu_glu)")
        self.gated = self.activation in ("clamped_glu", "silu_glu")
        self.limit = float(p["limit"]) if self.activation == "clamped_glu" else 0.0
        if self.activation == "clamped_glu" and not self.limit > 0:
            raise ValueError(f"moe: the gated activation's limit must be positive, got {self.limit}")
        # (limit, the sigmoid's slope, what is added to the up value) of g sigmoid(slope g) (u + offset)
        self.glu = None if not self.gated else ((self.limit, self.GLU_SLOPE, 1.0) if self.activation == "clamped_glu"
                                                else (float("inf"), 1.0, 0.0))
        self.routing = str(p.get("routing", "softmax_of_all"))
        if self.routing not in ("softmax_of_all", "softmax_of_chosen", "sigmoid_normalized"):
            raise ValueError(f"moe: unknown routing {self.routing!r}")
        self.weight_floor = float(p.get("weight_floor", 0.0))
        self.shared = build_part("ffn", p["shared"]) if p.get("shared") is not None else None
        if self.experts < 0 or self.identity < 0 or self.experts + self.identity < 1:
            raise ValueError("moe: there must be at least one expert")
        if not 1 <= self.top <= self.experts + self.identity:
            raise ValueError(f"moe: top {self.top} of {self.experts + self.identity} experts")
        if self.experts + self.identity > 1024:
            raise ValueError("moe: more than 1024 router outputs are beyond the kernel")
        self.has_correction = bool(p.get("correction", True))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_router = self.correction = self.w_up = self.w_down = None

    def param_specs(self):
        n, outs = self.names, self.experts + self.identity
        specs = {n["router"]: TensorSpec((outs, self.hidden))}
        if self.has_correction:
            specs[n["correction"]] = TensorSpec((outs,), init="zeros")
        for e in range(self.experts):
            if self.gated:
                specs[n["gate"].format(e=e)] = TensorSpec((self.ff, self.hidden))
            specs[n["up"].format(e=e)] = TensorSpec((self.ff, self.hidden))
            specs[n["down"].format(e=e)] = TensorSpec((self.hidden, self.ff))
        if self.shared is not None:
            specs.update(self.shared.param_specs())
        return specs

    def load(self, tensors, dtype, device):
        n, outs = self.names, self.experts + self.identity
        if self.shared is not None:
            self.shared.load({name: tensors[name] for name in self.shared.param_specs()}, dtype, device)
        layout = {"router": ((outs, self.hidden), dtype), "correction": ((outs,), torch.float32)}
        if self.experts:
            layout["up"] = ((self.experts, (2 if self.gated else 1) * self.ff, self.hidden), dtype)
            layout["down"] = ((self.experts, self.hidden, self.ff), dtype)
        self.buffers = buf = WeightBuffers(device, layout)
        buf["router"].copy_(tensors[n["router"]])
        if self.has_correction:
            buf["correction"].copy_(tensors[n["correction"]])
        else:
            buf["correction"].zero_()
        for e in range(self.experts):                    # each expert into its slice of the stack
            if self.gated:
                buf["up"][e][:self.ff].copy_(tensors[n["gate"].format(e=e)])
                buf["up"][e][self.ff:].copy_(tensors[n["up"].format(e=e)])
            else:
                buf["up"][e].copy_(tensors[n["up"].format(e=e)])
            buf["down"][e].copy_(tensors[n["down"].format(e=e)])
        self.w_router, self.correction = buf["router"], buf["correction"]
        self.w_up = buf["up"] if self.experts else None
        self.w_down = buf["down"] if self.experts else None

    def forward(self, h, ctx):
        k = ctx.kernels
        z = k.linear(h, self.w_router, out_dtype=torch.float32)                   # [T, experts + identity]
        if self.routing == "sigmoid_normalized":
            ids, weights = k.moe_route(z, self.correction if self.has_correction else None, self.top,
                                       kind="sigmoid_normalized", floor=self.weight_floor)
            y = k.moe_experts(h, self.w_up, self.w_down, ids, weights, self.experts, ctx.dtype, glu=self.glu)
            return y if self.shared is None else (y, self.shared.forward(h, ctx))
        if self.shared is not None:
            raise ValueError("moe: a shared expert beside softmax routing is not built")
        if self.routing == "softmax_of_chosen" or self.gated:
            ids, weights = k.moe_route(z, self.correction if self.has_correction else None, self.top,
                                       of_chosen=self.routing == "softmax_of_chosen")
            return k.moe_experts(h, self.w_up, self.w_down, ids, weights, self.experts, ctx.dtype,
                                 glu=self.glu)
        ids, weights = k.moe_route(z, self.correction, self.top)
        return k.moe_experts(h, self.w_up, self.w_down, ids, weights, self.experts, ctx.dtype)
