"""Grouped-query causal attention over a paged key/value cache.

q, k, v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv (biases by tensor presence,
runtime/backends/cuda/native/weight_map.cpp:55-58); q and k are rotated after the
bias (runtime/backends/cuda/native/transformer_forward.cu:2024-2089); rotated keys
and raw values go to the cache at the token's position (runtime/backends/cuda/native/
kernels/fused_rope_kv_append.cuh:110-143); query head h uses key/value head
h // (heads / kv_heads), score = q.k * scale, every token sees the keys up to its
own position, or the last `window` of them (runtime/backends/cuda/kernels/
flash_attention.cu:71-86, 152-172); then the output projection.

The three projections are stacked at load so that one product makes q, k and v.

Options that other designs use, all off by default: values of their own head size (`v_head_dim`), an RMS
norm of every query and key head before the rotation with one weight per side (`qk_norm`), a mask in
chunks (`chunk`: position p sees the keys from (p // chunk) * chunk on), one more unit in the softmax's
denominator (`sink`; "learned": exp of a learned number per head instead of one), a layer that projects queries only
and reads the keys and values another layer's cache holds (`own_kv` False), a short causal convolution over time on
every channel of q, k and v right behind the projection (`conv_taps`; the last taps - 1 projected rows are the
request's state), a query multiplier 1 + coef ln(floor((p + 1) / every) + 1) at position p (`q_temp`), a gate
sigmoid(W_g h) on the heads' outputs in front of the output projection (`gate`), and other tensor names (`names`).
"""
from __future__ import annotations

import math

import torch

from ..weights.loader import TensorSpec
from .base import KVCacheSpec, Mixer, StateSpec, WeightBuffers, build_part, register_part


def materialized_rows(kernels, h):
    """`h` as a tensor, also when the norm in front left its row scale to the product that follows."""
    make = getattr(kernels, "materialize_rows", None)
    return make(h) if make is not None and not isinstance(h, torch.Tensor) else h


@register_part("mixer", "attention")
class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, window (None or int),
    position (a PartSpec of role `position`, or None), qkv_bias (True, False or
    "if_present"), invent_bias (with "if_present": whether random-weights mode makes
    the biases up; default True), scale (None for 1/sqrt(head_dim)), v_head_dim (None: head_dim),
    qk_norm (None, or {eps}), chunk (None or int), sink (bool, or "learned": a tensor [heads]), own_kv (default True),
    conv_taps (None or int), q_temp (None, or {coef, every}), gate (None or "sigmoid"),
    names (tensor names of q, k, v, o, q_bias, k_bias, v_bias, q_norm, k_norm, sink, gate, q_conv, k_conv, v_conv)."""

    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
              "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
              "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sink", "gate": "gate_proj.weight",
              "q_conv": "q_conv.weight", "k_conv": "k_conv.weight", "v_conv": "v_conv.weight"}

    takes_scaled_rows = True          # h goes only into the stacked projection

    @staticmethod
    def check_head_dim(d: int) -> None:
        """The attention kernels (tiled or per-token) take head sizes that are multiples of 8 up
        to 256; anything else is refused when the model is planned, not at the first step."""
        if d <= 0 or d % 8 or d > 256:
            raise ValueError(f"attention: head size {d} is not supported (multiples of 8 up to 256)")

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.dv = int(p["v_head_dim"]) if p.get("v_head_dim") is not None else self.d
        self.general = (any(p.get(k) for k in ("qk_norm", "chunk", "sink", "conv_taps", "q_temp", "gate"))
                        or self.dv != self.d or not p.get("own_kv", True))
        if self.general:                   # the general kernels take any even size up to 256
            for size in (self.d, self.dv):
                if size <= 0 or size % 2 or size > 256:
                    raise ValueError(f"attention: head size {size} is not supported (even sizes up to 256)")
        else:
            self.check_head_dim(self.d)
        if self.nq % self.nkv:
            raise ValueError(f"attention: {self.nq} heads are not a multiple of {self.nkv} kv heads")
        self.window = None if p.get("window") is None else int(p["window"])
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.d)
        self.qkv_bias = p.get("qkv_bias", "if_present")
        self.invent_bias = bool(p.get("invent_bias", True))
        pos = p.get("position")
        self.position = build_part("position", pos) if pos is not None else None
        self.qk_norm_eps = None if not p.get("qk_norm") else float(p["qk_norm"]["eps"])
        self.chunk = None if not p.get("chunk") else int(p["chunk"])
        if self.chunk is not None and self.chunk <= 0:
            raise ValueError(f"attention: chunk must be positive, got {self.chunk}")
        self.sink = bool(p.get("sink", False))
        self.learned_sink = p.get("sink") == "learned"
        self.own_kv = bool(p.get("own_kv", True))
        self.taps = None if not p.get("conv_taps") else int(p["conv_taps"])
        if self.taps is not None and not (self.own_kv and 1 <= self.taps <= 16):
            raise ValueError("attention: a convolution behind the projections needs keys of its own and 1 to 16 taps")
        qt = p.get("q_temp")
        self.q_temp = None if not qt else (float(qt["coef"]), int(qt["every"]))
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"attention: q_temp.every must be at least 1, got {self.q_temp[1]}")
        self.gate = p.get("gate") or None
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"attention: unknown gate {self.gate!r} (known: sigmoid)")
        if self.general and self.qkv_bias == "if_present":
            self.qkv_bias = False
        if self.general and self.qkv_bias:
            raise ValueError("attention: biases together with head norms, chunks, a sink or a shared cache are not built")
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.sink_values = self.w_gate = self.w_conv = None

    # ---------------------------------------------------------------- declarations
    def cache_spec(self):
        """Rows that hold a key or a value, whichever is longer (a multiple of 8 elements); the cache of a layer
        that stores nothing is never asked for (its schedule entry names the storing layer's)."""
        row = self.d if not self.general else -(-max(self.d, self.dv) // 8) * 8
        return KVCacheSpec(self.nkv, row, self.window, chunk=self.retain_chunk)

    # The stretch of positions after which the cache may drop pages: the mask's own chunk, unless the
    # configuration says that a reader of this cache looks further back (it then sets this to None).
    @property
    def retain_chunk(self):
        return self.spec.params.get("retain_chunk", self.chunk)

    def state_spec(self):
        """The last taps - 1 rows of the stacked projection, the convolution's inputs before a step's first token."""
        if self.taps is None or self.taps < 2:
            return None
        return StateSpec(((self.taps - 1) * sum(self._sizes()),), torch.float32)

    def _sizes(self):
        """Rows of the stacked projection: (query rows, key rows, value rows)."""
        kv = self.nkv if self.own_kv else 0
        return self.nq * self.d, kv * self.d, kv * self.dv

    def param_specs(self):
        n = self.names
        q, k, v = self._sizes()
        specs = {n["q"]: TensorSpec((q, self.hidden)), n["o"]: TensorSpec((self.hidden, self.nq * self.dv))}
        if self.own_kv:
            specs[n["k"]] = TensorSpec((k, self.hidden))
            specs[n["v"]] = TensorSpec((v, self.hidden))
        if self.qkv_bias is not False:
            optional = self.qkv_bias == "if_present"
            for side, size in (("q", q), ("k", k), ("v", v)):
                specs[n[side + "_bias"]] = TensorSpec((size,), optional=optional, invent=self.invent_bias)
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((self.d,), init="ones")
            if self.own_kv:
                specs[n["k_norm"]] = TensorSpec((self.d,), init="ones")
        if self.learned_sink:
            specs[n["sink"]] = TensorSpec((self.nq,))
        if self.gate is not None:
            specs[n["gate"]] = TensorSpec((self.nq * self.dv, self.hidden))
        if self.taps is not None:
            for side, size in (("q", q), ("k", k), ("v", v)):
                specs[n[side + "_conv"]] = TensorSpec((size, self.taps))
        return specs

    def load(self, tensors, dtype, device):
        n = self.names
        q, k, v = self._sizes()
        sides = [("q", q)] + ([("k", k), ("v", v)] if self.own_kv else [])
        has_bias = any(n[side + "_bias"] in tensors for side, _ in sides)
        layout = {"w_qkv": ((q + k + v, self.hidden), dtype), "w_o": ((self.hidden, self.nq * self.dv), dtype)}
        if has_bias:
            layout["b_qkv"] = ((q + k + v,), torch.float32)               # added in float32
        if self.qk_norm_eps is not None:
            layout["q_norm"] = ((self.d,), torch.float32)
            layout["k_norm"] = ((self.d,), torch.float32)
        if self.learned_sink:
            layout["sink"] = ((self.nq,), torch.float32)
        if self.gate is not None:
            layout["w_gate"] = ((self.nq * self.dv, self.hidden), dtype)
        if self.taps is not None:
            layout["w_conv"] = ((q + k + v, self.taps), torch.float32)
        self.buffers = buf = WeightBuffers(device, layout)
        if self.learned_sink:
            buf["sink"].copy_(tensors[n["sink"]])
            self.sink_values = buf["sink"]
        if self.gate is not None:
            buf["w_gate"].copy_(tensors[n["gate"]])
            self.w_gate = buf["w_gate"]
        if self.taps is not None:                                          # the three convolutions as one over the stacked rows
            at = 0
            for side, size in (("q", q), ("k", k), ("v", v)):
                buf["w_conv"][at:at + size].copy_(tensors[n[side + "_conv"]])
                at += size
            self.w_conv = buf["w_conv"]
        at = 0
        for side, size in sides:                                          # each projection into its rows of the stack
            buf["w_qkv"][at:at + size].copy_(tensors[n[side]])
            if has_bias:
                b = tensors.get(n[side + "_bias"])
                if b is None:
                    buf["b_qkv"][at:at + size].zero_()
                else:
                    buf["b_qkv"][at:at + size].copy_(b)
            at += size
        buf["w_o"].copy_(tensors[n["o"]])
        self.w_qkv, self.w_o = buf["w_qkv"], buf["w_o"]
        self.b_qkv = buf["b_qkv"] if has_bias else None
        if self.qk_norm_eps is not None:
            buf["q_norm"].copy_(tensors[n["q_norm"]])
            self.q_norm_w = buf["q_norm"]
            if self.own_kv:
                buf["k_norm"].copy_(tensors[n["k_norm"]])
                self.k_norm_w = buf["k_norm"]

    def step_sections(self, ctx):
        """The work lists of the kernel table's attention kernels, if it has any."""
        make = getattr(ctx.kernels, "attention_sections", None)
        return make(ctx) if make is not None else {}

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        qkv = k.linear(h, self.w_qkv, allow_partial=True)                    # [T, (nq + 2 nkv) d], maybe in K slices
        rotary = self.position.rotary(ctx.device) if self.position is not None else None
        if not self.general:
            q = k.rope_append(qkv, self.b_qkv, rotary, self.nq, self.nkv, self.d, ctx, cache)   # [T, nq d]
            a = k.attention(q, self.nq, self.nkv, self.d, self.window, self.scale, ctx, cache)  # [T, nq d]
            return k.linear(a, self.w_o, allow_partial=True)
        if self.own_kv != bool(cache.writes):
            raise ValueError("attention: a layer with keys and values of its own writes its cache, one without reads another's")
        more = {}
        if self.taps is not None:                          # every channel of q, k and v over time, the state moved on
            state = None if self.taps < 2 else cache.state.unflatten(1, (1, self.taps - 1, sum(self._sizes())))
            qkv = k.short_conv(k.materialize(qkv), self.w_conv, self.taps, state, 0, ctx, add_input=False)
        if self.q_temp is not None:
            more["q_temp"] = self.q_temp
        q = k.rope_append(qkv, None, rotary, self.nq, self.nkv, self.d, ctx, cache, q_norm=self.q_norm_w,
                          k_norm=self.k_norm_w, norm_eps=self.qk_norm_eps or 0.0, dv=self.dv, own_kv=self.own_kv, **more)
        a = k.attention(q, self.nq, self.nkv, self.d, self.window, self.scale, ctx, cache, chunk=self.chunk,
                        sink=self.sink_values if self.learned_sink else self.sink, dv=self.dv)   # [T, nq dv]
        if self.gate is not None:
            a = k.gate_mul(a, k.linear(materialized_rows(k, h), self.w_gate), self.gate)
        return k.linear(a, self.w_o, allow_partial=True)
