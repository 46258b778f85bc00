"""Two mixers side by side that read the same rows; their outputs become one:

    combine = plain    y = a * left(h) + b * right(h)
    combine = normed   y = a * left(h) / rms(left(h)) * w_l + b * right(h) / rms(right(h)) * w_r      (over the width)

The left mixer may keep a key/value cache and state, the right one state only; the layer's state row per request
is [the left one's, then the right one's].  The result is float32: the norms, the weights and the sum happen in one
kernel, and the block adds it to the stream as it is.
"""
from __future__ import annotations

import dataclasses

import torch

from ..weights.loader import TensorSpec
from .base import Mixer, StateSpec, build_part, register_part


def _floats(spec) -> int:
    if spec is None:
        return 0
    if spec.dtype != torch.float32:
        raise ValueError("pair: both mixers' states must be float32 to share the layer's state row")
    n = 1
    for d in spec.shape:
        n *= int(d)
    return n


@register_part("mixer", "pair")
class PairMixer(Mixer):
    """params: hidden_size, left, right (PartSpecs of role `mixer`; tensors under `left.` / `right.`), combine
    (`plain` or `normed`), left_weight, right_weight (a, b), norm_eps, names (tensor names of left_norm, right_norm)."""

    _NAMES = {"left_norm": "left_norm.weight", "right_norm": "right_norm.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.left = build_part("mixer", p["left"])
        self.right = build_part("mixer", p["right"])
        self.combine = str(p.get("combine", "plain"))
        if self.combine not in ("plain", "normed"):
            raise ValueError(f"pair: unknown combine {self.combine!r} (known: plain, normed)")
        self.a, self.b = float(p.get("left_weight", 1.0)), float(p.get("right_weight", 1.0))
        self.eps = float(p.get("norm_eps", 1e-6))
        self.names = dict(self._NAMES)
        self.names.update(p.get("names") or {})
        if self.right.cache_spec() is not None:
            raise ValueError("pair: only the left mixer may keep a key/value cache")
        self.left_floats, self.right_floats = _floats(self.left.state_spec()), _floats(self.right.state_spec())
        self.graph_safe = self.left.graph_safe and self.right.graph_safe
        self.w_left = self.w_right = None

    def sub_parts(self):
        return [self.left, self.right]

    # ---------------------------------------------------------------- declarations
    def cache_spec(self):
        return self.left.cache_spec()

    def state_spec(self):
        total = self.left_floats + self.right_floats
        return StateSpec((total,), torch.float32) if total else None

    def param_specs(self):
        specs = {"left." + n: s for n, s in self.left.param_specs().items()}
        specs.update({"right." + n: s for n, s in self.right.param_specs().items()})
        if self.combine == "normed":
            specs[self.names["left_norm"]] = TensorSpec((self.hidden,), init="ones")
            specs[self.names["right_norm"]] = TensorSpec((self.hidden,), init="ones")
        return specs

    def load(self, tensors, dtype, device):
        for side, part in (("left.", self.left), ("right.", self.right)):
            part.load({n[len(side):]: t for n, t in tensors.items() if n.startswith(side) and n[len(side):] in part.param_specs()},
                      dtype, device)
        if self.combine == "normed":
            self.w_left = tensors[self.names["left_norm"]].to(device=device, dtype=torch.float32).contiguous()
            self.w_right = tensors[self.names["right_norm"]].to(device=device, dtype=torch.float32).contiguous()

    # --------------------------------------------------------------------- forward
    def forward(self, h, ctx, cache):
        k = ctx.kernels
        st = cache.state
        lf, rf = self.left_floats, self.right_floats
        if (lf or rf) and (st is None or st.shape[1] != lf + rf):
            raise ValueError("pair: the layer's state row does not fit the two mixers")
        left_cache = dataclasses.replace(cache, state=st[:, :lf] if lf else None)
        right_cache = dataclasses.replace(cache, kv=None, block_table=None, state=st[:, lf:lf + rf] if rf else None)
        yl = self.left.forward(h, ctx, left_cache)
        yr = self.right.forward(h, ctx, right_cache)
        return k.pair_combine(k.materialize(yl), k.materialize(yr), self.w_left, self.w_right, self.a, self.b, self.eps)
