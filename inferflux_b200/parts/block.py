"""Pre-norm residual block: x += mixer(norm(x)); x += ffn(norm(x))
(runtime/backends/cuda/native/llama_forward.h:88-90).  The block hands its last
delta on unadded, so that whatever normalises next adds it in the same kernel
(runtime/backends/cuda/native/transformer_forward.cu:2203-2211, 2564-2586)."""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..weights.loader import TensorSpec
from .base import Block, NormedDelta, StateSpec, StreamMerge, VectorScaledDelta, register_part, settle_pending
from .norm import RMSNorm


@register_part("block", "prenorm")
class PreNormBlock(Block):
    sub_parts = {"norm_mixer": "norm", "mixer": "mixer", "norm_ffn": "norm", "ffn": "ffn"}

    def forward(self, x, pending, ctx, cache):
        if isinstance(pending, NormedDelta):                         # the layer before norms its output itself
            pending.add_to(x, ctx)
            pending = None
        fused = getattr(ctx.kernels, "fused_prenorm_layer", None)    # a kernel table may run the whole layer itself
        if fused is not None:
            done = fused(self, x, pending, ctx, cache)
            if done is not None:
                return done
        h = self.norm_mixer.forward(x, pending, ctx, lazy=self.mixer.takes_scaled_rows)   # x += pending; h = norm(x)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norm_ffn.forward(x, a, ctx, lazy=self.ffn.takes_scaled_rows)             # x += a; h = norm(x)
        f = self.ffn.forward(h, ctx)
        return x, f


class _StoresForBlock:
    """What a layer stores when its block keeps state of its own beside the mixer's cache."""

    def __init__(self, mixer, state: Optional[StateSpec]):
        self.mixer, self.state = mixer, state

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.state


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """Norms on both sides of every sublayer, and optionally a short convolution over time in front of it:

        x += norm_b(mixer(conv(norm_a(x))));   x += norm_d(ffn(conv(norm_c(x))))

    params: ffn (False: the layer ends after the mixer), conv (False: no convolutions).  Parts, as far as
    present: norm_mixer, conv_mixer, mixer, postnorm_mixer, norm_ffn, conv_ffn, ffn, postnorm_ffn.  The
    convolutions' inputs of the last few tokens are the layer's state, [convolutions, rows, width] per request.
    A sublayer's output is handed on unadded with its norm (`NormedDelta`), so that sum, that norm and the
    next one run as one kernel."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        self.has_conv = bool(spec.params.get("conv", True))
        names = {"norm_mixer": "norm", "mixer": "mixer", "postnorm_mixer": "norm"}
        if self.has_ffn:
            names.update({"norm_ffn": "norm", "ffn": "ffn", "postnorm_ffn": "norm"})
        if self.has_conv:
            names["conv_mixer"] = "conv"
            if self.has_ffn:
                names["conv_ffn"] = "conv"
        self.sub_parts = names
        super().__init__(spec, parts)
        for name, role in names.items():
            if role == "norm" and not isinstance(parts[name], RMSNorm):
                raise ValueError(f"sandwich block: {name} must be an RMS norm (its weight and eps go into fused kernels)")
        self.convs = [parts[n] for n in ("conv_mixer", "conv_ffn") if n in parts]
        rows = {c.state_rows for c in self.convs}
        if len(rows) > 1:
            raise ValueError("sandwich block: the layer's convolutions must keep the same number of inputs")
        self.state_rows = rows.pop() if rows else None

    def cache_part(self):
        if self.mixer.state_spec() is not None and self.state_rows:
            raise ValueError("sandwich block: a mixer with state of its own beside convolutions is not built")
        if not self.state_rows:
            return self.mixer
        width = self.convs[0].channels
        return _StoresForBlock(self.mixer, StateSpec((len(self.convs), self.state_rows, width), torch.float32))

    def _sublayer_input(self, x, pending, norm, conv, index, ctx, cache):
        k = ctx.kernels
        if isinstance(pending, NormedDelta):
            if conv is not None and ctx.max_span == 1 and getattr(k, "fuses_single_token_conv", False):
                # decoded tokens only: sum, both norms and the convolution (its history is all state) in one kernel
                return k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype,
                                      conv=(conv.weight, conv.taps, cache.state, index, ctx))
            h = k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype)
        else:
            h = norm.forward(x, pending, ctx)
        return conv.forward(h, ctx, cache.state, index) if conv is not None else h

    def forward(self, x, pending, ctx, cache):
        conv = self.parts.get("conv_mixer")
        h = self._sublayer_input(x, pending, self.norm_mixer, conv, 0, ctx, cache)
        y = self.mixer.forward(h, ctx, cache)
        pending = NormedDelta(y, self.postnorm_mixer.weight, self.postnorm_mixer.eps)
        if not self.has_ffn:
            return x, pending
        h = self._sublayer_input(x, pending, self.norm_ffn, self.parts.get("conv_ffn"), 1, ctx, cache)
        y = self.ffn.forward(h, ctx)
        return x, NormedDelta(y, self.postnorm_ffn.weight, self.postnorm_ffn.eps)


@register_part("block", "postnorm")
class PostNormBlock(Block):
    """A norm on each sublayer's output only; the sublayers read the residual stream itself:

        x += norm_a(mixer(x));   x += norm_b(ffn(x))

    params: ffn (False: the layer ends after the mixer).  Parts: mixer, postnorm_mixer and, with a feed-forward,
    ffn, postnorm_ffn.  A sublayer's output travels unadded with its norm (`NormedDelta`); the sum, that norm
    and the rounding of x to the run's dtype for the next sublayer are one kernel.  A sublayer that sets
    `takes_stream` gets the float32 rows themselves."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        names = {"mixer": "mixer", "postnorm_mixer": "norm"}
        if self.has_ffn:
            names.update({"ffn": "ffn", "postnorm_ffn": "norm"})
        self.sub_parts = names
        super().__init__(spec, parts)
        for name, role in names.items():
            if role == "norm" and not isinstance(parts[name], RMSNorm):
                raise ValueError(f"postnorm block: {name} must be an RMS norm (its weight and eps go into a fused kernel)")

    @staticmethod
    def _sublayer_input(x, pending, reader, ctx):
        """Settle what is pending and give the reader its rows."""
        k = ctx.kernels
        as_stream = reader.takes_stream or ctx.dtype == torch.float32
        if isinstance(pending, NormedDelta):
            if as_stream:
                pending.add_to(x, ctx)
                return x
            return k.postnorm_add(x, pending.y, pending.weight, pending.eps, out_dtype=ctx.dtype, cast_out=True)
        settle_pending(x, pending, ctx)
        return x if as_stream else k.cast_rows(x, ctx.dtype)

    def forward(self, x, pending, ctx, cache):
        h = self._sublayer_input(x, pending, self.mixer, ctx)
        y = self.mixer.forward(h, ctx, cache)
        pending = NormedDelta(y, self.postnorm_mixer.weight, self.postnorm_mixer.eps)
        if not self.has_ffn:
            return x, pending
        h = self._sublayer_input(x, pending, self.ffn, ctx)
        y = self.ffn.forward(h, ctx)
        return x, NormedDelta(y, self.postnorm_ffn.weight, self.postnorm_ffn.eps)


@register_part("block", "parallel")
class ParallelBlock(Block):
    """One norm that both sublayers read, their outputs added together, then optionally a token input:

        h = norm(x);   x += m * (mixer(h + conv(h)) + ffn(h));   x += side(x)

    params: ffn, conv, side (whether the layer has each; defaults True, False, False), residual_mult (m, default 1).
    Parts, as far as present: norm, conv, mixer, ffn, side.  The convolution's inputs of the last few tokens and
    the mixer's own state share the layer's state row per request: [convolution rows, then the mixer's].  What the
    token input returns travels unadded (`pending`), so that its sum, its norm and the next layer's norm are one
    kernel; in steps of single tokens that kernel does the convolution too and hands back both h and h + conv(h)."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        self.has_conv = bool(spec.params.get("conv", False))
        self.has_side = bool(spec.params.get("side", False))
        self.mult = float(spec.params.get("residual_mult", 1.0))
        names = {"norm": "norm", "mixer": "mixer"}
        if self.has_ffn:
            names["ffn"] = "ffn"
        if self.has_conv:
            names["conv"] = "conv"
        if self.has_side:
            names["side"] = "token_input"
        self.sub_parts = names
        super().__init__(spec, parts)
        if not isinstance(self.norm, RMSNorm):
            raise ValueError("parallel block: norm must be an RMS norm (its weight and eps go into a fused kernel)")
        conv = parts.get("conv")
        self.conv_floats = (conv.state_rows or 0) * conv.channels if conv is not None else 0

    def cache_part(self):
        own = self.mixer.state_spec()
        if own is not None and own.dtype != torch.float32:
            raise ValueError("parallel block: the mixer's state must be float32 to share the layer's state row")
        if not self.conv_floats:
            return self.mixer
        size = 1
        for d in (own.shape if own is not None else (0,)):
            size *= int(d)
        return _StoresForBlock(self.mixer, StateSpec((self.conv_floats + (size if own is not None else 0),), torch.float32))

    def _views(self, cache):
        """(the convolution's state [slots, 1, rows, width], the cache as the mixer sees it)."""
        if not self.conv_floats or cache.state is None:
            return None, cache
        conv = self.conv
        conv_state = cache.state[:, :self.conv_floats].unflatten(1, (1, conv.state_rows, conv.channels))
        rest = cache.state[:, self.conv_floats:] if cache.state.shape[1] > self.conv_floats else None
        return conv_state, dataclasses.replace(cache, state=rest)

    def forward(self, x, pending, ctx, cache):
        k = ctx.kernels
        conv = self.parts.get("conv")
        conv_state, mixer_cache = self._views(cache)
        norm = self.norm
        hc = None
        if isinstance(pending, NormedDelta):
            if conv is not None and ctx.max_span == 1 and getattr(k, "fuses_single_token_conv", False):
                # decoded tokens only: sum, both norms and the convolution (its history is all state) in one kernel
                h, hc = k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype,
                                       conv=(conv.weight, conv.taps, conv_state, 0, ctx), groups=norm.groups, both=True)
            else:
                h = k.postnorm_add(x, pending.y, pending.weight, pending.eps, norm.weight, norm.eps, ctx.dtype,
                                   groups=norm.groups)
        else:
            h = norm.forward(x, pending, ctx)
        if hc is None:
            hc = conv.forward(h, ctx, conv_state, 0) if conv is not None else h
        y = self.mixer.forward(hc, ctx, mixer_cache)
        f = self.ffn.forward(h, ctx) if self.has_ffn else None
        if not self.has_side:
            k.residual_add_scaled(x, y, f, self.mult)
            return x, None
        rows = k.residual_add_scaled(x, y, f, self.mult, out_dtype=ctx.dtype)      # x in the run's dtype, for the gate
        return x, self.side.forward(x, ctx, rows=rows)


@register_part("block", "parallel_norms")
class ParallelNormsBlock(Block):
    """Two norms of the same stream, one in front of each sublayer, and both outputs added at once, each multiplied
    element by element by a learned vector of the block's own:

        x += s_m * mixer(norm_m(x)) + s_f * ffn(norm_f(x))

    params: ffn (False: the layer has a mixer only), hidden_size, layer_scale (None: no vectors; or tensor names
    {mixer, ffn}).  Parts: norm_mixer, mixer and, with a feed-forward, norm_ffn, ffn.  A feed-forward may hand back two
    outputs (a pair: a mixture's and a shared expert's); the sum takes both.  The sum travels unadded (`pending`), so that
    the next layer of this kind adds it in the kernel that makes its two norms."""

    def __init__(self, spec, parts):
        self.has_ffn = bool(spec.params.get("ffn", True))
        names = {"norm_mixer": "norm", "mixer": "mixer"}
        if self.has_ffn:
            names.update({"norm_ffn": "norm", "ffn": "ffn"})
        self.sub_parts = names
        super().__init__(spec, parts)
        self.hidden = int(spec.params["hidden_size"])
        self.scale_names = spec.params.get("layer_scale") or None
        self.s_mixer = self.s_ffn = None

    def param_specs(self):
        if not self.scale_names:
            return {}
        specs = {self.scale_names["mixer"]: TensorSpec((self.hidden,), init="ones")}
        if self.has_ffn:
            specs[self.scale_names["ffn"]] = TensorSpec((self.hidden,), init="ones")
        return specs

    def load(self, tensors, dtype, device):
        if not self.scale_names:
            return
        self.s_mixer = tensors[self.scale_names["mixer"]].to(device=device, dtype=torch.float32).contiguous()
        if self.has_ffn:
            self.s_ffn = tensors[self.scale_names["ffn"]].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, pending, ctx, cache):
        k = ctx.kernels
        if self.has_ffn:
            if isinstance(pending, VectorScaledDelta):
                h_m, h_f = k.rmsnorm_pair(x, self.norm_mixer.weight, self.norm_mixer.eps, self.norm_ffn.weight,
                                          self.norm_ffn.eps, ctx.dtype, vectors=pending)
            else:
                h_m, h_f = k.rmsnorm_pair(x, self.norm_mixer.weight, self.norm_mixer.eps, self.norm_ffn.weight,
                                          self.norm_ffn.eps, ctx.dtype, delta=_settled(x, pending, ctx))
        else:
            h_m, h_f = self.norm_mixer.forward(x, _settled(x, pending, ctx), ctx), None
        y = self.mixer.forward(h_m, ctx, cache)
        f = self.ffn.forward(h_f, ctx) if self.has_ffn else None
        f, f2 = f if isinstance(f, tuple) else (f, None)
        return x, VectorScaledDelta(y, self.s_mixer, f, self.s_ffn, f2)


def _settled(x, pending, ctx):
    """What is left to add inside the next norm kernel: a plain delta is; one with a norm or vectors of its own is added here."""
    if isinstance(pending, (NormedDelta, VectorScaledDelta)):
        pending.add_to(x, ctx)
        return None
    return pending


@register_part("merge", "linear_reinject")
class LinearReinject(StreamMerge):
    """x' = W [x; x0] + step[repeat]: the stream and the embedding output side by side through one matrix
    [width, 2 width] (x first), plus a learned vector per run.  The product takes its inputs in the run's
    dtype; its result and the sum stay float32, as the residual stream is.
    params: width, times, names (tensor names of `in`, `step`)."""

    _NAMES = {"in": "in", "step": "step"}

    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.times = int(spec.params["times"])
        self.names = dict(self._NAMES)
        self.names.update(spec.params.get("names") or {})
        self.w_in = self.steps = None

    def param_specs(self):
        return {self.names["in"]: TensorSpec((self.width, 2 * self.width)),
                self.names["step"]: TensorSpec((self.times, self.width))}

    def load(self, tensors, dtype, device):
        self.w_in = tensors[self.names["in"]].to(device=device, dtype=dtype).contiguous()
        self.steps = tensors[self.names["step"]].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, x0, repeat, ctx):
        if not 0 <= repeat < self.times:
            raise ValueError(f"linear_reinject: run {repeat} of {self.times}")
        k = ctx.kernels
        both = k.concat_cast(x, x0, ctx.dtype)                                  # [T, 2 width]
        return k.linear(both, self.w_in, bias=self.steps[repeat], out_dtype=torch.float32)


@register_part("block", "reinject")
class ReinjectBlock(Block):
    """Not a layer of sublayers: replaces the residual stream by a merge of it with the embedding output
    (`ctx.embedding_output`); which run of a looped stretch this is comes from the schedule entry
    (`ctx.entry.repeat`).  Stores nothing."""

    sub_parts = {"merge": "merge"}

    def cache_part(self):
        return None

    def forward(self, x, pending, ctx, cache):
        settle_pending(x, pending, ctx)
        return self.merge.forward(x, ctx.embedding_output, ctx.entry.repeat, ctx), None
