"""Typed configuration of the Benarax decoder, read from config.json.

Keys: `architecture` ("Benarax"), `vocab`, `width`, `norm` {`eps`, `groups`}, `embedding.scale`, `logit_scale`,
`residual_mult`, `canon.taps` (the short convolution in front of the mixer; absent: none), `token_side.dim`
(a per-layer token input; absent: none), `loop` {`start`, `stop`, `times`} (absent: every layer runs once) and
`layers`, a list whose entries have `type`, the mixer's sizes under `mixer`, and `mlp` (null or {`kind`: `moe`,
`expert`: {`ff`, `limit`}, `router`: {`experts`, `top`}}).

    general_delta                       mixer: heads, dim            (the decay's inner size is the shape of `mix.w1`)
    latent_attention, latent_attention_2
                                        mixer: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale,
                                        rot {base, dims, scaling {factor, original, fast, slow}}

The design, as the plan states it: the embedding's rows are multiplied by a constant; a layer has one norm (an RMS
norm over equal consecutive groups of the width) that both sublayers read, the mixer behind a causal depthwise
convolution over time, and adds m * (mixer + feed-forward); then a gated projection of the layer's columns of a
second token table joins the stream through an RMS norm of its own, times m.  The recurrent mixer keeps a matrix
per head that decays per key channel, loses what it holds along the unit key, and gains k v^T.  The attention mixers
make queries through a normed latent and keys and values of all heads from one normed latent per token, with one
rotated key part that all heads share; the two differ in which elements a rotation pairs (neighbours, or the two
halves), and frequencies may be slowed by wavelength with cos and sin made longer.  The feed-forward is a mixture
of clamped gated experts weighted by a softmax over the chosen router outputs.  Layers `start .. stop - 1` run `times`
times in a row with the same weights and a cache and state of their own per run.  The model's norm, a head of its
own, and logits times a constant.  Tensor names: `embed`, `side.embed`, `final.norm`, `head`, and per layer i
`l<i>.norm1`, `.canon1`, `.mix.*`, `.mlp.*`, `.side.gate`, `.side.proj`, `.side.norm`.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry, SubPart
from .registry import ConfigError, register_architecture

_ATTENTIONS = {"latent_attention": "interleaved", "latent_attention_2": "split_half"}     # type -> how a rotation pairs
_TYPES = ("general_delta",) + tuple(_ATTENTIONS)
_MLPS = ("moe",)


def _integer(where: str, raw, key: str, least: int = 1) -> int:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json (Benarax): {where}`{key}` must be an integer, got {v!r}")
    if int(v) < least:
        raise ConfigError(f"config.json (Benarax): {where}`{key}` must be at least {least}, got {v}")
    return int(v)


def _number(where: str, raw, key: str) -> float:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json (Benarax): {where}`{key}` must be a number, got {v!r}")
    return float(v)


@register_architecture("Benarax", "benarax")
@dataclass
class BenaraxConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm_eps: float = 1e-6
    norm_groups: int = 1
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    residual_mult: float = 1.0
    canon_taps: Optional[int] = None
    side_dim: Optional[int] = None
    loop: Optional[Dict[str, int]] = None
    max_positions: int = 1 << 20            # nothing in the design bounds a sequence

    architecture = "Benarax"
    model_type = "benarax"

    @property
    def vocab_size(self) -> int:            # the name generic callers use
        return self.vocab

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "BenaraxConfig":
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                raise ConfigError(f"config.json (Benarax): missing key `{key}`")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json (Benarax): `layers` must be a non-empty list")
        norm = raw.get("norm") or {}
        canon, side, loop = raw.get("canon"), raw.get("token_side"), raw.get("loop")
        emb = raw.get("embedding") or {}
        cfg = cls(
            vocab=_integer("", raw, "vocab"), width=_integer("", raw, "width"), layers=copy.deepcopy(raw["layers"]),
            norm_eps=float(norm.get("eps", 1e-6)),
            norm_groups=_integer("norm.", norm, "groups") if norm.get("groups") is not None else 1,
            embedding_scale=_number("embedding.", emb, "scale") if emb.get("scale") is not None else 1.0,
            logit_scale=_number("", raw, "logit_scale") if raw.get("logit_scale") is not None else 1.0,
            residual_mult=_number("", raw, "residual_mult") if raw.get("residual_mult") is not None else 1.0,
            canon_taps=None if not canon else _integer("canon.", canon, "taps"),
            side_dim=None if not side else _integer("token_side.", side, "dim"),
            loop=None if not loop else {k: _integer("loop.", loop, k, least=0) for k in ("start", "stop", "times")},
            max_positions=_integer("", raw, "max_positions") if raw.get("max_positions") is not None else 1 << 20)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.norm_eps > 0:
            raise ConfigError(f"Benarax config: norm.eps must be positive, got {self.norm_eps}")
        if self.width % self.norm_groups:
            raise ConfigError(f"Benarax config: width {self.width} is not cut evenly by norm.groups {self.norm_groups}")
        if self.canon_taps is not None and self.canon_taps > 16:
            raise ConfigError(f"Benarax config: canon.taps {self.canon_taps} is beyond the kernels' 16")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in _TYPES:
                raise ConfigError(f"Benarax config: {where}type must be one of {_TYPES}, got {kind!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict):
                raise ConfigError(f"Benarax config: {where}mixer is missing")
            _integer(where + "mixer.", m, "heads")
            _integer(where + "mixer.", m, "dim")
            if kind == "general_delta":
                if m["dim"] > 256:
                    raise ConfigError(f"Benarax config: {where}mixer.dim {m['dim']} is beyond the kernel's 256")
            else:
                self._validate_attention(m, where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in _MLPS:
                raise ConfigError(f"Benarax config: {where}mlp.kind must be one of {_MLPS}")
            _integer(where + "mlp.expert.", mlp.get("expert"), "ff")
            if not _number(where + "mlp.expert.", mlp.get("expert"), "limit") > 0:
                raise ConfigError(f"Benarax config: {where}mlp.expert.limit must be positive")
            r = mlp.get("router")
            n = _integer(where + "mlp.router.", r, "experts")
            top = _integer(where + "mlp.router.", r, "top")
            if not 1 <= top <= n or n > 1024:
                raise ConfigError(f"Benarax config: {where}mlp.router chooses {top} of {n} experts (at most 1024)")
        if self.loop is not None:
            lo, hi, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= lo <= hi <= len(self.layers):
                raise ConfigError(f"Benarax config: loop {lo} .. {hi} does not lie inside the {len(self.layers)} layers")
            if hi > lo and times < 1:
                raise ConfigError(f"Benarax config: loop.times must be at least 1, got {times}")

    @staticmethod
    def _validate_attention(m: dict, where: str) -> None:
        for key in ("vdim", "kv_rank", "q_rank"):
            _integer(where, m, key)
        rot_dim = _integer(where, m, "rot_dim", least=0)
        if m["kv_rank"] + rot_dim > 1024:
            raise ConfigError(f"Benarax config: {where}kv_rank + rot_dim {m['kv_rank'] + rot_dim} is beyond the kernels' 1024")
        _number(where, m, "scale")
        rot = m.get("rot")
        if rot_dim and not isinstance(rot, dict):
            raise ConfigError(f"Benarax config: {where}rot is missing")
        if rot_dim:
            dims = _integer(where + "rot.", rot, "dims", least=2)
            if dims % 2 or dims > rot_dim:
                raise ConfigError(f"Benarax config: {where}rot.dims {dims} must be even and at most rot_dim {rot_dim}")
            if not _number(where + "rot.", rot, "base") > 1:
                raise ConfigError(f"Benarax config: {where}rot.base must be above 1")
            sc = rot.get("scaling")
            if sc:
                vals = {k: _number(where + "rot.scaling.", sc, k) for k in ("factor", "original", "fast", "slow")}
                if not (vals["factor"] > 0 and vals["original"] > 0 and vals["fast"] > 0 and vals["slow"] > 0):
                    raise ConfigError(f"Benarax config: {where}rot.scaling {sc!r} is not usable")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                             "residual_mult": self.residual_mult, "layers": copy.deepcopy(self.layers)}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        if self.side_dim is not None:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # --------------------------------------------------------------------- plan
    def run_order(self) -> List[int]:
        """The layers in the order they run."""
        n = len(self.layers)
        if self.loop is None or self.loop["stop"] <= self.loop["start"]:
            return list(range(n))
        lo, hi = self.loop["start"], self.loop["stop"]
        return list(range(lo)) + list(range(lo, hi)) * self.loop["times"] + list(range(hi, n))

    def _norm_spec(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "groups": self.norm_groups,
                                    "tensor_name": name})

    def _mixer_spec(self, i: int) -> PartSpec:
        layer, w = self.layers[i], self.width
        m = layer["mixer"]
        if layer["type"] == "general_delta":
            return PartSpec("delta_rule", {"hidden_size": w, "num_heads": m["heads"], "head_dim": m["dim"],
                                           "decay_rank": m.get("rank"), "norm_eps": self.norm_eps})
        rot = m.get("rot") or {}
        position = None
        if m["rot_dim"]:
            sc = rot.get("scaling")
            position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                         "pairing": _ATTENTIONS[layer["type"]],
                                         "scaling": None if not sc else {"kind": "ramp", **sc}})
        return PartSpec("latent_attention", {
            "hidden_size": w, "num_heads": m["heads"], "qk_dim": m["dim"], "rot_dim": m["rot_dim"], "v_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "window": None, "scale": float(m["scale"]),
            "latent_norm_eps": self.norm_eps, "sink": False, "position": position,
            "names": {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq"}})

    def _ffn_spec(self, mlp: dict) -> PartSpec:
        r = mlp["router"]
        return PartSpec("moe", {"hidden_size": self.width, "expert_size": mlp["expert"]["ff"], "num_experts": r["experts"],
                                "top": r["top"], "activation": "clamped_glu", "limit": float(mlp["expert"]["limit"]),
                                "routing": "softmax_of_chosen", "correction": False})

    def _layer_spec(self, i: int) -> LayerSpec:
        mlp = self.layers[i].get("mlp")
        parts = {"norm": SubPart("norm", self._norm_spec("norm1")),
                 "mixer": SubPart("mixer", self._mixer_spec(i), "mix.")}
        if mlp is not None:
            parts["ffn"] = SubPart("ffn", self._ffn_spec(mlp), "mlp.")
        if self.canon_taps is not None:
            parts["conv"] = SubPart("conv", PartSpec("causal_depthwise", {"channels": self.width, "taps": self.canon_taps,
                                                                           "tensor_name": "canon1"}))
        if self.side_dim is not None:
            parts["side"] = SubPart("token_input", PartSpec("gated_table", {
                "hidden_size": self.width, "dim": self.side_dim, "first_column": i * self.side_dim, "eps": self.norm_eps,
                "scale": self.residual_mult}), "side.")
        block = PartSpec("parallel", {"ffn": mlp is not None, "conv": self.canon_taps is not None,
                                      "side": self.side_dim is not None, "residual_mult": self.residual_mult})
        return LayerSpec(f"l{i}.", block, parts)

    def to_plan(self) -> ModelPlan:
        layers = [self._layer_spec(i) for i in range(len(self.layers))]
        seen: Dict[int, int] = {}
        schedule: List[ScheduleEntry] = []
        for i in self.run_order():                          # every run has a cache and state of its own
            schedule.append(ScheduleEntry(layer=i, cache=len(schedule), repeat=seen.get(i, 0)))
            seen[i] = seen.get(i, 0) + 1
        embedding = {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_name": "embed",
                     "scale": self.embedding_scale}
        if self.side_dim is not None:
            embedding["side_table"] = {"tensor_name": "side.embed", "width": len(self.layers) * self.side_dim}
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=self.max_positions, embedding=PartSpec("embedding", embedding),
            layers=layers, schedule=schedule, final_norm=self._norm_spec("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": False,
                                         "tensor_name": "head", "scale": self.logit_scale}),
            final_norm_prefix="", embedding_prefix="", lm_head_prefix="")
        plan.validate()
        return plan
