"""Typed configuration of the Radalix decoder, read from config.json.

Keys: `architecture` ("Radalix"), `vocab`, `width`, `norm.eps`, `embedding` {`scale`, `bigram` {`buckets`, `mul_prev`,
`mul_cur`}} (no `bigram`: no second table), `logit_softcap` (absent: none) and `layers`, a list whose entries have
`type`, the two mixers' sizes under `mixer.left` / `mixer.right`, and `mlp` (null or {`kind`: `moe`, `expert`: {`ff`},
`router`: {`experts`, `top`}, `shared`: {`ff`} or absent}).

    parallel      left:  heads, kv_heads, dim, vdim, scale and optionally conv (taps), q_temp {coef, every}, rot, mask {size}
                  right: heads, dim, vdim, tau                              (linear attention with a decay per key channel)
    parallel_2    left:  as above, with a learned sink per head and no output gate
                  right: heads, vdim, state, groups, norm_groups, conv      (selective state-space recurrence)
                  and left_scale, right_scale beside them

The design, as the plan states it: the embedding's rows are multiplied by a constant and a row of a second table,
found by a hash of the token before and the token itself, is added.  A layer has two RMS norms of the same stream, one
in front of the mixer and one in front of the feed-forward, and adds both outputs, each multiplied element by element
by a learned vector.  A mixer is a pair of mixers that read the same rows.  In both kinds the left one is grouped-query
attention whose queries, keys and values pass a short causal convolution over time behind their projections; `parallel`
has no rotation but a query multiplier that grows with the position, sees every earlier key and gates its heads'
outputs by a sigmoid of a projection of its input; `parallel_2` turns a part of every head (neighbouring elements pair
up; frequencies may be slowed by wavelength with cos and sin made longer), sees a window of keys and has a learned
number per head in the softmax's denominator.  The right one keeps a matrix of state per head: in `parallel` it
decays per key channel by sigmoid(.)^(1/tau) of a low-rank projection, the heads' outputs are normed, gated and
projected, and the pair's result is half the sum of the two outputs after an RMS norm of each; in `parallel_2` it
decays per head by exp(-exp(A) dt) with dt = softplus(. + bias), takes dt B x^T, is read by C, and the pair's result is
a weighted sum.  The feed-forward is a mixture of gated SiLU experts, weighted by their sigmoid scores divided by the
chosen scores' sum, plus an expert every token uses.  The model's norm, the embedding table as head, and a cap on the
logits.  Tensor names: `embed`, `bigram`, `final.norm`, and per layer i `l<i>.norm1`, `.norm2`, `.ls1`, `.ls2`,
`.mix.left.*`, `.mix.right.*`, `.mix.left.out`, `.mix.right.out`, `.mlp.*`.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from .plan import LayerSpec, ModelPlan, PartSpec, SubPart, default_schedule
from .registry import ConfigError, register_architecture

_TYPES = ("parallel", "parallel_2")
_MLPS = ("moe",)
SIGMOID_WEIGHT_FLOOR = 1e-20        # added to the sum of the chosen scores before the division


def _integer(where: str, raw, key: str, least: int = 1) -> int:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json (Radalix): {where}`{key}` must be an integer, got {v!r}")
    if int(v) < least:
        raise ConfigError(f"config.json (Radalix): {where}`{key}` must be at least {least}, got {v}")
    return int(v)


def _number(where: str, raw, key: str) -> float:
    v = raw.get(key) if isinstance(raw, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json (Radalix): {where}`{key}` must be a number, got {v!r}")
    return float(v)


@register_architecture("Radalix", "radalix")
@dataclass
class RadalixConfig:
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    bigram: Optional[Dict[str, int]] = None
    logit_softcap: Optional[float] = None
    max_positions: int = 1 << 20            # nothing in the design bounds a sequence

    architecture = "Radalix"
    model_type = "radalix"

    @property
    def vocab_size(self) -> int:            # the name generic callers use
        return self.vocab

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "RadalixConfig":
        for key in ("vocab", "width", "layers"):
            if raw.get(key) is None:
                raise ConfigError(f"config.json (Radalix): missing key `{key}`")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json (Radalix): `layers` must be a non-empty list")
        norm = raw.get("norm") or {}
        emb = raw.get("embedding") or {}
        big = emb.get("bigram")
        cfg = cls(
            vocab=_integer("", raw, "vocab"), width=_integer("", raw, "width"), layers=copy.deepcopy(raw["layers"]),
            norm_eps=float(norm.get("eps", 1e-6)),
            embedding_scale=_number("embedding.", emb, "scale") if emb.get("scale") is not None else 1.0,
            bigram=None if not big else {"buckets": _integer("embedding.bigram.", big, "buckets"),
                                         "mul_prev": _integer("embedding.bigram.", big, "mul_prev", least=0),
                                         "mul_cur": _integer("embedding.bigram.", big, "mul_cur", least=0)},
            logit_softcap=_number("", raw, "logit_softcap") if raw.get("logit_softcap") is not None else None,
            max_positions=_integer("", raw, "max_positions") if raw.get("max_positions") is not None else 1 << 20)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if not self.norm_eps > 0:
            raise ConfigError(f"Radalix config: norm.eps must be positive, got {self.norm_eps}")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError(f"Radalix config: logit_softcap must be positive, got {self.logit_softcap}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in _TYPES:
                raise ConfigError(f"Radalix config: {where}type must be one of {_TYPES}, got {kind!r}")
            m = layer.get("mixer")
            if not isinstance(m, dict) or not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                raise ConfigError(f"Radalix config: {where}mixer must have `left` and `right`")
            self._validate_attention(m["left"], where + "mixer.left.")
            r, rw = m["right"], where + "mixer.right."
            if kind == "parallel":
                for key in ("heads", "dim", "vdim"):
                    _integer(rw, r, key)
                if not _number(rw, r, "tau") > 0:
                    raise ConfigError(f"Radalix config: {rw}tau must be positive")
                if r["dim"] > 512:
                    raise ConfigError(f"Radalix config: {rw}dim {r['dim']} is beyond the scan kernel's 512")
            else:
                for key in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
                    _integer(rw, r, key)
                if r["heads"] % r["groups"]:
                    raise ConfigError(f"Radalix config: {rw}heads {r['heads']} are not a multiple of groups {r['groups']}")
                if (r["heads"] * r["vdim"]) % r["norm_groups"]:
                    raise ConfigError(f"Radalix config: {rw}norm_groups {r['norm_groups']} do not cut {r['heads'] * r['vdim']} evenly")
                if r["state"] > 512 or r["conv"] > 16:
                    raise ConfigError(f"Radalix config: {rw}state {r['state']} / conv {r['conv']} are beyond the kernels' 512 / 16")
                _number(where + "mixer.", m, "left_scale")
                _number(where + "mixer.", m, "right_scale")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in _MLPS:
                raise ConfigError(f"Radalix config: {where}mlp.kind must be one of {_MLPS}")
            _integer(where + "mlp.expert.", mlp.get("expert"), "ff")
            rt = mlp.get("router")
            n = _integer(where + "mlp.router.", rt, "experts")
            top = _integer(where + "mlp.router.", rt, "top")
            if not 1 <= top <= n or n > 1024:
                raise ConfigError(f"Radalix config: {where}mlp.router chooses {top} of {n} experts (at most 1024)")
            if mlp.get("shared"):
                _integer(where + "mlp.shared.", mlp["shared"], "ff")

    @staticmethod
    def _validate_attention(m: dict, where: str) -> None:
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _integer(where, m, key)
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"Radalix config: {where}heads {m['heads']} are not a multiple of kv_heads {m['kv_heads']}")
        for key in ("dim", "vdim"):
            if m[key] % 2 or m[key] > 256:
                raise ConfigError(f"Radalix config: {where}{key} {m[key]} must be even and at most 256")
        _number(where, m, "scale")
        if m.get("conv") is not None and _integer(where, m, "conv") > 16:
            raise ConfigError(f"Radalix config: {where}conv {m['conv']} is beyond the kernels' 16 taps")
        if m.get("q_temp"):
            _number(where + "q_temp.", m["q_temp"], "coef")
            _integer(where + "q_temp.", m["q_temp"], "every")
        if m.get("mask"):
            _integer(where + "mask.", m["mask"], "size")
        rot = m.get("rot")
        if rot:
            dims = _integer(where + "rot.", rot, "dims", least=2)
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"Radalix config: {where}rot.dims {dims} must be even and at most dim {m['dim']}")
            if not _number(where + "rot.", rot, "base") > 1:
                raise ConfigError(f"Radalix config: {where}rot.base must be above 1")
            sc = rot.get("scaling")
            if sc:
                vals = {k: _number(where + "rot.scaling.", sc, k) for k in ("factor", "original", "fast", "slow")}
                if not min(vals.values()) > 0:
                    raise ConfigError(f"Radalix config: {where}rot.scaling {sc!r} is not usable")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(self.bigram)
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                             "norm": {"eps": self.norm_eps}, "embedding": emb, "layers": copy.deepcopy(self.layers)}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # --------------------------------------------------------------------- plan
    def _norm_spec(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "tensor_name": name})

    def _attention_spec(self, m: dict, kind: str) -> PartSpec:
        rot = m.get("rot")
        position = None
        if rot:
            sc = rot.get("scaling")
            position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "pairing": "interleaved",
                                         "scaling": None if not sc else {"kind": "ramp", **sc}})
        return PartSpec("attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_head_dim": m["vdim"], "window": None if not m.get("mask") else int(m["mask"]["size"]),
            "scale": float(m["scale"]), "position": position, "qkv_bias": False,
            "sink": "learned" if kind == "parallel_2" else False, "gate": "sigmoid" if kind == "parallel" else None,
            "conv_taps": m.get("conv"), "q_temp": None if not m.get("q_temp") else dict(m["q_temp"]),
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "sink": "sink", "q_conv": "q.conv",
                      "k_conv": "k.conv", "v_conv": "v.conv"}})

    def _mixer_spec(self, i: int) -> PartSpec:
        layer, w = self.layers[i], self.width
        m = layer["mixer"]
        left = self._attention_spec(m["left"], layer["type"])
        r = m["right"]
        if layer["type"] == "parallel":
            right = PartSpec("decayed_linear_attention", {"hidden_size": w, "num_heads": r["heads"], "key_dim": r["dim"],
                                                          "value_dim": r["vdim"], "tau": float(r["tau"]),
                                                          "norm_eps": self.norm_eps})
            return PartSpec("pair", {"hidden_size": w, "left": left, "right": right, "combine": "normed",
                                     "left_weight": 0.5, "right_weight": 0.5, "norm_eps": self.norm_eps,
                                     "names": {"left_norm": "left.out", "right_norm": "right.out"}})
        right = PartSpec("state_space", {"hidden_size": w, "num_heads": r["heads"], "value_dim": r["vdim"],
                                         "state_dim": r["state"], "groups": r["groups"], "norm_groups": r["norm_groups"],
                                         "conv_taps": r["conv"], "norm_eps": self.norm_eps})
        return PartSpec("pair", {"hidden_size": w, "left": left, "right": right, "combine": "plain",
                                 "left_weight": float(m["left_scale"]), "right_weight": float(m["right_scale"])})

    def _ffn_spec(self, mlp: dict) -> PartSpec:
        r = mlp["router"]
        shared = None
        if mlp.get("shared"):
            shared = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp["shared"]["ff"],
                                         "names": {"gate": "shared.gate", "up": "shared.up", "down": "shared.down"}})
        return PartSpec("moe", {"hidden_size": self.width, "expert_size": mlp["expert"]["ff"], "num_experts": r["experts"],
                                "top": r["top"], "activation": "silu_glu", "routing": "sigmoid_normalized",
                                "weight_floor": SIGMOID_WEIGHT_FLOOR, "correction": False, "shared": shared})

    def _layer_spec(self, i: int) -> LayerSpec:
        mlp = self.layers[i].get("mlp")
        parts = {"norm_mixer": SubPart("norm", self._norm_spec("norm1")),
                 "mixer": SubPart("mixer", self._mixer_spec(i), "mix.")}
        if mlp is not None:
            parts["norm_ffn"] = SubPart("norm", self._norm_spec("norm2"))
            parts["ffn"] = SubPart("ffn", self._ffn_spec(mlp), "mlp.")
        block = PartSpec("parallel_norms", {"ffn": mlp is not None, "hidden_size": self.width,
                                            "layer_scale": {"mixer": "ls1", "ffn": "ls2"}})
        return LayerSpec(f"l{i}.", block, parts)

    def to_plan(self) -> ModelPlan:
        layers = [self._layer_spec(i) for i in range(len(self.layers))]
        embedding = {"vocab_size": self.vocab, "hidden_size": self.width, "tensor_name": "embed",
                     "scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = {"tensor_name": "bigram", **self.bigram}
        plan = ModelPlan(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=self.max_positions, embedding=PartSpec("embedding", embedding),
            layers=layers, schedule=default_schedule(len(layers)), final_norm=self._norm_spec("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied": True,
                                         "softcap": self.logit_softcap}),
            final_norm_prefix="", embedding_prefix="", lm_head_prefix="lm_head.")
        plan.validate()
        return plan
