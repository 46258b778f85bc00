"""Token embedding and LM head.

x0[t] = E[token[t]] with no scaling (runtime/backends/cuda/native/
cuda_kernels.cu:256-270, 675-689: the residual stream is float32).  The head is
lm_head.weight, or the embedding table when the model ties them
(runtime/backends/cuda/native/weight_map.cpp:33-37); here the configuration's
tie_word_embeddings decides, and logits are produced in float32 for whichever rows
the step asks for.
"""
from __future__ import annotations

import torch

from ..weights.loader import TensorSpec
from .base import Part, StateSpec, register_part


@register_part("embedding", "embedding")
class Embedding(Part):
    """params: vocab_size, hidden_size, tensor_name (default `weight`), norm (None, or {tensor_name, eps}:
    the gathered rows are RMS-normed with that weight, in float32, before they become the residual stream),
    scale (default 1: the gathered rows are multiplied by it, in float32), side_table (None, or {tensor_name, width}:
    a second table [vocab, width] whose rows layers read by token id; a step finds it in `ctx.side_table`),
    bigram (None, or {tensor_name, buckets, mul_prev, mul_cur}: a table [buckets + 1, hidden] of which row
    (token before * mul_prev + token * mul_cur) mod buckets is added, the last row for a sequence's first token; the
    token before a step's first one is the request's state, `ctx.embedding_state`, int32 [slots, 1])."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tensor_name = str(spec.params.get("tensor_name", "weight"))
        norm = spec.params.get("norm")
        self.norm_name = None if not norm else str(norm.get("tensor_name", "norm.weight"))
        self.norm_eps = float(norm["eps"]) if norm else 0.0
        self.scale = float(spec.params.get("scale", 1.0))
        side = spec.params.get("side_table")
        self.side_name = None if not side else str(side["tensor_name"])
        self.side_width = int(side["width"]) if side else 0
        big = spec.params.get("bigram")
        self.bigram = None if not big else {"tensor_name": str(big.get("tensor_name", "bigram")), "buckets": int(big["buckets"]),
                                            "mul_prev": int(big["mul_prev"]), "mul_cur": int(big["mul_cur"])}
        if self.bigram is not None and (self.bigram["buckets"] < 1 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0
                                        or (self.vocab - 1) * (self.bigram["mul_prev"] + self.bigram["mul_cur"]) >= 1 << 62):
            raise ValueError(f"embedding: bad bigram hash {big!r}")
        self.table = self.norm_weight = self.side_table = self.bigram_table = None

    def state_spec(self):
        """The last token of a request, for the hash of the next step's first token."""
        return None if self.bigram is None else StateSpec((1,), torch.int32)

    def param_specs(self):
        specs = {self.tensor_name: TensorSpec((self.vocab, self.hidden))}
        if self.bigram is not None:
            specs[self.bigram["tensor_name"]] = TensorSpec((self.bigram["buckets"] + 1, self.hidden))
        if self.side_name is not None:
            specs[self.side_name] = TensorSpec((self.vocab, self.side_width))
        if self.norm_name is not None:
            specs[self.norm_name] = TensorSpec((self.hidden,), init="ones")
        return specs

    def load(self, tensors, dtype, device):
        self.table = tensors[self.tensor_name].to(device=device, dtype=dtype).contiguous()
        if self.norm_name is not None:
            self.norm_weight = tensors[self.norm_name].to(device=device, dtype=torch.float32).contiguous()
        if self.side_name is not None:
            self.side_table = tensors[self.side_name].to(device=device, dtype=dtype).contiguous()
        if self.bigram is not None:
            self.bigram_table = tensors[self.bigram["tensor_name"]].to(device=device, dtype=dtype).contiguous()

    def forward(self, ctx):
        ctx.side_table = self.side_table
        if self.scale != 1.0:
            x = ctx.kernels.embed(self.table, ctx.token_ids, self.vocab, scale=self.scale)
        else:
            x = ctx.kernels.embed(self.table, ctx.token_ids, self.vocab)
        if self.bigram is not None:
            b = self.bigram
            ctx.kernels.bigram_add(x, self.bigram_table, ctx.token_ids, ctx.embedding_state, b["mul_prev"], b["mul_cur"],
                                   b["buckets"], self.vocab, ctx)
        if self.norm_weight is not None:
            x = ctx.kernels.rmsnorm(x, self.norm_weight, self.norm_eps, torch.float32)
        return x


@register_part("lm_head", "lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied, softcap (None, or c: logits become c tanh(logits / c)),
    scale (default 1: the float32 logits are multiplied by it), tensor_name (default `weight`)."""

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        cap = spec.params.get("softcap")
        self.softcap = None if cap is None else float(cap)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"lm_head: softcap must be positive, got {self.softcap}")
        self.scale = float(spec.params.get("scale", 1.0))
        self.tensor_name = str(spec.params.get("tensor_name", "weight"))
        self.weight = None

    def param_specs(self):
        return {self.tensor_name: TensorSpec((self.vocab, self.hidden), ignored=self.tied)}

    def load(self, tensors, dtype, device, tied_table=None):
        if self.tied:
            if tied_table is None:
                raise ValueError("lm_head: tied head needs the embedding table")
            self.weight = tied_table
        else:
            self.weight = tensors[self.tensor_name].to(device=device, dtype=dtype).contiguous()

    def forward(self, h, ctx):
        """h: normed rows [R, hidden] -> float32 logits [R, vocab]."""
        logits = ctx.kernels.linear(h, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            ctx.kernels.scale_(logits, self.scale)
        if self.softcap is not None:
            ctx.kernels.softcap(logits, self.softcap)
        return logits
