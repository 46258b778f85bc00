"""Small Radalix models for the tests: configurations that differ in every size and option, random weights made sharp,
and the plain implementation's logits for a set of requests."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import plain_radalix


def _moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _left(heads, kv_heads, dim, vdim, scale, conv=None, q_temp=None, mask=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = rot
    return m


def _gated(left, heads, dim, vdim, tau, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}, "mlp": mlp}


def _ssm(left, heads, vdim, state, groups, norm_groups, conv, mlp, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel_2", "mixer": {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                                            "right": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                                      "norm_groups": norm_groups, "conv": conv}}, "mlp": mlp}


def configs():
    """name -> (config.json as a dict, page size).  Between them: both layer kinds in every order; grouped, ungrouped and
    single key heads; values longer and shorter than keys; convolutions of 1 to 5 taps and none; query multipliers that
    change every 1, 5 and 9 positions and none; windows of 1, below, at and above a page and longer than any prompt;
    rotation of a part and of the whole head, with and without slowed frequencies; recurrent heads whose key and value
    sizes are no multiples of anything; state-space groups of one head, several and all; norms over 1, 2 and 3 parts;
    routers choosing one, some and all, of one expert and several, with and without the expert every token uses; a layer
    without feed-forward; with and without the second embedding table (also one of so few rows that rows are shared),
    with and without a cap on the logits."""
    ramp = {"factor": 4.0, "original": 40, "fast": 4.0, "slow": 1.0}
    a = {"architecture": "Radalix", "vocab": 300, "width": 64, "norm": {"eps": 1e-6}, "logit_softcap": 12.0,
         "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 11}}, "layers": [
             _gated(_left(4, 2, 16, 8, 0.3, conv=3, q_temp=(0.4, 5)), 3, 8, 16, 4.0, _moe(24, 5, 2, shared=40)),
             _ssm(_left(2, 1, 8, 16, 0.5, conv=2, mask=7, rot={"base": 100.0, "dims": 4, "scaling": ramp}), 4, 8, 12, 2, 2, 3,
                  _moe(16, 3, 1), left_scale=0.9, right_scale=1.3),
             _ssm(_left(3, 3, 12, 12, 0.4, conv=4, mask=21, rot={"base": 50.0, "dims": 12}), 2, 24, 8, 1, 1, 2, None,
                  left_scale=1.1, right_scale=0.7),
             _gated(_left(1, 1, 32, 32, 0.2), 1, 24, 8, 1.0, _moe(8, 4, 4, shared=8))]}
    b = {"architecture": "Radalix", "vocab": 257, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": [
             _ssm(_left(6, 2, 8, 8, 0.6, conv=1, mask=1, rot={"base": 30.0, "dims": 2}), 6, 16, 16, 6, 3, 1, _moe(32, 4, 2)),
             _gated(_left(2, 2, 24, 48, 0.25, conv=5, q_temp=(1.5, 9)), 4, 16, 24, 16.0, None),
             _ssm(_left(4, 1, 16, 24, 0.35, conv=2, mask=200, rot={"base": 1000.0, "dims": 8,
                                                                  "scaling": {"factor": 8.0, "original": 24, "fast": 3.0, "slow": 0.5}}),
                  3, 32, 24, 3, 1, 4, _moe(16, 7, 3, shared=24), left_scale=0.5, right_scale=2.0)]}
    c = {"architecture": "Radalix", "vocab": 190, "width": 48, "norm": {"eps": 3e-4}, "logit_softcap": 50.0,
         "embedding": {"scale": 0.7, "bigram": {"buckets": 7, "mul_prev": 0, "mul_cur": 3}}, "layers": [
             _gated(_left(5, 1, 6, 10, 0.7, conv=2, q_temp=(0.8, 1)), 5, 6, 10, 2.5, _moe(20, 1, 1)),
             _gated(_left(2, 2, 14, 6, 0.45, conv=3), 2, 20, 14, 7.0, _moe(12, 6, 6, shared=10)),
             _ssm(_left(3, 1, 10, 14, 0.5, conv=3, mask=16, rot={"base": 20.0, "dims": 6,
                                                                "scaling": {"factor": 2.0, "original": 16, "fast": 2.0, "slow": 1.0}}),
                  5, 6, 5, 1, 5, 3, _moe(24, 2, 1, shared=6), left_scale=1.4, right_scale=0.6)]}
    return {"A": (a, 8), "B": (b, 4), "C": (c, 16)}


def medium_config():
    """A model of a few hundred columns whose prompts are long enough for the kernels of many rows: attention heads of 64
    and 128 with equal key and value sizes (the tiled attention kernels) on pages of 16, a window of 100, experts with more
    than 512 (token, choice) pairs a step, recurrent heads of 32 to 128 key channels."""
    ramp = {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 1.0}
    return {"architecture": "Radalix", "vocab": 700, "width": 320, "norm": {"eps": 1e-6}, "logit_softcap": 25.0,
            "embedding": {"scale": 4.0, "bigram": {"buckets": 509, "mul_prev": 13, "mul_cur": 5}}, "layers": [
                _gated(_left(4, 2, 64, 64, 0.2, conv=3, q_temp=(0.3, 64)), 3, 64, 32, 8.0, _moe(96, 8, 3, shared=128)),
                _ssm(_left(4, 1, 128, 128, 0.12, conv=4, mask=100, rot={"base": 10000.0, "dims": 32, "scaling": ramp}),
                     6, 48, 40, 2, 2, 4, _moe(64, 6, 2), left_scale=1.2, right_scale=0.9),
                _gated(_left(6, 3, 32, 64, 0.25, conv=2), 2, 128, 64, 16.0, None),
                _ssm(_left(8, 4, 64, 64, 0.15, conv=4, mask=33, rot={"base": 500.0, "dims": 64}), 4, 64, 128, 1, 4, 2,
                     _moe(96, 8, 3, shared=64))]}, 16


def write_model(raw, out_dir, seed):
    """Random weights for `raw`, then made sharp: the queries' and keys' projections are large so that attention is
    peaked, both embedding tables so that tokens and pairs of tokens differ, norm weights and the layers' output vectors
    are spread, the convolutions' taps are not small, decays spread from slow to fast, step sizes from small to large,
    sinks from negligible to dominant, and the router's scores are spread without reaching one."""
    from inferflux_b200.config import config_from_dict
    from inferflux_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    cfg = config_from_dict(raw)
    write_random_model(cfg, out_dir, seed=seed, dtype=torch.float32, std=0.08, norm_jitter=0.2)
    path = Path(out_dir) / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith(".left.q") or n.endswith(".left.k"):
            tensors[n] = t * 5.0
        elif n in ("embed", "bigram"):
            tensors[n] = t * 6.0
        elif n.endswith(".conv") and t.dim() == 2:
            tensors[n] = 0.6 * torch.randn(t.shape, generator=g)
        elif n.endswith(".conv.b"):
            tensors[n] = 0.3 * torch.randn(t.shape, generator=g)
        elif n.endswith(".right.a2.b"):
            tensors[n] = 1.0 + 2.0 * torch.randn(t.shape, generator=g)
        elif n.endswith(".right.a1") or n.endswith(".right.a2"):
            tensors[n] = t * 6.0
        elif n.endswith(".right.dt_bias"):
            tensors[n] = 1.5 * torch.randn(t.shape, generator=g)
        elif n.endswith(".right.A_log"):
            tensors[n] = torch.rand(t.shape, generator=g) * 2.5 - 1.0
        elif n.endswith(".right.D"):
            tensors[n] = torch.randn(t.shape, generator=g)
        elif n.endswith(".right.in") or n.endswith(".right.k") or n.endswith(".right.q"):
            tensors[n] = t * 3.0
        elif n.endswith(".left.sink"):
            tensors[n] = 2.0 * torch.randn(t.shape, generator=g)
        elif n.endswith(".ls1") or n.endswith(".ls2"):
            tensors[n] = 0.5 + torch.rand(t.shape, generator=g)
        elif n.endswith(".mlp.router"):
            tensors[n] = t * 1.5                           # sigmoid scores must stay apart: far-out logits all round to one
        elif ".mlp.e" in n or ".mlp.shared." in n:
            tensors[n] = t * 3.0
    write_safetensors(path, tensors, metadata={"format": "pt"})
    (Path(out_dir) / "config.json").write_text(json.dumps(raw, indent=1))
    return Path(out_dir)


def load(model_dir):
    return plain_radalix.load_model_dir(model_dir)


def plain_logits(model_dir, requests, weights_as=None, dtype=torch.float64):
    raw, W = load(model_dir)
    if weights_as is not None:
        W = {k: (v.to(weights_as) if v.is_floating_point() else v) for k, v in W.items()}
    return {rid: plain_radalix.forward(raw, W, toks, dtype=dtype).double().numpy() for rid, toks in requests.items()}


def requests_for(raw, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
