"""Small Benarax models for the tests: configurations that differ in every size and option, random
weights made sharp, and the plain implementation's logits for a set of requests."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from plain import plain_benarax


def _moe(ff, experts, top, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _delta(heads, dim, mlp):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def _latent(kind, heads, dim, rot_dim, vdim, kv_rank, q_rank, mlp, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                                    "q_rank": q_rank, "scale": scale, "rot": rot}, "mlp": mlp}


def configs():
    """name -> (config.json as a dict, page size).  Between them: norms over 1, 2, 3 and 5 groups; convolutions of 2, 3
    and 4 taps and none; token side inputs of 5, 8 and 16 columns and none; loops in the middle, at the start, at the
    end, run once, and none; both pairings of rotated elements, with and without slowed frequencies (ramps that leave
    some frequencies alone, blend some and slow some); one head and several; values longer and shorter than keys;
    latents smaller and larger than a head, no multiple of 16; rotated parts longer than the plain part; recurrent
    heads whose product is below, equal to and above the width; layers without feed-forward; routers choosing one,
    some and all; multipliers that are 1 and that are not; and one model (F) in which no size is a multiple of 8, the
    convolution has one tap, a router has one expert and the whole model is the loop."""
    ramp = {"factor": 4.0, "original": 40, "fast": 4.0, "slow": 1.0}
    a = {"architecture": "Benarax", "vocab": 300, "width": 64, "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 3},
         "embedding": {"scale": 2.0}, "logit_scale": 0.5, "residual_mult": 0.5, "token_side": {"dim": 8},
         "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
             _latent("latent_attention", 4, 16, 8, 24, 24, 40, _moe(40, 5, 2), 0.9, base=100.0, scaling=ramp),
             _delta(2, 16, _moe(24, 3, 1)),
             _latent("latent_attention_2", 2, 8, 16, 8, 40, 16, _moe(40, 5, 2), 1.2, base=500.0),
             _delta(3, 24, None)]}
    b = {"architecture": "Benarax", "vocab": 257, "width": 96, "norm": {"eps": 1e-5, "groups": 1}, "canon": {"taps": 2},
         "embedding": {"scale": 1.0}, "logit_scale": 1.0, "residual_mult": 1.0,
         "loop": {"start": 0, "stop": 2, "times": 3}, "layers": [
             _delta(3, 32, _moe(32, 4, 4, limit=0.7)),
             _latent("latent_attention_2", 6, 8, 8, 16, 24, 40, _moe(16, 7, 3), 1.5, base=50.0,
                     scaling={"factor": 8.0, "original": 24, "fast": 3.0, "slow": 0.5}),
             _latent("latent_attention", 3, 24, 4, 8, 40, 16, None, 0.6)]}
    c = {"architecture": "Benarax", "vocab": 190, "width": 48, "norm": {"eps": 3e-4, "groups": 3},
         "embedding": {"scale": 0.7}, "logit_scale": 2.0, "residual_mult": 0.8, "token_side": {"dim": 5}, "layers": [
             _latent("latent_attention_2", 1, 16, 32, 16, 8, 12, _moe(24, 2, 1), 0.7, base=3000.0),
             _delta(8, 8, _moe(16, 6, 6, limit=3.0)),
             _latent("latent_attention", 5, 8, 6, 40, 20, 28, None, 1.1, base=20.0,
                     scaling={"factor": 2.0, "original": 16, "fast": 2.0, "slow": 1.0})]}
    d = {"architecture": "Benarax", "vocab": 128, "width": 80, "norm": {"eps": 1e-6, "groups": 5}, "canon": {"taps": 4},
         "embedding": {"scale": 1.5}, "logit_scale": 0.3, "residual_mult": 0.4, "token_side": {"dim": 16},
         "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
             _delta(2, 40, _moe(48, 3, 2)),
             _delta(5, 16, None),
             _latent("latent_attention", 2, 32, 2, 16, 16, 8, _moe(20, 6, 3, limit=1.0), 0.8, base=7.0,
                     scaling={"factor": 3.0, "original": 4, "fast": 2.0, "slow": 1.0})]}
    e = {"architecture": "Benarax", "vocab": 150, "width": 32, "norm": {"eps": 1e-6, "groups": 4}, "canon": {"taps": 3},
         "loop": {"start": 0, "stop": 1, "times": 1}, "layers": [_delta(1, 32, _moe(8, 2, 2))]}
    f = {"architecture": "Benarax", "vocab": 203, "width": 100, "norm": {"eps": 1e-6, "groups": 5}, "canon": {"taps": 1},
         "embedding": {"scale": 1.3}, "logit_scale": 0.7, "residual_mult": 0.9, "token_side": {"dim": 6},
         "loop": {"start": 0, "stop": 3, "times": 2}, "layers": [
             _latent("latent_attention", 3, 10, 6, 14, 20, 12, _moe(10, 1, 1), 0.5, base=77.0,
                     scaling={"factor": 3.0, "original": 32, "fast": 4.0, "slow": 1.0}),
             _delta(3, 12, _moe(18, 5, 5)),
             _latent("latent_attention_2", 7, 12, 4, 6, 36, 44, None, 0.8, base=1000.0)]}
    return {"A": (a, 8), "B": (b, 16), "C": (c, 4), "D": (d, 16), "E": (e, 8), "F": (f, 16)}


def medium_config():
    """A model of a few hundred columns whose prompts are long enough for the kernels of many rows: latents of 64 and
    128 with rotated parts of 16 and 32 on pages of 16, experts with more than 512 (token, choice) pairs a step,
    recurrent heads of 32, 64 and 128 channels."""
    ramp = {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 1.0}
    return {"architecture": "Benarax", "vocab": 700, "width": 320, "norm": {"eps": 1e-6, "groups": 5}, "canon": {"taps": 4},
            "embedding": {"scale": 1.5}, "logit_scale": 0.5, "residual_mult": 0.6, "token_side": {"dim": 24},
            "loop": {"start": 2, "stop": 4, "times": 2}, "layers": [
                _latent("latent_attention", 6, 48, 16, 32, 64, 96, _moe(96, 8, 3), 0.5, base=20000.0, scaling=ramp),
                _delta(5, 64, _moe(64, 6, 2)),
                _latent("latent_attention_2", 10, 32, 32, 64, 128, 72, _moe(96, 8, 3), 0.4, base=5000.0),
                _delta(2, 128, None),
                _delta(9, 32, _moe(64, 6, 2))]}, 16


def write_model(raw, out_dir, seed):
    """Random weights for `raw`, then made sharp: the queries' and keys' projections are large so that attention is
    peaked, the embedding and the side table so that tokens differ, norm weights are spread, the convolution's taps
    are not small, decays spread from slow to fast and the erased share from little to much, the router decides
    clearly, and the experts' inputs reach both sides of the clamp."""
    from inferflux_b200.config import config_from_dict
    from inferflux_b200.weights import SafetensorsFile, write_random_model, write_safetensors
    cfg = config_from_dict(raw)
    write_random_model(cfg, out_dir, seed=seed, dtype=torch.float32, std=0.08, norm_jitter=0.2)
    path = Path(out_dir) / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    g = torch.Generator().manual_seed(seed)
    for n, t in tensors.items():
        if n.endswith(".mix.uq") or n.endswith(".mix.uk"):
            tensors[n] = t * 4.0
        elif n.endswith(".mix.dkv"):
            tensors[n] = t * 2.5
        elif n in ("embed", "side.embed"):
            tensors[n] = t * 8.0
        elif n.endswith(".canon1"):
            tensors[n] = 0.6 * torch.randn(t.shape, generator=g)
        elif n.endswith(".mix.w0"):
            tensors[n] = 1.5 * torch.randn(t.shape, generator=g)
        elif n.endswith(".mix.a.b"):
            tensors[n] = 1.0 * torch.randn(t.shape, generator=g)
        elif n.endswith(".mix.w2") or n.endswith(".mix.w1"):
            tensors[n] = t * 6.0
        elif n.endswith(".mix.k") or n.endswith(".mix.a"):
            tensors[n] = t * 3.0
        elif n.endswith(".mlp.router"):
            tensors[n] = t * 10.0
        elif ".mlp.e" in n or n.endswith(".side.gate"):
            tensors[n] = t * 3.0
    write_safetensors(path, tensors, metadata={"format": "pt"})
    (Path(out_dir) / "config.json").write_text(json.dumps(raw, indent=1))
    return Path(out_dir)


def load(model_dir):
    return plain_benarax.load_model_dir(model_dir)


def plain_logits(model_dir, requests, weights_as=None, dtype=torch.float64):
    raw, W = load(model_dir)
    if weights_as is not None:
        W = {k: (v.to(weights_as) if v.is_floating_point() else v) for k, v in W.items()}
    return {rid: plain_benarax.forward(raw, W, toks, dtype=dtype).double().numpy() for rid, toks in requests.items()}


def requests_for(raw, lens, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, raw["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lens)}
