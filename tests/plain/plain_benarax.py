"""The Benarax decoder stated plainly: one function per mechanism, whole sequences at once, no cache,
no batching, nothing shared with the package.  Slow on purpose; the tests hold the engine to it.

A model is (raw, W): config.json as a dict and name -> tensor.  Every function computes in the dtype of
its inputs (the tests use float64).

    x = embed[tokens] * s_e
    per layer run:  h = groupnorm(x, norm1)
                    x = x + m * (mixer(h + conv(h)) + ff(h))                 (ff may be absent)
                    x = x + m * rmsnorm(P (gelu(G x) * side[tokens, layer's columns]), side.norm)
    logits = s_l * head . groupnorm(x, final.norm)

Layers lo .. hi - 1 of `loop` run `times` times in a row with the same weights.  Mixers: `general_delta`
(a matrix per head that decays per key channel, loses part of what it holds along the present unit key,
and gains k v^T) and two latent attentions (queries through a normed latent; keys and values of all heads
from one normed latent per token, plus one rotated key part that all heads share), which differ in how
rotated elements pair up.  Feed-forward: a mixture of clamped gated experts whose weights are a softmax
over the chosen router outputs only.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ------------------------------------------------------------------------------ norms

def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rmsnorm(x, w, eps):
    return unit_rms(x, eps) * w


def groupnorm(x, w, eps, groups):
    """The last axis in `groups` equal consecutive parts, each divided by its own root mean square."""
    n = x.shape[-1]
    parts = x.reshape(*x.shape[:-1], groups, n // groups)
    return unit_rms(parts, eps).reshape(x.shape) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------ convolution over time

def causal_conv(h, w):
    """h: [n, C]; w: [C, taps].  out_t = sum_j w[:, j] h_(t - taps + 1 + j), rows before the first are zeros."""
    n, taps = h.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, h.shape[1], dtype=h.dtype), h], dim=0)
    out = torch.zeros_like(h)
    for j in range(taps):
        out = out + padded[j:j + n] * w[:, j]
    return out


# ------------------------------------------------------------------------------ the delta-rule recurrence

DECAY_FLOOR = math.exp(-0.5)            # the decay lies in (exp(-exp(-1/2)), 1)


def delta_decay(raw):
    return torch.exp(-DECAY_FLOOR * torch.sigmoid(raw))


def unit_key(k):
    return k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)


def delta_scan(r, k, v, w, a, state=None):
    """r, k, w, a: [n, H, D]; v: [n, H, Dv].  Per head a matrix S [key channel, value channel]:
    S <- w_t * S (rows) - (a_t u_t) (u_t^T S) + k_t v_t^T with u_t the unit key and both products taken of the
    old S; out_t = S^T r_t with the new S."""
    n, H, D = r.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=r.dtype) if state is None else state.clone()
    u = unit_key(k)
    out = []
    for t in range(n):
        along = torch.einsum("hi,hij->hj", u[t], S)                      # what S holds along the unit key
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * along[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hij,hi->hj", S, r[t]))
    return torch.stack(out), S


def delta_mixer(h, W, p, mixer, eps):
    H, D = mixer["heads"], mixer["dim"]
    n = h.shape[0]
    r, k, v = ((h @ W[p + s].T).view(n, H, D) for s in "rkv")
    w = delta_decay(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]).view(n, H, D)
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(n, H, D)
    o, _S = delta_scan(r, k, v, w, a)
    o = unit_rms(o, eps).reshape(n, H * D)
    return (o * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------------------ rotation

def rotary_frequencies(rot):
    """(frequencies [dims / 2], what cos and sin are multiplied by).  With `scaling` {factor, original, fast, slow}:
    frequencies that turn fewer than `slow` times within `original` positions are divided by factor, those that
    turn more than `fast` times stay, a ramp in the index between."""
    base, dims = float(rot["base"]), int(rot["dims"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, positions, freqs, mult, interleaved):
    """x: [n, heads, d]; the first 2 len(freqs) elements turn, pair i being (2i, 2i + 1) or (i, i + len(freqs))."""
    out = x.clone()
    pos = torch.as_tensor(positions, dtype=x.dtype)
    half = len(freqs)
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = (torch.cos(a) * mult)[:, None], (torch.sin(a) * mult)[:, None]
        i0, i1 = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        u, v = x[:, :, i0], x[:, :, i1]
        out[:, :, i0] = u * c - v * s
        out[:, :, i1] = v * c + u * s
    return out


# ------------------------------------------------------------------------------ latent attention

def latent_attention(h, W, p, mixer, eps, positions, interleaved):
    H, D, R, Dv, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    n = h.shape[0]
    freqs, mult = rotary_frequencies(mixer["rot"])
    q = (rmsnorm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps) @ W[p + "uq"].T).view(n, H, D + R)
    q_plain, q_turned = q[:, :, :D], rotate(q[:, :, D:], positions, freqs, mult, interleaved)
    down = h @ W[p + "dkv"].T
    c = rmsnorm(down[:, :rank], W[p + "dkv.norm"], eps)
    k_turned = rotate(down[:, None, rank:], positions, freqs, mult, interleaved)[:, 0]       # one for all heads
    k_plain = (c @ W[p + "uk"].T).view(n, H, D)
    v = (c @ W[p + "uv"].T).view(n, H, Dv)
    out = torch.zeros(n, H, Dv, dtype=h.dtype)
    for t in range(n):
        for a in range(H):
            s = (k_plain[:t + 1, a] @ q_plain[t, a] + k_turned[:t + 1] @ q_turned[t, a]) * mixer["scale"]
            out[t, a] = torch.softmax(s, dim=0) @ v[:t + 1, a]
    return out.reshape(n, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------ feed-forward

def route(h, W, p, router):
    """(chosen experts [n, top], weights [n, top]): the largest router outputs, softmax among them alone."""
    z = h @ W[p + "router"].T
    top = torch.topk(z, router["top"], dim=-1)
    return top.indices, torch.softmax(top.values, dim=-1)


def expert(h, W, p, e, limit):
    g = torch.clamp(h @ W[f"{p}e{e}.gate"].T, max=limit)
    u = torch.clamp(h @ W[f"{p}e{e}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[f"{p}e{e}.down"].T


def moe_ff(h, W, p, mlp):
    chosen, weight = route(h, W, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            out[t] += g * expert(h[t:t + 1], W, p, e, mlp["expert"]["limit"])[0]
    return out


# ------------------------------------------------------------------------------ token side input

def side_input(x, W, p, side_rows, eps):
    """The normed delta that a layer adds from its columns of the side table."""
    y = (gelu_tanh(x @ W[p + "side.gate"].T) * side_rows) @ W[p + "side.proj"].T
    return rmsnorm(y, W[p + "side.norm"], eps)


# ------------------------------------------------------------------------------ the model

def run_order(raw):
    n = len(raw["layers"])
    loop = raw.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return list(range(n))
    inner = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + inner * loop["times"] + list(range(loop["stop"], n))


def forward(raw, W, tokens, dtype=torch.float64, streams=None):
    """Logits [len(tokens), vocab].  `streams`, a list, receives the residual stream after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps, groups = float(raw["norm"]["eps"]), int(raw["norm"].get("groups", 1))
    m = float(raw.get("residual_mult", 1.0))
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = list(range(len(tokens)))
    x = W["embed"][ids] * float((raw.get("embedding") or {}).get("scale", 1.0))
    side = raw.get("token_side")
    for i in run_order(raw):
        layer, p = raw["layers"][i], f"l{i}."
        h = groupnorm(x, W[p + "norm1"], eps, groups)
        hm = h + causal_conv(h, W[p + "canon1"]) if raw.get("canon") else h
        if layer["type"] == "general_delta":
            y = delta_mixer(hm, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] in ("latent_attention", "latent_attention_2"):
            y = latent_attention(hm, W, p + "mix.", layer["mixer"], eps, positions, layer["type"] == "latent_attention")
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        if layer.get("mlp") is not None:
            y = y + moe_ff(h, W, p + "mlp.", layer["mlp"])
        x = x + m * y
        if side:
            d = int(side["dim"])
            x = x + m * side_input(x, W, p, W["side.embed"][ids][:, i * d:(i + 1) * d], eps)
        if streams is not None:
            streams.append(x.clone())
    return groupnorm(x, W["final.norm"], eps, groups) @ W["head"].T * float(raw.get("logit_scale", 1.0))


def load_model_dir(model_dir):
    """(config.json as a dict, name -> tensor) read with nothing but the file format: 8 bytes of length,
    that much JSON (name -> dtype, shape, offsets), then the data."""
    import numpy as np
    model_dir = Path(model_dir)
    raw = json.loads((model_dir / "config.json").read_text())
    blob = (model_dir / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8:8 + n])
    data = memoryview(blob)[8 + n:]
    W = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = bytes(data[lo:hi])
        if info["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f4").copy())
        elif info["dtype"] == "F64":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<f8").copy())
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(buf, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {info['dtype']} is not read here")
        W[name] = t.view(*info["shape"])
    return raw, W
