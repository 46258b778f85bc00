"""The Radalix decoder stated plainly: one function per mechanism, whole sequences at once, no cache,
no batching, nothing shared with the package.  Slow on purpose; the tests hold the engine to it.

A model is (raw, W): config.json as a dict and name -> tensor.  Every function computes in the dtype of
its inputs (the tests use float64).

    x = embed[tokens] * s_e + bigram[hash(previous token, token)]
    per layer:  m = mixer(rmsnorm(x, norm1));   f = ff(rmsnorm(x, norm2))     (both of the same x; ff may be absent)
                x = x + ls1 * m + ls2 * f
    logits = c * tanh(embed . rmsnorm(x, final.norm) / c)

A mixer is a pair of two mixers that read the same rows.  `parallel`: causal attention without positions but
with a position-dependent query temperature and an output gate, beside a linear attention whose state decays
per key channel; the result is half the sum of the two after an RMS norm of each.  `parallel_2`: attention
with a partial rotation, a sliding window and a sink, beside a selective state-space recurrence; the result is a
weighted sum of the two.  In both attentions queries, keys and values pass a short causal convolution over
time right behind their projections.  Feed-forward: a mixture of gated experts weighted by their sigmoid
scores, normalised over the chosen, plus an expert that every token uses.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ------------------------------------------------------------------------------ small pieces

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


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u, w, bias=None):
    """u: [n, C]; w: [C, taps].  out_t = sum_j w[:, j] u_(t - taps + 1 + j) (+ bias), rows before the first are zeros."""
    n, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out = out + padded[j:j + n] * w[:, j]
    return out if bias is None else out + bias


# ------------------------------------------------------------------------------ embedding

def bigram_rows(tokens, bigram):
    """Row of the second table for every token: a hash of the token before and the token itself; a sequence's
    first token takes the table's last row."""
    b = bigram
    rows = []
    for i, t in enumerate(tokens):
        rows.append(b["buckets"] if i == 0 else (int(tokens[i - 1]) * b["mul_prev"] + int(t) * b["mul_cur"]) % b["buckets"])
    return rows


def embed(raw, W, tokens, dtype):
    e = raw.get("embedding") or {}
    x = W["embed"].to(dtype)[list(tokens)] * float(e.get("scale", 1.0))
    if e.get("bigram"):
        x = x + W["bigram"].to(dtype)[bigram_rows(tokens, e["bigram"])]
    return x


# ------------------------------------------------------------------------------ positions

def rotary_frequencies(rot):
    """(frequencies as Python floats, what cos and sin are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])

    def index_of(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(index_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_neighbours(x, positions, freqs, mult):
    """x: [n, H, d]; elements (2i, 2i + 1) of the first 2 len(freqs) turn by position * freqs[i]."""
    out = x.clone()
    pos = torch.tensor(list(positions), dtype=x.dtype)
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = (torch.cos(a) * mult)[:, None], (torch.sin(a) * mult)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def query_temperature(positions, qt, dtype):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    return torch.tensor([1.0 + float(qt["coef"]) * math.log((p + 1) // int(qt["every"]) + 1) for p in positions], dtype=dtype)


# ------------------------------------------------------------------------------ attention

def attention(h, W, p, m, positions, gated):
    """Grouped-query attention over one sequence.  m: heads, kv_heads, dim, vdim, scale and optionally conv (taps),
    rot, q_temp, mask {size}.  A sink (tensor `sink`) joins the softmax's denominator if the tensor exists."""
    n = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, W[p + "q.conv"]), causal_conv(k, W[p + "k.conv"]), causal_conv(v, W[p + "v.conv"])
    q, k, v = q.reshape(n, H, d), k.reshape(n, G, d), v.reshape(n, G, dv)
    if m.get("rot"):
        freqs, mult = rotary_frequencies(m["rot"])
        q, k = rotate_neighbours(q, positions, freqs, mult), rotate_neighbours(k, positions, freqs, mult)
    if m.get("q_temp"):
        q = q * query_temperature(positions, m["q_temp"], q.dtype)[:, None, None]
    window = int(m["mask"]["size"]) if m.get("mask") else None
    sink = W.get(p + "sink")
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for i in range(n):
        first = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[first:i + 1, g] @ q[i, hh]) * float(m["scale"])
            top = s.max() if sink is None else torch.maximum(s.max(), sink[hh].to(s.dtype))
            e = torch.exp(s - top)
            denom = e.sum() + (torch.exp(sink[hh].to(s.dtype) - top) if sink is not None else 0.0)
            out[i, hh] = (e / denom) @ v[first:i + 1, g]
    out = out.reshape(n, H * dv)
    if gated:
        out = out * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


# ------------------------------------------------------------------------------ the two recurrences

def decayed_scan(q, k, v, decay, state=None):
    """q, k, decay: [n, H, D]; v: [n, H, Dv].  Per head a matrix S [key channel, value channel]:
    S <- decay_t * S (rows) + k_t v_t^T; out_t = S^T q_t with the new S."""
    n, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(n, H, v.shape[2], dtype=q.dtype)
    for t in range(n):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


def gated_linear_attention(h, W, p, m, eps):
    n = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T).reshape(n, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).reshape(n, H, d)
    v = (h @ W[p + "v"].T).reshape(n, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).reshape(n, H, d)
    o, _S = decayed_scan(q, k, v, decay)
    o = rmsnorm(o, W[p + "norm"], eps).reshape(n, H * dv)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def state_space(h, W, p, m, eps):
    n = h.shape[0]
    H, dv, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = H * dv
    zx = h @ W[p + "in"].T
    z, xbc, dt = zx[:, :inner], zx[:, inner:2 * inner + 2 * G * N], zx[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(n, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(n, G, N)
    C = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                                            # [n, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)                               # [n, H]
    of_head = [hh // (H // G) for hh in range(H)]
    k = B[:, of_head] * dt[:, :, None]                                               # [n, H, N]
    y, _S = decayed_scan(C[:, of_head], k, x, decay[:, :, None].expand(n, H, N))
    y = (y + W[p + "D"][None, :, None] * x).reshape(n, inner)
    y = groupnorm(y * silu(z), W[p + "norm"], eps, int(m["norm_groups"]))
    return y @ W[p + "o"].T


# ------------------------------------------------------------------------------ the pair

def mixer(h, W, p, layer, eps, positions):
    m = layer["mixer"]
    if layer["type"] == "parallel":
        left = attention(h, W, p + "left.", m["left"], positions, gated=True)
        right = gated_linear_attention(h, W, p + "right.", m["right"], eps)
        return 0.5 * (rmsnorm(left, W[p + "left.out"], eps) + rmsnorm(right, W[p + "right.out"], eps))
    if layer["type"] == "parallel_2":
        left = attention(h, W, p + "left.", m["left"], positions, gated=False)
        right = state_space(h, W, p + "right.", m["right"], eps)
        return float(m["left_scale"]) * left + float(m["right_scale"]) * right
    raise ValueError(layer["type"])


# ------------------------------------------------------------------------------ feed-forward

def gated_expert(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, W, p, router):
    """(chosen experts [n, top], weights [n, top]): sigmoid scores, the largest chosen, weights = scores over their sum."""
    s = torch.sigmoid(h @ W[p + "router"].T)
    val, idx = torch.topk(s, int(router["top"]), dim=-1)
    return idx, val / (val.sum(dim=-1, keepdim=True) + 1e-20)


def moe_ff(h, W, p, mlp):
    idx, wgt = route(h, W, p, mlp["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] = out[t] + wgt[t, j] * gated_expert(h[t:t + 1], W, f"{p}e{int(idx[t, j])}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


# ------------------------------------------------------------------------------ the model

def forward(raw, W, tokens, dtype=torch.float64, streams=None):
    """Logits [n, vocab] of one sequence.  `streams`: a list that receives the residual stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = float(raw["norm"]["eps"])
    positions = list(range(len(tokens)))
    x = embed(raw, W, tokens, dtype)
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        delta = W[p + "ls1"] * mixer(rmsnorm(x, W[p + "norm1"], eps), W, p + "mix.", layer, eps, positions)
        if layer.get("mlp") is not None:
            delta = delta + W[p + "ls2"] * moe_ff(rmsnorm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        x = x + delta
        if streams is not None:
            streams.append(x.clone())
    logits = rmsnorm(x, W["final.norm"], eps) @ W["embed"].T
    cap = raw.get("logit_softcap")
    return logits if not cap else float(cap) * torch.tanh(logits / float(cap))


def load_model_dir(model_dir):
    """(config.json as a dict, name -> tensor) of a model folder, read without the package."""
    import numpy as np
    model_dir = Path(model_dir)
    raw = json.loads((model_dir / "config.json").read_text())
    blob = (model_dir / "model.safetensors").read_bytes()
    n = int.from_bytes(blob[:8], "little")
    header = json.loads(blob[8:8 + n])
    W = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        data = blob[8 + n + lo:8 + n + hi]
        if info["dtype"] == "BF16":
            u = np.frombuffer(data, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(u.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(data, dtype="<f4").copy())
        elif info["dtype"] == "F64":
            t = torch.from_numpy(np.frombuffer(data, dtype="<f8").copy())
        elif info["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(data, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        W[name] = t.reshape(info["shape"])
    return raw, W
