"""Plain PyTorch statement of every kernel's contract, on any device.

Two uses: the GPU tests compare each CUDA kernel with the function of the same name
here, and the CPU tests hand this table to the engine in place of the CUDA one so
that the cache manager, the batch packing and the step function can be checked
without a GPU.  It is test code: the engine itself has no such path.  All math is
done in float32 (float64 where `wide` is set) and rounded once to the output dtype.
"""
from __future__ import annotations

import math

import torch


class PlainKernels:
    name = "plain-torch"

    def __init__(self, wide: bool = False):
        self.acc = torch.float64 if wide else torch.float32
        self.launches = 0

    # ------------------------------------------------------------- elementwise
    def embed(self, table, token_ids, vocab, scale=1.0):
        return (table[token_ids.long()].to(self.acc) * scale).to(torch.float32)

    def rmsnorm(self, x, w, eps, out_dtype, groups=1):
        xa = x.to(self.acc)
        parts = xa.reshape(*xa.shape[:-1], groups, xa.shape[-1] // groups)
        y = (parts * torch.rsqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(xa.shape) * w.to(self.acc)
        return y.to(out_dtype)

    def rmsnorm_columns(self, rows, col0, n, w, eps):
        """Columns col0 .. col0 + n of `rows`, RMS-normed with weight `w`, as a tensor of their own."""
        return self.rmsnorm(rows[:, col0:col0 + n], w, eps, rows.dtype)

    def residual_add_scaled(self, x, a, b, scale, out_dtype=None):
        """x += scale * (a + b) (b may be None); with `out_dtype` also returns the updated rows in that dtype."""
        total = a.to(self.acc) if b is None else a.to(self.acc) + b.to(self.acc)
        x += (scale * total).to(torch.float32)
        return None if out_dtype is None else x.to(out_dtype)

    def scale_(self, values, factor):
        values.mul_(factor)

    def gelu_mul_table(self, z, table, token_ids, first_column):
        """gelu_tanh(z) * table[token, first_column : first_column + z.shape[1]] in z's dtype."""
        za = z.to(self.acc)
        e = table[token_ids.long()][:, first_column:first_column + z.shape[1]].to(self.acc)
        g = 0.5 * za * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (za + 0.044715 * za ** 3)))
        return (g * e).to(z.dtype)

    def add_rmsnorm(self, x, delta, w, eps, out_dtype):
        x += delta.to(torch.float32)
        return self.rmsnorm(x, w, eps, out_dtype)

    def residual_add(self, x, delta):
        x += delta.to(torch.float32)

    def silu_mul(self, gate_up):
        inter = gate_up.shape[1] // 2
        g, u = gate_up[:, :inter].to(self.acc), gate_up[:, inter:].to(self.acc)
        return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def scatter_i32(self, table, index, value):
        if index.numel():
            table.view(-1)[index.long()] = value

    def relay_i32(self, dst, dst_index, src, src_index):
        if dst_index.numel():
            dst[dst_index.long()] = src[src_index.long()]

    # ------------------------------------------------------------------ linear
    def linear(self, a, w, bias=None, out_dtype=None, allow_partial=False):
        y = a.to(self.acc) @ w.to(self.acc).t()
        if bias is not None:
            y = y + bias.to(self.acc)
        return y.to(out_dtype or a.dtype)

    linear_generic = linear

    def linear_swiglu(self, a, w_gate_up):
        return self.silu_mul(self.linear(a, w_gate_up))

    def materialize(self, value, bias=None):
        return value if bias is None else value + bias.to(value.dtype)

    # --------------------------------------------------------------- attention
    def rope_append(self, qkv, bias, rotary, nq, nkv, d, ctx, cache, q_norm=None, k_norm=None, norm_eps=0.0, dv=None,
                    own_kv=True, q_temp=None):
        if (q_norm is not None or k_norm is not None or (dv is not None and dv != d) or not own_kv or q_temp is not None
                or (rotary is not None and rotary.magnitude != 1.0) or (cache.kv is not None and cache.kv.shape[-1] != d)):
            return self._norm_rope_append(qkv, rotary, nq, nkv, d, d if dv is None else dv, ctx, cache, q_norm, k_norm,
                                          norm_eps, own_kv, q_temp)
        T = qkv.shape[0]
        x = qkv.to(self.acc)
        if bias is not None:
            x = x + bias.to(self.acc)
        x = x.view(T, nq + 2 * nkv, d)
        pos = ctx.positions.long()
        if rotary is not None:
            rot = rotary.rotary_dim
            ang = pos.to(torch.float32)[:, None] * rotary.inv_freq[None, :].to(torch.float32)
            cos, sin = torch.cos(ang).to(self.acc)[:, None, :], torch.sin(ang).to(self.acc)[:, None, :]
            qk = x[:, :nq + nkv, :rot]
            if rotary.interleaved:
                a, b = qk[..., 0::2], qk[..., 1::2]
                turned = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
            else:
                a, b = qk[..., :rot // 2], qk[..., rot // 2:]
                turned = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
            x = x.clone()
            x[:, :nq + nkv, :rot] = turned
        x = x.to(qkv.dtype)
        if cache.writes and cache.kv is not None:
            P = cache.page_size
            slot = ctx.req_slot.long()[ctx.token_req.long()]
            page = cache.block_table[slot, pos // P].long()
            off = pos % P
            cache.kv[page, 0, :, off, :] = x[:, nq:nq + nkv, :].to(cache.kv.dtype)
            cache.kv[page, 1, :, off, :] = x[:, nq + nkv:, :].to(cache.kv.dtype)
        return x[:, :nq, :].reshape(T, nq * d).contiguous()

    def _turn(self, x, rotary, pos):
        """x [T, heads, d]: the first rotary_dim elements of every head turned by position * inv_freq."""
        if rotary is None:
            return x
        rot = rotary.rotary_dim
        ang = pos.to(torch.float32)[:, None] * rotary.inv_freq[None, :].to(torch.float32)
        cos, sin = torch.cos(ang).to(self.acc)[:, None, :], torch.sin(ang).to(self.acc)[:, None, :]
        cos, sin = cos * rotary.magnitude, sin * rotary.magnitude
        part = x[..., :rot]
        if rotary.interleaved:
            a, b = part[..., 0::2], part[..., 1::2]
            turned = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
        else:
            a, b = part[..., :rot // 2], part[..., rot // 2:]
            turned = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
        return torch.cat([turned, x[..., rot:]], dim=-1)

    def _norm_rope_append(self, qkv, rotary, nq, nkv, d, dv, ctx, cache, q_norm, k_norm, norm_eps, own_kv, q_temp=None):
        """`q_temp` = (coef, every): the queries are multiplied by 1 + coef ln(floor((p + 1) / every) + 1) at position p."""
        T = qkv.shape[0]
        x = qkv.to(self.acc)
        pos = ctx.positions.long()

        def head_norm(v, w):
            if w is None:
                return v
            return v * torch.rsqrt((v * v).mean(-1, keepdim=True) + norm_eps) * w.to(self.acc)
        q = self._turn(head_norm(x[:, :nq * d].view(T, nq, d), q_norm), rotary, pos)
        if q_temp is not None:
            mult = 1.0 + q_temp[0] * torch.log((torch.div(pos + 1, q_temp[1], rounding_mode="floor") + 1).to(torch.float32))
            q = q * mult.to(self.acc)[:, None, None]
        if own_kv:
            k = self._turn(head_norm(x[:, nq * d:(nq + nkv) * d].view(T, nkv, d), k_norm), rotary, pos)
            v = x[:, (nq + nkv) * d:].view(T, nkv, dv)
            if cache.writes and cache.kv is not None:
                P = cache.page_size
                slot = ctx.req_slot.long()[ctx.token_req.long()]
                page = cache.block_table[slot, pos // P].long()
                off = pos % P
                cache.kv[page, 0, :, off, :d] = k.to(cache.kv.dtype)
                cache.kv[page, 1, :, off, :dv] = v.to(cache.kv.dtype)
        return q.to(qkv.dtype).reshape(T, nq * d).contiguous()

    def attention(self, q, nq, nkv, d, window, scale, ctx, cache, chunk=None, sink=False, dv=None):
        dv = d if dv is None else dv
        T = q.shape[0]
        P = cache.page_size
        if chunk or torch.is_tensor(sink) or sink or dv != d or cache.kv.shape[-1] != d:
            out = torch.empty((T, nq, dv), dtype=q.dtype, device=q.device)
            qv = q.view(T, nq, d).to(self.acc)
            pos_all, req_all, slots = ctx.positions.tolist(), ctx.token_req.tolist(), ctx.req_slot.tolist()
            for t in range(T):
                pos, slot = pos_all[t], slots[req_all[t]]
                first = max(0, pos - window + 1) if window else 0
                if chunk:
                    first = max(first, pos // chunk * chunk)
                keys = torch.arange(first, pos + 1, device=q.device)
                pages = cache.block_table[slot, keys // P].long()
                K = cache.kv[pages, 0, :, keys % P, :d].to(self.acc)
                V = cache.kv[pages, 1, :, keys % P, :dv].to(self.acc)
                for h in range(nq):
                    g = h // (nq // nkv)
                    s = (K[:, g, :] @ qv[t, h]) * scale
                    if torch.is_tensor(sink):                    # a learned number per head in the denominator
                        s = torch.cat([s, sink[h].to(s.dtype).reshape(1)])
                    elif sink:
                        s = torch.cat([s, torch.zeros(1, dtype=s.dtype)])
                    p = torch.softmax(s, dim=0)[:keys.numel()]
                    out[t, h] = (p @ V[:, g, :]).to(q.dtype)
            return out.reshape(T, nq * dv)
        out = torch.empty((T, nq, d), dtype=q.dtype, device=q.device)
        qv = q.view(T, nq, d).to(self.acc)
        pos_all = ctx.positions.tolist()
        req_all = ctx.token_req.tolist()
        slots = ctx.req_slot.tolist()
        group = nq // nkv
        for t in range(T):
            pos, slot = pos_all[t], slots[req_all[t]]
            first = max(0, pos - window + 1) if window else 0
            keys = torch.arange(first, pos + 1, device=q.device)
            pages = cache.block_table[slot, keys // P].long()
            K = cache.kv[pages, 0, :, keys % P, :].to(self.acc)          # [n, nkv, d]
            V = cache.kv[pages, 1, :, keys % P, :].to(self.acc)
            for h in range(nq):
                g = h // group
                s = (K[:, g, :] @ qv[t, h]) * scale
                p = torch.softmax(s, dim=0)
                out[t, h] = (p @ V[:, g, :]).to(q.dtype)
        return out.reshape(T, nq * d)

    # ------------------------------------------- layers that norm a sublayer's output
    def postnorm_add(self, x, y, w_post, eps_post, w_next=None, eps_next=0.0, out_dtype=None, cast_out=False, groups=1):
        ya = y.to(self.acc)
        x += (ya * torch.rsqrt((ya * ya).mean(-1, keepdim=True) + eps_post) * w_post.to(self.acc)).to(torch.float32)
        if w_next is None:
            return x.to(out_dtype or y.dtype) if cast_out else None
        return self.rmsnorm(x, w_next, eps_next, out_dtype or y.dtype, groups=groups)

    def concat_cast(self, a, b, dtype):
        return torch.cat([a, b], dim=-1).to(dtype)

    def xielu(self, z, a_pos, a_neg):
        za = z.to(self.acc)
        neg = a_neg * (torch.expm1(torch.clamp(za, max=0.0)) - za) + 0.5 * za
        return torch.where(za > 0, a_pos * za * za + 0.5 * za, neg).to(z.dtype)

    def linear_xielu(self, a, w, a_pos, a_neg):
        return self.xielu(self.linear(a, w), a_pos, a_neg)

    def softcap(self, logits, cap):
        logits.copy_(cap * torch.tanh(logits.to(self.acc) / cap))

    def short_conv(self, h, w, taps, state, index, ctx, add_input=True, bias=None, act=None, columns=None):
        """`add_input` False: the convolution alone; `bias` [channels] is added and `act` ("silu") applied behind it;
        `columns` = (first, count): the convolution runs over those columns of `h` and returns them alone."""
        if columns is not None:
            h = h[:, columns[0]:columns[0] + columns[1]]
        ha, wa = h.to(self.acc), w.to(self.acc)
        out = ha * ((1.0 if add_input else 0.0) + wa[:, taps - 1])
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        for r in range(ctx.num_requests):
            lo, hi = cu[r], cu[r + 1]
            if taps == 1:
                continue
            old = state[slots[r], index].to(self.acc)                       # [taps - 1, C]
            seq = torch.cat([old, ha[lo:hi]], dim=0)                        # inputs from taps - 1 before the span
            for k in range(1, taps):
                out[lo:hi] += wa[:, taps - 1 - k] * seq[taps - 1 - k:taps - 1 - k + (hi - lo)]
            state[slots[r], index] = seq[-(taps - 1):].to(state.dtype)
        if bias is not None:
            out = out + bias.to(self.acc)
        if act == "silu":
            out = out * torch.sigmoid(out)
        return out.to(h.dtype).contiguous()

    # ------------------------------------------------- recurrence with matrix state
    def cast_rows(self, x, dtype):
        return x if dtype == torch.float32 else x.to(dtype)

    def tanh(self, z):
        z.copy_(torch.tanh(z.to(self.acc)))
        return z

    def token_shift_mix(self, x, mu, state, prev_offset, ctx, out_dtype):
        T, C = x.shape
        before = torch.empty_like(x)
        before[1:] = x[:-1]
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        for r in range(ctx.num_requests):
            before[cu[r]] = state[slots[r], prev_offset:prev_offset + C]
        xa, ba = x.to(self.acc), before.to(self.acc)
        return (xa[None] + (ba - xa)[None] * mu.to(self.acc)[:, None, :]).to(out_dtype)

    def wkv_scan(self, r, k, v, w_raw, g, w0, u, norm_w, eps, heads, dim, state, prev_offset, x, ctx, out_dtype):
        T = r.shape[0]
        A = self.acc
        shape = (T, heads, dim)
        ra, ka, va = r.to(A).view(shape), k.to(A).view(shape), v.to(A).view(shape)
        decay = torch.exp(-torch.exp(w_raw.to(A) + w0.to(A))).view(shape)
        ua = u.to(A).view(heads, dim)
        out = torch.empty(shape, dtype=A)
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        for q in range(ctx.num_requests):
            S = state[slots[q], :prev_offset].to(A).view(heads, dim, dim).clone()
            for t in range(cu[q], cu[q + 1]):
                kv = ka[t][:, :, None] * va[t][:, None, :]
                out[t] = torch.einsum("hij,hi->hj", S + ua[:, :, None] * kv, ra[t])
                S = decay[t][:, :, None] * S + kv
            state[slots[q], :prev_offset] = S.reshape(-1).to(state.dtype)
            state[slots[q], prev_offset:] = x[cu[q + 1] - 1]
        out = out * torch.rsqrt((out * out).mean(-1, keepdim=True) + eps)
        ga = g.to(A)
        y = out.reshape(T, heads * dim) * norm_w.to(A) * (ga / (1.0 + torch.exp(-ga)))
        return y.to(out_dtype)

    def delta_rule_scan(self, proj, w_raw, w0, a_bias, norm_w, eps, heads, dim, state, ctx, out_dtype):
        """`proj`: float32 [T, 5 heads dim], the projections r, k, v, g, a side by side; `state`: float32 [slots, >= heads
        dim dim] (rows may be further apart than that), the matrices S [head, key channel, value channel], moved on."""
        T, A, HD = proj.shape[0], self.acc, heads * dim
        shape = (T, heads, dim)
        r, k, v, g, a = (proj[:, i * HD:(i + 1) * HD].to(A) for i in range(5))
        r, k, v = r.view(shape), k.view(shape), v.view(shape)
        decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(w_raw.to(A) + w0.to(A))).view(shape)
        erase = torch.sigmoid(a + a_bias.to(A)).view(shape)
        unit = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        out = torch.empty(shape, dtype=A)
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        for q in range(ctx.num_requests):
            S = state[slots[q], :HD * dim].to(A).view(heads, dim, dim).clone()
            for t in range(cu[q], cu[q + 1]):
                along = torch.einsum("hi,hij->hj", unit[t], S)
                S = decay[t][:, :, None] * S - (erase[t] * unit[t])[:, :, None] * along[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
                out[t] = torch.einsum("hij,hi->hj", S, r[t])
            state[slots[q], :HD * dim] = S.reshape(-1).to(state.dtype)
        out = out * torch.rsqrt((out * out).mean(-1, keepdim=True) + eps)
        return (out.reshape(T, HD) * norm_w.to(A) * torch.sigmoid(g)).to(out_dtype)

    # ------------------------------------------- pairs of mixers, scans with a decayed matrix state
    def bigram_add(self, x, table, token_ids, state, mul_prev, mul_cur, buckets, vocab, ctx):
        """x[t] += table[(token before * mul_prev + token * mul_cur) mod buckets], the last row (`buckets`) at position 0;
        the token before a span's first one is state[slot, 0] (int32), which then takes the span's last token."""
        ids, pos = token_ids.long(), ctx.positions.long()
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        before = torch.empty_like(ids)
        for r in range(ctx.num_requests):
            lo, hi = cu[r], cu[r + 1]
            before[lo] = state[slots[r], 0]
            before[lo + 1:hi] = ids[lo:hi - 1]
            state[slots[r], 0] = ids[hi - 1].to(state.dtype)
        rows = torch.where(pos == 0, torch.full_like(ids, buckets), (before * mul_prev + ids * mul_cur) % buckets)
        x += table[rows].to(torch.float32)

    def rmsnorm_pair(self, x, w_a, eps_a, w_b, eps_b, out_dtype, delta=None, vectors=None):
        """x += delta (if any; `vectors`: s_a * a + s_b * (b + b2), see residual_add_vectors); two RMS norms of the same rows."""
        if vectors is not None:
            self.residual_add_vectors(x, vectors.a, vectors.s_a, vectors.b, vectors.s_b, vectors.b2)
        if delta is not None:
            x += delta.to(torch.float32)
        return self.rmsnorm(x, w_a, eps_a, out_dtype), self.rmsnorm(x, w_b, eps_b, out_dtype)

    def gate_mul(self, a, g, kind):
        """a * sigmoid(g) (`sigmoid`) or a * silu(g) (`silu`), in a's dtype."""
        ga = g.to(self.acc)
        gate = torch.sigmoid(ga) if kind == "sigmoid" else ga * torch.sigmoid(ga)
        return (a.to(self.acc) * gate).to(a.dtype)

    def decay_scan(self, q, k, v, raw, state, ctx, heads, groups, dk, dv, decay, tau=1.0, q_scale=1.0, step_bias=None,
                   log_rate=None, skip=None):
        """Per request and head a float32 matrix S, kept in `state` [slots, heads dv dk] as [head, value channel, key
        channel]: S <- diag(w_t) S + k_t v_t^T, o_t = S^T (q_scale q_t) with the new S.  q, k: float32 [T, groups dk]
        (head h reads group h // (heads / groups)); v: [T, heads dv]; returns float32 [T, heads dv].
        decay `sigmoid_root`: raw [T, heads dk], w = sigmoid(raw)^(1/tau).
        decay `softplus_step`: raw [T, heads], dt = softplus(raw + step_bias), w = exp(-exp(log_rate) dt) for the whole
        head, k is multiplied by dt, and skip[h] v_t is added to o_t."""
        T, A = q.shape[0], self.acc
        per = heads // groups
        of_head = torch.arange(heads) // per
        qa = q.to(A).reshape(T, groups, dk)[:, of_head] * q_scale
        ka = k.to(A).reshape(T, groups, dk)[:, of_head]
        va = v.to(A).reshape(T, heads, dv)
        if decay == "sigmoid_root":
            w = torch.exp(torch.nn.functional.logsigmoid(raw.to(A)) / tau).reshape(T, heads, dk)
        elif decay == "softplus_step":
            dt = torch.nn.functional.softplus(raw.to(A) + step_bias.to(A), threshold=30.0)
            w = torch.exp(-torch.exp(log_rate.to(A)) * dt)[:, :, None].expand(T, heads, dk)
            ka = ka * dt[:, :, None]
        else:
            raise ValueError(decay)
        out = torch.empty((T, heads, dv), dtype=A)
        cu, slots = ctx.cu_seqlens.tolist(), ctx.req_slot.tolist()
        for r in range(ctx.num_requests):
            S = state[slots[r], :heads * dv * dk].to(A).view(heads, dv, dk).clone()
            for t in range(cu[r], cu[r + 1]):
                S = w[t][:, None, :] * S + va[t][:, :, None] * ka[t][:, None, :]
                out[t] = torch.einsum("hvd,hd->hv", S, qa[t])
            state[slots[r], :heads * dv * dk] = S.reshape(-1).to(state.dtype)
        if skip is not None:
            out = out + skip.to(A)[None, :, None] * va
        return out.reshape(T, heads * dv).to(torch.float32)

    def gated_groupnorm(self, y, gate, w, eps, groups, gate_first, out_dtype):
        """Rows of y [T, C] in `groups` equal parts, each over its own root mean square, times w (of size C, or of a
        part's size and then the same for every part) and silu(gate): the gate multiplies before the norm
        (`gate_first`) or behind it."""
        A = self.acc
        ya, ga = y.to(A), gate.to(A)
        ga = ga * torch.sigmoid(ga)
        if gate_first:
            ya = ya * ga
        T, C = ya.shape
        parts = ya.reshape(T, groups, C // groups)
        normed = parts * torch.rsqrt((parts * parts).mean(-1, keepdim=True) + eps)
        wa = w.to(A)
        normed = (normed * wa).reshape(T, C) if wa.numel() == C // groups else normed.reshape(T, C) * wa
        if not gate_first:
            normed = normed * ga
        return normed.to(out_dtype)

    def pair_combine(self, a, b, w_a, w_b, c_a, c_b, eps):
        """float32 [T, C]: c_a a + c_b b, or with weights c_a a / rms(a) * w_a + c_b b / rms(b) * w_b."""
        A = self.acc
        aa, ba = a.to(A), b.to(A)
        if w_a is not None:
            aa = aa * torch.rsqrt((aa * aa).mean(-1, keepdim=True) + eps) * w_a.to(A)
            ba = ba * torch.rsqrt((ba * ba).mean(-1, keepdim=True) + eps) * w_b.to(A)
        return (c_a * aa + c_b * ba).to(torch.float32)

    def residual_add_vectors(self, x, a, s_a, b=None, s_b=None, b2=None):
        """x += s_a * a + s_b * (b + b2), element by element along a row (a vector None: ones; b, b2 may be None)."""
        A = self.acc
        total = a.to(A) if s_a is None else a.to(A) * s_a.to(A)
        if b is not None:
            bb = b.to(A) if b2 is None else b.to(A) + b2.to(A)
            total = total + (bb if s_b is None else bb * s_b.to(A))
        x += total.to(torch.float32)

    # ------------------------------------------------------- mixture of experts
    def moe_route(self, z, correction, top, of_chosen=False, kind=None, floor=0.0):
        if kind == "sigmoid_normalized":                    # sigmoid scores; the chosen scores over their sum
            s = torch.sigmoid(z.to(self.acc))
            choice = s if correction is None else s + correction.to(self.acc)
            ids = torch.topk(choice, top, dim=-1).indices
            w = torch.gather(s, 1, ids)
            return ids.to(torch.int32), (w / (w.sum(-1, keepdim=True) + floor)).to(torch.float32)
        if of_chosen:                                       # the largest logits; softmax among them alone
            za = z.to(self.acc) if correction is None else z.to(self.acc) + correction.to(self.acc)
            best = torch.topk(za, top, dim=-1)
            return best.indices.to(torch.int32), torch.softmax(torch.gather(z.to(self.acc), 1, best.indices), dim=-1).to(torch.float32)
        s = torch.softmax(z.to(self.acc), dim=-1)
        choice = s if correction is None else s + correction.to(self.acc)
        ids = torch.topk(choice, top, dim=-1).indices
        return ids.to(torch.int32), torch.gather(s, 1, ids).to(torch.float32)

    def moe_experts(self, h, w_up, w_down, ids, weights, experts, out_dtype, glu=None):
        """`glu` = (limit, slope[, offset = 1]): w_up holds an expert's gate rows above its up rows, and the activation is
        g sigmoid(slope g) (u + offset) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
        ha = h.to(self.acc)
        out = torch.zeros_like(ha)
        for t in range(h.shape[0]):
            for e, wgt in zip(ids[t].tolist(), weights[t].to(self.acc)):
                if e >= experts:
                    out[t] += wgt * ha[t]
                elif glu is not None:
                    both = w_up[e].to(self.acc) @ ha[t]
                    ff = both.shape[0] // 2
                    gate, up = torch.clamp(both[:ff], max=glu[0]), torch.clamp(both[ff:], min=-glu[0], max=glu[0])
                    a = gate * torch.sigmoid(glu[1] * gate) * (up + (glu[2] if len(glu) > 2 else 1.0))
                    out[t] += wgt * (w_down[e].to(self.acc) @ a.to(h.dtype).to(self.acc))
                else:
                    a = torch.relu(w_up[e].to(self.acc) @ ha[t]) ** 2
                    out[t] += wgt * (w_down[e].to(self.acc) @ a.to(h.dtype).to(self.acc))
        return out.to(out_dtype)

    # -------------------------------------------------------- latent attention
    def latent_norm_append(self, rows, col0, rank, w, eps, ctx, cache):
        xa = rows[:, col0:col0 + rank].to(self.acc)
        c = xa * torch.rsqrt((xa * xa).mean(-1, keepdim=True) + eps) * w.to(self.acc)
        if cache.writes:
            P, pos = cache.page_size, ctx.positions.long()
            slot = ctx.req_slot.long()[ctx.token_req.long()]
            page = cache.block_table[slot, pos // P].long()
            cache.kv[page, 0, 0, pos % P, :] = c.to(cache.kv.dtype)

    def latent_rope_append(self, rows, col0, rank, rot, w, eps, q, heads, dim, rotary, ctx, cache, vdim=None):
        """The cached row of every token: [columns col0 .. + rank of `rows`, RMS-normed with `w`; the `rot` columns
        behind them, turned by the token's position].  Returns `q` [T, heads (dim + rot)] with every head's last `rot`
        elements turned the same way (q itself may be changed)."""
        A = self.acc
        xa = rows[:, col0:col0 + rank].to(A)
        c = xa * torch.rsqrt((xa * xa).mean(-1, keepdim=True) + eps) * w.to(A)
        T = rows.shape[0]
        pos = ctx.positions.to(A)

        def turn(x):                                         # x: [T, n, rot]
            if not rot or rotary is None:
                return x
            half = rotary.rotary_dim // 2
            ang = pos[:, None] * rotary.inv_freq.to(A)[None, :]
            cos, sin = (torch.cos(ang) * rotary.magnitude)[:, None, :], (torch.sin(ang) * rotary.magnitude)[:, None, :]
            out = x.clone()
            if rotary.interleaved:
                u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
                out[..., 0:2 * half:2], out[..., 1:2 * half:2] = u * cos - v * sin, v * cos + u * sin
            else:
                u, v = x[..., :half], x[..., half:2 * half]
                out[..., :half], out[..., half:2 * half] = u * cos - v * sin, v * cos + u * sin
            return out
        kt = turn(rows[:, None, col0 + rank:col0 + rank + rot].to(A))[:, 0]
        if cache.writes:
            P, p = cache.page_size, ctx.positions.long()
            slot = ctx.req_slot.long()[ctx.token_req.long()]
            page = cache.block_table[slot, p // P].long()
            cache.kv[page, 0, 0, p % P, :] = torch.cat([c, kt], dim=-1).to(cache.kv.dtype)
        qa = q[:, :heads * (dim + rot)].to(A).reshape(T, heads, dim + rot).clone()
        qa[:, :, dim:] = turn(qa[:, :, dim:])
        return qa.reshape(T, heads * (dim + rot)).to(q.dtype)

    def latent_attention(self, q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache, rot=0):
        if rot:
            return self._latent_attention_rot(q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache, rot)
        T, P = q_rows.shape[0], cache.page_size
        q = q_rows[:, :heads * dim].to(self.acc).view(T, heads, dim)
        uk, uv = w_uk.to(self.acc).view(heads, dim, rank), w_uv.to(self.acc).view(heads, vdim, rank)
        out = torch.empty((T, heads, vdim), dtype=q_rows.dtype, device=q_rows.device)
        pos_all, req_all, slots = ctx.positions.tolist(), ctx.token_req.tolist(), ctx.req_slot.tolist()
        for t in range(T):
            pos, slot = pos_all[t], slots[req_all[t]]
            first = max(0, pos - window + 1) if window else 0
            keys = torch.arange(first, pos + 1, device=q_rows.device)
            pages = cache.block_table[slot, keys // P].long()
            C = cache.kv[pages, 0, 0, keys % P, :].to(self.acc)            # [n, rank]
            for h in range(heads):
                s = (C @ (uk[h].t() @ q[t, h])) * scale
                if sinks is not None:
                    s = torch.cat([s, sinks[h:h + 1].to(self.acc)])
                p = torch.softmax(s, dim=0)[:keys.numel()]
                out[t, h] = (uv[h] @ (p @ C)).to(q_rows.dtype)
        return out.reshape(T, heads * vdim)

    def _latent_attention_rot(self, q_rows, w_uk, w_uv, sinks, heads, dim, vdim, rank, window, scale, ctx, cache, rot):
        """Cached rows are [latent; turned key part]; a query head is [dim plain; rot turned] elements."""
        T, P = q_rows.shape[0], cache.page_size
        q = q_rows[:, :heads * (dim + rot)].to(self.acc).view(T, heads, dim + rot)
        uk, uv = w_uk.to(self.acc).view(heads, dim, rank), w_uv.to(self.acc).view(heads, vdim, rank)
        out = torch.empty((T, heads, vdim), dtype=q_rows.dtype, device=q_rows.device)
        pos_all, req_all, slots = ctx.positions.tolist(), ctx.token_req.tolist(), ctx.req_slot.tolist()
        for t in range(T):
            pos, slot = pos_all[t], slots[req_all[t]]
            first = max(0, pos - window + 1) if window else 0
            keys = torch.arange(first, pos + 1, device=q_rows.device)
            pages = cache.block_table[slot, keys // P].long()
            rows = cache.kv[pages, 0, 0, keys % P, :].to(self.acc)         # [n, rank + rot]
            C, Kt = rows[:, :rank], rows[:, rank:]
            for h in range(heads):
                s = (C @ (uk[h].t() @ q[t, h, :dim]) + Kt @ q[t, h, dim:]) * scale
                if sinks is not None:
                    s = torch.cat([s, sinks[h:h + 1].to(self.acc)])
                p = torch.softmax(s, dim=0)[:keys.numel()]
                out[t, h] = (uv[h] @ (p @ C)).to(q_rows.dtype)
        return out.reshape(T, heads * vdim)

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def penalties(self, logits, tokens, counts, rep, freq, pres):
        R = logits.shape[0]
        for r in range(R):
            for tok, cnt in zip(tokens[r].tolist(), counts[r].tolist()):
                if tok < 0 or cnt <= 0:
                    continue
                v = logits[r, tok]
                v = v / rep[r] if v > 0 else v * rep[r]
                logits[r, tok] = v - freq[r] * cnt - pres[r]

    def logit_bias(self, logits, rows, tokens, bias):
        for r, t, b in zip(rows.tolist(), tokens.tolist(), bias.tolist()):
            logits[r, t] += b

    def sample(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step, features=3):
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        for r in range(R):
            t = float(temperature[r])
            if not t > 0:
                out[r] = int(torch.argmax(logits[r]))
                continue
            p = torch.softmax(logits[r].to(torch.float32) / t, dim=-1)
            keep = kept_mask(p, int(top_k[r]), float(top_p[r]), float(min_p[r]))
            u = philox_uniform(int(seed_lo[r]), int(seed_hi[r]), int(step[r]))
            kept = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
            c = torch.cumsum(kept, 0)
            target = u * float(c[-1])
            idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64), right=True))
            idx = min(idx, V - 1)
            while not bool(keep[idx]):
                idx -= 1
            out[r] = idx
        return out


def kept_mask(p, top_k, top_p, min_p):
    """Which probabilities survive top-k, then min-p, then the nucleus (ties at a
    threshold are kept)."""
    V = p.numel()
    thr = 0.0
    if 0 < top_k < V:
        thr = float(torch.topk(p, top_k).values[-1])
    if min_p > 0:
        thr = max(thr, min_p * float(p.max()))
    keep = p >= thr
    if 0 < top_p < 1:
        kept = torch.where(keep, p, torch.zeros_like(p))
        need = top_p * float(kept.sum())
        vals, _ = torch.sort(kept, descending=True)
        c = torch.cumsum(vals, 0)
        n = int(torch.searchsorted(c, torch.tensor(need, dtype=c.dtype))) + 1
        n = min(n, V)
        thr = max(thr, float(vals[n - 1]))
        keep = p >= thr
    return keep


def philox_uniform(key0, key1, c0, c1=0, c2=0, c3=0):
    """First word of Philox4x32-10 as a float in [0, 1) with 24 bits."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    key0, key1, c0, c1, c2, c3 = (v & mask for v in (key0, key1, c0, c1, c2, c3))
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & mask, p1 >> 32, p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ key0) & mask, lo1, (hi0 ^ c3 ^ key1) & mask, lo0
        key0, key1 = (key0 + W0) & mask, (key1 + W1) & mask
    return (c0 >> 8) / 16777216.0
