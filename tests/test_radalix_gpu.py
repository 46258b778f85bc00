"""Radalix on the GPU: every new kernel alone against the plain kernel statements (themselves held to the plain
implementation by the CPU tests), attention with planted keys, then whole models through the step function, the
replay program and the engine."""
import math

import numpy as np
import pytest
import torch

import helpers
import radalix_models as rm
from plain import plain_radalix as P
from plain.plain_kernels import PlainKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def radalix_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(rm.configs().items()):
        out[name] = (rm.write_model(raw, tmp_path_factory.mktemp(f"radalix_{name}"), seed=31 + i), page, raw)
    return out


class _Ctx:
    """The few fields of a step context that the kernels of this file read, on a device."""

    def __init__(self, spans, slots, device):
        cu, pos, req = [0], [], []
        for r, (start, n) in enumerate(spans):
            cu.append(cu[-1] + n)
            pos += list(range(start, start + n))
            req += [r] * n
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        self.cu_seqlens, self.positions, self.token_req, self.req_slot = mk(cu), mk(pos), mk(req), mk(slots)
        self.num_requests, self.num_tokens = len(spans), cu[-1]
        self.spans, self.slots_host = list(spans), list(slots)
        self.max_span = max(n for _s, n in spans)
        self.max_kv_len = max(s + n for s, n in spans)
        self.extra, self.extra_len = {}, {}


def _steps(lens_per_step, slot_of):
    """[(spans, slots)] for requests that bring lens_per_step[step][request] tokens (0: the request sits the step out)."""
    starts = [0] * len(slot_of)
    for lens in lens_per_step:
        spans, slots = [], []
        for q, n in enumerate(lens):
            if n:
                spans.append((starts[q], n))
                slots.append(slot_of[q])
                starts[q] += n
        yield spans, slots


# ------------------------------------------------------------------ the scan with a decayed matrix state

@pytest.mark.parametrize("mode", ["sigmoid_root", "softplus_step"])
@pytest.mark.parametrize("H,G,dk,dv", [(3, 3, 8, 16), (4, 2, 12, 8), (2, 1, 56, 24), (6, 6, 16, 16), (1, 1, 6, 10), (5, 1, 5, 6),
                                       (2, 2, 128, 64), (4, 4, 64, 128), (2, 1, 200, 24), (3, 3, 32, 1), (8, 2, 24, 40)])
def test_decay_scan_over_steps_and_requests(cuda_kernels, mode, H, G, dk, dv):
    """Three requests over four steps: portions of 1 to 37 tokens (more and fewer than the kernel stages at once), a request
    that sits a step out, states in slots that lie inside longer rows, inputs that are slices of wider rows; against the
    plain statement, outputs and states."""
    if mode == "sigmoid_root" and G != H:
        G = H                                                              # the channel decay's keys are per head
    front = 24                                                             # floats of another part's state first
    plain = PlainKernels(wide=True)
    state_g = torch.zeros(4, front + H * dk * dv, dtype=torch.float32, device=DEV)
    state_p = torch.zeros(4, front + H * dk * dv, dtype=F64)
    g = torch.Generator().manual_seed(H * 1000 + dk * 10 + dv)
    bias, rate, skip = 1.5 * torch.randn(H, generator=g), torch.rand(H, generator=g) * 2.5 - 1.0, torch.randn(H, generator=g)
    kw = {"decay": mode, "tau": 3.0, "q_scale": dk ** -0.5} if mode == "sigmoid_root" else \
        {"decay": mode, "step_bias": bias, "log_rate": rate, "skip": skip}
    to_dev = lambda d: {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in d.items()}
    for step, (spans, slots) in enumerate(_steps([(37, 1, 5), (1, 16, 0), (2, 17, 1), (1, 1, 1)], [3, 0, 2])):
        T = sum(n for _s, n in spans)
        wide = torch.randn(T, 2 * G * dk + H * dv + 5, generator=g)         # q | k | v side by side in one wider row
        q, k, v = wide[:, :G * dk], wide[:, G * dk:2 * G * dk], wide[:, 2 * G * dk:2 * G * dk + H * dv]
        raw = 2.0 * torch.randn(T, H * dk if mode == "sigmoid_root" else H, generator=g)
        want = plain.decay_scan(q.double(), k.double(), v.double(), raw.double(), state_p[:, front:], _Ctx(spans, slots, "cpu"),
                                heads=H, groups=G, dk=dk, dv=dv, **kw)
        wg = wide.to(DEV)
        got = cuda_kernels.decay_scan(wg[:, :G * dk], wg[:, G * dk:2 * G * dk], wg[:, 2 * G * dk:2 * G * dk + H * dv], raw.to(DEV),
                                      state_g[:, front:], _Ctx(spans, slots, DEV), heads=H, groups=G, dk=dk, dv=dv, **to_dev(kw))
        scale = max(1.0, float(want.abs().max()))
        assert got.dtype == torch.float32 and float((got.double().cpu() - want.double()).abs().max()) <= 3e-5 * scale, (step, H, dk, dv)
        assert float((state_g.double().cpu() - state_p).abs().max()) <= 3e-5 * max(1.0, float(state_p.abs().max()))
    assert float(state_g[1].abs().max()) == 0.0 and float(state_g[:, :front].abs().max()) == 0.0


@pytest.mark.parametrize("mode", ["sigmoid_root", "softplus_step"])
def test_decay_scan_is_the_same_however_it_is_cut(cuda_kernels, mode):
    H, dk, dv, T = 2, 48, 40, 53
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(T, H * d, generator=g).to(DEV) for d in (dk, dk, dv))
    raw = torch.randn(T, H * dk if mode == "sigmoid_root" else H, generator=g).to(DEV)
    vec = [torch.randn(H, generator=g).to(DEV) for _ in range(3)]
    kw = {"decay": mode, "tau": 5.0} if mode == "sigmoid_root" else {"decay": mode, "step_bias": vec[0], "log_rate": vec[1], "skip": vec[2]}

    def run(cuts, others=0):
        state = torch.zeros(3, H * dk * dv, dtype=torch.float32, device=DEV)
        out, pos = [], 0
        for n in cuts:
            sl = slice(pos, pos + n)
            spans, slots = [(pos, n)], [1]
            parts = [q[sl], k[sl], v[sl], raw[sl]]
            if others:                                                   # another request's tokens in front, in the same step
                spans, slots = [(0, others)] + spans, [2, 1]
                parts = [torch.cat([full[:others] * 0.5, p]) for full, p in zip((q, k, v, raw), parts)]
            y = cuda_kernels.decay_scan(*[p.contiguous() for p in parts], state, _Ctx(spans, slots, DEV), heads=H, groups=H, dk=dk, dv=dv, **kw)
            out.append(y[others:])
            pos += n
        return torch.cat(out), state[1].clone()
    whole, s0 = run([T])
    for cuts, others in (([1] * T, 0), ([16, 16, 16, 5], 0), ([2, 31, 1, 17, 2], 0), ([20, 33], 7)):
        got, s1 = run(cuts, others)
        assert torch.equal(got, whole) and torch.equal(s0, s1), cuts


def test_decay_scan_keeps_what_was_written_long_ago(cuda_kernels):
    """Decays next to one: what token 3 wrote is read back by token 600 (q along k_3), through dozens of stretches of
    staged tokens, in a prompt and in single decoded tokens."""
    H, dk, dv, T = 2, 32, 24, 601
    g = torch.Generator().manual_seed(4)
    q, k, v = torch.randn(T, H * dk, generator=g), 0.02 * torch.randn(T, H * dk, generator=g), torch.randn(T, H * dv, generator=g)
    k[3] = 3.0 * torch.randn(H * dk, generator=g)                           # little is written, but by token 3
    k3 = k[3].view(H, dk)
    q[600] = (k3 / (k3 * k3).sum(-1, keepdim=True)).reshape(-1) * 50.0
    raw = torch.full((T, H * dk), 14.0)                                     # sigmoid(14)^(1/2): 0.9999996
    plain = PlainKernels(wide=True)
    sp = torch.zeros(1, H * dk * dv, dtype=F64)
    want = plain.decay_scan(q.double(), k.double(), v.double(), raw.double(), sp, _Ctx([(0, T)], [0], "cpu"), heads=H, groups=H,
                            dk=dk, dv=dv, decay="sigmoid_root", tau=2.0).double()
    cos = torch.nn.functional.cosine_similarity(want[600].view(H, dv), v[3].view(H, dv).double(), dim=-1)
    assert float(cos.min()) > 0.97, "the test's own construction does not read token 3 back"
    for cuts in ([T], [590] + [1] * 11):
        sg = torch.zeros(1, H * dk * dv, dtype=torch.float32, device=DEV)
        out, pos = [], 0
        for n in cuts:
            sl = slice(pos, pos + n)
            out.append(cuda_kernels.decay_scan(q[sl].to(DEV), k[sl].to(DEV), v[sl].to(DEV), raw[sl].to(DEV), sg, _Ctx([(pos, n)], [0], DEV),
                                               heads=H, groups=H, dk=dk, dv=dv, decay="sigmoid_root", tau=2.0))
            pos += n
        got = torch.cat(out).double().cpu()
        assert float((got - want).abs().max()) < 2e-4 * float(want.abs().max()), cuts
        assert float((sg.double().cpu() - sp).abs().max()) < 2e-4 * float(sp.abs().max())


# ------------------------------------------------------------------ rows: two norms, gated norms, the pair's sum, vectors

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("C", [48, 64, 320, 4104])
def test_two_norms_pair_sum_and_vector_sum(cuda_kernels, dtype, tol, C):
    plain = PlainKernels(wide=True)
    g = torch.Generator().manual_seed(C)
    T = 7
    x = 3.0 * torch.randn(T, C, generator=g)
    wa, wb = 1 + 0.3 * torch.randn(C, generator=g), 1 + 0.3 * torch.randn(C, generator=g)
    want = plain.rmsnorm_pair(x.double().clone(), wa, 1e-6, wb, 1e-3, F64)
    got = cuda_kernels.rmsnorm_pair(x.to(DEV), wa.to(DEV), 1e-6, wb.to(DEV), 1e-3, dtype)
    for a, b in zip(got, want):
        assert a.dtype == dtype and float((a.double().cpu() - b).abs().max()) <= tol * float(b.abs().max())
    a, b = torch.randn(T, C, generator=g).to(dtype), (5.0 * torch.randn(T, C, generator=g))
    for w in ((wa, wb), (None, None)):
        want = plain.pair_combine(a.double(), b.double(), w[0], w[1], 0.5, 1.7, 1e-6)
        got = cuda_kernels.pair_combine(a.to(DEV), b.to(DEV), None if w[0] is None else w[0].to(DEV), None if w[1] is None else w[1].to(DEV),
                                        0.5, 1.7, 1e-6)
        assert got.dtype == torch.float32 and float((got.double().cpu() - want.double()).abs().max()) <= 3e-6 * float(want.abs().max())
    f, f2 = torch.randn(T, C, generator=g).to(dtype), torch.randn(T, C, generator=g).to(dtype)
    from inferflux_b200.parts import VectorScaledDelta
    for args in ((b, wa, f, wb, f2), (b, wa, f, wb, None), (b, wa, None, None, None), (b, None, f, None, f2)):
        xp, xg = x.double().clone(), x.clone().to(DEV)
        plain.residual_add_vectors(xp, *[None if t is None else t.double() for t in args])
        cuda_kernels.residual_add_vectors(xg, *[None if t is None else t.to(DEV) for t in args])
        assert float((xg.double().cpu() - xp).abs().max()) <= 3e-6 * float(xp.abs().max())
        # the same sum inside the kernel of the two norms
        xq = x.clone().to(DEV)
        got = cuda_kernels.rmsnorm_pair(xq, wa.to(DEV), 1e-6, wb.to(DEV), 1e-3, dtype,
                                        vectors=VectorScaledDelta(*[None if t is None else t.to(DEV) for t in args]))
        want = plain.rmsnorm_pair(xp.clone(), wa, 1e-6, wb, 1e-3, F64)
        assert float((xq.double().cpu() - xp).abs().max()) <= 3e-6 * float(xp.abs().max())
        for u, v_ in zip(got, want):
            assert float((u.double().cpu() - v_).abs().max()) <= tol * float(v_.abs().max())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("C,groups,shared", [(64, 4, True), (48, 1, False), (320, 5, False), (96, 3, True), (30, 5, True), (2048, 2, False)])
def test_gated_norm_over_parts_and_gates(cuda_kernels, dtype, tol, C, groups, shared):
    plain = PlainKernels(wide=True)
    g = torch.Generator().manual_seed(C + groups)
    T = 9
    y = 2.0 * torch.randn(T, C, generator=g)
    wide = 2.0 * torch.randn(T, C + 11, generator=g)                         # the gate: a slice of wider rows
    w = 1 + 0.3 * torch.randn(C // groups if shared else C, generator=g)
    for first in (True, False):
        want = plain.gated_groupnorm(y.double(), wide[:, 3:3 + C].double(), w, 1e-5, groups, first, F64)
        got = cuda_kernels.gated_groupnorm(y.to(DEV), wide.to(DEV)[:, 3:3 + C], w.to(DEV), 1e-5, groups, first, dtype)
        assert got.dtype == dtype and float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    a, gate = torch.randn(T, C, generator=g).to(dtype), (3.0 * torch.randn(T, C, generator=g)).to(dtype)
    for kind in ("sigmoid", "silu"):
        want = plain.gate_mul(a.double(), gate.double(), kind)
        got = cuda_kernels.gate_mul(a.to(DEV), gate.to(DEV), kind)
        assert got.dtype == dtype and float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bigram_rows_and_the_token_before_a_step(cuda_kernels, dtype):
    """Three requests over four steps; the token before a step's first one comes from the request's slot, position 0 takes the
    table's last row, hashes beyond 32 bits are taken in 64."""
    plain = PlainKernels(wide=True)
    vocab, H, buckets, mp, mc = 50000, 40, 2039, 1_000_003, 999_983
    g = torch.Generator().manual_seed(2)
    table = torch.randn(buckets + 1, H, generator=g).to(dtype)
    sg, sp = torch.zeros(4, 1, dtype=torch.int32, device=DEV), torch.zeros(4, 1, dtype=torch.int32)
    for spans, slots in _steps([(5, 1, 2), (1, 3, 0), (2, 1, 1), (1, 1, 7)], [3, 0, 2]):
        T = sum(n for _s, n in spans)
        ids = torch.randint(0, vocab, (T,), generator=g, dtype=torch.int32)
        x = torch.randn(T, H, generator=g)
        xp, xg = x.double().clone(), x.clone().to(DEV)
        cp, cg = _Ctx(spans, slots, "cpu"), _Ctx(spans, slots, DEV)
        plain.bigram_add(xp, table.double(), ids, sp, mp, mc, buckets, vocab, cp)
        cuda_kernels.bigram_add(xg, table.to(DEV), ids.to(DEV), sg, mp, mc, buckets, vocab, cg)
        assert float((xg.double().cpu() - xp).abs().max()) <= 1e-6 and torch.equal(sg.cpu(), sp)
        assert float((xp - x.double()).abs().max()) > 0.1


# ------------------------------------------------------------------ convolution with its options

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("taps,C,col0,width", [(3, 64, 0, 64), (4, 80, 32, 120), (2, 37, 5, 50), (1, 16, 0, 16), (5, 24, 8, 40), (4, 384, 128, 600)])
def test_convolution_alone_with_bias_activation_and_column_slices(cuda_kernels, dtype, tol, taps, C, col0, width):
    plain = PlainKernels(wide=True)
    g = torch.Generator().manual_seed(taps * 100 + C)
    w, bias = 0.6 * torch.randn(C, taps, generator=g), 0.5 * torch.randn(C, generator=g)
    front = 12
    sg = torch.zeros(4, front + max(1, taps - 1) * C, dtype=torch.float32, device=DEV)
    sp = torch.zeros(4, front + max(1, taps - 1) * C, dtype=F64)
    view = lambda s: None if taps < 2 else s[:, front:front + (taps - 1) * C].unflatten(1, (1, taps - 1, C))
    for opts in ({"add_input": False}, {"add_input": False, "bias": bias, "act": "silu"}, {"add_input": True, "bias": bias}):
        sg.zero_(), sp.zero_()
        for spans, slots in _steps([(9, 1, 2), (1, 3, 0), (2, 17, 1), (1, 1, 1)], [3, 0, 2]):
            T = sum(n for _s, n in spans)
            h = torch.randn(T, width, generator=g).to(dtype)
            cols = None if (col0 == 0 and width == C) else (col0, C)
            want = plain.short_conv(h.double(), w, taps, view(sp), 0, _Ctx(spans, slots, "cpu"), columns=cols, **opts)
            go = {k: (v.to(DEV) if torch.is_tensor(v) else v) for k, v in opts.items()}
            got = cuda_kernels.short_conv(h.to(DEV), w.to(DEV), taps, view(sg), 0, _Ctx(spans, slots, DEV), columns=cols, **go)
            assert got.shape == (T, C) and float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
            assert float((sg.double().cpu() - sp).abs().max()) <= 1e-6
        assert float(sg[:, :front].abs().max()) == 0.0


# ------------------------------------------------------------------ sigmoid routing, plain gated experts

@pytest.mark.parametrize("n,top", [(5, 1), (20, 3), (7, 7), (300, 8), (1, 1), (2, 2), (14, 5)])
def test_router_sigmoid_scores_over_the_chosen_sum(cuda_kernels, n, top):
    plain = PlainKernels(wide=True)
    z = 3.0 * torch.randn(33, n, generator=torch.Generator().manual_seed(n * 10 + top))
    ids_p, w_p = plain.moe_route(z.double(), None, top, kind="sigmoid_normalized", floor=1e-20)
    ids_g, w_g = cuda_kernels.moe_route(z.to(DEV), None, top, kind="sigmoid_normalized", floor=1e-20)
    assert torch.equal(ids_g.cpu(), ids_p) and float((w_g.cpu() - w_p).abs().max()) < 2e-6
    assert float((w_g.sum(-1) - 1).abs().max()) < 1e-5
    lone = torch.full((2, n), -200.0)                                          # every score underflows: the floor keeps the division finite
    _i, w0 = cuda_kernels.moe_route(lone.to(DEV), None, top, kind="sigmoid_normalized", floor=1e-20)
    assert bool(torch.isfinite(w0).all())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,width,ff,experts,top", [(5, 64, 40, 5, 2), (1, 48, 24, 1, 1), (33, 96, 16, 7, 7), (9, 192, 56, 10, 3)])
def test_plain_gated_experts_few_tokens(cuda_kernels, dtype, tol, T, width, ff, experts, top):
    plain = PlainKernels(wide=True)
    g = torch.Generator().manual_seed(T + width)
    h = torch.randn(T, width, generator=g).to(dtype)
    w_up, w_down = (0.3 * torch.randn(experts, 2 * ff, width, generator=g)).to(dtype), (0.3 * torch.randn(experts, width, ff, generator=g)).to(dtype)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, top, generator=g)
    glu = (float("inf"), 1.0, 0.0)
    want = plain.moe_experts(h, w_up, w_down, ids, wts, experts, F64, glu=glu)
    got = cuda_kernels.moe_experts(h.to(DEV), w_up.to(DEV), w_down.to(DEV), ids.to(DEV), wts.to(DEV), experts, dtype, glu=glu)
    assert float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    silu = lambda z: z * torch.sigmoid(z)                                      # the activation itself, from its definition
    t, e = 0, int(ids[0, 0])
    both = w_up[e].double() @ h[t].double()
    assert torch.allclose(plain.moe_experts(h[:1], w_up, w_down, ids[:1, :1], torch.ones(1, 1), experts, F64, glu=glu)[0],
                          w_down[e].double() @ (silu(both[:ff]) * both[ff:]).to(dtype).double(), atol=1e-9)


@pytest.mark.parametrize("T,width,ff,experts,top", [(300, 128, 96, 6, 2), (700, 320, 72, 8, 3), (256, 64, 200, 3, 3)])
def test_plain_gated_experts_sorted_tiles_against_the_per_token_kernels(cuda_kernels, monkeypatch, T, width, ff, experts, top):
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, width, generator=g).to(torch.bfloat16).to(DEV)
    w_up = (0.2 * torch.randn(experts, 2 * ff, width, generator=g)).to(torch.bfloat16).to(DEV)
    w_down = (0.2 * torch.randn(experts, width, ff, generator=g)).to(torch.bfloat16).to(DEV)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, top, generator=g).to(DEV)
    glu = (float("inf"), 1.0, 0.0)
    tiles = cuda_kernels.moe_experts(h, w_up, w_down, ids, wts, experts, torch.bfloat16, glu=glu)
    monkeypatch.setenv("INFERFLUX_B200_MOE_TILES", "0")
    rows = cuda_kernels.moe_experts(h, w_up, w_down, ids, wts, experts, torch.bfloat16, glu=glu)
    cuda_kernels.check_errors()
    assert float((tiles.double() - rows.double()).abs().max()) <= 3e-2 * max(1.0, float(rows.double().abs().max()))


# ------------------------------------------------------------------ attention with planted keys

def _cache(dtype, nkv, row, page, window, device, tokens=400):
    pages = -(-tokens // page)
    from inferflux_b200.cache.manager import CacheManager
    from inferflux_b200.parts.base import KVCacheSpec
    return CacheManager([(KVCacheSpec(nkv, row, window), None)], page_size=page, num_pages=pages, max_seqs=4, max_seq_len=page * pages,
                        dtype=dtype, device=device)


def _step_ctx(kernels, dtype, cache, spans, device):
    from inferflux_b200.engine.batch import StepContext, StepEntry
    entries, starts, slots = [], [], []
    for rid, n in spans:
        if rid not in cache:
            cache.add_request(rid)
        start = cache.length(rid)
        cache.reserve(rid, start + n)
        entries.append(StepEntry(rid, [0] * n, []))
        starts.append(start)
        slots.append(cache.slot(rid))
    ctx = StepContext.build(kernels, dtype, device, entries, starts, slots, cache.drain_table_updates())
    for g, (idx, page) in zip(cache.groups, ctx.table_updates):
        kernels.scatter_i32(g.table, idx, page)
    for (rid, n), s in zip(spans, starts):
        cache.commit(rid, s + n)
    return ctx


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("nq,nkv,d,dv,page,window,rot,q_temp", [
    (4, 2, 16, 8, 8, 21, 8, None), (2, 1, 64, 32, 16, 150, 16, None), (3, 3, 12, 12, 4, 7, 12, None), (4, 2, 64, 64, 16, None, 0, (0.3, 128)),
    (2, 2, 24, 48, 16, 16, 0, (1.5, 9)), (8, 4, 64, 64, 16, 100, 32, None)])
def test_attention_planted_keys_window_edges_sink_and_far_keys(cuda_kernels, dtype, tol, nq, nkv, d, dv, page, window, rot, q_temp):
    """A prompt of 300 tokens and then 40 decoded ones.  For sixteen queries one key is planted (a large product with that
    query alone, along a direction of its own in the part of a head that no rotation turns): as far back as the query
    sees, at the first key of its window, just outside the window, and at a page's border.  The kernels' output must be
    the planted key's value when the key is seen and must not be when it is not, in prompt rows and in decoded rows, with
    a learned sink per head in the denominator; and it must agree with the plain statement."""
    from inferflux_b200.config.plan import ScheduleEntry
    from inferflux_b200.parts.base import RotaryTable
    n_prompt, n_all = 300, 340
    g = torch.Generator().manual_seed(nq * 100 + d)
    q = 0.3 * torch.randn(n_all, nq, d, generator=g)
    k = 0.3 * torch.randn(n_all, nkv, d, generator=g)
    v = torch.randn(n_all, nkv, dv, generator=g)
    sink = 2.0 * torch.randn(nq, generator=g)
    w = window or 10 ** 6
    free = d - rot                                                           # elements of a head that stay unturned
    plants = {}                                                              # query position -> (key position, seen)
    if free >= 8:
        count, used = 0, set()
        for base in (240, 284, 302, 326):                                   # queries in the prompt and among the decoded tokens
            for j in range(4):
                p = base + 3 * j
                first = max(0, p - w + 1)
                # a key well inside what is seen (far back without a window), the first key seen, the last one not seen
                # any more, and the first key of the page before the query's
                kp, seen = [(first + 2 if window else 3 + count, True), (first, True), (p - w, False),
                            (max(first, (p // page - 1) * page), True)][j]
                if kp < 0 or kp in used:                                     # every planted key serves one query
                    continue
                used.add(kp)
                direction = torch.zeros(d)
                direction[rot + count % free] = 12.0 if count < free else -12.0     # a signed axis of its own
                count += 1
                q[p] = 0.05 * torch.randn(nq, d, generator=g) + direction
                k[kp] = 0.05 * torch.randn(nkv, d, generator=g) + direction
                plants[p] = (kp, seen)
        assert len(plants) >= 8 and count <= 2 * free and any(not seen for _k, seen in plants.values()) == bool(window)
    scale = 1.0 / math.sqrt(d)
    freqs = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    outs = {}
    for name, kern, dev, dt in (("plain", PlainKernels(wide=True), "cpu", F64), ("cuda", cuda_kernels, DEV, dtype)):
        cache = _cache(dt, nkv, -(-max(d, dv) // 8) * 8, page, window, dev)
        rt = None if not rot else RotaryTable(freqs.to(dev), rot, True, 1.07)
        got, pos = [], 0
        for n in [n_prompt] + [1] * (n_all - n_prompt):
            ctx = _step_ctx(kern, dt, cache, [("r", n)], dev)
            view = cache.view(ScheduleEntry(layer=0, cache=0))
            sl = slice(pos, pos + n)
            qkv = torch.cat([q[sl].reshape(n, -1), k[sl].reshape(n, -1), v[sl].reshape(n, -1)], dim=1).to(dt).to(dev)
            qq = kern.rope_append(qkv, None, rt, nq, nkv, d, ctx, view, dv=dv, q_temp=q_temp)
            got.append(kern.attention(qq, nq, nkv, d, window, scale, ctx, view, sink=sink.to(dev), dv=dv).double().cpu())
            pos += n
        outs[name] = torch.cat(got).view(n_all, nq, dv)
    err = float((outs["cuda"] - outs["plain"]).abs().max())
    assert err <= tol * max(1.0, float(outs["plain"].abs().max())), err
    per = nq // nkv
    for p, (kp, seen) in plants.items():
        for h in range(nq):
            close = float((outs["cuda"][p, h] - v[kp, h // per].double()).abs().max())
            assert (close < 0.1) == seen, (p, kp, seen, h, close)


# ------------------------------------------------------------------ whole models

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


@pytest.fixture(scope="module")
def oracle(radalix_dirs):
    memo = {}

    def get(name):
        if name not in memo:
            d, _page, raw = radalix_dirs[name]
            reqs = rm.requests_for(raw, LENS, 100)
            memo[name] = {"reqs": reqs, "float32": rm.plain_logits(d, reqs),
                          "bfloat16": rm.plain_logits(d, reqs, weights_as=torch.bfloat16),
                          "yard": rm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16)}
        return memo[name]
    return get


def _runner(d, dtype, page, kernels, pages=None, **kw):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype=dtype, device=DEV)
    return ModelRunner(model, kernels, page_size=page, num_pages=pages or 256 // page, max_seqs=4, max_seq_len=512, **kw)


def _bf16_close(name, got, want, yard):
    """bfloat16 logits against the exact ones, with the plain implementation in bfloat16 arithmetic on the same rounded
    weights as the yardstick.  The test models are sharp and their routers decide by small margins, so two correct
    bfloat16 computations differ by about as much as either differs from the exact result: up to three times the
    yardstick's worst row, twice on average.  A router whose margin is below what rounding moves sends a token to
    another expert in one computation and not in the other; both are right, so one row in fifty may lie further out."""
    err, bound = np.abs(got - want).max(axis=1), np.abs(yard - want).max(axis=1)
    far = int((err > 3.0 * float(bound.max())).sum())
    assert far <= max(1, len(err) // 50) and float(err.max()) <= 12.0 * float(bound.max()), \
        f"{name}: row {int(err.argmax())} is off by {float(err.max()):.4f} ({far} rows far out); rounding alone gives {float(bound.max()):.4f}"
    assert float(err.mean()) <= 2.0 * float(bound.mean()), f"{name}: mean error {float(err.mean()):.4f} against {float(bound.mean()):.4f}"


def _check(name, dtype, got, o):
    if dtype == "float32":
        top = max(float(np.abs(v).max()) for v in o["float32"].values())
        bad = helpers.first_bad(got, o["float32"], 2e-4 + 1e-5 * top)
        assert bad is None, f"{name}: first wrong row (request, position, diff): {bad}"
    else:
        for rid in o["reqs"]:
            _bf16_close(f"{name} {rid}", got[rid], o["bfloat16"][rid], o["yard"][rid])


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_step_function_cuttings(name, dtype, cutting, radalix_dirs, oracle, cuda_kernels):
    d, page, raw = radalix_dirs[name]
    o = oracle(name)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](o["reqs"])
    runner = _runner(d, dtype, page, cuda_kernels, cuda_graphs=(cutting == "tail"))
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    cuda_kernels.check_errors()
    _check(f"{name} {cutting}", dtype, got, o)
    assert not runner.cache.live_requests()


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_is_the_same_under_every_cutting(name, radalix_dirs, oracle, cuda_kernels):
    d, page, raw = radalix_dirs[name]
    reqs = oracle(name)["reqs"]
    results = []
    for make in (helpers.trace_whole, helpers.trace_tail, helpers.trace_portions, lambda r: helpers.trace_mixed(r, 256)):
        steps = make(reqs)
        runner = _runner(d, "float32", page, cuda_kernels)
        results.append(helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"]))
    for other in results[1:]:
        for rid in reqs:
            assert np.array_equal(results[0][rid], other[rid]), rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens_from_the_first_token_on(dtype, radalix_dirs, cuda_kernels):
    from inferflux_b200.engine import StepEntry
    d, page, raw = radalix_dirs["A"]
    toks = rm.requests_for(raw, [60], 3)["r0"]
    rounded = torch.bfloat16 if dtype == "bfloat16" else None
    want = rm.plain_logits(d, {"r0": toks}, weights_as=rounded)["r0"]
    yard = rm.plain_logits(d, {"r0": toks}, weights_as=torch.bfloat16, dtype=torch.bfloat16)["r0"]
    runner = _runner(d, dtype, page, cuda_kernels)
    got, pos, sizes, i = [], 0, [2, 1, 3, 2, 2, 5, 1, 1, 2, 17], 0
    while pos < len(toks):
        n = min(sizes[i % len(sizes)], len(toks) - pos)
        i += 1
        got += list(runner.step([StepEntry("r0", toks[pos:pos + n], list(range(n)))]).cpu().numpy())
        pos += n
    runner.end_request("r0")
    cuda_kernels.check_errors()
    if dtype == "float32":
        assert float(np.abs(np.stack(got) - want).max()) < 3e-4
    else:
        _bf16_close("short portions", np.stack(got), want, yard)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_medium_model_with_long_prompts(dtype, tmp_path, cuda_kernels):
    """Prompts of 700 and 300 tokens through a model of four layers: whole, then in portions of 200 and 128 beside each
    other's decoded tokens.  These steps reach the kernels of many rows (library and tcgen05 products, sorted expert tiles
    with the gated activation, the tiled attention kernels with a learned sink and a window, the scan's long spans) inside
    a whole model."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    raw, page = rm.medium_config()
    d = rm.write_model(raw, tmp_path / "medium", seed=77)
    reqs = rm.requests_for(raw, [700, 300], 12)
    rows = {"r0": [0, 1, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512, 640, 698, 699], "r1": [0, 63, 64, 127, 128, 200, 298, 299]}
    rounded = torch.bfloat16 if dtype == "bfloat16" else None
    want = {k: v[rows[k]] for k, v in rm.plain_logits(d, reqs, weights_as=rounded).items()}
    yard = {k: v[rows[k]] for k, v in rm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16).items()} \
        if dtype == "bfloat16" else None

    def compare(name, got):
        for rid in reqs:
            if dtype == "float32":
                assert float(np.abs(got[rid] - want[rid]).max()) < 5e-4, (name, rid, float(np.abs(got[rid] - want[rid]).max()))
            else:
                _bf16_close(f"{name} {rid}", got[rid], want[rid], yard[rid])
    _c, model = load_model(d, dtype=dtype, device=DEV)
    runner = ModelRunner(model, cuda_kernels, page_size=page, num_pages=80, max_seqs=4, max_seq_len=1024)
    got = {}
    for rid, toks in reqs.items():
        got[rid] = runner.step([StepEntry(rid, toks, rows[rid])]).cpu().numpy()
        runner.end_request(rid)
    cuda_kernels.check_errors()
    compare("whole", got)
    got = {rid: {} for rid in reqs}
    at = {"r0": 0, "r1": 0}
    size = {"r0": 200, "r1": 128}
    while any(at[r] < len(reqs[r]) for r in reqs):
        entries, asked = [], []
        for rid, toks in reqs.items():
            if at[rid] >= len(toks):
                continue
            n = 1 if len(toks) - at[rid] <= 20 else min(size[rid], len(toks) - 20 - at[rid])
            w = [p - at[rid] for p in rows[rid] if at[rid] <= p < at[rid] + n]
            entries.append(StepEntry(rid, toks[at[rid]:at[rid] + n], w))
            asked += [(rid, p) for p in rows[rid] if at[rid] <= p < at[rid] + n]
            at[rid] += n
        out = runner.step(entries).cpu().numpy()
        for (rid, p), row in zip(asked, out):
            got[rid][p] = row
        for rid in reqs:
            if at[rid] == len(reqs[rid]) and rid in runner.cache:
                runner.end_request(rid)
        runner.cache.check()
    cuda_kernels.check_errors()
    compare("portions", {rid: np.stack([got[rid][p] for p in rows[rid]]) for rid in reqs})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_reused_pages_slots_and_graphs(dtype, radalix_dirs, cuda_kernels):
    """12 prompt tokens, then 300 decoded one by one beside requests that join and leave: page borders and windows are
    crossed by decoded tokens, the pages and the slot of a request that left serve the next one, decode steps replay a
    CUDA graph."""
    from inferflux_b200.engine import StepEntry
    d, page, raw = radalix_dirs["A"]
    reqs = rm.requests_for(raw, [312, 90, 60], 9)
    want = rm.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    yard = rm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16) if dtype == "bfloat16" else None
    runner = _runner(d, dtype, page, cuda_kernels, pages=52, cuda_graphs=True)     # 40 pages for r0, 12 for one of the others
    a = reqs["r0"]
    got = {rid: [] for rid in reqs}
    got["r0"] += list(runner.step([StepEntry("r0", a[:12], list(range(12)))]).cpu().numpy())
    at = {"r1": 0, "r2": 0}
    for i in range(12, len(a)):
        entries, order = [StepEntry("r0", [a[i]], [0])], ["r0"]
        other = "r1" if at["r1"] < len(reqs["r1"]) else ("r2" if at["r2"] < len(reqs["r2"]) else None)
        if i >= 100 and other is not None:
            n = 7 if at[other] < 49 else 1
            n = min(n, len(reqs[other]) - at[other])
            entries.append(StepEntry(other, reqs[other][at[other]:at[other] + n], list(range(n))))
            order += [other] * n
            at[other] += n
        out = runner.step(entries).cpu().numpy()
        for rid, row in zip(order, out):
            got[rid].append(row)
        if other is not None and at[other] == len(reqs[other]) and other in runner.cache:
            runner.end_request(other)
        runner.cache.check()
    cuda_kernels.check_errors()
    assert runner.graph_replays > 50
    got = {k: np.stack(v) for k, v in got.items()}
    for rid in reqs:
        if dtype == "float32":
            assert float(np.abs(got[rid] - want[rid]).max()) < 3e-4, rid
        else:
            _bf16_close(rid, got[rid], want[rid], yard[rid])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, radalix_dirs, oracle, tmp_path):
    d, page, raw = radalix_dirs["B"]
    o = oracle("B")
    steps = helpers.trace_mixed(o["reqs"], 256)
    got = helpers.collect(steps, helpers.run_trace_cli(d, dtype, steps, tmp_path / "out", 256, raw["vocab"], page_size=page),
                          raw["vocab"])
    _check("B through the program", dtype, got, o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_engine_and_scheduler(dtype, radalix_dirs, tmp_path):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = radalix_dirs["A"]
    if dtype == "bfloat16":
        # a router that decides by less than rounding moves its outputs sends a token to another expert in one correct
        # computation and not in another, and every later token inherits the difference through the cache and the state:
        # the bfloat16 run generates with routers that choose all their experts
        raw = {**raw, "layers": [l if l["mlp"] is None else {**l, "mlp": {**l["mlp"], "router": {**l["mlp"]["router"], "top": l["mlp"]["router"]["experts"]}}}
                                 for l in raw["layers"]]}
        d = rm.write_model(raw, tmp_path / "all_chosen", seed=31)
    _raw, W = rm.load(d)
    if dtype == "bfloat16":
        W = {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in W.items()}
    prompts = list(rm.requests_for(raw, [7, 19, 33, 4, 1, 70], 40).values())
    for pages in (64, 14):                                 # 14 pages of 8: the requests do not all fit at once
        eng = Engine(d, dtype=dtype, device=DEV, kv_page_size=page, kv_num_pages=pages, kv_max_batch=4, kv_max_seq=128,
                     chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=24)
        for prompt, r in zip(prompts, res):
            seq = list(prompt) + list(r.token_ids)
            exact = P.forward(raw, W, seq)
            rough = P.forward(raw, W, seq, dtype=torch.bfloat16).double() if dtype == "bfloat16" else None
            for i, tok in enumerate(r.token_ids):
                row = len(prompt) - 1 + i
                gap = float(exact[row].max() - exact[row, tok])
                slack = 1e-3 if rough is None else 4.0 * float((rough - exact).abs().max())
                assert gap <= slack, f"token {i}: {gap:.4f} below the best logit, rounding allows {slack:.4f}"
        assert not eng.runner.cache.live_requests()
