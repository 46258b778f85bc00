"""Benarax on the GPU: every new kernel alone against the plain kernel statements (themselves held to the plain
implementation by the CPU tests), the attention part alone with planted keys, then whole models through the step
function, the replay program and the engine."""
import math

import numpy as np
import pytest
import torch

import benarax_models as bm
import helpers
from plain import plain_benarax as P
from plain.plain_kernels import PlainKernels

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


def _rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.fixture(scope="module")
def benarax_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(bm.configs().items()):
        out[name] = (bm.write_model(raw, tmp_path_factory.mktemp(f"benarax_{name}"), seed=71 + i), page, raw)
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


# ------------------------------------------------------------------ rows: norms in groups, sums, the side input's gate

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,groups", [(64, 2), (80, 5), (96, 1), (4104, 3), (48, 48)])
def test_norm_in_groups_alone_and_behind_a_normed_delta(cuda_kernels, dtype, tol, H, groups):
    plain = PlainKernels(wide=True)
    for T in (1, 7, 300):
        x, y = _rnd(T, H, seed=T, scale=2.0), _rnd(T, H, seed=T + 1).to(dtype)
        w_post, w_next = 1 + 0.2 * _rnd(H, seed=3), 1 + 0.2 * _rnd(H, seed=4)
        want = plain.rmsnorm(x.double(), w_next, 1e-5, F64, groups=groups)
        got = cuda_kernels.rmsnorm(x.to(DEV), w_next.to(DEV), 1e-5, dtype, groups=groups)
        assert got.dtype == dtype and float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
        xp = x.clone().double()
        want = plain.postnorm_add(xp, y, w_post, 1e-6, w_next, 1e-5, out_dtype=F64, groups=groups)
        xg = x.to(DEV)
        got = cuda_kernels.postnorm_add(xg, y.to(DEV), w_post.to(DEV), 1e-6, w_next.to(DEV), 1e-5, dtype, groups=groups)
        assert float((xg.cpu().double() - xp).abs().max()) < 1e-5
        # the norm of the rows as the kernel's float32 sum left them (a group of one element near zero turns the
        # sum's last bit into much more)
        want = plain.rmsnorm(xg.cpu().double(), w_next, 1e-5, F64, groups=groups)
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("taps", [2, 3, 4])
def test_single_tokens_sum_norm_and_convolution_in_one_kernel(cuda_kernels, dtype, tol, taps):
    """Steps of one token per request: the kernel that adds the normed delta and norms the row also makes h + conv(h)
    from the state's rows and moves the state on; against the two kernels one after the other, and the plain ones."""
    H, groups, slots = 80, 5, [2, 0, 3]
    plain = PlainKernels(wide=True)
    w_post, w_next, cw = 1 + 0.2 * _rnd(H, seed=3), 1 + 0.2 * _rnd(H, seed=4), _rnd(H, taps, seed=5, scale=0.6)
    state_p = torch.zeros(4, 1, taps - 1, H, dtype=F64)
    state_a = torch.zeros(4, 1, taps - 1, H, dtype=torch.float32, device=DEV)
    state_b = state_a.clone()
    for step in range(taps + 2):
        ctx_p, ctx_g = _Ctx([(step, 1)] * 3, slots, "cpu"), _Ctx([(step, 1)] * 3, slots, DEV)
        x, y = _rnd(3, H, seed=10 + step, scale=2.0), _rnd(3, H, seed=20 + step).to(dtype)
        xp = x.clone().double()
        h_p = plain.postnorm_add(xp, y, w_post, 1e-6, w_next, 1e-5, out_dtype=F64, groups=groups)
        hc_p = plain.short_conv(h_p if dtype == torch.float32 else h_p.to(dtype).double(), cw, taps, state_p, 0, ctx_p)
        xa, xb = x.to(DEV), x.to(DEV)
        h_a, hc_a = cuda_kernels.postnorm_add(xa, y.to(DEV), w_post.to(DEV), 1e-6, w_next.to(DEV), 1e-5, dtype,
                                              conv=(cw.to(DEV), taps, state_a, 0, ctx_g), groups=groups, both=True)
        h_b = cuda_kernels.postnorm_add(xb, y.to(DEV), w_post.to(DEV), 1e-6, w_next.to(DEV), 1e-5, dtype, groups=groups)
        hc_b = cuda_kernels.short_conv(h_b, cw.to(DEV), taps, state_b, 0, ctx_g)
        top = float(hc_p.abs().max())
        assert torch.equal(xa, xb) and float((h_a.float() - h_b.float()).abs().max()) <= tol * 4
        assert float((hc_a.double().cpu() - hc_p).abs().max()) <= tol * top, step
        assert float((hc_b.double().cpu() - hc_p).abs().max()) <= tol * top, step
        assert float((state_a.double().cpu() - state_p).abs().max()) <= tol * top
        assert float(state_a[1].abs().max()) == 0.0                        # a slot nobody had stays untouched


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_scaled_sum_gate_times_table_and_scaled_embedding(cuda_kernels, dtype, tol):
    plain = PlainKernels(wide=True)
    T, H = 37, 72
    x, a, b = _rnd(T, H, seed=1), _rnd(T, H, seed=2).to(dtype), _rnd(T, H, seed=3).to(dtype)
    for second in (b, None):
        xp, xg = x.clone().double(), x.to(DEV)
        want = plain.residual_add_scaled(xp, a, second, 0.37, out_dtype=F64)
        got = cuda_kernels.residual_add_scaled(xg, a.to(DEV), None if second is None else second.to(DEV), 0.37, out_dtype=dtype)
        assert float((xg.cpu().double() - xp).abs().max()) < 2e-6
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
        assert cuda_kernels.residual_add_scaled(xg, a.to(DEV), None, 1.0) is None
    table, ids = _rnd(50, 40, seed=4).to(dtype), torch.randint(0, 50, (T,), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    for first, dim in ((0, 8), (13, 5), (24, 16)):
        z = _rnd(T, dim, seed=6, scale=2.0).to(dtype)
        want = plain.gelu_mul_table(z.double(), table.double(), ids, first)
        got = cuda_kernels.gelu_mul_table(z.to(DEV), table.to(DEV), ids.to(DEV), first)
        assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    emb = cuda_kernels.embed(table.to(DEV), ids.to(DEV), 50, scale=1.7)
    assert emb.dtype == torch.float32 and float((emb.cpu().double() - table[ids.long()].double() * 1.7).abs().max()) < 1e-6
    v = _rnd(9, 33, seed=7)
    vg = v.to(DEV)
    cuda_kernels.scale_(vg, 0.3)
    assert float((vg.cpu() - v * 0.3).abs().max()) < 1e-7
    rows, w = _rnd(T, 90, seed=8).to(dtype), 1 + 0.2 * _rnd(24, seed=9)
    want = plain.rmsnorm(rows[:, 40:64].double(), w, 1e-5, F64)
    got = cuda_kernels.rmsnorm_columns(rows.to(DEV), 40, 24, w.to(DEV), 1e-5)
    assert tuple(got.shape) == (T, 24) and float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())


# ------------------------------------------------------------------ the delta-rule recurrence

@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,D", [(3, 8), (2, 24), (4, 32), (2, 64), (1, 128), (2, 160), (5, 40), (1, 6)])
def test_delta_rule_over_steps_and_requests(cuda_kernels, dtype, tol, H, D):
    """Three requests over four steps: portions of 1 to 37 tokens (more and fewer than the 16 the kernel stages), a
    request that sits a step out, states carried in slots that lie inside longer rows; against the plain statement."""
    HD, front = H * D, 24                                                   # `front` floats of another part's state first
    plain = PlainKernels(wide=True)
    state_g = torch.zeros(4, front + H * D * D, dtype=torch.float32, device=DEV)
    state_p = torch.zeros(4, front + H * D * D, dtype=F64)
    g = torch.Generator().manual_seed(H * 100 + D)
    w0, ab, nw = 1.5 * torch.randn(HD, generator=g), torch.randn(HD, generator=g), 1 + 0.2 * torch.randn(HD, generator=g)
    starts = [0, 0, 0]
    for step, lens in enumerate([(37, 1, 5), (1, 16, 0), (2, 17, 1), (1, 1, 1)]):
        spans, slots = [], []
        for q, n in enumerate(lens):
            if n:
                spans.append((starts[q], n))
                slots.append([3, 0, 2][q])
                starts[q] += n
        T = sum(n for _s, n in spans)
        proj = torch.randn(T, 5 * HD + 3, generator=g)                      # rows wider than the five projections
        w_raw = 2.0 * torch.randn(T, HD, generator=g)
        want = plain.delta_rule_scan(proj.double(), w_raw.double(), w0, ab, nw, 1e-5, H, D, state_p[:, front:], _Ctx(spans, slots, "cpu"), F64)
        got = cuda_kernels.delta_rule_scan(proj.to(DEV), w_raw.to(DEV), w0.to(DEV), ab.to(DEV), nw.to(DEV), 1e-5, H, D,
                                           state_g[:, front:], _Ctx(spans, slots, DEV), dtype)
        scale = float(want.abs().max())
        assert got.dtype == dtype and float((got.double().cpu() - want).abs().max()) <= tol * max(1.0, scale), (step, H, D)
        assert float((state_g.double().cpu() - state_p).abs().max()) <= 3e-5 * max(1.0, float(state_p.abs().max()))
    assert float(state_g[1].abs().max()) == 0.0 and float(state_g[:, :front].abs().max()) == 0.0


def test_delta_rule_is_the_same_however_it_is_cut(cuda_kernels):
    H, D, T = 2, 32, 53
    g = torch.Generator().manual_seed(9)
    proj, wr = torch.randn(T, 5 * H * D, generator=g).to(DEV), torch.randn(T, H * D, generator=g).to(DEV)
    w0, ab, nw = (torch.randn(H * D, generator=g).to(DEV) for _ in range(3))

    def run(cuts, others=0):
        state = torch.zeros(3, H * D * D, dtype=torch.float32, device=DEV)
        out, pos = [], 0
        for n in cuts:
            sl = slice(pos, pos + n)
            spans, slots = [(pos, n)], [1]
            p, w = proj[sl], wr[sl]
            if others:                                                   # another request's tokens in front, in the same step
                spans, slots = [(0, others)] + spans, [2, 1]
                p, w = torch.cat([proj[:others] * 0.5, p]), torch.cat([wr[:others], w])
            y = cuda_kernels.delta_rule_scan(p.contiguous(), w.contiguous(), w0, ab, nw, 1e-6, H, D, state, _Ctx(spans, slots, DEV),
                                             torch.float32)
            out.append(y[others:])
            pos += n
        return torch.cat(out), state[1].clone()
    whole, s0 = run([T])
    for cuts, others in (([1] * T, 0), ([16, 16, 16, 5], 0), ([2, 31, 1, 17, 2], 0), ([20, 33], 7)):
        got, s1 = run(cuts, others)
        assert torch.equal(got, whole) and torch.equal(s0, s1), cuts


def test_delta_rule_keeps_what_was_written_long_ago(cuda_kernels):
    """Decays next to one and almost nothing erased: what token 3 wrote is read back by token 600 (r along k_3),
    through 38 stretches of staged tokens, in a prompt and in single decoded tokens."""
    H, D, T = 2, 32, 601
    HD = H * D
    g = torch.Generator().manual_seed(4)
    proj = torch.randn(T, 5 * HD, generator=g)
    proj[:, HD:2 * HD] *= 0.05                                             # small keys: little is written ...
    proj[3, HD:2 * HD] = 3.0 * torch.randn(HD, generator=g)                 # ... but by token 3
    k3 = proj[3, HD:2 * HD].view(H, D)
    proj[600, :HD] = (k3 / (k3 * k3).sum(-1, keepdim=True)).reshape(-1) * 50.0
    w_raw = torch.full((T, HD), -12.0)                                      # decay = exp(-0.6 sigmoid(-12)): 0.999996
    w0, ab, nw = torch.zeros(HD), torch.full((HD,), -12.0), torch.ones(HD)
    plain = PlainKernels(wide=True)
    sp = torch.zeros(1, HD * D, dtype=F64)
    want = plain.delta_rule_scan(proj.double(), w_raw.double(), w0, ab, nw, 1e-6, H, D, sp, _Ctx([(0, T)], [0], "cpu"), F64)
    # the per-head norm hides the size but not the direction: the last row points along v_3
    v3 = proj[3, 2 * HD:3 * HD].view(H, D).double()
    gate = torch.sigmoid(proj[600, 3 * HD:4 * HD].double()).view(H, D)
    cos = torch.nn.functional.cosine_similarity(want[600].view(H, D) / gate, v3, dim=-1)
    assert float(cos.min()) > 0.97, "the test's own construction does not read token 3 back"
    for cuts in ([T], [590] + [1] * 11):
        sg = torch.zeros(1, HD * D, dtype=torch.float32, device=DEV)
        out, pos = [], 0
        for n in cuts:
            out.append(cuda_kernels.delta_rule_scan(proj[pos:pos + n].to(DEV).contiguous(), w_raw[pos:pos + n].to(DEV).contiguous(),
                                                    w0.to(DEV), ab.to(DEV), nw.to(DEV), 1e-6, H, D, sg, _Ctx([(pos, n)], [0], DEV),
                                                    torch.float32))
            pos += n
        got = torch.cat(out).double().cpu()
        assert float((got - want).abs().max()) < 2e-4 * float(want.abs().max()), cuts
        assert float((sg.double().cpu() - sp).abs().max()) < 2e-4 * float(sp.abs().max())


# ------------------------------------------------------------------ routing over the chosen, gated experts

@pytest.mark.parametrize("n,top", [(5, 1), (20, 3), (7, 7), (300, 8), (1, 1), (2, 2)])
def test_router_softmax_over_the_chosen_alone(cuda_kernels, n, top):
    T = 19
    z = _rnd(T, n, seed=n, scale=2.0)
    ids, w = cuda_kernels.moe_route(z.to(DEV), None, top, of_chosen=True)
    want_ids, want_w = PlainKernels(wide=True).moe_route(z, None, top, of_chosen=True)
    assert torch.equal(ids.cpu().sort(dim=1).values, want_ids.sort(dim=1).values)
    chosen = torch.gather(z.double(), 1, ids.cpu().long())
    assert float((w.cpu().double() - torch.softmax(chosen, dim=-1)).abs().max()) < 1e-6
    assert float((w.sum(dim=1) - 1.0).abs().max()) < 1e-6
    if top < n:                                                            # not the softmax over all
        assert float((w.cpu().double() - torch.gather(torch.softmax(z.double(), -1), 1, ids.cpu().long())).abs().max()) > 1e-3


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,width,ff,experts,top,limit", [(5, 64, 40, 5, 2, 1.5), (1, 48, 24, 2, 1, 0.7), (33, 96, 16, 7, 7, 3.0),
                                                          (8, 320, 96, 8, 3, 1.0)])
def test_gated_experts_few_tokens(cuda_kernels, dtype, tol, T, width, ff, experts, top, limit):
    h = _rnd(T, width, seed=1).to(dtype)
    w_up, w_down = _rnd(experts, 2 * ff, width, seed=2, scale=0.3).to(dtype), _rnd(experts, width, ff, seed=3, scale=0.2).to(dtype)
    z = _rnd(T, experts, seed=4, scale=2.0)
    plain = PlainKernels(wide=True)
    ids, wts = plain.moe_route(z, None, top, of_chosen=True)
    want = plain.moe_experts(h.double(), w_up.double(), w_down.double(), ids, wts, experts, F64, glu=(limit, 1.702))
    got = cuda_kernels.moe_experts(h.to(DEV), w_up.to(DEV), w_down.to(DEV), ids.to(DEV), wts.to(DEV), experts, dtype, glu=(limit, 1.702))
    assert float((got.double().cpu() - want).abs().max()) <= tol * float(want.abs().max())
    both = w_up.double() @ h.double().T                                     # the clamp is met from both sides
    assert float(both[:, :ff].max()) > limit and float(both[:, ff:].max()) > limit and float(both[:, ff:].min()) < -limit


@pytest.mark.parametrize("T,width,ff,experts,top", [(300, 128, 96, 6, 2), (700, 320, 72, 8, 3), (256, 64, 200, 3, 3), (520, 96, 128, 16, 1)])
def test_gated_experts_sorted_tiles_against_the_per_token_kernels(cuda_kernels, monkeypatch, T, width, ff, experts, top):
    """From 512 (token, choice) pairs on, bfloat16 runs sorted 128-row tiles with the gated activation in the first
    product's epilogue: against the per-token kernels and the plain statement; experts nobody chose, expert sizes
    that are no multiple of the tile."""
    bf = torch.bfloat16
    h = _rnd(T, width, seed=1).to(bf)
    w_up, w_down = _rnd(experts, 2 * ff, width, seed=2, scale=0.2).to(bf), _rnd(experts, width, ff, seed=3, scale=0.2).to(bf)
    z = _rnd(T, experts, seed=4, scale=2.0)
    z[:, experts - 1] -= 100.0 if top < experts - 1 else 0.0              # an expert that nobody chooses
    plain = PlainKernels(wide=True)
    ids, wts = plain.moe_route(z, None, top, of_chosen=True)
    want = plain.moe_experts(h.double(), w_up.double(), w_down.double(), ids, wts, experts, F64, glu=(1.2, 1.702))
    outs = []
    for tiles in ("1", "0"):
        monkeypatch.setenv("INFERFLUX_B200_MOE_TILES", tiles)
        before = cuda_kernels.launches
        outs.append(cuda_kernels.moe_experts(h.to(DEV), w_up.to(DEV), w_down.to(DEV), ids.to(DEV), wts.to(DEV), experts, bf,
                                             glu=(1.2, 1.702)).double().cpu())
        assert cuda_kernels.launches - before == (5 if tiles == "1" else 2)
    cuda_kernels.check_errors()
    top_v = float(want.abs().max())
    assert float((outs[0] - want).abs().max()) <= 2e-2 * top_v and float((outs[1] - want).abs().max()) <= 2e-2 * top_v


# ------------------------------------------------------------------ latent attention with a rotated part

def _step_ctx(kernels, dtype, cache, spans, providers=()):
    """A step context for `spans` = [(request, number of tokens)], pages reserved and the table updated."""
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
    ctx = StepContext.build(kernels, dtype, DEV, entries, starts, slots, cache.drain_table_updates(), providers=providers)
    for g, (idx, page) in zip(cache.groups, ctx.table_updates):
        kernels.scatter_i32(g.table, idx, page)
    return ctx, starts


def _attention_part(dtype, width, H, dk, rot, dv, rank, q_rank, pairing, scaling, scale, seed):
    from inferflux_b200.config import PartSpec
    from inferflux_b200.parts import build_part
    position = PartSpec("rope", {"theta": 300.0, "rotary_dim": rot, "pairing": pairing,
                                 "scaling": None if scaling is None else {"kind": "ramp", **scaling}})
    mixer = build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": H, "qk_dim": dk, "rot_dim": rot, "v_dim": dv, "kv_rank": rank, "q_rank": q_rank,
        "window": None, "scale": scale, "latent_norm_eps": 1e-5, "sink": False, "position": position,
        "names": {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq"}}))
    tensors = {n: _rnd(*s.shape, seed=seed + i, scale=0.3).to(dtype) for i, (n, s) in enumerate(mixer.param_specs().items())}
    for n in ("dq.norm", "dkv.norm"):
        tensors[n] = (1 + 0.2 * _rnd(*tensors[n].shape, seed=seed + 50)).to(dtype)
    tensors["dkv"][rank:] *= 0.08            # the rotated key part is not normed: kept small, it moves scores by a few units
    return mixer, tensors


def _plant(h, tensors, mixer_raw, pairs, eps):
    """For every (query position i, head, key position j): the input row j is replaced by one whose latent, after the
    norm, points along head's query i carried into latent space, and whose rotated key part is nothing."""
    W = {k: v.double() for k, v in tensors.items()}
    H, D, R, rank = mixer_raw["heads"], mixer_raw["dim"], mixer_raw["rot_dim"], mixer_raw["kv_rank"]
    back = torch.linalg.pinv(W["dkv"])                                      # [width, rank + rot]
    for i, head, j in pairs:
        q = (P.rmsnorm(h[i:i + 1].double() @ W["dq"].T, W["dq.norm"], eps) @ W["uq"].T).view(H, D + R)[head, :D]
        ql = W["uk"].view(H, D, rank)[head].T @ q
        target = torch.cat([ql / ql.norm() * 3.0 / W["dkv.norm"], torch.zeros(R, dtype=F64)])
        h[j] = (back @ target).to(h.dtype)
    return h


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("sizes", [
    # width, heads, dim, rot, vdim, kv_rank, q_rank, pairing, page
    (96, 3, 16, 16, 24, 32, 40, "interleaved", 16),        # tiles in bfloat16
    (128, 4, 24, 32, 16, 64, 24, "split_half", 16),        # tiles, values shorter than keys
    (160, 2, 8, 64, 40, 48, 56, "interleaved", 8),         # tiles, a rotated part longer than the latent's plain keys
    (384, 2, 16, 64, 24, 256, 48, "split_half", 16),       # tiles at their largest latent and rotated part
    (96, 5, 12, 6, 20, 20, 28, "split_half", 4),           # sizes the tiles do not take: the per-token kernel
    (96, 1, 16, 8, 16, 40, 16, "interleaved", 16)])
def test_latent_attention_with_rotated_part_planted_keys(cuda_kernels, dtype, tol, sizes):
    """The mixer over its own cache, whole, in portions and with its last tokens decoded alone, against the plain
    function that makes keys and values of every head explicitly.  Single keys are made to stand out: the first
    token, one far back, the last of a page and the first of the next, the token itself and the one before."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    width, H, dk, rot, dv, rank, q_rank, pairing, page = sizes
    T, eps = 700, 1e-5
    scaling = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}
    scale = 2.0 / math.sqrt(rank)            # planted scores near 25, the largest of the others near 13
    mixer, tensors = _attention_part(dtype, width, H, dk, rot, dv, rank, q_rank, pairing, scaling, scale, seed=40)
    mixer.load(tensors, dtype, DEV)
    raw = {"heads": H, "dim": dk, "rot_dim": rot, "vdim": dv, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
           "rot": {"base": 300.0, "dims": rot, "scaling": scaling}}
    h0 = _rnd(T, width, seed=60)
    h = h0.clone()
    pairs = [(699, 0, 3), (698, H - 1, 0), (697, 0, 25 * page - 1), (696, H - 1, 25 * page), (650, 0, 650), (640, H - 1, 639),
             (300, 0, 5), (301, H - 1, 17 * page), (302, 0, 17 * page - 1), (40, 0, 2 * page), (41, H - 1, 2 * page - 1)]
    h = _plant(h, tensors, raw, pairs, eps).to(dtype)
    want = P.latent_attention(h.double(), {k: v.double() for k, v in tensors.items()}, "", raw, eps, list(range(T)),
                              pairing == "interleaved")
    # the planted keys do stand out: without them the rows that ask for them come out quite differently
    plain0 = P.latent_attention(h0.to(dtype).double(), {k: v.double() for k, v in tensors.items()}, "", raw, eps, list(range(T)),
                                pairing == "interleaved")
    for i, _head, _j in pairs:
        assert float((plain0[i] - want[i]).norm()) > 0.2 * float(want[i].norm()), f"the key planted for row {i} does not show"
    for cuts in ([T], [300, 339, 61], [690] + [1] * 10, [2, 5, 57, 1, 1, 2, 632]):
        cache = CacheManager([(mixer.cache_spec(), None)], page_size=page, num_pages=T // page + 2, max_seqs=2, max_seq_len=T + page,
                             dtype=dtype, device=DEV)
        outs, pos = [], 0
        for n in cuts:
            ctx, starts = _step_ctx(cuda_kernels, dtype, cache, [("r", n)], providers=[mixer])
            outs.append(cuda_kernels.materialize(mixer.forward(h[pos:pos + n].to(DEV).contiguous(), ctx,
                                                               cache.view(ScheduleEntry(0, 0)))))
            cache.commit("r", starts[0] + n)
            pos += n
        cuda_kernels.check_errors()
        got = torch.cat(outs).float().cpu().double()
        err = (got - want).abs().max(dim=1).values
        assert float(err.max()) < tol * float(want.abs().max()), f"cuts {cuts}: row {int(err.argmax())} is off by {float(err.max())}"


def test_latent_attention_rotated_tiles_against_the_per_token_kernel(cuda_kernels):
    """The two bfloat16 paths on the same steps: prompt portions beside decoded tokens of other requests."""
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    bf = torch.bfloat16
    mixer, tensors = _attention_part(bf, 128, 6, 16, 32, 24, 64, 48, "split_half", None, 0.4, seed=80)
    mixer.load(tensors, bf, DEV)
    outs, tiled_calls = {}, []
    inner = cuda_kernels._latent_attention_tiles

    def counting(*a, **kw):
        tiled_calls.append(kw.get("rot", 0))
        return inner(*a, **kw)
    cuda_kernels._latent_attention_tiles = counting
    try:
        for tiles in (True, False):
            cuda_kernels.latent_tiles = tiles
            cache = CacheManager([(mixer.cache_spec(), None)], page_size=16, num_pages=80, max_seqs=4, max_seq_len=600, dtype=bf, device=DEV)
            got = []
            for step, spans in enumerate([[("a", 500), ("b", 70)], [("a", 1), ("b", 1), ("c", 130)], [("c", 2), ("a", 1)], [("b", 1), ("a", 1), ("c", 1)]]):
                T = sum(n for _r, n in spans)
                ctx, starts = _step_ctx(cuda_kernels, bf, cache, spans, providers=[mixer])
                before = len(tiled_calls)
                got.append(cuda_kernels.materialize(mixer.forward(_rnd(T, 128, seed=step).to(bf).to(DEV), ctx, cache.view(ScheduleEntry(0, 0)))).float().cpu())
                assert (len(tiled_calls) - before == 1) == tiles and all(r == 32 for r in tiled_calls)
                for (rid, n), st in zip(spans, starts):
                    cache.commit(rid, st + n)
            outs[tiles] = torch.cat(got)
    finally:
        cuda_kernels.latent_tiles = True
        del cuda_kernels._latent_attention_tiles
    cuda_kernels.check_errors()
    assert float((outs[True] - outs[False]).abs().max()) < 3e-2 * float(outs[False].abs().max())


# ------------------------------------------------------------------ whole models

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


@pytest.fixture(scope="module")
def oracle(benarax_dirs):
    memo = {}

    def get(name):
        if name not in memo:
            d, _page, raw = benarax_dirs[name]
            reqs = bm.requests_for(raw, LENS, 100)
            memo[name] = {"reqs": reqs, "float32": bm.plain_logits(d, reqs),
                          "bfloat16": bm.plain_logits(d, reqs, weights_as=torch.bfloat16),
                          "yard": bm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16)}
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


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_step_function_cuttings(name, dtype, cutting, benarax_dirs, oracle, cuda_kernels):
    d, page, raw = benarax_dirs[name]
    o = oracle(name)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](o["reqs"])
    runner = _runner(d, dtype, page, cuda_kernels, cuda_graphs=(cutting == "tail"))
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    cuda_kernels.check_errors()
    _check(f"{name} {cutting}", dtype, got, o)
    assert not runner.cache.live_requests()


@pytest.mark.parametrize("name", ["A", "D"])
def test_float32_is_the_same_under_every_cutting(name, benarax_dirs, oracle, cuda_kernels):
    d, page, raw = benarax_dirs[name]
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
def test_portions_down_to_two_tokens_from_the_first_token_on(dtype, benarax_dirs, cuda_kernels):
    from inferflux_b200.engine import StepEntry
    d, page, raw = benarax_dirs["A"]
    toks = bm.requests_for(raw, [60], 3)["r0"]
    rounded = torch.bfloat16 if dtype == "bfloat16" else None
    want = bm.plain_logits(d, {"r0": toks}, weights_as=rounded)["r0"]
    yard = bm.plain_logits(d, {"r0": toks}, weights_as=torch.bfloat16, dtype=torch.bfloat16)["r0"]
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
    """Prompts of 700 and 300 tokens through a model of five layers (seven runs): whole, then in portions of 200 and 128
    beside each other's decoded tokens.  These steps reach the kernels of many rows (library and tcgen05 products, sorted
    expert tiles with the gated activation, the tensor-core latent attention with a rotated part, the scan's long spans)
    inside a whole model."""
    from inferflux_b200.engine import ModelRunner, StepEntry
    from inferflux_b200.models import load_model
    raw, page = bm.medium_config()
    d = bm.write_model(raw, tmp_path / "medium", seed=77)
    reqs = bm.requests_for(raw, [700, 300], 12)
    rows = {"r0": [0, 1, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512, 640, 698, 699], "r1": [0, 63, 64, 127, 128, 200, 298, 299]}
    rounded = torch.bfloat16 if dtype == "bfloat16" else None
    want = {k: v[rows[k]] for k, v in bm.plain_logits(d, reqs, weights_as=rounded).items()}
    yard = {k: v[rows[k]] for k, v in bm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16).items()} \
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
def test_long_decoding_with_reused_pages_slots_and_graphs(dtype, benarax_dirs, cuda_kernels):
    """12 prompt tokens, then 300 decoded one by one beside requests that join and leave: page borders are crossed by
    decoded tokens, the pages and the slot of a request that left serve the next one, decode steps replay a CUDA graph."""
    from inferflux_b200.engine import StepEntry
    d, page, raw = benarax_dirs["A"]
    reqs = bm.requests_for(raw, [312, 90, 60], 9)
    want = bm.plain_logits(d, reqs, weights_as=torch.bfloat16 if dtype == "bfloat16" else None)
    yard = bm.plain_logits(d, reqs, weights_as=torch.bfloat16, dtype=torch.bfloat16) if dtype == "bfloat16" else None
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
def test_trace_run_program(dtype, benarax_dirs, oracle, tmp_path):
    d, page, raw = benarax_dirs["B"]
    o = oracle("B")
    steps = helpers.trace_mixed(o["reqs"], 256)
    got = helpers.collect(steps, helpers.run_trace_cli(d, dtype, steps, tmp_path / "out", 256, raw["vocab"], page_size=page),
                          raw["vocab"])
    _check("B through the program", dtype, got, o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_engine_and_scheduler(dtype, benarax_dirs, tmp_path):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = benarax_dirs["A"]
    if dtype == "bfloat16":
        # a router that decides by less than rounding moves its outputs sends a token to another expert in one correct
        # computation and not in another, and every later token inherits the difference through the cache and the state:
        # the bfloat16 run generates with routers that choose all their experts
        raw = {**raw, "layers": [l if l["mlp"] is None else {**l, "mlp": {**l["mlp"], "router": {**l["mlp"]["router"], "top": l["mlp"]["router"]["experts"]}}}
                                 for l in raw["layers"]]}
        d = bm.write_model(raw, tmp_path / "all_chosen", seed=71)
    _raw, W = bm.load(d)
    if dtype == "bfloat16":
        W = {k: v.to(torch.bfloat16) for k, v in W.items()}
    prompts = list(bm.requests_for(raw, [7, 19, 33, 4, 1, 70], 40).values())
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
                # bfloat16: the logits tests allow the engine three times what rounding does to the plain computation
                # (its worst row of this sequence); the chosen token may lie that much, and the rounding itself, below
                slack = 1e-3 if rough is None else 4.0 * float((rough - exact).abs().max())
                assert gap <= slack, f"token {i}: {gap:.4f} below the best logit, rounding allows {slack:.4f}"
        assert not eng.runner.cache.live_requests()
