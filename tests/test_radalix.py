"""Radalix without a GPU: the plain implementation's mechanisms against values worked out by hand, the
configuration and plan, and the engine's host logic (plan, cache and state manager, batching, scheduler)
run on the plain kernel table against the plain implementation."""
import math

import numpy as np
import pytest
import torch

import helpers
import radalix_models as rm
from plain import plain_radalix as P
from plain.plain_kernels import PlainKernels

F64 = torch.float64


@pytest.fixture(scope="module")
def radalix_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(rm.configs().items()):
        out[name] = (rm.write_model(raw, tmp_path_factory.mktemp(f"radalix_{name}"), seed=31 + i), page, raw)
    return out


# ------------------------------------------------------------------ mechanisms, by hand

def test_bigram_rows_by_hand():
    b = {"buckets": 10, "mul_prev": 3, "mul_cur": 7}
    assert P.bigram_rows([4, 9, 0, 9], b) == [10, (4 * 3 + 9 * 7) % 10, (9 * 3) % 10, (0 * 3 + 9 * 7) % 10]
    assert P.bigram_rows([5], b) == [10]                                   # a sequence's first token: the table's last row
    raw = {"embedding": {"scale": 2.0, "bigram": b}}
    W = {"embed": torch.arange(20, dtype=F64).reshape(10, 2), "bigram": 100.0 * torch.arange(22, dtype=F64).reshape(11, 2)}
    x = P.embed(raw, W, [4, 9], F64)
    assert x.tolist() == [[2 * 8 + 2000, 2 * 9 + 2100], [2 * 18 + 1000, 2 * 19 + 1100]]


def test_convolution_over_time_by_hand():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=F64)
    w = torch.tensor([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]], dtype=F64)          # the last tap meets the present token
    got = P.causal_conv(u, w)
    assert got[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0] and got[:, 1].tolist() == [20.0, 40.0, 60.0, 80.0]
    assert P.causal_conv(u, w, torch.tensor([0.5, -1.0], dtype=F64))[1].tolist() == [12.5, 39.0]
    assert torch.equal(P.causal_conv(u, torch.tensor([[3.0], [0.5]], dtype=F64)), u * torch.tensor([3.0, 0.5], dtype=F64))


def test_query_temperature_and_rotation_by_hand():
    t = P.query_temperature([0, 3, 4, 9, 14], {"coef": 0.5, "every": 5}, F64)
    assert torch.allclose(t, torch.tensor([1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(4)], dtype=F64))
    x = torch.tensor([[[1.0, 0.0, 5.0, 6.0, 7.0, 8.0]]], dtype=F64)              # one token, one head of six
    near = P.rotate_neighbours(x, [1], [math.pi / 2, math.pi], 1.0)             # pairs (0, 1), (2, 3); the rest stays
    assert torch.allclose(near[0, 0], torch.tensor([0.0, 1.0, -5.0, -6.0, 7.0, 8.0], dtype=F64), atol=1e-12)
    assert torch.equal(P.rotate_neighbours(x, [0], [0.3, 0.7], 1.0), x)
    assert torch.allclose(P.rotate_neighbours(x, [0], [0.3, 0.7], 1.5)[0, 0, :4], x[0, 0, :4] * 1.5)
    plain, one = P.rotary_frequencies({"base": 100.0, "dims": 8})
    assert plain == [100.0 ** (-2.0 * i / 8) for i in range(4)] and one == 1.0
    f, mult = P.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}})
    lo, hi = 0, 3                                                              # the indices that turn 4 times and once in 64 positions
    assert abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    for i in range(4):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f[i] - (plain[i] / 4.0 * ramp + plain[i] * (1 - ramp))) < 1e-15


def test_attention_window_sink_and_gate_by_hand():
    # one head of one channel, keys 1 everywhere: scores are all q * scale, weights uniform over what is seen
    W = {"a.q": torch.ones(1, 1, dtype=F64), "a.k": torch.zeros(1, 1, dtype=F64), "a.v": torch.ones(1, 1, dtype=F64),
         "a.o": torch.ones(1, 1, dtype=F64)}
    h = torch.tensor([[1.0], [2.0], [4.0], [8.0]], dtype=F64)
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "scale": 1.0}
    assert torch.allclose(P.attention(h, W, "a.", m, range(4), False)[:, 0], torch.tensor([1.0, 1.5, 7 / 3, 15 / 4], dtype=F64))
    win = P.attention(h, W, "a.", {**m, "mask": {"size": 2}}, range(4), False)[:, 0]
    assert torch.allclose(win, torch.tensor([1.0, 1.5, 3.0, 6.0], dtype=F64))            # itself and one token before it
    one = P.attention(h, W, "a.", {**m, "mask": {"size": 1}}, range(4), False)[:, 0]
    assert torch.allclose(one, h[:, 0])
    W["a.sink"] = torch.tensor([math.log(2.0)], dtype=F64)                               # counts as two keys of score 0, no value
    sunk = P.attention(h, W, "a.", {**m, "mask": {"size": 2}}, range(4), False)[:, 0]
    assert torch.allclose(sunk, torch.tensor([1 / 3, 3 / 4, 6 / 4, 12 / 4], dtype=F64))
    del W["a.sink"]
    W["a.g"] = torch.tensor([[0.0]], dtype=F64)                                          # sigmoid(0) = 1/2
    assert torch.allclose(P.attention(h, W, "a.", m, range(4), True)[:, 0], torch.tensor([0.5, 0.75, 7 / 6, 15 / 8], dtype=F64))


def test_decayed_scan_by_hand():
    q = torch.tensor([[[2.0]], [[3.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[-2.0]]], dtype=F64)
    v = torch.tensor([[[10.0]], [[1.0]]], dtype=F64)
    w = torch.tensor([[[0.5]], [[0.25]]], dtype=F64)
    out, S = P.decayed_scan(q, k, v, w)
    # S: 0 -> 10 -> 0.25 * 10 - 2 = 0.5; the read-out takes the new S
    assert out[:, 0, 0].tolist() == [20.0, 1.5] and float(S) == 0.5
    g = torch.Generator().manual_seed(1)
    mk = lambda *s: torch.rand(*s, generator=g, dtype=F64)
    q, k, v, w = mk(9, 2, 3), mk(9, 2, 3) - 0.5, mk(9, 2, 5), mk(9, 2, 3)
    whole, S_whole = P.decayed_scan(q, k, v, w)
    first, S_mid = P.decayed_scan(q[:4], k[:4], v[:4], w[:4])
    second, S_end = P.decayed_scan(q[4:], k[4:], v[4:], w[4:], state=S_mid)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S_end, S_whole)
    # the decay scales rows (key channels), not columns
    _o, S1 = P.decayed_scan(torch.ones(1, 1, 2, dtype=F64), torch.zeros(1, 1, 2, dtype=F64), torch.zeros(1, 1, 2, dtype=F64),
                            torch.tensor([[[0.5, 1.0]]], dtype=F64), state=torch.tensor([[[1.0, 2.0], [3.0, 4.0]]], dtype=F64))
    assert S1[0].tolist() == [[0.5, 1.0], [3.0, 4.0]]


def test_router_and_expert_by_hand():
    W = {"m.router": torch.eye(4, dtype=F64)}
    h = torch.tensor([[0.0, math.log(3.0), math.log(1 / 3), -50.0]], dtype=F64)           # scores 1/2, 3/4, 1/4, ~0
    chosen, weight = P.route(h, W, "m.", {"top": 2})
    assert chosen[0].tolist() == [1, 0] and torch.allclose(weight[0], torch.tensor([0.6, 0.4], dtype=F64))
    one, w1 = P.route(h, W, "m.", {"top": 1})
    assert one[0].tolist() == [1] and abs(float(w1) - 1.0) < 1e-12
    W.update({"m.gate": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0]], dtype=F64), "m.up": torch.tensor([[0, 0, 1.0, 0], [2.0, 0, 0, 0]], dtype=F64),
              "m.down": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=F64)})
    x = torch.tensor([[2.0, -1.0, 3.0, 0.0]], dtype=F64)
    a = [2.0 / (1 + math.exp(-2.0)) * 3.0, -1.0 / (1 + math.exp(1.0)) * 4.0]
    assert torch.allclose(P.gated_expert(x, W, "m.")[0], torch.tensor([a[0], a[1], a[0] + a[1]], dtype=F64))


# ------------------------------------------------------------------ every option changes the result

def test_every_option_matters(radalix_dirs):
    for name in ("A", "B", "C"):
        d, _page, raw = radalix_dirs[name]
        _raw, W = rm.load(d)
        toks = rm.requests_for(raw, [45], 9)["r0"]
        base = P.forward(raw, W, toks)

        def differs(other_raw=None, other_W=None):
            return float((P.forward(other_raw or raw, other_W or W, toks) - base).abs().max())

        def scaled(suffix, f):
            assert any(k.endswith(suffix) for k in W), suffix
            return {k: (v * f if k.endswith(suffix) else v) for k, v in W.items()}

        def edit(change):
            layers = []
            for l in raw["layers"]:
                m = {**l["mixer"], "left": {**l["mixer"]["left"]}, "right": {**l["mixer"]["right"]}}
                change(l["type"], m)
                layers.append({**l, "mixer": m})
            return {**raw, "layers": layers}
        for suffix in (".ls1", ".left.o", ".right.o", ".right.norm", ".norm1", "final.norm"):
            assert differs(other_W=scaled(suffix, 1.3)) > 1e-6, (name, suffix)
        if any(k.endswith(".left.out") for k in W):
            assert differs(other_W={k: (v.roll(1) if k.endswith(".left.out") else v) for k, v in W.items()}) > 1e-6
        if any(k.endswith(".sink") for k in W):
            assert differs(other_W={k: (v + 1.0 if k.endswith(".sink") else v) for k, v in W.items()}) > 1e-6
        if raw["embedding"].get("bigram"):
            assert differs(other_W={k: (v.roll(1, 0) if k == "bigram" else v) for k, v in W.items()}) > 1e-6
            assert differs(other_raw={**raw, "embedding": {"scale": raw["embedding"]["scale"]}}) > 1e-6
        assert differs(other_raw={**raw, "embedding": {**raw["embedding"], "scale": raw["embedding"]["scale"] * 1.1}}) > 1e-6
        if raw.get("logit_softcap"):
            assert differs(other_raw={k: v for k, v in raw.items() if k != "logit_softcap"}) > 1e-6

        def no_q_temp(kind, m):
            m["left"].pop("q_temp", None)

        def wider_window(kind, m):
            if m["left"].get("mask"):
                m["left"]["mask"] = {"size": m["left"]["mask"]["size"] + 1}

        def other_scales(kind, m):
            if kind == "parallel_2":
                m["left_scale"], m["right_scale"] = m["left_scale"] * 1.2, m["right_scale"] * 0.8
            else:
                m["right"]["tau"] = m["right"]["tau"] * 2.0

        def unscaled(kind, m):
            if m["left"].get("rot"):
                m["left"]["rot"] = {k: v for k, v in m["left"]["rot"].items() if k != "scaling"}
        if any(l["mixer"]["left"].get("q_temp") for l in raw["layers"]):
            assert differs(other_raw=edit(no_q_temp)) > 1e-6, name
        if any((l["mixer"]["left"].get("mask") or {}).get("size", 1 << 30) < 44 for l in raw["layers"]):
            assert differs(other_raw=edit(wider_window)) > 1e-6, name
        assert differs(other_raw=edit(other_scales)) > 1e-6, name
        if any((l["mixer"]["left"].get("rot") or {}).get("scaling") for l in raw["layers"]):
            assert differs(other_raw=edit(unscaled)) > 1e-6, name


# ------------------------------------------------------------------ configuration and plan

def test_config_round_trip_and_plan(radalix_dirs):
    from inferflux_b200.config import ConfigError, RadalixConfig, config_from_dict, load_config
    from inferflux_b200.models.model import Model
    d, _page, raw = radalix_dirs["A"]
    cfg = load_config(d)
    assert isinstance(cfg, RadalixConfig) and cfg.to_dict() == raw
    plan = cfg.to_plan()
    assert [l.block.kind for l in plan.layers] == ["parallel_norms"] * 4 and [l.mixer.kind for l in plan.layers] == ["pair"] * 4
    assert [l.mixer.params["right"].kind for l in plan.layers] == ["decayed_linear_attention", "state_space", "state_space",
                                                                   "decayed_linear_attention"]
    model = Model(plan)
    exp = model.expected_tensors()
    names = set(exp)
    assert {"embed", "bigram", "final.norm", "l0.norm1", "l0.norm2", "l0.ls1", "l0.ls2", "l0.mix.left.q", "l0.mix.left.q.conv",
            "l0.mix.left.k.conv", "l0.mix.left.v.conv", "l0.mix.left.g", "l0.mix.left.o", "l0.mix.left.out", "l0.mix.right.out",
            "l0.mix.right.a1", "l0.mix.right.a2", "l0.mix.right.a2.b", "l0.mix.right.norm", "l0.mlp.router", "l0.mlp.e4.gate",
            "l0.mlp.shared.down", "l1.mix.left.sink", "l1.mix.right.in", "l1.mix.right.conv", "l1.mix.right.conv.b",
            "l1.mix.right.dt_bias", "l1.mix.right.A_log", "l1.mix.right.D", "l1.mix.right.norm", "l2.ls1", "l3.mix.left.g"} <= names
    assert not {"l0.mix.left.sink", "l1.mix.left.g", "l1.mix.left.out", "l1.mlp.shared.gate", "l2.norm2", "l2.ls2", "l2.mlp.router",
                "l3.mix.left.q.conv", "l0.mlp.e5.up", "head"} & names
    assert exp["bigram"].shape == (54, 64) and exp["l0.mix.left.q.conv"].shape == (64, 3) and exp["l0.mix.right.norm"].shape == (16,)
    assert exp["l1.mix.right.in"].shape == (2 * 32 + 2 * 2 * 12 + 4, 64) and exp["l1.mix.right.conv"].shape == (32 + 48, 3)
    assert exp["l0.mix.right.a1"].shape == (-1, 64) and exp["l0.mix.right.a1"].fits((11, 64))     # the decay's inner size: the file's
    specs = model.cache_specs()
    kv, st = specs[0]
    assert (kv.num_kv_heads, kv.head_dim, kv.window) == (2, 16, None) and st.shape == (2 * (64 + 32 + 16) + 3 * 8 * 16,)
    kv, st = specs[1]
    assert (kv.num_kv_heads, kv.head_dim, kv.window) == (1, 16, 7) and st.shape == (1 * (16 + 8 + 16) + 2 * 80 + 4 * 12 * 8,)
    assert specs[3][1].shape == (24 * 8,)                                     # no convolution: the recurrence's matrix alone
    assert specs[4] == (None, model.embedding.state_spec()) and specs[4][1].dtype == torch.int32
    _d, _p, raw_b = radalix_dirs["B"]
    assert len(Model(config_from_dict(raw_b).to_plan()).cache_specs()) == 3   # without the second table the embedding keeps nothing
    lay = raw["layers"][1]
    for bad in ({**raw, "layers": []}, {**raw, "layers": [{**lay, "type": "other"}]}, {k: v for k, v in raw.items() if k != "width"},
                {**raw, "layers": [{**lay, "mixer": {k: v for k, v in lay["mixer"].items() if k != "right"}}]},
                {**raw, "layers": [{**lay, "mixer": {**lay["mixer"], "left": {**lay["mixer"]["left"], "kv_heads": 3}}}]},
                {**raw, "layers": [{**lay, "mixer": {**lay["mixer"], "left": {**lay["mixer"]["left"], "rot": {"base": 100.0, "dims": 7}}}}]},
                {**raw, "layers": [{**lay, "mixer": {**lay["mixer"], "right": {**lay["mixer"]["right"], "groups": 3}}}]},
                {**raw, "layers": [{**lay, "mixer": {k: v for k, v in lay["mixer"].items() if k != "left_scale"}}]},
                {**raw, "layers": [{**lay, "mlp": {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 3}}}]},
                {**raw, "logit_softcap": 0.0}):
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_wrong_weights_are_refused_and_the_decay_rank_comes_from_the_file(radalix_dirs, tmp_path):
    from inferflux_b200.models import load_model
    from inferflux_b200.weights import WeightError, write_safetensors
    d, _page, raw = radalix_dirs["A"]
    _raw, W = rm.load(d)
    (tmp_path / "config.json").write_text((d / "config.json").read_text())
    W2 = {k: v for k, v in W.items() if k not in ("l0.mlp.e1.gate", "l1.mix.left.sink")}
    W2["l1.mix.right.in"] = W["l1.mix.right.in"][:-1].contiguous()
    W2["bigram"] = W["bigram"][:-1].contiguous()
    write_safetensors(tmp_path / "model.safetensors", W2)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, dtype="float32", device="cpu")
    assert e.value.missing == ["l0.mlp.e1.gate", "l1.mix.left.sink"]
    assert sorted(w[0] for w in e.value.wrong_shape) == ["bigram", "l1.mix.right.in"]
    W3 = dict(W)                                            # another inner size of the decay: taken from the tensors
    W3["l0.mix.right.a1"] = torch.cat([W["l0.mix.right.a1"], W["l0.mix.right.a1"][:3] * 0.5])
    W3["l0.mix.right.a2"] = torch.cat([W["l0.mix.right.a2"], W["l0.mix.right.a2"][:, :3] * 0.5], dim=1)
    write_safetensors(tmp_path / "model.safetensors", W3)
    _c, model = load_model(tmp_path, dtype="float32", device="cpu")
    assert model.layers[0].mixer.right.rank == W["l0.mix.right.a1"].shape[0] + 3


# ------------------------------------------------------------------ the engine's host logic on plain kernels

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


def _plain_runner(d, page, pages=None, max_seqs=4, max_seq_len=512):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype="float32", device="cpu")
    return ModelRunner(model, PlainKernels(wide=True), page_size=page, num_pages=pages or 256 // page, max_seqs=max_seqs,
                       max_seq_len=max_seq_len)


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_engine_host_logic_on_plain_kernels(name, cutting, radalix_dirs):
    d, page, raw = radalix_dirs[name]
    reqs = rm.requests_for(raw, LENS, 100)
    want = rm.plain_logits(d, reqs)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](reqs)
    runner = _plain_runner(d, page)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    bad = helpers.first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong row (request, position, diff): {bad}"
    pools = [256 // page] * len(runner.cache.groups)
    assert not runner.cache.live_requests() and runner.cache.free_pages() == pools


def test_portions_down_to_two_tokens_and_the_first_tokens(radalix_dirs):
    """Portions of 2, 1, 3, 2, 2, 5 ... tokens from the first token on: the convolutions read the rows that the
    portion before left (and zeros before the sequence's start), the recurrences their state, the second embedding
    table the token before, attention its pages."""
    from inferflux_b200.engine import StepEntry
    for name in ("A", "C"):
        d, page, raw = radalix_dirs[name]
        toks = rm.requests_for(raw, [60], 3)["r0"]
        want = rm.plain_logits(d, {"r0": toks})["r0"]
        runner = _plain_runner(d, page)
        got, pos, sizes, i = [], 0, [2, 1, 3, 2, 2, 5, 1, 1, 2, 17], 0
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            got += list(runner.step([StepEntry("r0", toks[pos:pos + n], list(range(n)))]).double().numpy())
            pos += n
        runner.end_request("r0")
        assert float(np.abs(np.stack(got) - want).max()) < 2e-4, name


def test_a_slot_and_pages_that_are_used_again_start_clean(radalix_dirs):
    from inferflux_b200.engine import StepEntry
    d, page, raw = radalix_dirs["A"]
    reqs = rm.requests_for(raw, [9, 1, 3, 2, 30, 5], 7)
    want = rm.plain_logits(d, reqs)
    runner = _plain_runner(d, page, pages=4, max_seqs=1, max_seq_len=32)
    for rid, toks in reqs.items():                         # one slot, four pages: everybody inherits them
        got = runner.step([StepEntry(rid, toks, list(range(len(toks))))]).double().numpy()
        assert float(np.abs(got - want[rid]).max()) < 2e-4, rid
        assert all(float(s[0].double().abs().max()) > 0 for s in runner.cache.state[:-1] if s is not None)
        assert int(runner.cache.state[-1][0, 0]) == toks[-1]                 # the embedding's memory: the last token
        runner.end_request(rid)
        runner.cache.check()
    assert all(g.alloc.allocations > 4 for g in runner.cache.groups)


def test_greedy_generation_through_engine_and_scheduler(radalix_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = radalix_dirs["A"]
    _raw, W = rm.load(d)
    prompts = list(rm.requests_for(raw, [7, 19, 33, 4, 1], 40).values())

    def greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(P.forward(raw, W, seq)[-1].argmax()))
        return seq[len(prompt):]
    want = [greedy(p, 12) for p in prompts]
    for pages in (64, 8):                                  # 8 pages of 8: the requests do not all fit at once
        eng = Engine(d, dtype="float32", device="cpu", kernels=PlainKernels(wide=True), kv_page_size=page,
                     kv_num_pages=pages, kv_max_batch=4, kv_max_seq=128, chunked_prefill_tokens=16, max_batch_tokens=48)
        res = eng.generate(prompts, SamplingParams(temperature=0.0), max_tokens=12)
        assert [r.token_ids for r in res] == want
        assert not eng.runner.cache.live_requests()
