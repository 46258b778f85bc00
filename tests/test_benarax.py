"""Benarax without a GPU: the plain implementation's mechanisms against values worked out by hand, the
configuration and plan, and the engine's host logic (plan, cache and state manager, batching, scheduler)
run on the plain kernel table against the plain implementation."""
import math

import numpy as np
import pytest
import torch

import benarax_models as bm
import helpers
from plain import plain_benarax as P
from plain.plain_kernels import PlainKernels

F64 = torch.float64


@pytest.fixture(scope="module")
def benarax_dirs(tmp_path_factory):
    out = {}
    for i, (name, (raw, page)) in enumerate(bm.configs().items()):
        out[name] = (bm.write_model(raw, tmp_path_factory.mktemp(f"benarax_{name}"), seed=71 + i), page, raw)
    return out


# ------------------------------------------------------------------ mechanisms, by hand

def test_norm_in_groups_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 5.0, 0.5], dtype=F64)
    got = P.groupnorm(x, w, 0.0, 2)
    assert torch.allclose(got, torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5), 0.0, 1 / math.sqrt(2.0)]], dtype=F64))
    assert torch.allclose(P.groupnorm(x, w, 0.0, 1), x / math.sqrt(29 / 4) * w)
    # eps under the root, per group
    tiny = torch.tensor([[1e-3, 0.0]], dtype=F64)
    assert abs(float(P.groupnorm(tiny, torch.ones(2, dtype=F64), 1e-6, 2)[0, 0]) - 1e-3 / math.sqrt(2e-6)) < 1e-12
    assert float(P.groupnorm(torch.zeros(1, 6, dtype=F64), torch.ones(6, dtype=F64), 1e-6, 3).abs().max()) == 0.0


def test_convolution_over_time_by_hand():
    h = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]], dtype=F64)
    w = torch.tensor([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]], dtype=F64)          # the last tap meets the present token
    got = P.causal_conv(h, w)
    assert got[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0]
    assert got[:, 1].tolist() == [20.0, 40.0, 60.0, 80.0]
    assert torch.equal(P.causal_conv(h, torch.tensor([[3.0], [0.5]], dtype=F64)), h * torch.tensor([3.0, 0.5], dtype=F64))


def test_delta_rule_by_hand():
    # one head, one channel: u = k / sqrt(k^2 + 1e-6) is +-1 up to 5e-7, S is a number
    r = torch.tensor([[[2.0]], [[3.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[-2.0]]], dtype=F64)
    v = torch.tensor([[[10.0]], [[1.0]]], dtype=F64)
    w = torch.tensor([[[0.5]], [[0.25]]], dtype=F64)
    a = torch.tensor([[[0.3]], [[0.1]]], dtype=F64)
    out, S = P.delta_scan(r, k, v, w, a)
    # S: 0 -> 10 -> 0.25 * 10 - 0.1 * 10 + (-2) * 1 = -0.5
    assert abs(float(out[0, 0, 0]) - 20.0) < 1e-9 and abs(float(S) + 0.5) < 1e-5 and abs(float(out[1, 0, 0]) + 1.5) < 1e-4
    # two key channels: the decay scales rows, the erased part lies along the unit key, both read the old state
    S0 = torch.tensor([[[1.0, 2.0], [3.0, 4.0]]], dtype=F64)
    k2 = torch.tensor([[[3.0, 4.0]]], dtype=F64)
    w2 = torch.tensor([[[0.5, 1.0]]], dtype=F64)
    a2 = torch.tensor([[[1.0, 0.5]]], dtype=F64)
    v2 = torch.tensor([[[1.0, 0.0]]], dtype=F64)
    _o, S1 = P.delta_scan(torch.ones(1, 1, 2, dtype=F64), k2, v2, w2, a2, state=S0)
    u = torch.tensor([0.6, 0.8], dtype=F64)
    along = u @ S0[0]                                                           # [3.0, 4.4]
    want = torch.stack([0.5 * S0[0, 0] - 1.0 * 0.6 * along + 3.0 * v2[0, 0], 1.0 * S0[0, 1] - 0.5 * 0.8 * along + 4.0 * v2[0, 0]])
    assert torch.allclose(S1[0], want, atol=1e-6)
    assert torch.allclose(_o[0, 0], S1[0].sum(dim=0))                            # out = S^T r of the new S
    # the decay's range
    assert abs(float(P.delta_decay(torch.tensor(0.0, dtype=F64))) - math.exp(-0.5 * math.exp(-0.5))) < 1e-15
    assert float(P.delta_decay(torch.tensor(50.0, dtype=F64))) > math.exp(-math.exp(-0.5)) - 1e-12
    assert float(P.delta_decay(torch.tensor(-50.0, dtype=F64))) > 1 - 1e-12
    # carried state: two halves give what the whole gives
    g = torch.Generator().manual_seed(1)
    mk = lambda *s: torch.rand(*s, generator=g, dtype=F64)
    r, k, v, w, a = mk(9, 2, 3), mk(9, 2, 3) - 0.5, mk(9, 2, 3), mk(9, 2, 3), mk(9, 2, 3)
    whole, S_whole = P.delta_scan(r, k, v, w, a)
    first, S_mid = P.delta_scan(r[:4], k[:4], v[:4], w[:4], a[:4])
    second, S_end = P.delta_scan(r[4:], k[4:], v[4:], w[4:], a[4:], state=S_mid)
    assert torch.allclose(torch.cat([first, second]), whole) and torch.allclose(S_end, S_whole)


def test_rotation_pairings_and_slowed_frequencies_by_hand():
    x = torch.tensor([[[1.0, 0.0, 5.0, 6.0, 7.0, 8.0]]], dtype=F64)              # one token, one head of six
    near = P.rotate(x, [1], [math.pi / 2, math.pi], 1.0, True)                   # pairs (0, 1), (2, 3)
    assert torch.allclose(near[0, 0], torch.tensor([0.0, 1.0, -5.0, -6.0, 7.0, 8.0], dtype=F64), atol=1e-12)
    halves = P.rotate(x, [1], [math.pi / 2, math.pi], 1.0, False)                # pairs (0, 2), (1, 3)
    assert torch.allclose(halves[0, 0], torch.tensor([-5.0, 0.0, 1.0, -6.0, 7.0, 8.0], dtype=F64), atol=1e-12)
    assert torch.equal(P.rotate(x, [0], [0.3, 0.7], 1.0, True), x)
    assert torch.allclose(P.rotate(x, [0], [0.3, 0.7], 1.5, False)[0, 0, :4], x[0, 0, :4] * 1.5)      # cos and sin are made longer
    plain, one = P.rotary_frequencies({"base": 100.0, "dims": 8})
    assert plain == [100.0 ** (-2.0 * i / 8) for i in range(4)] and one == 1.0
    sc = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 1.0}
    f, mult = P.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": sc})
    # the index at which a frequency turns 4 times in 64 positions is 0.81 (floor 0), once: 2.01 (ceil 3)
    lo, hi = 0, 3
    assert abs(mult - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    for i in range(4):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(f[i] - (plain[i] / 4.0 * ramp + plain[i] * (1 - ramp))) < 1e-15
    assert f[0] == plain[0] and abs(f[3] - plain[3] / 4.0) < 1e-18 and plain[1] / 4 < f[1] < plain[1]
    # both ends of the ramp below the first index: a ramp of no width, the first frequency stays, the others are slowed
    g, _m = P.rotary_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 2.0, "original": 4, "fast": 2.0, "slow": 1.0}})
    assert g[0] == plain[0] and all(abs(g[i] - plain[i] / 2.0) < 1e-18 for i in (1, 2, 3))


def test_router_and_clamped_expert_by_hand():
    W = {"m.router": torch.eye(4, dtype=F64)}
    h = torch.tensor([[1.0, 3.0, 2.0, -1.0]], dtype=F64)
    chosen, weight = P.route(h, W, "m.", {"top": 2})
    assert chosen[0].tolist() == [1, 2]
    assert torch.allclose(weight[0], torch.tensor([math.e / (1 + math.e), 1 / (1 + math.e)], dtype=F64))   # among the chosen alone
    one, w1 = P.route(h, W, "m.", {"top": 1})
    assert one[0].tolist() == [1] and float(w1) == 1.0
    # an expert: the gate is cut from above only, the up value on both sides, and (u + 1) multiplies
    W.update({"m.e0.gate": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0], [0, 0, 0, 4.0]], dtype=F64),
              "m.e0.up": torch.tensor([[0, 0, 1.0, 0], [0, 0, 0, 3.0], [0, 1.0, 0, 0]], dtype=F64),
              "m.e0.down": torch.eye(3, dtype=F64)[[0, 1, 2, 0]]})
    y = P.expert(h, W, "m.", 0, 1.5)[0]
    sig = lambda z: 1 / (1 + math.exp(-1.702 * z))
    want = [1.0 * sig(1.0) * (1.5 + 1), 1.5 * sig(1.5) * (-1.5 + 1), -4.0 * sig(-4.0) * (1.5 + 1)]
    assert torch.allclose(y[:3], torch.tensor(want, dtype=F64)) and abs(float(y[3]) - want[0]) < 1e-12


def test_token_side_input_by_hand():
    W = {"l0.side.gate": torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64), "l0.side.proj": torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=F64),
         "l0.side.norm": torch.tensor([1.0, 3.0], dtype=F64)}
    x = torch.tensor([[0.5, -1.0]], dtype=F64)
    e = torch.tensor([[2.0, 1.0]], dtype=F64)
    y = torch.tensor([float(P.gelu_tanh(torch.tensor(0.5, dtype=F64))) * 2.0, float(P.gelu_tanh(torch.tensor(-1.0, dtype=F64))) * 2.0])
    rms = math.sqrt(float((y * y).mean()))
    got = P.side_input(x, W, "l0.", e, 0.0)
    assert torch.allclose(got[0], torch.tensor([y[0] / rms, 3.0 * y[1] / rms], dtype=F64))
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=F64))) - 0.5 * (1 + math.tanh(math.sqrt(2 / math.pi) * 1.044715))) < 1e-15


# ------------------------------------------------------------------ the whole model, stated plainly

@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_model_is_causal_and_its_options_matter(name, benarax_dirs):
    d, _page, raw = benarax_dirs[name]
    _raw, W = bm.load(d)
    toks = bm.requests_for(raw, [45], 5)["r0"]
    streams = []
    full = P.forward(raw, W, toks, streams=streams)
    assert len(streams) == len(P.run_order(raw))
    assert torch.allclose(full[:19], P.forward(raw, W, toks[:19]), atol=1e-9), "a position depends on later tokens"
    assert float(full.abs().max()) > 0.5, "the test model's logits are too flat to show anything"
    assert float((P.forward(raw, W, toks, dtype=torch.float32).double() - full).abs().max()) < 2e-3

    def differs(other_raw=None, other_W=None):
        return float((P.forward(other_raw or raw, other_W or W, toks) - full).abs().max())

    def scaled(suffix, by):
        return {k: (v * by if k.endswith(suffix) else v) for k, v in W.items()}
    assert differs(other_W={k: (v + 1.0 if k.endswith(".mix.w0") else v) for k, v in W.items()}) > 1e-5          # the decay
    assert differs(other_W={k: (v + 1.0 if k.endswith(".mix.a.b") else v) for k, v in W.items()}) > 1e-5         # the erased share
    assert differs(other_W=scaled(".dq.norm", 1.5)) > 1e-5 and differs(other_W=scaled(".dkv.norm", 1.5)) > 1e-5
    if raw.get("canon"):
        assert differs(other_W=scaled(".canon1", 0.0)) > 1e-5
        assert differs(other_raw={k: v for k, v in raw.items() if k != "canon"}) > 1e-5
    if raw.get("token_side"):
        assert differs(other_W=scaled(".side.norm", 0.0)) > 1e-5
        assert differs(other_W={k: (v.roll(1, 1) if k == "side.embed" else v) for k, v in W.items()}) > 1e-5     # whose columns
    assert differs(other_raw={**raw, "residual_mult": raw["residual_mult"] * 1.1}) > 1e-5
    assert differs(other_raw={**raw, "norm": {**raw["norm"], "groups": 1 if raw["norm"]["groups"] > 1 else 2}}) > 1e-5
    if raw.get("loop") and raw["loop"]["times"] > 1:
        assert differs(other_raw={**raw, "loop": {**raw["loop"], "times": raw["loop"]["times"] - 1}}) > 1e-5

    def edit(change):
        layers = []
        for l in raw["layers"]:
            m = {**l["mixer"], "rot": dict(l["mixer"].get("rot") or {})}
            if l["type"] != "general_delta":
                l = {**l, **(change(l["type"], m) or {})}
            layers.append({**l, "mixer": m if l["type"] != "general_delta" else l["mixer"]})
        return {**raw, "layers": layers}

    def other_pairing(kind, m):
        return {"type": "latent_attention_2" if kind == "latent_attention" else "latent_attention"}

    def unscaled(kind, m):
        m["rot"].pop("scaling", None)

    def other_scale(kind, m):
        m["scale"] = m["scale"] * 1.2
    if any(l["mixer"].get("rot_dim", 0) >= 4 for l in raw["layers"]):          # one pair alone is the same pair either way
        assert differs(other_raw=edit(other_pairing)) > 1e-5, "both pairings of rotated elements give the same logits"
    assert differs(other_raw=edit(other_scale)) > 1e-5
    if any((l["mixer"].get("rot") or {}).get("scaling") for l in raw["layers"]):
        assert differs(other_raw=edit(unscaled)) > 1e-5


def test_every_run_of_a_looped_layer_has_its_own_memory(benarax_dirs):
    """The second run of a layer must not see the keys or the state that its first run left: with the loop's layers
    written out as layers of their own (same weights under other names) the logits are the same."""
    d, _page, raw = benarax_dirs["A"]
    _raw, W = bm.load(d)
    toks = bm.requests_for(raw, [30], 6)["r0"]
    order = P.run_order(raw)
    flat = {k: v for k, v in raw.items() if k != "loop"}
    flat["layers"] = [raw["layers"][i] for i in order]
    W2 = {k: v for k, v in W.items() if not k.startswith("l")}
    dim = raw["token_side"]["dim"]
    side = []
    for new, old in enumerate(order):
        for k, v in W.items():
            if k.startswith(f"l{old}."):
                W2[f"l{new}." + k.split(".", 1)[1]] = v
        side.append(W["side.embed"][:, old * dim:(old + 1) * dim])          # every run reads its layer's columns
    W2["side.embed"] = torch.cat(side, dim=1)
    assert torch.allclose(P.forward(raw, W, toks), P.forward(flat, W2, toks), atol=1e-10)


# ------------------------------------------------------------------ configuration and plan

def test_config_round_trip_and_plan(benarax_dirs):
    from inferflux_b200.config import BenaraxConfig, ConfigError, config_from_dict, load_config
    from inferflux_b200.models.model import Model
    d, _page, raw = benarax_dirs["A"]
    cfg = load_config(d)
    assert isinstance(cfg, BenaraxConfig) and cfg.to_dict() == raw
    assert cfg.run_order() == [0, 1, 2, 1, 2, 3] == P.run_order(raw)
    plan = cfg.to_plan()
    assert [plan.layers[e.layer].block.kind for e in plan.schedule] == ["parallel"] * 6
    assert [(e.layer, e.cache, e.repeat) for e in plan.schedule] == [(0, 0, 0), (1, 1, 0), (2, 2, 0), (1, 3, 1), (2, 4, 1), (3, 5, 0)]
    model = Model(plan)
    names = set(model.expected_tensors())
    assert {"embed", "side.embed", "final.norm", "head", "l0.norm1", "l0.canon1", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq",
            "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.o", "l0.mlp.router", "l0.mlp.e0.gate",
            "l0.mlp.e4.up", "l0.mlp.e4.down", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l1.mix.r", "l1.mix.k", "l1.mix.v",
            "l1.mix.g", "l1.mix.a", "l1.mix.a.b", "l1.mix.w1", "l1.mix.w2", "l1.mix.w0", "l1.mix.norm", "l1.mix.o",
            "l3.norm1", "l3.mix.r"} <= names
    assert not {"l0.mix.q", "l0.norm2", "l3.mlp.router", "l0.mlp.e5.up", "l1.mlp.e3.gate", "l0.mix.sink"} & names
    exp = model.expected_tensors()
    assert exp["side.embed"].shape == (300, 4 * 8) and exp["l0.canon1"].shape == (64, 3) and exp["l0.mix.dkv"].shape == (24 + 8, 64)
    assert exp["l1.mix.w1"].shape == (-1, 64) and exp["l1.mix.w1"].fits((11, 64))        # the decay's inner size: the file's
    specs = model.cache_specs()
    conv = 2 * 64                                            # taps - 1 rows of the width, in every layer's state
    kv, st = specs[0]
    assert (kv.planes, kv.num_kv_heads, kv.head_dim, kv.window) == (1, 1, 24 + 8, None) and st.shape == (conv,)
    assert specs[1][0] is None and specs[1][1].shape == (conv + 2 * 16 * 16,) and specs[3][1].shape == specs[1][1].shape
    assert specs[2][0].head_dim == 40 + 16 and specs[4][0].head_dim == 56 and specs[5][1].shape == (conv + 3 * 24 * 24,)
    # without a convolution an attention layer has no state at all
    _d, _p, raw_c = benarax_dirs["C"]
    specs_c = Model(config_from_dict(raw_c).to_plan()).cache_specs()
    assert specs_c[0][1] is None and specs_c[1][0] is None and specs_c[1][1].shape == (8 * 8 * 8,)
    lat = raw["layers"][0]
    for bad in ({**raw, "layers": []}, {**raw, "layers": [{**lat, "type": "other"}]},
                {k: v for k, v in raw.items() if k != "width"}, {**raw, "norm": {"eps": 1e-6, "groups": 3}},
                {**raw, "loop": {"start": 2, "stop": 5, "times": 2}}, {**raw, "loop": {"start": 1, "stop": 3, "times": 0}},
                {**raw, "layers": [{**lat, "mixer": {k: v for k, v in lat["mixer"].items() if k != "kv_rank"}}]},
                {**raw, "layers": [{**lat, "mixer": {**lat["mixer"], "rot": {"base": 100.0, "dims": 7}}}]},
                {**raw, "layers": [{**lat, "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 2, "top": 3}}}]},
                {**raw, "layers": [{**lat, "mlp": {"kind": "moe", "expert": {"ff": 8, "limit": 0.0}, "router": {"experts": 2, "top": 1}}}]}):
        with pytest.raises(ConfigError):
            config_from_dict(bad)


def test_wrong_weights_are_refused_and_the_decay_rank_comes_from_the_file(benarax_dirs, tmp_path):
    from inferflux_b200.models import load_model
    from inferflux_b200.weights import WeightError, write_safetensors
    d, _page, raw = benarax_dirs["D"]
    _raw, W = bm.load(d)
    (tmp_path / "config.json").write_text((d / "config.json").read_text())
    W2 = {k: v for k, v in W.items() if k != "l0.mlp.e1.gate"}
    W2["l2.mix.dkv"] = W["l2.mix.dkv"][:-1].contiguous()
    W2["side.embed"] = W["side.embed"][:, :-1].contiguous()
    write_safetensors(tmp_path / "model.safetensors", W2)
    with pytest.raises(WeightError) as e:
        load_model(tmp_path, dtype="float32", device="cpu")
    assert e.value.missing == ["l0.mlp.e1.gate"] and sorted(w[0] for w in e.value.wrong_shape) == ["l2.mix.dkv", "side.embed"]
    W3 = dict(W)                                            # another inner size of the decay: taken from the tensors
    W3["l0.mix.w1"] = torch.cat([W["l0.mix.w1"], W["l0.mix.w1"][:3] * 0.5])
    W3["l0.mix.w2"] = torch.cat([W["l0.mix.w2"], W["l0.mix.w2"][:, :3] * 0.5], dim=1)
    write_safetensors(tmp_path / "model.safetensors", W3)
    _c, model = load_model(tmp_path, dtype="float32", device="cpu")
    assert model.layers[0].mixer.rank == W["l0.mix.w1"].shape[0] + 3


# ------------------------------------------------------------------ the engine's host logic on plain kernels

LENS = [40, 33, 50, 61, 97, 70, 25, 64, 1, 2]


def _plain_runner(d, page, pages=None, max_seqs=4, max_seq_len=512):
    from inferflux_b200.engine import ModelRunner
    from inferflux_b200.models import load_model
    _c, model = load_model(d, dtype="float32", device="cpu")
    return ModelRunner(model, PlainKernels(wide=True), page_size=page, num_pages=pages or 256 // page, max_seqs=max_seqs,
                       max_seq_len=max_seq_len)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("cutting", ["whole", "tail", "portions", "mixed"])
def test_engine_host_logic_on_plain_kernels(name, cutting, benarax_dirs):
    d, page, raw = benarax_dirs[name]
    reqs = bm.requests_for(raw, LENS, 100)
    want = bm.plain_logits(d, reqs)
    steps = {"whole": helpers.trace_whole, "tail": helpers.trace_tail, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, 256)}[cutting](reqs)
    runner = _plain_runner(d, page)
    got = helpers.collect(steps, helpers.run_steps_in_process(runner, steps), raw["vocab"])
    bad = helpers.first_bad(got, want, 2e-4)
    assert bad is None, f"first wrong row (request, position, diff): {bad}"
    assert not runner.cache.live_requests() and runner.cache.free_pages() == [256 // page] * len(runner.cache.groups)


def test_portions_down_to_two_tokens_and_the_first_tokens(benarax_dirs):
    """Portions of 2, 1, 3, 2, 2, 5 ... tokens from the first token on: the convolution reads the rows that the
    portion before left (and zeros before the sequence's start), the recurrence its state, attention its pages."""
    from inferflux_b200.engine import StepEntry
    for name in ("A", "D"):
        d, page, raw = benarax_dirs[name]
        toks = bm.requests_for(raw, [60], 3)["r0"]
        want = bm.plain_logits(d, {"r0": toks})["r0"]
        runner = _plain_runner(d, page)
        got, pos, sizes, i = [], 0, [2, 1, 3, 2, 2, 5, 1, 1, 2, 17], 0
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            i += 1
            got += list(runner.step([StepEntry("r0", toks[pos:pos + n], list(range(n)))]).double().numpy())
            pos += n
        runner.end_request("r0")
        assert float(np.abs(np.stack(got) - want).max()) < 2e-4, name


def test_a_slot_and_pages_that_are_used_again_start_clean(benarax_dirs):
    from inferflux_b200.engine import StepEntry
    d, page, raw = benarax_dirs["A"]
    reqs = bm.requests_for(raw, [9, 1, 3, 2, 30, 5], 7)
    want = bm.plain_logits(d, reqs)
    runner = _plain_runner(d, page, pages=4, max_seqs=1, max_seq_len=32)
    for rid, toks in reqs.items():                         # one slot, four pages: everybody inherits them
        got = runner.step([StepEntry(rid, toks, list(range(len(toks))))]).double().numpy()
        assert float(np.abs(got - want[rid]).max()) < 2e-4, rid
        assert all(float(s[0].abs().max()) > 0 for s in runner.cache.state if s is not None)
        runner.end_request(rid)
        runner.cache.check()
    assert all(g.alloc.allocations > 4 for g in runner.cache.groups)


def test_greedy_generation_through_engine_and_scheduler(benarax_dirs):
    from inferflux_b200 import Engine, SamplingParams
    d, page, raw = benarax_dirs["A"]
    _raw, W = bm.load(d)
    prompts = list(bm.requests_for(raw, [7, 19, 33, 4, 1], 40).values())

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
