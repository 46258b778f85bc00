#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on the Qwen2.5-7B shape, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with the
context ending at 4,096 tokens, timed on the device with CUDA events around K decode
steps of the step function; the K-step loop is repeated until about half a second has
been timed and the median repeat is reported (`repeats`, `repeat_ms`, the SM clock
beside each).  `e2e` is the same through the Python entry point (`Engine.step`: host
token ids in through pinned memory, sampled ids read back, every step).  `prefill` is
one 2,048-token prompt in one step; `points` holds decode at batch 1 and 64, at
context 2,048 and averaged over 2,048 to 4,096, the prefill as four portions of 512,
and decode and a served workload at the Qwen2.5-1.5B shape; `roofline` compares the
bytes a decode step has to read (every weight once and the cache of the live requests)
with the measured HBM peak; `baselines` times the same model in plain PyTorch (matmul +
scaled_dot_product_attention) on the same GPU; `checked` compares the engine's logits at
the benchmarked depth, batch and context with a float32 PyTorch forward.
Weights are random (N(0, 0.02), norms 1.0), prompts are uniform random token ids.
A decode step reads ~14 GB of weights, far more than the 126 MB L2, so no L2 flush
is needed between timed steps (`l2` in `config` says so).

`--impl reference` runs the unmodified reference (its LlamaForwardTyped<bf16> model
path, built by baseline/build_ref.py with a small driver, baseline/ref_harness.cu) on
the same shape, batch, context and step counts and prints the same line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
CONTEXT = 4096
PREFILL_TOKENS = 2048


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            raw = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in raw.items() if isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (ValueError, OSError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.times = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        try:                                    # NVML in this process: a sample every 20 ms (reading only)
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            try:
                get_reasons = pynvml.nvmlDeviceGetCurrentClocksEventReasons
            except AttributeError:
                get_reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop.is_set():
                bits = int(get_reasons(h))
                self.times.append(time.time())
                self.rows.append([str(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), str(mx), "",
                                  "Active" if bits & 0x8 else "Not Active", "Active" if bits & 0x40 else "Not Active",
                                  "Active" if bits & 0x20 else "Not Active", "Active" if bits & 0x4 else "Not Active"])
                self._stop.wait(0.02)
            return
        except Exception:
            pass
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.times.append(time.time())
                    self.rows.append([c.strip() for c in out.stdout.strip().splitlines()[0].split(",")])
            except (OSError, subprocess.SubprocessError):
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self, begin=None, end=None):
        """Median SM clock and the reasons seen, over all samples or those taken in [begin, end]."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, r in zip(self.times, self.rows):
            if begin is not None and not (begin <= t <= end):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


SHAPES = {   # the three real-sized shapes of the benchmark description
    "7b": dict(hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False),
    "1.5b": dict(hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True),
    "32b": dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=40, num_key_value_heads=8,
                intermediate_size=27648, vocab_size=152064, tie_word_embeddings=False),
}


def qwen7b_config(shape="7b"):
    from inferflux_b200.config import Qwen2Config
    return Qwen2Config(head_dim=128, max_position_embeddings=32768, rope_theta=1000000.0, rms_norm_eps=1e-6,
                       **SHAPES[shape])


def weight_bytes(cfg, batch):
    """Bytes of weights a decode step reads once: every layer matrix, bias and norm,
    the final norm and the head; of the embedding table only the batch's rows."""
    h, i, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads * cfg.head_dim, \
        cfg.num_key_value_heads * cfg.head_dim
    per_layer = 2 * (h * (q + 2 * kv) + q * h + 3 * h * i) + 4 * (q + 2 * kv) + 4 * 2 * h
    head = 2 * cfg.vocab_size * h                       # tied or not, the head's table is read once
    return cfg.num_hidden_layers * per_layer + head + 4 * h + batch * h * 2


def kv_bytes_per_token(cfg):
    return 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2


def prefill_flops(cfg, tokens):
    h, i, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads * cfg.head_dim, \
        cfg.num_key_value_heads * cfg.head_dim
    linear = 2 * tokens * cfg.num_hidden_layers * (h * (q + 2 * kv) + q * h + 3 * h * i)
    attn = cfg.num_hidden_layers * 4 * cfg.num_attention_heads * cfg.head_dim * (tokens * (tokens + 1) // 2)
    head = 2 * cfg.vocab_size * h                       # logits of the last position only
    return linear + attn + head


def random_prompts(cfg, n, length, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (length,), generator=g).tolist() for _ in range(n)]


def bring_to_decode(engine, prompts, max_tokens):
    """Prefill every prompt through the engine until all requests are decoding."""
    from inferflux_b200.sampling import SamplingParams
    for p in prompts:
        engine.add_request(p, SamplingParams(temperature=0.0), max_tokens=max_tokens)
    guard = 0
    while engine.scheduler.waiting or any(r.remaining > 1 or not r.output for r in engine.scheduler.running):
        engine.step()
        guard += 1
        if guard > 100000:
            raise RuntimeError("prefill did not finish")


def end_all(engine):
    """End every live request outside the scheduler's books (their lengths were moved by direct steps)."""
    engine.drain()
    for r in list(engine.scheduler.running):
        r.status = "finished"
        engine.scheduler.running.remove(r)
        if r.request_id in engine.runner.cache:
            engine.runner.end_request(r.request_id)
    engine.scheduler.waiting.clear()


def time_decode(engine, cfg, batch, steps, warmup, repeats=1, context=4096, clock=None, e2e=True):
    """Decode at `batch` with the last timed step ending at `context` tokens.  Returns a dict:
    dev_ms (median over `repeats` loops of exactly `steps` steps, CUDA events around each loop),
    repeat_ms, repeat_spans (wall-clock begin/end of each loop), e2e_ms (through Engine.step),
    launches per step, h2d/d2h bytes per step, ctx (tokens per request after the last step)."""
    import torch
    from inferflux_b200.engine import StepEntry
    timed = repeats * steps
    total = warmup + timed
    # The last timed step ends at `context`: the prompt leaves room for both timed loops and for the tokens
    # the first requests decode while the last prompts are still prefilled (8,192 prompt tokens a step).
    # So no step of the timed loops is the first of a longer context class (its CUDA graph would be
    # captured inside the timing).
    loops = 2 if e2e else 1
    prompt_len = context - loops * total - 2 - (-(-batch * context // 8192) + 2)
    prompts = random_prompts(cfg, batch, prompt_len, seed=batch)
    bring_to_decode(engine, prompts, max_tokens=4 * total + 8 + batch)   # the first ones decode while the last prefill
    runner, kernels = engine.runner, engine.kernels
    out = {}

    # ---- end to end through the entry point: scheduler, step, sampling, ids back to the host
    if e2e:
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        h2d0, d2h0 = engine.stats.h2d_bytes, engine.stats.d2h_bytes
        walls = []
        for _ in range(repeats):
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            walls.append((time.perf_counter() - t0) * 1000.0 / steps)
        out["e2e_ms"] = statistics.median(walls)
        out["h2d"] = (engine.stats.h2d_bytes - h2d0) / timed
        out["d2h"] = (engine.stats.d2h_bytes - d2h0) / timed

    # ---- the step function alone, timed on the device
    engine.drain()
    rids = [r.request_id for r in engine.scheduler.running]
    assert len(rids) == batch, f"{len(rids)} of {batch} requests are still decoding"
    g = torch.Generator().manual_seed(1)
    feed = torch.randint(0, cfg.vocab_size, (total, batch), generator=g).tolist()

    def one(i):
        logits = runner.step([StepEntry(rid, [feed[i][b]], [0]) for b, rid in enumerate(rids)])
        return kernels.argmax(logits)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = kernels.launches
    ms, spans = [], []
    with (clock if clock is not None else _Null()):
        for r in range(repeats):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.time()
            start.record()
            for i in range(warmup + r * steps, warmup + (r + 1) * steps):
                one(i)
            end.record()
            torch.cuda.synchronize()
            spans.append((t0, time.time()))
            ms.append(start.elapsed_time(end) / steps)
    out["dev_ms"] = statistics.median(ms)
    out["repeat_ms"] = ms
    out["repeat_spans"] = spans
    out["launches"] = (kernels.launches - l0) / timed
    out["ctx"] = runner.cache.length(rids[0])
    kernels.check_errors()
    end_all(engine)
    return out


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


def time_prefill(engine, cfg, tokens, warmup, reps, portion=0):
    """Median ms of one prompt of `tokens` tokens: in one step, or in portions of `portion`."""
    import torch
    from inferflux_b200.engine import StepEntry
    runner = engine.runner
    prompts = random_prompts(cfg, warmup + reps, tokens, seed=99)
    portion = portion or tokens
    times = []
    for i, p in enumerate(prompts):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for at in range(0, tokens, portion):
            part = p[at:at + portion]
            runner.step([StepEntry(f"prefill-{i}", part, [len(part) - 1] if at + portion >= tokens else [])])
        end.record()
        torch.cuda.synchronize()
        runner.end_request(f"prefill-{i}")
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def serve_workload(engine, cfg, requests, new_tokens, seed=3, prompt_len=0):
    """Many requests with prompts of uniform random length through the scheduler: chunked
    prefill mixed with decode, as a server would run them.  Returns (seconds, prompt tokens,
    generated tokens, steps, preemptions)."""
    import torch
    from inferflux_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    lens = [prompt_len] * requests if prompt_len else torch.randint(128, 2049, (requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    for p in prompts:
        engine.add_request(p, SamplingParams(temperature=0.0), max_tokens=new_tokens)
    torch.cuda.synchronize()
    steps0 = engine.stats.steps
    t0 = time.perf_counter()
    done = 0
    while engine.has_unfinished():
        done += len(engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert done == requests, f"{done} of {requests} requests finished"
    return dt, sum(lens), requests * new_tokens, engine.stats.steps - steps0, engine.stats.preemptions


def check_logits(engine, cfg, batch, context, rows, steps=4):
    """The engine's logits at the benchmarked depth, batch and context against a float32 PyTorch
    forward of the whole sequence: `batch` requests are prefilled through the engine to just under
    `context` tokens, then decoded for `steps` steps with given tokens through the step function (the
    path the timing uses: CUDA-graph replay from the second step on), and the last step's logits of
    `rows` are compared.  The yardstick for the error is the same model in plain bfloat16 PyTorch."""
    import torch
    from inferflux_b200.engine import StepEntry
    from baseline.torch_plain import TorchPlain
    torch.backends.cuda.matmul.allow_tf32 = False
    prompt_len = context - steps - 2 - (-(-batch * context // 8192) + 2)
    prompts = random_prompts(cfg, batch, prompt_len, seed=1000 + batch)
    bring_to_decode(engine, prompts, max_tokens=steps + 64 + batch)
    engine.drain()
    reqs = list(engine.scheduler.running)
    assert len(reqs) == batch
    g = torch.Generator().manual_seed(2)
    feed = torch.randint(0, cfg.vocab_size, (steps, batch), generator=g).tolist()
    # what each request holds so far: its prompt and the tokens it decoded while the others were prefilled;
    # its last sampled token has not been run yet and is replaced by the fed ones
    history = {b: list(r.prompt) + list(r.output[:engine.runner.cache.length(r.request_id) - len(r.prompt)])
               for b, r in enumerate(reqs)}
    logits = None
    for i in range(steps):
        logits = engine.runner.step([StepEntry(r.request_id, [feed[i][b]], [0]) for b, r in enumerate(reqs)])
        for b in range(batch):
            history[b].append(feed[i][b])
    engine.kernels.check_errors()
    got = logits.float()
    exact, plain16 = TorchPlain(engine.model, torch.float32), TorchPlain(engine.model, torch.bfloat16)
    worst = yard = scale = 0.0
    agree = 0
    for b in rows:
        want = exact.logits_last(history[b])[0]
        mine, theirs = got[b], plain16.logits_last(history[b])[0]
        worst = max(worst, float((mine - want).abs().max()))
        yard = max(yard, float((theirs - want).abs().max()))
        scale = max(scale, float(want.abs().max()))
        agree += int(int(mine.argmax()) == int(want.argmax()))
    ctx = engine.runner.cache.length(reqs[0].request_id)
    graphs = engine.runner.graph_replays
    end_all(engine)
    return {"batch": batch, "ctx": ctx, "rows": len(rows), "steps": steps, "max_err": round(worst, 4),
            "torch_bf16_err": round(yard, 4), "logit_scale": round(scale, 2), "argmax_agree": agree,
            "graph_replays": graphs, "ok": bool(worst <= 2.0 * yard + 1e-3 * scale)}


def run_reference(args, pk):
    """The reference arm: the unmodified reference model path (LlamaForwardTyped<bf16>::Forward /
    BatchForward + GpuSampler) driven by baseline/ref_harness at the same shape, batch, context and
    step counts.  None of this repository's kernels is loaded: the harness is a program of its own."""
    sys.path.insert(0, str(ROOT / "baseline"))
    try:
        from build_ref import build as build_reference
        exe = build_reference()
    except Exception as e:                                   # no sources, no nvcc, compile error
        print(json.dumps({"impl": "reference", "unavailable": f"the reference arm cannot be built: {e}"[:300]}))
        return 0
    cfg = qwen7b_config(args.shape)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    cmd = [str(exe), "bench", "dtype=bf16", f"hidden={cfg.hidden_size}", f"layers={cfg.num_hidden_layers}",
           f"heads={cfg.num_attention_heads}", f"kv_heads={cfg.num_key_value_heads}", f"head_dim={cfg.head_dim}",
           f"inter={cfg.intermediate_size}", f"vocab={cfg.vocab_size}", f"theta={cfg.rope_theta}",
           f"eps={cfg.rms_norm_eps}", f"tied={int(cfg.tie_word_embeddings)}", "bias=1", f"max_pos={CONTEXT}",
           f"ctx_end={CONTEXT}", f"steps={steps}", f"warmup={warmup}", f"prefill_tokens={PREFILL_TOKENS}",
           "batches=" + ",".join(map(str, batches))]
    clock = ClockSampler()
    with clock:
        proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference harness exited with {proc.returncode}: {proc.stderr.strip()[-200:]}"}))
        return 0
    raw = json.loads(proc.stdout.strip().splitlines()[-1])
    main = raw[f"b{args.batch}"]
    value = args.batch * 1000.0 / main["dev_ms"]
    step_bytes = weight_bytes(cfg, args.batch) + args.batch * main["ctx_end"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (main["dev_ms"] * 1e-3) / 1e9
    pf = prefill_flops(cfg, PREFILL_TOKENS) / (raw["prefill_ms"] * 1e-3)
    line = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B bf16 (also batch 1/64 and prefill tok/s at 2,048 tokens)",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["dev_ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": f"Qwen2.5-{args.shape.upper()} shape", "layers": cfg.num_hidden_layers,
                   "layers_full": SHAPES[args.shape]["num_hidden_layers"], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": CONTEXT, "context_at_timing": main["ctx_end"], "kv_cache": "contiguous (the reference's)",
                   "parallelism": "single GPU", "l2": "inputs larger than L2 (GBs of weights per step), no flush",
                   "peaks": pk["source"], "cuda_graph": bool(main["graph"])},
        "form": "stock model path: the reference's LlamaForwardTyped<bf16> (Forward, BatchForward), KvCacheGpuTyped, "
                "CublasGemm and GpuSampler, unmodified, driven by baseline/ref_harness.cu; the executor, scheduler and "
                "HTTP server above them are not built (they need llama.cpp)",
        "clocks": clock.summary(main["timed_begin"], main["timed_end"]),
        "e2e": {"value": round(args.batch * 1000.0 / main["e2e_ms"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main["h2d_bytes"], "d2h_bytes_per_step": main["d2h_bytes"],
                "ms_per_step": round(main["e2e_ms"], 4)},
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / raw["prefill_ms"], 1), "tokens": PREFILL_TOKENS,
                    "ms": round(raw["prefill_ms"], 3), "frac": round(pf / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {f"decode_b{b}": round(b * 1000.0 / raw[f"b{b}"]["dev_ms"], 2) for b in batches if b != args.batch},
        "impl": "reference",
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------- another design beside the closest existing model
# Dafolorn at sizes that resemble real layers, and the Qwen2 shape of equal size: the same width, heads, vocabulary and
# number of layer runs (2 + 6 looped 4 times + 2 = 28); the feed-forward has two matrices instead of three, so it is
# 1.5 times as wide; key/value heads of 128 against a latent of 256 per token; a window of 4,096.
DESIGN_SHAPES = {
    "1.5b": dict(width=1536, heads=12, ff=13440, vocab=151936, qwen="1.5b"),
    "7b": dict(width=3584, heads=28, ff=28416, vocab=152064, qwen="7b"),
}


def dafolorn_config(shape, window=4096, rank=256):
    from inferflux_b200.config import DafolornConfig
    s = DESIGN_SHAPES[shape]
    layer = {"type": "latent_attention",
             "mixer": {"heads": s["heads"], "dim": 128, "vdim": 128, "kv_rank": rank, "mask": {"size": window},
                       "scale": 128 ** -0.5},
             "mlp": {"kind": "dense", "ff": s["ff"]}}
    return DafolornConfig.from_dict({"architecture": "Dafolorn", "vocab": s["vocab"], "width": s["width"],
                                     "norm": {"eps": 1e-6}, "canon": {"taps": 4}, "logit_softcap": 30.0,
                                     "loop": {"start": 2, "stop": 8, "times": 4}, "layers": [layer] * 10})


def dafolorn_step_bytes(cfg, batch, context):
    """Bytes a decode step must read: every matrix of every layer run, the merges, the head, the cached latents."""
    w, total = cfg.width, 0
    runs = cfg.run_order()
    for i, _rep, first in runs:
        m, mlp = cfg.layers[i]["mixer"], cfg.layers[i]["mlp"]
        q, v, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["kv_rank"]
        total += 2 * (w * (q + r) + q * r + v * r + v * w + (2 * w * mlp["ff"] if mlp else 0))
        total += 2 * w * 2 * w if first else 0
        keys = min(context, (m.get("mask") or {}).get("size") or context)
        total += batch * keys * r * 2
    return total + 2 * cfg.vocab * w


def dafolorn_prefill_flops(cfg, tokens):
    w, total = cfg.width, 0
    for i, _rep, first in cfg.run_order():
        m, mlp = cfg.layers[i]["mixer"], cfg.layers[i]["mlp"]
        q, v, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["kv_rank"]
        total += 2 * tokens * (w * (q + r) + q * r + v * r + v * w + (2 * w * mlp["ff"] if mlp else 0) + (2 * w * w if first else 0))
        total += 4 * m["heads"] * r * (tokens * (tokens + 1) // 2)       # scores and sums over latents (window >= tokens)
    return total + 2 * cfg.vocab * w


def _event_times(fn, reps=15, warm=3):
    """Median ms of fn() alone on the device: captured into a CUDA graph (so that the host's time between its
    launches does not count) and replayed with the L2 flushed (a 512 MB write) before every timed replay."""
    import torch
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda:0")
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    times = []
    for i in range(warm + reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        if i >= warm:
            times.append(a.elapsed_time(b))
    return statistics.median(times)


def design_kernels(kernels, dcfg, qcfg, pk, batch, context, tokens):
    """The new design's kernels beside the like kernels of the closest model, each alone at the layer's sizes:
    microseconds and the fraction of its roofline (HBM bytes, or tensor FLOPs where those take longer)."""
    import torch
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import KVCacheSpec
    dev, bf = "cuda:0", torch.bfloat16
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    m = dcfg.layers[0]["mixer"]
    H, dk, dv, r, w = m["heads"], m["dim"], m["vdim"], m["kv_rank"], dcfg.width
    nq, nkv, d = qcfg.num_attention_heads, qcfg.num_key_value_heads, qcfg.head_dim
    page, out = 16, {}

    def row(name, ms, bytes_=0, flops=0):
        roof = max(bytes_ / hbm, flops / tf)
        out[name] = {"us": round(ms * 1000, 1), "roofline_us": round(roof * 1e6, 1), "frac": round(roof / (ms * 1e-3), 3),
                     "bound": "hbm" if bytes_ / hbm >= flops / tf else "tensor"}

    def ctx_for(cache, spans):
        entries, starts, slots = [], [], []
        for rid, n in spans:
            if rid not in cache:
                cache.add_request(rid)
            start = cache.length(rid)
            cache.reserve(rid, start + n)
            entries.append(StepEntry(rid, [0] * n, []))
            starts.append(start)
            slots.append(cache.slot(rid))
        ctx = StepContext.build(kernels, bf, dev, entries, starts, slots, cache.drain_table_updates())
        for g, (idx, pg) in zip(cache.groups, ctx.table_updates):
            kernels.scatter_i32(g.table, idx, pg)
        for (rid, n), start in zip(spans, starts):
            cache.commit(rid, start + n)
        return ctx

    for what, spans_a, spans_b in (("decode", [(f"r{i}", context - 1) for i in range(batch)], [(f"r{i}", 1) for i in range(batch)]),
                                   ("prefill", [], [("p", tokens)])):
        T = sum(n for _r, n in spans_b)
        keys = sum((context if what == "decode" else (n * (n + 1)) // 2) for _r, n in spans_b)
        pages = (batch * context if what == "decode" else tokens) // page + 2 * batch + 2
        # the new design: one latent plane
        cache = CacheManager([(KVCacheSpec(1, r, None, planes=1), None)], page_size=page, num_pages=pages, max_seqs=batch,
                             max_seq_len=max(context, tokens) + 16, dtype=bf, device=dev)
        cache.groups[0].pool.normal_()
        if spans_a:
            ctx_for(cache, spans_a)
        ctx = ctx_for(cache, spans_b)
        view = cache.view(ScheduleEntry(0, 0))
        q_rows = torch.randn(T, H * dk + r, device=dev).to(bf)
        w_uk, w_uv = (torch.randn(H * dk, r, device=dev) * 0.05).to(bf), (torch.randn(H * dv, r, device=dev) * 0.05).to(bf)
        sinks = torch.zeros(H, device=dev)
        ms = _event_times(lambda: kernels.latent_attention(q_rows, w_uk, w_uv, sinks, H, dk, dv, r, None, dk ** -0.5, ctx, view))
        row(f"latent attention, {what} (3 launches: into latent space, tiles, values)", ms,
            bytes_=(batch * context if what == "decode" else tokens) * r * 2 + 2 * T * H * (dk + r + r + dv),
            flops=4 * H * r * keys + 2 * T * H * r * (dk + dv))
        del cache
        # the closest model: keys and values of nkv heads
        cache = CacheManager([(KVCacheSpec(nkv, d, None), None)], page_size=page, num_pages=pages, max_seqs=batch,
                             max_seq_len=max(context, tokens) + 16, dtype=bf, device=dev)
        cache.groups[0].pool.normal_()
        if spans_a:
            ctx_for(cache, spans_a)
        ctx = ctx_for(cache, spans_b)
        view = cache.view(ScheduleEntry(0, 0))
        q = torch.randn(T, nq * d, device=dev).to(bf)
        ms = _event_times(lambda: kernels.attention(q, nq, nkv, d, None, d ** -0.5, ctx, view))
        row(f"attention of the closest model, {what}", ms,
            bytes_=(batch * context if what == "decode" else tokens) * 2 * nkv * d * 2 + 4 * T * nq * d, flops=4 * nq * d * keys)
        del cache
        # rows: sum + norms; convolution; activation
        x = torch.randn(T, w, device=dev)
        y = torch.randn(T, w, device=dev).to(bf)
        wn = torch.ones(w, device=dev)
        ms = _event_times(lambda: kernels.postnorm_add(x, y, wn, 1e-6, wn, 1e-6, bf))
        row(f"sum of the normed delta + next norm, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        ms = _event_times(lambda: kernels.add_rmsnorm(x, y, wn, 1e-6, bf))
        row(f"sum + norm of the closest model, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        state = torch.zeros(batch, 2, 3, w, device=dev)
        wc = torch.randn(w, 4, device=dev)
        ms = _event_times(lambda: kernels.short_conv(y, wc, 4, state, 0, ctx))
        row(f"short convolution, {T} rows", ms, bytes_=T * w * 4)
        ff = dcfg.layers[0]["mlp"]["ff"]
        z = torch.randn(T, ff, device=dev).to(bf)
        ms = _event_times(lambda: kernels.xielu(z, 0.69, 1.19))
        row(f"xIELU, {T} rows", ms, bytes_=T * ff * 4)
        gu = torch.randn(T, 2 * qcfg.intermediate_size, device=dev).to(bf)
        ms = _event_times(lambda: kernels.silu_mul(gu))
        row(f"SiLU * up of the closest model, {T} rows", ms, bytes_=T * qcfg.intermediate_size * 6)
    kernels.check_errors()
    return out


def run_design(args, pk):
    """`--design dafolorn`: decode and prefill throughput of the design at real layer sizes beside the Qwen2 shape of
    equal size, and its kernels beside the like kernels, one JSON line."""
    import torch
    page, batch, context = 16, args.batch, min(args.context, 4096)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    result = {"metric": "decode and prefill tokens/s of another design beside the closest model at equal size",
              "design": args.design, "dtype": "bf16", "n_gpus": 1, "data": "synthetic: random weights, uniform random token ids",
              "batch": batch, "context": context, "prefill_tokens": PREFILL_TOKENS, "peaks": pk["source"], "shapes": {}}
    kernels_table = None
    for shape in ([args.shape] if args.shape in DESIGN_SHAPES else sorted(DESIGN_SHAPES)):
        entry = {}
        for name in ("dafolorn", "qwen2"):
            cfg = dafolorn_config(shape) if name == "dafolorn" else qwen7b_config(DESIGN_SHAPES[shape]["qwen"])
            if args.layers and name == "qwen2":
                cfg.num_hidden_layers = args.layers
            longest = context + 4 * (warmup + 3 * steps) + 16 + batch
            engine = _engine(cfg, page, batch, longest)
            r = time_decode(engine, cfg, batch, steps, warmup, repeats=3, context=context, e2e=False)
            pre_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=5)
            if name == "dafolorn":
                step_bytes, flops = dafolorn_step_bytes(cfg, batch, r["ctx"]), dafolorn_prefill_flops(cfg, PREFILL_TOKENS)
            else:
                step_bytes = weight_bytes(cfg, batch) + batch * r["ctx"] * kv_bytes_per_token(cfg)
                flops = prefill_flops(cfg, PREFILL_TOKENS)
            entry[name] = {"decode_tok_s": round(batch * 1000.0 / r["dev_ms"], 1), "decode_ms_per_step": round(r["dev_ms"], 3),
                           "decode_hbm_frac": round(step_bytes / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
                           "launches_per_step": round(r["launches"], 1),
                           "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 2),
                           "prefill_tensor_frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3)}
            if name == "dafolorn" and kernels_table is None:
                kernels_table = design_kernels(engine.kernels, cfg, qwen7b_config(DESIGN_SHAPES[shape]["qwen"]), pk, batch,
                                               context, PREFILL_TOKENS)
                entry["kernels"] = kernels_table
            del engine
            torch.cuda.empty_cache()
        result["shapes"][shape] = entry
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------- Zeluzen beside the closest existing model
# Layers in the pattern recurrence, recurrence, attention, recurrence, recurrence, attention that reads the cache of the
# attention layer before it; feed-forwards alternate between the gated one of the Qwen2 shape and a mixture of 16 + 2
# experts of which a token uses 4, sized so that a token's active feed-forward parameters equal the gated one's.
def zeluzen_config(shape, layers=0, chunk=8192):
    from inferflux_b200.config import ZeluzenConfig
    s = DESIGN_SHAPES[shape]
    q = qwen7b_config(s["qwen"])
    w, inter = s["width"], q.intermediate_size
    n = layers or q.num_hidden_layers
    dense = {"kind": "dense", "ff": inter}
    moe = {"kind": "moe", "expert": {"ff": (3 * inter // 8) // 64 * 64}, "router": {"experts": 16, "identity": 2, "top": 4}}
    rot = {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    out, last_attention = [], None
    for i in range(n):
        mlp = dense if i % 2 == 0 else moe
        if i % 3 != 2:
            out.append({"type": "wkv", "mixer": {"heads": w // 64, "dim": 64, "rank": 64}, "mlp": mlp})
            continue
        mixer = {"heads": s["heads"], "kv_heads": q.num_key_value_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                 "mask": {"size": chunk}, "rot": rot}
        if last_attention is not None and (i // 3) % 2 == 1:
            mixer["kv_from"] = last_attention
        else:
            last_attention = i
        out.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return ZeluzenConfig.from_dict({"architecture": "Zeluzen", "vocab": s["vocab"], "width": w, "norm": {"eps": 1e-6}, "layers": out})


def zeluzen_costs(cfg, batch, context, tokens):
    """(bytes a decode step must read or write, FLOPs of a prefill of `tokens`): matrices (a token's 4 experts, and at
    most all of them), recurrent state in and out, cached keys and values."""
    w, step_bytes, flops = cfg.width, 0, 0
    for layer in cfg.layers:
        m, mlp = layer["mixer"], layer["mlp"]
        if layer["type"] == "wkv":
            hd, rank = m["heads"] * m["dim"], m.get("rank") or 16
            params = 5 * hd * w + 2 * rank * max(w, hd)
            step_bytes += 2 * batch * m["heads"] * m["dim"] * m["dim"] * 4
            flops += 4 * tokens * hd * m["dim"]
        else:
            own = m.get("kv_from") is None
            params = w * m["heads"] * m["dim"] + m["heads"] * m["vdim"] * w + (w * m["kv_heads"] * (m["dim"] + m["vdim"]) if own else 0)
            keys = min(context, m["mask"]["size"]) if m.get("mask") else context
            step_bytes += batch * keys * m["kv_heads"] * (m["dim"] + m["vdim"]) * 2
            flops += 2 * m["heads"] * (m["dim"] + m["vdim"]) * (tokens * (tokens + 1) // 2)
        step_bytes += 2 * params
        flops += 2 * tokens * params
        if mlp and mlp["kind"] == "dense":
            step_bytes += 2 * 3 * w * mlp["ff"]
            flops += 2 * tokens * 3 * w * mlp["ff"]
        elif mlp:
            r = mlp["router"]
            step_bytes += 2 * 2 * w * mlp["expert"]["ff"] * min(r["experts"], batch * r["top"])
            flops += 2 * tokens * 2 * w * mlp["expert"]["ff"] * r["top"]
    return step_bytes + 2 * cfg.vocab * w, flops + 2 * cfg.vocab * w


def zeluzen_kernels(kernels, zcfg, qcfg, pk, batch, context, tokens):
    """The new design's kernels beside the like kernels of the closest model, each alone at the layer's sizes."""
    import torch
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import KVCacheSpec
    dev, bf = "cuda:0", torch.bfloat16
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    wk = next(l for l in zcfg.layers if l["type"] == "wkv")["mixer"]
    at = next(l for l in zcfg.layers if l["type"] == "attention")["mixer"]
    moe = next(l["mlp"] for l in zcfg.layers if l["mlp"] and l["mlp"]["kind"] == "moe")
    w, H, D = zcfg.width, wk["heads"], wk["dim"]
    nq, nkv, d = qcfg.num_attention_heads, qcfg.num_key_value_heads, qcfg.head_dim
    page, out = 16, {}

    def row(name, ms, bytes_=0, flops=0):
        roof = max(bytes_ / hbm, flops / tf)
        out[name] = {"us": round(ms * 1000, 1), "roofline_us": round(roof * 1e6, 1), "frac": round(roof / (ms * 1e-3), 3),
                     "bound": "hbm" if bytes_ / hbm >= flops / tf else "tensor"}

    def ctx_for(cache, spans):
        entries, starts, slots = [], [], []
        for rid, n in spans:
            if rid not in cache:
                cache.add_request(rid)
            start = cache.length(rid)
            cache.reserve(rid, start + n)
            entries.append(StepEntry(rid, [0] * n, []))
            starts.append(start)
            slots.append(cache.slot(rid))
        ctx = StepContext.build(kernels, bf, dev, entries, starts, slots, cache.drain_table_updates())
        for g, (idx, pg) in zip(cache.groups, ctx.table_updates):
            kernels.scatter_i32(g.table, idx, pg)
        for (rid, n), start in zip(spans, starts):
            cache.commit(rid, start + n)
        return ctx

    for what, spans_a, spans_b in (("decode", [(f"r{i}", context - 1) for i in range(batch)], [(f"r{i}", 1) for i in range(batch)]),
                                   ("prefill", [], [("p", tokens)])):
        T = sum(n for _r, n in spans_b)
        keys = sum((context if what == "decode" else (n * (n + 1)) // 2) for _r, n in spans_b)
        pages = (batch * context if what == "decode" else tokens) // page + 2 * batch + 2
        cached = batch * context if what == "decode" else tokens
        for name, spec, kw in (("attention with chunks and a sink", KVCacheSpec(at["kv_heads"], 128, None, chunk=at["mask"]["size"]),
                                dict(chunk=at["mask"]["size"], sink=True, dv=128)),
                               ("attention of the closest model", KVCacheSpec(nkv, d, None), {})):
            cache = CacheManager([(spec, None)], page_size=page, num_pages=pages, max_seqs=batch,
                                 max_seq_len=max(context, tokens) + 16, dtype=bf, device=dev)
            cache.groups[0].pool.normal_()
            if spans_a:
                ctx_for(cache, spans_a)
            ctx = ctx_for(cache, spans_b)
            view = cache.view(ScheduleEntry(0, 0))
            heads, kvh, hd = (at["heads"], at["kv_heads"], 128) if kw else (nq, nkv, d)
            q = torch.randn(T, heads * hd, device=dev).to(bf)
            ms = _event_times(lambda: kernels.attention(q, heads, kvh, hd, None, hd ** -0.5, ctx, view, **kw))
            row(f"{name}, {what}", ms, bytes_=cached * 2 * kvh * hd * 2 + 4 * T * heads * hd, flops=4 * heads * hd * keys)
            del cache
        # the recurrence: state in and out, five float32 inputs, a scratch row and the output
        state = torch.zeros(batch, H * D * D + w, device=dev)
        ins = [torch.randn(T, H * D, device=dev) * 0.1 for _ in range(5)]
        consts = [torch.zeros(H * D, device=dev), torch.zeros(H * D, device=dev), torch.ones(H * D, device=dev)]
        x = torch.randn(T, w, device=dev)
        ms = _event_times(lambda: kernels.wkv_scan(*ins, *consts, 1e-6, H, D, state, H * D * D, x, ctx, bf))
        row(f"recurrence over {T} tokens ({what})", ms, bytes_=2 * len(spans_b) * H * D * D * 4 + T * H * D * (5 * 4 + 8 + 2),
            flops=0)
        mu = torch.rand(5, w, device=dev)
        ms = _event_times(lambda: kernels.token_shift_mix(x, mu, state, H * D * D, ctx, bf))
        row(f"five mixes of a token and the one before, {T} rows", ms, bytes_=T * w * (4 + 5 * 2))
        y = torch.randn(T, w, device=dev).to(bf)
        wn = torch.ones(w, device=dev)
        ms = _event_times(lambda: kernels.postnorm_add(x, y, wn, 1e-6, out_dtype=bf, cast_out=True))
        row(f"sum of the normed delta + rows in bfloat16, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        ms = _event_times(lambda: kernels.add_rmsnorm(x, y, wn, 1e-6, bf))
        row(f"sum + norm of the closest model, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        # the experts against the closest model's gated feed-forward (both: all matrices a token uses)
        E, top, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
        up = (torch.randn(E, ff, w, device=dev) * 0.02).to(bf)
        down = (torch.randn(E, w, ff, device=dev) * 0.02).to(bf)
        h = torch.randn(T, w, device=dev).to(bf)
        z = torch.randn(T, E + moe["router"]["identity"], device=dev)
        corr = torch.zeros(E + moe["router"]["identity"], device=dev)
        ids, wts = kernels.moe_route(z, corr, top)
        ms = _event_times(lambda: kernels.moe_route(z, corr, top))
        row(f"router, {T} rows", ms, bytes_=T * (E + 2) * 4)
        used = min(E, T * top)
        ms = _event_times(lambda: kernels.moe_experts(h, up, down, ids, wts, E, bf))
        row(f"experts, {T} rows", ms, bytes_=used * 2 * ff * w * 2, flops=2 * T * top * 2 * ff * w)
        inter = qcfg.intermediate_size
        wgu, wd = (torch.randn(2 * inter, w, device=dev) * 0.02).to(bf), (torch.randn(w, inter, device=dev) * 0.02).to(bf)
        ms = _event_times(lambda: kernels.materialize(kernels.linear(kernels.linear_swiglu(h, wgu), wd, allow_partial=True)))
        row(f"gated feed-forward of the closest model, {T} rows", ms, bytes_=3 * inter * w * 2, flops=2 * T * 3 * inter * w)
        del up, down, wgu, wd
    kernels.check_errors()
    return out


def run_design_zeluzen(args, pk):
    """`--design zeluzen`: decode and prefill throughput of the design at real layer sizes beside the Qwen2 shape of
    equal width, layer count and vocabulary, and its kernels beside the like kernels, one JSON line."""
    import torch
    page, batch, context = 16, args.batch, min(args.context, 4096)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    result = {"metric": "decode and prefill tokens/s of another design beside the closest model at equal size",
              "design": args.design, "dtype": "bf16", "n_gpus": 1, "data": "synthetic: random weights, uniform random token ids",
              "batch": batch, "context": context, "prefill_tokens": PREFILL_TOKENS, "peaks": pk["source"], "shapes": {}}
    kernels_table = None
    for shape in ([args.shape] if args.shape in DESIGN_SHAPES else sorted(DESIGN_SHAPES)):
        entry = {}
        for name in ("zeluzen", "qwen2"):
            cfg = zeluzen_config(shape, args.layers) if name == "zeluzen" else qwen7b_config(DESIGN_SHAPES[shape]["qwen"])
            if args.layers and name == "qwen2":
                cfg.num_hidden_layers = args.layers
            longest = context + 4 * (warmup + 3 * steps) + 16 + batch
            engine = _engine(cfg, page, batch, longest)
            r = time_decode(engine, cfg, batch, steps, warmup, repeats=3, context=context, e2e=False)
            pre_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=5)
            if name == "zeluzen":
                step_bytes, flops = zeluzen_costs(cfg, batch, r["ctx"], PREFILL_TOKENS)
            else:
                step_bytes = weight_bytes(cfg, batch) + batch * r["ctx"] * kv_bytes_per_token(cfg)
                flops = prefill_flops(cfg, PREFILL_TOKENS)
            entry[name] = {"decode_tok_s": round(batch * 1000.0 / r["dev_ms"], 1), "decode_ms_per_step": round(r["dev_ms"], 3),
                           "decode_hbm_frac": round(step_bytes / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
                           "launches_per_step": round(r["launches"], 1),
                           "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 2),
                           "prefill_tensor_frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3)}
            if name == "zeluzen" and kernels_table is None:
                kernels_table = zeluzen_kernels(engine.kernels, cfg, qwen7b_config(DESIGN_SHAPES[shape]["qwen"]), pk, batch,
                                                context, PREFILL_TOKENS)
                entry["kernels"] = kernels_table
            del engine
            torch.cuda.empty_cache()
        result["shapes"][shape] = entry
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------- Benarax beside Zeluzen
def benarax_config(shape, layers=0):
    """Benarax at the sizes of `zeluzen_config`: two delta-rule layers (heads of 64), then a latent attention layer (heads of
    128 + 64 rotated, a latent of 256, queries through a latent of 1,536), the two pairings taking turns; every layer a
    mixture of 16 gated experts of which a token uses 4, sized so that a token's active feed-forward parameters equal the
    Qwen2 shape's; norms over 8 groups, a convolution of 4 taps, a token side input of 256 columns a layer."""
    from inferflux_b200.config import BenaraxConfig
    s = DESIGN_SHAPES[shape]
    q = qwen7b_config(s["qwen"])
    w, inter = s["width"], q.intermediate_size
    n = layers or q.num_hidden_layers
    moe = {"kind": "moe", "expert": {"ff": (inter // 4) // 64 * 64, "limit": 7.0}, "router": {"experts": 16, "top": 4}}
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    out = []
    for i in range(n):
        if i % 3 != 2:
            out.append({"type": "general_delta", "mixer": {"heads": w // 64, "dim": 64, "rank": 64}, "mlp": moe})
            continue
        kind = "latent_attention" if (i // 3) % 2 == 0 else "latent_attention_2"
        out.append({"type": kind, "mixer": {"heads": s["heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 256,
                                            "q_rank": 1536, "scale": 192 ** -0.5, "rot": rot}, "mlp": moe})
    return BenaraxConfig.from_dict({"architecture": "Benarax", "vocab": s["vocab"], "width": w, "norm": {"eps": 1e-6, "groups": 8},
                                    "canon": {"taps": 4}, "token_side": {"dim": 256}, "embedding": {"scale": 1.0},
                                    "logit_scale": 1.0, "residual_mult": 1.0, "layers": out})


def benarax_costs(cfg, batch, context, tokens):
    """(bytes a decode step must read or write, FLOPs of a prefill of `tokens`): matrices (a token's experts, and at most
    all of them), recurrent state in and out, cached latent rows."""
    w, step_bytes, flops = cfg.width, 0, 0
    side = cfg.side_dim or 0
    for layer in cfg.layers:
        m, mlp = layer["mixer"], layer["mlp"]
        if layer["type"] == "general_delta":
            hd, rank = m["heads"] * m["dim"], m.get("rank") or 16
            params = 6 * hd * w + rank * (w + hd)
            step_bytes += 2 * batch * m["heads"] * m["dim"] * m["dim"] * 4
            flops += 6 * tokens * hd * m["dim"]
        else:
            H, dq, row = m["heads"], m["dim"] + m["rot_dim"], m["kv_rank"] + m["rot_dim"]
            params = w * (m["q_rank"] + row) + m["q_rank"] * H * dq + H * (m["dim"] + m["vdim"]) * m["kv_rank"] + H * m["vdim"] * w
            step_bytes += batch * context * row * 2
            flops += 2 * H * (row + m["kv_rank"]) * (tokens * (tokens + 1) // 2)
        params += 2 * side * w
        step_bytes += 2 * params
        flops += 2 * tokens * params
        if mlp:
            r = mlp["router"]
            step_bytes += 2 * 3 * w * mlp["expert"]["ff"] * min(r["experts"], batch * r["top"])
            flops += 2 * tokens * 3 * w * mlp["expert"]["ff"] * r["top"]
    return step_bytes + 2 * cfg.vocab * w, flops + 2 * cfg.vocab * w


def benarax_kernels(kernels, bcfg, zcfg, pk, batch, context, tokens):
    """The new design's kernels beside the like kernels of the closest models, each alone at the layer's sizes: the
    delta-rule scan beside Zeluzen's recurrence, latent attention with a rotated part beside Dafolorn's latent attention,
    gated experts beside Zeluzen's, the norm over groups behind a normed delta beside the norm over the row."""
    import torch
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import KVCacheSpec
    from inferflux_b200.parts.base import RotaryTable
    dev, bf = "cuda:0", torch.bfloat16
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    dl = next(l for l in bcfg.layers if l["type"] == "general_delta")["mixer"]
    at = next(l for l in bcfg.layers if l["type"] != "general_delta")["mixer"]
    moe = next(l["mlp"] for l in bcfg.layers if l["mlp"])
    zmoe = next(l["mlp"] for l in zcfg.layers if l["mlp"] and l["mlp"]["kind"] == "moe")
    w, H, D = bcfg.width, dl["heads"], dl["dim"]
    page, out = 16, {}

    def row(name, ms, bytes_=0, flops=0):
        roof = max(bytes_ / hbm, flops / tf)
        out[name] = {"us": round(ms * 1000, 1), "roofline_us": round(roof * 1e6, 1), "frac": round(roof / (ms * 1e-3), 3),
                     "bound": "hbm" if bytes_ / hbm >= flops / tf else "tensor"}

    def ctx_for(cache, spans, providers=()):
        entries, starts, slots = [], [], []
        for rid, n in spans:
            if rid not in cache:
                cache.add_request(rid)
            start = cache.length(rid)
            cache.reserve(rid, start + n)
            entries.append(StepEntry(rid, [0] * n, []))
            starts.append(start)
            slots.append(cache.slot(rid))
        ctx = StepContext.build(kernels, bf, dev, entries, starts, slots, cache.drain_table_updates(), providers=providers)
        for g, (idx, pg) in zip(cache.groups, ctx.table_updates):
            kernels.scatter_i32(g.table, idx, pg)
        for (rid, n), start in zip(spans, starts):
            cache.commit(rid, start + n)
        return ctx

    class _Sections:                                       # asks the kernel table for the latent kernels' work lists
        def step_sections(self, ctx):
            return ctx.kernels.latent_attention_sections(ctx)

    AH, dk, rot, dv, rank = at["heads"], at["dim"], at["rot_dim"], at["vdim"], at["kv_rank"]
    for what, spans_a, spans_b in (("decode", [(f"r{i}", context - 1) for i in range(batch)], [(f"r{i}", 1) for i in range(batch)]),
                                   ("prefill", [], [("p", tokens)])):
        T = sum(n for _r, n in spans_b)
        keys = sum((context if what == "decode" else (n * (n + 1)) // 2) for _r, n in spans_b)
        pages = (batch * context if what == "decode" else tokens) // page + 2 * batch + 2
        cached = batch * context if what == "decode" else tokens
        for name, extra in (("latent attention with a rotated part", rot), ("latent attention of the closest model", 0)):
            cache = CacheManager([(KVCacheSpec(1, rank + extra, None, planes=1), None)], page_size=page, num_pages=pages,
                                 max_seqs=batch, max_seq_len=max(context, tokens) + 16, dtype=bf, device=dev)
            cache.groups[0].pool.normal_()
            if spans_a:
                ctx_for(cache, spans_a)
            ctx = ctx_for(cache, spans_b, providers=[_Sections()])
            view = cache.view(ScheduleEntry(0, 0))
            uk, uv = (torch.randn(AH * dk, rank, device=dev) * 0.05).to(bf), (torch.randn(AH * dv, rank, device=dev) * 0.05).to(bf)
            q = (torch.randn(T, AH * (dk + extra), device=dev) * 0.3).to(bf)
            if extra:
                down = torch.randn(T, rank + extra, device=dev).to(bf)
                table = RotaryTable(torch.rand(extra // 2, device=dev), extra, True, 1.0)
                lw = torch.ones(rank, device=dev)
                queries = kernels.latent_rope_append(down, 0, rank, extra, lw, 1e-6, q, AH, dk, table, ctx, view, vdim=dv)
                ms = _event_times(lambda: kernels.latent_rope_append(down, 0, rank, extra, lw, 1e-6, q, AH, dk, table, ctx, view, vdim=dv))
                row(f"latent row: norm, rotation, append, {what}", ms, bytes_=T * (2 * (rank + extra) * 2 + 2 * AH * extra * 2))
            else:
                queries = q
            ms = _event_times(lambda: kernels.latent_attention(queries, uk, uv, None, AH, dk, dv, rank, None, (dk + rot) ** -0.5, ctx,
                                                               view, rot=extra))
            row(f"{name}, {what}", ms, bytes_=cached * (rank + extra) * 2 + 2 * T * AH * (dk + dv) * 2 + AH * (dk + dv) * rank * 2,
                flops=2 * AH * (2 * rank + extra) * keys + 2 * T * AH * (dk + dv) * rank)
            del cache
        # the recurrences: state in and out, float32 inputs, scratch rows and the output
        ctx = type("C", (), {})()
        cu = [0]
        for _r, n in spans_b:
            cu.append(cu[-1] + n)
        ctx.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
        ctx.req_slot = torch.arange(len(spans_b), dtype=torch.int32, device=dev)
        ctx.num_requests, ctx.num_tokens = len(spans_b), T
        state = torch.zeros(batch, H * D * D + w, device=dev)
        proj = torch.randn(T, 5 * H * D, device=dev) * 0.1
        w_raw = torch.randn(T, H * D, device=dev)
        consts = [torch.zeros(H * D, device=dev), torch.zeros(H * D, device=dev), torch.ones(H * D, device=dev)]
        ms = _event_times(lambda: kernels.delta_rule_scan(proj, w_raw, *consts, 1e-6, H, D, state, ctx, bf))
        row(f"delta-rule recurrence over {T} tokens ({what})", ms,
            bytes_=2 * len(spans_b) * H * D * D * 4 + T * H * D * (6 * 4 + 4 * 8 + 2))
        ins = [torch.randn(T, H * D, device=dev) * 0.1 for _ in range(5)]
        x = torch.randn(T, w, device=dev)
        ms = _event_times(lambda: kernels.wkv_scan(*ins, *consts, 1e-6, H, D, state, H * D * D, x, ctx, bf))
        row(f"recurrence of the closest model over {T} tokens ({what})", ms,
            bytes_=2 * len(spans_b) * H * D * D * 4 + T * H * D * (5 * 4 + 8 + 2))
        y = torch.randn(T, w, device=dev).to(bf)
        wn = torch.ones(w, device=dev)
        ms = _event_times(lambda: kernels.postnorm_add(x, y, wn, 1e-6, wn, 1e-6, bf, groups=bcfg.norm_groups))
        row(f"sum of the normed delta + norm over groups, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        ms = _event_times(lambda: kernels.postnorm_add(x, y, wn, 1e-6, wn, 1e-6, bf))
        row(f"sum of the normed delta + norm of the closest model, {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        a, b = torch.randn(T, w, device=dev).to(bf), torch.randn(T, w, device=dev).to(bf)
        ms = _event_times(lambda: kernels.residual_add_scaled(x, a, b, 0.5, out_dtype=bf))
        row(f"scaled sum of both sublayers + rows in bfloat16, {T} rows", ms, bytes_=T * w * (8 + 2 + 2 + 2))
        # the gated experts against the closest model's (both: all matrices a token uses)
        h = torch.randn(T, w, device=dev).to(bf)
        for name, cfg_moe, gated in (("gated experts", moe, True), ("experts of the closest model", zmoe, False)):
            E, top, ff = cfg_moe["router"]["experts"], cfg_moe["router"]["top"], cfg_moe["expert"]["ff"]
            n_out = E + (0 if gated else cfg_moe["router"].get("identity", 0))
            up = (torch.randn(E, (2 if gated else 1) * ff, w, device=dev) * 0.02).to(bf)
            down = (torch.randn(E, w, ff, device=dev) * 0.02).to(bf)
            z = torch.randn(T, n_out, device=dev)
            if gated:
                ids, wts = kernels.moe_route(z, None, top, of_chosen=True)
                ms = _event_times(lambda: kernels.moe_route(z, None, top, of_chosen=True))
                row(f"router over the chosen, {T} rows", ms, bytes_=T * (E + 2) * 4)
                ms = _event_times(lambda: kernels.moe_experts(h, up, down, ids, wts, E, bf, glu=(7.0, 1.702)))
            else:
                ids, wts = kernels.moe_route(z, torch.zeros(n_out, device=dev), top)
                ms = _event_times(lambda: kernels.moe_experts(h, up, down, ids, wts, E, bf))
            mats = 3 if gated else 2
            row(f"{name}, {T} rows", ms, bytes_=min(E, T * top) * mats * ff * w * 2, flops=2 * T * top * mats * ff * w)
            del up, down
    kernels.check_errors()
    return out


def run_design_benarax(args, pk):
    """`--design benarax`: decode and prefill throughput of the design at real layer sizes beside Zeluzen, the closest
    model, at equal width, layer count, vocabulary and active feed-forward parameters, and its kernels beside the like
    kernels, one JSON line."""
    import torch
    page, batch, context = 16, args.batch, min(args.context, 4096)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    result = {"metric": "decode and prefill tokens/s of another design beside the closest model at equal size",
              "design": args.design, "dtype": "bf16", "n_gpus": 1, "data": "synthetic: random weights, uniform random token ids",
              "batch": batch, "context": context, "prefill_tokens": PREFILL_TOKENS, "peaks": pk["source"], "shapes": {}}
    kernels_table = None
    for shape in ([args.shape] if args.shape in DESIGN_SHAPES and args.shape != "7b" else sorted(DESIGN_SHAPES)):
        entry = {}
        for name in ("benarax", "zeluzen"):
            cfg = benarax_config(shape, args.layers) if name == "benarax" else zeluzen_config(shape, args.layers)
            longest = context + 4 * (warmup + 3 * steps) + 16 + batch
            engine = _engine(cfg, page, batch, longest)
            r = time_decode(engine, cfg, batch, steps, warmup, repeats=3, context=context, e2e=False)
            pre_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=5)
            step_bytes, flops = (benarax_costs if name == "benarax" else zeluzen_costs)(cfg, batch, r["ctx"], PREFILL_TOKENS)
            entry[name] = {"decode_tok_s": round(batch * 1000.0 / r["dev_ms"], 1), "decode_ms_per_step": round(r["dev_ms"], 3),
                           "decode_hbm_frac": round(step_bytes / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
                           "launches_per_step": round(r["launches"], 1),
                           "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 2),
                           "prefill_tensor_frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3)}
            if name == "benarax" and kernels_table is None:
                kernels_table = benarax_kernels(engine.kernels, cfg, zeluzen_config(shape, args.layers), pk, batch, context,
                                                PREFILL_TOKENS)
                entry["kernels"] = kernels_table
            del engine
            torch.cuda.empty_cache()
        result["shapes"][shape] = entry
    print(json.dumps(result))
    return 0


# ---------------------------------------------------------------- Radalix beside Benarax, the closest existing model
def radalix_config(shape, layers=0):
    """Radalix at the sizes of `benarax_config`: layers of a pair of mixers, the two kinds taking turns.  Left: attention
    with the Qwen2 shape's query heads of 128 over two (1.5B) or four (7B) key/value heads, four taps behind the
    projections; without positions, with a query multiplier and an output gate in one kind, with 64 turned elements,
    slowed frequencies, a window of 8,192 and a learned sink in the other.  Right: a matrix state per head with a decay per
    key channel (heads of 64 keys x 128 values) or a selective state-space recurrence (heads of 64 values, a state of
    128, one group, four taps).  Every layer a mixture of 16 gated experts of which a token uses 3, plus one that every
    token uses, sized so that a token's active feed-forward parameters equal the Qwen2 shape's."""
    from inferflux_b200.config import RadalixConfig
    s = DESIGN_SHAPES[shape]
    q = qwen7b_config(s["qwen"])
    w, inter = s["width"], q.intermediate_size
    n = layers or q.num_hidden_layers
    ff = (inter // 4) // 64 * 64
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": 16, "top": 3}, "shared": {"ff": ff}}
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    left = {"heads": s["heads"], "kv_heads": q.num_key_value_heads, "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "conv": 4}
    out = []
    for i in range(n):
        if i % 2 == 0:
            out.append({"type": "parallel", "mlp": moe, "mixer": {
                "left": {**left, "q_temp": {"coef": 0.1, "every": 1024}},
                "right": {"heads": w // 128, "dim": 64, "vdim": 128, "tau": 16.0}}})
        else:
            out.append({"type": "parallel_2", "mlp": moe, "mixer": {
                "left": {**left, "mask": {"size": 8192}, "rot": rot}, "left_scale": 1.0, "right_scale": 1.0,
                "right": {"heads": w // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}}})
    return RadalixConfig.from_dict({"architecture": "Radalix", "vocab": s["vocab"], "width": w, "norm": {"eps": 1e-6},
                                    "embedding": {"scale": 1.0, "bigram": {"buckets": 65521, "mul_prev": 31, "mul_cur": 17}},
                                    "logit_softcap": 30.0, "layers": out})


def radalix_costs(cfg, batch, context, tokens):
    """(bytes a decode step must read or write, FLOPs of a prefill of `tokens`): matrices (a token's experts, and at most
    all of them), recurrent state in and out, cached keys and values."""
    w, step_bytes, flops = cfg.width, 0, 0
    for layer in cfg.layers:
        l, r, mlp = layer["mixer"]["left"], layer["mixer"]["right"], layer["mlp"]
        qd, kd, vd = l["heads"] * l["dim"], l["kv_heads"] * l["dim"], l["kv_heads"] * l["vdim"]
        params = w * (qd + kd + vd) + l["heads"] * l["vdim"] * w * (2 if layer["type"] == "parallel" else 1)
        keys = min(context, l["mask"]["size"]) if l.get("mask") else context
        step_bytes += batch * keys * (kd + vd) * 2
        flops += 2 * l["heads"] * (l["dim"] + l["vdim"]) * (tokens * (tokens + 1) // 2)
        if layer["type"] == "parallel":
            K, V = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            params += w * (2 * K + 2 * V) + 16 * (w + K) + V * w
            state = r["heads"] * r["dim"] * r["vdim"]
        else:
            inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
            params += w * (2 * inner + 2 * gn + r["heads"]) + inner * w
            state = r["heads"] * r["state"] * r["vdim"]
        step_bytes += 2 * batch * state * 4
        flops += 4 * tokens * state
        step_bytes += 2 * params
        flops += 2 * tokens * params
        if mlp:
            rt = mlp["router"]
            shared = (mlp.get("shared") or {}).get("ff", 0)
            step_bytes += 2 * 3 * w * (mlp["expert"]["ff"] * min(rt["experts"], batch * rt["top"]) + shared)
            flops += 2 * tokens * 3 * w * (mlp["expert"]["ff"] * rt["top"] + shared)
    return step_bytes + 2 * cfg.vocab * w, flops + 2 * cfg.vocab * w


def radalix_kernels(kernels, rcfg, bcfg, pk, batch, context, tokens):
    """The new design's kernels beside the like kernels of the closest models, each alone at the layer's sizes: the scan with
    a decayed matrix state (both decays) beside the delta-rule scan, attention with a learned sink beside attention with a
    plain one, the convolution behind the projections, the gated norm, the pair's sum and the vector-scaled residual sum
    beside the scaled sum of both sublayers, plain gated experts beside clamped ones."""
    import torch
    from inferflux_b200.cache import CacheManager
    from inferflux_b200.config import ScheduleEntry
    from inferflux_b200.engine.batch import StepContext, StepEntry
    from inferflux_b200.parts import KVCacheSpec
    dev, bf = "cuda:0", torch.bfloat16
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    gla = next(l for l in rcfg.layers if l["type"] == "parallel")["mixer"]["right"]
    ssm = next(l for l in rcfg.layers if l["type"] == "parallel_2")["mixer"]["right"]
    left = next(l for l in rcfg.layers if l["type"] == "parallel_2")["mixer"]["left"]
    moe = next(l["mlp"] for l in rcfg.layers if l["mlp"])
    dl = next(l for l in bcfg.layers if l["type"] == "general_delta")["mixer"]
    w = rcfg.width
    page, out = 16, {}

    def row(name, ms, bytes_=0, flops=0):
        roof = max(bytes_ / hbm, flops / tf)
        out[name] = {"us": round(ms * 1000, 1), "roofline_us": round(roof * 1e6, 1), "frac": round(roof / (ms * 1e-3), 3),
                     "bound": "hbm" if bytes_ / hbm >= flops / tf else "tensor"}

    def ctx_for(cache, spans, providers=()):
        entries, starts, slots = [], [], []
        for rid, n in spans:
            if rid not in cache:
                cache.add_request(rid)
            start = cache.length(rid)
            cache.reserve(rid, start + n)
            entries.append(StepEntry(rid, [0] * n, []))
            starts.append(start)
            slots.append(cache.slot(rid))
        ctx = StepContext.build(kernels, bf, dev, entries, starts, slots, cache.drain_table_updates(), providers=providers)
        for g, (idx, pg) in zip(cache.groups, ctx.table_updates):
            kernels.scatter_i32(g.table, idx, pg)
        for (rid, n), start in zip(spans, starts):
            cache.commit(rid, start + n)
        return ctx

    class _Sections:                                       # asks the kernel table for the attention kernels' work lists
        def step_sections(self, ctx):
            return ctx.kernels.attention_sections(ctx)

    nq, nkv, d = left["heads"], left["kv_heads"], left["dim"]
    for what, spans_a, spans_b in (("decode", [(f"r{i}", context - 1) for i in range(batch)], [(f"r{i}", 1) for i in range(batch)]),
                                   ("prefill", [], [("p", tokens)])):
        T = sum(n for _r, n in spans_b)
        keys = sum((context if what == "decode" else (n * (n + 1)) // 2) for _r, n in spans_b)
        pages = (batch * context if what == "decode" else tokens) // page + 2 * batch + 2
        cached = batch * context if what == "decode" else tokens
        cache = CacheManager([(KVCacheSpec(nkv, d, None), None)], page_size=page, num_pages=pages, max_seqs=batch,
                             max_seq_len=max(context, tokens) + 16, dtype=bf, device=dev)
        cache.groups[0].pool.normal_()
        if spans_a:
            ctx_for(cache, spans_a)
        ctx = ctx_for(cache, spans_b, providers=[_Sections()])
        view = cache.view(ScheduleEntry(0, 0))
        q = (torch.randn(T, nq * d, device=dev) * 0.3).to(bf)
        sinks = torch.randn(nq, device=dev)
        for name, sink in (("attention with a learned sink", sinks), ("attention with a plain sink (the closest model's)", True)):
            ms = _event_times(lambda: kernels.attention(q, nq, nkv, d, 8192, d ** -0.5, ctx, view, sink=sink))
            row(f"{name}, {what}", ms, bytes_=cached * nkv * 2 * d * 2 + 2 * T * nq * d * 2, flops=4 * nq * d * keys)
        # the convolution behind the stacked projections, then rotation, query multiplier and cache rows
        width = (nq + 2 * nkv) * d
        qkv = torch.randn(T, width, device=dev).to(bf)
        taps = torch.randn(width, 4, device=dev)
        cstate = torch.zeros(batch, 1, 3, width, device=dev)
        ms = _event_times(lambda: kernels.short_conv(qkv, taps, 4, cstate, 0, ctx, add_input=False))
        row(f"convolution behind the projections, {T} rows ({what})", ms, bytes_=T * width * 4 + (2 * len(spans_b) * 3 * width * 4 if what == "decode" else 0))
        del cache
        # the scans: state in and out, float32 inputs, the output
        sctx = type("C", (), {})()
        cu = [0]
        for _r, n in spans_b:
            cu.append(cu[-1] + n)
        sctx.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=dev)
        sctx.req_slot = torch.arange(len(spans_b), dtype=torch.int32, device=dev)
        sctx.num_requests, sctx.num_tokens, sctx.max_span = len(spans_b), T, max(n for _r, n in spans_b)
        H, dk, dv = gla["heads"], gla["dim"], gla["vdim"]
        state = torch.zeros(batch, H * dk * dv, device=dev)
        qq, kk, raw = (torch.randn(T, H * dk, device=dev) * 0.1 for _ in range(3))
        vv = torch.randn(T, H * dv, device=dev) * 0.1
        ms = _event_times(lambda: kernels.decay_scan(qq, kk, vv, raw, state, sctx, heads=H, groups=H, dk=dk, dv=dv, decay="sigmoid_root",
                                                     tau=16.0, q_scale=dk ** -0.5))
        row(f"scan, decay per key channel, {T} tokens ({what})", ms, bytes_=2 * len(spans_b) * H * dk * dv * 4 + T * H * (3 * dk + 2 * dv) * 4)
        H2, n2, dv2, G2 = ssm["heads"], ssm["state"], ssm["vdim"], ssm["groups"]
        state2 = torch.zeros(batch, H2 * n2 * dv2, device=dev)
        bc = [torch.randn(T, G2 * n2, device=dev) * 0.1 for _ in range(2)]
        xx, dt = torch.randn(T, H2 * dv2, device=dev) * 0.1, torch.randn(T, H2, device=dev)
        vec = [torch.zeros(H2, device=dev) for _ in range(3)]
        ms = _event_times(lambda: kernels.decay_scan(bc[0], bc[1], xx, dt, state2, sctx, heads=H2, groups=G2, dk=n2, dv=dv2,
                                                     decay="softplus_step", step_bias=vec[0], log_rate=vec[1], skip=vec[2]))
        row(f"scan, decay per head from a step size, {T} tokens ({what})", ms,
            bytes_=2 * len(spans_b) * H2 * n2 * dv2 * 4 + T * (2 * G2 * n2 + 2 * H2 * dv2 + H2) * 4)
        HB, DB = dl["heads"], dl["dim"]
        state3 = torch.zeros(batch, HB * DB * DB, device=dev)
        proj = torch.randn(T, 5 * HB * DB, device=dev) * 0.1
        w_raw = torch.randn(T, HB * DB, device=dev)
        consts = [torch.zeros(HB * DB, device=dev), torch.zeros(HB * DB, device=dev), torch.ones(HB * DB, device=dev)]
        ms = _event_times(lambda: kernels.delta_rule_scan(proj, w_raw, *consts, 1e-6, HB, DB, state3, sctx, bf))
        row(f"delta-rule scan of the closest model, {T} tokens ({what})", ms,
            bytes_=2 * len(spans_b) * HB * DB * DB * 4 + T * HB * DB * (6 * 4 + 4 * 8 + 2))
        # rows: the two norms, the gated norms, the pair's sum, the residual sum
        x = torch.randn(T, w, device=dev)
        wn = torch.ones(w, device=dev)
        ms = _event_times(lambda: kernels.rmsnorm_pair(x, wn, 1e-6, wn, 1e-6, bf))
        row(f"two norms of one row, {T} rows", ms, bytes_=T * w * (4 + 2 + 2))
        ms = _event_times(lambda: kernels.rmsnorm(x, wn, 1e-6, bf))
        row(f"one norm of a row (the closest model's), {T} rows", ms, bytes_=T * w * (4 + 2))
        inner = H2 * dv2
        y, gate = torch.randn(T, inner, device=dev), torch.randn(T, inner, device=dev)
        wi = torch.ones(inner, device=dev)
        ms = _event_times(lambda: kernels.gated_groupnorm(y, gate, wi, 1e-6, 1, True, bf))
        row(f"gate and norm behind the scan, {T} rows", ms, bytes_=T * inner * (4 + 4 + 2))
        a, b = torch.randn(T, w, device=dev).to(bf), torch.randn(T, w, device=dev)
        ms = _event_times(lambda: kernels.pair_combine(a, b, wn, wn, 0.5, 0.5, 1e-6))
        row(f"the pair's sum with both norms, {T} rows", ms, bytes_=T * w * (2 + 4 + 4))
        f1, f2 = torch.randn(T, w, device=dev).to(bf), torch.randn(T, w, device=dev).to(bf)
        ms = _event_times(lambda: kernels.residual_add_vectors(x, b, wn, f1, wn, f2))
        row(f"residual sum with vectors, {T} rows", ms, bytes_=T * w * (8 + 4 + 2 + 2))
        ms = _event_times(lambda: kernels.residual_add_scaled(x, f1, f2, 0.5))
        row(f"scaled sum of both sublayers (the closest model's), {T} rows", ms, bytes_=T * w * (8 + 2 + 2))
        # the experts: plain gated beside clamped gated (the same kernels)
        h = torch.randn(T, w, device=dev).to(bf)
        E, top, ff = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
        up = (torch.randn(E, 2 * ff, w, device=dev) * 0.02).to(bf)
        down = (torch.randn(E, w, ff, device=dev) * 0.02).to(bf)
        z = torch.randn(T, E, device=dev)
        ids, wts = kernels.moe_route(z, None, top, kind="sigmoid_normalized", floor=1e-20)
        ms = _event_times(lambda: kernels.moe_route(z, None, top, kind="sigmoid_normalized", floor=1e-20))
        row(f"router, sigmoid scores over their sum, {T} rows", ms, bytes_=T * (E + 2) * 4)
        for name, glu in (("plain gated experts", (float("inf"), 1.0, 0.0)), ("clamped gated experts (the closest model's)", (7.0, 1.702, 1.0))):
            ms = _event_times(lambda: kernels.moe_experts(h, up, down, ids, wts, E, bf, glu=glu))
            row(f"{name}, {T} rows", ms, bytes_=min(E, T * top) * 3 * ff * w * 2, flops=2 * T * top * 3 * ff * w)
        del up, down
    kernels.check_errors()
    return out


def run_design_radalix(args, pk):
    """`--design radalix`: decode and prefill throughput of the design at real layer sizes beside Benarax, the closest
    model, at equal width, layer count, vocabulary and active feed-forward parameters, and its kernels beside the like
    kernels, one JSON line."""
    import torch
    page, batch, context = 16, args.batch, min(args.context, 4096)
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    result = {"metric": "decode and prefill tokens/s of another design beside the closest model at equal size",
              "design": args.design, "dtype": "bf16", "n_gpus": 1, "data": "synthetic: random weights, uniform random token ids",
              "batch": batch, "context": context, "prefill_tokens": PREFILL_TOKENS, "peaks": pk["source"], "shapes": {}}
    kernels_table = None
    for shape in ([args.shape] if args.shape in DESIGN_SHAPES and args.shape != "7b" else sorted(DESIGN_SHAPES)):
        entry = {}
        for name in ("radalix", "benarax"):
            cfg = radalix_config(shape, args.layers) if name == "radalix" else benarax_config(shape, args.layers)
            longest = context + 4 * (warmup + 3 * steps) + 16 + batch
            engine = _engine(cfg, page, batch, longest)
            r = time_decode(engine, cfg, batch, steps, warmup, repeats=3, context=context, e2e=False)
            pre_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=5)
            step_bytes, flops = (radalix_costs if name == "radalix" else benarax_costs)(cfg, batch, r["ctx"], PREFILL_TOKENS)
            entry[name] = {"decode_tok_s": round(batch * 1000.0 / r["dev_ms"], 1), "decode_ms_per_step": round(r["dev_ms"], 3),
                           "decode_hbm_frac": round(step_bytes / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
                           "launches_per_step": round(r["launches"], 1),
                           "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "prefill_ms": round(pre_ms, 2),
                           "prefill_tensor_frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 3)}
            if name == "radalix" and kernels_table is None:
                kernels_table = radalix_kernels(engine.kernels, cfg, benarax_config(shape, args.layers), pk, batch, context,
                                                PREFILL_TOKENS)
                entry["kernels"] = kernels_table
            del engine
            torch.cuda.empty_cache()
        result["shapes"][shape] = entry
    print(json.dumps(result))
    return 0



def _engine(cfg, page, slots, longest, pages=None, chunk=2048):
    import torch
    from inferflux_b200 import Engine
    return Engine(config=cfg, seed=0, dtype="bfloat16", device=torch.device("cuda:0"), kv_page_size=page,
                  kv_num_pages=pages or slots * (longest // page + 2), kv_max_batch=slots, kv_max_seq=longest,
                  max_batch_size=slots, max_batch_tokens=8192, chunked_prefill_tokens=chunk)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="tokens per request at the last timed decode step (default: the headline's 4,096)")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the shape has (named in config)")
    ap.add_argument("--shape", default="7b", choices=sorted(SHAPES), help="model shape (default: the 7B headline shape)")
    ap.add_argument("--timed-seconds", type=float, default=0.5,
                    help="repeat the K-step loop until about this much has been timed (the median repeat is reported)")
    ap.add_argument("--serve", type=int, default=0, metavar="REQUESTS",
                    help="instead of the decode/prefill numbers: REQUESTS prompts of 128..2048 tokens, 256 new tokens "
                         "each, chunked prefill of 512 mixed with decode, through the scheduler")
    ap.add_argument("--serve-prompt", type=int, default=0, metavar="TOKENS",
                    help="with --serve: every prompt has this length (default: uniform in [128, 2048])")
    ap.add_argument("--serve-new", type=int, default=256, metavar="TOKENS", help="with --serve: new tokens per request")
    ap.add_argument("--no-points", action="store_true", help="skip the other decode points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill (for profiling decode)")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of logits with the float32 PyTorch forward")
    ap.add_argument("--no-extras", action="store_true", help="skip the PyTorch baseline and the 1.5B-shape points")
    ap.add_argument("--prefill-only", action="store_true",
                    help="time only the 2,048-token prefill and print a short line (for profiling prefill)")
    ap.add_argument("--design", default="", choices=["", "dafolorn", "zeluzen", "benarax", "radalix"],
                    help="instead of the headline numbers: this design at real layer sizes beside the Qwen2 shape of equal "
                         "size (decode and prefill tokens/s, and its kernels beside the like kernels); --shape picks one size")
    args = ap.parse_args()

    pk = peaks()
    if args.impl == "reference":
        return run_reference(args, pk)
    if args.design == "zeluzen":
        return run_design_zeluzen(args, pk)
    if args.design == "benarax":
        return run_design_benarax(args, pk)
    if args.design == "radalix":
        return run_design_radalix(args, pk)
    if args.design:
        return run_design(args, pk)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup, steps = max(3, args.warmup), max(1, args.steps)
    context = args.context
    if context != CONTEXT:          # another context length: the headline's other points and checks do not apply
        args.no_points = args.no_check = args.no_extras = True

    import torch

    cfg = qwen7b_config(args.shape)
    full_layers = cfg.num_hidden_layers
    if args.layers:
        cfg.num_hidden_layers = args.layers
    page = 16
    model_name = f"Qwen2.5-{args.shape.upper()} shape"
    if args.serve:
        n = args.serve
        longest = (args.serve_prompt or 2048) + args.serve_new
        engine = _engine(cfg, page, n, longest + 64, chunk=512)
        serve_workload(engine, cfg, min(n, 8), 16, prompt_len=min(args.serve_prompt, 1024))   # warm-up: kernels, graphs
        dt, pt, gt, steps_run, pre = serve_workload(engine, cfg, n, args.serve_new, prompt_len=args.serve_prompt)
        print(json.dumps({"metric": "served tokens/s (prompt + generated), chunked prefill mixed with decode",
                          "value": round((pt + gt) / dt, 1), "generated_tok_s": round(gt / dt, 1), "unit": "tokens/s",
                          "seconds": round(dt, 3), "steps": steps_run, "requests": n, "prompt_tokens": pt,
                          "generated_tokens": gt, "preemptions": pre, "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": model_name, "layers": cfg.num_hidden_layers,
                                     "prompts": args.serve_prompt or "uniform in [128, 2048]", "prefill_chunk": 512,
                                     "new_tokens": args.serve_new, "kv_page": page}, "impl": "ours"}))
        return 0
    if args.prefill_only:
        engine = _engine(cfg, page, 2, PREFILL_TOKENS + 64, chunk=PREFILL_TOKENS)
        ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=warmup, reps=steps)
        fl = prefill_flops(cfg, PREFILL_TOKENS) / (ms * 1e-3)
        print(json.dumps({"metric": "prefill tok/s at 2,048 tokens", "value": round(PREFILL_TOKENS * 1000.0 / ms, 1),
                          "unit": "tokens/s", "ms": round(ms, 3), "frac": round(fl / (pk["bf16_tflops"] * 1e12), 4),
                          "dtype": "bf16", "n_gpus": 1,
                          "config": {"model": model_name, "layers": cfg.num_hidden_layers,
                                     "layers_full": full_layers, "kv_page": page, "peaks": pk["source"]},
                          "impl": "ours"}))
        return 0

    # how often the K-step loop is repeated: about --timed-seconds at the rate the bytes allow
    est_ms = (weight_bytes(cfg, args.batch) + args.batch * context * kv_bytes_per_token(cfg)) / (0.7 * pk["hbm_gbs"] * 1e6)
    repeats = max(1, min(12, int(-(-args.timed_seconds * 1000.0 // (steps * est_ms)))))
    biggest = max(args.batch, 1 if args.no_points else 64)
    longest = context + 4 * (warmup + repeats * steps) + 8 + biggest   # a prompt plus the most new tokens time_decode allows
    cfg.max_position_embeddings = max(cfg.max_position_embeddings, longest)
    engine = _engine(cfg, page, biggest, longest)

    clock = ClockSampler()
    main_run = time_decode(engine, cfg, args.batch, steps, warmup, repeats=repeats, context=context, clock=clock)
    dev_ms = main_run["dev_ms"]
    value = args.batch * 1000.0 / dev_ms
    step_bytes = weight_bytes(cfg, args.batch) + args.batch * main_run["ctx"] * kv_bytes_per_token(cfg)
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    repeat_clocks = [clock.summary(b, e)["sm_mhz"] for b, e in main_run["repeat_spans"]]

    prefill = None
    points = {}
    if not args.no_prefill:
        pclock = ClockSampler()
        with pclock:
            prefill_ms = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=3, reps=9)
        pf = prefill_flops(cfg, PREFILL_TOKENS) / (prefill_ms * 1e-3) / 1e12
        pc = pclock.summary()
        prefill = {"value": round(PREFILL_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                   "ms": round(prefill_ms, 3), "frac": round(pf / pk["bf16_tflops"], 4), "frac_of": "burst peak",
                   "frac_sustained": round(pf / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]), 4),
                   "sm_mhz": pc["sm_mhz"], "reasons": pc["reasons"]}
        if not args.no_points:
            ms4 = time_prefill(engine, cfg, PREFILL_TOKENS, warmup=2, reps=3, portion=512)
            points["prefill_4x512"] = round(PREFILL_TOKENS * 1000.0 / ms4, 1)
    if not args.no_points:
        k = min(steps, 20)
        for b in (1, 64):
            r = time_decode(engine, cfg, b, k, 5, repeats=5, e2e=False)
            points[f"decode_b{b}"] = round(b * 1000.0 / r["dev_ms"], 1)
        window = [value]
        for ctx in (2048, 3072):
            r = time_decode(engine, cfg, args.batch, k, 5, repeats=4, context=ctx, e2e=False)
            window.append(args.batch * 1000.0 / r["dev_ms"])
            if ctx == 2048:
                points[f"decode_b{args.batch}_ctx2048"] = round(window[-1], 1)
        points[f"decode_b{args.batch}_avg_ctx2048_4096"] = round((window[1] + 2 * window[2] + window[0]) / 4, 1)

    checked = None
    if not args.no_check:
        checked = {"b%d" % args.batch: check_logits(engine, cfg, args.batch, context, rows=[0, args.batch - 1])}
        if not args.no_points:
            checked["b64"] = check_logits(engine, cfg, 64, context, rows=[0, 37])

    baselines = None
    if not args.no_extras:
        from baseline.torch_plain import time_torch_plain
        dec_ms, pre_ms = time_torch_plain(engine.model, cfg.vocab_size, args.batch, context, PREFILL_TOKENS)
        baselines = {"torch_plain": {"what": "the same weights in plain PyTorch (matmul + scaled_dot_product_attention, "
                                             "contiguous cache, eager)", "decode_tok_s": round(args.batch * 1000.0 / dec_ms, 1),
                                     "decode_ms_per_step": round(dec_ms, 3), "prefill_tok_s": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1),
                                     "prefill_ms": round(pre_ms, 3)}}

    if not args.no_extras and args.shape == "7b" and not args.layers:
        # the 1.5B shape (64 requests, chunks of 512 mixed with decode) on the same GPU
        del engine
        torch.cuda.empty_cache()
        small = qwen7b_config("1.5b")
        eng = _engine(small, page, 64, context + 4 * (5 + 2 * 20) + 80, chunk=512)
        r = time_decode(eng, small, 8, 20, 5, repeats=4, e2e=False)
        b15 = weight_bytes(small, 8) + 8 * r["ctx"] * kv_bytes_per_token(small)
        points["decode_b8_1p5b"] = round(8 * 1000.0 / r["dev_ms"], 1)
        points["decode_b8_1p5b_hbm_frac"] = round(b15 / (r["dev_ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        serve_workload(eng, small, 8, 16, prompt_len=1024)
        runs = sorted(serve_workload(eng, small, 64, 256) for _ in range(3))      # the median of three: a shared host
        dt, pt, gt, _s, _p = runs[1]                                                # now and then stalls a run
        points["serve_1p5b"] = round((pt + gt) / dt, 1)
        points["serve_1p5b_generated"] = round(gt / dt, 1)

    line = {
        "metric": "decode tok/s at batch 8, Qwen2.5-7B bf16 (also batch 1/64 and prefill tok/s at 2,048 tokens)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "rope_theta": cfg.rope_theta, "rms_norm_eps": cfg.rms_norm_eps, "global_batch": args.batch,
                   "seq_len": context, "context_at_timing": main_run["ctx"], "kv_page": page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (GBs of weights per step), no flush",
                   "peaks": pk["source"]},
        "repeats": repeats, "repeat_ms": [round(m, 4) for m in main_run["repeat_ms"]], "repeat_sm_mhz": repeat_clocks,
        "clocks": clock.summary(),
        "e2e": {"value": round(args.batch * 1000.0 / main_run["e2e_ms"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": int(main_run["h2d"]), "d2h_bytes_per_step": int(main_run["d2h"]),
                "ms_per_step": round(main_run["e2e_ms"], 4)},
        "gpu_launches": int(round(main_run["launches"] * steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "checked": checked,
        "baselines": baselines,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
