#!/usr/bin/env python3
"""Headline benchmark: decode tokens/s of the Llama-3.2-1B shape in bfloat16 on one
B200 (batch 8 at the stated context length), with prefill of 2,048 tokens, decode
at batch 1 and 64, the same metric end to end through the Python entry point, and
roofline fractions.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of the whole batch (model forward over the paged
cache plus on-device sampling).  Weights are random (seeded normal, std 0.02),
token ids are seeded uniform: there is no network for checkpoints or datasets.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the headline configuration: the Llama-3.2-1B shape
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}
# the other shapes that the reference's benchmark configurations name (--shape, for measurements
# beside the headline; the default run is the 1B shape)
LLAMA_3B = dict(LLAMA_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, head_dim=128,
                intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": ("Llama-3.2-1B", LLAMA_1B), "3b": ("Llama-3.2-3B", LLAMA_3B), "8b": ("Llama-3.1-8B", LLAMA_8B)}
CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}

REFERENCE_UNAVAILABLE = ("hvasconcelos/mlxforge builds only on Apple (CMakeLists.txt:14-16 errors elsewhere) and "
                         "computes through Apple MLX/Metal, which this box does not have; it has no pip package")


def peaks():
    """HBM copy bandwidth and the library's bfloat16 product throughput as a burst (the divisor for
    a region of a few milliseconds timed alone between synchronisations, as the prefill here is)
    and sustained under the power cap."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                j = json.load(f)
            hbm, burst = j.get("hbm_gbs"), j.get("bf16_tflops")
            if hbm and burst:
                return {"hbm_gbs": float(hbm), "bf16_tflops": float(burst),
                        "bf16_tflops_sustained": float(j.get("bf16_tflops_sustained") or burst), "source": "measured"}
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi sampling SM clocks and throttle reasons while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        self.f = open(self.path, "w")
        self.proc = subprocess.Popen([exe, "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    c = [x.strip() for x in line.split(",")]
                    if len(c) < 7:
                        continue
                    try:
                        sm.append(float(c[0]))
                        mx.append(float(c[1]))
                    except ValueError:
                        continue
                    for n, v in zip(names, c[3:7]):
                        if v.lower().startswith("active"):
                            reasons.add(n)
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}
        return out


def decode_device(engine, batch, ctx, steps, warmup, seed=0, segments=5):
    """Device-timed decode: `batch` sequences whose cache holds ~ctx tokens (filled
    with random keys and values, no forward pass needed for that), `warmup` + `steps`
    decode steps of the step function with greedy sampling on the device.  The `steps`
    timed steps are one region between two events; events in between cut it into
    `segments` pieces whose ms per step show the spread.  Returns (seconds per step,
    kernel launches per step, cache tokens read per step, [ms per step of every piece])."""
    import numpy as np
    import torch
    from mlxforge_b200.csrc import binding, ops
    from mlxforge_b200.engine.step import StepEntry
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(seed)
    vocab = engine.model.spec.vocab_size
    start_len = ctx - (warmup + steps)
    seqs = [cache.open_sequence() for _ in range(batch)]
    for s in seqs:
        cache.reserve([(s, start_len)])
        cache.commit(s, start_len)
    out = torch.empty(batch, dtype=torch.int32, device="cuda")
    toks = rng.integers(0, vocab, size=(warmup + steps, batch))

    def one(i):
        logits = runner.step([StepEntry(s, [int(toks[i, b])], [0]) for b, s in enumerate(seqs)])
        ops.sample(logits, None, None, out)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    l0 = binding.launch_count()
    segments = max(1, min(segments, steps))
    cuts = [round(k * steps / segments) for k in range(segments + 1)]
    events = [torch.cuda.Event(enable_timing=True) for _ in cuts]
    events[0].record()
    for k in range(segments):
        for i in range(warmup + cuts[k], warmup + cuts[k + 1]):
            one(i)
        events[k + 1].record()
    torch.cuda.synchronize()
    ops.check_kernel_status()
    sec = events[0].elapsed_time(events[-1]) / 1e3 / steps
    pieces = [events[k].elapsed_time(events[k + 1]) / (cuts[k + 1] - cuts[k]) for k in range(segments)]
    launches = (binding.launch_count() - l0) / steps
    mean_ctx = start_len + warmup + (steps + 1) / 2.0
    for s in seqs:
        cache.close(s)
    return sec, launches, mean_ctx * batch, pieces


def prefill_products_device(engine, tokens, runs=5, warmup=3):
    """The matrix products of a prefill of `tokens` tokens alone (every layer's QKV, output,
    gate|up with its gated epilogue, down; the head's one row is left out), through the same
    dispatch the model uses, on scratch operands.  Returns (seconds, FLOPs)."""
    import torch
    rt = engine.model.rt
    blocks = [engine.model.blocks[item.layer] for item in engine.model.spec.schedule]
    flops = 0.0
    plan = []
    for b in blocks:
        m, f = b.mixer, b.feed_forward
        xs = {}
        for w in (m.w_qkv, m.w_o, f.w_gu, f.w_down):
            k = w.shape[1]
            if k not in xs:
                xs[k] = torch.randn((tokens, k), device=rt.device).to(torch.bfloat16)
            flops += 2.0 * tokens * w.shape[0] * k
        plan.append((m, f, xs))
    outs = {}

    def out(name, shape):
        if name not in outs:
            outs[name] = torch.empty(shape, dtype=torch.bfloat16, device=rt.device)
        return outs[name]

    def once():
        for m, f, xs in plan:
            rt.linear(xs[m.w_qkv.shape[1]], m.w_qkv, out("qkv", (tokens, m.w_qkv.shape[0])))
            rt.linear(xs[m.w_o.shape[1]], m.w_o, out("o", (tokens, m.w_o.shape[0])))
            rt.linear_swiglu(xs[f.w_gu.shape[1]], f.w_gu, f.group, out("act", (tokens, f.inter)))
            rt.linear(xs[f.w_down.shape[1]], f.w_down, out("down", (tokens, f.w_down.shape[0])))

    times = []
    for i in range(warmup + runs):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        once()
        e1.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(e0.elapsed_time(e1) / 1e3)
    return statistics.median(times), flops


def prefill_device(engine, tokens, runs=5, warmup=3):
    import numpy as np
    import torch
    from mlxforge_b200.engine.step import StepEntry
    runner, cache = engine.runner, engine.cache
    rng = np.random.default_rng(1)
    ids = rng.integers(0, engine.model.spec.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + runs):
        s = cache.open_sequence()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry(s, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.close(s)
        if i >= warmup:
            times.append(e0.elapsed_time(e1) / 1e3)
    return statistics.median(times)


def decode_e2e(engine, batch, ctx, steps, warmup):
    """The same metric through the Python entry point: requests with host token ids
    in, generated ids out; every step copies its inputs from pinned host memory and
    reads the sampled ids back."""
    import numpy as np
    import torch
    import mlxforge_b200 as mf
    rng = np.random.default_rng(2)
    vocab = engine.model.spec.vocab_size
    # requests finish their prompts in different steps: every one gets room to decode through
    # the whole timed region, and is cancelled after it
    plen = ctx - (warmup + steps) - 1 - 2 * batch
    reqs = [engine.submit_ids(rng.integers(0, vocab, size=plen).tolist(), mf.GREEDY,
                              warmup + steps + 4 * batch + 64, eos_ids=[]) for _ in range(batch)]
    while any(len(r.output_ids) < 1 for r in reqs):          # prefill and first token, untimed
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    n0 = sum(len(r.output_ids) for r in reqs)
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    n1 = sum(len(r.output_ids) for r in reqs)
    h2d = engine.runner.last_meta_bytes
    assert all(not r.finished for r in reqs), "a request ended inside the timed region"
    for r in reqs:
        r.cancel()
    engine.run_until_idle()
    return (n1 - n0) / (t1 - t0), h2d, batch * 4 + 4      # the sampled ids and the kernels' status word


def serving_workload(engine, n_requests, lo, hi, out_tokens, seed=4):
    """The continuous-batching run of the reference's benchmark (bench/config.py:34-47 gives the
    load shapes; apps/mlxforge_cli.cpp:311-349 the protocol): `n_requests` requests with
    uniform-random prompt lengths in [lo, hi] submitted at once, `out_tokens` generated tokens
    each (EOS off), prompts run in portions beside decoding.  Host token ids in, ids out."""
    import numpy as np
    import torch
    import mlxforge_b200 as mf
    rng = np.random.default_rng(seed)
    vocab = engine.model.spec.vocab_size
    lens = rng.integers(lo, hi + 1, size=n_requests)
    prompts = [rng.integers(0, vocab, size=int(n)).tolist() for n in lens]
    torch.cuda.synchronize()
    steps_before = int(engine.metrics()["steps"])
    t0 = time.perf_counter()
    reqs = [engine.submit_ids(p, mf.GREEDY, out_tokens, eos_ids=[]) for p in prompts]
    first = [None] * n_requests
    while not engine.idle:
        engine.step()
        now = time.perf_counter()
        for i, r in enumerate(reqs):
            if first[i] is None and len(r.output_ids) > 0:
                first[i] = now
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    assert all(r.finish_reason == "length" for r in reqs), [r.finish_reason for r in reqs]
    ttft = sorted((f - t0) * 1e3 for f in first)
    gen = sum(len(r.output_ids) for r in reqs)
    m = engine.metrics()
    return {"seconds": round(t1 - t0, 3), "prompt_tokens": int(lens.sum()), "generated_tokens": gen,
            "tokens_per_s": round((int(lens.sum()) + gen) / (t1 - t0), 1), "generated_per_s": round(gen / (t1 - t0), 1),
            "ttft_ms_p50": round(ttft[len(ttft) // 2], 1), "ttft_ms_p99": round(ttft[min(len(ttft) - 1, int(0.99 * len(ttft)))], 1),
            "steps": int(m["steps"]) - steps_before, "preemptions": int(m["preemptions"]), "peak_running": int(m["peak_running"])}


def run_workload(args) -> int:
    """`--workload serving`: the Llama-3.2-3B shape, 64 requests with prompts of 128 to 4096
    tokens and 256 generated tokens each, portions of 512 beside decoding.  `--workload longctx`:
    the Llama-3.1-8B shape, 8 requests of 16,384 prompt tokens and 512 generated tokens each.
    Both print one JSON line; the first run on an engine also captures its CUDA graphs and
    sizes its buffers, so the load runs twice and both runs are reported."""
    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json
    from mlxforge_b200.csrc import ops
    serving = args.workload == "serving"
    shape_key = args.shape if args.shape_given else ("3b" if serving else "8b")
    shape_name, shape = SHAPES[shape_key]
    layers = args.layers or shape["num_hidden_layers"]
    cfg_json = dict(shape, num_hidden_layers=layers)
    if serving:
        n, lo, hi, out, chunk, running = 64, 128, 4096, 256, 512, 64
    else:
        n, lo, hi, out, chunk, running = 8, 16384, 16384, 512, 2048, 8
    tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
    try:
        model_dir = mf.write_random_model(os.path.join(tmp, "model"), config_from_json(cfg_json), seed=0, dtype="bfloat16")
        engine = mf.Engine(model_spec=model_dir, dtype="bfloat16", kv_pool_tokens=n * (hi + out + 64), max_running=running,
                           token_budget=max(2048, chunk + running), prefill_chunk=chunk)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    clocks = ClockSampler()
    clocks.start()
    runs = [serving_workload(engine, n, lo, hi, out) for _ in range(2)]
    clk = clocks.stop()
    ops.check_kernel_status()
    print(json.dumps({
        "workload": args.workload, "model": f"{shape_name} shape", "layers": layers,
        "layers_of_named_config": shape["num_hidden_layers"], "requests": n, "prompt_tokens": [lo, hi],
        "generated_tokens_each": out, "prefill_chunk": chunk, "max_running": running, "dtype": "bf16",
        "data": "synthetic: seeded normal(0, 0.02) weights, seeded uniform token ids", "first_run": runs[0],
        "second_run": runs[1], "clocks": clk}))
    return 0


# Kinds of launches that `--without` leaves out of a decode step, to see what each costs inside it.
LEFT_OUT = ("norms", "rotation", "attention", "qkv", "o", "gate_up", "down", "head", "products")


def leave_out(kind: str, shape: dict) -> None:
    """Replace the launcher of one kind of kernel by nothing (the step's numbers are then wrong and
    only its time means something)."""
    from mlxforge_b200.csrc import ops
    hidden, inter = shape["hidden_size"], shape["intermediate_size"]
    qkv_rows = (shape["num_attention_heads"] + 2 * shape["num_key_value_heads"]) * shape["head_dim"]
    stream = ops.stream_linear

    def nothing(*a, **k):
        return None

    def products(pred):
        def f(x, w, out, swiglu=False):
            return None if pred(w, swiglu) else stream(x, w, out, swiglu=swiglu)
        return f

    if kind == "norms":
        ops.add_rmsnorm = nothing
    elif kind == "rotation":
        ops.rope_kv_write = nothing
    elif kind == "attention":
        ops.attention_decode = nothing
    elif kind == "products":
        ops.stream_linear = nothing
    else:
        pred = {"qkv": lambda w, s: not s and tuple(w.shape) == (qkv_rows, hidden),
                "o": lambda w, s: not s and tuple(w.shape) == (hidden, shape["num_attention_heads"] * shape["head_dim"])
                and tuple(w.shape) != (qkv_rows, hidden),
                "gate_up": lambda w, s: s,
                "down": lambda w, s: not s and tuple(w.shape) == (hidden, inter),
                "head": lambda w, s: w.shape[0] == shape["vocab_size"]}[kind]
        ops.stream_linear = products(pred)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default=None, choices=sorted(SHAPES), help="layer sizes (default: the 1B shape)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has (0: all)")
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="decode / prefill: run just that part and print a short line (for profiling small cases)")
    ap.add_argument("--without", default=None, choices=sorted(LEFT_OUT),
                    help="with --only decode: time the step with the launches of one kind left out (its results are "
                         "wrong; the difference to the full step is what that kind costs inside the step)")
    ap.add_argument("--workload", default="headline", choices=["headline", "serving", "longctx"],
                    help="serving: 64 requests on the 3B shape; longctx: 8 x 16,384 tokens on the 8B shape")
    args = ap.parse_args()
    args.shape_given = args.shape is not None
    args.shape = args.shape or "1b"

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"unavailable": f"this engine runs on one GPU; --gpus {args.gpus} is not supported"}))
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload != "headline":
        return run_workload(args)

    import torch
    import mlxforge_b200 as mf
    from mlxforge_b200.config import config_from_json

    shape_name, shape = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]
    cfg_json = dict(shape, num_hidden_layers=args.layers)
    tmp = tempfile.mkdtemp(prefix="mlxforge_bench_")
    try:
        t0 = time.time()
        model_dir = mf.write_random_model(os.path.join(tmp, f"llama_{args.shape}_random"), config_from_json(cfg_json), seed=0,
                                          dtype="bfloat16")
        ctx = args.context
        pool_seqs = 64 if args.only == "all" and not args.skip_points else max(args.batch, 1)
        engine = mf.Engine(model_spec=model_dir, dtype="bfloat16", kv_pool_tokens=pool_seqs * (ctx + 64),
                           max_running=64, token_budget=8192, prefill_chunk=2048)
        print(f"[bench] model written and loaded in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    # the synthetic cache: random keys and values everywhere (reading zeros is as slow, but keep it honest)
    for pool in engine.cache._k + engine.cache._v:
        pool.normal_(0.0, 1.0)

    pk = peaks()
    weight_bytes = engine.model.weight_bytes()
    kv_per_token = engine.model.cache_layout.bytes_per_token(2)

    if args.only == "prefill":
        t_pre = prefill_device(engine, PREFILL_TOKENS, runs=max(1, args.steps), warmup=args.warmup)
        print(json.dumps({"only": "prefill", "shape": args.shape, "tokens": PREFILL_TOKENS, "ms": round(t_pre * 1e3, 3),
                          "layers": args.layers}))
        return 0
    BATCH_ = args.batch
    if args.without:
        if args.only != "decode":
            print("--without goes with --only decode", file=sys.stderr)
            return 2
        leave_out(args.without, shape)
    clocks = ClockSampler()
    clocks.start()
    sec, launches, kv_tokens, pieces = decode_device(engine, BATCH_, ctx, args.steps, args.warmup)
    clk = clocks.stop()
    value = BATCH_ / sec
    bytes_step = weight_bytes + kv_tokens * kv_per_token
    achieved = bytes_step / sec / 1e9
    if args.only == "decode":
        line = {"only": "decode", "shape": args.shape, "batch": BATCH_, "context": ctx, "layers": args.layers,
                "ms_per_step": round(sec * 1e3, 4), "launches_per_step": launches, "gbs": round(achieved, 1)}
        if args.without:
            line = dict(line, without=args.without, gbs=None, note="a kind of kernel was left out: a timing, not a result")
        print(json.dumps(line))
        return 0

    # the other batch sizes the metric names, at the headline context and at the 1024 tokens its
    # decode line names; each with the fraction of the HBM peak that its bytes over its time are
    points, point_fracs = {}, {}
    if not args.skip_points:
        for b, c in ((1, ctx), (64, ctx), (1, 1024), (8, 1024), (64, 1024)):
            s_b, _, kv_b, _ = decode_device(engine, b, c, max(8, args.steps // 2), args.warmup, seed=b)
            name = f"decode_b{b}" if c == ctx else f"decode_b{b}_ctx{c}"
            points[name] = round(b / s_b, 1)
            point_fracs[name] = round((weight_bytes + kv_b * kv_per_token) / s_b / 1e9 / pk["hbm_gbs"], 4)

    t_pre = prefill_device(engine, PREFILL_TOKENS)
    t_gemm, gemm_flops = prefill_products_device(engine, PREFILL_TOKENS)
    c = cfg_json
    L, H, I, V = c["num_hidden_layers"], c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nh, nkv, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    mat = L * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I)
    T = PREFILL_TOKENS
    flops = 2.0 * T * mat + 2.0 * V * H + L * 2.0 * T * T * hd * nh     # products + one head row + causal attention
    # the whole prefill is timed alone between synchronisations: the burst peak is its divisor
    prefill = {"value": round(T / t_pre, 1), "tokens": T, "ms": round(t_pre * 1e3, 3),
               "frac": round(flops / t_pre / (pk["bf16_tflops"] * 1e12), 4),
               "frac_of_sustained": round(flops / t_pre / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "products_ms": round(t_gemm * 1e3, 3),
               "products_frac": round(gemm_flops / t_gemm / (pk["bf16_tflops"] * 1e12), 4)}

    e2e_value, h2d, d2h = decode_e2e(engine, BATCH_, ctx, args.steps, args.warmup)
    # what the Python host costs at the other batch sizes, and what launching a step before the tokens of
    # the one before are on the host is worth: the same metric through the entry point
    e2e_points = {}
    if not args.skip_points:
        half = max(8, args.steps // 2)
        e2e_points["decode_b1"] = round(decode_e2e(engine, 1, ctx, half, args.warmup)[0], 1)
        e2e_points["decode_b64_ctx1024"] = round(decode_e2e(engine, 64, 1024, half, args.warmup)[0], 1)
        engine.pipeline = False
        try:
            e2e_points["decode_b8_unpipelined"] = round(decode_e2e(engine, BATCH_, ctx, half, args.warmup)[0], 1)
            e2e_points["decode_b1_unpipelined"] = round(decode_e2e(engine, 1, ctx, half, args.warmup)[0], 1)
        finally:
            engine.pipeline = True

    line = {
        "metric": f"decode tok/s @ batch {BATCH_} ({shape_name} bf16)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded normal(0, 0.02) weights, seeded uniform token ids, random cache contents",
        "config": {
            "model": f"{shape_name} shape (LlamaForCausalLM)", "layers": L,
            "layers_of_named_config": shape["num_hidden_layers"],
            "hidden": H, "heads": nh, "kv_heads": nkv, "head_dim": hd, "intermediate": I, "vocab": V,
            "global_batch": BATCH_, "seq_len": ctx, "context_len": ctx, "kv_block": engine.cache.page_size,
            "prefill_tokens": T, "parallelism": "single GPU",
            "l2": "working set per step (weights + live cache) exceeds L2 many times; no flush needed",
            "peaks": pk["source"],
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(round(launches * args.steps)),
        "clocks": clk,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "point_fracs": point_fracs,
        "e2e_points": e2e_points,
        "ms_per_step_pieces": {"median": round(statistics.median(pieces), 4), "min": round(min(pieces), 4),
                               "max": round(max(pieces), 4), "pieces": len(pieces)},
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
