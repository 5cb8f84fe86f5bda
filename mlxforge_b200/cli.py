"""Command line, in the manner of the reference's ``mlxforge-cli``
(apps/mlxforge_cli.cpp:9-38,521-656):

    generate <model> <ids.npy | "1,2,3"> [max_tokens=64] [--temperature T] [--seed S] ...
        token ids in (a .npy of int ids, as the reference accepts, or a comma
        list), generated ids streamed to stdout; statistics to stderr
    bench <model> [max_tokens=128] [runs=3]
        one discarded warm-up, EOS disabled, time to first token and decode tok/s
    dump-weights <dir>
        ``key [shape] dtype`` for every tensor of the checkpoint
    random-weights <config.json> <out_dir> [--seed S] [--dtype bfloat16|float32]
        write a model folder with random weights (not in the reference)
    replay ...
        the same program as bin/trace_run

Tokenizers are out of scope: prompts are token ids.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np


def _read_ids(arg: str):
    if arg.endswith(".npy"):
        return [int(t) for t in np.load(arg).reshape(-1)]
    return [int(t) for t in arg.replace(" ", "").split(",") if t]


def _engine(args, **over):
    from .engine.engine import Engine, EngineConfig
    cfg = EngineConfig(model_spec=args.model, dtype=args.dtype, kv_block_size=args.kv_block_size,
                       prefill_chunk=args.prefill_chunk, skinny_mm=not args.no_skinny_mm,
                       rope_scaling=args.rope_scaling or "", cuda_graphs=not args.no_cuda_graphs,
                       pipeline=not args.no_pipeline, gemm=args.gemm, **over)
    return Engine(cfg)


def _common(ap):
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--kv-block-size", type=int, default=16)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--no-skinny-mm", action="store_true", help="few-row products by the library instead")
    ap.add_argument("--rope-scaling", default="", help="JSON object replacing the checkpoint's rope_scaling")
    ap.add_argument("--no-cuda-graphs", action="store_true", help="launch every kernel of a decode step one by one")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="collect a step's tokens before the next step is launched")
    ap.add_argument("--gemm", default="", choices=["", "auto", "library", "tcgen05"],
                    help="many-row products: own tcgen05 kernel for gate|up (auto), the library, or the own kernel for all")


def run_generate(args) -> int:
    from .sampling.params import SamplingParams
    prompt = _read_ids(args.prompt)
    eng = _engine(args, kv_pool_tokens=max(4096, len(prompt) + args.max_tokens + 64))
    params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                            repetition_penalty=args.repetition_penalty,
                            frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty,
                            seed=args.seed)
    t0 = time.perf_counter()
    req = eng.submit_ids(prompt, params, args.max_tokens)
    first = None
    n = 0
    while not req.finished:
        eng.step()
        while n < len(req.output_ids):
            if first is None:
                first = time.perf_counter()
            sys.stdout.write(("" if n == 0 else " ") + str(req.output_ids[n]))
            sys.stdout.flush()
            n += 1
    sys.stdout.write("\n")
    t1 = time.perf_counter()
    if req.finish_reason == "error":
        print(f"error: {req.error}", file=sys.stderr)
        return 1
    ttft = (first - t0) * 1e3 if first else float("nan")
    dec = n - 1
    tps = dec / (t1 - first) if first and dec > 0 and t1 > first else 0.0
    print(f"generated {n} tokens ({req.finish_reason})", file=sys.stderr)
    print(f"time to first token {ttft:.1f}ms; decode {tps:.1f} tok/s ({dec} tokens in {(t1 - (first or t1)) * 1e3:.1f}ms)",
          file=sys.stderr)
    return 0


def run_bench(args) -> int:
    from .sampling.params import GREEDY
    eng = _engine(args, kv_pool_tokens=max(4096, args.prompt_tokens + args.max_tokens + 64))
    vocab = eng.model.spec.vocab_size
    prompt = np.random.default_rng(0).integers(0, vocab, size=args.prompt_tokens).tolist()

    def one():
        t0 = time.perf_counter()
        req = eng.submit_ids(prompt, GREEDY, args.max_tokens, eos_ids=[])
        first = None
        while not req.finished:
            eng.step()
            if first is None and req.output_ids:
                first = time.perf_counter()
        t1 = time.perf_counter()
        dec = len(req.output_ids) - 1
        return (first - t0) * 1e3, dec / (t1 - first) if dec > 0 else 0.0, dec

    print(f"bench: prompt={len(prompt)} tokens, max_tokens={args.max_tokens}, warmup=1, runs={args.runs}")
    one()
    ttfts, tpss = [], []
    for i in range(args.runs):
        ttft, tps, dec = one()
        ttfts.append(ttft)
        tpss.append(tps)
        print(f"  run {i + 1}/{args.runs}:  ttft {ttft:.1f} ms   decode {tps:.1f} tok/s  ({dec} tokens)", flush=True)
    print(f"\nttft     mean {np.mean(ttfts):.1f} ms   (min {min(ttfts):.1f}, max {max(ttfts):.1f})")
    print(f"decode   mean {np.mean(tpss):.1f} tok/s   (min {min(tpss):.1f}, max {max(tpss):.1f})")
    return 0


def run_dump_weights(args) -> int:
    from .weights.safetensors_io import SafetensorsFile, model_files
    total = 0
    for path in model_files(args.dir):
        f = SafetensorsFile(path)
        for e in sorted(f.entries, key=lambda e: e.name):
            print(f"{e.name} {list(e.shape)} {e.dtype}")
            total += e.end - e.begin
        f.close()
    print(f"{total / 2**20:.1f} MiB of tensor data")
    return 0


def run_random_weights(args) -> int:
    from .config.registry import config_from_json
    from .weights.random_init import write_random_model
    with open(args.config) as f:
        cfg = config_from_json(json.load(f))
    write_random_model(args.out_dir, cfg, args.seed, dtype=args.dtype, std=args.std, norm_std=args.norm_std)
    print(args.out_dir)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mlxforge_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)

    g = sub.add_parser("generate", help="generate token ids from a prompt of token ids")
    g.add_argument("model")
    g.add_argument("prompt", help="ids.npy or a comma-separated list of token ids")
    g.add_argument("max_tokens", nargs="?", type=int, default=64)
    g.add_argument("--temperature", type=float, default=0.0, help="<= 0: greedy (the default, as the reference's CLI)")
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0)
    _common(g)
    g.set_defaults(fn=run_generate)

    b = sub.add_parser("bench", help="time to first token and decode tok/s")
    b.add_argument("model")
    b.add_argument("max_tokens", nargs="?", type=int, default=128)
    b.add_argument("runs", nargs="?", type=int, default=3)
    b.add_argument("--prompt-tokens", type=int, default=32)
    _common(b)
    b.set_defaults(fn=run_bench)

    d = sub.add_parser("dump-weights", help="list the tensors of a checkpoint")
    d.add_argument("dir")
    d.set_defaults(fn=run_dump_weights)

    r = sub.add_parser("random-weights", help="write a model folder with random weights")
    r.add_argument("config")
    r.add_argument("out_dir")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.set_defaults(fn=run_random_weights)

    p = sub.add_parser("replay", help="replay a trace of steps (same as bin/trace_run)", add_help=False)
    p.set_defaults(fn=None)

    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
