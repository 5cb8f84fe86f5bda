"""Trace replay: feed given token ids through the model step by step and write
logits.  It samples nothing and has no forward pass, cache or loader of its own:
it drives ``load_model``, ``CacheManager`` and ``ModelRunner.step``, the ones
generation uses.

Steps come one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at
the wanted places, in the order of the entries and of ``want``, as little-endian
float32 ``[wanted, vocab]``.  After every step a line ``done <step>`` is printed
and flushed.  The reference's nearest tool is its golden dump
(reference/dump_ref.py:535-715), which runs whole prompts only.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..csrc import ops
from .loading import load_model, parse_dtype
from .step import ModelRunner, StepEntry

REPLAY_PAGE_SIZE = 16
MAX_LIVE = 8


def make_runner(model_dir: str, dtype, max_tokens: int, page_size: int = REPLAY_PAGE_SIZE,
                max_seqs: int = MAX_LIVE) -> ModelRunner:
    model, _ = load_model(model_dir, dtype)
    # each live request's count is rounded up to a multiple of 64 by the caller, so
    # whole pages of 16 always suffice for max_tokens
    cache = CacheManager(model.cache_layout, page_size=page_size, max_tokens=max_tokens, max_seqs=max_seqs,
                         dtype=parse_dtype(dtype), device=str(model.rt.device))
    return ModelRunner(model, cache, model.rt, cuda_graphs=True)


def replay(runner: ModelRunner, lines: IO[str], out_dir: str, done: IO[str] = sys.stdout) -> None:
    os.makedirs(out_dir, exist_ok=True)
    live: Dict[str, object] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in live:
                live[rid] = runner.cache.open_sequence()
            entries.append(StepEntry(live[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = runner.step(entries)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            ops.check_kernel_status()       # the copy has waited for the step: a kernel that gave up shows now
            arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            seq = live.pop(str(rid), None)
            if seq is not None:
                runner.cache.close(seq)
        done.write(f"done {step}\n")
        done.flush()
    ops.check_kernel_status()


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay a trace of steps and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    args = ap.parse_args(argv)
    runner = make_runner(args.model, args.dtype, args.max_tokens)
    replay(runner, sys.stdin, args.out)
    return 0
