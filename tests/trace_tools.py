"""Builds traces (lists of step records in trace_run's format) for given requests
and compares what a replay wrote with the plain implementation's whole-sequence
logits."""
from __future__ import annotations

import io
import json
import os

import numpy as np


class Trace:
    def __init__(self):
        self.steps = []          # records as trace_run reads them
        self.wanted = []         # per step: list of (request id, position in the request)

    def add(self, entries, end=()):
        """entries: list of (id, start position, tokens, want indices)."""
        rec = {"step": len(self.steps), "entries": [], "end": list(end)}
        wanted = []
        for rid, start, tokens, want in entries:
            rec["entries"].append({"id": rid, "tokens": list(map(int, tokens)), "want": list(map(int, want))})
            wanted += [(rid, start + w) for w in want]
        self.steps.append(rec)
        self.wanted.append(wanted)

    def lines(self):
        return io.StringIO("".join(json.dumps(s) + "\n" for s in self.steps))

    def live_tokens_rounded(self, to=64):
        """Most tokens live requests hold at any time, each rounded up to a multiple of ``to``."""
        held, peak = {}, 0
        for rec in self.steps:
            for e in rec["entries"]:
                held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
            peak = max(peak, sum((n + to - 1) // to * to for n in held.values()))
            for rid in rec["end"]:
                held.pop(rid, None)
        return peak


def whole(requests):
    t = Trace()
    for rid, toks in requests.items():
        t.add([(rid, 0, toks, range(len(toks)))], end=[rid])
    return t


def decode_tail(requests, tail=32):
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    t = Trace()
    for rid, toks in requests.items():
        n = len(toks)
        head = max(1, n - tail)
        t.add([(rid, 0, toks[:head], [head - 1])])
        for p in range(head, n):
            t.add([(rid, p, toks[p:p + 1], [0])], end=[rid] if p == n - 1 else [])
        if head == n:
            t.steps[-1]["end"] = [rid]
    return t


def lockstep(requests):
    """Every request from its first token on, one token a step, all live requests in every
    step: the first tokens of a sequence, long decoding, a batch that shrinks as requests end."""
    t = Trace()
    longest = max(len(toks) for toks in requests.values())
    for p in range(longest):
        entries = [(rid, p, toks[p:p + 1], [0]) for rid, toks in requests.items() if p < len(toks)]
        t.add(entries, end=[rid for rid, toks in requests.items() if p == len(toks) - 1])
    return t


def portions(requests, sizes=(7, 2, 5, 3, 2, 11, 4, 2, 16, 1, 9)):
    """Every request alone, in portions of changing size, down to two tokens."""
    t = Trace()
    for k, (rid, toks) in enumerate(requests.items()):
        p, i = 0, k
        while p < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - p)
            t.add([(rid, p, toks[p:p + n], range(n))], end=[rid] if p + n == len(toks) else [])
            p += n
            i += 1
    return t


def total_tokens(requests):
    return sum(len(t) for t in requests.values())


def mixed(requests, max_live=4, seed=0, decode_last=8, want_all=True, max_portion=9):
    """Up to ``max_live`` live requests: portions of some (2 to ``max_portion`` tokens) beside
    single decoded tokens of others in the same step, a request now and then left out of a
    step, new ones admitted as others end."""
    rng = np.random.default_rng(seed)
    t = Trace()
    waiting = list(requests.items())
    live = {}      # id -> [tokens, position]
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, end = [], []
        for rid in list(live):
            toks, p = live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue                                   # sits this step out
            left = len(toks) - p
            n = 1 if left <= decode_last else int(min(left - decode_last, rng.integers(2, max_portion + 1)))
            want = range(n) if want_all else ([n - 1] if p + n >= len(toks) - decode_last else [])
            entries.append((rid, p, toks[p:p + n], want))
            live[rid][1] = p + n
            if p + n == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            t.add(entries, end)
    return t


def read_outputs(trace, out_dir, vocab):
    """{(request id, position): logits row} from the files a replay wrote."""
    got = {}
    for rec, wanted in zip(trace.steps, trace.wanted):
        path = os.path.join(out_dir, f"{rec['step']}.f32")
        if not wanted:
            assert not os.path.exists(path), f"step {rec['step']} wanted nothing but wrote a file"
            continue
        a = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
        for row, key in zip(a, wanted):
            assert key not in got, key
            got[key] = row
    return got


def worst(got, expected):
    """(max abs diff, (request, position) where it is, scale of the logits there)."""
    worst_d, where = 0.0, None
    for (rid, pos), row in got.items():
        d = float(np.max(np.abs(row.astype(np.float64) - expected[rid][pos])))
        if not np.isfinite(d):
            return float("inf"), (rid, pos)
        if d > worst_d:
            worst_d, where = d, (rid, pos)
    return worst_d, where


def first_bad(got, expected, tol):
    """The earliest (request, position) beyond the tolerance: where to start looking."""
    bad = [(rid, pos) for (rid, pos), row in got.items()
           if not np.max(np.abs(row.astype(np.float64) - expected[rid][pos])) <= tol]
    return min(bad, key=lambda k: (k[1], k[0])) if bad else None
