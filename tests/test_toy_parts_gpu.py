"""Generality of the parts: a toy architecture defined HERE — a mixer with
fixed-size state of its own, a feed-forward with routing, a position encoding with
tensors of its own, layers with different mixers, a windowed attention layer
without position encoding, a schedule that
runs one layer twice and lets one run read another run's cache — is registered,
built from a model folder and stepped through the engine's own loader, cache
manager and step function, with no change to the framework's files.  Its logits,
in portions and token by token, are compared with a plain NumPy forward of the
same toy model written below."""
import json
import os

import numpy as np
import pytest

import plain_llama as P
from helpers import bf16_round, write_model_dir

pytestmark = pytest.mark.gpu

H, V, D_STATE, N_EXPERTS, INTER = 48, 97, 24, 3, 40
NH, NKV, HD, WINDOW = 3, 1, 16, 21
N_POS = 29
DECAY = 0.8
EPS = 1e-5


# ----------------------------------------------------------------------------- the toy parts (torch ops: tests may)

def _register():
    import torch
    from mlxforge_b200.config.model_config import ModelConfig
    from mlxforge_b200.config.registry import register_architecture
    from mlxforge_b200.parts.base import (Block, FeedForward, FixedState, LayerSpec, Mixer, ModelSpec, PartSpec,
                                          PositionEncoding, ScheduleItem, TensorSpec, register_block,
                                          register_feed_forward, register_mixer, register_position)

    class DecayStateMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t W_in^T ;  out_t = s_t W_out^T.  The state s lives in
        the request's slot, so a sequence must be fed in order, each token once."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.h, self.d, self.decay = params["hidden_size"], params["state_size"], params["decay"]
            self.state_dtype = params.get("state_dtype", "float32")

        def tensor_specs(self):
            return {self.prefix + "in.weight": TensorSpec((self.d, self.h)),
                    self.prefix + "out.weight": TensorSpec((self.h, self.d))}

        def bind(self, tensors):
            self.w_in = tensors[self.prefix + "in.weight"].float()
            self.w_out = tensors[self.prefix + "out.weight"].float()

        def cache_need(self):
            return FixedState((self.d,), tag="decay", dtype=self.state_dtype)

        def forward(self, x, batch, cache, writes_cache=True):
            sd = cache.tensor.dtype                      # the state's own precision, as this mixer asked for it
            u = (x.float() @ self.w_in.t()).to(sd)
            w_out = self.w_out.to(sd)
            out = torch.empty((x.shape[0], self.h), dtype=torch.float32, device=x.device)
            for start, n, slot in zip(batch.q_start, batch.q_len, batch.slot_ids):
                s = cache.tensor[slot].clone()
                for t in range(start, start + n):
                    s = self.decay * s + u[t]
                    out[t] = (s @ w_out.t()).float()
                cache.tensor[slot] = s
            return out.to(x.dtype)

    class Top1Experts(FeedForward):
        """Router logits in 32-bit, the best expert's ReLU MLP, weighted by its softmax probability."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.h, self.i, self.e = params["hidden_size"], params["intermediate_size"], params["n_experts"]

        def tensor_specs(self):
            specs = {self.prefix + "router.weight": TensorSpec((self.e, self.h))}
            for k in range(self.e):
                specs[f"{self.prefix}experts.{k}.up.weight"] = TensorSpec((self.i, self.h))
                specs[f"{self.prefix}experts.{k}.down.weight"] = TensorSpec((self.h, self.i))
            return specs

        def bind(self, tensors):
            self.router = tensors[self.prefix + "router.weight"].float()
            self.up = [tensors[f"{self.prefix}experts.{k}.up.weight"].float() for k in range(self.e)]
            self.down = [tensors[f"{self.prefix}experts.{k}.down.weight"].float() for k in range(self.e)]

        def forward(self, x, batch):
            xf = x.float()
            probs = torch.softmax(xf @ self.router.t(), dim=-1)
            best = probs.argmax(dim=-1)
            out = torch.zeros_like(xf)
            for k in range(self.e):
                rows = (best == k).nonzero().flatten()
                if rows.numel():
                    y = torch.relu(xf[rows] @ self.up[k].t()) @ self.down[k].t()
                    out[rows] = y * probs[rows, k:k + 1]
            return out.to(x.dtype)

    class LearnedPositions(PositionEncoding):
        """Learned vectors added to queries and keys: q += A[pos mod n], k += B[pos mod n], the same
        for every head.  It owns two tensors and implements ``encode`` alone: storing keys and values
        in pages is the cache lane's business."""

        def __init__(self, params, prefix, runtime):
            super().__init__(params, prefix, runtime)
            self.hd, self.n = params["head_dim"], params["n_positions"]

        def tensor_specs(self):
            return {self.prefix + "q.weight": TensorSpec((self.n, self.hd)),
                    self.prefix + "k.weight": TensorSpec((self.n, self.hd))}

        def bind(self, tensors):
            self.a = tensors[self.prefix + "q.weight"].float()
            self.b = tensors[self.prefix + "k.weight"].float()

        def encode(self, q, k, batch):
            pos = batch.positions.long()
            q += self.a[pos % self.n][:, None].to(q.dtype)
            k += self.b[pos % self.n][:, None].to(k.dtype)

    class ParallelSandwich(Block):
        """Another arrangement: the mixer and the feed-forward read the same normalised input, and
        their sum goes through a norm of its own before it joins the stream:
        ``h += out_norm( mixer(norm(h)) + feed_forward(norm(h)) )``.  One input norm, no
        feed-forward norm, and a part in a role that the usual layer does not have."""

        roles = ("mixer", "mixer_norm", "feed_forward", "out_norm")

        def forward(self, residual, pending, batch, cache, writes_cache=True):
            x = self.mixer_norm.add_forward(residual, pending)
            total = self.mixer.forward(x, batch, cache, writes_cache).float() + self.feed_forward.forward(x, batch).float()
            out = self.rt.buffer("toy.sandwich", tuple(total.shape))     # not the buffer the input norm writes
            return residual, self.by_role["out_norm"].forward(total, out=out)

    class MixerOnly(Block):
        """A layer without a feed-forward: ``h += mixer(norm(h))``."""

        roles = ("mixer", "mixer_norm")

        def forward(self, residual, pending, batch, cache, writes_cache=True):
            x = self.mixer_norm.add_forward(residual, pending)
            return residual, self.mixer.forward(x, batch, cache, writes_cache)

    register_block("toy_parallel_sandwich", ParallelSandwich, replace=True)
    register_block("toy_mixer_only", MixerOnly, replace=True)
    register_position("toy_learned", LearnedPositions, replace=True)
    register_mixer("toy_decay_state", DecayStateMixer, replace=True)
    register_feed_forward("toy_top1_experts", Top1Experts, replace=True)

    class ToyConfig(ModelConfig):
        @classmethod
        def from_json(cls, j):
            return cls(architecture="ToyForCausalLM", raw=dict(j))

    def norm(prefix):
        return PartSpec("rmsnorm", {"size": H, "eps": EPS}, prefix=prefix)

    def build(cfg):
        rope = PartSpec("rope", {"head_dim": HD, "rotary_dim": HD, "theta": 10000.0, "scaling": None})
        nope = PartSpec("none", {"head_dim": HD})
        learned = PartSpec("toy_learned", {"head_dim": HD, "n_positions": N_POS}, prefix="layers.4.pos.")

        def attn(i, position, window):
            return PartSpec("attention", {"hidden_size": H, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD,
                                          "softmax_scale": HD ** -0.5, "window": window, "position": position},
                            prefix=f"layers.{i}.attn.")

        swiglu = lambda i: PartSpec("swiglu", {"hidden_size": H, "intermediate_size": INTER}, prefix=f"layers.{i}.mlp.")
        layers = (
            LayerSpec("prenorm", attn(0, rope, 0), norm("layers.0.n1."), swiglu(0), norm("layers.0.n2.")),
            LayerSpec("prenorm", PartSpec("toy_decay_state", {"hidden_size": H, "state_size": D_STATE, "decay": DECAY},
                                          prefix="layers.1.mix."), norm("layers.1.n1."),
                      PartSpec("toy_top1_experts", {"hidden_size": H, "intermediate_size": INTER,
                                                    "n_experts": N_EXPERTS}, prefix="layers.1.moe."),
                      norm("layers.1.n2.")),
            LayerSpec("prenorm", attn(2, nope, WINDOW), norm("layers.2.n1."), swiglu(2), norm("layers.2.n2.")),
            LayerSpec("prenorm", attn(3, rope, 0), norm("layers.3.n1."), swiglu(3), norm("layers.3.n2.")),
            LayerSpec("prenorm", attn(4, learned, 0), norm("layers.4.n1."), swiglu(4), norm("layers.4.n2.")),
            # another arrangement, with a norm in a role of its own and no feed-forward norm
            LayerSpec("toy_parallel_sandwich", mixer=attn(5, rope, 0), mixer_norm=norm("layers.5.n1."),
                      feed_forward=swiglu(5), extra=(("out_norm", "norm", norm("layers.5.out_norm.")),)),
            # a layer without a feed-forward, whose state is kept in float64
            LayerSpec("toy_mixer_only",
                      mixer=PartSpec("toy_decay_state", {"hidden_size": H, "state_size": D_STATE, "decay": DECAY,
                                                         "state_dtype": "float64"}, prefix="layers.6.mix."),
                      mixer_norm=norm("layers.6.n1.")),
        )
        # layer 0 runs twice (two caches of its own); the last run of layer 3 reads the cache
        # that the first run of layer 0 wrote and writes none
        schedule = (ScheduleItem(0), ScheduleItem(1), ScheduleItem(2), ScheduleItem(0), ScheduleItem(3, cache_of=0),
                    ScheduleItem(4), ScheduleItem(5), ScheduleItem(6))
        return ModelSpec(hidden_size=H, vocab_size=V,
                         embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}, prefix="embed."),
                         layers=layers, schedule=schedule, final_norm=norm("final_norm."),
                         head=PartSpec("linear_head", {"vocab_size": V, "hidden_size": H, "tied_to": "embed.weight",
                                                       "require_own": False}, prefix="head."))

    register_architecture("ToyForCausalLM", ToyConfig, build, replace=True)


def toy_weights(seed=3):
    rng = np.random.default_rng(seed)
    r = lambda *s, std=0.08: bf16_round(rng.standard_normal(s).astype(np.float32) * std)
    w = {"embed.weight": r(V, H, std=0.5), "final_norm.weight": bf16_round(1 + 0.1 * rng.standard_normal(H).astype(np.float32))}
    for i in range(5):
        for n in ("n1", "n2"):
            w[f"layers.{i}.{n}.weight"] = bf16_round(1 + 0.1 * rng.standard_normal(H).astype(np.float32))
    for n in ("layers.5.n1", "layers.5.out_norm", "layers.6.n1"):
        w[f"{n}.weight"] = bf16_round(1 + 0.1 * rng.standard_normal(H).astype(np.float32))
    w["layers.6.mix.in.weight"] = r(D_STATE, H)
    w["layers.6.mix.out.weight"] = r(H, D_STATE)
    w["layers.4.pos.q.weight"] = r(N_POS, HD, std=0.5)
    w["layers.4.pos.k.weight"] = r(N_POS, HD, std=0.5)
    for i in (0, 2, 3, 4, 5):
        w[f"layers.{i}.attn.q_proj.weight"] = r(NH * HD, H, std=0.3)
        w[f"layers.{i}.attn.k_proj.weight"] = r(NKV * HD, H, std=0.3)
        w[f"layers.{i}.attn.v_proj.weight"] = r(NKV * HD, H)
        w[f"layers.{i}.attn.o_proj.weight"] = r(H, NH * HD)
        w[f"layers.{i}.mlp.gate_proj.weight"] = r(INTER, H)
        w[f"layers.{i}.mlp.up_proj.weight"] = r(INTER, H)
        w[f"layers.{i}.mlp.down_proj.weight"] = r(H, INTER)
    w["layers.1.mix.in.weight"] = r(D_STATE, H)
    w["layers.1.mix.out.weight"] = r(H, D_STATE)
    w["layers.1.moe.router.weight"] = r(N_EXPERTS, H, std=0.5)
    for k in range(N_EXPERTS):
        w[f"layers.1.moe.experts.{k}.up.weight"] = r(INTER, H)
        w[f"layers.1.moe.experts.{k}.down.weight"] = r(H, INTER)
    return w


# ----------------------------------------------------------------------------- plain forward of the toy model

def plain_forward(w, tokens):
    w = {k: v.astype(np.float64) for k, v in w.items()}
    T = len(tokens)
    pos = np.arange(T)
    freqs = np.power(np.float32(10000.0), np.arange(0, HD, 2, dtype=np.float32) / np.float32(HD))
    h = P.embed(w["embed.weight"], tokens)
    kept = {}

    def attn_block(h, i, item, rope, window, kv_from=None):
        p = f"layers.{i}."
        xn = P.rms_norm(h, w[p + "n1.weight"], EPS)
        q, k, v = P.project_qkv(xn, w[p + "attn.q_proj.weight"], w[p + "attn.k_proj.weight"],
                                w[p + "attn.v_proj.weight"], NH, NKV, HD)
        if rope == "learned":
            q = q + w["layers.4.pos.q.weight"][pos % N_POS][None]
            k = k + w["layers.4.pos.k.weight"][pos % N_POS][None]
        elif rope:
            q, k = P.apply_rope(q, pos, freqs), P.apply_rope(k, pos, freqs)
        if kv_from is not None:
            k, v = kept[kv_from]
        kept[item] = (k, v)
        h = h + P.attention(q, k, v, HD ** -0.5, window) @ w[p + "attn.o_proj.weight"].T
        xn = P.rms_norm(h, w[p + "n2.weight"], EPS)
        return h + P.swiglu_mlp(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                w[p + "mlp.down_proj.weight"])

    h = attn_block(h, 0, 0, True, 0)
    # layer 1: decaying state, then top-1 experts
    xn = P.rms_norm(h, w["layers.1.n1.weight"], EPS)
    u = xn @ w["layers.1.mix.in.weight"].T
    s = np.zeros(D_STATE)
    mix = np.empty((T, H))
    for t in range(T):
        s = DECAY * s + u[t]
        mix[t] = s @ w["layers.1.mix.out.weight"].T
    h = h + mix
    xn = P.rms_norm(h, w["layers.1.n2.weight"], EPS)
    logits = xn @ w["layers.1.moe.router.weight"].T
    probs = np.exp(logits - logits.max(-1, keepdims=True))
    probs /= probs.sum(-1, keepdims=True)
    moe = np.zeros((T, H))
    for t in range(T):
        k = int(np.argmax(probs[t]))
        moe[t] = np.maximum(xn[t] @ w[f"layers.1.moe.experts.{k}.up.weight"].T, 0) @ \
            w[f"layers.1.moe.experts.{k}.down.weight"].T * probs[t, k]
    h = h + moe
    h = attn_block(h, 2, 2, False, WINDOW)
    h = attn_block(h, 0, 3, True, 0)
    h = attn_block(h, 3, 4, True, 0, kv_from=0)
    h = attn_block(h, 4, 5, "learned", 0)
    # layer 5: attention and feed-forward side by side on one normalised input, their sum normalised
    xn = P.rms_norm(h, w["layers.5.n1.weight"], EPS)
    q, k, v = P.project_qkv(xn, w["layers.5.attn.q_proj.weight"], w["layers.5.attn.k_proj.weight"],
                            w["layers.5.attn.v_proj.weight"], NH, NKV, HD)
    q, k = P.apply_rope(q, pos, freqs), P.apply_rope(k, pos, freqs)
    both = P.attention(q, k, v, HD ** -0.5, 0) @ w["layers.5.attn.o_proj.weight"].T + \
        P.swiglu_mlp(xn, w["layers.5.mlp.gate_proj.weight"], w["layers.5.mlp.up_proj.weight"],
                     w["layers.5.mlp.down_proj.weight"])
    h = h + P.rms_norm(both, w["layers.5.out_norm.weight"], EPS)
    # layer 6: the decaying state alone
    u = P.rms_norm(h, w["layers.6.n1.weight"], EPS) @ w["layers.6.mix.in.weight"].T
    s = np.zeros(D_STATE)
    for t in range(T):
        s = DECAY * s + u[t]
        h[t] = h[t] + s @ w["layers.6.mix.out.weight"].T
    return P.rms_norm(h, w["final_norm.weight"], EPS) @ w["embed.weight"].T


# ----------------------------------------------------------------------------- the test

def test_toy_architecture_is_registered_built_and_stepped(tmp_path):
    import torch
    _register()
    from mlxforge_b200.engine.replay import make_runner
    from mlxforge_b200.engine.step import StepEntry
    from mlxforge_b200.parts.base import FixedState, PagedKV
    w = toy_weights()
    d = write_model_dir(str(tmp_path / "toy"), {"architectures": ["ToyForCausalLM"]}, w, "bfloat16")
    runner = make_runner(d, "float32", max_tokens=192)
    layout = runner.model.cache_layout
    # two paged groups (full attention: four lanes; windowed: one) and two state groups (the two
    # decaying states differ in precision, so each has slots of its own)
    assert sorted((g.need.window, g.n_lanes) for g in layout.paged) == [(0, 4), (WINDOW, 1)]
    assert sorted((g.need.dtype, g.n_lanes) for g in layout.state) == [("float32", 1), ("float64", 1)]
    assert {str(t.dtype) for t in runner.cache._state} == {"torch.float32", "torch.float64"}
    assert layout.item_lane[4] == layout.item_lane[0], "the last run reads the first run's lane"

    rng = np.random.default_rng(0)
    seqs = {"a": rng.integers(0, V, size=70).tolist(), "b": rng.integers(0, V, size=45).tolist()}
    want = {k: plain_forward(w, t) for k, t in seqs.items()}
    # a in portions of changing size with b's tokens beside it, one by one towards the end
    live = {k: runner.cache.open_sequence() for k in seqs}
    done = {k: 0 for k in seqs}
    got = {k: {} for k in seqs}
    sizes = {"a": [7, 2, 16, 5, 1, 1, 9, 2, 1, 1, 1, 3, 1, 20], "b": [1, 11, 2, 2, 1, 13, 1, 1, 1, 12]}
    step = 0
    while any(done[k] < len(seqs[k]) for k in seqs):
        entries, keys = [], []
        for k in seqs:
            if done[k] >= len(seqs[k]) or (k == "b" and step % 3 == 2):
                continue
            n = min(sizes[k][(step) % len(sizes[k])], len(seqs[k]) - done[k])
            entries.append(StepEntry(live[k], seqs[k][done[k]:done[k] + n], list(range(n))))
            keys.append((k, done[k], n))
            done[k] += n
        step += 1
        if not entries:
            continue
        logits = runner.step(entries).cpu().numpy()
        row = 0
        for k, start, n in keys:
            for j in range(n):
                got[k][start + j] = logits[row]
                row += 1
        runner.cache.check()
    worst = max(float(np.max(np.abs(got[k][p] - want[k][p]))) for k in seqs for p in range(len(seqs[k])))
    scale = max(float(np.max(np.abs(v))) for v in want.values())
    assert worst <= 1e-4 * max(1.0, scale), worst
    # the windowed group gave pages back as the window moved on; the full groups kept theirs
    win = [g for g, gl in enumerate(layout.paged) if gl.need.window][0]
    full = 1 - win
    assert live["a"].pages_held(win) < live["a"].pages_held(full) == (70 + 15) // 16
    for s in live.values():
        runner.cache.close(s)
    assert runner.cache.free_pages() == runner.cache.total_pages()
