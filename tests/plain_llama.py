"""A plain, slow implementation of the Llama dense decoder in NumPy float64.

Whole sequences, no cache, one function for each part, written from the
reference's formulas (hvasconcelos/mlxforge; every function cites file:line of
that project).  It shares no code with ``mlxforge_b200``: it has its own
safetensors reader, its own config reading and its own sampler.

The reference's model code needs Apple MLX (``CMakeLists.txt:14-16`` refuses
other hosts, every model source includes ``mlx/...``), so it cannot be imported
or compiled here and this file rests on the formulas.  Three of the reference's
committed fixtures need no weights: ``reference/fixtures/rope_freqs.npy`` and
``q_pre0.npy -> q_rope0.npy`` anchor the position encoding, ``embeddings.npy ->
attn_norm0.npy`` the RMSNorm (its weight is the same vector for every position);
small copies of what they check are under ``tests/golden/`` with the scripts that
cut them, and ``tests/test_plain.py`` holds this file against them.  The one part
of the reference that does compile here, its configuration parser, is compared
with this build's parser in ``tests/test_config_reference.py``.  Attention and the
feed-forward have no fixture without weights and stay pinned by their formulas.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------- files

def read_safetensors(path):
    """{name: float64 or int array}.  Format: 8-byte LE header length, JSON header,
    raw bytes (src/inspect/safetensors_header.cpp:21-63)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[b:e]
        dt = info["dtype"]
        if dt == "BF16":
            u = np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif dt == "F32":
            a = np.frombuffer(raw, dtype=np.float32).astype(np.float64)
        elif dt == "F16":
            a = np.frombuffer(raw, dtype=np.float16).astype(np.float64)
        else:
            raise ValueError(dt)
        out[name] = a.reshape(info["shape"])
    return out


def load_model_dir(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ----------------------------------------------------------------------------- rounding model

ROUND = None
"""None: everything in float64.  A function (e.g. ``round_bf16``): applied to every
activation a 16-bit engine would store in 16 bits (normed inputs, projections,
rotated queries and keys, probabilities, attention output, feed-forward
intermediates and the deltas added to the residual stream; never the residual
stream, the softmax sums or the logits).  The gap between the two runs of this
same plain implementation is the noise floor of bfloat16 activations for a given
model and prompt; the tests derive their bfloat16 tolerance from it."""


def round_bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
    return r.view(np.float32).astype(np.float64)


def _r(x):
    return x if ROUND is None else ROUND(x)


# ----------------------------------------------------------------------------- parts

def rope_frequencies(cfg):
    """float32 [head_dim/2]: ``theta ** (arange(0, hd, 2) / hd)`` with the llama3 /
    linear rescaling, all in float32 as the reference computes it
    (src/model/decoder_model.cpp:44-49 base schedule, :65-70 linear, :116-146 llama3).
    An angle is ``position / freq`` (src/model/decoder_model.cpp:220-228)."""
    hd = cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    base = np.float32(cfg["rope_theta"])
    idx = np.arange(0, hd, 2, dtype=np.float32)
    freqs = np.power(base, idx / np.float32(hd)).astype(np.float32)
    rs = cfg.get("rope_scaling") or cfg.get("rope_parameters")
    kind = "default"
    if isinstance(rs, dict):
        kind = rs.get("rope_type", rs.get("type", "")) or "default"
    if kind == "default":
        return freqs
    factor = np.float32(rs.get("factor", 1.0))
    if kind == "linear":
        return (freqs * factor).astype(np.float32)
    assert kind == "llama3", kind
    low_ff = np.float32(rs.get("low_freq_factor", 1.0))
    high_ff = np.float32(rs.get("high_freq_factor", 1.0))
    old_ctx = np.float32(rs["original_max_position_embeddings"])
    low_wl = old_ctx / low_ff
    high_wl = old_ctx / high_ff
    two_pi = np.float32(6.283185307179586)                      # src/model/decoder_model.cpp:21
    wavelens = (two_pi * freqs).astype(np.float32)
    scaled = np.where(wavelens > low_wl, freqs * factor, freqs).astype(np.float32)
    is_medium = (wavelens > high_wl) & (wavelens < low_wl)
    smooth = ((old_ctx / wavelens - low_ff) / (high_ff - low_ff)).astype(np.float32)
    denom = ((np.float32(1.0) - smooth) / factor + smooth).astype(np.float32)
    smooth_freqs = (scaled / denom).astype(np.float32)
    return np.where(is_medium, smooth_freqs, scaled).astype(np.float32)


def embed(table, tokens):
    """``h[t] = E[token[t]]`` (src/model/decoder_model.cpp:194-204)."""
    return table[np.asarray(tokens, dtype=np.int64)]


def rms_norm(x, w, eps):
    """``x * rsqrt(mean(x^2) + eps) * w`` over the last axis; the weight multiplies
    directly, no ``1 + w`` (src/model/decoder_model.cpp:206-208)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return _r(x / np.sqrt(ms + eps) * w)


def project_qkv(xn, wq, wk, wv, n_heads, n_kv_heads, head_dim):
    """``x @ W^T`` with HF ``(out, in)`` weights, no bias, then split into heads:
    head ``h`` is output rows ``[h*hd, (h+1)*hd)`` (src/model/decoder_model.cpp:174-192,234-253).
    Returns q [nh, T, hd], k [nkv, T, hd], v [nkv, T, hd]."""
    T = xn.shape[0]
    q = _r(xn @ wq.T).reshape(T, n_heads, head_dim).transpose(1, 0, 2)
    k = _r(xn @ wk.T).reshape(T, n_kv_heads, head_dim).transpose(1, 0, 2)
    v = _r(xn @ wv.T).reshape(T, n_kv_heads, head_dim).transpose(1, 0, 2)
    return q, k, v


def apply_rope(x, positions, freqs):
    """Half-split rotation (``traditional=false``) over the full head:
    ``out[i] = x[i] cos - x[i+hd/2] sin``; ``out[i+hd/2] = x[i] sin + x[i+hd/2] cos``
    with angle ``p / f_i`` (src/model/decoder_model.cpp:220-228; pairing checked
    against reference/fixtures/q_pre0.npy -> q_rope0.npy).  x: [heads, T, hd]."""
    hd = x.shape[-1]
    half = hd // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] / freqs.astype(np.float64)[None, :]
    c, s = np.cos(ang), np.sin(ang)
    x1, x2 = x[..., :half], x[..., half:]
    return _r(np.concatenate([x1 * c - x2 * s, x1 * s + x2 * c], axis=-1))


def attention(q, k, v, scale, window=0):
    """Causal GQA attention over the whole sequence: ``softmax(q k^T * scale) v``;
    query head ``h`` reads KV head ``h // (nh / nkv)`` (src/model/sdpa.cpp:27);
    query ``j`` sees keys ``<= j`` (src/model/sdpa.cpp:44-46, src/model/decoder_model.cpp:260-275).
    ``window`` > 0 also hides keys older than ``j - window + 1`` (not a Llama
    option; it is here for the windowed cache groups the engine supports).
    q: [nh, T, hd]; k, v: [nkv, T, hd] -> [T, nh*hd]."""
    nh, T, hd = q.shape
    nkv = k.shape[0]
    rep = nh // nkv
    out = np.empty((T, nh, hd), dtype=q.dtype)
    jj = np.arange(T)
    visible = jj[None, :] <= jj[:, None]
    if window and window > 0:
        visible &= jj[None, :] > (jj[:, None] - window)
    for h in range(nh):
        s = (q[h] @ k[h // rep].T) * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        out[:, h, :] = (_r(p) @ v[h // rep]) / p.sum(axis=-1, keepdims=True)
    return _r(out.reshape(T, nh * hd))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """``down( silu(gate(x)) * up(x) )``, ``silu(g) = g * sigmoid(g)``
    (src/model/decoder_model.cpp:277-282)."""
    g = _r(x @ w_gate.T)
    u = _r(x @ w_up.T)
    return _r(_r((g / (1.0 + np.exp(-g))) * u) @ w_down.T)


def decoder_block(h, w, cfg, layer, positions, freqs, window=0):
    """Pre-norm block with two residuals: ``h + attn(norm(h))`` then
    ``+ mlp(norm(.))`` (src/model/decoder_model.cpp:288-293)."""
    p = f"model.layers.{layer}."
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim", cfg["hidden_size"] // nh)
    eps = cfg["rms_norm_eps"]
    xn = rms_norm(h, w[p + "input_layernorm.weight"], eps)
    q, k, v = project_qkv(xn, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                          w[p + "self_attn.v_proj.weight"], nh, nkv, hd)
    q = apply_rope(q, positions, freqs)
    k = apply_rope(k, positions, freqs)                       # v is never rotated
    a = attention(q, k, v, 1.0 / np.sqrt(hd), window)         # scale 1/sqrt(hd): decoder_model.cpp:265
    h = h + _r(a @ w[p + "self_attn.o_proj.weight"].T)        # :273-274,290
    xn = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    return h + swiglu_mlp(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])


def forward_logits(cfg, w, tokens):
    """Logits [T, V] of one whole sequence (src/model/decoder_model.cpp:330-351,363-369):
    embed, all blocks, final norm, head = ``lm_head.weight`` if present else the
    embedding table (:348-349)."""
    T = len(tokens)
    positions = np.arange(T)
    freqs = rope_frequencies(cfg)
    h = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_block(h, w, cfg, layer, positions, freqs)
    hn = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return hn @ head.T


# ----------------------------------------------------------------------------- sampling

def greedy(logits_row):
    """argmax over the vocabulary (src/sample/sampler.cpp:59-61); ties go to the
    lowest index (the reference leaves ties to MLX)."""
    return int(np.argmax(logits_row))


def uniform_for(seed, index):
    """The engine's counter-based draw: a splitmix64 hash of (seed, output index)
    mapped to [0, 1) with 24 bits.  Restated here, not imported."""
    mask = (1 << 64) - 1
    z = (int(seed) * 0x9E3779B97F4A7C15 + (int(index) + 1) * 0xD1B54A32D192ED03) & mask
    z = (z + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def filter_logits(logits_row, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """``logits / T`` then top-k, top-p, min-p in the reference's order, removed
    entries at -inf (src/sample/sampler.cpp:63-93,156-163)."""
    x = np.asarray(logits_row, dtype=np.float64) / temperature
    V = x.shape[0]
    if top_k > 0:
        k = min(top_k, V)
        kth = np.sort(x)[V - k]
        x = np.where(x < kth, -np.inf, x)
    if top_p < 1.0:
        order = np.argsort(-x, kind="stable")
        sl = x[order]
        p = np.exp(sl - sl.max())
        p /= p.sum()
        prior = np.cumsum(p) - p
        keep = prior < top_p
        y = np.full(V, -np.inf)
        y[order[keep]] = sl[keep]
        x = y
    if min_p > 0.0:
        p = np.exp(x - x.max())
        p /= p.sum()
        x = np.where(p < min_p * p.max(), -np.inf, x)
    return x


def sample_token(logits_row, temperature, u, top_k=0, top_p=1.0, min_p=0.0):
    """``temperature <= 0`` is greedy; else a categorical draw from
    ``softmax(filtered logits / T)`` (src/sample/sampler.cpp:141-166) by inverse
    CDF in index order: the first index whose cumulative probability exceeds
    ``u``.  Returns (token, distance of u to the nearest CDF edge)."""
    if temperature <= 0.0:
        return greedy(logits_row), 1.0
    x = filter_logits(logits_row, temperature, top_k, top_p, min_p)
    p = np.exp(x - x.max())
    p /= p.sum()
    cdf = np.cumsum(p)
    tok = int(np.searchsorted(cdf, u, side="right"))
    tok = min(tok, len(p) - 1)
    while p[tok] == 0.0 and tok > 0:
        tok -= 1
    lo = cdf[tok] - p[tok]
    return tok, float(min(u - lo, cdf[tok] - u))


def apply_penalties(logits_row, history, repetition=1.0, frequency=0.0, presence=0.0):
    """Repetition (divide positive / multiply negative logits of seen tokens), then
    frequency (``- f * count``) and presence (``- p * seen``) penalties
    (src/sample/sampler.cpp:95-135)."""
    x = np.array(logits_row, dtype=np.float64)
    hist = np.asarray(history, dtype=np.int64)
    if repetition != 1.0 and hist.size:
        ids = np.unique(hist)
        x[ids] = np.where(x[ids] > 0, x[ids] / repetition, x[ids] * repetition)
    if (frequency != 0.0 or presence != 0.0) and hist.size:
        counts = np.bincount(hist, minlength=x.shape[0]).astype(np.float64)
        x = x - counts * frequency - (counts > 0) * presence
    return x


def generate(cfg, w, prompt, max_tokens, temperature=0.0, seed=0, eos_ids=()):
    """Full-recompute generation, no cache, as the reference's oracle loop does
    (reference/dump_ref.py:202-213).  EOS stops and is not emitted
    (src/runtime/single_stream.cpp:86-89)."""
    seq = list(prompt)
    out = []
    for i in range(max_tokens):
        row = forward_logits(cfg, w, seq)[-1]
        tok, _ = sample_token(row, temperature, uniform_for(seed, i))
        if tok in eos_ids:
            break
        out.append(tok)
        seq.append(tok)
    return out
