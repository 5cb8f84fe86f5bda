"""Shared by the tests: tiny configurations of the architecture that differ in
every size and option, model folders with random weights written into a
temporary directory (never committed), and comparison helpers.  The weights are
made here with NumPy and written with a writer of the tests' own, so that a test
of the engine does not rest on the engine's own random-weights mode."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

# ---------------------------------------------------------------------------- configurations

TINY_A = {   # 2 layers, GQA 4:2, head_dim = hidden/heads, no rope scaling, tied head
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "max_position_embeddings": 128, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
TINY_B = {   # 3 layers, MQA 6:1, head_dim != hidden/heads, llama3 scaling hitting all three branches, untied
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}
TINY_C = {   # sizes that are no power of two anywhere: MHA 5:5, head_dim 48, odd vocabulary, linear scaling
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 136, "vocab_size": 307, "rope_theta": 1000000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "max_position_embeddings": 512, "rms_norm_eps": 3e-5, "tie_word_embeddings": False,
}
TINY_D = {   # a width, an intermediate size and a vocabulary that are no multiple of 8: the scalar kernel paths
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 3, "num_key_value_heads": 3,
    "head_dim": 16, "intermediate_size": 52, "vocab_size": 131, "rope_theta": 20000.0,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
# The two below are still small, but have the shapes that the serving kernels are written for, so
# that those kernels run inside a model: head size 64 (decode attention with tensor copies, the
# tcgen05 prefill attention two tiles ahead), widths that are whole stages of the few-row product
# (one tensor copy per stage), an intermediate size of at least 256 rows' worth of tcgen05 tiles.
SMALL_E = {  # head_dim 64, GQA 8:2, llama3 scaling, tied head
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 1024, "num_attention_heads": 8, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 2048, "vocab_size": 2048, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "max_position_embeddings": 1024, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
SMALL_F = {  # head_dim 128, GQA 12:4, a width of three half-stages, a vocabulary that is no multiple of 16, untied
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 4,
    "head_dim": 128, "intermediate_size": 3072, "vocab_size": 3000, "rope_theta": 250000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 4.0},
    "max_position_embeddings": 1024, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": SMALL_E, "F": SMALL_F}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 5}
NORM_STD = {"A": 0.0, "B": 0.1, "C": 0.2, "D": 0.05, "E": 0.1, "F": 0.15}

# The benchmark's shape itself (Llama 3.2 1B)
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 16, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "tie_word_embeddings": True,
}


def tensor_shapes(cfg):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hd = cfg.get("head_dim", H // cfg["num_attention_heads"])
    nq, nkv = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    out = [("model.embed_tokens.weight", (V, H))]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (H,)), (p + "self_attn.q_proj.weight", (nq, H)),
                (p + "self_attn.k_proj.weight", (nkv, H)), (p + "self_attn.v_proj.weight", (nkv, H)),
                (p + "self_attn.o_proj.weight", (H, nq)), (p + "post_attention_layernorm.weight", (H,)),
                (p + "mlp.gate_proj.weight", (I, H)), (p + "mlp.up_proj.weight", (I, H)),
                (p + "mlp.down_proj.weight", (H, I))]
    out.append(("model.norm.weight", (H,)))
    if not cfg.get("tie_word_embeddings", True):
        out.append(("lm_head.weight", (V, H)))
    return out


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_round(a):
    return (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32)


def random_weights(cfg, seed, norm_std=0.0, std=0.02, qk_gain=1.0, draw32=False):
    """float32 arrays whose values are exact in bfloat16, so that the 32-bit and the
    bfloat16 engine and the plain implementation all start from the same numbers.
    ``qk_gain`` scales the query and key projections: a gain of some tens makes the
    softmax peaked, so that one wrong or missing key changes the logits.  ``draw32`` draws in
    float32 (another stream of numbers, several times faster: for models of a billion values)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg):
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            a = np.ones(shape, dtype=np.float32) + rng.standard_normal(shape).astype(np.float32) * norm_std
        else:
            a = (rng.standard_normal(shape, dtype=np.float32) if draw32
                 else rng.standard_normal(shape).astype(np.float32)) * np.float32(std)
            if "q_proj" in name or "k_proj" in name:
                a = a * qk_gain
        w[name] = bf16_round(a)
    return w


def write_model_dir(path, cfg, weights, dtype="bfloat16"):
    """config.json + model.safetensors, written by hand (8-byte length, JSON header, bytes)."""
    os.makedirs(path, exist_ok=True)
    header, blobs, off = {}, [], 0
    for name, a in weights.items():
        raw = to_bf16_bits(a).tobytes() if dtype == "bfloat16" else np.ascontiguousarray(a, np.float32).tobytes()
        header[name] = {"dtype": "BF16" if dtype == "bfloat16" else "F32", "shape": list(a.shape),
                        "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return path


def make_tiny(tmp_path, which, dtype="bfloat16", qk_gain=1.0):
    cfg = TINY[which]
    w = random_weights(cfg, SEEDS[which], NORM_STD[which], qk_gain=qk_gain)
    d = write_model_dir(str(tmp_path / f"tiny_{which}_{dtype}_{qk_gain}"), cfg, w, dtype)
    return d, cfg, {k: v.astype(np.float64) for k, v in w.items()}


def random_prompt(cfg, n, seed):
    return np.random.default_rng(1000 + seed).integers(0, cfg["vocab_size"], size=n).tolist()


def max_abs_diff(a, b):
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64))))
