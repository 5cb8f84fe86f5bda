"""Configuration, registry, safetensors container, weight binding errors and the
random-weights mode.  CPU only."""
import json
import os

import numpy as np
import pytest

import plain_llama as P
from helpers import TINY_A, TINY_B, random_weights, tensor_shapes, write_model_dir
from mlxforge_b200.config import (ConfigError, LlamaConfig, config_from_dir, config_from_json,
                                  registered_architectures)
from mlxforge_b200.parts.base import TensorSpec
from mlxforge_b200.weights import (SafetensorsError, WeightError, check_names, clean_name, read_header,
                                   write_random_model)

LLAMA_1B = {   # the Llama-3.2-1B config.json the reference tests parse (tests/core/config_test.cpp:16-64)
    "architectures": ["LlamaForCausalLM"], "attention_bias": False, "bos_token_id": 128000,
    "eos_token_id": [128001, 128008, 128009], "head_dim": 64, "hidden_act": "silu", "hidden_size": 2048,
    "intermediate_size": 8192, "max_position_embeddings": 131072, "mlp_bias": False, "model_type": "llama",
    "num_attention_heads": 32, "num_hidden_layers": 16, "num_key_value_heads": 8, "rms_norm_eps": 1e-05,
    "rope_scaling": {"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "rope_theta": 500000.0, "tie_word_embeddings": True, "vocab_size": 128256,
}


def test_llama_1b_config_fields():
    c = config_from_json(LLAMA_1B)
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (16, 2048, 32, 8)
    assert (c.head_dim, c.vocab_size, c.intermediate_size) == (64, 128256, 8192)
    assert c.rope_theta == 500000.0 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings
    assert c.eos_token_ids == (128001, 128008, 128009) and c.bos_token_id == 128000
    rs = c.rope_scaling
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == ("llama3", 32.0, 1.0, 4.0, 8192)
    assert config_from_json(c.to_json()) == c


def test_defaults_and_scalar_eos():
    j = dict(TINY_A)
    del j["head_dim"], j["tie_word_embeddings"]
    j["eos_token_id"] = 7
    j["bos_token_id"] = None
    c = config_from_json(j)
    assert c.head_dim == 16 and c.tie_word_embeddings and c.eos_token_ids == (7,) and c.bos_token_id == -1
    assert c.rope_scaling is None


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "intermediate_size", "rope_theta",
                                 "rms_norm_eps"])
def test_missing_required_field_is_named(key):
    j = dict(TINY_A)
    del j[key]
    with pytest.raises(ConfigError, match=f"missing required field '{key}'"):
        config_from_json(j)


def test_wrong_type_and_bad_values():
    with pytest.raises(ConfigError, match="field 'hidden_size' has wrong type"):
        config_from_json(dict(TINY_A, hidden_size="64"))
    with pytest.raises(ConfigError, match="must be a multiple"):
        config_from_json(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="unsupported architecture 'FooForCausalLM'"):
        config_from_json(dict(TINY_A, architectures=["FooForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_json({k: v for k, v in TINY_A.items() if k != "architectures"})
    for k in ("attention_bias", "mlp_bias"):
        with pytest.raises(ConfigError, match=k):
            config_from_json(dict(TINY_A, **{k: True}))
    with pytest.raises(ConfigError, match="hidden_act"):
        config_from_json(dict(TINY_A, hidden_act="gelu"))
    assert "LlamaForCausalLM" in registered_architectures()


def test_rope_scaling_validation():
    ok = dict(TINY_B)
    config_from_json(ok)
    with pytest.raises(ConfigError, match="unsupported rope_scaling rope_type 'yarn'"):
        config_from_json(dict(TINY_A, rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="original_max_position_embeddings"):
        config_from_json(dict(TINY_A, rope_scaling={"rope_type": "llama3", "factor": 8.0, "high_freq_factor": 4.0}))
    with pytest.raises(ConfigError, match="high_freq_factor != low_freq_factor"):
        config_from_json(dict(TINY_A, rope_scaling={"rope_type": "llama3", "factor": 8.0,
                                                    "original_max_position_embeddings": 32}))
    with pytest.raises(ConfigError, match="factor > 0"):
        config_from_json(dict(TINY_A, rope_scaling={"type": "linear", "factor": 0.0}))
    # legacy "type" key and typeless object (src/core/config.cpp:53-57)
    assert config_from_json(dict(TINY_A, rope_scaling={"type": "linear", "factor": 2.0})).rope_scaling.rope_type == "linear"
    assert config_from_json(dict(TINY_A, rope_scaling={})).rope_scaling.rope_type == "default"
    # nested rope_parameters.rope_theta wins (src/core/config.cpp:83-88)
    j = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    j["rope_parameters"] = {"rope_theta": 12345.0}
    assert config_from_json(j).rope_theta == 12345.0


def test_config_file_errors(tmp_path):
    with pytest.raises(ConfigError, match="cannot open file"):
        config_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="parse error"):
        config_from_dir(str(tmp_path))


def test_rope_frequencies_match_reference_fixture():
    from mlxforge_b200.parts.rope import rope_frequencies
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_anchor.npz"))
    f = rope_frequencies(64, 500000.0, LLAMA_1B["rope_scaling"])
    assert f.dtype == np.float32
    assert np.max(np.abs(f - g["rope_freqs"]) / g["rope_freqs"]) < 1e-6
    # the plain implementation states the same formula on its own
    assert np.array_equal(f, P.rope_frequencies(LLAMA_1B))
    for cfg in (TINY_A, TINY_B):
        hd = cfg["head_dim"]
        assert np.array_equal(rope_frequencies(hd, cfg["rope_theta"], cfg.get("rope_scaling")),
                              P.rope_frequencies(cfg))
    # Tiny B reaches all three llama3 branches: untouched, smoothed, scaled by the factor
    base = np.power(np.float32(500000.0), np.arange(0, 32, 2, dtype=np.float32) / np.float32(32))
    ratio = P.rope_frequencies(TINY_B) / base
    assert ratio[0] == 1.0 and 1.0 < ratio[1] < 8.0 and np.allclose(ratio[2:], 8.0)


# ----------------------------------------------------------------------------- container

def test_safetensors_malformed(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x00\x00\x00")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_header(str(p))
    p.write_bytes((0).to_bytes(8, "little"))
    with pytest.raises(SafetensorsError, match="invalid header length"):
        read_header(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="invalid header length"):
        read_header(str(p))
    bad = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [8, 0]}}).encode()
    p.write_bytes(len(bad).to_bytes(8, "little") + bad + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="invalid data offsets"):
        read_header(str(p))
    bad = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(bad).to_bytes(8, "little") + bad + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not fill"):
        read_header(str(p))


def test_weight_error_lists_everything():
    specs = {"a.weight": TensorSpec((2, 3)), "b.weight": TensorSpec((4,), role="vector"),
             "c.weight": TensorSpec((5, 5)), "opt.weight": TensorSpec((1,), optional=True)}
    found = {"a.weight": (2, 3), "b.weight": (5,), "zzz.bias": (3,), "extra": (1,)}
    with pytest.raises(WeightError) as ei:
        check_names(specs, found, "'x'")
    e = ei.value
    assert e.missing == ["c.weight"] and e.unexpected == ["extra", "zzz.bias"]
    assert e.wrong_shape == [("b.weight", (5,), (4,))]
    msg = str(e)
    assert "missing tensors (1): c.weight" in msg and "unexpected tensors (2): extra, zzz.bias" in msg
    assert "b.weight is [5], expected [4]" in msg
    check_names(specs, {"a.weight": (2, 3), "b.weight": (4,), "c.weight": (5, 5)})


def test_clean_name():
    assert clean_name("model.layers.0.self_attn.rotary_emb.inv_freq") is None
    assert clean_name("language_model.model.norm.weight") == "model.norm.weight"
    assert clean_name("model.language_model.layers.1.mlp.up_proj.weight") == "model.layers.1.mlp.up_proj.weight"
    assert clean_name("lm_head.weight") == "lm_head.weight"


def test_model_declares_the_checkpoint_tensors():
    """The tensors the built model asks for are exactly those of a Llama checkpoint
    (untied: with lm_head; tied: lm_head optional)."""
    import torch
    from mlxforge_b200.config import get_architecture
    from mlxforge_b200.engine.runtime import Runtime
    from mlxforge_b200.models.decoder import DecoderModel
    for cfg in (TINY_A, TINY_B):
        c = config_from_json(cfg)
        model = DecoderModel(get_architecture(c.architecture).build_spec(c), Runtime(torch.float32, "cpu"))
        specs = model.tensor_specs()
        want = dict(tensor_shapes(cfg))
        check_names(specs, want)
        if cfg["tie_word_embeddings"]:
            assert specs["lm_head.weight"].optional
            check_names(specs, dict(want, **{"lm_head.weight": (cfg["vocab_size"], cfg["hidden_size"])}))
        else:
            with pytest.raises(WeightError, match="missing tensors .*lm_head.weight"):
                check_names(specs, {k: v for k, v in want.items() if k != "lm_head.weight"})
        with pytest.raises(WeightError, match="unexpected tensors .*q_proj.bias"):
            check_names(specs, dict(want, **{"model.layers.0.self_attn.q_proj.bias": (4,)}))
        assert [g.n_lanes for g in model.cache_layout.paged] == [cfg["num_hidden_layers"]]


def test_random_weights_mode_roundtrip(tmp_path):
    c = config_from_json(TINY_B)
    d = write_random_model(str(tmp_path / "m"), c, seed=5, dtype="bfloat16", norm_std=0.1)
    cfg, w = P.load_model_dir(d)
    assert config_from_json(cfg) == c
    assert {k: v.shape for k, v in w.items()} == dict(tensor_shapes(TINY_B))
    m = w["model.layers.1.mlp.gate_proj.weight"]
    assert abs(m.std() - 0.02) < 0.002 and abs(m.mean()) < 0.002
    n = w["model.layers.0.input_layernorm.weight"]
    assert abs(n.mean() - 1.0) < 0.05 and 0.05 < n.std() < 0.2
    d2 = write_random_model(str(tmp_path / "m2"), c, seed=5, dtype="bfloat16", norm_std=0.1)
    assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()
    d3 = write_random_model(str(tmp_path / "m3"), c, seed=6, dtype="float32")
    _, w3 = P.load_model_dir(d3)
    assert not np.array_equal(w3["model.norm.weight"], n[:0]) and np.all(w3["model.norm.weight"] == 1.0)
    assert not np.allclose(w3["model.embed_tokens.weight"], w["model.embed_tokens.weight"])


def test_command_line_without_a_gpu(tmp_path):
    """The commands that need no device work on the CPU (random-weights writes a model folder,
    dump-weights lists it as ``key [shape] dtype``, apps/mlxforge_cli.cpp:147-191); generate says
    loudly that there is no device instead of computing anything on the CPU."""
    import json
    import subprocess
    import sys
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 48,
           "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 80,
           "vocab_size": 101, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}
    (tmp_path / "cfg.json").write_text(json.dumps(cfg))

    def run(*args):
        return subprocess.run([sys.executable, "-m", "mlxforge_b200", *args], capture_output=True, text=True, cwd=root)

    r = run("random-weights", str(tmp_path / "cfg.json"), str(tmp_path / "m"), "--seed", "3")
    assert r.returncode == 0, r.stderr
    assert sorted(os.listdir(tmp_path / "m")) == ["config.json", "model.safetensors"]
    r = run("dump-weights", str(tmp_path / "m"))
    assert r.returncode == 0, r.stderr
    lines = r.stdout.splitlines()
    assert "lm_head.weight [101, 48] BF16" in lines and "model.layers.1.self_attn.k_proj.weight [16, 48] BF16" in lines
    assert len([l for l in lines if l.endswith("BF16")]) == 2 * 9 + 3      # nine per layer, embedding, norm, head
    if not torch.cuda.is_available():
        r = run("generate", str(tmp_path / "m"), "1,2,3", "4")
        assert r.returncode != 0 and "no CPU fallback" in r.stderr


def _split_into_shards(tmp_path, cfg, weights, n_first):
    """A folder with config.json, two shard files and model.safetensors.index.json, as the
    reference reads it (src/core/weights.cpp:208-249; its own test: tests/core/weights_test.cpp:23-106)."""
    names = list(weights)
    first, second = {n: weights[n] for n in names[:n_first]}, {n: weights[n] for n in names[n_first:]}
    d = str(tmp_path)
    for fname, part in (("model-00001-of-00002.safetensors", first), ("model-00002-of-00002.safetensors", second)):
        write_model_dir(os.path.join(d, "_part"), cfg, part)
        os.replace(os.path.join(d, "_part", "model.safetensors"), os.path.join(d, fname))
    index = {"metadata": {"total_size": 0},
             "weight_map": {**{n: "model-00001-of-00002.safetensors" for n in first},
                            **{n: "model-00002-of-00002.safetensors" for n in second}}}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def test_a_folder_of_two_shards_loads_like_one_file(tmp_path):
    import torch
    from mlxforge_b200.config import get_architecture
    from mlxforge_b200.engine.runtime import Runtime
    from mlxforge_b200.models.decoder import DecoderModel
    from mlxforge_b200.weights import load_tensors
    from mlxforge_b200.weights.safetensors_io import model_files
    w = random_weights(TINY_B, seed=9, norm_std=0.1)
    d = _split_into_shards(tmp_path / "sharded", TINY_B, w, n_first=11)
    files = model_files(d)
    assert [os.path.basename(f) for f in files] == ["model-00001-of-00002.safetensors",
                                                    "model-00002-of-00002.safetensors"]
    c = config_from_json(TINY_B)
    model = DecoderModel(get_architecture(c.architecture).build_spec(c), Runtime(torch.float32, "cpu"))
    got = load_tensors(d, model.tensor_specs(), "cpu", exact=True)
    assert set(got) == set(w)
    for name, a in w.items():
        assert np.array_equal(got[name].float().numpy(), a), name
    model.bind(got)        # every part finds its tensors, whichever file they came from

    # a tensor that neither shard has and one that the model does not know: still ONE error for both
    os.remove(os.path.join(d, "model-00002-of-00002.safetensors"))
    second = {n: a for n, a in list(w.items())[11:] if n != "model.norm.weight"}
    second["model.layers.0.self_attn.q_proj.bias"] = np.zeros(4, dtype=np.float32)
    write_model_dir(os.path.join(d, "_part"), TINY_B, second)
    os.replace(os.path.join(d, "_part", "model.safetensors"), os.path.join(d, "model-00002-of-00002.safetensors"))
    with pytest.raises(WeightError) as ei:
        load_tensors(d, model.tensor_specs(), "cpu")
    assert ei.value.missing == ["model.norm.weight"]
    assert ei.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]


def test_an_index_with_a_missing_shard_falls_back_to_the_single_file_or_fails(tmp_path):
    from mlxforge_b200.weights.safetensors_io import model_files
    w = random_weights(TINY_A, seed=9)
    d = _split_into_shards(tmp_path / "sharded", TINY_A, w, n_first=5)
    os.remove(os.path.join(d, "model-00001-of-00002.safetensors"))
    with pytest.raises(SafetensorsError, match=r"no model.safetensors\[.index.json\]"):
        model_files(d)
    write_model_dir(d, TINY_A, w)                      # a whole model.safetensors beside the broken index
    assert [os.path.basename(f) for f in model_files(d)] == ["model.safetensors"]
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        f.write('{"metadata": {}}')
    with pytest.raises(SafetensorsError, match="has no 'weight_map' object"):
        model_files(d)


def test_rope_scaling_override_replaces_the_checkpoints_wholesale():
    """``rope_scaling`` given to the engine or on the command line replaces the checkpoint's
    object; nothing of the old one survives (src/core/config.cpp:282-300; the reference's test:
    tests/model/rope_scaling_test.cpp:116-221).  The frequencies the position encoding is built
    with are those of the plain implementation for a config that had the override to begin with."""
    from mlxforge_b200.config.model_config import apply_rope_scaling_override
    from mlxforge_b200.models.llama import build_llama_spec
    from mlxforge_b200.parts.rope import rope_frequencies
    assert TINY_B["rope_scaling"]["rope_type"] == "llama3"
    j = apply_rope_scaling_override(TINY_B, '{"rope_type": "linear", "factor": 4.0}')
    c = config_from_json(j)
    rs = c.rope_scaling
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == ("linear", 4.0, 1.0, 1.0, 0)
    position = build_llama_spec(c).layers[0].mixer.params["position"]
    got = rope_frequencies(position.params["rotary_dim"], position.params["theta"], position.params["scaling"])
    want = P.rope_frequencies(dict(TINY_B, rope_scaling={"rope_type": "linear", "factor": 4.0}))
    assert np.array_equal(got, want)
    assert not np.array_equal(got, P.rope_frequencies(TINY_B))
    # onto a checkpoint without scaling, and an override the engine cannot compute
    c2 = config_from_json(apply_rope_scaling_override(TINY_A, json.dumps(TINY_B["rope_scaling"])))
    assert c2.rope_scaling.rope_type == "llama3" and c2.rope_scaling.original_max_position_embeddings == 32
    with pytest.raises(ConfigError, match="unsupported rope_scaling rope_type 'yarn'"):
        config_from_json(apply_rope_scaling_override(TINY_A, '{"rope_type": "yarn", "factor": 2.0}'))
    with pytest.raises(ConfigError, match="invalid rope_scaling override JSON"):
        apply_rope_scaling_override(TINY_A, '{"rope_type": ')
    with pytest.raises(ConfigError, match="must be a JSON object"):
        apply_rope_scaling_override(TINY_A, '[4.0]')
