"""The configuration parser against hvasconcelos/mlxforge's own: ``src/core/config.cpp`` is pure
C++ over nlohmann/json (no MLX), so it compiles on any host.  This test builds it at test time
with a small driver (tests/support/config_probe.cpp), feeds both parsers the same objects — the
reference's Llama-3.2-1B fixture, every required key removed in turn, wrong types, the optional
keys, the rope-scaling variants and the rope-scaling override — and compares every field and
every error text (cases follow the reference's tests/core/config_test.cpp:16-64 and
tests/model/rope_scaling_test.cpp).

Where the two differ on purpose it is said at the case: this engine computes no yarn scaling and
refuses it; it also refuses non-positive sizes that the reference would accept and divide by.

Skipped when the reference's sources, a C++ compiler or nlohmann's header is not there.  The
reference is looked for in ``$MLXFORGE_REFERENCE_DIR``, else in a folder ``reference`` beside the
repository."""
import copy
import json
import os
import shutil
import subprocess
import sysconfig

import pytest

from mlxforge_b200.config import config_from_json
from mlxforge_b200.config.model_config import ConfigError, apply_rope_scaling_override

HERE = os.path.dirname(os.path.abspath(__file__))


def _reference_dir():
    cand = os.environ.get("MLXFORGE_REFERENCE_DIR") or os.path.join(HERE, "..", "..", "reference")
    return cand if os.path.isfile(os.path.join(cand, "src", "core", "config.cpp")) else None


def _json_include():
    cands = [os.environ.get("NLOHMANN_INCLUDE"),
             os.path.join(sysconfig.get_paths()["purelib"], "include", "cudnn_frontend", "thirdparty"),
             "/usr/include", "/usr/local/include"]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "nlohmann", "json.hpp")):
            return c
    return None


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    ref, inc, cxx = _reference_dir(), _json_include(), shutil.which("g++") or shutil.which("c++")
    if not (ref and inc and cxx):
        pytest.skip("needs the reference's sources, a C++ compiler and nlohmann/json.hpp")
    exe = str(tmp_path_factory.mktemp("config_probe") / "config_probe")
    cmd = [cxx, "-std=c++17", "-O0", "-I", os.path.join(ref, "src"), "-I", inc,
           os.path.join(ref, "src", "core", "config.cpp"), os.path.join(HERE, "support", "config_probe.cpp"),
           "-o", exe]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert p.returncode == 0, p.stdout

    def run(cases):
        text = "".join(json.dumps(c) + "\n" for c in cases)
        r = subprocess.run([exe], input=text, stdout=subprocess.PIPE, text=True, check=True)
        lines = [json.loads(x) for x in r.stdout.splitlines() if x.strip()]
        assert len(lines) == len(cases)
        return lines
    run.fixture = os.path.join(ref, "tests", "fixtures", "config_llama32_1b.json")
    return run


def ours(case):
    """This engine's parser on the same case, as the probe prints it."""
    j = dict(case["config"])
    j.setdefault("architectures", ["LlamaForCausalLM"])     # the registry dispatches on it; the reference ignores it
    try:
        if "override" in case:
            j = apply_rope_scaling_override(j, case["override"])
        c = config_from_json(j)
    except ConfigError as e:
        return {"error": str(e)}
    rs = c.rope_scaling
    return {
        "model_type": c.model_type, "num_hidden_layers": c.num_hidden_layers, "hidden_size": c.hidden_size,
        "num_attention_heads": c.num_attention_heads, "num_key_value_heads": c.num_key_value_heads,
        "head_dim": c.head_dim, "vocab_size": c.vocab_size, "intermediate_size": c.intermediate_size,
        "rope_theta": c.rope_theta, "rms_norm_eps": c.rms_norm_eps,
        "max_position_embeddings": c.max_position_embeddings, "tie_word_embeddings": c.tie_word_embeddings,
        "bos_token_id": c.bos_token_id, "eos_token_ids": list(c.eos_token_ids),
        "rope_scaling": None if rs is None else {
            "rope_type": rs.rope_type, "factor": rs.factor, "low_freq_factor": rs.low_freq_factor,
            "high_freq_factor": rs.high_freq_factor,
            "original_max_position_embeddings": rs.original_max_position_embeddings},
    }


def same(a, b):
    """Fields equal; the reference holds its reals in float32."""
    if isinstance(a, dict) and isinstance(b, dict):
        return a.keys() == b.keys() and all(same(a[k], b[k]) for k in a)
    if isinstance(a, float) or isinstance(b, float):
        return abs(float(a) - float(b)) <= 1e-6 * max(1.0, abs(float(a)))
    return a == b


BASE = {"num_hidden_layers": 2, "hidden_size": 8, "num_attention_heads": 4, "num_key_value_heads": 2,
        "vocab_size": 100, "intermediate_size": 16, "rope_theta": 10000.0, "rms_norm_eps": 1e-6}
REQUIRED = list(BASE)


def with_(**kw):
    j = copy.deepcopy(BASE)
    j.update(kw)
    return {"config": j}


def test_fields_agree_with_the_reference_parser(probe):
    with open(probe.fixture) as f:
        fixture = json.load(f)
    llama3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
              "original_max_position_embeddings": 32}
    cases = [
        {"config": fixture},
        with_(some_future_field=123, torch_dtype="bfloat16"),          # unknown keys; head_dim derived; no eos
        with_(head_dim=6, max_position_embeddings=77, tie_word_embeddings=False, model_type="llama"),
        with_(eos_token_id=5), with_(eos_token_id=[5, 9]), with_(eos_token_id=None),
        with_(bos_token_id=None), with_(bos_token_id=3),
        with_(rope_scaling=llama3),
        with_(rope_scaling={"type": "linear", "factor": 2.0}),          # the legacy key for the type
        with_(rope_scaling={"factor": 4.0}),                            # no type at all: "default"
        with_(rope_scaling={"rope_type": "default"}),
        with_(rope_scaling=None),
        with_(rope_parameters={"rope_theta": 250000.0, "rope_type": "linear", "factor": 3.0}),
        dict(with_(rope_scaling=llama3), override='{"rope_type":"linear","factor":4.0}'),
        dict(with_(), override='{"rope_type":"llama3","factor":2.0,"low_freq_factor":1.0,"high_freq_factor":4.0,'
                               '"original_max_position_embeddings":64}'),
    ]
    for case, ref in zip(cases, probe(cases)):
        assert "error" not in ref, (case, ref)
        mine = ours(case)
        assert same(mine, ref), f"\ncase {case}\nours {mine}\nref  {ref}"
    # the fixture's values, spelled out (tests/core/config_test.cpp:16-37)
    c = ours(cases[0])
    assert (c["num_hidden_layers"], c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"],
            c["head_dim"], c["vocab_size"], c["intermediate_size"], c["max_position_embeddings"]) == \
        (16, 2048, 32, 8, 64, 128256, 8192, 131072)
    assert c["eos_token_ids"] == [128001, 128008, 128009] and c["bos_token_id"] == 128000


def test_errors_agree_with_the_reference_parser(probe):
    missing = [{"config": {k: v for k, v in BASE.items() if k != key}} for key in REQUIRED]
    wrong = [with_(num_hidden_layers="two"), with_(rms_norm_eps="small"), with_(hidden_size=[8])]
    exact = missing + [
        with_(rope_scaling={"rope_type": "linear", "factor": 0.0}),
        with_(rope_scaling={"rope_type": "linear", "factor": -1.0}),
    ]
    for case, ref in zip(exact, probe(exact)):
        assert "error" in ref, (case, ref)
        assert ours(case) == ref, (case, ours(case), ref)
    # same sentence up to the part that names the JSON library's own wording or the list of types
    prefix = wrong + [
        with_(rope_scaling={"rope_type": "dynamic", "factor": 2.0}),
        dict(with_(), override='{"rope_type": "linear", '),
        dict(with_(), override='[1, 2]'),
        dict(with_(), override='{"rope_type":"ntk"}'),
    ]
    cuts = ["has wrong type: "] * len(wrong) + ["(supported:", "override JSON: ", "must be a JSON object", "(supported:"]
    for case, ref, cut in zip(prefix, probe(prefix), cuts):
        mine = ours(case)
        assert "error" in ref and "error" in mine, (case, mine, ref)
        assert cut in ref["error"] and cut in mine["error"], (mine, ref)
        assert mine["error"].split(cut)[0] == ref["error"].split(cut)[0], (mine, ref)


def test_where_this_engine_is_stricter_on_purpose(probe):
    """The reference accepts these and this engine refuses them; both facts are pinned."""
    yarn = with_(rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64})
    zero_heads = with_(num_key_value_heads=0)
    flat = with_(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 2.0, "high_freq_factor": 2.0,
                               "original_max_position_embeddings": 32})
    refs = probe([yarn, zero_heads, flat])
    assert all("error" not in r for r in refs), refs
    assert "unsupported rope_scaling rope_type 'yarn'" in ours(yarn)["error"]       # no yarn schedule in this engine
    assert "must be positive" in ours(zero_heads)["error"]                            # it would divide by it
    assert "high_freq_factor != low_freq_factor" in ours(flat)["error"]              # the formula divides by the difference
