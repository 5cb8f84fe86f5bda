"""mlxforge_b200: a small, whole inference engine for one B200, for the dense GQA
decoder (``LlamaForCausalLM``) that hvasconcelos/mlxforge runs.

    import mlxforge_b200 as mf
    engine = mf.Engine(model_spec="/path/to/model", dtype="bfloat16")
    ids = engine.generate([1, 2, 3], max_tokens=16)                 # greedy
    req = engine.submit_ids([1, 2, 3], mf.SamplingParams(temperature=0.8, seed=1), max_tokens=16)
    engine.run_until_idle(); print(req.output_ids, req.finish_reason)
"""
__version__ = "0.1.0"

from .config import (ConfigError, LlamaConfig, ModelConfig, config_from_dir, config_from_json,  # noqa: F401
                     register_architecture)
from .sampling import GREEDY, SamplingParams  # noqa: F401
from .weights import WeightError, write_random_model  # noqa: F401


def __getattr__(name):
    # the engine pulls in torch.cuda state; import it on first use
    if name in ("Engine", "EngineConfig", "QueueFull"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name in ("load_model",):
        from .engine.loading import load_model
        return load_model
    raise AttributeError(name)


def generate(model_spec, prompt_ids, max_tokens=64, params=None, **engine_options):
    """One call from a model folder and token ids to generated token ids."""
    from .engine.engine import Engine
    return Engine(model_spec=model_spec, **engine_options).generate(prompt_ids, params, max_tokens)
