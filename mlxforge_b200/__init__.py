"""mlxforge_b200: a small, whole inference engine for one B200, for the dense GQA
decoder (LlamaForCausalLM) that hvasconcelos/mlxforge runs."""
__version__ = "0.1.0"
