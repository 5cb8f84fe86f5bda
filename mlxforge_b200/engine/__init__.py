from .loading import load_model, parse_dtype, require_gpu
from .runtime import Runtime
from .step import ModelRunner, StepBatch, StepEntry
