from .decoder import DecoderModel
from . import llama  # noqa: F401
