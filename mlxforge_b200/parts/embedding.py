"""Token embedding (``h[t] = E[token[t]]``, src/model/decoder_model.cpp:194-204)
into the 32-bit residual stream, and the output head (``logits = hn W^T`` with
``W = lm_head.weight`` when the checkpoint has it, else the embedding table,
:346-350), computed only for the rows that were asked for, in float32."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import Part, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.table = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.prefix + "weight": TensorSpec((self.vocab, self.hidden))}

    def bind(self, tensors) -> None:
        self.table = tensors[self.prefix + "weight"].to(self.rt.dtype).contiguous()

    def weight_bytes(self) -> int:
        return 0     # a step reads one row per token, not the table

    def forward(self, tokens, out):
        ops.embed(self.table, tokens, out)
        return out


@register_head("linear_head")
class LinearHead(Part):
    graph_safe = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.require_own = bool(params.get("require_own", False))
        self.weight = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        own = TensorSpec((self.vocab, self.hidden), optional=not self.require_own and self.tied_to is not None)
        specs = {self.prefix + "weight": own}
        if self.tied_to and not self.require_own:
            specs[self.tied_to] = TensorSpec((self.vocab, self.hidden))
        return specs

    def bind(self, tensors) -> None:
        w = tensors.get(self.prefix + "weight")
        if w is None:
            w = tensors[self.tied_to]
        self.weight = w.to(self.rt.dtype).contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, out):
        """x [n, H] in the compute dtype -> float32 logits [n, V]."""
        return self.rt.linear(x, self.weight, out)
