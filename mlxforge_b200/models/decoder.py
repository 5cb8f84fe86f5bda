"""The model every architecture becomes: parts built from a ``ModelSpec`` and run
in the order its schedule gives.  Nothing here knows Llama; the layer loop is
the reference's (src/model/decoder_model.cpp:330-351: embed, blocks, final norm,
head) with the head applied only to the rows whose logits were asked for.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheLayout, GroupLayout
from ..parts.base import (EMBEDDINGS, HEADS, NORMS, FixedState, ModelSpec, PagedKV, TensorSpec, build_layer,
                          build_part)
from ..weights.loader import WeightError, load_tensors


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime):
        self.spec = spec
        self.rt = runtime
        self.embedding = build_part(EMBEDDINGS, spec.embedding, runtime)
        self.blocks = [build_layer(ls, runtime) for ls in spec.layers]
        self.final_norm = build_part(NORMS, spec.final_norm, runtime)
        self.head = build_part(HEADS, spec.head, runtime)
        for i, item in enumerate(spec.schedule):
            if not (0 <= item.layer < len(self.blocks)):
                raise ValueError(f"schedule item {i} names layer {item.layer}, the model has {len(self.blocks)}")
            if item.cache_of is not None and not (0 <= item.cache_of < i):
                raise ValueError(f"schedule item {i} reads the cache of item {item.cache_of}, which does not run before it")
        self.cache_layout = self._layout()

    # ------------------------------------------------------------------ weights
    def parts(self):
        yield self.embedding
        for b in self.blocks:
            yield from b.parts()
        yield self.final_norm
        yield self.head

    @property
    def graph_safe(self) -> bool:
        """Whether every part (the attention mixers' position encodings included) can be
        recorded into a CUDA graph."""
        for p in self.parts():
            if not getattr(p, "graph_safe", False):
                return False
            pos = getattr(p, "position", None)
            if pos is not None and not getattr(pos, "graph_safe", False):
                return False
        return True

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for p in self.parts():
            for name, s in p.tensor_specs().items():
                old = specs.get(name)
                if old is not None and tuple(old.shape) != tuple(s.shape):
                    raise ValueError(f"tensor '{name}' is declared with shapes {old.shape} and {s.shape}")
                # a tensor is optional only if every part that reads it says so
                specs[name] = s if old is None else TensorSpec(s.shape, old.optional and s.optional, s.role)
        return specs

    def load(self, model_dir: str) -> None:
        tensors = load_tensors(model_dir, self.tensor_specs(), self.rt.device, exact=self.rt.precise)
        self.bind(tensors)

    def bind(self, tensors) -> None:
        for p in self.parts():
            p.bind(tensors)

    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads: every part once per run of its layer."""
        total = self.final_norm.weight_bytes() + self.head.weight_bytes()
        for item in self.spec.schedule:
            total += sum(p.weight_bytes() for p in self.blocks[item.layer].parts())
        return total

    # ------------------------------------------------------------------ cache
    def _layout(self) -> CacheLayout:
        paged: List[list] = []     # [need, lanes]
        state: List[list] = []
        item_lane: List[Optional[tuple]] = []
        for i, item in enumerate(self.spec.schedule):
            if item.cache_of is not None:
                src = item_lane[item.cache_of]
                need = self.blocks[item.layer].cache_need()
                if src is None or src[0] != "paged":
                    raise ValueError(f"schedule item {i} reads the cache of item {item.cache_of}, which has none to share")
                src_need = paged[src[1]][0]
                if not isinstance(need, PagedKV) or (need.n_kv_heads, need.head_dim) != (src_need.n_kv_heads, src_need.head_dim):
                    raise ValueError(f"schedule item {i} cannot read a cache of another geometry")
                item_lane.append(src)
                continue
            need = self.blocks[item.layer].cache_need()
            if need is None:
                item_lane.append(None)
            elif isinstance(need, PagedKV):
                for g, (n, lanes) in enumerate(paged):
                    if n == need:
                        item_lane.append(("paged", g, lanes))
                        paged[g][1] += 1
                        break
                else:
                    paged.append([need, 1])
                    item_lane.append(("paged", len(paged) - 1, 0))
            elif isinstance(need, FixedState):
                for g, (n, lanes) in enumerate(state):
                    if n == need:
                        item_lane.append(("state", g, lanes))
                        state[g][1] += 1
                        break
                else:
                    state.append([need, 1])
                    item_lane.append(("state", len(state) - 1, 0))
            else:
                raise TypeError(f"mixer of layer {item.layer} declares an unknown cache need {need!r}")
        return CacheLayout(tuple(GroupLayout(n, l) for n, l in paged), tuple(GroupLayout(n, l) for n, l in state),
                           tuple(item_lane))

    # ------------------------------------------------------------------ forward
    def forward(self, batch, cache) -> Optional[torch.Tensor]:
        """Run the tokens of ``batch`` through every item of the schedule, writing
        the cache, and return float32 logits [n_wanted, vocab] (None if nothing
        was asked for)."""
        rt = self.rt
        T = batch.n_tokens
        residual = rt.buffer("residual", (T, self.spec.hidden_size), torch.float32)
        self.embedding.forward(batch.tokens, residual)
        pending = None
        for i, item in enumerate(self.spec.schedule):
            residual, pending = self.blocks[item.layer].forward(
                residual, pending, batch, cache.lane(i), writes_cache=item.cache_of is None)
        if batch.n_wanted == 0:
            return None
        hn = self.final_norm.add_forward(residual, pending, rows=batch.want_rows,
                                         out=rt.buffer("final.norm", (batch.n_wanted, self.spec.hidden_size)))
        logits = rt.buffer("logits", (batch.n_wanted, self.spec.vocab_size), torch.float32)
        return self.head.forward(hn, logits)
