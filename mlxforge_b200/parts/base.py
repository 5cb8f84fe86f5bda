"""What a model is made of, as data, and the interfaces its parts implement.

A model is a ``ModelSpec``: an embedding, a list of ``LayerSpec`` (each naming a
mixer, a feed-forward, their norms and the arrangement of the four in a block,
every one by *kind* with its sizes and constants as parameters), a *schedule*
that says in which order layers run (a layer may appear twice; a run may read
the cache another run wrote), a final norm and an output head.  The reference
builds the same thing with virtual methods on one class (``attention /
decoder_block / feed_forward``, src/model/decoder_model.h:83-93,134-139); here
the seams are registries so that a new mixer, feed-forward, norm, position
encoding, block arrangement or architecture is one ``register_*`` call and no
part knows which model it is in.

Every part is built as ``cls(spec.params, prefix=spec.prefix, runtime=rt)``,
declares the tensors it reads with ``tensor_specs()``, receives them through
``bind()`` and then runs on the flat token batch of one engine step.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Union


# --------------------------------------------------------------------------- specs

@dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its sizes and constants and its tensor-name prefix."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def __hash__(self):  # params is a dict
        return hash((self.kind, self.prefix, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its four parts and how a block arranges them."""

    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class ScheduleItem:
    """One run of a layer.  ``cache_of`` names an earlier item of the schedule
    whose cache this run reads instead of owning one (it then writes nothing)."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleItem, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()
    max_position_embeddings: int = 0


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part reads: its shape, whether it may be absent, and whether it
    is a matrix used in products (kept in the compute dtype) or a vector of
    per-channel constants (kept in 32-bit)."""

    shape: Tuple[int, ...]
    optional: bool = False
    role: str = "matrix"           # "matrix" | "vector" | "table" (integer)


# --------------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class PagedKV:
    """Keys and values that grow with the sequence, kept in pages.  ``window`` > 0
    means a run only ever reads the last ``window`` positions, so older pages are
    given back."""

    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size, one tensor of ``shape`` (32-bit floats)
    per run of the layer, zeroed when a request is admitted."""

    shape: Tuple[int, ...]
    tag: str = ""


CacheNeed = Union[PagedKV, FixedState, None]


# --------------------------------------------------------------------------- interfaces

class Part:
    """Common base: construction, tensor declaration, binding."""

    # True if ``forward`` only launches work that a CUDA graph can record and replay:
    # no host decision that depends on the step's data (lengths, slots), no read-back,
    # no allocation.  The engine replays decode steps from graphs only when every part
    # of the model says so; a part that does not say so is simply run eagerly.
    graph_safe = False

    def __init__(self, params: Dict[str, Any], prefix: str, runtime: "Any"):
        self.params = dict(params)
        self.prefix = prefix
        self.rt = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        """Full tensor names this part reads, with expected shapes."""
        return {}

    def bind(self, tensors: Dict[str, Any]) -> None:
        """Receive the loaded tensors (device tensors keyed by full name) and
        pack whatever operand layout the kernels want."""

    def weight_bytes(self) -> int:
        """Bytes of weights one step reads from this part (for the roofline)."""
        return 0


class Norm(Part):
    def forward(self, x, out=None):
        """Normalise each row of ``x`` ([T, H], 32-bit residual stream) into the
        compute dtype."""
        raise NotImplementedError

    def add_forward(self, residual, delta, out=None, rows=None):
        """``residual += delta`` (in 32-bit, in place) and return the normalised
        sum; ``delta`` may be None.  With ``rows`` (int32 device indices) only
        those rows are produced and the residual is left as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns integer positions into whatever the mixer applies to queries and keys."""

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache: bool) -> None:
        """``qkv``: [T, (n_heads + 2 n_kv_heads) * head_dim], the step's projections side by
        side.  Writes the encoded queries to ``q_out`` [T, n_heads * head_dim] and, if
        ``writes_cache``, the encoded keys and the values of token ``t`` into page
        ``batch.block_table(lane.group)[batch.seq_of_token[t], p // lane.page_size]``, slot
        ``p % lane.page_size`` of ``lane.k`` / ``lane.v`` ([page, kv_head, slot, head_dim]),
        with ``p = batch.positions[t]``.  The mixer forwards this part's ``tensor_specs`` and
        ``bind``, so an encoding may own tensors."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return None

    def forward(self, x, batch, cache, writes_cache: bool = True):
        """``x``: [T, H] normalised tokens of the step in the compute dtype;
        ``batch``: the step's ``StepBatch``; ``cache``: this run's view of the
        cache (a ``KVLane``, a state tensor, or None).  Returns the delta [T, H]
        to add to the residual stream."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, batch):
        """[T, H] -> delta [T, H]."""
        raise NotImplementedError


class Block:
    """Arrangement of a layer's parts around the residual stream.  The stream
    travels as ``(residual, pending)``: ``pending`` is a delta not yet added, so
    that the add can be fused with the next norm."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward,
                 feed_forward_norm: Norm, runtime: "Any"):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.rt = runtime

    def parts(self) -> List[Part]:
        return [self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm]

    def forward(self, residual, pending, batch, cache, writes_cache: bool = True):
        raise NotImplementedError


# --------------------------------------------------------------------------- registries

class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Any] = {}

    def register(self, kind: str, obj: Any = None, *, replace: bool = False):
        def put(o):
            if kind in self._items and not replace and self._items[kind] is not o:
                raise KeyError(f"{self.what} kind '{kind}' is already registered")
            self._items[kind] = o
            return o
        return put if obj is None else put(obj)

    def get(self, kind: str):
        try:
            return self._items[kind]
        except KeyError:
            known = ", ".join(sorted(self._items)) or "none"
            raise KeyError(f"unknown {self.what} kind '{kind}' (registered: {known})") from None

    def kinds(self) -> List[str]:
        return sorted(self._items)


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
BLOCKS = _Registry("block arrangement")
EMBEDDINGS = _Registry("embedding")
HEADS = _Registry("output head")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


def build_part(registry: _Registry, spec: PartSpec, runtime) -> Part:
    return registry.get(spec.kind)(spec.params, prefix=spec.prefix, runtime=runtime)
