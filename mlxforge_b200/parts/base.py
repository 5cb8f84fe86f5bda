"""What a model is made of, as data, and the interfaces its parts implement.

A model is a ``ModelSpec``: an embedding, a list of ``LayerSpec`` (each naming its
parts by role -- usually a mixer, a feed-forward and their norms, but a layer may
leave one out or carry further ones -- and the arrangement that runs them, every
one by *kind* with its sizes and constants as parameters), a *schedule*
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
    """One layer: its parts by role and the arrangement (``block``) that runs them.

    The four usual roles have fields of their own; any of them may be None (a layer
    without a feed-forward, an arrangement with one norm).  ``extra`` holds further
    parts as ``(role, family, spec)``, ``family`` being the registry the part is
    built from: "mixer", "feed_forward" or "norm" (a norm after the mixer, a second
    feed-forward, ...).  The arrangement finds all of them under their roles."""

    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    extra: Tuple[Tuple[str, str, PartSpec], ...] = ()

    def part_specs(self) -> List[Tuple[str, str, PartSpec]]:
        """Every part of the layer as (role, family, spec), in a fixed order."""
        usual = (("mixer", "mixer", self.mixer), ("mixer_norm", "norm", self.mixer_norm),
                 ("feed_forward", "feed_forward", self.feed_forward),
                 ("feed_forward_norm", "norm", self.feed_forward_norm))
        out = [(role, family, spec) for role, family, spec in usual if spec is not None]
        seen = {role for role, _, _ in out}
        for role, family, spec in self.extra:
            if role in seen:
                raise ValueError(f"layer names the role '{role}' twice")
            seen.add(role)
            out.append((role, family, spec))
        return out


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
    """Per-request state of fixed size, one tensor of ``shape`` and ``dtype`` (a torch
    dtype's name; 32-bit floats unless said otherwise) per run of the layer, zeroed
    when a request is admitted."""

    shape: Tuple[int, ...]
    tag: str = ""
    dtype: str = "float32"


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
    """Turns integer positions into whatever the mixer applies to queries and keys.

    An encoding implements ``encode`` and knows nothing of pages: the cache lane stores
    keys and values (``KVLane.store``).  One that has a kernel doing both at once (the
    rotary encoding has) overrides ``rotate_and_store`` as well.  The mixer forwards this
    part's ``tensor_specs`` and ``bind``, so an encoding may own tensors."""

    def encode(self, q, k, batch) -> None:
        """Apply the encoding in place.  ``q``: [T, n_heads, head_dim] and ``k``:
        [T, n_kv_heads, head_dim] (views into the step's projections, compute dtype);
        token ``t`` stands at ``batch.positions[t]`` of its sequence."""
        raise NotImplementedError

    def rotate_and_store(self, qkv, batch, q_out, lane, n_heads, n_kv_heads, writes_cache: bool) -> None:
        """``qkv``: [T, (n_heads + 2 n_kv_heads) * head_dim], the step's projections side by
        side.  Leaves the encoded queries in ``q_out`` [T, n_heads * head_dim] and, if
        ``writes_cache``, the encoded keys and the values in the lane's pages.  The default
        encodes in place and lets the lane store."""
        T, hd = qkv.shape[0], lane.need.head_dim
        nq, nk = n_heads * hd, n_kv_heads * hd
        self.encode(qkv[:, :nq].view(T, n_heads, hd), qkv[:, nq:nq + nk].view(T, n_kv_heads, hd), batch)
        lane.store(qkv, batch, q_out, n_heads, n_kv_heads, writes_cache, precise=self.rt.precise)


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
    that the add can be fused with the next norm.

    ``by_role`` holds the layer's parts under the roles its ``LayerSpec`` named; the
    four usual ones are also attributes (None where the layer has none).  An
    arrangement says with ``roles`` which parts it needs and fails at build time,
    not in the middle of a step, when a layer does not bring them."""

    roles: Tuple[str, ...] = ()

    def __init__(self, by_role: Dict[str, Part], runtime: "Any"):
        self.by_role = dict(by_role)
        missing = [r for r in self.roles if r not in self.by_role]
        if missing:
            raise ValueError(f"{type(self).__name__} needs parts in the roles {missing}, the layer has "
                             f"{sorted(self.by_role)}")
        self.mixer = self.by_role.get("mixer")
        self.mixer_norm = self.by_role.get("mixer_norm")
        self.feed_forward = self.by_role.get("feed_forward")
        self.feed_forward_norm = self.by_role.get("feed_forward_norm")
        self.rt = runtime

    def parts(self) -> List[Part]:
        return list(self.by_role.values())

    def cache_need(self) -> CacheNeed:
        """What this layer keeps per request: its mixer's need."""
        return self.mixer.cache_need() if self.mixer is not None else None

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


FAMILIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS}


def build_layer(spec: LayerSpec, runtime) -> Block:
    """The layer's parts, each from its family's registry, in the arrangement it names."""
    by_role = {}
    for role, family, part in spec.part_specs():
        if family not in FAMILIES:
            raise KeyError(f"role '{role}': unknown family '{family}' (one of {sorted(FAMILIES)})")
        by_role[role] = build_part(FAMILIES[family], part, runtime)
    return BLOCKS.get(spec.block)(by_role, runtime)
