"""The typed description of a model that the engine builds from.

An architecture's ``config.json`` is parsed by its own adapter into a
:class:`ModelSpec`.  Nothing below the adapter knows which architecture it is
in: a block is a list of :class:`PartSpec` (``kind`` + parameters) and the
engine looks every ``kind`` up in the part registries.  The order in which
layers run is data too (:class:`ScheduleEntry`): it may name a layer twice, or
let one entry read the cache another entry writes.

The reference keeps the same information in ``ArchitectureSpec``
(src/Inference/architecture_spec.jl:218-364) with a per-layer mixer symbol
(``layer_mixer``, :251-257); here the per-layer choice is the part spec itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: a registered ``kind`` and its sizes and constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: which arrangement, and the parts it is put together from.

    ``prefix`` is the internal name prefix of the layer's tensors
    (``layers.3.``); the architecture adapter maps internal names to the names
    in the checkpoint.
    """

    arrangement: str                 # registered block arrangement, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ff_norm: PartSpec
    prefix: str


@dataclass(frozen=True)
class ScheduleEntry:
    """One step of the layer order.

    ``layer`` indexes ``ModelSpec.blocks``.  ``cache_of`` is ``None`` when the
    entry owns a cache of its own, or the index (into the schedule) of an
    earlier entry whose cache this entry reads without writing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    tie_embedding: bool
    embedding_scale: float = 1.0
    # logits = softcap * tanh(logit_scale * logits / softcap); no cap when None (LFM2 has neither)
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    # internal tensor name -> names it may carry in a checkpoint (first is canonical)
    tensor_names: Mapping[str, Tuple[str, ...]] = field(default_factory=dict)
    # checkpoint tensor names (regular expressions) that are ignored when present
    ignorable_tensors: Tuple[str, ...] = ()
    # token ids the configuration declares (may be None)
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    max_position: Optional[int] = None
    # the architecture's own typed configuration, kept for describe()/bench
    source: Any = None

    def external_names(self, internal: str) -> Tuple[str, ...]:
        names = self.tensor_names.get(internal)
        return names if names else (internal,)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(i) for i in range(n_layers))
