"""A model as data: parts chosen layer by layer, and the order they run in."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

from ..parts.base import PartSpec


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its block arrangement and the parts inside it."""

    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None


@dataclass(frozen=True)
class Run:
    """One entry of the run order: which layer runs and which cache it uses.

    `cache` names a cache (keys/values and state) by number. The entry that
    `owns` it writes it; an entry with `owns=False` reads what an earlier entry
    wrote (its mixer must be built with `shares_cache`). A layer named twice
    runs twice, each run with a cache of its own unless it names a shared one.
    """

    layer: int
    cache: int
    owns: bool = True


@dataclass(frozen=True)
class Between:
    """A run-order entry that is no layer: stream operation `op` (an index into `ModelSpec.stream_ops`) happens to
    the residual stream at this point, with `arg` telling it which of its occasions this is (the pass of a loop)."""

    op: int
    arg: int = 0


@dataclass
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: tuple = ()
    ignorable_tensor: Callable[[str], bool] = field(default=lambda name: False)
    stream_ops: list = field(default_factory=list)  # PartSpecs of what `Between` entries of the schedule name
    streams: Optional[int] = None  # copies of the residual stream the blocks carry side by side (None: the one stream)

    def runs(self):
        """The schedule's layer runs, without what happens between them."""
        return [e for e in self.schedule if isinstance(e, Run)]

    def validate(self) -> None:
        owners = {}
        for i, run in enumerate(self.schedule):
            if isinstance(run, Between):
                if not 0 <= run.op < len(self.stream_ops):
                    raise ValueError(f"run order entry {i} names stream operation {run.op}; the model has "
                                     f"{len(self.stream_ops)}")
                continue
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {run.layer}; the model has {len(self.layers)}")
            if run.owns:
                if run.cache in owners:
                    raise ValueError(f"cache {run.cache} is written by run entries {owners[run.cache]} and {i}")
                owners[run.cache] = i
            elif run.cache not in owners:
                raise ValueError(f"run order entry {i} reads cache {run.cache} before any entry writes it")


def default_schedule(n_layers: int) -> list:
    return [Run(layer=i, cache=i, owns=True) for i in range(n_layers)]
