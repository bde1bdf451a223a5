"""Typed configuration of the Dupenex decoder, read from its config.json.

The file is nested: `layers` is a list with one entry per layer (`type` names the mixer, `mixer` holds the mixer's
sizes and constants, `mlp` the feed-forward's or null), `loop` (optional) names a stretch of layers that runs several
times in a row, `streams` (optional) the number of copies of the residual stream that the layers carry side by side,
`norm.eps`, `vocab`, `width`. Every size and constant comes from there (two ranks come from the stored tensors); a key
the file does not have switches its feature off where that makes sense (no `loop`: every layer once; no `streams`:
the plain residual sum; no `mask`: every earlier key is seen; no `rot`: no rotation; `mlp` null: no feed-forward) and
is an error otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .bananex_config import LoopConfig, _get
from .model_config import ConfigError

MIXER_TYPES = ("channel_delta", "parallel")
MAX_POSITIONS = 1 << 20  # the file gives no longest sequence: nothing in the model depends on one


def _positive(where, **sizes):
    for k, v in sizes.items():
        if v < 1:
            raise ConfigError(f"config.json `{where}.{k}` must be positive")


@dataclass(frozen=True)
class ChannelDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: Optional[int]  # only for folders of random weights: a stored model's tensors give the ranks
    gate_rank: Optional[int]

    @staticmethod
    def from_json(m, where):
        heads = _get(m, "heads", int, where)
        c = ChannelDeltaConfig(heads=heads, kv_heads=int(m["kv_heads"]) if m.get("kv_heads") is not None else heads,
                               dim=_get(m, "dim", int, where), vdim=_get(m, "vdim", int, where),
                               conv=_get(m, "conv", int, where),
                               decay_rank=int(m["decay_rank"]) if m.get("decay_rank") else None,
                               gate_rank=int(m["gate_rank"]) if m.get("gate_rank") else None)
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim, conv=c.conv)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json `{where}`: {c.kv_heads} kv_heads do not divide {c.heads} heads")
        return c


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: Optional[float]
    window: Optional[int]
    rot_base: float
    rot_dims: int

    @staticmethod
    def from_json(m, where):
        if not isinstance(m, dict):
            raise ConfigError(f"config.json is missing `{where}`")
        rot, mask = m.get("rot"), m.get("mask")
        heads = _get(m, "heads", int, where)
        dim = _get(m, "dim", int, where)
        c = WindowAttentionConfig(
            heads=heads, kv_heads=int(m["kv_heads"]) if m.get("kv_heads") is not None else heads, dim=dim,
            vdim=int(m["vdim"]) if m.get("vdim") is not None else dim,
            scale=float(m["scale"]) if m.get("scale") is not None else None,
            window=_get(mask, "size", int, where + ".mask") if mask else None,
            rot_base=_get(rot, "base", float, where + ".rot") if rot else 10000.0,
            rot_dims=_get(rot, "dims", int, where + ".rot") if rot else 0)
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json `{where}`: {c.kv_heads} kv_heads do not divide {c.heads} heads")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim:
            raise ConfigError(f"config.json `{where}.rot.dims` = {c.rot_dims} must be even and at most dim")
        if c.window is not None and c.window < 1:
            raise ConfigError(f"config.json `{where}.mask.size` must be at least 1")
        return c


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @staticmethod
    def from_json(m, where):
        if not isinstance(m, dict):
            raise ConfigError(f"config.json is missing `{where}`")
        c = MatrixMemoryConfig(heads=_get(m, "heads", int, where), dim=_get(m, "dim", int, where),
                               vdim=_get(m, "vdim", int, where), gate_cap=_get(m, "gate_cap", float, where))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim)
        if c.gate_cap <= 0:
            raise ConfigError(f"config.json `{where}.gate_cap` must be positive")
        return c


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: MatrixMemoryConfig

    @staticmethod
    def from_json(m, where):
        return ParallelConfig(WindowAttentionConfig.from_json(m.get("left"), where + ".left"),
                              MatrixMemoryConfig.from_json(m.get("right"), where + ".right"))


_MIXERS = {"channel_delta": ChannelDeltaConfig, "parallel": ParallelConfig}


@dataclass(frozen=True)
class MlpConfig:
    kind: str  # "dense" | "moe"
    ff: int  # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0

    @staticmethod
    def from_json(m, where):
        kind = str(m.get("kind", "dense"))
        if kind == "dense":
            c = MlpConfig("dense", _get(m, "ff", int, where))
        elif kind == "moe":
            c = MlpConfig("moe", _get(m.get("expert"), "ff", int, where + ".expert"),
                          _get(m.get("router"), "experts", int, where + ".router"),
                          _get(m.get("router"), "top", int, where + ".router"))
            if not 1 <= c.top <= c.experts:
                raise ConfigError(f"config.json `{where}.router`: top = {c.top} must lie in 1..experts = {c.experts}")
        else:
            raise ConfigError(f"config.json `{where}.kind` = `{kind}`; this engine knows: dense, moe")
        _positive(where, ff=c.ff)
        return c


@dataclass(frozen=True)
class DupenexLayer:
    type: str
    mixer: object
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class DupenexConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]
    layers: tuple
    loop: Optional[LoopConfig]

    @staticmethod
    def from_json(cfg: dict) -> "DupenexConfig":
        layers = cfg.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json `layers` must be a non-empty list")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = _get(entry, "type", str, where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json `{where}.type` = `{kind}`; this engine knows: {', '.join(MIXER_TYPES)}")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"config.json is missing `{where}.mixer`")
            mlp = entry.get("mlp")
            out.append(DupenexLayer(kind, _MIXERS[kind].from_json(entry["mixer"], where + ".mixer"),
                                    MlpConfig.from_json(mlp, where + ".mlp") if mlp else None))
        loop = None
        if cfg.get("loop"):
            lp = cfg["loop"]
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"), _get(lp, "times", int, "loop"))
            if not 0 <= loop.start <= loop.stop <= len(out) or loop.times < 1:
                raise ConfigError(f"config.json `loop` = {lp!r} does not fit {len(out)} layers")
        streams = int(cfg["streams"]) if cfg.get("streams") is not None else None
        if streams is not None and streams < 1:
            raise ConfigError("config.json `streams` must be at least 1")
        c = DupenexConfig(vocab=_get(cfg, "vocab", int, ""), width=_get(cfg, "width", int, ""),
                          eps=_get(cfg.get("norm"), "eps", float, "norm"), streams=streams, layers=tuple(out), loop=loop)
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json `vocab` and `width` must be positive")
        return c

    def run_order(self) -> list:
        """Layer numbers in the order they run: the layers before the loop, the looped stretch `times` times, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        lp = self.loop
        return list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))
