"""Typed configuration of the Bananex decoder, read from its config.json.

The file is nested: `layers` is a list with one entry per layer (`type` names the mixer, `mixer` holds the mixer's
sizes and constants, `mlp` the feed-forward's or null), `loop` (optional) names a stretch of layers that runs
several times, `norm.eps`, `logit_scale`, `vocab`, `width`. Every size and constant comes from there; a key the file
does not have switches its feature off where that makes sense (no `loop`: every layer once; no `mask`: every earlier
key is seen; `mlp` null: no feed-forward) and is an error otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .model_config import ConfigError

MIXER_TYPES = ("latent_attention", "mingru", "mamba2")
MAX_POSITIONS = 1 << 20  # the file gives no longest sequence: nothing in the model depends on one


def _get(obj, key, kind, where):
    if not isinstance(obj, dict) or obj.get(key) is None:
        raise ConfigError(f"config.json is missing `{where}.{key}`")
    try:
        return kind(obj[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json `{where}.{key}` = {obj[key]!r} is not {kind.__name__}") from e


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: Optional[float]
    window: Optional[int]
    rot_base: float
    rot_dims: int

    @staticmethod
    def from_json(m, where):
        rot = m.get("rot") if isinstance(m, dict) else None
        rot_dim = _get(m, "rot_dim", int, where)
        mask = m.get("mask")
        c = LatentAttentionConfig(
            heads=_get(m, "heads", int, where), dim=_get(m, "dim", int, where), rot_dim=rot_dim,
            vdim=_get(m, "vdim", int, where), kv_rank=_get(m, "kv_rank", int, where),
            scale=float(m["scale"]) if m.get("scale") is not None else None,
            window=_get(mask, "size", int, where + ".mask") if mask else None,
            rot_base=_get(rot, "base", float, where + ".rot") if rot else 10000.0,
            rot_dims=_get(rot, "dims", int, where + ".rot") if rot else 0)
        if min(c.heads, c.dim, c.vdim, c.kv_rank) < 1 or c.rot_dim < 0:
            raise ConfigError(f"config.json `{where}`: sizes must be positive")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.rot_dim:
            raise ConfigError(f"config.json `{where}.rot.dims` = {c.rot_dims} must be even and at most rot_dim")
        if c.window is not None and c.window < 1:
            raise ConfigError(f"config.json `{where}.mask.size` must be at least 1")
        return c


@dataclass(frozen=True)
class MinGRUConfig:
    width: int

    @staticmethod
    def from_json(m, where):
        c = MinGRUConfig(width=_get(m, "width", int, where))
        if c.width < 1:
            raise ConfigError(f"config.json `{where}.width` must be positive")
        return c


@dataclass(frozen=True)
class Mamba2Config:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @staticmethod
    def from_json(m, where):
        c = Mamba2Config(heads=_get(m, "heads", int, where), vdim=_get(m, "vdim", int, where),
                         state=_get(m, "state", int, where), groups=_get(m, "groups", int, where),
                         conv=_get(m, "conv", int, where), norm_groups=_get(m, "norm_groups", int, where))
        if min(c.heads, c.vdim, c.state, c.groups, c.conv, c.norm_groups) < 1:
            raise ConfigError(f"config.json `{where}`: sizes must be positive")
        if c.heads % c.groups:
            raise ConfigError(f"config.json `{where}`: {c.groups} groups do not divide {c.heads} heads")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"config.json `{where}`: {c.norm_groups} norm groups do not divide heads * vdim")
        return c


_MIXERS = {"latent_attention": LatentAttentionConfig, "mingru": MinGRUConfig, "mamba2": Mamba2Config}


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int

    @staticmethod
    def from_json(m, where):
        kind = str(m.get("kind", "dense"))
        if kind != "dense":
            raise ConfigError(f"config.json `{where}.kind` = `{kind}`; this engine knows: dense")
        c = DenseMlpConfig(ff=_get(m, "ff", int, where))
        if c.ff < 1:
            raise ConfigError(f"config.json `{where}.ff` must be positive")
        return c


@dataclass(frozen=True)
class BananexLayer:
    type: str
    mixer: object
    mlp: Optional[DenseMlpConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BananexConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: tuple
    loop: Optional[LoopConfig]

    @staticmethod
    def from_json(cfg: dict) -> "BananexConfig":
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
            out.append(BananexLayer(kind, _MIXERS[kind].from_json(entry["mixer"], where + ".mixer"),
                                    DenseMlpConfig.from_json(mlp, where + ".mlp") if mlp else None))
        loop = None
        if cfg.get("loop"):
            lp = cfg["loop"]
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"), _get(lp, "times", int, "loop"))
            if not 0 <= loop.start <= loop.stop <= len(out) or loop.times < 1:
                raise ConfigError(f"config.json `loop` = {lp!r} does not fit {len(out)} layers")
        c = BananexConfig(vocab=_get(cfg, "vocab", int, ""), width=_get(cfg, "width", int, ""),
                          eps=_get(cfg.get("norm"), "eps", float, "norm"),
                          logit_scale=float(cfg["logit_scale"]) if cfg.get("logit_scale") is not None else 1.0,
                          layers=tuple(out), loop=loop)
        if c.vocab < 1 or c.width < 1:
            raise ConfigError("config.json `vocab` and `width` must be positive")
        return c

    def run_order(self) -> list:
        """[(layer, pass number or None)]: the layers before the loop, the looped stretch `times` times, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        order = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            order += [(i, t) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, n)]
