"""Two mixers side by side on the same input: out = c (n(left(h)) * w_l + n(right(h)) * w_r), each output
RMS-normed over the model's width with a weight of its own before they are joined."""
from __future__ import annotations

import dataclasses

from ..kernels import ops
from ..runtime import ResidualStream
from .base import MIXERS, CacheNeeds, Mixer, StateNeeds, TensorNeed, register_mixer


def _named(state, prefix: str) -> dict:
    if state is None:
        return {}
    if isinstance(state, StateNeeds):
        return {prefix: state}
    return {f"{prefix}.{k}": v for k, v in state.items()}


@register_mixer("parallel")
class ParallelMixers(Mixer):
    """params: width, eps, scale (c, default 1/2), left, right (the `PartSpec`s of the two mixers).
    tensors: left_out [width], right_out [width]. At most one of the two may keep paged keys and values; their
    per-request states live side by side in the layer run's slot, named `left.*` and `right.*`."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.eps = int(p["width"]), float(p["eps"])
        self.scale = float(p.get("scale", 0.5))
        self.sides = {name: MIXERS.get(p[name].kind)(p[name], runtime) for name in ("left", "right")}
        self.w_left = self.w_right = None

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.sides.values())

    def cache_needs(self):
        needs = {name: m.cache_needs() for name, m in self.sides.items()}
        kvs = [n.kv for n in needs.values() if n.kv is not None]
        if len(kvs) > 1:
            raise ValueError("parallel mixers: only one of the two may keep paged keys and values")
        state = {}
        for name, n in needs.items():
            state.update(_named(n.state, name))
        return CacheNeeds(kv=kvs[0] if kvs else None, state=state or None)

    def tensors(self):
        t = self.spec.tensors
        out = {t["left_out"]: TensorNeed((self.width,), keep_fp32=True, init="ones"),
               t["right_out"]: TensorNeed((self.width,), keep_fp32=True, init="ones")}
        for m in self.sides.values():
            out.update(m.tensors())
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_left, self.w_right = get(t["left_out"]), get(t["right_out"])
        for m in self.sides.values():
            m.load(get)

    def prepare(self, context_length: int) -> None:
        for m in self.sides.values():
            m.prepare(context_length)

    def weight_bytes(self):
        return (self.w_left.numel() + self.w_right.numel()) * 4 + sum(m.weight_bytes() for m in self.sides.values())

    def _view(self, cache, name: str):
        """The side's share of the layer run's cache: the pages if it is the one that keeps them, its own states."""
        needs = self.sides[name].cache_needs()
        state = cache.state if isinstance(cache.state, dict) else {}
        if isinstance(needs.state, StateNeeds):
            mine = state.get(name)
        else:
            mine = {k[len(name) + 1:]: v for k, v in state.items() if k.startswith(name + ".")} or None
        if needs.kv is None:
            return dataclasses.replace(cache, k=None, v=None, tables=None, state=mine)
        return dataclasses.replace(cache, state=mine)

    def forward(self, h, stream, step, cache) -> None:
        rt, rows = self.rt, h.shape[0]
        outs = {}
        for name, m in self.sides.items():
            y = ResidualStream.unwritten(rt, rows, self.width)
            m.forward(h, y, step, self._view(cache, name))
            outs[name] = y.data
        stream = rt.stream(stream)
        x, fresh = stream.claim()
        ops.pair_norm_add(x, outs["left"], outs["right"], self.w_left, self.w_right, self.scale, self.eps, store=fresh)
