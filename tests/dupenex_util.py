"""Small Dupenex configurations with weights that exercise every mechanism, for the engine and for the plain
implementation alike (the same values, bfloat16-rounded, as a folder and as 64-bit arrays)."""
from __future__ import annotations

import copy

import numpy as np
import torch

import plain_dupenex
from bananex_util import bf16_round, plain_weights, random_tokens, write_model  # noqa: F401  (shared helpers)


def delta(heads=4, kv_heads=2, dim=24, vdim=20, conv=3, decay_rank=6, gate_rank=10):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                                               "conv": conv, "decay_rank": decay_rank, "gate_rank": gate_rank}}


def par(heads=4, kv_heads=2, dim=16, vdim=24, window=12, base=10000.0, dims=8, scale=None, r_heads=3, r_dim=12,
        r_vdim=20, cap=6.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        left["mask"] = {"size": window}
    if dims:
        left["rot"] = {"base": base, "dims": dims}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim,
                                                                 "gate_cap": cap}}}


def dense(ff=72):
    return {"kind": "dense", "ff": ff}


def moe(ff=24, experts=6, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def config(layers, mlps, width=64, vocab=199, streams=3, loop=None, eps=1e-5):
    out = []
    for l, m in zip(layers, mlps):
        l = copy.deepcopy(l)
        l["mlp"] = copy.deepcopy(m)
        out.append(l)
    cfg = {"architecture": "Dupenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# sizes that differ in every respect: copies of the stream (none, 1, 2, 3, 5), looped or not and where, layers
# without a feed-forward, key heads shared or not, one head, 1 to 5 taps, windows of 1, 5, 12, 33 and none, rotation of
# all, half or none of a head, values wider and narrower than keys, one expert of one, all experts chosen
CONFIGS = {
    "mix": config([delta(), par(), delta(heads=2, kv_heads=2, dim=16, vdim=40, conv=4), par(window=5, dims=16, vdim=8)],
                  [dense(), moe(), moe(ff=16, experts=5, top=5), dense(40)], loop=(1, 3, 2)),
    "plain": config([par(window=None, dims=0, heads=3, kv_heads=3, r_heads=1), delta(heads=3, kv_heads=1, conv=1),
                     delta(heads=1, kv_heads=1, dim=40, vdim=8, conv=2)],
                    [None, moe(ff=32, experts=3, top=1), dense(56)], width=48, vocab=131, streams=None),
    "one": config([delta(dim=36, vdim=12, conv=5, kv_heads=4), par(heads=1, kv_heads=1, dim=32, vdim=16, window=1, dims=32,
                                                                    r_heads=2, r_dim=20, r_vdim=8, cap=2.5)],
                  [moe(ff=8, experts=1, top=1), None], width=40, vocab=97, streams=1, loop=(0, 2, 3)),
    # (its attention is one the tensor-core kernels take in bfloat16: values twice as wide as keys of 64)
    "wide": config([par(heads=6, kv_heads=2, dim=64, vdim=128, window=33, dims=32, base=250000.0, r_heads=2, r_dim=96,
                        r_vdim=40, cap=15.0), delta(heads=4, kv_heads=2, dim=128, vdim=96, conv=4, decay_rank=16,
                                                    gate_rank=8), delta(heads=2, dim=48, vdim=72, kv_heads=1)],
                   [moe(ff=40, experts=16, top=3), dense(136), moe(ff=24, experts=4, top=2)], width=96, vocab=257,
                   streams=5, loop=(1, 2, 2), eps=1e-6),
    "two": config([delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=2), delta()], [dense(48), dense(48)], width=56,
                  vocab=89, streams=2),
}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> bfloat16 tensor. Matrices N(0, 1/fan_in) so activations stay of order one; norm gains 1 + N(0, 0.2);
    the copies' read, write and mix tables away from 0, 1 and the unit matrix; decays and gate biases spread so that
    no mechanism is near a no-op; router rows large so that few choices are close calls."""
    from cuca_b200.config.registry import build_spec
    from cuca_b200.models.model import Model

    needs = Model(build_spec(cfg), runtime=None).tensor_needs()
    rng = np.random.default_rng(seed)
    out = {}
    for name, need in sorted(needs.items()):
        shape = tuple(need.shape)
        if ".hc" in name and name.endswith(".mix"):
            v = np.eye(shape[0]) * 0.8 + rng.normal(0.0, 0.25, shape)
        elif ".hc" in name and name.endswith(".in"):
            v = rng.uniform(0.3, 1.0, shape) * rng.choice([-1.0, 1.0], shape, p=[0.2, 0.8])
        elif ".hc" in name and name.endswith(".out"):
            v = rng.normal(0.8, 0.4, shape)
        elif name.endswith("A_log"):
            v = rng.uniform(-1.5, 1.0, shape)
        elif name.endswith("dt_bias"):
            v = rng.uniform(-2.0, 1.0, shape)
        elif name.endswith(".conv"):
            v = rng.normal(0.0, 0.5, shape)
        elif name.endswith(".f.b"):
            v = rng.normal(2.0, 1.0, shape)
        elif name.endswith(".i.b"):
            v = rng.normal(0.0, 1.0, shape)
        elif need.init == "ones":
            v = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name.endswith(".router"):
            v = rng.normal(0.0, 3.0, shape) / np.sqrt(shape[-1])
        elif name.endswith(".right.i") or name.endswith(".right.f"):
            v = rng.normal(0.0, 2.0, shape) / np.sqrt(shape[-1])
        elif name == "embed":
            v = rng.normal(0.0, 1.0, shape)
        else:
            v = rng.normal(0.0, 1.0, shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16)
    return out


class Oracle:
    """Whole-sequence logits of the plain implementation, cached per request (the interface `replay_util.compare`
    takes)."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg, self.w = cfg, plain_weights(weights)
        self._cache = {}

    def logits(self, rid: str, tokens: list) -> np.ndarray:
        if rid not in self._cache:
            self._cache[rid] = plain_dupenex.forward(self.cfg, self.w, tokens)
        return self._cache[rid]

    def tolerance(self, dtype: str, requests: dict) -> float:
        """What a replay may differ by, relative to a row's largest logit. 32-bit: a fixed small number. bfloat16:
        three times what rounding alone does to these very requests (the plain implementation run once more with
        everything that enters a contraction, and the cached keys and values, rounded to bfloat16), at least 3e-2."""
        if dtype == "float32":
            return 1e-4
        errs = []
        for rid, tokens in requests.items():
            key = ("rounded", rid)
            if key not in self._cache:
                plain_dupenex.ROUND = bf16_round
                try:
                    self._cache[key] = plain_dupenex.forward(self.cfg, self.w, tokens)
                finally:
                    plain_dupenex.ROUND = None
            exact = self.logits(rid, tokens)
            errs.append(np.abs(self._cache[key] - exact).max(axis=1) / np.abs(exact).max(axis=1))
        # the median row: a routed layer takes another expert here and there once its input is rounded, and such a
        # row's error says nothing about rounding
        return max(3e-2, 3.0 * float(np.median(np.concatenate(errs))) * 2.0)


def compare(steps, got, requests, oracle, dtype, allow=0.10, tol32=None):
    """`replay_util.compare` for a model with routed layers: in bfloat16 a token whose router logits nearly tie at
    the cut may go to another expert than in the plain implementation (and what it then leaves in the layers' states
    and keys moves the tokens after it a little), so up to `allow` of the wanted places may be off by more than the
    tolerance while the median place stays well inside it (never in 32-bit, and never by a non-finite value)."""
    import replay_util as ru
    tol = oracle.tolerance(dtype, requests)
    if dtype == "float32":
        return ru.compare(steps, got, requests, oracle, tol32 or tol)
    pos = {rid: 0 for rid in requests}
    errs = []
    for s in steps:
        row = 0
        for e in s["entries"]:
            ref = oracle.logits(e["id"], requests[e["id"]])
            for w in e.get("want", []):
                r, g = ref[pos[e["id"]] + w], got[s["step"]][row]
                assert np.isfinite(g).all(), (s["step"], e["id"])
                errs.append((float(np.abs(g - r).max()) / float(np.abs(r).max()), s["step"], e["id"], pos[e["id"]] + w))
                row += 1
            pos[e["id"]] += len(e["tokens"])
    over = [x for x in errs if x[0] > tol]
    assert len(over) <= max(1, allow * len(errs)), f"{len(over)} of {len(errs)} places over {tol:.2e}; first: {over[:3]}"
    assert float(np.median([x[0] for x in errs])) < 0.5 * tol
    return max(x[0] for x in errs)
