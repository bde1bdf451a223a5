"""Small Bananex configurations with weights that exercise every mechanism, for the engine and for the plain
implementation alike (the same values, bfloat16-rounded, as a folder and as 64-bit arrays)."""
from __future__ import annotations

import copy
import json
from pathlib import Path

import numpy as np
import torch

import plain_bananex


def latent(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=12, base=10000.0, dims=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims},
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def mingru(width=48):
    return {"type": "mingru", "mixer": {"width": width}}


def mamba2(heads=4, vdim=8, state=16, groups=2, conv=4, norm_groups=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def config(layers, width=64, vocab=199, ff=96, loop=None, logit_scale=1.5, eps=1e-5, no_mlp=()):
    out = []
    for i, l in enumerate(layers):
        l = copy.deepcopy(l)
        l["mlp"] = None if i in no_mlp else {"kind": "dense", "ff": ff + 8 * i}
        out.append(l)
    cfg = {"architecture": "Bananex", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "logit_scale": logit_scale, "layers": out}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# sizes that differ in every respect: looped or not, the loop at the start or in the middle, layers without a
# feed-forward, one head / one group / one tap / one norm group, windows of 1 and none, rotation of a part of rot_dim
CONFIGS = {
    "mix": config([latent(), mingru(), mamba2(), latent(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=24, window=5)],
                  loop=(1, 3, 2)),
    "loop0": config([mamba2(heads=2, vdim=16, state=8, groups=1, conv=2, norm_groups=1), latent(window=None, dims=4),
                     mingru(width=40)], width=48, vocab=131, loop=(0, 2, 3), logit_scale=0.7, no_mlp=(1,)),
    "flat": config([mingru(width=72), latent(heads=1, dim=32, rot_dim=4, vdim=16, kv_rank=136, window=1),
                    mamba2(heads=3, vdim=20, state=40, groups=3, conv=1, norm_groups=3),
                    latent(heads=5, dim=12, rot_dim=6, vdim=10, kv_rank=33, window=40, base=250000.0)],
                   width=80, vocab=257, ff=72, logit_scale=1.0, eps=1e-6),
    # latent sizes that the tensor-core attention takes in bfloat16: 64 + 16 and 96 + 32 values per cached row, more
    # heads than one group of 16 holds, a window that ends inside a key tile and none
    "wide": config([latent(heads=5, dim=16, rot_dim=16, vdim=16, kv_rank=64, window=23, scale=0.6), mamba2(),
                    latent(heads=18, dim=8, rot_dim=32, vdim=8, kv_rank=96, window=None, scale=0.5), mingru(24)],
                   width=72, vocab=211, loop=(2, 4, 2)),
    "once": config([latent(window=17), mamba2(conv=7, state=6, groups=4, heads=4, vdim=12)], width=56, vocab=97,
                   loop=(0, 2, 1)),
}


def make_weights(cfg: dict, seed: int) -> dict:
    """name -> bfloat16 tensor (int32 for none). Matrices N(0, 1/fan_in) so activations stay of order one; norm gains
    1 + N(0, 0.2); shift mixes U(0, 1); decays, step sizes and biases spread so that no mechanism is near a no-op."""
    from cuca_b200.config.registry import build_spec
    from cuca_b200.models.model import Model

    needs = Model(build_spec(cfg), runtime=None).tensor_needs()
    rng = np.random.default_rng(seed)
    out = {}
    for name, need in sorted(needs.items()):
        shape = tuple(need.shape)
        if name.endswith(".shift"):
            v = rng.uniform(0.0, 1.0, shape)
        elif name.endswith("A_log"):
            v = rng.uniform(-1.5, 1.0, shape)
        elif name.endswith("dt_bias"):
            v = rng.uniform(-2.0, 1.0, shape)
        elif name.endswith(".D"):
            v = rng.normal(1.0, 0.3, shape)
        elif name.endswith(".conv"):
            v = rng.normal(0.0, 0.5, shape)
        elif need.init == "ones":
            v = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name.endswith(".b") or name == "loop.step":
            v = rng.normal(0.0, 0.3, shape)
        elif name in ("embed",):
            v = rng.normal(0.0, 1.0, shape)
        else:
            v = rng.normal(0.0, 1.0, shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16)
    return out


def write_model(folder, cfg: dict, weights: dict) -> Path:
    from cuca_b200.weights.safetensors_io import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    write_safetensors(folder / "model.safetensors", weights)
    return folder


def plain_weights(weights: dict) -> dict:
    return {k: v.to(torch.float64).numpy() for k, v in weights.items()}


class Oracle:
    """Whole-sequence logits of the plain implementation, cached per request (the interface `replay_util.compare`
    takes)."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg, self.w = cfg, plain_weights(weights)
        self._cache = {}

    def logits(self, rid: str, tokens: list) -> np.ndarray:
        if rid not in self._cache:
            self._cache[rid] = plain_bananex.forward(self.cfg, self.w, tokens)
        return self._cache[rid]

    def tolerance(self, dtype: str, requests: dict) -> float:
        """What a replay may differ by, relative to a row's largest logit. 32-bit: a fixed small number. bfloat16:
        three times what rounding alone does to these very requests (the plain implementation run once more with
        everything that enters a contraction, and the cached latent, rounded to bfloat16), and at least 3e-2."""
        if dtype == "float32":
            return 2e-5
        worst = 0.0
        for rid, tokens in requests.items():
            key = ("rounded", rid)
            if key not in self._cache:
                plain_bananex.ROUND = bf16_round
                try:
                    self._cache[key] = plain_bananex.forward(self.cfg, self.w, tokens)
                finally:
                    plain_bananex.ROUND = None
            exact = self.logits(rid, tokens)
            err = np.abs(self._cache[key] - exact).max(axis=1) / np.abs(exact).max(axis=1)
            worst = max(worst, float(err.max()))
        return max(3e-2, 3.0 * worst)


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(torch.float64).numpy()


def random_tokens(n: int, vocab: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
