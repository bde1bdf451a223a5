"""The Bananex decoder as a `ModelSpec`.

Every layer is a `sandwich_shift` block (a single-number RMSNorm before and after each sublayer, the mixer's input
mixed with the previous token's) around one of three mixers, `latent_attention`, `mingru` or `mamba2`, and an
optional dense GELU feed-forward with biases. A stretch of layers may run several passes with the same weights:
each pass is entered through `loop_entry` (the stream is remixed with the embedding output and a per-pass vector
is added) and each run of a layer has a cache and state of its own. The final norm has a single gain too and the
logits are scaled by `logit_scale`. Tensor names: `embed`, `head`, `final.norm`, `loop.in`, `loop.step`, and per
layer i `l<i>.norm1|norm1b|norm2|norm2b|shift`, `l<i>.mix.*`, `l<i>.mlp.up|up.b|down|down.b`.
"""
from __future__ import annotations

import re

from ..config.bananex_config import MAX_POSITIONS, BananexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import Between, LayerSpec, ModelSpec, Run


def _mixer_spec(layer, E: int, eps: float, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        position = None
        if m.rot_dims:
            position = PartSpec("rope", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                         "pairs": "adjacent"})
        return PartSpec("latent_attention",
                        {"width": E, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                         "kv_rank": m.kv_rank, "window": m.window, "scale": m.scale, "eps": eps, "position": position},
                        {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                         "g": p + "g", "o": p + "o"})
    if layer.type == "mingru":
        return PartSpec("mingru", {"width": E, "inner": m.width},
                        {"z": p + "z", "z_bias": p + "z.b", "x": p + "x", "x_bias": p + "x.b", "g": p + "g",
                         "o": p + "o"})
    if layer.type == "mamba2":
        return PartSpec("mamba2", {"width": E, "heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups,
                                   "conv": m.conv, "norm_groups": m.norm_groups, "eps": eps},
                        {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
                         "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"})
    raise ValueError(layer.type)


def bananex_spec(cfg: BananexConfig) -> ModelSpec:
    E, eps = cfg.width, cfg.eps

    def norm(name):
        return PartSpec("rmsnorm_scalar", {"width": E, "eps": eps}, {"weight": name})

    layers, no_mlp = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"mix": p + "shift", "mixer_post": p + "norm1b"}
        ff = ffn_norm = None
        if layer.mlp is not None:
            names["ffn_post"] = p + "norm2b"
            ff = PartSpec("dense_act", {"width": E, "inner": layer.mlp.ff, "act": "gelu", "bias": True},
                          {"up": p + "mlp.up", "up_bias": p + "mlp.up.b", "down": p + "mlp.down",
                           "down_bias": p + "mlp.down.b"})
            ffn_norm = norm(p + "norm2")
        else:
            no_mlp.append(i)
        layers.append(LayerSpec(block=PartSpec("sandwich_shift", {"width": E, "eps": eps, "post_gain": "scalar"}, names),
                                mixer=_mixer_spec(layer, E, eps, p + "mix."), mixer_norm=norm(p + "norm1"),
                                feed_forward=ff, ffn_norm=ffn_norm))
    schedule, stream_ops = [], []
    looped = cfg.loop is not None and cfg.loop.stop > cfg.loop.start
    if looped:
        stream_ops.append(PartSpec("loop_entry", {"width": E, "times": cfg.loop.times},
                                   {"mix": "loop.in", "step": "loop.step"}))
    for n, (i, t) in enumerate(cfg.run_order()):
        if looped and t is not None and i == cfg.loop.start:
            schedule.append(Between(op=0, arg=t))
        schedule.append(Run(layer=i, cache=n, owns=True))
    # a layer without feed-forward has no use for the norms around one, should a file carry them
    spare = re.compile(r"^l(%s)\.norm2b?$" % "|".join(str(i) for i in no_mlp)) if no_mlp else None
    return ModelSpec(
        architecture="Bananex", vocab_size=cfg.vocab, width=E, max_positions=MAX_POSITIONS,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "width": E}, {"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("head", {"vocab": cfg.vocab, "width": E, "scale": cfg.logit_scale}, {"weight": "head"}),
        # ... nor has a model without a looped stretch any use for the loop's tensors
        ignorable_tensor=lambda name: (bool(spare and spare.match(name))
                                       or (not looped and name in ("loop.in", "loop.step"))),
        stream_ops=stream_ops)


@register_architecture("Bananex")
def build_bananex(config_json: dict) -> ModelSpec:
    return bananex_spec(BananexConfig.from_json(config_json))
