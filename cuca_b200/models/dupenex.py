"""The Dupenex decoder as a `ModelSpec`.

Every layer is a mixer and an optional feed-forward, each behind an RMSNorm. With `streams` in the configuration the
layers carry that many copies of the residual stream (`hyper_connections` blocks: a sublayer reads a weighted sum of
the copies and writes into all of them; the model's output is the copies' sum), else the plain pre-norm residual.
Mixers: `channel_delta` (the `gated_delta` part: a delta rule with a decay per key channel behind short convolutions)
and `parallel` (the `parallel` part around a sliding-window `attention` with rotary adjacent pairs, value heads of
their own size and an output gate, and an `mlstm` matrix memory; each side's output is normed and the two are
averaged). Feed-forwards: dense SwiGLU, or `routed` experts with a squared-relu activation. A stretch of layers
may run several passes in a row with the same weights, each run with a cache and state of its own, nothing between.
Tensor names: `embed`, `head`, `final.norm` and per layer i `l<i>.norm1|norm2`, `l<i>.hc1|hc2.in|out|mix`,
`l<i>.mix.*`, `l<i>.mlp.*`.
"""
from __future__ import annotations

from ..config.dupenex_config import MAX_POSITIONS, DupenexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, Run


def _mixer_spec(layer, E: int, eps: float, p: str) -> PartSpec:
    m = layer.mixer
    if layer.type == "channel_delta":
        return PartSpec("gated_delta",
                        {"width": E, "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                         "conv": m.conv, "eps": eps, "decay_rank": m.decay_rank, "gate_rank": m.gate_rank},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "q_conv": p + "q.conv", "k_conv": p + "k.conv",
                         "v_conv": p + "v.conv", "b": p + "b", "A_log": p + "A_log", "dt_bias": p + "dt_bias",
                         "a1": p + "a1", "a2": p + "a2", "g1": p + "g1", "g2": p + "g2", "norm": p + "norm",
                         "o": p + "o"})
    if layer.type == "parallel":
        a, r = m.left, m.right
        position = None
        if a.rot_dims:
            position = PartSpec("rope", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base,
                                         "pairs": "adjacent"})
        lp, rp = p + "left.", p + "right."
        left = PartSpec("attention",
                        {"width": E, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim,
                         "v_head_dim": a.vdim, "window": a.window, "scale": a.scale, "position": position, "gate": True},
                        {"q": lp + "q", "k": lp + "k", "v": lp + "v", "g": lp + "g", "o": lp + "o"})
        right = PartSpec("mlstm", {"width": E, "heads": r.heads, "dim": r.dim, "vdim": r.vdim, "gate_cap": r.gate_cap,
                                   "eps": eps},
                         {"q": rp + "q", "k": rp + "k", "v": rp + "v", "g": rp + "g", "i": rp + "i",
                          "i_bias": rp + "i.b", "f": rp + "f", "f_bias": rp + "f.b", "norm": rp + "norm", "o": rp + "o"})
        return PartSpec("parallel", {"width": E, "eps": eps, "scale": 0.5, "left": left, "right": right},
                        {"left_out": lp + "out", "right_out": rp + "out"})
    raise ValueError(layer.type)


def _mlp_spec(mlp, E: int, p: str) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"width": E, "inner": mlp.ff}, {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    names = {"router": p + "router"}
    for e in range(mlp.experts):
        names[f"up{e}"] = f"{p}e{e}.up"
        names[f"down{e}"] = f"{p}e{e}.down"
    return PartSpec("routed", {"width": E, "inner": mlp.ff, "experts": mlp.experts, "top": mlp.top, "act": "relu2"}, names)


def dupenex_spec(cfg: DupenexConfig) -> ModelSpec:
    E, eps, S = cfg.width, cfg.eps, cfg.streams

    def norm(name):
        return PartSpec("rmsnorm", {"width": E, "eps": eps}, {"weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ff = layer.mlp is not None
        if S is None:
            block = PartSpec("pre_norm")
        else:
            names = {"read1": p + "hc1.in", "write1": p + "hc1.out", "mix1": p + "hc1.mix"}
            if has_ff:
                names.update({"read2": p + "hc2.in", "write2": p + "hc2.out", "mix2": p + "hc2.mix"})
            block = PartSpec("hyper_connections", {"width": E, "streams": S, "eps": eps}, names)
        layers.append(LayerSpec(block=block, mixer=_mixer_spec(layer, E, eps, p + "mix."), mixer_norm=norm(p + "norm1"),
                                feed_forward=_mlp_spec(layer.mlp, E, p + "mlp.") if has_ff else None,
                                ffn_norm=norm(p + "norm2") if has_ff else None))
    schedule = [Run(layer=i, cache=n, owns=True) for n, i in enumerate(cfg.run_order())]
    final = norm("final.norm") if S is None else PartSpec("rmsnorm_streams", {"width": E, "eps": eps, "streams": S},
                                                          {"weight": "final.norm"})
    no_ff = {i for i, layer in enumerate(cfg.layers) if layer.mlp is None}
    return ModelSpec(
        architecture="Dupenex", vocab_size=cfg.vocab, width=E, max_positions=MAX_POSITIONS,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "width": E}, {"weight": "embed"}),
        layers=layers, schedule=schedule, final_norm=final,
        head=PartSpec("head", {"vocab": cfg.vocab, "width": E}, {"weight": "head"}),
        # a layer without feed-forward has no use for what stands around one, should a file carry it
        ignorable_tensor=lambda name: any(name.startswith(f"l{i}.norm2") or name.startswith(f"l{i}.hc2.") for i in no_ff),
        streams=S)


@register_architecture("Dupenex")
def build_dupenex(config_json: dict) -> ModelSpec:
    return dupenex_spec(DupenexConfig.from_json(config_json))
