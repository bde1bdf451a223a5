"""Dense SwiGLU feed-forward: y = down(silu(gate f) * (up f))
(src/provider/local/model/cpu.rs:3554-3565). gate and up are stacked into one
weight at load so one contraction with a SwiGLU epilogue yields the activation
(the reference accepts the stacked form too: model/cpu.rs:3131-3136)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, TensorNeed, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """params: width, inner. tensors: gate [inner, width], up [inner, width], down [width, inner]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.w_gate_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        return {t["gate"]: TensorNeed((self.inner, self.width)), t["up"]: TensorNeed((self.inner, self.width)),
                t["down"]: TensorNeed((self.width, self.inner))}

    def load(self, get):
        t = self.spec.tensors
        self.w_gate_up = torch.cat([get(t["gate"]), get(t["up"])], dim=0).contiguous()
        self.w_down = get(t["down"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        act = self.rt.linear(h, self.w_gate_up, epilogue=ops.EPI_SWIGLU)
        self.rt.stream(stream).add_linear(act, self.w_down)


@register_feed_forward("dense_act")
class DenseActivation(FeedForward):
    """y = down(act(up f + b_up)) + b_down with act the exact (erf) GELU or its tanh form.
    params: width, inner, act ("gelu" | "gelu_tanh"), bias (bool). tensors: up [inner, width], down [width, inner]
    and, with bias, up_bias [inner], down_bias [width]."""

    graph_safe = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        self.act = str(spec.params.get("act", "gelu"))
        if self.act not in ("gelu", "gelu_tanh"):
            raise ValueError(f"dense feed-forward: activation `{self.act}` is unknown; known: gelu, gelu_tanh")
        self.bias = bool(spec.params.get("bias", True))
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["up"]: TensorNeed((self.inner, self.width)), t["down"]: TensorNeed((self.width, self.inner))}
        if self.bias:
            out[t["up_bias"]] = TensorNeed((self.inner,))
            out[t["down_bias"]] = TensorNeed((self.width,))
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_up, self.w_down = get(t["up"]), get(t["down"])
        if self.bias:
            self.b_up, self.b_down = get(t["up_bias"]), get(t["down_bias"])

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_up, self.w_down, self.b_up, self.b_down)
                   if w is not None)

    def forward(self, h, stream, step) -> None:
        a = self.rt.linear(h, self.w_up, bias=self.b_up)
        ops.gelu_(a, tanh_form=self.act == "gelu_tanh")
        self.rt.stream(stream).add_linear(a, self.w_down, bias=self.b_down)
