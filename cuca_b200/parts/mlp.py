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


@register_feed_forward("routed")
class RoutedExperts(FeedForward):
    """Every token goes to the `top` of `experts` small feed-forwards with the largest router logits z = W_r f
    (32-bit), with weights p = softmax of just those `top` logits: y = sum_e p_e down_e(act(up_e f)), act the
    square of relu. The experts' weights are stacked at load (`up` [experts * inner, width], `down` [width,
    experts * inner]). Many tokens: all experts' up-projections in one contraction, the activation weighted per
    expert (0 for the ones a token did not choose), one contraction over (expert, inner) down. Few tokens: only the
    chosen experts' rows are read, a warp per output. Both sum a token's experts in a fixed order.

    params: width, inner, experts, top, act ("relu2"). tensors: router [experts, width], `up{e}` [inner, width] and
    `down{e}` [width, inner] for every expert e."""

    graph_safe = True
    SPARSE_MAX_TOKENS = 32  # up to this many tokens only the chosen experts are read

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        p = spec.params
        self.width, self.inner = int(p["width"]), int(p["inner"])
        self.experts, self.top = int(p["experts"]), int(p["top"])
        if str(p.get("act", "relu2")) != "relu2":
            raise ValueError(f"routed feed-forward: activation `{p.get('act')}` is unknown; known: relu2")
        if not 1 <= self.top <= min(self.experts, ops.MOE_MAX_TOP) or self.experts > ops.MOE_MAX_EXPERTS:
            raise ValueError(f"routed feed-forward: {self.top} of {self.experts} experts is outside what the kernels "
                             f"take (experts <= {ops.MOE_MAX_EXPERTS}, chosen <= {ops.MOE_MAX_TOP})")
        self.w_router = self.w_up = self.w_down = None

    def tensors(self):
        t = self.spec.tensors
        out = {t["router"]: TensorNeed((self.experts, self.width))}
        for e in range(self.experts):
            out[t[f"up{e}"]] = TensorNeed((self.inner, self.width))
            out[t[f"down{e}"]] = TensorNeed((self.width, self.inner))
        return out

    def load(self, get):
        t = self.spec.tensors
        self.w_router = get(t["router"])
        self.w_up = torch.cat([get(t[f"up{e}"]) for e in range(self.experts)], dim=0).contiguous()
        self.w_down = torch.cat([get(t[f"down{e}"]) for e in range(self.experts)], dim=1).contiguous()

    def weight_bytes(self):
        """What a step of several tokens reads at most: the router and every expert once."""
        return sum(w.numel() * w.element_size() for w in (self.w_router, self.w_up, self.w_down))

    def forward(self, h, stream, step) -> None:
        rt, T = self.rt, h.shape[0]
        logits = rt.linear(h, self.w_router, out_dtype=torch.float32)
        idx = torch.empty(T, self.top, dtype=torch.int32, device=rt.device)
        wts = torch.empty(T, self.top, dtype=torch.float32, device=rt.device)
        if T <= self.SPARSE_MAX_TOKENS:
            ops.moe_route(logits, self.top, idx, wts)
            a = rt.empty(T * self.top, self.inner)
            y, fresh = rt.stream(stream).claim()
            ops.moe_sparse(h, self.w_up, self.w_down, idx, wts, a, y, fresh, self.top, self.experts, self.inner)
            return
        spread = torch.empty(T, self.experts, dtype=torch.float32, device=rt.device)
        ops.moe_route(logits, self.top, idx, wts, spread)
        u = rt.linear(h, self.w_up)
        a = torch.empty_like(u)
        ops.moe_act_dense(u, spread, a, self.experts, self.inner)
        rt.stream(stream).add_linear(a, self.w_down)
