"""Operations on the whole residual stream between layers (`StreamOp`)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import StreamOp, TensorNeed, register_stream_op


@register_stream_op("loop_entry")
class LoopEntry(StreamOp):
    """Entering pass t of a stretch of layers that runs several times with the same weights:
    x <- W [x; e] + s_t, with e the embedding output and s_t row t of a table.
    params: width, times. tensors: mix [width, 2 width] (x's columns first), step [times, width]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.times = int(spec.params["times"])
        self.w = self.steps = None

    def tensors(self):
        t = self.spec.tensors
        return {t["mix"]: TensorNeed((self.width, 2 * self.width)), t["step"]: TensorNeed((self.times, self.width))}

    def load(self, get):
        t = self.spec.tensors
        self.w, self.steps = get(t["mix"]), get(t["step"])

    def weight_bytes(self):
        return self.w.numel() * self.w.element_size() + self.width * self.steps.element_size()

    def forward(self, stream, origin, step, arg: int) -> None:
        rt = self.rt
        x = stream.data
        both = rt.empty(x.shape[0], 2 * self.width)
        ops.concat2(x, origin, both)
        new = torch.empty_like(x)
        ops.gemm(both, self.w, new, ops.EPI_STORE, self.steps[arg], rt.err)
        stream.replace(new)
