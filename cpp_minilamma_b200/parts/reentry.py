"""Re-entry into a stretch of layers: the stream is mixed with the embedding's output before a pass.

    x <- W_in [x ; x0] + step[r]           x0 the stream as the embedding left it, r the number of the pass

A model that runs a stretch of its layers several times gives every pass the original input again, and a vector
of its own so that the passes can tell each other apart.  W_in is [D, 2 D] with x's columns first; `step` is
[passes, D].  The sum x + (pending output of the layer before) is formed in float32 and the result is written to
the float32 stream; the product itself runs in the activation dtype like every other projection.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, PendingSum, PreNormed, StreamOp, WeightSpec, register_part
from .linear import Linear


class Reentry(StreamOp):
    """params: passes, names {"in": tensor name of W_in, "step": tensor name of the per-pass vectors}, optional (True:
    a folder may leave the tensors out - a model whose stretch is empty never enters it)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.passes = int(params["passes"])
        self.names = dict(params["names"])
        self.optional = bool(params.get("optional", False))
        self.linear: Optional[Linear] = None
        self.step_vectors: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        D = self.ctx.hidden_size
        return [WeightSpec(self.names["in"], (D, 2 * D), optional=self.optional),
                WeightSpec(self.names["step"], (self.passes, D), kind="vector", init="normal", optional=self.optional)]

    def bind(self, store) -> None:
        self.linear = Linear(store.take(self.names["in"]), self.names["in"])
        self.step_vectors = store.take(self.names["step"])

    def parameter_bytes(self) -> int:
        return self.linear.parameter_bytes() + self.ctx.hidden_size * 4

    def forward(self, step, x, pending, x0, pass_number: int) -> None:
        if not 0 <= pass_number < self.passes:
            raise ValueError(f"{self.names['in']}: pass {pass_number} of {self.passes}")
        if isinstance(pending, PreNormed):
            pending = None  # the part before has added its output to the stream already
        if isinstance(pending, PendingSum):
            raise RuntimeError(f"{self.names['in']}: two pending outputs in front of a re-entry are not supported")
        T, D = x.shape
        both = step.ws.buffer("reentry.in", (T, 2 * D), self.ctx.act_dtype)
        K.stream_concat(x, pending, x0, both)
        self.linear.forward(step, both, "reentry.out", out_dtype=torch.float32, out=x)
        K.add_bias(x, self.step_vectors[pass_number])


register_part("stream_op", "reentry", Reentry)
