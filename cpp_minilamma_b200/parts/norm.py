"""RMSNorm and layer norm, each fused with the residual add that precedes it.

y_i = x_i * w_i / sqrt(mean_j(x_j^2) + eps): eps inside the root, the weight multiplies
(no 1 + w), no bias - src/ops.cc:95-110.  The residual stream x is float32; the add of
the previous part's output and the norm are one kernel.

`layer_norm` (not in the reference): y_i = (x_i - mean) / sqrt(var + eps) * w_i + b_i with var the mean of the
squared deviations; weight and bias are tensors of their own.  It has no factor that the products around it could
apply, so it is never folded away (`prenorm_weight` stays None).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import kernels as K
from .base import BuildContext, Norm, PendingSum, PreNormed, WeightSpec, register_part


class RMSNorm(Norm):
    """params: width, eps, name (tensor name of the weight)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = params["name"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.width,), kind="vector", init="norm")]

    def bind(self, store) -> None:
        self.weight = store.take(self.name)

    def parameter_bytes(self) -> int:
        return self.width * 4

    def prenorm_weight(self):
        return self.weight, self.eps

    def forward(self, step, x, delta, rows=None, out_name: str = "h"):
        if isinstance(delta, PreNormed):
            if delta.norm is not self or rows is not None:
                raise RuntimeError(f"{self.name}: given rows that were prepared for another norm")
            return delta  # x is up to date; the product that reads the rows applies the factor
        n = x.shape[0] if rows is None else rows.shape[0]
        out = step.ws.buffer(out_name, (n, self.width), self.ctx.act_dtype)
        if isinstance(delta, PendingSum):
            K.add_rmsnorm(x, delta.first, self.weight, out, self.eps, rows, delta2=delta.second)
        else:
            K.add_rmsnorm(x, delta, self.weight, out, self.eps, rows)
        return out

    def forward_in_place(self, x) -> None:
        """x <- norm(x) on the float32 stream itself (a norm that sits on the stream, not beside it)."""
        K.add_rmsnorm(x, None, self.weight, x, self.eps)


class LayerNorm(Norm):
    """params: width, eps, name (tensor name of the weight), bias (tensor name of the bias, or None for none),
    optional (True: a folder may leave both tensors out)."""

    capturable = True

    def __init__(self, params, ctx: BuildContext):
        super().__init__(params, ctx)
        self.width = int(params["width"])
        self.eps = float(params["eps"])
        self.name = params["name"]
        self.bias_name = params.get("bias")
        self.optional = bool(params.get("optional", False))  # a folder may leave the tensors out (a norm nothing reads)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.name, (self.width,), kind="vector", init="norm", optional=self.optional)]
        if self.bias_name:
            specs.append(WeightSpec(self.bias_name, (self.width,), kind="vector", init="normal", optional=self.optional))
        return specs

    def bind(self, store) -> None:
        self.weight = store.take(self.name)
        self.bias = store.take(self.bias_name) if self.bias_name else None

    def parameter_bytes(self) -> int:
        return self.width * (8 if self.bias_name else 4)

    def forward(self, step, x, delta, rows=None, out_name: str = "h"):
        if isinstance(delta, PreNormed):
            raise RuntimeError(f"{self.name}: a layer norm cannot finish rows that were prepared for another norm")
        n = x.shape[0] if rows is None else rows.shape[0]
        out = step.ws.buffer(out_name, (n, self.width), self.ctx.act_dtype)
        if isinstance(delta, PendingSum):
            # two parts that read one norm: add the first to the stream here, the second with the norm
            K.add_layernorm(x, delta.first, self.weight, self.bias, out, self.eps, rows)
            if rows is not None:
                raise RuntimeError(f"{self.name}: two pending outputs cannot be added to gathered rows")
            delta = delta.second
        K.add_layernorm(x, delta, self.weight, self.bias, out, self.eps, rows)
        return out


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm", LayerNorm)
