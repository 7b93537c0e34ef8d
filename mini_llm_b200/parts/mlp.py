"""Dense feed-forward: ``act(x W_up + b_up) W_down + b_down``, added onto the
residual stream (engine/src/transformer_block.c:64-71).  The activation is a
parameter: the tanh form of gelu (engine/include/gelu_math.h:6-11) or the erf
form (engine/src/gelu.c:5-9), or the square of relu.  Biases are optional, and the tensors'
names are parameters (``weight_suffix=""`` for files that name a matrix by its layer alone).
``compute`` returns the output itself, in 32-bit, for arrangements that norm it before the sum."""

from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .spec import WeightSpec

ACTIVATION_EPILOGUES = ("gelu_tanh", "gelu_erf", "relu_squared", "silu")


class DenseMlp(FeedForward):
    graph_safe = True
    def __init__(self, prefix, width: int, inner: int, activation: str,
                 up_name: str = "c_fc", down_name: str = "c_proj", stored_in_out: bool = True, bias: bool = True,
                 weight_suffix: str = ".weight"):
        super().__init__(prefix)
        self.width, self.inner = int(width), int(inner)
        if activation not in ACTIVATION_EPILOGUES:
            raise ValueError(f"{prefix}: unknown activation '{activation}' (known: {', '.join(ACTIVATION_EPILOGUES)})")
        self.activation = activation
        self.up_name, self.down_name = up_name, down_name
        self.stored_in_out = bool(stored_in_out)
        self.bias, self.weight_suffix = bool(bias), weight_suffix

    def _matrix_shape(self, n_in, n_out):
        return (n_in, n_out) if self.stored_in_out else (n_out, n_in)

    def weight_specs(self):
        t, suffix = self.stored_in_out, self.weight_suffix
        specs = [
            WeightSpec(self.full_name(f"{self.up_name}{suffix}"), self._matrix_shape(self.width, self.inner), transpose=t),
            WeightSpec(self.full_name(f"{self.down_name}{suffix}"), self._matrix_shape(self.inner, self.width), transpose=t,
                       init="residual_matrix"),
        ]
        if self.bias:
            specs.insert(1, WeightSpec(self.full_name(f"{self.up_name}.bias"), (self.inner,), role="vector", init="bias"))
            specs.append(WeightSpec(self.full_name(f"{self.down_name}.bias"), (self.width,), role="vector", init="bias"))
        return specs

    accepts_deferred_norm = True

    def _bias(self, name):
        return self.w(f"{name}.bias") if self.bias else None

    def _up(self, ctx, x):
        up = ctx.buffer("mlp_up", (x.shape[0], self.inner), ctx.act_dtype)
        ctx.kernels.linear(ctx, up, x, self.w(f"{self.up_name}{self.weight_suffix}"), self._bias(self.up_name),
                           epilogue=self.activation)
        return up

    def forward(self, ctx, x, hidden):
        ctx.kernels.linear(ctx, hidden, self._up(ctx, x), self.w(f"{self.down_name}{self.weight_suffix}"),
                           self._bias(self.down_name), epilogue="add")

    def compute(self, ctx, x):
        out = ctx.buffer("mlp_out", (x.shape[0], self.width), torch.float32)
        ctx.kernels.linear(ctx, out, self._up(ctx, x), self.w(f"{self.down_name}{self.weight_suffix}"),
                           self._bias(self.down_name))
        return out


register_part("dense_mlp", DenseMlp)
