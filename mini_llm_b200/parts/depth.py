"""Weighted sum over depth: what a layer hands on is not its own result alone but
``sum_j w[j] * X_j`` over the embedding output X_0 and the results X_1 .. X_n of all layers so
far (its own is X_n), with learned weights per layer.  The model keeps the results at hand
(``ModelSpec.keeps_layer_results``, ``ctx.kept_results`` [T, planes, width] in 32-bit); an
arrangement calls this part last."""

from __future__ import annotations

from .base import Part, register_part
from .spec import WeightSpec


class DepthWeightedSum(Part):
    graph_safe = True

    def __init__(self, prefix, n_inputs: int, name: str = "weight"):
        super().__init__(prefix)
        self.n_inputs, self.name = int(n_inputs), name
        if self.n_inputs < 2:
            raise ValueError(f"{self.full_name(name)}: a layer's result and at least the embedding output are summed")

    def weight_specs(self):
        return [WeightSpec(self.full_name(self.name), (self.n_inputs,), role="vector", init="gain")]

    def forward(self, ctx, hidden):
        if ctx.kept_results is None or ctx.kept_results.shape[1] < self.n_inputs:
            raise RuntimeError(f"{self.full_name(self.name)}: the model keeps no layer results to sum over "
                               f"(ModelSpec.keeps_layer_results)")
        ctx.kernels.depth_mix(hidden, ctx.kept_results, self.w(self.name), self.n_inputs - 1)


register_part("depth_weighted_sum", DepthWeightedSum)
