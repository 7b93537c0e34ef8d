"""Routed feed-forward (mixture of experts) with sigmoid scores.

Router logits ``z = W_router x`` and scores ``s = sigmoid(z)`` in 32-bit; each token takes the
``top`` experts with the largest scores.  The weight of a chosen expert is its score (not
renormalized) and multiplies the expert's INPUT: the layer adds ``sum_e expert_e(s_e * x)`` onto
the stream, with ``expert(u) = W_down (silu(W_gate u) * (W_up u))`` and no biases.  A shared expert of
the same form (with an inner size of its own) may run for every token; its output is multiplied
by ``sigmoid(w_sg . x)``, one number per token.

Experts are named by tables of pointers and inner sizes, so the shared expert goes through the
kernels as one more chosen expert with input weight 1 and its gate as the output weight.
"""

from __future__ import annotations

import torch

from .base import FeedForward, register_part
from .spec import WeightSpec


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, prefix, width: int, n_experts: int, top: int, expert_inner: int, shared_inner: int | None = None,
                 names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_experts, self.top, self.inner = int(width), int(n_experts), int(top), int(expert_inner)
        self.shared_inner = int(shared_inner) if shared_inner else None
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"{prefix}: every token takes between 1 and {self.n_experts} experts, got {self.top}")
        if self.inner <= 0:
            raise ValueError(f"{prefix}: the experts' inner size must be positive")
        self.names = dict(router="router", expert="e{index}", shared="shared", shared_gate="shared.sg", gate="gate", up="up",
                          down="down")
        self.names.update(names or {})
        self.pairs = self.top + (1 if self.shared_inner else 0)

    def _expert_names(self):
        found = [(self.names["expert"].format(index=e), self.inner) for e in range(self.n_experts)]
        if self.shared_inner:
            found.append((self.names["shared"], self.shared_inner))
        return found

    def weight_specs(self):
        n = self.names
        specs = [WeightSpec(self.full_name(n["router"]), (self.n_experts, self.width))]
        for name, inner in self._expert_names():
            specs += [WeightSpec(self.full_name(f"{name}.{n['gate']}"), (inner, self.width)),
                      WeightSpec(self.full_name(f"{name}.{n['up']}"), (inner, self.width)),
                      WeightSpec(self.full_name(f"{name}.{n['down']}"), (self.width, inner), init="residual_matrix")]
        if self.shared_inner:
            specs.append(WeightSpec(self.full_name(n["shared_gate"]), (1, self.width)))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        experts = self._expert_names()
        device = self.w(n["router"]).device

        def table(which):
            return torch.tensor([self.w(f"{name}.{n[which]}").data_ptr() for name, _ in experts], dtype=torch.int64, device=device)

        self.gate_of, self.up_of, self.down_of = table("gate"), table("up"), table("down")
        self.inner_of = torch.tensor([inner for _, inner in experts], dtype=torch.int32, device=device)
        self.max_inner = max(inner for _, inner in experts)

    def forward(self, ctx, x, hidden):
        k, n = ctx.kernels, x.shape[0]
        choice = ctx.buffer("expert_choice", (n * self.pairs,), torch.int32)
        in_weight = ctx.buffer("expert_in_weight", (n * self.pairs,), torch.float32)
        out_weight = ctx.buffer("expert_out_weight", (n * self.pairs,), torch.float32)
        k.route(x, self.w(self.names["router"]), self.w(self.names["shared_gate"]) if self.shared_inner else None, self.top,
                choice, in_weight, out_weight)
        act = ctx.buffer("expert_act", (n * self.pairs, self.max_inner), ctx.act_dtype)
        k.experts(hidden, act, x, choice, in_weight, out_weight, self.gate_of, self.up_of, self.down_of, self.inner_of,
                  self.max_inner, self.pairs)

    def compute(self, ctx, x):
        out = ctx.buffer("mlp_out", (x.shape[0], self.width), torch.float32)
        out.zero_()
        self.forward(ctx, x, out)
        return out


register_part("routed_experts", RoutedExperts)
