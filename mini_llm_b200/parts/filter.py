"""Input filters: what stands between a sublayer's norm and its mixer.

``causal_taps``: a short causal convolution over time on every channel, added onto its input:
``out_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)`` with zeros before the sequence's start.
The last ``taps - 1`` inputs of a request are its state (32-bit, in the request's slot), so a
prompt may be cut anywhere and a decoded token finds its predecessors.
"""

from __future__ import annotations

import torch

from .base import InputFilter, register_part
from .spec import FixedState, NoCache, WeightSpec


class CausalTaps(InputFilter):
    graph_safe = True
    accepts_deferred_norm = True      # a step of single tokens norms on the way in (one kernel with the filter)

    def __init__(self, prefix, width: int, taps: int, name: str = "weight"):
        super().__init__(prefix)
        self.width, self.taps, self.name = int(width), int(taps), name
        if self.taps < 1:
            raise ValueError(f"{self.full_name(name)}: a convolution has at least one tap")

    def weight_specs(self):
        # kept in 32-bit: the taps enter 32-bit sums only
        return [WeightSpec(self.full_name(self.name), (self.width, self.taps), role="vector", init="matrix")]

    def cache_need(self):
        return FixedState((self.taps - 1, self.width), "float32") if self.taps > 1 else NoCache()

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self._no_state = None

    def forward(self, ctx, x, cache):
        out = ctx.buffer("filtered", (x.shape[0], self.width), ctx.act_dtype)
        if self.taps > 1:
            state, writes = cache.state, cache.writes
        else:
            if self._no_state is None:
                self._no_state = torch.zeros((1, 0, self.width), dtype=torch.float32, device=ctx.device)
            state, writes = self._no_state, False
        ctx.kernels.causal_taps(ctx, out, x, self.w(self.name), state, writes)
        return out


register_part("causal_taps", CausalTaps)
