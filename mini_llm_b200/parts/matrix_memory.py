"""Mixers whose memory is a matrix per head: ``S <- a S + b k v^T``, read as ``S^T q``.

Two kinds share the projections, the recurrence kernel and the gated output
(``norm(out) * gain * sigmoid(W_g x)``, then ``W_o``):

``decaying_matrix_memory`` (lightning attention): ``a`` is a fixed decay per head, ``b = 1``;
    q, k and v pass through silu; the heads' outputs are normed together by their root mean square.
``gated_matrix_memory`` (the matrix memory of xLSTM, mLSTM): per head a log input gate
    ``li = cap * tanh((w_i . x + b_i) / cap)`` and a log forget gate
    ``lf = logsigmoid(cap * tanh((w_f . x + b_f) / cap))``; with a running maximum ``m`` (from 0):
    ``m' = max(lf + m, li)``, ``a = exp(lf + m - m')``, ``b = exp(li - m')``; a vector ``n`` follows
    the same recurrence with ``k`` alone and the output is ``S^T q / (max(|n . q|, exp(-m')) + 1e-6)``,
    ``q`` scaled by ``dim^(-1/2)``; each head's output is normed by its own root mean square.

State (32-bit, in the request's slot): S [heads, dim, vdim], and for the gated kind n [heads, dim]
and m [heads].  Gates, decays and the state never leave 32-bit; q, k, v and the output gate are
read in the engine's element type.  The projections q, k, v, g are one product (their matrices
are stacked once at load), the two gate projections another whose result stays 32-bit.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, register_part
from .spec import FixedState, WeightSpec


class MatrixMemory(Mixer):
    graph_safe = True
    gated = False

    def __init__(self, prefix, width: int, n_heads: int, key_size: int, value_size: int, eps: float,
                 names: dict | None = None):
        super().__init__(prefix)
        self.width, self.n_heads, self.dim, self.vdim = int(width), int(n_heads), int(key_size), int(value_size)
        self.eps = float(eps)
        if min(self.n_heads, self.dim, self.vdim) <= 0:
            raise ValueError(f"{prefix}: heads, key size and value size must be positive")
        self.names = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", i="i", i_bias="i.b", f="f", f_bias="f.b")
        self.names.update(names or {})
        self.qk, self.vw = self.n_heads * self.dim, self.n_heads * self.vdim

    def weight_specs(self):
        n = self.names
        return [
            WeightSpec(self.full_name(n["q"]), (self.qk, self.width)),
            WeightSpec(self.full_name(n["k"]), (self.qk, self.width)),
            WeightSpec(self.full_name(n["v"]), (self.vw, self.width)),
            WeightSpec(self.full_name(n["g"]), (self.vw, self.width)),
            WeightSpec(self.full_name(n["o"]), (self.width, self.vw), init="residual_matrix"),
            WeightSpec(self.full_name(n["norm"]), (self.vw,), role="vector", init="gain"),
        ]

    def cache_need(self):
        return FixedState((ops.memory_state_floats(self.n_heads, self.dim, self.vdim, self.gated),), "float32")

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        self.stacked = torch.cat([self.w(n["q"]), self.w(n["k"]), self.w(n["v"]), self.w(n["g"])]).contiguous()

    # what the recurrence is told besides q, k, v: the subclasses differ here only
    def recurrence(self, ctx, x):
        raise NotImplementedError

    norm_groups = 1

    def compute(self, ctx, x, cache):
        k, n = ctx.kernels, x.shape[0]
        projected = ctx.buffer("memory_qkvg", (n, 2 * self.qk + 2 * self.vw), ctx.act_dtype)
        k.linear(ctx, projected, x, self.stacked)
        q, keys = projected[:, :self.qk], projected[:, self.qk:2 * self.qk]
        values, gate = projected[:, 2 * self.qk:2 * self.qk + self.vw], projected[:, 2 * self.qk + self.vw:]
        read = ctx.buffer("memory_read", (n, self.vw), torch.float32)
        k.memory_scan(ctx, read, q, keys, values, cache.state, self.n_heads, self.dim, self.vdim, writes=cache.writes,
                      **self.recurrence(ctx, x))
        mixed = ctx.buffer("attn_out", (n, self.vw), ctx.act_dtype)
        k.grouped_rms_norm(mixed, read, self.w(self.names["norm"]), self.norm_groups, self.eps, gate=gate)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        hidden += self.compute(ctx, x, cache)


class DecayingMatrixMemory(MatrixMemory):
    def __init__(self, prefix, width, n_heads, key_size, value_size, eps, decay, names=None):
        super().__init__(prefix, width, n_heads, key_size, value_size, eps, names)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.n_heads:
            raise ValueError(f"{prefix}: {len(self.decay_values)} decays for {self.n_heads} heads")

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.stacked.device)

    def recurrence(self, ctx, x):
        return dict(decay=self.decay, silu=True)


class GatedMatrixMemory(MatrixMemory):
    gated = True

    def __init__(self, prefix, width, n_heads, key_size, value_size, eps, gate_cap, names=None):
        super().__init__(prefix, width, n_heads, key_size, value_size, eps, names)
        self.gate_cap = float(gate_cap)
        if self.gate_cap <= 0:
            raise ValueError(f"{prefix}: the gates' cap must be positive")
        self.norm_groups = self.n_heads

    def weight_specs(self):
        n, h = self.names, self.n_heads
        return super().weight_specs() + [
            WeightSpec(self.full_name(n["i"]), (h, self.width)),
            WeightSpec(self.full_name(n["i_bias"]), (h,), role="vector", init="bias"),
            WeightSpec(self.full_name(n["f"]), (h, self.width)),
            WeightSpec(self.full_name(n["f_bias"]), (h,), role="vector", init="bias"),
        ]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.names
        # the two gate projections as one product; rows of zeros fill it up to sixteen output
        # features, the least the tensor-core kernel's tiles take
        stacked = torch.cat([self.w(n["i"]), self.w(n["f"])])
        self.gate_width = max(16, 2 * self.n_heads)
        self.gate_matrix = torch.zeros((self.gate_width, self.width), dtype=stacked.dtype, device=stacked.device)
        self.gate_matrix[:2 * self.n_heads] = stacked
        self.gate_bias = torch.cat([self.w(n["i_bias"]), self.w(n["f_bias"])]).contiguous()

    def recurrence(self, ctx, x):
        gates = ctx.buffer("memory_gates", (x.shape[0], self.gate_width), torch.float32)
        ctx.kernels.linear(ctx, gates, x, self.gate_matrix)
        return dict(gates=gates[:, :2 * self.n_heads], gate_bias=self.gate_bias, gate_cap=self.gate_cap,
                    q_scale=self.dim ** -0.5)


register_part("decaying_matrix_memory", DecayingMatrixMemory)
register_part("gated_matrix_memory", GatedMatrixMemory)
