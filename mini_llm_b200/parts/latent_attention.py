"""Causal attention over a shared low-rank latent.

Per token one projection gives ``rank + rot`` numbers: the first ``rank``, normed by their root
mean square and multiplied by a gain, are the latent ``c``; the last ``rot``, with rotary
positions, are a key part ``r`` that all heads share.  Head ``h`` has the key
``[U_k[h] c | r]`` and the value ``U_v[h] c``; its query is ``[q_h | rotated q'_h]`` with
``dim`` and ``rot`` entries.  Only ``[c | r]`` is cached, one row per token for all heads.

The products with U_k and U_v are moved to the query's side (both are linear in ``c``):
``q_h . (U_k[h] c) = (U_k[h]^T q_h) . c``, and ``sum_j p_j U_v[h] c_j = U_v[h] (sum_j p_j c_j)``.
So the step computes, per token and head, the effective query ``[U_k[h]^T q_h | rotated q'_h]``
in 32-bit, attends over the cached rows (score = effective query . row * scale, value = the row's
first ``rank`` entries; softmax in 32-bit), and expands the result with U_v[h].  A prompt portion
and a single decoded token take the same path, and no key or value per head is ever stored.

Rotary positions use the interleaved layout: among the first ``rotary_dims`` entries of the
rotated part, entries 2i and 2i+1 form a pair that turns by ``position * base^(-2i/rotary_dims)``.
"""

from __future__ import annotations

import torch

from .base import Mixer, register_part
from .spec import PagedKV, WeightSpec


class LatentAttention(Mixer):
    graph_safe = True
    wants_attention_tiles = True      # its prompt kernel reads the step's work list of (up to 128 tokens, entry) tiles

    def __init__(self, prefix, width: int, n_heads: int, head_size: int, rotated_size: int, value_size: int,
                 latent_size: int, score_scale: float, rotary_base: float, rotary_dims: int, eps: float,
                 q_name: str = "q", down_name: str = "dkv", latent_norm_name: str = "dkv.norm",
                 key_up_name: str = "uk", value_up_name: str = "uv", out_name: str = "o"):
        super().__init__(prefix)
        self.width, self.n_heads = int(width), int(n_heads)
        self.dim, self.rot, self.vdim, self.rank = int(head_size), int(rotated_size), int(value_size), int(latent_size)
        self.score_scale, self.rotary_base, self.rotary_dims = float(score_scale), float(rotary_base), int(rotary_dims)
        self.eps = float(eps)
        if self.rotary_dims % 2 != 0 or not 0 <= self.rotary_dims <= self.rot:
            raise ValueError(f"{prefix}: {self.rotary_dims} rotated dimensions do not fit a rotated part of {self.rot} "
                             f"(an even number, at most the part)")
        if min(self.n_heads, self.dim, self.vdim, self.rank) <= 0:
            raise ValueError(f"{prefix}: heads, head size, value size and latent size must be positive")
        self.names = dict(q=q_name, down=down_name, norm=latent_norm_name, uk=key_up_name, uv=value_up_name, o=out_name)
        self.row = self.rank + self.rot

    def weight_specs(self):
        n, h = self.names, self.n_heads
        return [
            WeightSpec(self.full_name(n["q"]), (h * (self.dim + self.rot), self.width)),
            WeightSpec(self.full_name(n["down"]), (self.row, self.width)),
            WeightSpec(self.full_name(n["norm"]), (self.rank,), role="vector", init="gain"),
            WeightSpec(self.full_name(n["uk"]), (h * self.dim, self.rank)),
            WeightSpec(self.full_name(n["uv"]), (h * self.vdim, self.rank)),
            WeightSpec(self.full_name(n["o"]), (self.width, h * self.vdim), init="residual_matrix"),
        ]

    def cache_need(self):
        return PagedKV(1, self.row, None, has_values=False)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        h = self.n_heads
        uk = self.w(self.names["uk"])
        # per head, [rank, dim]: the key expansion as the product's weight on the query's side
        self.key_up_t = uk.view(h, self.dim, self.rank).transpose(1, 2).contiguous()
        self.value_up = self.w(self.names["uv"]).view(h, self.vdim, self.rank)
        half = self.rotary_dims // 2
        exponent = -2.0 * torch.arange(half, dtype=torch.float64) / max(self.rotary_dims, 1)
        self.inv_freq = (torch.tensor(self.rotary_base, dtype=torch.float64) ** exponent).to(uk.device)
        if half == 0:
            self.inv_freq = torch.zeros(1, dtype=torch.float64, device=uk.device)

    def compute(self, ctx, x, cache):
        k, n, h = ctx.kernels, x.shape[0], self.n_heads
        q = ctx.buffer("latent_q", (n, h * (self.dim + self.rot)), ctx.act_dtype)
        k.linear(ctx, q, x, self.w(self.names["q"]))
        down = ctx.buffer("latent_down", (n, self.row), torch.float32)
        k.linear(ctx, down, x, self.w(self.names["down"]))
        q_eff = ctx.buffer("latent_q_eff", (n, h * self.row), torch.float32)
        k.latent_prepare(ctx, cache, q_eff, down, q, self.w(self.names["norm"]), self.inv_freq, self.rank, self.rot,
                         self.rotary_dims, h, self.dim, self.eps)
        k.head_linear(ctx, q_eff, q, self.key_up_t, h, self.dim + self.rot, self.row)
        mixed_latent = ctx.buffer("latent_mixed", (n, h * self.rank), k.latent_mixed_dtype(cache, self.rank, self.rot))
        k.latent_attention(ctx, mixed_latent, q_eff, cache, h, self.rank, self.rot, self.score_scale)
        mixed = ctx.buffer("attn_out", (n, h * self.vdim), ctx.act_dtype)
        k.head_linear(ctx, mixed, mixed_latent, self.value_up, h, self.rank, self.vdim)
        out = ctx.buffer("mixer_out", (n, self.width), torch.float32)
        k.linear(ctx, out, mixed, self.w(self.names["o"]))
        return out

    def forward(self, ctx, x, hidden, cache):
        hidden += self.compute(ctx, x, cache)


register_part("latent_attention", LatentAttention)
