"""Latent attention mixer: softmax attention whose keys and values are up-projections of
one cached latent row per token.

A token leaves ``kv_rank`` normalised latent features c and ``rot_dim`` rotated key features
in its cache row; nothing per head is cached.  The key up-projection is folded into the
query (a_h = W_uk[h]^T q_h, so that q_h . (W_uk[h] c) = a_h . c) and the value up-projection
is applied to the attention's output (sum_j p_j W_uv[h] c_j = W_uv[h] sum_j p_j c_j): the
attention kernel then reads the same rows for every head, in prompts and in decoding alike.
One product gives the queries, the down-projection and the output gate.  Scores,
probabilities and the weighted sum are float; the folded query is kept in float as well.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, KVNeed, LayerCache, Runtime, StepContext
from .registry import register_part


class LatentAttention:
    graph_safe = True       # nothing per-step is read from the host

    @classmethod
    def param_specs(cls, spec) -> dict:
        h = spec.num_heads
        rows = h * (spec.qk_dim + spec.rot_dim) + spec.kv_rank + spec.rot_dim
        if spec.gated:
            rows += h * spec.v_dim
        return {
            "in.weight": ParamSpec((rows, spec.hidden_size)),
            "kv_norm.weight": ParamSpec((spec.kv_rank,), role="vector", init="ones"),
            "uk.weight": ParamSpec((h * spec.qk_dim, spec.kv_rank)),
            "uv.weight": ParamSpec((h * spec.v_dim, spec.kv_rank)),
            "o.weight": ParamSpec((spec.hidden_size, h * spec.v_dim)),
        }

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        return CacheNeed(kv=KVNeed(num_kv_heads=1, head_dim=spec.kv_rank + spec.rot_dim,
                                   window=spec.window, planes=1))

    def __init__(self, spec, params: dict, runtime: Runtime):
        p = spec.position
        if p.kind != "rope" or not p.interleaved:
            raise ValueError("latent attention rotates interleaved pairs (a rope position spec "
                             "with interleaved=True)")
        if p.rotary_dim % 2 or p.rotary_dim > spec.rot_dim:
            raise ValueError(f"rotary_dim {p.rotary_dim} must be even and at most rot_dim "
                             f"{spec.rot_dim}")
        self.spec = spec
        self.runtime = runtime
        h = spec.num_heads
        self.w_in = params["in.weight"]
        self.w_out = params["o.weight"]
        self.norm_weight = params["kv_norm.weight"].float().contiguous()
        # per head: [rank, qk_dim] rows so that a = q @ uk_t[h]^T, and [v_dim, rank]
        self.uk_t = params["uk.weight"].view(h, spec.qk_dim, spec.kv_rank).transpose(1, 2).contiguous()
        self.uv = params["uv.weight"].view(h, spec.v_dim, spec.kv_rank)
        half = p.rotary_dim // 2
        self.freq = torch.tensor([p.theta ** (-(2.0 * i) / p.rotary_dim) for i in range(half)],
                                 dtype=torch.float64, device=runtime.device)
        self.scale = spec.scale if spec.scale is not None else (spec.qk_dim + spec.rot_dim) ** -0.5

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        h, per_head = s.num_heads, s.qk_dim + s.rot_dim
        q_cols = h * per_head
        proj = ops.linear(x, self.w_in, static_weights=True)
        ops.latent_fill(proj, q_cols, self.norm_weight, self.freq, ctx.positions, ctx.cache_pos,
                        ctx.token_req, cache.block_table, cache.kv, h, s.qk_dim, s.rot_dim,
                        s.position.rotary_dim, s.kv_rank, cache.page_size, s.norm_eps)
        q = proj[:, :q_cols].view(-1, h, per_head)
        q_abs = ops.linear_per_head(q[:, :, :s.qk_dim], self.uk_t, out_dtype=torch.float32)
        lat = ops.latent_attention(q_abs, q[:, :, s.qk_dim:], cache.kv, cache.block_table,
                                   ctx.token_req, ctx.cache_pos, h, s.kv_rank, s.rot_dim,
                                   cache.page_size, s.window or 0, self.scale,
                                   max_keys=ctx.max_kv_len)
        y = ops.linear_per_head(ops.convert(lat, self.runtime.dtype), self.uv)
        y = y.view(-1, h * s.v_dim)
        if s.gated:
            ops.sigmoid_gate_mul(y, proj[:, q_cols + s.kv_rank + s.rot_dim:])
        return ops.linear(y, self.w_out, static_weights=True)


register_part("mixer", "latent_attention", LatentAttention)
