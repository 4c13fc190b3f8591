"""Matrix-memory mixer (the mLSTM cell): a recurrent layer whose per-request state lives in
a state slot instead of key/value pages.

One product gives q, k, v and the output gate g, a second one, with float output, the two
gate pre-activations per head (everything that enters the recurrence beyond q, k and v is
float).  The scan kernel walks each entry's tokens from the state its slot holds and leaves
the new state there; a second kernel divides each head's output by its root mean square,
scales it by the cell's norm weight and gates it; the output product follows.  A prompt
portion, a single decoded token and any mix of the two are the same launches.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, LayerCache, Runtime, StateNeed, StepContext
from .registry import register_part


class MatrixMemory:
    # the forward pass reads the step's device arrays only
    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        qk, vv = spec.num_heads * spec.qk_dim, spec.num_heads * spec.v_dim
        return {
            "in.weight": ParamSpec((2 * qk + 2 * vv, spec.hidden_size)),
            "gates.weight": ParamSpec((2 * spec.num_heads, spec.hidden_size)),
            "gates.bias": ParamSpec((2 * spec.num_heads,), role="vector", init="zeros"),
            "norm.weight": ParamSpec((vv,), role="vector", init="ones"),
            "o.weight": ParamSpec((spec.hidden_size, vv)),
        }

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        size = ops.matrix_memory_state_size(spec.num_heads, spec.qk_dim, spec.v_dim)
        return CacheNeed(state=StateNeed(shape=(size,), dtype="float32"))

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.w_in = params["in.weight"]
        self.w_gates = params["gates.weight"]
        self.w_out = params["o.weight"]
        self.bias = params["gates.bias"].float().contiguous()
        self.norm_weight = params["norm.weight"].float().contiguous()
        self.q_scale = spec.qk_dim ** -0.5

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        qk, vv = s.num_heads * s.qk_dim, s.num_heads * s.v_dim
        proj = ops.linear(x, self.w_in, static_weights=True)
        gates = ops.linear(x, self.w_gates, out_dtype=torch.float32, static_weights=True)
        o = ops.matrix_memory_scan(proj, gates, self.bias, ctx.qo_indptr, ctx.slots, cache.state,
                                   ctx.num_entries, s.num_heads, s.qk_dim, s.v_dim, s.gate_cap,
                                   self.q_scale, s.denom_floor)
        y = ops.head_norm_gate(o, proj[:, 2 * qk + vv:], self.norm_weight, s.num_heads, s.v_dim,
                               s.norm_eps, self.runtime.dtype)
        return ops.linear(y, self.w_out, static_weights=True)


register_part("mixer", "mlstm", MatrixMemory)
