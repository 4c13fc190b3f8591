"""Selective-scan mixer (Mamba): a recurrent layer whose per-request state, the diagonal
state S of every channel and the last inputs of its short convolution, lives in a state
slot.

One product gives [x | z]; a kernel runs the causal convolution with SiLU over x (inputs
before a portion's start come from the slot); a second product, with float output, gives
[dt_in | B | C]; the scan kernel makes the step sizes (softplus(W_dt dt_in + b), float),
walks each entry's tokens from the state in its slot, gates with silu(z) and moves the
convolution's window on; the output product follows.  Long portions are cut into pieces that
run side by side (the recurrence is linear in the state, so a piece's effect is its own end
state plus a decay of whatever came before).  A prompt portion, a decoded token and
any mix are the same launches.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, LayerCache, Runtime, StateNeed, StepContext
from .registry import register_part


class SelectiveScan:
    graph_safe = True       # the forward pass reads the step's device arrays only

    @classmethod
    def param_specs(cls, spec) -> dict:
        inner = spec.inner
        return {
            "in.weight": ParamSpec((2 * inner, spec.hidden_size)),
            "conv.weight": ParamSpec((inner, spec.conv), role="vector"),
            "conv.bias": ParamSpec((inner,), role="vector", init="zeros"),
            "x.weight": ParamSpec((spec.dt_rank + 2 * spec.state, inner)),
            "dt.weight": ParamSpec((inner, spec.dt_rank), role="vector"),
            "dt.bias": ParamSpec((inner,), role="vector", init="zeros"),
            "A_log": ParamSpec((inner, spec.state), role="vector", init="zeros"),
            "D": ParamSpec((inner,), role="vector", init="ones"),
            "o.weight": ParamSpec((spec.hidden_size, inner)),
        }

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        size = ops.selective_scan_state_size(spec.inner, spec.state, spec.conv)
        return CacheNeed(state=StateNeed(shape=(size,), dtype="float32"))

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.w_in = params["in.weight"]
        self.w_x = params["x.weight"]
        self.w_out = params["o.weight"]
        self.conv_w = params["conv.weight"].contiguous()
        self.conv_b = params["conv.bias"].to(self.conv_w.dtype).contiguous()
        # for the kernel that takes 8 channels a thread: taps-major float weights
        self.conv_wt = self.conv_w.float().t().contiguous()
        self.conv_bf = self.conv_b.float().contiguous()
        # everything that enters the recurrence beside x, B and C is float
        self.w_dt = params["dt.weight"].float().contiguous()
        self.dt_bias = params["dt.bias"].float().contiguous()
        self.a_neg = (-torch.exp(params["A_log"].float())).contiguous()
        self.d_skip = params["D"].float().contiguous()

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        s = self.spec
        xz = ops.linear(x, self.w_in, static_weights=True)
        xc = ops.conv_silu(xz, self.conv_w, self.conv_b, ctx.token_req, ctx.qo_indptr, ctx.slots,
                           cache.state, s.inner, s.conv, weight_t=self.conv_wt,
                           bias_f32=self.conv_bf)
        proj = ops.linear(xc, self.w_x, out_dtype=torch.float32, static_weights=True)
        y = ops.selective_scan(xc, xz, proj, self.w_dt, self.dt_bias, self.a_neg, self.d_skip,
                               ctx.qo_indptr, ctx.slots, cache.state, ctx.num_entries, s.inner,
                               s.state, s.dt_rank, s.conv, max_q_len=ctx.max_q_len)
        return ops.linear(y, self.w_out, static_weights=True)


register_part("mixer", "selective_scan", SelectiveScan)
