"""Parallel mixer: several mixers side by side on the same input.  The result is the mean of
their outputs, each divided by its root mean square over the model width and scaled by a
weight of its own; the mean is float.  At most one branch may keep keys and values in pages
and at most one a state slot: the layer's cache entry then serves both.
"""
from __future__ import annotations

from .. import ops
from ..weights.names import ParamSpec
from .base import CacheNeed, LayerCache, Runtime, StepContext
from .registry import build_part, part_class, register_part


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class ParallelMixer:
    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for b, branch in enumerate(spec.branches):
            for local, ps in part_class("mixer", branch).param_specs(branch).items():
                out[f"branch{b}.{local}"] = ps
            out[f"out{b}.weight"] = ParamSpec((spec.hidden_size,), role="vector", init="ones")
        return out

    @classmethod
    def cache_need(cls, spec) -> CacheNeed:
        kv = state = None
        for branch in spec.branches:
            need = part_class("mixer", branch).cache_need(branch)
            if need is None:
                continue
            if need.kv is not None:
                if kv is not None:
                    raise ValueError("two branches of a parallel mixer ask for key/value pages")
                kv = need.kv
            if need.state is not None:
                if state is not None:
                    raise ValueError("two branches of a parallel mixer ask for a state slot")
                state = need.state
        return CacheNeed(kv=kv, state=state)

    def __init__(self, spec, params: dict, runtime: Runtime):
        if not 1 <= len(spec.branches) <= 4:
            raise ValueError("a parallel mixer has one to four branches")
        self.spec = spec
        self.runtime = runtime
        self.branches = [build_part("mixer", branch, _sub(params, f"branch{b}"), runtime)
                         for b, branch in enumerate(spec.branches)]
        self.weights = [params[f"out{b}.weight"].float().contiguous()
                        for b in range(len(spec.branches))]
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.branches)

    def forward(self, x, ctx: StepContext, cache: LayerCache):
        outs = [branch.forward(x, ctx, cache) for branch in self.branches]
        return ops.mean_of_norms(outs, self.weights, self.spec.norm_eps)


register_part("mixer", "parallel", ParallelMixer)
