"""Block arrangements: how a mixer, a feed-forward and norms are wired.

"prenorm" is the reference's DecoderLayer (mstar/model/components/decoder_layer.py:
58-71): h += mixer(norm1(h)); h += ffn(norm2(h)).  The two adds are not separate
passes: each part's output stays pending on the residual stream and the next norm
(the next block's norm1, or the final norm) adds it in float while normalising.
"""
from __future__ import annotations

from .base import ResidualStream, Runtime
from .registry import build_part, part_class, register_part


def _sub(params: dict, prefix: str) -> dict:
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


class PreNormBlock:
    SUBPARTS = (("norm1", "norm"), ("mixer", "mixer"), ("norm2", "norm"), ("ffn", "ffn"))

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls.SUBPARTS:
            sub = getattr(spec, name)
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1, _sub(params, "norm1"), runtime)
        self.mixer = build_part("mixer", spec.mixer, _sub(params, "mixer"), runtime)
        self.norm2 = build_part("norm", spec.norm2, _sub(params, "norm2"), runtime)
        self.ffn = build_part("ffn", spec.ffn, _sub(params, "ffn"), runtime)
        # replayable as part of a captured decode step only if every sub-part says so itself
        self.graph_safe = all(getattr(p, "graph_safe", False) is True
                              for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.norm1.add_norm(stream)
        stream.push(self.mixer.forward(x, ctx, cache))
        y = self.norm2.add_norm(stream)
        stream.push(self.ffn.forward(y, ctx))


class SandwichBlock:
    """h += norm1_post(mixer(norm1(h))); h += norm2_post(ffn(norm2(h))).  A sublayer's output
    is pushed together with its own norm; the next norm on the stream (this block's norm2, the
    next block's norm1, or the model's final norm) applies it, adds and normalises in one
    kernel.  A block without a feed-forward has the first sublayer only."""

    @staticmethod
    def _subparts(spec):
        parts = [("norm1", "norm"), ("mixer", "mixer"), ("norm1_post", "norm")]
        if spec.ffn is not None:
            parts += [("norm2", "norm"), ("ffn", "ffn"), ("norm2_post", "norm")]
        return parts

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls._subparts(spec):
            sub = getattr(spec, name)
            if sub is None:
                raise ValueError(f"a sandwich block needs {name}")
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.parts = {name: build_part(category, getattr(spec, name), _sub(params, name), runtime)
                      for name, category in self._subparts(spec)}
        self.norm1, self.mixer, self.norm1_post = (self.parts[k] for k in
                                                   ("norm1", "mixer", "norm1_post"))
        self.norm2, self.ffn, self.norm2_post = (self.parts.get(k) for k in
                                                 ("norm2", "ffn", "norm2_post"))
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.parts.values())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        x = self.norm1.add_norm(stream)
        stream.push(self.mixer.forward(x, ctx, cache), post=self.norm1_post)
        if self.ffn is not None:
            y = self.norm2.add_norm(stream)
            stream.push(self.ffn.forward(y, ctx), post=self.norm2_post)


class PostNormBlock:
    """h += m * norm1_post(mixer(h)); h += m * norm2_post(ffn(h)): the sublayers read the
    residual itself, only their outputs are normed (and multiplied by ``residual_mult``).  A
    sublayer's output stays pending with its norm; the kernel that adds it also hands the new
    residual, in the compute dtype, to the sublayer that reads it next."""

    @staticmethod
    def _subparts(spec):
        parts = [("mixer", "mixer"), ("norm1_post", "norm")]
        if spec.ffn is not None:
            parts += [("ffn", "ffn"), ("norm2_post", "norm")]
        return parts

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {}
        for name, category in cls._subparts(spec):
            sub = getattr(spec, name)
            if sub is None:
                raise ValueError(f"a postnorm block needs {name}")
            for local, ps in part_class(category, sub).param_specs(sub).items():
                out[f"{name}.{local}"] = ps
        return out

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.parts = {name: build_part(category, getattr(spec, name), _sub(params, name), runtime)
                      for name, category in self._subparts(spec)}
        self.mixer, self.norm1_post = self.parts["mixer"], self.parts["norm1_post"]
        self.ffn, self.norm2_post = self.parts.get("ffn"), self.parts.get("norm2_post")
        self.graph_safe = all(getattr(p, "graph_safe", False) is True for p in self.parts.values())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        m = self.spec.residual_mult
        x = stream.rows(self.runtime.dtype)
        stream.push(self.mixer.forward(x, ctx, cache), post=self.norm1_post, scale=m)
        if self.ffn is not None:
            y = stream.rows(self.runtime.dtype)
            stream.push(self.ffn.forward(y, ctx), post=self.norm2_post, scale=m)


register_part("block", "prenorm", PreNormBlock)
register_part("block", "postnorm", PostNormBlock)
register_part("block", "sandwich", SandwichBlock)
