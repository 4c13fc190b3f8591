"""Typed configuration of the Vudivik decoder (``"architecture": "Vudivik"``).

config.json gives ``width``, ``vocab``, ``norm.eps``, ``residual_mult`` and the layers one
by one: ``layers[i] = {"type": "parallel", "mixer": {"left": {...}, "right": {...}},
"mlp": {...} | null}``, optionally with ``"weights_of": j``: such a layer has no tensors of
its own and runs layer j's, with a cache and a state of its own.

A layer norms only what its sublayers put out: ``h += m * norm1(mixer(h))``, then ``h += m *
norm2(ff(h))``.  The mixer runs two mixers side by side: a grouped-query attention
(``left``: biased projections, an RMS norm per query and key head, rotate-half rotary
encoding over ``rot.dims`` features with the frequency scaling of ``rot.scaling``, a sliding
window ``mask.size`` that keeps the first ``mask.keep_first`` tokens visible) and a selective
scan (``right``); their RMS-normed outputs are averaged.  The feed-forward is
``down(relu(up h)^2)``, dense or as routed experts (softmax scores, a correction added for
the choice only, the last ``router.identity`` outputs standing for identity experts).
Nothing has a size default; every size may differ from layer to layer.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .base import ConfigError, ModelConfig
from .layout import (AttentionSpec, BlockSpec, MLPSpec, ModelLayout, NormSpec, ParallelMixerSpec,
                     PositionSpec, RopeScalingSpec, RoutedExpertsSpec, RunEntry,
                     SelectiveScanSpec)
from .tifosun import _Reader

LAYER_TYPES = ("parallel",)


@dataclass
class VudivikConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    layers: list = field(default_factory=list)        # the raw layer objects of config.json
    stop_tokens: tuple = ()

    architecture = "Vudivik"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "VudivikConfig":
        rd = _Reader()
        width = rd.get(raw, "config", "width", int)
        vocab = rd.get(raw, "config", "vocab", int)
        eps = rd.get(rd.get(raw, "config", "norm", dict), "config.norm", "eps", float)
        mult = rd.get(raw, "config", "residual_mult", float)
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            rd.problems.append("config.layers must be a non-empty list")
            layers = []
        stops = raw.get("eos_token_id")
        if stops is None:
            stops = ()
        elif not isinstance(stops, (list, tuple)):
            stops = (stops,)
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, residual_mult=mult,
                  layers=copy.deepcopy(list(layers)), stop_tokens=tuple(int(t) for t in stops))
        rd.positive("config", width=width, vocab=vocab, **{"norm.eps": eps})
        if width > 0:
            cfg._plan(rd)
        if rd.problems:
            raise ConfigError("unusable Vudivik configuration: " + "; ".join(rd.problems))
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "layers": copy.deepcopy(self.layers)}
        if self.stop_tokens:
            out["eos_token_id"] = list(self.stop_tokens)
        return out

    # -- layers -------------------------------------------------------------
    def _left(self, rd: _Reader, path: str, m: Mapping) -> AttentionSpec:
        heads, kv_heads, dim, vdim = (rd.get(m, path, k, int)
                                      for k in ("heads", "kv_heads", "dim", "vdim"))
        scale = rd.get(m, path, "scale", float)
        rd.positive(path, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
        if kv_heads > 0 and heads % kv_heads:
            rd.problems.append(f"{path}.heads ({heads}) is no multiple of kv_heads ({kv_heads})")
        position = PositionSpec(kind="none", head_dim=dim)
        rot = rd.get(m, path, "rot", dict, default=None, required=False)
        if rot is not None:
            base = rd.get(rot, path + ".rot", "base", float)
            dims = rd.get(rot, path + ".rot", "dims", int)
            rd.positive(path, **{"rot.base": base})
            if dims % 2 or not 0 <= dims <= dim:
                rd.problems.append(f"{path}.rot.dims must be even and at most dim, got {dims}")
            scaling = None
            sc = rd.get(rot, path + ".rot", "scaling", dict, default=None, required=False)
            if sc is not None:
                sp = path + ".rot.scaling"
                factor, low, high = (rd.get(sc, sp, k, float) for k in ("factor", "low", "high"))
                original = rd.get(sc, sp, "original", float)
                rd.positive(sp, factor=factor, original=original)
                if high == low:
                    rd.problems.append(f"{sp}.high and .low must differ")
                scaling = RopeScalingSpec(rope_type="llama3", factor=factor, low_freq_factor=low,
                                          high_freq_factor=high,
                                          original_max_position_embeddings=original)
            if dims:
                position = PositionSpec(kind="rope", head_dim=dim, rotary_dim=dims, theta=base,
                                        scaling=scaling, interleaved=False)
        window, keep = None, 0
        mask = rd.get(m, path, "mask", dict, default=None, required=False)
        if mask is not None:
            window = rd.get(mask, path + ".mask", "size", int)
            keep = rd.get(mask, path + ".mask", "keep_first", int, default=0, required=False)
            rd.positive(path, **{"mask.size": window})
            if keep < 0:
                rd.problems.append(f"{path}.mask.keep_first must not be negative, got {keep}")
        return AttentionSpec(hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads,
                             head_dim=dim, position=position, window=window, scale=scale,
                             keep_first=keep, v_head_dim=vdim, bias=True,
                             qk_norm_eps=self.norm_eps)

    def _right(self, rd: _Reader, path: str, m: Mapping) -> SelectiveScanSpec:
        inner, state, rank, taps = (rd.get(m, path, k, int)
                                    for k in ("inner", "state", "dt_rank", "conv"))
        rd.positive(path, inner=inner, state=state, dt_rank=rank, conv=taps)
        return SelectiveScanSpec(hidden_size=self.width, inner=inner, state=state, dt_rank=rank,
                                 conv=taps)

    def _mixer(self, rd: _Reader, i: int, layer: Mapping):
        kind = rd.get(layer, f"layers[{i}]", "type", str)
        if kind not in LAYER_TYPES:
            rd.problems.append(f"layers[{i}].type {kind!r} is not known (known: {LAYER_TYPES})")
            return None
        path = f"layers[{i}].mixer"
        m = rd.get(layer, f"layers[{i}]", "mixer", dict)
        left = self._left(rd, path + ".left", rd.get(m, path, "left", dict))
        right = self._right(rd, path + ".right", rd.get(m, path, "right", dict))
        return ParallelMixerSpec(hidden_size=self.width, branches=(left, right),
                                 norm_eps=self.norm_eps)

    def _ffn(self, rd: _Reader, i: int, layer: Mapping):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        path = f"layers[{i}].mlp"
        kind = rd.get(mlp, path, "kind", str)
        if kind == "dense":
            ff = rd.get(mlp, path, "ff", int)
            rd.positive(path, ff=ff)
            return MLPSpec(hidden_size=self.width, intermediate_size=ff, activation="relu2")
        if kind == "moe":
            router = rd.get(mlp, path, "router", dict)
            experts = rd.get(router, path + ".router", "experts", int)
            top = rd.get(router, path + ".router", "top", int)
            identity = rd.get(router, path + ".router", "identity", int, default=0,
                              required=False)
            ff = rd.get(rd.get(mlp, path, "expert", dict), path + ".expert", "ff", int)
            rd.positive(path, experts=experts, top=top, **{"expert.ff": ff})
            if identity < 0:
                rd.problems.append(f"{path}.router.identity must not be negative")
            if top > experts + identity:
                rd.problems.append(f"{path}.router.top ({top}) exceeds the router's outputs "
                                   f"({experts + identity})")
            return RoutedExpertsSpec(hidden_size=self.width, num_experts=experts, top=top,
                                     expert_size=ff, shared_size=0, score="softmax",
                                     renormalize=False, scale_input=False, activation="relu2",
                                     gated=False, choice_bias=True, identity_experts=identity)
        rd.problems.append(f"{path}.kind {kind!r} is not known (known: dense, moe)")
        return None

    def _plan(self, rd: Optional[_Reader] = None):
        """(blocks, order, owners): one block per layer that has tensors of its own,
        ``owners[b]`` its layer index, and the run order with a cache per layer."""
        rd = rd or _Reader()
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks, owners, block_of, order = [], [], {}, []
        # first the layers that have tensors, then whose tensors every layer runs: a layer may
        # name one before or after it, and one that borrows itself passes the name on
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                rd.problems.append(f"layers[{i}] must be an object")
                continue
            if layer.get("weights_of") is not None:
                continue
            mixer = self._mixer(rd, i, layer)
            ffn = self._ffn(rd, i, layer)
            block_of[i] = len(blocks)
            owners.append(i)
            blocks.append(BlockSpec(kind="postnorm", mixer=mixer, ffn=ffn, norm1=None, norm2=None,
                                    norm1_post=norm, norm2_post=None if ffn is None else norm,
                                    residual_mult=self.residual_mult))
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                continue
            at, seen = i, set()
            while isinstance(self.layers[at], Mapping) and self.layers[at].get("weights_of") is not None:
                nxt = self.layers[at]["weights_of"]
                seen.add(at)
                if isinstance(nxt, bool) or not isinstance(nxt, int) \
                        or not 0 <= nxt < len(self.layers) or nxt in seen:
                    rd.problems.append(f"layers[{i}].weights_of must lead to a layer with tensors "
                                       f"of its own, got {self.layers[at]['weights_of']!r}")
                    at = None
                    break
                at = nxt
            if at is None or at not in block_of:
                continue
            order.append(RunEntry(block=block_of[at], cache=i))
        return blocks, order, owners

    def block_owners(self) -> list:
        """Layer index whose tensors each block of the layout holds."""
        return self._plan()[2]

    def layout(self) -> ModelLayout:
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps)
        blocks, order, _ = self._plan()
        layout = ModelLayout(vocab_size=self.vocab, hidden_size=self.width, blocks=blocks,
                             order=order, final_norm=norm, tie_word_embeddings=False,
                             max_positions=None)
        layout.validate()
        return layout

    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)

    def max_positions(self):
        return None
