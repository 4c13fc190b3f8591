"""Typed configuration of the Tifosun decoder (``"architecture": "Tifosun"``).

config.json lists the layers one by one: ``layers[i] = {"type", "mixer": {...}, "mlp":
{...} | null}``; beside it stand ``width``, ``vocab`` and ``norm.eps``.  A layer's mixer is
a matrix memory (types "mlstm" and "mlstm_2", the same cell under two names) or a
windowed latent attention ("latent_attention"); its feed-forward is dense, routed experts,
or absent.  Every layer is a sandwich block: a norm before and after each sublayer, each
with its weight stored as an offset from one.  Nothing has a size default: what config.json
does not give is an error, and every size may differ from layer to layer.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .base import ConfigError, ModelConfig
from .layout import (BlockSpec, GatedMLPSpec, LatentAttentionSpec, MatrixMemorySpec, ModelLayout,
                     NormSpec, PositionSpec, RoutedExpertsSpec, RunEntry)

MATRIX_MEMORY_TYPES = ("mlstm", "mlstm_2")
LATENT_ATTENTION_TYPES = ("latent_attention",)


class _Reader:
    """Fetches typed keys of nested objects and collects what is absent or of a wrong
    type, so that one error names everything."""

    def __init__(self):
        self.problems: list = []

    def get(self, obj, path: str, key: str, kind: type, default=None, required=True):
        if not isinstance(obj, Mapping) or key not in obj or obj[key] is None:
            if required:
                self.problems.append(f"{path}.{key} is missing")
                return kind()
            return default
        v = obj[key]
        if kind is int:
            if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
                self.problems.append(f"{path}.{key} must be an integer, got {v!r}")
                return 0
            return int(v)
        if kind is float:
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                self.problems.append(f"{path}.{key} must be a number, got {v!r}")
                return 0.0
            return float(v)
        if kind is str and not isinstance(v, str):
            self.problems.append(f"{path}.{key} must be a string, got {v!r}")
            return ""
        if kind is dict and not isinstance(v, Mapping):
            self.problems.append(f"{path}.{key} must be an object, got {v!r}")
            return {}
        return v

    def positive(self, path: str, **values) -> None:
        for name, v in values.items():
            if not v > 0:
                self.problems.append(f"{path}.{name} must be positive, got {v!r}")


@dataclass
class TifosunConfig(ModelConfig):
    width: int
    vocab: int
    norm_eps: float
    layers: list = field(default_factory=list)        # the raw layer objects of config.json
    stop_tokens: tuple = ()

    architecture = "Tifosun"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TifosunConfig":
        rd = _Reader()
        width = rd.get(raw, "config", "width", int)
        vocab = rd.get(raw, "config", "vocab", int)
        eps = rd.get(rd.get(raw, "config", "norm", dict), "config.norm", "eps", float)
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            rd.problems.append("config.layers must be a non-empty list")
            layers = []
        stops = raw.get("eos_token_id")
        if stops is None:
            stops = ()
        elif not isinstance(stops, (list, tuple)):
            stops = (stops,)
        cfg = cls(width=width, vocab=vocab, norm_eps=eps, layers=copy.deepcopy(list(layers)),
                  stop_tokens=tuple(int(t) for t in stops))
        rd.positive("config", width=width, vocab=vocab, **{"norm.eps": eps})
        if not rd.problems:
            cfg._blocks(rd)
        if rd.problems:
            raise ConfigError("unusable Tifosun configuration: " + "; ".join(rd.problems))
        return cfg

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.stop_tokens:
            out["eos_token_id"] = list(self.stop_tokens)
        return out

    # -- layers -------------------------------------------------------------
    def _mixer(self, rd: _Reader, i: int, layer: Mapping):
        path = f"layers[{i}].mixer"
        kind = rd.get(layer, f"layers[{i}]", "type", str)
        m = rd.get(layer, f"layers[{i}]", "mixer", dict)
        if kind in MATRIX_MEMORY_TYPES:
            heads, dim, vdim = (rd.get(m, path, k, int) for k in ("heads", "dim", "vdim"))
            cap = rd.get(m, path, "gate_cap", float)
            rd.positive(path, heads=heads, dim=dim, vdim=vdim, gate_cap=cap)
            return MatrixMemorySpec(hidden_size=self.width, num_heads=heads, qk_dim=dim,
                                    v_dim=vdim, gate_cap=cap, norm_eps=self.norm_eps)
        if kind in LATENT_ATTENTION_TYPES:
            heads, dim, vdim, rank, rot_dim = (rd.get(m, path, k, int)
                                               for k in ("heads", "dim", "vdim", "kv_rank", "rot_dim"))
            rot = rd.get(m, path, "rot", dict)
            base = rd.get(rot, path + ".rot", "base", float)
            dims = rd.get(rot, path + ".rot", "dims", int, default=rot_dim, required=False)
            mask = rd.get(m, path, "mask", dict, default=None, required=False)
            window = None if mask is None else rd.get(mask, path + ".mask", "size", int)
            scale = rd.get(m, path, "scale", float, default=None, required=False)
            rd.positive(path, heads=heads, dim=dim, vdim=vdim, kv_rank=rank, rot_dim=rot_dim,
                        **{"rot.base": base})
            if window is not None:
                rd.positive(path, **{"mask.size": window})
            if dims % 2 or not 0 <= dims <= rot_dim:
                rd.problems.append(f"{path}.rot.dims must be even and at most rot_dim, got {dims}")
            position = PositionSpec(kind="rope", head_dim=rot_dim, rotary_dim=dims, theta=base,
                                    interleaved=True)
            return LatentAttentionSpec(hidden_size=self.width, num_heads=heads, qk_dim=dim,
                                       rot_dim=rot_dim, v_dim=vdim, kv_rank=rank,
                                       position=position, window=window, scale=scale,
                                       norm_eps=self.norm_eps, gated=True)
        rd.problems.append(f"layers[{i}].type {kind!r} is not known (known: "
                           f"{MATRIX_MEMORY_TYPES + LATENT_ATTENTION_TYPES})")
        return None

    def _ffn(self, rd: _Reader, i: int, layer: Mapping):
        mlp = layer.get("mlp") if isinstance(layer, Mapping) else None
        if mlp is None:
            return None
        path = f"layers[{i}].mlp"
        kind = rd.get(mlp, path, "kind", str)
        if kind == "dense":
            ff = rd.get(mlp, path, "ff", int)
            rd.positive(path, ff=ff)
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=ff, activation="silu")
        if kind == "moe":
            router = rd.get(mlp, path, "router", dict)
            experts = rd.get(router, path + ".router", "experts", int)
            top = rd.get(router, path + ".router", "top", int)
            ff = rd.get(rd.get(mlp, path, "expert", dict), path + ".expert", "ff", int)
            shared = mlp.get("shared")
            shared_ff = 0 if shared is None else rd.get(shared, path + ".shared", "ff", int)
            rd.positive(path, experts=experts, top=top, **{"expert.ff": ff})
            if top > experts:
                rd.problems.append(f"{path}.router.top ({top}) exceeds experts ({experts})")
            return RoutedExpertsSpec(hidden_size=self.width, num_experts=experts, top=top,
                                     expert_size=ff, shared_size=shared_ff, score="sigmoid",
                                     renormalize=False, scale_input=True, activation="silu")
        rd.problems.append(f"{path}.kind {kind!r} is not known (known: dense, moe)")
        return None

    def _blocks(self, rd: Optional[_Reader] = None) -> list:
        rd = rd or _Reader()
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps, weight_offset=1.0)
        blocks = []
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, Mapping):
                rd.problems.append(f"layers[{i}] must be an object")
                continue
            mixer = self._mixer(rd, i, layer)
            ffn = self._ffn(rd, i, layer)
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, ffn=ffn, norm1=norm,
                                    norm2=None if ffn is None else norm, norm1_post=norm,
                                    norm2_post=None if ffn is None else norm))
        return blocks

    def layout(self) -> ModelLayout:
        """Layers run once each in the listed order; every layer has a cache entry of its
        own (pages of latents for an attention layer, a state slot for a matrix memory)."""
        norm = NormSpec(kind="rmsnorm", size=self.width, eps=self.norm_eps, weight_offset=1.0)
        blocks = self._blocks()
        order = [RunEntry(block=i, cache=i) for i in range(len(blocks))]
        layout = ModelLayout(vocab_size=self.vocab, hidden_size=self.width, blocks=blocks,
                             order=order, final_norm=norm, tie_word_embeddings=False,
                             max_positions=None)
        layout.validate()
        return layout

    def stop_token_ids(self) -> tuple:
        return tuple(self.stop_tokens)

    def max_positions(self):
        return None
