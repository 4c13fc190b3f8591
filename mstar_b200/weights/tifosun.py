"""Checkpoint tensor names of the Tifosun decoder and where each goes.

Layer i's tensors start with ``l<i>.``: its four norms (``norm1``, ``norm1b``, ``norm2``,
``norm2b``), its mixer under ``mix.`` and its feed-forward under ``mlp.``; the model's
ends are ``embed``, ``final.norm`` and ``head``.  Matrices that read the same input are
stacked into one engine parameter so that one product serves them:

  matrix memory     in    = [q; k; v; g]      gates = [i; f] (with their biases)
  latent attention  in    = [q; dkv; g]
  gated feed-forward gate_up = [gate; up]     (per expert for routed experts, expert
                                               after expert; ``e<j>.down`` likewise)
"""
from __future__ import annotations

from ..config.layout import ModelLayout
from .names import CheckpointMap, TensorSource


def _stack(sources: list, param: str, parts: list) -> None:
    row = 0
    for name, rows in parts:
        sources.append(TensorSource(name, param, row, rows))
        row += rows


def tifosun_checkpoint_map(config, layout: ModelLayout) -> CheckpointMap:
    src: list = []
    width = layout.hidden_size
    src.append(TensorSource("embed", "embed.weight", 0, layout.vocab_size))
    for i, block in enumerate(layout.blocks):
        ck, me = f"l{i}", f"blocks.{i}"
        for ck_norm, part in (("norm1", "norm1"), ("norm1b", "norm1_post"), ("norm2", "norm2"),
                              ("norm2b", "norm2_post")):
            spec = getattr(block, part)
            if spec is not None:
                src.append(TensorSource(f"{ck}.{ck_norm}", f"{me}.{part}.weight", 0, spec.size))
        m = block.mixer
        if m.kind == "mlstm":
            qk, vv = m.num_heads * m.qk_dim, m.num_heads * m.v_dim
            _stack(src, f"{me}.mixer.in.weight", [(f"{ck}.mix.q", qk), (f"{ck}.mix.k", qk),
                                                  (f"{ck}.mix.v", vv), (f"{ck}.mix.g", vv)])
            _stack(src, f"{me}.mixer.gates.weight", [(f"{ck}.mix.i", m.num_heads),
                                                     (f"{ck}.mix.f", m.num_heads)])
            _stack(src, f"{me}.mixer.gates.bias", [(f"{ck}.mix.i.b", m.num_heads),
                                                   (f"{ck}.mix.f.b", m.num_heads)])
            src.append(TensorSource(f"{ck}.mix.norm", f"{me}.mixer.norm.weight", 0, vv))
            src.append(TensorSource(f"{ck}.mix.o", f"{me}.mixer.o.weight", 0, width))
        elif m.kind == "latent_attention":
            q_rows = m.num_heads * (m.qk_dim + m.rot_dim)
            vv = m.num_heads * m.v_dim
            parts = [(f"{ck}.mix.q", q_rows), (f"{ck}.mix.dkv", m.kv_rank + m.rot_dim)]
            if m.gated:
                parts.append((f"{ck}.mix.g", vv))
            _stack(src, f"{me}.mixer.in.weight", parts)
            src.append(TensorSource(f"{ck}.mix.dkv.norm", f"{me}.mixer.kv_norm.weight", 0,
                                    m.kv_rank))
            src.append(TensorSource(f"{ck}.mix.uk", f"{me}.mixer.uk.weight", 0,
                                    m.num_heads * m.qk_dim))
            src.append(TensorSource(f"{ck}.mix.uv", f"{me}.mixer.uv.weight", 0, vv))
            src.append(TensorSource(f"{ck}.mix.o", f"{me}.mixer.o.weight", 0, width))
        else:
            raise ValueError(f"no checkpoint names for a mixer of kind {m.kind!r}")
        f = block.ffn
        if f is None:
            continue
        if f.kind == "gated_mlp":
            _stack(src, f"{me}.ffn.gate_up.weight", [(f"{ck}.mlp.gate", f.intermediate_size),
                                                     (f"{ck}.mlp.up", f.intermediate_size)])
            src.append(TensorSource(f"{ck}.mlp.down", f"{me}.ffn.down.weight", 0, width))
        elif f.kind == "routed_experts":
            src.append(TensorSource(f"{ck}.mlp.router", f"{me}.ffn.router.weight", 0,
                                    f.num_experts))
            gate_up, down = [], []
            for e in range(f.num_experts):
                gate_up += [(f"{ck}.mlp.e{e}.gate", f.expert_size),
                            (f"{ck}.mlp.e{e}.up", f.expert_size)]
                down.append((f"{ck}.mlp.e{e}.down", width))
            _stack(src, f"{me}.ffn.experts.gate_up.weight", gate_up)
            _stack(src, f"{me}.ffn.experts.down.weight", down)
            if f.shared_size:
                _stack(src, f"{me}.ffn.shared.gate_up.weight",
                       [(f"{ck}.mlp.shared.gate", f.shared_size),
                        (f"{ck}.mlp.shared.up", f.shared_size)])
                src.append(TensorSource(f"{ck}.mlp.shared.down", f"{me}.ffn.shared.down.weight",
                                        0, width))
        else:
            raise ValueError(f"no checkpoint names for a feed-forward of kind {f.kind!r}")
    src.append(TensorSource("final.norm", "final_norm.weight", 0, layout.final_norm.size))
    src.append(TensorSource("head", "head.weight", 0, layout.vocab_size))
    return CheckpointMap(sources=src)
