"""Checkpoint tensor names of the Vudivik decoder and where each goes.

Layer i's tensors start with ``l<i>.`` (a layer that runs another layer's tensors has none):
``norm1`` / ``norm2`` (the norms after the sublayers), the attention under ``mix.left.``, the
selective scan under ``mix.right.``, the two merge norms ``mix.left.out`` / ``mix.right.out``,
the feed-forward under ``mlp.``; the model's ends are ``embed``, ``final.norm``, ``head``.
Stacked into one engine parameter: ``[q; k; v]`` with their biases, and the experts' ``up``
and ``down`` matrices expert after expert.
"""
from __future__ import annotations

from ..config.layout import ModelLayout
from .names import CheckpointMap, TensorSource
from .tifosun import _stack


def vudivik_checkpoint_map(config, layout: ModelLayout) -> CheckpointMap:
    src: list = []
    width = layout.hidden_size
    src.append(TensorSource("embed", "embed.weight", 0, layout.vocab_size))
    for b, (block, layer) in enumerate(zip(layout.blocks, config.block_owners())):
        ck, me = f"l{layer}", f"blocks.{b}"
        src.append(TensorSource(f"{ck}.norm1", f"{me}.norm1_post.weight", 0, width))
        mixer = block.mixer
        if mixer.kind != "parallel" or len(mixer.branches) != 2:
            raise ValueError(f"no checkpoint names for a mixer of kind {mixer.kind!r}")
        left, right = mixer.branches
        lp, rp = f"{ck}.mix.left", f"{ck}.mix.right"
        lm, rm = f"{me}.mixer.branch0", f"{me}.mixer.branch1"
        q_rows = left.num_heads * left.head_dim
        k_rows = left.num_kv_heads * left.head_dim
        v_rows = left.num_kv_heads * left.value_dim
        _stack(src, f"{lm}.qkv.weight", [(f"{lp}.q", q_rows), (f"{lp}.k", k_rows),
                                         (f"{lp}.v", v_rows)])
        _stack(src, f"{lm}.qkv.bias", [(f"{lp}.q.b", q_rows), (f"{lp}.k.b", k_rows),
                                       (f"{lp}.v.b", v_rows)])
        src.append(TensorSource(f"{lp}.q.norm", f"{lm}.q_norm.weight", 0, left.head_dim))
        src.append(TensorSource(f"{lp}.k.norm", f"{lm}.k_norm.weight", 0, left.head_dim))
        src.append(TensorSource(f"{lp}.o", f"{lm}.o.weight", 0, width))
        src.append(TensorSource(f"{rp}.in", f"{rm}.in.weight", 0, 2 * right.inner))
        src.append(TensorSource(f"{rp}.conv", f"{rm}.conv.weight", 0, right.inner))
        src.append(TensorSource(f"{rp}.conv.b", f"{rm}.conv.bias", 0, right.inner))
        src.append(TensorSource(f"{rp}.x", f"{rm}.x.weight", 0, right.dt_rank + 2 * right.state))
        src.append(TensorSource(f"{rp}.dt", f"{rm}.dt.weight", 0, right.inner))
        src.append(TensorSource(f"{rp}.dt.b", f"{rm}.dt.bias", 0, right.inner))
        src.append(TensorSource(f"{rp}.A_log", f"{rm}.A_log", 0, right.inner))
        src.append(TensorSource(f"{rp}.D", f"{rm}.D", 0, right.inner))
        src.append(TensorSource(f"{rp}.o", f"{rm}.o.weight", 0, width))
        src.append(TensorSource(f"{lp}.out", f"{me}.mixer.out0.weight", 0, width))
        src.append(TensorSource(f"{rp}.out", f"{me}.mixer.out1.weight", 0, width))
        f = block.ffn
        if f is None:
            continue
        src.append(TensorSource(f"{ck}.norm2", f"{me}.norm2_post.weight", 0, width))
        if f.kind == "mlp":
            src.append(TensorSource(f"{ck}.mlp.up", f"{me}.ffn.up.weight", 0, f.intermediate_size))
            src.append(TensorSource(f"{ck}.mlp.down", f"{me}.ffn.down.weight", 0, width))
        elif f.kind == "routed_experts":
            outputs = f.num_experts + f.identity_experts
            src.append(TensorSource(f"{ck}.mlp.router", f"{me}.ffn.router.weight", 0, outputs))
            src.append(TensorSource(f"{ck}.mlp.correction", f"{me}.ffn.router.correction", 0,
                                    outputs))
            _stack(src, f"{me}.ffn.experts.up.weight",
                   [(f"{ck}.mlp.e{e}.up", f.expert_size) for e in range(f.num_experts)])
            _stack(src, f"{me}.ffn.experts.down.weight",
                   [(f"{ck}.mlp.e{e}.down", width) for e in range(f.num_experts)])
        else:
            raise ValueError(f"no checkpoint names for a feed-forward of kind {f.kind!r}")
    src.append(TensorSource("final.norm", "final_norm.weight", 0, layout.final_norm.size))
    src.append(TensorSource("head", "head.weight", 0, layout.vocab_size))
    return CheckpointMap(sources=src)
