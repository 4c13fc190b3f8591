"""Configuration, layout and checkpoint map of the Tifosun decoder (no GPU needed)."""
import copy

import pytest
import torch

import tifosun_util as U
from mstar_b200.config.base import ConfigError
from mstar_b200.config.registry import config_from_dict, known_architectures
from mstar_b200.engine.model import cache_needs, model_param_specs


def test_architecture_is_found_by_its_single_name():
    assert "Tifosun" in known_architectures()
    cfg = config_from_dict(U.MIXED)
    assert cfg.architecture == "Tifosun" and cfg.to_dict()["layers"] == U.MIXED["layers"]
    assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
    with pytest.raises(ConfigError, match="architecture"):
        config_from_dict({"width": 8})


def test_layout_reads_every_size_per_layer():
    lay = config_from_dict(U.MIXED).layout()
    kinds = [(b.kind, b.mixer.kind, None if b.ffn is None else b.ffn.kind) for b in lay.blocks]
    assert kinds == [("sandwich", "mlstm", "routed_experts"),
                     ("sandwich", "latent_attention", "gated_mlp"),
                     ("sandwich", "mlstm", None),
                     ("sandwich", "latent_attention", "routed_experts")]
    m0, a1, m2, a3 = (b.mixer for b in lay.blocks)
    assert (m0.num_heads, m0.qk_dim, m0.v_dim, m0.gate_cap) == (3, 24, 40, 6.0)
    assert (m2.num_heads, m2.qk_dim, m2.v_dim, m2.gate_cap) == (2, 72, 33, 9.0)
    assert (a1.num_heads, a1.qk_dim, a1.rot_dim, a1.v_dim, a1.kv_rank, a1.window) == (5, 24, 8, 16, 48, 11)
    assert a1.position.rotary_dim == 6 and a1.position.interleaved and a1.scale == 0.9
    assert (a3.window, a3.position.theta, a3.position.rotary_dim) == (7, 50.0, 16)
    f0, f3 = lay.blocks[0].ffn, lay.blocks[3].ffn
    assert (f0.num_experts, f0.top, f0.expert_size, f0.shared_size) == (5, 2, 24, 40)
    assert (f3.num_experts, f3.top, f3.expert_size, f3.shared_size) == (7, 3, 16, 0)
    assert lay.blocks[2].norm2 is None and lay.blocks[2].norm2_post is None
    assert lay.final_norm.weight_offset == 1.0 and lay.blocks[0].norm1_post.weight_offset == 1.0
    needs = cache_needs(lay)
    assert needs[0].kv is None and needs[0].state.shape == (3 * (24 * 40 + 24 + 1),)
    assert needs[1].state is None and (needs[1].kv.planes, needs[1].kv.head_dim,
                                       needs[1].kv.window) == (1, 56, 11)
    assert needs[3].kv.window == 7


def test_checkpoint_map_covers_every_tensor_once():
    cfg = config_from_dict(U.MIXED)
    lay = cfg.layout()
    from mstar_b200.weights.tifosun import tifosun_checkpoint_map

    cmap = tifosun_checkpoint_map(cfg, lay)
    weights = U.random_weights(U.MIXED, 0)
    assert sorted(s.name for s in cmap.sources) == sorted(weights)
    specs = model_param_specs(lay)
    rows = {}
    for s in cmap.sources:
        assert tuple(weights[s.name].shape) == (s.rows,) + tuple(specs[s.param].shape[1:]), s.name
        rows[s.param] = rows.get(s.param, 0) + s.rows
    assert rows == {k: v.shape[0] for k, v in specs.items()}
    # gate rows of expert 1 follow the up rows of expert 0
    src = {s.name: s for s in cmap.sources}
    assert src["l0.mlp.e1.gate"].row_start == 2 * 24 and src["l0.mlp.e1.up"].row_start == 3 * 24
    assert src["l0.mix.i.b"].param == src["l0.mix.f.b"].param and src["l0.mix.f.b"].row_start == 3


@pytest.mark.parametrize("change,match", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0].update(type="conv"), "not known"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=5), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "not known"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_unusable_configurations_are_named(change, match):
    raw = copy.deepcopy(U.MIXED)
    change(raw)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_plain_cut_anywhere_agrees_with_itself():
    """The oracle itself: a sequence fed in pieces equals the sequence fed at once."""
    import plain_tifosun as P

    w = U.random_weights(U.MIXED, 5)
    toks = U.tokens(U.MIXED, 30, 6)
    whole = P.PlainTifosun(U.MIXED, w).forward(toks)
    m = P.PlainTifosun(U.MIXED, w)
    pieces = torch.cat([m.forward(toks[:13]), m.forward(toks[13:15]), m.forward(toks[15:16]),
                        m.forward(toks[16:])])
    assert (whole - pieces).abs().max() < 1e-9
